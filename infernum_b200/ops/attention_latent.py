"""The tensor-core kernel for attention over a latent cache
(``attention_latent_mma.cu``), one compiled module per (kv_rank, width), built
when a model first needs it.

``run`` returns False when the sizes have no variant (kv_rank a multiple of 32,
width a multiple of 16 and at most 576, bfloat16, 16-byte aligned rows); the
caller then takes the plain kernel.  How a step's rows are spread is worked out
once per step and layer geometry and kept in ``ctx.scratch``: 16 or 32 packed
rows (rows x heads; or 64 with eight warps) per CTA, and - when those CTAs would leave most SMs idle, as
with a few decoded rows - the key tiles of each shared out over several CTAs
whose partial sums a second kernel merges.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch

from ..csrc.build import load_module
from ..errors import KernelError
from . import core

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
_libs: Dict[Tuple[int, int], ctypes.CDLL] = {}
SM_COUNT_FALLBACK = 148
MAX_WIDTH = 576
KEY_TILE = 32


def supported(kv_rank: int, width: int) -> bool:
    return kv_rank % 32 == 0 and width % 16 == 0 and 32 <= kv_rank <= width <= MAX_WIDTH


def lib_for(kv_rank: int, width: int) -> ctypes.CDLL:
    lib = _libs.get((kv_rank, width))
    if lib is None:
        lib = load_module(f"attn_latent_kv{kv_rank}_w{width}", ["attention_latent_mma.cu"],
                          [f"-DLAT_KV={kv_rank}", f"-DLAT_W={width}"])
        lib.ib_attention_latent.argtypes = [
            _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p, _c_ll,
            _c_void_p, _c_void_p]
        lib.ib_attention_latent.restype = _c_int
        lib.ib_attention_latent_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        lib.ib_attention_latent_scratch_bytes.restype = _c_ll
        if lib.ib_attention_latent_kv() != kv_rank or lib.ib_attention_latent_width() != width:
            raise KernelError(f"latent attention module for ({kv_rank}, {width}) was built for other sizes")
        _libs[(kv_rank, width)] = lib
    return lib


def choose_plan(rows_per_entry, heads: int, max_kv_len: int, window: int, kv_rank: int, sm_count: int) -> Tuple[int, int]:
    """(packed rows per CTA in sixteens: 1, 2 or 4; splits of the keys).  More rows
    per CTA share a tile of keys among more rows, and are taken when an entry has
    the packed rows to fill them (4: eight warps in two groups).  Splits: while the CTAs leave SMs idle, the keys a CTA
    walks (at most the window plus its rows) are shared out, each slice keeping
    at least two tiles of keys."""
    most = max(rows_per_entry) * heads if rows_per_entry else heads
    mt = 4 if most >= 64 else 2 if most >= 32 else 1
    m = 16 * mt
    ctas = max(1, sum(-(-(r * heads) // m) for r in rows_per_entry if r > 0))
    reach = max_kv_len if window <= 0 else min(max_kv_len, window + max(rows_per_entry, default=1))
    tiles = max(1, -(-reach // KEY_TILE))
    splits = 1
    if ctas < sm_count and tiles >= 4:
        splits = max(1, min(-(-2 * sm_count // ctas), tiles // 2, 64))
    return mt, splits


def run(q_abs: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, kv_rank: int, ctx, tables: torch.Tensor,
        scale: float, window: int, rt) -> bool:
    num_pages, one, page_size, width = pool.shape
    N, heads, _ = q_abs.shape
    if not supported(kv_rank, width) or q_abs.dtype != torch.bfloat16:
        return False
    if q_abs.stride(0) % 8 or q_abs.stride(1) % 8 or out.stride(0) % 2 or out.stride(1) % 2 \
            or q_abs.data_ptr() % 16 or pool.data_ptr() % 16 or out.data_ptr() % 4:
        return False
    core.require_cuda(q_abs, pool, out, tables)
    key = ("latent_plan", heads, kv_rank, width, int(window))
    plan = ctx.scratch.get(key)
    if plan is None:
        cu = ctx.host_cu_rows
        rows = [cu[i + 1] - cu[i] for i in range(ctx.n_entries)]
        forced = rt.options.get("latent_plan")
        plan = tuple(forced) if forced else choose_plan(rows, heads, ctx.max_kv_len, window, kv_rank,
                                                        rt.options.get("sm_count") or SM_COUNT_FALLBACK)
        ctx.scratch[key] = plan
    mt, splits = plan
    lib = lib_for(kv_rank, width)
    scratch_ptr, scratch_bytes = None, 0
    if splits > 1:
        need = lib.ib_attention_latent_scratch_bytes(N, heads, splits)
        buf = ctx.scratch.get("latent_split")
        if buf is None or buf.numel() * 4 < need:
            buf = torch.empty((need + 3) // 4, dtype=torch.float32, device=q_abs.device)
            ctx.scratch["latent_split"] = buf
        scratch_ptr, scratch_bytes = buf.data_ptr(), buf.numel() * 4
    code = lib.ib_attention_latent(
        q_abs.data_ptr(), q_abs.stride(0), q_abs.stride(1), pool.data_ptr(), out.data_ptr(), out.stride(0),
        out.stride(1), ctx.cu_rows.data_ptr(), ctx.q_start.data_ptr(), tables.data_ptr(), tables.shape[1],
        ctx.n_entries, N, ctx.max_rows_per_entry, heads, page_size, num_pages, int(window), float(scale), mt, splits,
        scratch_ptr, scratch_bytes, rt.err.data_ptr(), core.stream_ptr(q_abs))
    core.check(code, "attention_latent_mma")
    return True
