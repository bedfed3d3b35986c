"""Small Nadozen configurations for the tests and their model folders."""

from __future__ import annotations

import os
from typing import Optional

import torch


def wkv(heads, dim, mlp=None, weights_of=None, rank=None):
    m = {"heads": heads, "dim": dim}
    if rank:
        m["decay_rank"] = rank
    d = {"type": "wkv", "mixer": m, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def parallel(left, right, left_scale, right_scale, mlp=None, weights_of=None):
    d = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                       "right_scale": right_scale}, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def left(heads, kv_heads, dim, scale, window):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return m


def right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
            "norm_groups": norm_groups}


DENSE = lambda ff: {"kind": "dense", "ff": ff}  # noqa: E731

# Three streams; a wkv layer with a feed-forward, a parallel layer without one, and both once
# more with the first two's tensors; grouped state-space heads and two norm groups; a window
# that is no multiple of a page.
_A_PAR = (left(6, 2, 16, 0.3, 21), right(4, 12, 20, 2, 3, 2), 0.7, 1.3)
CASE_A = {
    "architecture": "Nadozen", "vocab": 173, "width": 80, "logit_scale": 0.7, "norm": {"eps": 1e-5}, "streams": 3,
    "layers": [
        wkv(3, 16, DENSE(104), rank=12),
        parallel(*_A_PAR),
        wkv(3, 16, DENSE(104), weights_of=0, rank=12),
        parallel(*_A_PAR, weights_of=1),
    ],
}
# Values that are 1 or equal: no ``streams`` key (one plain residual stream), one head, as many
# key/value heads as heads, a window of one token and one longer than any sequence, a
# convolution of one tap and one of two, logit scale 1, sizes that are no multiple of 8.
CASE_B = {
    "architecture": "Nadozen", "vocab": 130, "width": 72, "logit_scale": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        parallel(left(2, 2, 12, 0.25, 1), right(1, 20, 10, 1, 1, 1), 1.0, 1.0, DENSE(40)),
        wkv(1, 28, None, rank=5),
        parallel(left(1, 1, 20, 0.5, 1000), right(3, 6, 14, 3, 2, 3), 0.4, 0.9, None),
        wkv(2, 10, DENSE(52), rank=9),
    ],
}
# Sizes the tensor-core kernels take (head sizes that are multiples of 16, pages of 16), two
# streams, a window that crosses pages and key tiles, attention without a window.
CASE_C = {
    "architecture": "Nadozen", "vocab": 384, "width": 128, "logit_scale": 0.5, "norm": {"eps": 1e-6}, "streams": 2,
    "layers": [
        parallel(left(8, 2, 32, 0.2, 45), right(4, 32, 64, 1, 4, 1), 0.5, 0.8, DENSE(192)),
        wkv(4, 32, None, rank=16),
        parallel(left(4, 4, 64, 0.15, 0), right(8, 16, 32, 2, 4, 4), 1.1, 0.6, None),
        wkv(4, 32, None, weights_of=1, rank=16),
    ],
}
# One stream that still goes through the streams' coefficients, and a state of 128 rows.
CASE_D = {
    "architecture": "Nadozen", "vocab": 97, "width": 64, "logit_scale": 2.0, "norm": {"eps": 1e-5}, "streams": 1,
    "layers": [
        wkv(2, 32, DENSE(48), rank=8),
        parallel(left(4, 1, 16, 0.3, 9), right(2, 24, 128, 1, 5, 2), 0.9, 0.9, DENSE(48)),
    ],
}
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D}
PAGE_SIZES = {"A": 4, "B": 8, "C": 16, "D": 4}


def make_folder(folder: str, config: dict, seed: int, sharpen: float = 0.0, drop: Optional[list] = None) -> str:
    """A random model through the package's writer, with the projections scaled up so
    that every sub-layer moves the streams noticeably.  ``sharpen`` scales the
    weights of the query norm so that attention is peaked and a single wrong key
    shows in the logits (the keys are normed, so scaling a projection would not)."""
    from infernum_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file

    write_random_model(folder, config, seed)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith(".q.norm") and sharpen:
            t = t * sharpen
        elif name.endswith((".left.k", ".left.o", ".left.g", ".right.o", ".mix.o", ".down", ".gate", ".up", "head",
                            "embed")):
            t = t * 6.0
        elif name.endswith((".right.in", ".mix.r", ".mix.k", ".mix.v", ".mix.g", ".mix.w1", ".mix.w2")):
            t = t * 3.0   # (what feeds a recurrence: its state sums these over many tokens)
        elif name.endswith(".mix") and ".hc" in name:
            t = t + torch.eye(t.shape[0]) * 0.8   # streams mostly keep themselves
        else:
            continue
        tensors[name] = t.to(torch.bfloat16)
    for name in drop or []:
        del tensors[name]
    save_file(tensors, path, metadata={"format": "pt"})
    return folder
