"""Small Rugesun configurations for the tests, their model folders, and a way
to make attention peaked so that a single wrong key shows in the logits."""

from __future__ import annotations

import os
from typing import Optional

import torch


def mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base=10000.0, kv_from=None,
          rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(m, mlp):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


DENSE = lambda ff: {"kind": "dense", "ff": ff}  # noqa: E731
MOE = lambda ff, experts, top: {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}  # noqa: E731

# Three layers: an owner with a mixture of experts; a reader of its cache whose window is
# wider than the owner's, with a dense feed-forward; an owner of other sizes without a
# feed-forward.
CASE_A = {
    "architecture": "Rugesun", "vocab": 211, "width": 96, "postln_alpha": 1.5, "logit_softcap": 12.0,
    "norm": {"eps": 1e-5}, "embedding": {"bigram": {"buckets": 97, "mul_prev": 7, "mul_cur": 13}},
    "layers": [
        layer(mixer(3, 16, 8, 24, 24, 40, 0.2, 20), MOE(24, 6, 2)),
        layer(mixer(3, 16, 8, 24, 24, 40, 0.2, 28, kv_from=0), DENSE(136)),
        layer(mixer(2, 8, 16, 8, 16, 16, 0.3, 9, base=500.0), None),
    ],
}
# Values that are 1 or equal to each other: one head, top 1, top = experts, a window of one
# token and a window longer than any sequence, alpha 1, no soft cap, sizes that are no
# multiple of 8, five bigram buckets.
CASE_B = {
    "architecture": "Rugesun", "vocab": 130, "width": 72, "postln_alpha": 1.0, "logit_softcap": None,
    "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 1}},
    "layers": [
        layer(mixer(1, 12, 4, 20, 10, 20, 0.25, 1000), MOE(12, 3, 1)),
        layer(mixer(2, 6, 6, 10, 14, 22, 0.4, 1), MOE(20, 2, 2)),
        layer(mixer(1, 12, 4, 20, 10, 20, 0.25, 5, kv_from=0), DENSE(40)),
        layer(mixer(4, 8, 4, 8, 12, 20, 0.3, 0, kv_from=0), DENSE(64)),
    ],
}
# Sizes the tensor-core kernels take (multiples of 16, pages of 16), a window that is no
# multiple of a page or a key tile, two owners with readers in between.
CASE_C = {
    "architecture": "Rugesun", "vocab": 384, "width": 128, "postln_alpha": 2.5, "logit_softcap": 20.0,
    "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 509, "mul_prev": 29, "mul_cur": 11}},
    "layers": [
        layer(mixer(4, 16, 16, 16, 48, 32, 0.18, 37), DENSE(192)),
        layer(mixer(4, 16, 16, 16, 48, 32, 0.18, 70, kv_from=0), MOE(32, 8, 3)),
        layer(mixer(8, 32, 32, 16, 64, 96, 0.12, 45), MOE(64, 4, 2)),
        layer(mixer(8, 32, 32, 16, 64, 96, 0.12, 45, kv_from=2), DENSE(128)),
    ],
}
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}
PAGE_SIZES = {"A": 4, "B": 8, "C": 16}


def make_folder(folder: str, config: dict, seed: int, sharpen: float = 0.0, drop: Optional[list] = None) -> str:
    """A random model through the package's writer.  ``sharpen`` scales the query
    up-projections so that attention is peaked; the value, output and feed-forward
    down projections are scaled so that every sub-layer moves the stream
    noticeably.  ``drop`` names tensors to leave out of the file."""
    from infernum_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file

    write_random_model(folder, config, seed)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith((".mix.uq", ".mix.dkv", ".mix.dq")):
            t = t * (6.0 if not sharpen else 6.0 * sharpen ** 0.5)
        elif name.endswith((".mix.uk", ".mix.uv", ".mix.o", ".down", ".gate", ".up", "head", "embed", "bigram")):
            t = t * 6.0
        else:
            continue
        tensors[name] = t.to(torch.bfloat16)
    for name in drop or []:
        del tensors[name]
    save_file(tensors, path, metadata={"format": "pt"})
    return folder
