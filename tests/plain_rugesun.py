"""A plain, slow implementation of the Rugesun decoder for whole sequences:
float64, no cache, no batching, one function per mechanism.  It shares no code
with the package: the tests hold the package against it.

Notation: T tokens, width D, H heads; weights are [out, in] and applied as W x.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F = torch.float64


def read_config(folder_or_dict) -> dict:
    if isinstance(folder_or_dict, dict):
        return folder_or_dict
    with open(os.path.join(folder_or_dict, "config.json")) as fh:
        return json.load(fh)


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return {k: (v.to(F) if v.is_floating_point() else v) for k, v in
            load_file(os.path.join(folder, "model.safetensors")).items()}


# ---- mechanisms -------------------------------------------------------------
def bigram_rows(tokens: Sequence[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the bigram table for every token; the first token takes row ``buckets``."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(w, cfg, tokens: Sequence[int]) -> torch.Tensor:
    b = cfg["embedding"]["bigram"]
    rows = bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])
    return w["embed"].to(F)[list(tokens)] + w["bigram"].to(F)[rows]


def layer_norm(x, weight, bias, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * weight.to(F) + bias.to(F)


def rms_norm(x, weight, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F)


def gelu_tanh(z) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate(x, positions, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., d]: pair (i, i + dims/2) of the last axis turns by position * base^(-2i/dims)."""
    half = dims // 2
    if half == 0:
        return x
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * torch.cos(angle) - v * torch.sin(angle),
                      v * torch.cos(angle) + u * torch.sin(angle), x[..., dims:]], dim=-1)


def window_mask(T: int, window: int) -> torch.Tensor:
    """[T, T] True where key j is visible from query i: 0 <= i - j < window (window 0: all earlier)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = (i - j) >= 0
    if window > 0:
        m &= (i - j) < window
    return m


def latent_kv(w, p: str, m: dict, h, eps: float):
    """The cached pair of a layer that owns a cache: the normed latent [T, kv_rank]
    and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    kv = h @ w[p + "dkv"].to(F).T
    c = rms_norm(kv[:, : m["kv_rank"]], w[p + "dkv.norm"], eps)
    r = rotate(kv[:, m["kv_rank"]:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    return c, r


def latent_attention(w, p: str, m: dict, h, c, r, eps: float) -> torch.Tensor:
    """The mixer with keys and values made explicitly, head by head."""
    T, H, d, rd, vd = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms_norm(h @ w[p + "dq"].to(F).T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].to(F).T).view(T, H, d + rd)
    q_plain = q[..., :d]
    q_rot = rotate(q[..., d:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    k = (c @ w[p + "uk"].to(F).T).view(T, H, d)
    v = (c @ w[p + "uv"].to(F).T).view(T, H, vd)
    window = (m.get("mask") or {}).get("size", 0)
    visible = window_mask(T, window)
    heads = []
    for a in range(H):
        s = (q_plain[:, a] @ k[:, a].T + q_rot[:, a] @ r.T) * m["scale"]
        s = s.masked_fill(~visible, -math.inf)
        heads.append(torch.softmax(s, dim=-1) @ v[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].to(F).T


def dense_ff(w, p: str, h) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].to(F).T) * (h @ w[p + "up"].to(F).T)) @ w[p + "down"].to(F).T


def route(w, p: str, h, top: int):
    """(indices [T, top], weights [T, top]): the largest logits (lower index among equals)."""
    z = h @ w[p + "router"].to(F).T + w[p + "router.b"].to(F)
    idx = torch.empty((h.shape[0], top), dtype=torch.long)
    zz = z.clone()
    for k in range(top):
        best = zz.max(-1).values
        first = (zz == best[:, None]).to(torch.int8).argmax(-1)  # the lowest index among equals
        idx[:, k] = first
        zz[torch.arange(h.shape[0]), first] = -math.inf
    chosen = torch.gather(z, 1, idx)
    return idx, torch.softmax(chosen, dim=-1)


def moe_ff(w, p: str, h, experts: int, top: int) -> torch.Tensor:
    idx, wts = route(w, p, h, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            q = f"{p}e{e}."
            a = silu(w[q + "gate"].to(F) @ h[t]) * (w[q + "up"].to(F) @ h[t])
            out[t] += wts[t, k] * (w[q + "down"].to(F) @ a)
    return out


def routing_margin(w, p: str, h, top: int) -> torch.Tensor:
    """Per token, how far the last chosen logit lies above the first one left out, in
    units of the row's spread; infinite when every expert is chosen.  A small margin
    says that rounding may choose otherwise."""
    z = h @ w[p + "router"].to(F).T + w[p + "router.b"].to(F)
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=F)
    s = torch.sort(z, dim=-1, descending=True).values
    return (s[:, top - 1] - s[:, top]) / z.std(dim=-1).clamp_min(1e-9)


def softcap(x, cap: Optional[float]) -> torch.Tensor:
    return x if not cap else cap * torch.tanh(x / cap)


# ---- the model ----------------------------------------------------------------
def forward(cfg, w, tokens: Sequence[int], layers_out: Optional[list] = None,
            margins_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] in float64; ``layers_out`` collects the stream after each layer,
    ``margins_out`` the routing margins [T] of every mixture of experts."""
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    x = embed(w, cfg, tokens)
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        src = m.get("kv_from")
        if src is None:
            cached[i] = latent_kv(w, p + "mix.", m, x, eps)
            c, r = cached[i]
        else:
            c, r = cached[src]
        x = layer_norm(alpha * x + latent_attention(w, p + "mix.", m, x, c, r, eps),
                       w[p + "norm1"], w[p + "norm1.b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                f = dense_ff(w, p + "mlp.", x)
            else:
                f = moe_ff(w, p + "mlp.", x, mlp["router"]["experts"], mlp["router"]["top"])
                if margins_out is not None:
                    margins_out.append(routing_margin(w, p + "mlp.", x, mlp["router"]["top"]))
            x = layer_norm(alpha * x + f, w[p + "norm2"], w[p + "norm2.b"], eps)
        elif p + "norm2" in w:
            x = layer_norm(alpha * x, w[p + "norm2"], w[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return softcap(x @ w["head"].to(F).T, cfg.get("logit_softcap"))


class Plain:
    """Logits by sequence, cached (the interface the trace comparison wants)."""

    def __init__(self, folder: Optional[str] = None, config: Optional[dict] = None, weights=None):
        self.cfg = read_config(folder if folder is not None else config)
        self.weights = read_weights(folder) if folder is not None else weights
        self._cache: Dict[tuple, torch.Tensor] = {}
        self._margins: Dict[tuple, torch.Tensor] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._cache:
            margins: list = []
            self._cache[key] = forward(self.cfg, self.weights, list(tokens), margins_out=margins).to(torch.float32)
            self._margins[key] = torch.stack(margins).min(0).values if margins else \
                torch.full((len(key),), math.inf, dtype=F)
        return self._cache[key]

    def margins(self, tokens: Sequence[int]) -> torch.Tensor:
        """Per position the smallest routing margin over the layers."""
        self.logits(tokens)
        return self._margins[tuple(tokens)]
