"""A plain, slow implementation of the Nadozen decoder for whole sequences:
float64, no cache, no state carried between calls, no batching, one function per
mechanism.  It shares no code with the package: the tests hold the package
against it.

Notation: T tokens, width D; weights are [out, in] and applied as W x; ``w`` maps
checkpoint names to tensors.
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


# ---- small functions ----------------------------------------------------------
def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def layer_norm(x, weight, bias, eps: float):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps: float):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---- mechanisms ---------------------------------------------------------------
def position_vectors(T: int, D: int, base: float = 10000.0, start: int = 0):
    """Row p: sin(p f_i) at 2i and cos(p f_i) at 2i+1, f_i = base^(-2i/D)."""
    pe = torch.zeros(T, D, dtype=F)
    for c in range(D):
        f = base ** (-(2 * (c // 2)) / D)
        for t in range(T):
            a = (start + t) * f
            pe[t, c] = math.cos(a) if c % 2 else math.sin(a)
    return pe


def embed(w, cfg, tokens: Sequence[int]):
    return w["embed"][list(tokens)] + position_vectors(len(tokens), cfg["width"])


def hyper_read(xs: List[torch.Tensor], a):
    """u = sum_s a[s] x_s."""
    return sum(a[s] * xs[s] for s in range(len(xs)))


def hyper_write(xs: List[torch.Tensor], M, c, y):
    """x_t' = sum_s M[s, t] x_s + c[t] y, all t from the old streams."""
    n = len(xs)
    return [sum(M[s, t] * xs[s] for s in range(n)) + c[t] * y for t in range(n)]


def token_shift(h, mu):
    """h + (h_prev - h) * mu with zeros before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu


def wkv_decay(m_w, w1, w2, w0):
    return torch.exp(-torch.exp(torch.tanh(m_w @ w1.T) @ w2.T + w0))


def wkv_recurrence(r, k, v, decay, u):
    """One head: r, k, v, decay [T, K], u [K].  Returns o [T, K] and the final state."""
    T, K = r.shape
    S = torch.zeros(K, K, dtype=F)
    o = torch.zeros(T, K, dtype=F)
    for t in range(T):
        kv = torch.outer(k[t], v[t])
        o[t] = (S + u[:, None] * kv).T @ r[t]
        S = decay[t][:, None] * S + kv
    return o, S


def wkv_mixer(w, p: str, m: dict, h, eps: float):
    T = h.shape[0]
    H, K = m["heads"], m["dim"]
    mixes = {s: token_shift(h, w[p + "mu." + s]) for s in "rkvgw"}
    r = (mixes["r"] @ w[p + "r"].T).view(T, H, K)
    k = (mixes["k"] @ w[p + "k"].T).view(T, H, K)
    v = (mixes["v"] @ w[p + "v"].T).view(T, H, K)
    gate = silu(mixes["g"] @ w[p + "g"].T)
    decay = wkv_decay(mixes["w"], w[p + "w1"], w[p + "w2"], w[p + "w0"]).view(T, H, K)
    heads = []
    for a in range(H):
        o, _ = wkv_recurrence(r[:, a], k[:, a], v[:, a], decay[:, a], w[p + "u"][a])
        heads.append(unit_rms(o, eps))
    y = torch.cat(heads, dim=-1) * w[p + "norm"] * gate
    return y @ w[p + "o"].T


def sink_attention_head(q, k, v, scale: float, window: Optional[int], sink):
    """One head: q, k [T, K] (already normed), v [T, V]; position i sees j with
    0 <= i - j < window; exp(sink) joins the denominator."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F)
    for i in range(T):
        lo = 0 if not window else max(0, i - window + 1)
        s = (k[lo: i + 1] @ q[i]) * scale
        top = torch.maximum(s.max(), sink)
        e = torch.exp(s - top)
        out[i] = (e / (e.sum() + torch.exp(sink - top))) @ v[lo: i + 1]
    return out


def sink_attention(w, p: str, m: dict, h, eps: float):
    T = h.shape[0]
    H, G, K = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, K)
    k = (h @ w[p + "k"].T).view(T, G, K)
    qn = unit_rms(q, eps) * w[p + "q.norm"]
    kn = unit_rms(k, eps) * w[p + "k.norm"]
    window = m["mask"]["size"] if m.get("mask") else None
    heads = [sink_attention_head(qn[:, a], kn[:, a // (H // G)], k[:, a // (H // G)], m["scale"], window,
                                 w[p + "sink"][a]) for a in range(H)]
    y = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def causal_conv(x, weight, bias):
    """Per channel: y_t = b + sum_j weight[:, j] x_{t - (taps-1-j)}, zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], dim=0)
    y = bias.expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j: j + T] * weight[:, j]
    return y


def ssd_recurrence(x, B, C, dt, a_log, d_skip):
    """One head: x [T, P], B, C [T, N], dt [T].  Returns y [T, P] and the final state."""
    T, P = x.shape
    S = torch.zeros(B.shape[1], P, dtype=F)
    y = torch.zeros(T, P, dtype=F)
    for t in range(T):
        S = torch.exp(-torch.exp(a_log) * dt[t]) * S + dt[t] * torch.outer(B[t], x[t])
        y[t] = S.T @ C[t] + d_skip * x[t]
    return y, S


def ssd_mixer(w, p: str, m: dict, h, eps: float):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    heads = []
    for a in range(H):
        g = a // (H // G)
        y, _ = ssd_recurrence(x[:, a], B[:, g], C[:, g], dt[:, a], w[p + "A_log"][a], w[p + "D"][a])
        heads.append(y)
    y = torch.cat(heads, dim=-1) * silu(z)
    parts = m.get("norm_groups", 1)
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(w, p: str, m: dict, h, eps: float):
    return m.get("left_scale", 1.0) * sink_attention(w, p + "left.", m["left"], h, eps) + \
        m.get("right_scale", 1.0) * ssd_mixer(w, p + "right.", m["right"], h, eps)


def feed_forward(w, p: str, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def final_logits(w, cfg, x):
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"])
    return (x @ w["head"].T) * cfg.get("logit_scale", 1.0)


# ---- the whole model ----------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], streams_out: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence.  ``streams_out`` collects the sum of
    the streams after every layer run."""
    eps = cfg["norm"]["eps"]
    n_streams = cfg.get("streams")
    x = embed(w, cfg, tokens)
    xs = [x.clone() for _ in range(n_streams)] if n_streams is not None else [x]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of")
        lp = f"l{i if src is None else src}."
        subs = [("1", lambda h: (wkv_mixer if layer["type"] == "wkv" else parallel_mixer)(
            w, lp + "mix.", layer["mixer"], h, eps))]
        if layer.get("mlp") is not None:
            subs.append(("2", lambda h: feed_forward(w, lp + "mlp.", h)))
        for q, f in subs:
            nw, nb = w[lp + "norm" + q], w[lp + "norm" + q + ".b"]
            if n_streams is None:
                xs = [xs[0] + f(layer_norm(xs[0], nw, nb, eps))]
            else:
                hc = lp + "hc" + q
                y = f(layer_norm(hyper_read(xs, w[hc + ".in"]), nw, nb, eps))
                xs = hyper_write(xs, w[hc + ".mix"], w[hc + ".out"], y)
        if streams_out is not None:
            streams_out.append(sum(xs))
    return final_logits(w, cfg, sum(xs))


def argmax(logits) -> int:
    return int(torch.argmax(logits).item())


class Plain:
    """The plain implementation over a model folder, logits cached by sequence."""

    def __init__(self, folder: Optional[str], config: Optional[dict] = None, weights=None):
        self.cfg = read_config(folder if folder is not None else config)
        self.weights = read_weights(folder) if folder is not None else weights
        self._cache: Dict[tuple, torch.Tensor] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._cache:
            self._cache[key] = forward(self.cfg, self.weights, list(tokens))
        return self._cache[key]
