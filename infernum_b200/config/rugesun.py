"""Typed configuration of the Rugesun decoder (``"architecture": "Rugesun"``).

config.json of this design is nested:

    architecture, vocab, width, postln_alpha, logit_softcap,
    norm.eps,
    embedding.bigram.{buckets, mul_prev, mul_cur},
    layers[i].type                      the mixer's kind ("latent_attention")
    layers[i].mixer.{heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
                     rot.{base, dims}, mask.size, kv_from (optional)}
    layers[i].mlp                       null, {kind: "dense", ff} or
                                        {kind: "moe", expert.ff, router.{experts, top}}

Every size and constant is read here and nowhere else; ``max_position`` (not a
key of the design, optional) bounds the scheduler's default sequence length.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .base import take_float, take_int


def _section(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: int  # 0: every earlier token is visible
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        rot = _section(d, "rot", where)
        mask = d.get("mask")
        window = 0
        if mask is not None:
            if not isinstance(mask, Mapping):
                raise ConfigError(f"config.json: {where}'mask' must be an object")
            window = take_int(mask, "size")
        kv_from = d.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"config.json: {where}'kv_from' must name a layer")
        cfg = cls(heads=take_int(d, "heads"), dim=take_int(d, "dim", minimum=0),
                  rot_dim=take_int(d, "rot_dim", minimum=0), vdim=take_int(d, "vdim"),
                  q_rank=take_int(d, "q_rank"), kv_rank=take_int(d, "kv_rank"), scale=take_float(d, "scale"),
                  rot_base=take_float(rot, "base"), rot_dims=take_int(rot, "dims", minimum=0), window=window,
                  kv_from=kv_from)
        if cfg.rot_dims % 2 or cfg.rot_dims > cfg.rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims {cfg.rot_dims} must be even and at most rot_dim")
        if cfg.dim + cfg.rot_dim == 0:
            raise ConfigError(f"config.json: {where}a head needs query/key dimensions")
        return cfg


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = d.get("kind")
        if kind == "dense":
            return cls("dense", take_int(d, "ff"))
        if kind == "moe":
            router = _section(d, "router", where)
            cfg = cls("moe", take_int(_section(d, "expert", where), "ff"), take_int(router, "experts"),
                      take_int(router, "top"))
            if cfg.top > cfg.experts:
                raise ConfigError(f"config.json: {where}top {cfg.top} exceeds the {cfg.experts} experts")
            return cfg
        raise ConfigError(f"config.json: {where}mlp.kind {kind!r} is not supported (dense, moe)")


@dataclass(frozen=True)
class RugesunLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class RugesunConfig:
    vocab: int
    width: int
    postln_alpha: float
    logit_softcap: Optional[float]
    norm_eps: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: Tuple[RugesunLayerConfig, ...]
    max_position: int = 32768
    architecture: str = "Rugesun"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RugesunConfig":
        if d.get("architecture") != "Rugesun":
            raise ConfigError(f"RugesunConfig cannot read architecture {d.get('architecture')!r}")
        bigram = _section(_section(d, "embedding", ""), "bigram", "embedding.")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, ld in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(ld, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = ld.get("type")
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (latent_attention)")
            mixer = LatentMixerConfig.from_dict(_section(ld, "mixer", where), where + "mixer.")
            mlp = ld.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(RugesunLayerConfig(kind, mixer,
                                             FeedForwardConfig.from_dict(mlp, where + "mlp.") if mlp else None))
        for i, layer in enumerate(layers):
            j = layer.mixer.kv_from
            if j is None:
                continue
            if j >= i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from must name an earlier layer")
            src = layers[j].mixer
            if src.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {j}, which keeps no cache")
            if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (
                    layer.mixer.kv_rank, layer.mixer.rot_dim, layer.mixer.rot_dims, layer.mixer.rot_base):
                raise ConfigError(f"config.json: layers[{i}] reads layer {j}'s cache but differs from it in "
                                  f"kv_rank, rot_dim or rotation")
        cap = d.get("logit_softcap")
        if cap is not None:
            cap = take_float(d, "logit_softcap")
            if not cap > 0.0:
                cap = None
        return cls(vocab=take_int(d, "vocab"), width=take_int(d, "width"),
                   postln_alpha=take_float(d, "postln_alpha", default=1.0), logit_softcap=cap,
                   norm_eps=take_float(_section(d, "norm", ""), "eps"),
                   bigram_buckets=take_int(bigram, "buckets"), bigram_mul_prev=take_int(bigram, "mul_prev", minimum=0),
                   bigram_mul_cur=take_int(bigram, "mul_cur", minimum=0), layers=tuple(layers),
                   max_position=take_int(d, "max_position", default=32768))
