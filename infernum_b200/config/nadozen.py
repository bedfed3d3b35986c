"""Typed configuration of the Nadozen decoder (``"architecture": "Nadozen"``).

config.json of this design is nested:

    architecture, vocab, width, logit_scale, norm.eps,
    streams                             residual streams per token (absent: one plain stream)
    layers[i].type                      "wkv" or "parallel"
    layers[i].weights_of                (optional) the layer whose tensors this one uses
    layers[i].mixer                     wkv:      {heads, dim}
                                        parallel: {left: {heads, kv_heads, dim, vdim, scale, mask.size},
                                                   right: {heads, vdim, state, groups, conv, norm_groups},
                                                   left_scale, right_scale}
    layers[i].mlp                       null or {kind: "dense", ff}

Every size and constant is read here and nowhere else.  Two keys are not the
design's and optional: ``max_position`` bounds the scheduler's default sequence
length, and ``mixer.decay_rank`` of a wkv layer names the rank of its decay's
low-rank pair for the random-weights mode (a checkpoint's tensors give it
otherwise).
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
class WkvConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "WkvConfig":
        return cls(heads=take_int(d, "heads"), dim=take_int(d, "dim"),
                   decay_rank=take_int(d, "decay_rank", default=None))


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int  # 0: every earlier token is visible

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "SinkAttentionConfig":
        mask = d.get("mask")
        window = 0
        if mask is not None:
            if not isinstance(mask, Mapping):
                raise ConfigError(f"config.json: {where}'mask' must be an object")
            window = take_int(mask, "size")
        heads = take_int(d, "heads")
        cfg = cls(heads=heads, kv_heads=take_int(d, "kv_heads", default=heads), dim=take_int(d, "dim"),
                  vdim=take_int(d, "vdim", default=None) or take_int(d, "dim"), scale=take_float(d, "scale"),
                  window=window)
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}{cfg.heads} heads are not a multiple of {cfg.kv_heads} kv_heads")
        if cfg.vdim != cfg.dim:
            raise ConfigError(f"config.json: {where}values are the keys, so vdim {cfg.vdim} must equal dim {cfg.dim}")
        return cfg


@dataclass(frozen=True)
class SsdConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "SsdConfig":
        cfg = cls(heads=take_int(d, "heads"), vdim=take_int(d, "vdim"), state=take_int(d, "state"),
                  groups=take_int(d, "groups", default=1), conv=take_int(d, "conv"),
                  norm_groups=take_int(d, "norm_groups", default=1))
        if cfg.heads % cfg.groups:
            raise ConfigError(f"config.json: {where}{cfg.heads} heads are not a multiple of {cfg.groups} groups")
        if (cfg.heads * cfg.vdim) % cfg.norm_groups:
            raise ConfigError(f"config.json: {where}{cfg.heads * cfg.vdim} channels do not split in "
                              f"{cfg.norm_groups} norm_groups")
        return cfg


@dataclass(frozen=True)
class ParallelConfig:
    left: SinkAttentionConfig
    right: SsdConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "ParallelConfig":
        return cls(left=SinkAttentionConfig.from_dict(_section(d, "left", where), where + "left."),
                   right=SsdConfig.from_dict(_section(d, "right", where), where + "right."),
                   left_scale=take_float(d, "left_scale", default=1.0),
                   right_scale=take_float(d, "right_scale", default=1.0))


@dataclass(frozen=True)
class NadozenLayerConfig:
    type: str  # "wkv" | "parallel"
    mixer: Any  # WkvConfig | ParallelConfig
    ff: Optional[int]  # the dense feed-forward's width, None for a layer without one
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class NadozenConfig:
    vocab: int
    width: int
    logit_scale: float
    norm_eps: float
    streams: Optional[int]  # None: one plain residual stream
    layers: Tuple[NadozenLayerConfig, ...]
    max_position: int = 32768
    architecture: str = "Nadozen"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "NadozenConfig":
        if d.get("architecture") != "Nadozen":
            raise ConfigError(f"NadozenConfig cannot read architecture {d.get('architecture')!r}")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, ld in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(ld, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = ld.get("type")
            mixer_d = _section(ld, "mixer", where)
            if kind == "wkv":
                mixer = WkvConfig.from_dict(mixer_d, where + "mixer.")
            elif kind == "parallel":
                mixer = ParallelConfig.from_dict(mixer_d, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (wkv, parallel)")
            mlp = ld.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"config.json: {where}mlp must be an object or null")
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind')!r} is not supported (dense)")
                ff = take_int(mlp, "ff")
            src = ld.get("weights_of")
            if src is not None and (isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(raw_layers)):
                raise ConfigError(f"config.json: {where}weights_of must name a layer")
            layers.append(NadozenLayerConfig(kind, mixer, ff, src))
        for i, layer in enumerate(layers):
            if layer.weights_of is None:
                continue
            src = layers[layer.weights_of]
            if layer.weights_of == i or src.weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of must name a layer with tensors of its own")
            if (src.type, src.mixer, src.ff) != (layer.type, layer.mixer, layer.ff):
                raise ConfigError(f"config.json: layers[{i}] uses layer {layer.weights_of}'s tensors "
                                  f"but differs from it")
        streams = d.get("streams")
        if streams is not None:
            streams = take_int(d, "streams")
            if streams > 8:
                raise ConfigError(f"config.json: 'streams' {streams} is beyond the 8 the kernels take")
        return cls(vocab=take_int(d, "vocab"), width=take_int(d, "width"),
                   logit_scale=take_float(d, "logit_scale", default=1.0),
                   norm_eps=take_float(_section(d, "norm", ""), "eps"), streams=streams, layers=tuple(layers),
                   max_position=take_int(d, "max_position", default=32768))
