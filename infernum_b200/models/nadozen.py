"""The Nadozen decoder as a model description.

A decoder-only model of pre-norm layers (layer norms with weight and bias) over
several residual streams per token (hyper-connections; one plain stream when the
configuration names none).  A layer's mixer is either ``wkv`` time mixing (a
recurrent matrix state per head with a data-dependent decay) or ``parallel``:
sliding-window attention without positions - normed queries and keys, values
that are the keys as projected, a sink logit per head, a sigmoid output gate -
side by side with a selective state space layer, their results added with fixed
weights.  Feed-forwards are gated SiLU layers; a layer may have none.  A layer
may run with another layer's tensors and a cache and state of its own.  The
embedding adds a sinusoidal position vector; the logits are scaled.

Checkpoint names: ``embed``, ``l<i>.norm1`` / ``.b``, ``l<i>.norm2`` / ``.b``,
``l<i>.hc<q>.{in, out, mix}``, ``l<i>.mix.*`` (wkv), ``l<i>.mix.left.{q, k, q.norm,
k.norm, sink, g, o}``, ``l<i>.mix.right.{in, conv, conv.b, dt_bias, A_log, D, norm,
o}``, ``l<i>.mlp.{gate, up, down}``, ``final.norm`` / ``.b``, ``head``.
"""

from __future__ import annotations

from ..config.nadozen import NadozenConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem
from ..registry import register_architecture


def build_nadozen_spec(cfg: NadozenConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "weight": name,
                                      "bias": name + ".b"})

    layers, index_of, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p, m = f"l{i}.", layer.mixer
        if layer.type == "wkv":
            mixer = PartSpec("wkv", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim,
                                     "eps": cfg.norm_eps, "decay_rank": m.decay_rank, "prefix": p + "mix."})
        else:
            left, right = m.left, m.right
            mixer = PartSpec("parallel", {
                "left": {"kind": "attention", "params": {
                    "hidden_size": cfg.width, "num_heads": left.heads, "num_kv_heads": left.kv_heads,
                    "head_dim": left.dim, "window": left.window, "scale": left.scale, "position": None,
                    "prefix": p + "mix.left.", "names": {"q": "q", "k": "k", "o": "o"},
                    "qk_norm": {"q": "q.norm", "k": "k.norm", "eps": cfg.norm_eps},
                    "value_from_key": True, "sink": "sink", "gate": "g"}},
                "right": {"kind": "ssd", "params": {
                    "hidden_size": cfg.width, "num_heads": right.heads, "vdim": right.vdim, "state": right.state,
                    "groups": right.groups, "conv": right.conv, "norm_groups": right.norm_groups,
                    "eps": cfg.norm_eps, "prefix": p + "mix.right."}},
                "left_scale": m.left_scale, "right_scale": m.right_scale})
        parts = {"norm1": norm(p + "norm1"), "mixer": mixer}
        if layer.ff is not None:
            parts["norm2"] = norm(p + "norm2")
            parts["ffn"] = PartSpec("swiglu", {
                "hidden_size": cfg.width, "intermediate_size": layer.ff, "prefix": p + "mlp.",
                "names": {"gate": "gate", "up": "up", "down": "down"}, "activation": "silu"})
        index_of[i] = len(layers)
        if cfg.streams is not None:
            layers.append(LayerSpec(block="hyper_prenorm", name=p, parts=parts,
                                    params={"streams": cfg.streams, "prefix": p}))
        else:
            layers.append(LayerSpec(block="prenorm", name=p, parts=parts))
    for i, layer in enumerate(cfg.layers):
        # a layer that uses another's tensors is a further run of that layer, with a cache and state of its own
        schedule.append(ScheduleItem(index_of[i if layer.weights_of is None else layer.weights_of]))
    return ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("sinusoidal_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed", "base": 10000.0,
            "streams": cfg.streams}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head",
                                         "scale": cfg.logit_scale}),
        max_position=cfg.max_position,
    )


register_architecture("Nadozen", NadozenConfig.from_dict, build_nadozen_spec)
