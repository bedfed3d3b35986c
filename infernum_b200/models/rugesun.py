"""The Rugesun decoder as a model description.

A decoder-only model of post-norm layers: ``x <- norm1(alpha x + mixer(x))``,
``x <- norm2(alpha x + ff(x))`` with layer norms (weight and bias); the mixer
is attention through a latent with a sliding window, some layers reading an
earlier layer's cached latents; the feed-forward is a gated GELU layer or a
mixture of SiLU experts; the embedding adds a hashed bigram row; the logits
are soft-capped.

Checkpoint names: ``embed``, ``bigram``, ``l<i>.norm1`` / ``.b``, ``l<i>.norm2`` /
``.b``, ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o}``,
``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{router, router.b, e<k>.gate, e<k>.up,
e<k>.down}``, ``final.norm`` / ``.b``, ``head``.
"""

from __future__ import annotations

from ..config.rugesun import RugesunConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem
from ..registry import register_architecture


def build_rugesun_spec(cfg: RugesunConfig) -> ModelSpec:
    def norm(name: str, optional: bool = False) -> PartSpec:
        return PartSpec("layernorm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "weight": name,
                                      "bias": name + ".b", "optional": optional})

    # pages of a cache are given back by the widest window among the layers that read it
    cache_window = {}
    for i, layer in enumerate(cfg.layers):
        owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
        w = layer.mixer.window
        prev = cache_window.get(owner)
        cache_window[owner] = w if prev is None else (0 if (w == 0 or prev == 0) else max(prev, w))

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        owner = i if m.kv_from is None else m.kv_from
        parts = {
            "mixer": PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim,
                "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale,
                "window": m.window, "cache_window": cache_window[owner], "eps": cfg.norm_eps,
                "rotary_dim": m.rot_dims, "theta": m.rot_base, "kv_shared": m.kv_from is not None,
                "prefix": p + "mix.",
            }),
            "norm1": norm(p + "norm1"),
        }
        if layer.mlp is None:
            # (no feed-forward: a second norm runs only if the checkpoint holds one)
            parts["norm2"] = norm(p + "norm2", optional=True)
        else:
            parts["norm2"] = norm(p + "norm2")
            if layer.mlp.kind == "dense":
                parts["ffn"] = PartSpec("swiglu", {
                    "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "prefix": p + "mlp.",
                    "names": {"gate": "gate", "up": "up", "down": "down"}, "activation": "gelu_tanh"})
            else:
                parts["ffn"] = PartSpec("moe", {
                    "hidden_size": cfg.width, "expert_size": layer.mlp.ff, "experts": layer.mlp.experts,
                    "top": layer.mlp.top, "activation": "silu", "prefix": p + "mlp."})
        layers.append(LayerSpec(block="postnorm", name=p, parts=parts, params={"alpha": cfg.postln_alpha}))
        schedule.append(ScheduleItem(i, cache_of=m.kv_from))
    return ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("hashed_bigram_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed", "bigram_weight": "bigram",
            "buckets": cfg.bigram_buckets, "mul_prev": cfg.bigram_mul_prev, "mul_cur": cfg.bigram_mul_cur}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head",
                                         "softcap": cfg.logit_softcap}),
        max_position=cfg.max_position,
    )


register_architecture("Rugesun", RugesunConfig.from_dict, build_rugesun_spec)
