"""Block arrangements.

``prenorm``: the Llama layer (infernum-llama/src/graph_builder.rs:451-507):
``h += mixer(norm1(h))``; ``h += ffn(norm2(h))``.  The two adds are not done
here: each output is pushed on the residual stream as a pending delta and the
next norm kernel folds it in (the reference's optimizer fuses add + rms_norm
the same way, infernum/src/graph/optimizer.rs:105-174).

Parts of a ``prenorm`` layer: ``norm1``, ``mixer``, ``norm2``, ``ffn``.
"""

from __future__ import annotations

from ..errors import ConfigError
from .base import BLOCKS, Block, ResidualStream


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        missing = [r for r in ("norm1", "mixer", "norm2", "ffn") if r not in parts]
        if missing:
            raise ConfigError(f"prenorm block {params.get('name', '')!r} lacks parts {missing}")

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        stream.push(p["mixer"].forward(p["norm1"].forward(stream), ctx, cache))
        stream.push(p["ffn"].forward(p["norm2"].forward(stream), ctx))


@BLOCKS.register("postnorm")
class PostNormBlock(Block):
    """Norm after the sum: ``h <- norm1(alpha * h + mixer(h))`` and then
    ``h <- norm2(alpha * h + ffn(h))``.  The sub-layers read the stream itself
    (``stream.act``, its rounding to the activation dtype); the normed sum is the
    new stream, kept in float32.  A layer without a feed-forward has no ``ffn``
    part; its ``norm2``, when the checkpoint holds one, norms ``alpha * h``.

    Parameters: ``alpha`` (default 1).  Parts: ``norm1``, ``mixer``, and
    optionally ``ffn`` and ``norm2``; the norms must offer ``renorm``.
    """

    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        self.alpha = float(params.get("alpha", 1.0))
        missing = [r for r in ("norm1", "mixer") if r not in parts]
        if "ffn" in parts and "norm2" not in parts:
            missing.append("norm2")
        if missing:
            raise ConfigError(f"postnorm block {params.get('name', '')!r} lacks parts {missing}")
        for role in ("norm1", "norm2"):
            if role in parts and not hasattr(parts[role], "renorm"):
                raise ConfigError(f"postnorm block: the {parts[role].kind!r} norm cannot norm a stream in place")

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        if stream.act is None:
            raise ConfigError("postnorm block: the stream carries no activation copy (wrong embedding?)")
        stream.push(p["mixer"].forward(stream.act, ctx, cache))
        p["norm1"].renorm(stream, self.alpha)
        ffn, norm2 = p.get("ffn"), p.get("norm2")
        if ffn is not None:
            stream.push(ffn.forward(stream.act, ctx))
            norm2.renorm(stream, self.alpha)
        elif norm2 is not None and getattr(norm2, "present", True):
            norm2.renorm(stream, self.alpha)
