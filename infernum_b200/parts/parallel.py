"""Two mixers side by side: both read the same input and their results are
added with fixed weights, ``left_scale * left(x) + right_scale * right(x)``.

Parameters: ``left``, ``right`` (each {"kind", "params"}: any registered mixer),
``left_scale``, ``right_scale``.  The pair may use the paged cache through one
member and a state slot through one member (the cache manager hands a run one
of each); both members see the run's ``LayerCache`` and take from it what they
declared.  When both members offer their input projection as a product of the
same input (``project`` / ``projected_rows``), the two weights are stacked and one
product feeds both.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from .base import MIXERS, Mixer, PagedCacheSpec, Runtime, StateSpec, WeightSpec
from .linear import Linear


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.members = []
        for side in ("left", "right"):
            spec = params[side]
            self.members.append(MIXERS.get(spec["kind"])(spec.get("params", {}), rt))
        self.scales = (float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0)))
        paged = [m for m in self.members if m.cache_spec() is not None]
        stateful = [m for m in self.members if m.state_spec() is not None]
        if len(paged) > 1 or len(stateful) > 1:
            raise ConfigError("parallel mixer: at most one member may use the paged cache and one a state slot")
        self.replayable = all(m.all_replayable() for m in self.members)
        self.fused_in: Optional[Linear] = None

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return next((m.cache_spec() for m in self.members if m.cache_spec() is not None), None)

    def state_spec(self) -> Optional[StateSpec]:
        return next((m.state_spec() for m in self.members if m.state_spec() is not None), None)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for m in self.members:
            specs.update(m.weight_specs())
        return specs

    def bind(self, weights) -> None:
        for m in self.members:
            m.bind(weights)
        ins = [getattr(m, "qkv", None) or getattr(m, "w_in", None) for m in self.members]
        if all(isinstance(l, Linear) for l in ins) and len({l.weight.dtype for l in ins}) == 1 \
                and len({l.weight.shape[1] for l in ins}) == 1 and all(l.out_features % 8 == 0 for l in ins[:-1]):
            # one product for both members' input projections (they read the same rows);
            # the members keep views of the stacked weight, so nothing is held twice
            stacked = torch.cat([l.weight for l in ins], dim=0)
            self.fused_in = Linear(stacked, self.rt)
            at = 0
            for l in ins:
                l.weight = self.fused_in.weight[at: at + l.out_features]
                at += l.out_features

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.members)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        outs = []
        if self.fused_in is not None:
            both = self.fused_in(x)
            at = 0
            for m in self.members:
                n = (getattr(m, "qkv", None) or m.w_in).out_features
                outs.append(m.forward(x, ctx, cache, projected=both[:, at: at + n]))
                at += n
        else:
            outs = [m.forward(x, ctx, cache) for m in self.members]
        core.pointwise(outs[0], outs[1], "axpby", self.scales[0], self.scales[1])
        return outs[0]
