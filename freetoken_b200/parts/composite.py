"""A mixer made of several mixers that read the same input.

``y = sum_j scale_j * mixer_j(h)``: every member runs on the block's normed rows with a
cache of its own (pages, state slots or nothing, whatever it asks for), writes its rows into
one ``[T, members, H]`` buffer, and the rows are added in float32 with their scales.  The
members are ordinary registered mixers, so any two (attention beside a state space,
attention beside attention with another window) can stand side by side.
"""

from __future__ import annotations

from typing import List

import torch

from ..cache.manager import CompositeNeed
from ..csrc import ops
from .base import MIXERS, CacheView, Mixer, StepContext, register_mixer


@register_mixer("mixer_sum")
class MixerSum(Mixer):
    """params: ``hidden_size``, ``members`` (PartSpecs of mixers, built below this mixer's
    prefix) and ``scales`` (one factor per member)."""

    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.hidden = int(spec.params["hidden_size"])
        self.members: List[Mixer] = [MIXERS.get(m.kind)(m, prefix) for m in spec.params["members"]]
        self.scales = [float(s) for s in spec.params["scales"]]
        if len(self.scales) != len(self.members) or not self.members:
            raise ValueError("mixer_sum: one scale per member, at least one member")
        self.scale_tensor = None

    @property
    def graph_capturable(self) -> bool:
        return True                      # records what its members record

    def children(self):
        return list(self.members)

    def cache_need(self):
        return CompositeNeed(tuple(m.cache_need() for m in self.members))

    def tensor_specs(self):
        return [s for m in self.members for s in m.tensor_specs()]

    def bind(self, tensors, dtype) -> None:
        for m in self.members:
            m.bind(tensors, dtype)
        device = next(iter(tensors.values())).device
        self.scale_tensor = torch.tensor(self.scales, dtype=torch.float32, device=device)

    def libraries(self, dtype):
        return ["rowwise"] + [lib for m in self.members for lib in m.libraries(dtype)]

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T, n = x.shape[0], len(self.members)
        rows = ctx.workspace.get("mixer_sum.rows", (T, n, self.hidden), ctx.dtype)
        for j, (member, view) in enumerate(zip(self.members, cache.members)):
            if member.writes_into_out:
                member.forward(ctx, x, view, out=rows[:, j])
            else:
                rows[:, j].copy_(member.forward(ctx, x, view))
        if out is None:
            out = ctx.workspace.get("mixer_sum.out", (T, self.hidden), ctx.dtype)
        if not out.is_contiguous():
            dense = ctx.workspace.get("mixer_sum.out", (T, self.hidden), ctx.dtype)
            ops.scaled_sum(rows, self.scale_tensor, dense)
            out.copy_(dense)
            return out
        ops.scaled_sum(rows, self.scale_tensor, out)
        return out
