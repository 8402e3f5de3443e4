"""A plain two-matrix feed-forward: ``y = Wdown f(Wup h)``.

``f`` is one of ``relu2`` (the square of relu), ``gelu_tanh`` and ``silu``,
evaluated in float32 on the up projection's output.  The reference's models
use gated, routed experts only (python/freetoken/layers/moe.py:83-92); its dense
linear layers (python/freetoken/layers/linear.py:31-32) are what this part is
made of.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from ..weights.spec import TensorSpec
from . import linear
from .base import FeedForward, StepContext, register_feed_forward


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """params: ``hidden_size, intermediate_size, activation``, ``scope`` and ``names``
    (up, down below the scope)."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.act = str(p.get("activation", "relu2"))
        if self.act not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.act!r} is not one of {sorted(ops.ACTIVATIONS)}")
        scope = self.name(p["scope"])
        self.n_up = f"{scope}.{p['names']['up']}"
        self.n_down = f"{scope}.{p['names']['down']}"
        self.w_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.n_up, (self.inter, self.hidden)),
                TensorSpec(self.n_down, (self.hidden, self.inter), tag="residual_out")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.w_up = tensors[self.n_up]
        self.w_down = tensors[self.n_down]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] + linear.libraries(dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor, out=None) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        # decode rows: the activation is the weight-streaming kernel's epilogue
        mid = linear.linear(x, self.w_up, ws.get("mlp.mid", (T, self.inter), ctx.dtype), activation=self.act)
        if out is None:
            out = ws.get("mlp.y", (T, self.hidden), ctx.dtype)
        return linear.linear(mid, self.w_down, out)
