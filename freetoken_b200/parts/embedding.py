"""Token embedding and output head.

Embedding: ``residual[t,:] = W[ids[t],:]`` with no scale
(python/freetoken/layers/embedding.py:39-47, kernel/csrc/jit/index.cu:31-59).
Head: ``logits = x @ Wlm^T`` in float32 for the rows asked for; with tied
weights ``Wlm`` is the embedding table (layers/embedding.py:107-115).

Two options the reference's models do not have: an RMS norm of the embedded rows
(``residual[t,:] = rms(W[ids[t],:]) * g``, gathered and normed in one kernel) and a
cap on the logits (``cap * tanh(logits / cap)``).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from ..weights.spec import Init, TensorSpec
from . import linear
from .base import Embedding, Head, StepContext, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size, hidden_size``, ``scope`` (the table is ``<scope>.weight``) or
    ``tensor`` (its whole name); ``norm_tensor`` and ``norm_eps``: the embedded rows are
    RMS-normed with that weight before they become the residual stream."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight_name = self.name(spec.get("tensor") or f"{spec.params['scope']}.weight")
        self.norm_name = self.name(spec.get("norm_tensor")) if spec.get("norm_tensor") else None
        self.norm_eps = float(spec.get("norm_eps", 1e-6))
        self.weight = self.norm_weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.weight_name, (self.vocab, self.hidden), tag="embedding")]
        if self.norm_name:
            specs.append(TensorSpec(self.norm_name, (self.hidden,), role="small32",
                                    init=Init(mean=1.0, std=0.0), tag="norm"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]
        if self.norm_name:
            self.norm_weight = tensors[self.norm_name]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] if self.norm_name else ["elementwise"]

    def forward(self, ctx: StepContext, residual: torch.Tensor) -> None:
        if self.norm_name:
            ops.embed_norm(ctx.token_ids, self.weight, self.norm_weight, residual, self.norm_eps)
        else:
            ops.embed_gather(ctx.token_ids, self.weight, residual)


@register_head("lm_head")
class LMHead(Head):
    """params: ``vocab_size, hidden_size, scope`` (the tensor is ``<scope>.weight``) or ``tensor``
    (its whole name), ``tied_to`` (full name of
    the embedding table, or None; a tied head with no ``scope`` has no tensor of its own,
    not even an optional one), ``softcap`` (None or 0: no cap on the logits)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied_to = spec.get("tied_to")
        scope = spec.get("scope")
        own = spec.get("tensor") or (f"{scope}.weight" if scope else None)
        if not own and not self.tied_to:
            raise ValueError("a head needs a tensor of its own ('scope' or 'tensor') or a table to share "
                             "('tied_to')")
        self.own_name = self.name(own) if own else None
        self.weight_name = self.tied_to or self.own_name
        self.softcap = float(spec.get("softcap") or 0.0)
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.tied_to and not self.own_name:
            return []
        if self.tied_to:
            # a checkpoint of a tied model may still carry the head's tensor; it
            # is accepted and dropped (python/freetoken/layers/embedding.py:74-90)
            return [TensorSpec(self.own_name, (self.vocab, self.hidden), optional=True, keep=False)]
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]

    def libraries(self, dtype) -> List[str]:
        return linear.libraries(dtype) + (["rowwise"] if self.softcap else [])

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor) -> None:
        linear.linear(x, self.weight, out)
        if self.softcap:
            ops.softcap(out, self.softcap)
