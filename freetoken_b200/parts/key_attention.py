"""Attention mixers that keep ONE tensor per token in the cache.

Both run causal softmax attention through the kernels of :mod:`.attention`
over pages that hold a single plane, read as keys and again as values.

``shared_kv_attention`` - grouped-query attention whose values are its keys::

    q_t = Wq h_t  (heads x dim),   k_t = Wk h_t  (kv_heads x dim),   v_t = k_t
    q_t <- q_t * (1 + coef * ln(floor((t + 1) / every) + 1))      (query temperature)
    o_t,i = sum_{j <= t} softmax_j(q_t,i . k_j,g(i) * scale) k_j,g(i);   y_t = Wo o_t

No rotation: the temperature is the only way a position enters.

``latent_attention`` - keys and values are made from a cached latent vector::

    c_t = rms(Wdkv h_t) * w_c                (rank numbers: all the cache keeps)
    k_j,i = Wuk,i c_j,   v_j,i = Wuv,i c_j,   score = q_t,i . k_j,i * scale
    o_t,i = sigmoid(Wg h_t)_i * sum_j softmax_j(score) v_j,i;   y_t = Wo o_t

Since ``q . (Wuk c) = (Wuk^T q) . c`` and ``sum_j p_j Wuv c_j = Wuv (sum_j p_j c_j)``,
the mixer multiplies the queries by ``Wuk^T`` per head, attends over the latent
pages as ONE shared key/value head of size ``rank``, and multiplies the result by
``Wuv`` per head: the keys and values themselves are never formed, for a prompt
portion no more than for a decoded token, so the logits at a position do not
depend on how the prompt was cut.

The reference's models have neither mixer; its attention layer
(python/freetoken/models/minimax_m2/attention.py:29-84) is the pattern both follow.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.manager import PagedKeyNeed
from ..csrc import ops
from ..weights.spec import Cat, Init, Name, TensorSpec
from . import linear
from .attention import PagedSoftmaxCore
from .base import CacheView, Mixer, StepContext, register_mixer


def _both_planes(pages: torch.Tensor) -> torch.Tensor:
    """``[pages, kv_heads, page, d]`` seen as the kernels' ``[2 (K, V), ...]``: the same
    plane twice."""
    return pages.unsqueeze(0).expand(2, *pages.shape)


@register_mixer("shared_kv_attention")
class SharedKVAttention(PagedSoftmaxCore, Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, head_dim, sm_scale``,
    ``q_temp_coef`` (0: no temperature), ``q_temp_every``, ``sliding_window`` (None: all
    keys), ``scope`` and ``names`` (q, k, o and the merged qk tensor below the scope)."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.scale = float(p["sm_scale"])
        self.temp_coef = float(p.get("q_temp_coef", 0.0))
        self.temp_every = int(p.get("q_temp_every", 1))
        self.window = p.get("sliding_window")
        if self.nkv <= 0 or self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} is not a multiple of num_kv_heads {self.nkv}")
        if self.d > 512:
            raise ValueError(f"head_dim {self.d} exceeds what the attention kernels take (512)")
        if self.temp_coef != 0.0 and self.temp_every <= 0:
            raise ValueError("q_temp_every must be positive")
        names = p["names"]
        scope = self.name(p["scope"])
        self.n_qk = f"{scope}.{names['qk']}"
        self.n_q, self.n_k, self.n_o = (f"{scope}.{names[k]}" for k in ("q", "k", "o"))
        self.w_qk = self.w_o = None

    def cache_need(self):
        return PagedKeyNeed(self.nkv, self.d, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        qn, kn = self.nq * self.d, self.nkv * self.d
        return [
            TensorSpec(self.n_qk, (qn + kn, self.hidden), sources=(Cat((
                Name(self.n_q, (qn, self.hidden)), Name(self.n_k, (kn, self.hidden))), 0),)),
            TensorSpec(self.n_o, (self.hidden, qn), tag="residual_out"),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.w_qk = tensors[self.n_qk]
        self.w_o = tensors[self.n_o]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] + self.attention_libraries(dtype) + linear.libraries(dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        qn, kn = self.nq * self.d, self.nkv * self.d
        qk = linear.linear(x, self.w_qk, ws.get("kattn.qk", (T, qn + kn), ctx.dtype))
        q = ws.get("kattn.q", (T, qn), ctx.dtype)
        table = ctx.block_tables[cache.block_table_index]
        ops.key_store(qk, q, cache.pages if cache.writes else None, None, ctx.token_pos, ctx.token_seg,
                      table, q_off=0, k_off=qn, num_heads=self.nq, q_dim=self.d, num_kv_heads=self.nkv,
                      k_dim=self.d, temp_coef=self.temp_coef, temp_every=self.temp_every)
        o = ws.get("kattn.o", (T, qn), ctx.dtype)
        self.attend(ctx, q, o, _both_planes(cache.pages), table)
        if out is None:
            out = ws.get("kattn.y", (T, self.hidden), ctx.dtype)
        return linear.linear(o, self.w_o, out)


@register_mixer("latent_attention")
class LatentAttention(PagedSoftmaxCore, Mixer):
    """params: ``hidden_size, num_heads, qk_dim, v_dim, rank, sm_scale, norm_eps``,
    ``output_gate`` (a sigmoid gate per head, read from the mixer's input),
    ``scope`` and ``names`` (q, down, gate, latent_norm, up_k, up_v, o and the merged input
    projection below the scope)."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = 1                       # every head attends over the one latent
        self.dq = int(p["qk_dim"])
        self.dv = int(p["v_dim"])
        self.d = self.rank = int(p["rank"])
        self.scale = float(p["sm_scale"])
        self.eps = float(p["norm_eps"])
        self.gated = bool(p.get("output_gate", True))
        self.window = None
        if self.rank > 512:
            raise ValueError(f"latent rank {self.rank} exceeds what the attention kernels take (512)")
        names = p["names"]
        scope = self.name(p["scope"])
        self.n = {k: f"{scope}.{v}" for k, v in names.items()}
        self.w_in = self.w_norm = self.w_uk = self.w_uv = self.w_ukt = self.w_o = None

    def cache_need(self):
        return PagedKeyNeed(1, self.rank, None)

    def tensor_specs(self) -> List[TensorSpec]:
        H, W, R = self.nq, self.hidden, self.rank
        pieces = [Name(self.n["q"], (H * self.dq, W)), Name(self.n["down"], (R, W))]
        if self.gated:
            pieces.append(Name(self.n["gate"], (H, W)))
        return [
            TensorSpec(self.n["in"], (H * self.dq + R + (H if self.gated else 0), W),
                       sources=(Cat(tuple(pieces), 0),)),
            TensorSpec(self.n["latent_norm"], (R,), role="small32", init=Init(mean=1.0, std=0.0), tag="norm"),
            TensorSpec(self.n["up_k"], (H * self.dq, R)),
            TensorSpec(self.n["up_v"], (H * self.dv, R)),
            TensorSpec(self.n["o"], (W, H * self.dv), tag="residual_out"),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        H, R = self.nq, self.rank
        self.w_in = tensors[self.n["in"]]
        self.w_norm = tensors[self.n["latent_norm"]]
        self.w_uk = tensors[self.n["up_k"]].view(H, self.dq, R)      # [head][dq, R]
        self.w_uv = tensors[self.n["up_v"]].view(H, self.dv, R)      # [head][dv, R]
        # the CUDA-core product wants [N, K] rows: Wuk^T per head
        self.w_ukt = self.w_uk.transpose(1, 2).contiguous() if dtype == torch.float32 else None
        self.w_o = tensors[self.n["o"]]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] + self.attention_libraries(dtype) + linear.libraries(dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        H, R, dq, dv = self.nq, self.rank, self.dq, self.dv
        width = self.w_in.shape[0]
        z = linear.linear(x, self.w_in, ws.get("lattn.in", (T, width), ctx.dtype))
        table = ctx.block_tables[cache.block_table_index]
        # the latent: RMS norm in float32, into the token's place of the page
        ops.key_store(z, None, cache.pages if cache.writes else None, self.w_norm, ctx.token_pos,
                      ctx.token_seg, table, q_off=0, k_off=H * dq, num_heads=H, q_dim=dq, num_kv_heads=1,
                      k_dim=R, eps=self.eps)
        # queries into the latent's space: q' = Wuk^T q per head
        q = ws.get("lattn.q", (T, H * R), ctx.dtype)
        q_heads = z[:, :H * dq].view(T, H, dq)
        if ctx.dtype == torch.float32:
            ops.gemm_heads(q_heads, self.w_ukt, q.view(T, H, R))
        else:
            torch.bmm(q_heads.transpose(0, 1), self.w_uk, out=q.view(T, H, R).transpose(0, 1))
        o = ws.get("lattn.o", (T, H * R), ctx.dtype)
        self.attend(ctx, q, o, _both_planes(cache.pages), table)
        # back out of the latent's space: Wuv per head, then the gate
        y = ws.get("lattn.v", (T, H * dv), ctx.dtype)
        if ctx.dtype == torch.float32:
            ops.gemm_heads(o.view(T, H, R), self.w_uv, y.view(T, H, dv))
        else:
            torch.bmm(o.view(T, H, R).transpose(0, 1), self.w_uv.transpose(1, 2),
                      out=y.view(T, H, dv).transpose(0, 1))
        if self.gated:
            ops.gate_heads(y, z[:, H * dq + R:], H, dv)
        if out is None:
            out = ws.get("lattn.y", (T, self.hidden), ctx.dtype)
        return linear.linear(y, self.w_o, out)
