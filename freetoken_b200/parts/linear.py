"""Matrix products ``y = x @ W^T`` for the parts, by compute dtype.

* float32 compute: the CUDA-core kernel of ``gemm_simt.cu`` - true 32-bit
  arithmetic with a fixed summation order (no tensor cores, no TF32), weights
  read as stored (float32 or bfloat16, upcast exactly in registers).
* bfloat16 compute, bfloat16 result: a library product (cuBLAS through
  ``torch.matmul``), as the reference does for its dense projections
  (python/freetoken/layers/linear.py:31-32).  Few rows (decode) go through the
  weight-streaming kernel of ``skinny_gemm.cu`` instead.
* bfloat16 compute, float32 result (logits of many rows, the router's logits
  of a long step): the library product with a float32 result where this
  PyTorch offers one (``torch.mm(..., out_dtype=float32)``), else the
  weight-streaming kernel; either way the result is the float32 accumulator,
  never a rounded bfloat16.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
           activation: Optional[str] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = f(x @ weight^T)``; ``weight`` is ``[N, K]``; ``out`` preallocated.  ``activation``
    names ``f`` (one of ``ops.ACTIVATIONS``; ``None``: the product itself): the weight-streaming
    kernel applies it to its float32 accumulator, behind the other products it is a launch
    of its own on the stored result.  ``bias`` (float32 ``[N]``; not together with an
    activation) is added to the product: by the library product itself where that runs (its
    float32 accumulator plus the bias, rounded once), by a launch of its own elsewhere."""
    if bias is not None:
        if activation is not None:
            raise ValueError("linear: a bias and an activation together are not offered")
        rows = x.shape[0]
        if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and out.is_contiguous()
                and not (rows <= SKINNY_ROWS and ops.skinny_gemm_takes(x, weight, out))):
            torch.addmm(_bias_as(bias, torch.bfloat16), x, weight.t(), out=out)
            return out
        linear(x, weight, out)
        ops.bias_add(out, bias)
        return out
    if activation is not None:
        if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
                and ops.skinny_gemm_takes(x, weight, out)):
            ops.skinny_gemm(x, weight, out, rows_per_pass=ops.pass_rows(x.shape[0]), unary=activation)
            return out
        linear(x, weight, out)
        ops.activation(out, activation)
        return out
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        rows = x.shape[0]
        takes = ops.skinny_gemm_takes(x, weight, out)
        if takes and rows <= SKINNY_ROWS:
            ops.skinny_gemm(x, weight, out, rows_per_pass=ops.pass_rows(rows))
            return out
        if out.dtype == torch.bfloat16:
            torch.matmul(x, weight.t(), out=out)
            return out
        if out.dtype == torch.float32 and library_f32_out(x, weight, out):
            return out
        if takes:
            ops.skinny_gemm(x, weight, out, rows_per_pass=32)
            return out
    ops.gemm_rows(x, weight, out)
    return out


_BIAS_COPIES = {}


def _bias_as(bias: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 bias in the library product's element type (made once per bias; exact for a
    bias that was stored in that type)."""
    key = (bias.data_ptr(), dtype)
    hit = _BIAS_COPIES.get(key)
    if hit is None or hit[0] is not bias:
        hit = (bias, bias.to(dtype))
        _BIAS_COPIES[key] = hit
    return hit[1]


_F32_OUT = {"ok": None}


def library_offers_f32_out(device) -> bool:
    """Whether ``torch.mm`` takes ``out_dtype`` (asked once, on a tiny product).
    Only "this PyTorch has no such argument" counts as no; any other error is
    a real one and is raised."""
    if _F32_OUT["ok"] is None:
        a = torch.zeros((16, 16), dtype=torch.bfloat16, device=device)
        try:
            torch.mm(a, a.t(), out_dtype=torch.float32)
            _F32_OUT["ok"] = True
        except (TypeError, NotImplementedError):
            _F32_OUT["ok"] = False
    return _F32_OUT["ok"]


def library_f32_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """bfloat16 x bfloat16 -> float32 through the library product, where this
    PyTorch offers it; the result is the float32 accumulator, not a rounded
    bfloat16.  False: the caller takes one of our kernels instead."""
    if not library_offers_f32_out(x.device):
        return False
    torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    return True


# Up to this many rows the weight-streaming kernel reads the weights once;
# above it the library's tiled product wins.
SKINNY_ROWS = 32


def libraries(compute: torch.dtype, bias: bool = False) -> list:
    libs = ["gemm_simt"] if compute == torch.float32 else ["gemm_simt", "skinny_gemm"]
    return libs + (["rowwise"] if bias else [])
