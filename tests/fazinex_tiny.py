"""Tiny Fazinex configurations, a model-folder writer of the tests' own, and helpers.

The configurations differ from each other in every size and constant: head counts
and group sizes (grouped, one key head, one key head per query head), head sizes
that the tensor-core kernels take (32, 64, 128) and that they refuse (16, 20, 24, 40),
value size equal to and different from the key size, latent rank equal to and
different from both, layers without feed-forward, feed-forward widths that differ
between layers, a loop over a middle span, over all layers, and none, a logit cap
and none, a query temperature with short and long periods and none.
"""

from __future__ import annotations

import json
import os
import struct
from typing import Dict, List

import torch

import plain_fazinex as plain


def attn(heads, kv_heads, dim, scale, coef=None, every=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent(heads, dim, vdim, rank, scale, ff=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# small heads of sizes no tensor-core kernel takes; a loop of three passes over the middle
FZ_A: Dict = {
    "architecture": "Fazinex", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 10.0,
    "layers": [attn(4, 2, 16, 0.3, coef=0.25, every=8, ff=96),
               latent(3, 16, 24, 40, 0.2, ff=80),
               attn(2, 2, 24, 0.25, ff=48),
               latent(2, 8, 8, 16, 0.4)],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

# head sizes 32, 64 and 128 with pages of 64: the tensor-core and TMA-fed kernels
FZ_B: Dict = {
    "architecture": "Fazinex", "vocab": 300, "width": 128, "norm": {"eps": 2e-6},
    "layers": [attn(4, 2, 64, 0.125, coef=0.4, every=16, ff=96),
               latent(4, 32, 32, 64, 0.18, ff=64),
               attn(8, 1, 32, 0.2, coef=0.1, every=3),
               latent(2, 64, 128, 128, 0.1, ff=160)],
}

# awkward sizes: nothing a multiple of 8; the loop covers every layer
FZ_C: Dict = {
    "architecture": "Fazinex", "vocab": 211, "width": 100, "norm": {"eps": 3e-6}, "logit_softcap": 30.0,
    "layers": [latent(5, 20, 12, 36, 0.22, ff=70),
               attn(5, 5, 20, 0.2, coef=0.6, every=1, ff=50)],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

FZ = {"A": FZ_A, "B": FZ_B, "C": FZ_C}
PAGE = {"A": 4, "B": 64, "C": 12}
SEEDS = {"A": 11, "B": 12, "C": 13}

_CODES = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """8-byte little-endian header length, JSON header, raw data."""
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _CODES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)


def write_model(folder: str, config: Dict, state: Dict[str, torch.Tensor]) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), state)
    return folder


def write_tiny(folder: str, which: str) -> str:
    return write_model(folder, FZ[which], plain.random_state(FZ[which], SEEDS[which]))


def tokens(seed: int, n: int, vocab: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# Largest allowed error of a position's logits: root mean square of the difference (its
# mean taken off) over the root mean square of the expected logits (their mean taken off).
# float32: summation orders differ.  bfloat16: every stored activation is rounded to 8 bits
# (2^-9 relative) and the models here run up to eight layers; the largest error seen with
# correct kernels is 0.032, a key that is lost or misplaced gives 0.3 and more.
TOL = {"float32": 3e-5, "bfloat16": 5e-2}


def position_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    g, w = got.double(), want.double()
    d = g - w
    d = d - d.mean(dim=-1, keepdim=True)
    scale = (w - w.mean(dim=-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(dim=-1).sqrt() / scale


def compare(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor], tol: float, what: str) -> None:
    for rid, w in want.items():
        g = got[rid]
        assert not torch.isnan(g).any(), f"{what}: request {rid} has positions without logits (or NaN)"
        err = position_errors(g, w)
        if (err > tol).any():
            pos = int((err > tol).nonzero()[0])
            raise AssertionError(f"{what}: request {rid}: first wrong position {pos} of {len(w)} "
                                 f"(error {float(err[pos]):.3e}, worst {float(err.max()):.3e}, allowed {tol:.1e})")


def make_engine(folder: str, dtype: str, page: int, max_tokens: int, live: int = 4, poison: bool = False):
    from freetoken_b200.engine import Engine, EngineArgs
    return Engine.from_folder(folder, EngineArgs(dtype=dtype, page_size=page, num_pages=-(-max_tokens // page),
                                                 max_running_requests=live, poison_freed_pages=poison))
