"""Tiny Tonapel configurations, random weights for them, and helpers of the tests.

The configurations differ from each other in every size and constant: widths, head counts
and group sizes, key sizes equal to, below and above value sizes, windows of 1, of a few
tokens, shorter and longer than a page, rotation of a part of a head, of all of it and of
none, state sizes below 32, between 32 and 64 and above 64, one and several norm groups,
convolutions of 2 to 5 taps, layers without feed-forward, dense and routed feed-forwards with
one, some and all experts chosen, every layer order.
"""

from __future__ import annotations

import copy
from typing import Dict, List

import torch

from fazinex_tiny import make_engine, position_errors, tokens, write_model, write_safetensors  # noqa: F401  (re-exported)


def left(heads, kv_heads, dim, vdim, window, rot_dims, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
            "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims}}


def right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
            "norm_groups": norm_groups}


def parallel(l, r, ls=1.0, rs=1.0, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def model(vocab, width, eps, mult, layers):
    return {"architecture": "Tonapel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "residual_mult": mult, "layers": layers}


# awkward sizes, nothing a multiple of 8; windows of 7 and of 1; a layer without feed-forward
TN_A: Dict = model(150, 40, 1e-5, 0.7, [
    parallel(left(4, 2, 12, 20, 7, 6, base=100.0), right(3, 10, 12, 1, 4, 1), 1.3, 0.6, moe(5, 2, 24, 0.8)),
    delta(4, 2, 12, 10, 2, dense(56)),
    delta(2, 2, 40, 36, 3),
    parallel(left(2, 2, 24, 8, 1, 24, base=500.0, scale=0.3), right(4, 6, 70, 2, 2, 4), 0.5, 1.0, moe(3, 3, 20, 2.5)),
])

# sizes the tensor-core attention kernels take (32, 64, 128; keys and values alike), pages of 64,
# windows shorter than, equal to and longer than a page
TN_B: Dict = model(320, 128, 2e-6, 1.0, [
    parallel(left(4, 2, 64, 64, 100, 32), right(4, 32, 64, 2, 4, 2), 0.75, 1.1, dense(256)),
    delta(4, 2, 64, 64, 4, moe(8, 2, 64, 7.0)),
    parallel(left(8, 1, 32, 32, 64, 16, base=5000.0), right(2, 64, 128, 1, 3, 1), 1.0, 0.4, moe(6, 1, 48, 1.5)),
    parallel(left(2, 2, 128, 128, 130, 128), right(8, 16, 16, 4, 5, 8), 0.6, 0.95, dense(192)),
])

# delta layers only first (no paged cache before the last layer); no rotation; one expert of one;
# a width that is no multiple of 4 (no 16-byte pieces anywhere along a row of the residual)
TN_C: Dict = model(97, 70, 1e-4, 0.35, [
    delta(3, 1, 20, 28, 5, moe(1, 1, 30, 0.5)),
    delta(6, 6, 8, 12, 2, dense(100)),
    parallel(left(6, 3, 16, 40, 33, 0), right(3, 24, 33, 3, 2, 3), 1.0, 1.0),
])

TN = {"A": TN_A, "B": TN_B, "C": TN_C}
PAGE = {"A": 4, "B": 64, "C": 12}
SEEDS = {"A": 21, "B": 22, "C": 23}


def random_state(config: Dict, seed: int, slow_decay: bool = False) -> Dict[str, torch.Tensor]:
    """Every tensor of a model of ``config`` by name, drawn so that activations stay of order one
    and rounded to bfloat16 (what the file holds), as float64.  ``slow_decay``: recurrent states
    that forget slowly, so that a token far back still counts."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]
    out: Dict[str, torch.Tensor] = {}

    def put(name, *shape, std=None, mean=0.0):
        fan_in = shape[-1] if len(shape) > 1 else 1
        s = std if std is not None else fan_in ** -0.5
        out[name] = (torch.randn(*shape, generator=g, dtype=torch.float64) * s + mean).to(torch.bfloat16).double()

    put("embed", config["vocab"], W, std=1.0)
    put("head", config["vocab"], W)
    put("final.norm", W, std=0.1)
    log_rate = -6.0 if slow_decay else -0.5
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer["mlp"] else ()):
            put(p + n, W, std=0.1)
        if layer["type"] == "parallel":
            a, s = m["left"], m["right"]
            q = p + "mix.left."
            for name, rows in (("q", a["heads"] * a["dim"]), ("k", a["kv_heads"] * a["dim"]),
                               ("v", a["kv_heads"] * a["vdim"])):
                put(q + name, rows, W)
                put(q + name + ".b", rows, std=0.3)
            put(q + "o", W, a["heads"] * a["vdim"])
            put(q + "o.b", W, std=0.3)
            r = p + "mix.right."
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            put(r + "in", 2 * inner + 2 * gn + s["heads"], W)
            put(r + "conv", inner + 2 * gn, s["conv"], std=0.5)
            put(r + "conv.b", inner + 2 * gn, std=0.2)
            put(r + "dt_bias", s["heads"], std=0.5, mean=-0.5)
            put(r + "A_log", s["heads"], std=0.5, mean=log_rate)
            put(r + "D", s["heads"], std=0.3, mean=1.0)
            put(r + "norm", inner, std=0.2, mean=1.0)
            put(r + "o", W, inner)
        else:
            q = p + "mix."
            kd, inner = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for name, rows in (("q", kd), ("k", kd), ("v", inner)):
                put(q + name, rows, W)
                put(q + name + ".conv", rows, m["conv"], std=0.5)
            put(q + "g", inner, W)
            put(q + "b", m["heads"], W)
            put(q + "a", m["heads"], W)
            put(q + "A_log", m["heads"], std=0.5, mean=log_rate)
            put(q + "dt_bias", m["heads"], std=0.5, mean=-0.5)
            put(q + "norm", m["vdim"], std=0.2, mean=1.0)
            put(q + "o", W, inner)
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            put(p + "mlp.gate", mlp["ff"], W)
            put(p + "mlp.up", mlp["ff"], W)
            put(p + "mlp.down", W, mlp["ff"])
        elif mlp:
            put(p + "mlp.router", mlp["router"]["experts"], W, std=2.0 * W ** -0.5)
            for e in range(mlp["router"]["experts"]):
                put(f"{p}mlp.e{e}.gate", mlp["expert"]["ff"], W)
                put(f"{p}mlp.e{e}.up", mlp["expert"]["ff"], W)
                put(f"{p}mlp.e{e}.down", W, mlp["expert"]["ff"])
    return out


def as_file(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.to(torch.bfloat16) for k, v in state.items()}


def write_tiny(folder: str, which: str) -> str:
    return write_model(folder, TN[which], as_file(random_state(TN[which], SEEDS[which])))


def one_layer(layer: Dict, vocab=90, width=48, eps=1e-6, mult=1.0) -> Dict:
    return model(vocab, width, eps, mult, [copy.deepcopy(layer)])


def routed_layers(config: Dict) -> List[int]:
    return [i for i, l in enumerate(config["layers"]) if l["mlp"] and l["mlp"]["kind"] == "moe"]


# Largest allowed error of a position's logits (see fazinex_tiny.position_errors).  float32:
# summation orders differ, and four recurrences in a row carry their rounding along.
# bfloat16: every stored activation is rounded to 8 bits; with correct kernels nearly all
# positions stay below 0.03 and single ones reach 0.08 (the delta rule's unit norms and read-out
# norm divide by small numbers now and then); a lost state, a window one token off or a lost key
# gives 0.2 and more, at every position behind the fault.
TOL = {"float32": 5e-5, "bfloat16": 6e-2}


def compare(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor], tol: float, what: str) -> None:
    """Every position of every request within ``tol``.  Above 1e-3 (bfloat16) the bound is on
    rounding noise, whose tail is long: then one position in fifty of a request (at least one) may
    lie between ``tol`` and twice ``tol``, none beyond."""
    for rid, w in want.items():
        g = got[rid]
        assert not torch.isnan(g).any(), f"{what}: request {rid} has positions without logits (or NaN)"
        err = position_errors(g, w)
        over = err > tol
        allowed = max(1, len(w) // 50) if tol > 1e-3 else 0
        if int(over.sum()) > allowed or (err > 2 * tol).any():
            pos = int(over.nonzero()[0])
            raise AssertionError(f"{what}: request {rid}: first wrong position {pos} of {len(w)} "
                                 f"(error {float(err[pos]):.3e}, worst {float(err.max()):.3e}, "
                                 f"{int(over.sum())} positions over {tol:.1e})")
