"""Tonapel beside the MiniMax-M3 decoder at equal size: step throughput and kernel rooflines.

    python bench.py --design tonapel [--sizes w2048,w4096] [--steps K] [--warmup W]

For every size a four-layer Tonapel model (parallel + dense, delta + experts, parallel + experts,
delta + dense; random weights) and a MiniMax-M3 decoder of the same width, head counts, head size,
layer count and vocabulary run the same workload through ``Engine.step`` (the method of
:mod:`.design_bench`): one prompt of ``--prefill-tokens`` tokens, and decode steps at batch 8 and 1
on contexts of ``--context`` tokens built by real prefill.

The second part times the design's own kernels beside the like kernel of the other model, each
replayed from a CUDA graph over inputs that are rotated so that no repetition finds them in L2,
as a fraction of the measured copy bandwidth: the scans of the two recurrent mixers (a prompt
portion of 8,192 tokens, and a decode batch of 64 whose traffic is the states) beside decode
attention over 2,048 keys; the short convolution and the gated norm beside ``qk_rope_store``; the
norm that adds a branch into the residual beside ``rmsnorm``; decode attention inside a window
beside the same kernel over the whole context.  One JSON line.
"""

from __future__ import annotations

import json
import time
from typing import Any, Callable, Dict, List

from .design_bench import LAYERS, _timed, measure_model, minimax_config

SIZES: Dict[str, Dict[str, int]] = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, ssd_heads=32, ssd_dim=64, state=128,
                  delta_heads=16, ff=8192, experts=8, top=2, vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=1024, ssd_heads=64, ssd_dim=64, state=128,
                  delta_heads=32, ff=14336, experts=8, top=2, vocab=32768),
}
TAPS = 4


def tonapel_config(s: Dict[str, int]) -> Dict[str, Any]:
    d = s["dim"]
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5,
            "mask": {"size": s["window"]}, "rot": {"base": 1e4, "dims": d // 2}}
    right = {"heads": s["ssd_heads"], "vdim": s["ssd_dim"], "state": s["state"], "groups": 1, "conv": TAPS,
             "norm_groups": 1}
    par = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.7}
    dl = {"heads": s["delta_heads"], "kv_heads": s["delta_heads"], "dim": d, "vdim": d, "conv": TAPS}
    inter = max(128, (s["ff"] // 3) // 128 * 128)           # a token uses about as much as the dense one holds
    dense = {"kind": "dense", "ff": s["ff"] * 2 // 3 // 128 * 128}
    moe = {"kind": "moe", "expert": {"ff": inter, "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]}}
    return {"architecture": "Tonapel", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "residual_mult": 0.7,
            "layers": [{"type": "parallel", "mixer": par, "mlp": dense}, {"type": "delta", "mixer": dl, "mlp": moe},
                       {"type": "parallel", "mixer": par, "mlp": moe}, {"type": "delta", "mixer": dl, "mlp": dense}]}


def kernel_pairs(s: Dict[str, int], peaks: Dict[str, Any], reps: int = 10) -> Dict[str, Any]:
    import torch

    from .csrc import ops
    from .parts.base import Workspace

    dev, bf = "cuda:0", torch.bfloat16
    hbm = peaks["hbm_gbs"] * 1e9
    W, d, P = s["width"], s["dim"], 64
    out: Dict[str, Any] = {}

    def rotate(make: Callable[[], Any], nbytes: int, most: int = 16) -> List[Any]:
        return [make() for _ in range(min(most, max(2, -(-(256 << 20) // max(1, nbytes)))))]

    def run(name: str, launch: Callable[[int], None], sets: int, nbytes: float) -> None:
        for i in range(min(sets, 3)):
            launch(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(sets):
                launch(i)
        graph.replay()
        ms = _timed(graph.replay, reps) / sets
        out[name] = {"us": round(ms * 1e3, 2), "gbs": round(nbytes / (ms / 1e3) / 1e9, 1),
                     "frac_of_measured_copy_peak": round(nbytes / (ms / 1e3) / hbm, 3)}

    def meta(lens):
        q = [0]
        for n in lens:
            q.append(q[-1] + n)
        seg = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(dev)
        return (seg, torch.arange(len(lens), dtype=torch.int32, device=dev),
                torch.tensor(q, dtype=torch.int32, device=dev))

    Hs, Ps, N = s["ssd_heads"], s["ssd_dim"], s["state"]
    inner, C = Hs * Ps, Hs * Ps + 2 * N
    Hd = s["delta_heads"]
    Cd = 3 * Hd * d
    for label, lens in (("one prompt portion of 8,192 tokens", [8192]), ("decode batch of 64", [1] * 64)):
        T, S = sum(lens), len(lens)
        seg, slot, q = meta(lens)
        # ---- state space ------------------------------------------------------------------
        state_b = Hs * N * Ps * 4
        xs = rotate(lambda: torch.randn(T, C, device=dev, dtype=bf) * 0.5, T * C * 2 + S * state_b)
        states = [torch.zeros(S, Hs * N * Ps, device=dev) for _ in xs]
        dt = torch.randn(T, Hs, device=dev, dtype=bf)
        small = [torch.zeros(Hs, device=dev) for _ in range(3)]
        y = torch.empty(T, inner, device=dev)
        run(f"ssd_scan, {label}", lambda i: ops.ssd_scan(xs[i], dt, small[0], small[1], small[2], states[i], y, slot, q,
                                                         Hs, Ps, N, 1), len(xs),
            nbytes=T * C * 2 + T * inner * 4 + 2 * S * state_b)
        conv_state = [torch.zeros(S, (TAPS - 1) * C, device=dev) for _ in xs]
        cw, cb = torch.randn(C, TAPS, device=dev), torch.zeros(C, device=dev)
        conv_out = torch.empty(T, C, device=dev, dtype=bf)
        run(f"conv_silu, {label}", lambda i: ops.conv_silu(xs[i], conv_out, cw, cb, conv_state[i], seg, slot, q), len(xs),
            nbytes=2 * T * C * 2 + 2 * S * (TAPS - 1) * C * 4)
        gate = torch.randn(T, inner, device=dev, dtype=bf)
        nw = torch.ones(inner, device=dev)
        ys = rotate(lambda: torch.randn(T, inner, device=dev), T * inner * 8, most=8)
        gout = torch.empty(T, inner, device=dev, dtype=bf)
        run(f"gated_norm, {label}", lambda i: ops.gated_norm(ys[i], gate, nw, gout, 1, 1e-6, True), len(ys),
            nbytes=T * inner * (4 + 2 + 2))
        del xs, states, conv_state, ys
        # ---- delta rule --------------------------------------------------------------------
        dstate_b = Hd * d * d * 4
        qs = rotate(lambda: torch.randn(T, Cd, device=dev, dtype=bf), T * Cd * 2 + S * dstate_b)
        dstates = [torch.zeros(S, Hd * d * d, device=dev) for _ in qs]
        gates = torch.randn(T, 2 * Hd, device=dev, dtype=bf)
        o = torch.empty(T, Hd * d, device=dev)
        run(f"delta_scan, {label}",
            lambda i: ops.delta_scan(qs[i], gates[:, :Hd], gates[:, Hd:], small[0][:Hd], small[1][:Hd], dstates[i], o,
                                     slot, q, Hd, Hd, d, d, 1e-6, d ** -0.5), len(qs),
            nbytes=T * Cd * 2 + T * Hd * d * 4 + 2 * S * dstate_b)
        del qs, dstates
        # ---- the norm that adds a branch, beside the norm that adds the residual ------------
        branches = rotate(lambda: torch.randn(T, W, device=dev, dtype=bf), T * W * (2 + 8 + 2), most=8)
        res = torch.zeros(T, W, device=dev)
        w1 = torch.zeros(W, device=dev)
        nout = torch.empty(T, W, device=dev, dtype=bf)
        run(f"norm_add + next norm, {label}",
            lambda i: ops.norm_add(branches[i], res, w1, 1e-6, True, 0.5, next_weight=w1, next_eps=1e-6,
                                   next_plus_one=True, next_out=nout), len(branches), nbytes=T * W * (2 + 8 + 2))
        run(f"rmsnorm (residual add + norm), {label}",
            lambda i: ops.rmsnorm(branches[i], res, w1, nout, 1e-6, True), len(branches), nbytes=T * W * (2 + 8 + 2))
        del branches

    # ---- projection rows -> queries + cache (the like kernel of the convolution) -------------
    T = 8192
    H, G = s["heads"], s["kv_heads"]
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seg0 = torch.zeros(T, dtype=torch.int32, device=dev)
    table = torch.arange(1, T // P + 1, dtype=torch.int32, device=dev).view(1, -1)
    qkv_bytes = T * (H + 2 * G) * d * 2
    srcs = rotate(lambda: torch.randn(T, (H + 2 * G) * d, device=dev, dtype=bf), 2 * qkv_bytes)
    q_out = torch.empty(T, H * d, device=dev, dtype=bf)
    kv_pages = torch.zeros(2, T // P + 1, G, P, d, device=dev, dtype=bf)
    cos_sin = torch.ones(T, d // 2, device=dev)
    run("qk_rope_store (rotary, keys and values to pages), 8,192 tokens",
        lambda i: ops.qk_rope_store(srcs[i], q_out, kv_pages, None, None, cos_sin, pos, seg0, table, H, G, d, d // 2,
                                    0, False, False, 1e-6), len(srcs), nbytes=2 * qkv_bytes)
    del srcs

    # ---- decode attention, 64 requests at position 2,047: inside a window, and all keys ----------
    B, ctx = 64, 2048
    ws = Workspace(dev)
    per_req = ctx // P
    n_pages = B * per_req
    dpos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    dseg = torch.arange(B, dtype=torch.int32, device=dev)
    dtable = torch.arange(1, n_pages + 1, dtype=torch.int32, device=dev).view(B, per_req)
    caches = rotate(lambda: torch.randn(2, n_pages + 1, G, P, d, device=dev, dtype=bf), 2 * (n_pages + 1) * G * P * d * 2,
                    most=3)
    qd = torch.randn(B, H * d, device=dev, dtype=bf)
    od = torch.empty_like(qd)
    for name, window in ((f"attn_decode inside a window of {s['window']}", s["window"]), ("attn_decode, all 2,048 keys", None)):
        keys = window or ctx
        run(name, lambda i, w=window: ops.attn_decode(qd, od, caches[i], None, B, dpos, dseg, dtable, H, G, d, d ** -0.5,
                                                      w, ctx, ws), len(caches), nbytes=B * keys * G * d * 2 * 2)
    return out


def main(a) -> int:
    import torch

    from .benchmark import ClockSampler, load_peaks

    peaks = load_peaks()
    names = [n for n in a.sizes.split(",") if n.strip()]
    for n in names:
        if n not in SIZES:
            print(f"unknown size '{n}' (known: {', '.join(SIZES)})")
            return 2
    t0 = time.time()
    sizes: Dict[str, Any] = {}
    with ClockSampler() as clocks:
        for n in names:
            s = SIZES[n]
            room = a.context + a.steps + a.warmup + 512
            sizes[n] = {"shape": s,
                        "tonapel": measure_model(tonapel_config(s), a),
                        "minimax_m3_equal_size": measure_model(minimax_config({**s, "rank": 0}, room), a)}
        kernels = kernel_pairs(SIZES[names[0]], peaks)
    torch.cuda.synchronize()
    line = {"bench": "design", "design": "Tonapel", "beside": "MiniMax-M3 decoder at equal size",
            "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids", "layers": LAYERS,
            "context": a.context, "steps": a.steps, "warmup": max(3, a.warmup), "sizes": sizes,
            "kernels_at": names[0], "kernels": kernels,
            "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": peaks["source"]},
            "clocks": clocks.summary(), "wall_s": round(time.time() - t0, 1)}
    print(json.dumps(line))
    return 0
