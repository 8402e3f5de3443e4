"""Fazinex beside the MiniMax-M3 decoder at equal size: step throughput and kernel rooflines.

    python bench.py --design fazinex [--sizes w2048,w4096] [--steps K] [--warmup W]

For every size a four-layer Fazinex model (attention, latent, latent, attention; random
weights) and a MiniMax-M3 decoder of the same width, head counts, head size, layer count
and vocabulary (eight experts, two per token, sized so that a token uses as many
feed-forward weights as the dense feed-forward has) run the same workload through
``Engine.step``: one prompt of ``--prefill-tokens`` tokens, and decode steps at batch 8 and
1 on contexts of ``--context`` tokens built by real prefill.  Device time between CUDA
events after warm-up; the weights of either model exceed the L2 cache.  Per-kernel device
times of one decode and one prefill step come from the profiler's kernel timestamps.

The second part times the design's own kernels beside the like kernel of the other model
on inputs that are rotated so that no repetition finds them in L2 (all launches of a
rotation replayed from one CUDA graph, so that the host's launch time is not measured), and gives each as a
fraction of the measured peak (copy bandwidth, or library bf16 throughput): ``key_store``
beside ``qk_rope_store``, ``embed_norm`` beside ``embed_gather``, decode and prefill
attention over one cached plane beside the same kernels over separate keys and values.
One JSON line.
"""

from __future__ import annotations

import json
import time
from typing import Any, Callable, Dict, List

SIZES: Dict[str, Dict[str, int]] = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, rank=128, ff=8192, vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, rank=128, ff=14336, vocab=32768),
}
LAYERS = 4


def fazinex_config(s: Dict[str, int]) -> Dict[str, Any]:
    attn = {"type": "attention", "mlp": {"kind": "dense", "ff": s["ff"]},
            "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                      "scale": s["dim"] ** -0.5, "q_temp": {"coef": 0.1, "every": 512}}}
    latent = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": s["ff"]},
              "mixer": {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "kv_rank": s["rank"],
                        "scale": s["dim"] ** -0.5}}
    return {"architecture": "Fazinex", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "logit_softcap": 30.0, "layers": [attn, latent, latent, attn]}


def minimax_config(s: Dict[str, int], max_positions: int) -> Dict[str, Any]:
    inter = max(128, (s["ff"] // 3) // 128 * 128)
    return dict(architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3", hidden_size=s["width"],
                num_hidden_layers=LAYERS, num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"],
                head_dim=s["dim"], rotary_dim=s["dim"] // 2, rope_theta=5e6, max_position_embeddings=max_positions,
                rms_norm_eps=1e-6, use_gemma_norm=True, use_qk_norm=True, qk_norm_type="per_head",
                num_local_experts=8, num_experts_per_tok=2, intermediate_size=inter, scoring_func="sigmoid",
                use_routing_bias=True, norm_topk_prob=True, routed_scaling_factor=1.0, hidden_act="silu",
                vocab_size=s["vocab"], tie_word_embeddings=False)


def _timed(fn: Callable[[], None], reps: int) -> float:
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps


def _kernel_times(fn: Callable[[], None], steps: int = 3) -> Dict[str, float]:
    """Device microseconds per step of every kernel ``fn`` launches (profiler timestamps)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
    rows: Dict[str, float] = {}
    for e in prof.key_averages():
        if e.device_time_total > 0:           # instantiations of one template are added up
            rows[_short(e.key)] = rows.get(_short(e.key), 0.0) + e.device_time_total / steps
    return dict(sorted(rows.items(), key=lambda kv: -kv[1]))


def _short(name: str) -> str:
    for cut in ("<", "("):
        if cut in name:
            name = name[:name.index(cut)]
    return name.replace("void ", "").replace("ft::", "")[:48]


def measure_model(config: Dict[str, Any], a, seed: int = 0) -> Dict[str, Any]:
    """Prefill and decode steps of one model through ``Engine.step``."""
    import numpy as np
    import torch

    from .benchmark import bench_random_options
    from .engine import Engine, EngineArgs, StepEntry

    page, batch = 64, 8
    room = a.context + a.steps + a.warmup + 16 + 2 * page
    pool = batch * (-(-room // page) * page) + (-(-a.prefill_tokens // page) * page)
    engine = Engine.from_config(config, seed, EngineArgs(
        dtype="bfloat16", page_size=page, max_tokens=pool, max_running_requests=batch + 1,
        max_seq_len=room + page), random_options=bench_random_options())
    V = engine.vocab_size
    rng = np.random.default_rng(seed)
    out: Dict[str, Any] = {"weights_gb": round(engine.weight_bytes / 1e9, 3)}

    def prefill_once():
        engine.step([StepEntry("p", rng.integers(0, V, a.prefill_tokens).tolist(), [a.prefill_tokens - 1])])
        engine.end_request("p")

    for _ in range(max(3, a.warmup)):
        prefill_once()
    ms = _timed(prefill_once, 5)
    out["prefill"] = {"tokens": a.prefill_tokens, "ms": round(ms, 3),
                      "tokens_per_s": round(a.prefill_tokens / (ms / 1e3))}
    kernels = _kernel_times(prefill_once)
    out["prefill"]["kernel_us"] = {k: round(v, 1) for k, v in list(kernels.items())[:10]}
    out["prefill"]["kernel_us_total"] = round(sum(kernels.values()), 1)

    ids = [f"d{i}" for i in range(batch)]
    per = max(1, 8192 // a.context)
    for i in range(0, batch, per):
        engine.step([StepEntry(r, rng.integers(0, V, a.context).tolist(), []) for r in ids[i:i + per]])
    for b in (batch, 1):
        live = ids[:b]

        def decode_once():
            toks = rng.integers(0, V, b)
            engine.step([StepEntry(r, [int(t)], [0]) for r, t in zip(live, toks)])

        for _ in range(max(3, a.warmup)):
            decode_once()
        ms = _timed(decode_once, a.steps)
        # a windowed group reads no more than its window; a request's state rows are read and written
        held = sum(min(engine.length(live[0]), g.need.window or engine.length(live[0])) * (
            t.numel() * t.element_size() // (t.shape[1 + g.need.page_axis] * page))
            for t, g in zip(engine.storage.paged, engine.cache.paged_groups))
        state_bytes = sum(2 * t[:, 0].numel() * t.element_size() for t in engine.storage.state)
        nbytes = engine.weight_bytes + b * (held + state_bytes)
        out[f"decode_b{b}"] = {"ms": round(ms, 4), "tokens_per_s": round(b / (ms / 1e3)),
                               "bytes_per_step": nbytes, "gbs": round(nbytes / (ms / 1e3) / 1e9, 1),
                               "graph_replays": engine.graph_replays}
        if b == batch:
            kernels = _kernel_times(decode_once)
            out[f"decode_b{b}"]["kernel_us"] = {k: round(v, 1) for k, v in list(kernels.items())[:10]}
            out[f"decode_b{b}"]["kernel_us_total"] = round(sum(kernels.values()), 1)
    for r in ids:
        engine.end_request(r)
    del engine
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------ kernels side by side
def kernel_pairs(s: Dict[str, int], peaks: Dict[str, Any], reps: int = 10) -> Dict[str, Any]:
    import torch

    from .csrc import ops
    from .parts.base import Workspace

    dev = "cuda:0"
    bf = torch.bfloat16
    H, G, d, W, V = s["heads"], s["kv_heads"], s["dim"], s["width"], s["vocab"]
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    P = 64
    out: Dict[str, Any] = {}

    def rotate(make: Callable[[], Any], nbytes: int) -> List[Any]:
        """Input sets whose total exceeds the L2 cache (126 MB) twice over."""
        return [make() for _ in range(max(2, -(-(256 << 20) // max(1, nbytes))))]

    def run(name: str, launch: Callable[[int], None], sets: int, nbytes: float = 0.0, flops: float = 0.0) -> None:
        """Time one launch per input set, recorded once into a CUDA graph and replayed: between
        events on the device, without the host's time to issue a launch (several of these
        kernels run for less than a Python call takes)."""
        for i in range(min(sets, 3)):
            launch(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(sets):
                launch(i)
        graph.replay()
        ms = _timed(graph.replay, reps) / sets
        row: Dict[str, Any] = {"us": round(ms * 1e3, 2)}
        if nbytes:
            row["gbs"] = round(nbytes / (ms / 1e3) / 1e9, 1)
            row["frac_of_measured_copy_peak"] = round(nbytes / (ms / 1e3) / hbm, 3)
        if flops:
            row["tflops"] = round(flops / (ms / 1e3) / 1e12, 1)
            row["frac_of_measured_bf16_peak"] = round(flops / (ms / 1e3) / tflops, 3)
        out[name] = row

    # ---- rows of a prompt portion: projection rows -> queries + cache ------------------
    T = 8192
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seg = torch.zeros(T, dtype=torch.int32, device=dev)
    pages_n = T // P
    table = torch.arange(1, pages_n + 1, dtype=torch.int32, device=dev).view(1, -1)
    qk_bytes = T * (H + G) * d * 2
    srcs = rotate(lambda: torch.randn(T, (H + G) * d, device=dev, dtype=bf), 2 * qk_bytes)
    q_out = torch.empty(T, H * d, device=dev, dtype=bf)
    key_pages = torch.zeros(pages_n + 1, G, P, d, device=dev, dtype=bf)
    run("key_store (queries x temperature, keys to pages)",
        lambda i: ops.key_store(srcs[i], q_out, key_pages, None, pos, seg, table, q_off=0, k_off=H * d,
                                num_heads=H, q_dim=d, num_kv_heads=G, k_dim=d, temp_coef=0.1, temp_every=512),
        len(srcs), nbytes=2 * qk_bytes)
    qkv_bytes = T * (H + 2 * G) * d * 2
    srcs3 = rotate(lambda: torch.randn(T, (H + 2 * G) * d, device=dev, dtype=bf), 2 * qkv_bytes)
    kv_pages = torch.zeros(2, pages_n + 1, G, P, d, device=dev, dtype=bf)
    qn = torch.ones(d, device=dev)
    cos_sin = torch.ones(T, d // 2, device=dev)
    run("qk_rope_store (per-head norm, rotary, keys and values to pages)",
        lambda i: ops.qk_rope_store(srcs3[i], q_out, kv_pages, qn, qn, cos_sin, pos, seg, table, H, G, d, d // 2,
                                    2, True, False, 1e-6),
        len(srcs3), nbytes=2 * qkv_bytes)
    R = s["rank"]
    lat_w = H * d + R + H
    lat_w += -lat_w % 8
    srcs_l = rotate(lambda: torch.randn(T, lat_w, device=dev, dtype=bf), T * lat_w * 2)
    lat_pages = torch.zeros(pages_n + 1, 1, P, R, device=dev, dtype=bf)
    wn = torch.ones(R, device=dev)
    run("key_store (latent: RMS norm, to pages)",
        lambda i: ops.key_store(srcs_l[i], None, lat_pages, wn, pos, seg, table, q_off=0, k_off=H * d, num_heads=H,
                                q_dim=d, num_kv_heads=1, k_dim=R, eps=1e-6),
        len(srcs_l), nbytes=2 * T * R * 2)
    del srcs, srcs3, srcs_l

    # ---- embedding ---------------------------------------------------------------------
    emb = torch.randn(V, W, device=dev, dtype=bf)
    ids = [torch.randint(0, V, (T,), device=dev, dtype=torch.int32) for _ in range(4)]
    res = torch.empty(T, W, device=dev, dtype=torch.float32)
    g = torch.ones(W, device=dev)
    emb_bytes = T * W * (2 + 4)
    run("embed_norm (gather + RMS norm)", lambda i: ops.embed_norm(ids[i], emb, g, res, 1e-6), 4, nbytes=emb_bytes)
    run("embed_gather", lambda i: ops.embed_gather(ids[i], emb, res), 4, nbytes=emb_bytes)
    mids = rotate(lambda: torch.randn(T, s["ff"], device=dev, dtype=bf), T * s["ff"] * 2)
    run("activation relu^2 (in place)", lambda i: ops.activation(mids[i], "relu2"), len(mids),
        nbytes=2 * T * s["ff"] * 2)
    del mids, emb, res

    # ---- decode attention: 64 requests x 2,048 keys ------------------------------------
    B, ctx = 64, 2048
    ws = Workspace(dev)
    per_req = ctx // P
    n_pages = B * per_req
    dpos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    dseg = torch.arange(B, dtype=torch.int32, device=dev)
    dtable = torch.arange(1, n_pages + 1, dtype=torch.int32, device=dev).view(B, per_req)

    def decode_case(name: str, heads: int, kv_heads: int, dim: int, shared: bool) -> None:
        plane = (n_pages + 1) * kv_heads * P * dim * 2
        one = B * ctx * kv_heads * dim * 2 * (1 if shared else 2)

        def make():
            if shared:
                t = torch.randn(n_pages + 1, kv_heads, P, dim, device=dev, dtype=bf)
                return t.unsqueeze(0).expand(2, *t.shape)
            return torch.randn(2, n_pages + 1, kv_heads, P, dim, device=dev, dtype=bf)
        caches = rotate(make, plane * (1 if shared else 2))
        q = torch.randn(B, heads * dim, device=dev, dtype=bf)
        o = torch.empty_like(q)
        run(name, lambda i: ops.attn_decode(q, o, caches[i], None, B, dpos, dseg, dtable, heads, kv_heads, dim,
                                            dim ** -0.5, None, ctx, ws), len(caches), nbytes=one)

    decode_case("attn_decode, keys are values (one plane)", H, G, d, True)
    decode_case("attn_decode, latent plane (one shared head)", H, 1, R, True)
    decode_case("attn_decode, keys and values (two planes)", H, G, d, False)
    decode_case("attn_decode, keys and values of one shared head (two planes)", H, 1, R, False)

    # ---- prefill attention: one 8,192-token prompt ---------------------------------------
    tiles = torch.arange(0, T, 64, dtype=torch.int32, device=dev)
    tile_seg = torch.zeros_like(tiles)
    seg_q = torch.tensor([0, T], dtype=torch.int32, device=dev)
    seg_p0 = torch.zeros(1, dtype=torch.int32, device=dev)

    def prefill_case(name: str, heads: int, kv_heads: int, dim: int, shared: bool) -> None:
        if shared:
            t = torch.randn(pages_n + 1, kv_heads, P, dim, device=dev, dtype=bf)
            cache = t.unsqueeze(0).expand(2, *t.shape)
        else:
            cache = torch.randn(2, pages_n + 1, kv_heads, P, dim, device=dev, dtype=bf)
        q = torch.randn(T, heads * dim, device=dev, dtype=bf)
        o = torch.empty_like(q)
        flops = 4.0 * heads * dim * T * (T + 1) / 2
        run(name, lambda i: ops.attn_prefill_tc(q, o, cache, tile_seg, tiles, seg_q, seg_p0, table, heads, kv_heads,
                                                dim, dim ** -0.5), 1, flops=flops)

    prefill_case("attn_prefill_tc, keys are values (one plane)", H, G, d, True)
    prefill_case("attn_prefill_tc, latent plane (one shared head)", H, 1, R, True)
    prefill_case("attn_prefill_tc, keys and values (two planes)", H, G, d, False)
    ops.check_tc_status(dev)
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
                        "fazinex": measure_model(fazinex_config(s), a),
                        "minimax_m3_equal_size": measure_model(minimax_config(s, room), a)}
        kernels = kernel_pairs(SIZES[names[0]], peaks)
    torch.cuda.synchronize()
    line = {"bench": "design", "design": "Fazinex", "beside": "MiniMax-M3 decoder at equal size",
            "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids", "layers": LAYERS,
            "context": a.context, "steps": a.steps, "warmup": max(3, a.warmup), "sizes": sizes,
            "kernels_at": names[0], "kernels": kernels,
            "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": peaks["source"]},
            "clocks": clocks.summary(), "wall_s": round(time.time() - t0, 1)}
    print(json.dumps(line))
    return 0
