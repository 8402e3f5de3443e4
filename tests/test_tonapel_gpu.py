"""Tonapel in the engine against the plain implementation: every new kernel alone, every
mechanism alone in a one-layer model, whole prompts against decoding, portions down to two
tokens, mixed batches with pages and state slots used again, a window's edge and a token far
back made decisive on purpose, the first tokens, long decoding, three configurations that
differ in every size, greedy generation through the scheduler, the trace replay tool."""

import copy

import pytest
import torch

import plain_tonapel as plain
import replay_driver as rd
import tonapel_tiny as tn

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 150, 66, 260, 21], "C": [2, 35, 77, 5]}
CUTS = {"whole": rd.whole, "decode_tail": rd.decode_tail, "portions": rd.portions, "mixed": rd.mixed}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def requests_of(which):
    vocab = tn.TN[which]["vocab"]
    return {f"r{i}": tn.tokens(30 * i + ord(which), n, vocab) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {which: tn.write_tiny(str(tmp_path_factory.mktemp(f"tn{which}")), which) for which in tn.TN}


def expected_for(config, state, reqs, dtype, routing=None):
    """The plain model's logits; in bfloat16 with the experts the engine chose (two correct
    implementations may choose differently where two router logits lie within rounding)."""
    out = {}
    for rid, toks in reqs.items():
        ids = routing[rid] if dtype == "bfloat16" and routing else None
        out[rid] = plain.forward(config, state, toks, expert_ids=ids)
    return out


def run_engine(engine, reqs, schedule, routing=None):
    """Drive ``engine.step`` through a schedule; logits of every position of every request.  With
    ``routing`` (a dict) the experts the engine chose are left there: ``routing[request][j]`` is
    ``[positions, top]`` of the j-th routed layer (layers may choose different numbers)."""
    from freetoken_b200.engine import StepEntry
    out = {rid: torch.full((len(t), engine.vocab_size), float("nan")) for rid, t in reqs.items()}
    for entries, ended in schedule:
        batch = [StepEntry(rid, reqs[rid][first:first + n], list(range(n))) for rid, first, n in entries]
        probe = {"router_ids": []} if routing is not None else None
        logits = engine.step(batch, probe=probe).float().cpu()
        row = 0
        for rid, first, n in entries:
            out[rid][first:first + n] = logits[row:row + n]
            if routing is not None:
                if rid not in routing:
                    routing[rid] = [torch.full((len(reqs[rid]), x.shape[1]), -1, dtype=torch.long)
                                    for x in probe["router_ids"]]
                for j, x in enumerate(probe["router_ids"]):
                    routing[rid][j][first:first + n] = x[row:row + n].cpu().long()
            row += n
        for rid in ended:
            engine.end_request(rid)
    engine.cache.check_integrity()
    return out


def run_and_compare(folder, config, state, reqs, schedule, dtype, page, what, tol=None, poison=True):
    engine = tn.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=poison)
    routing = {} if tn.routed_layers(config) else None
    got = run_engine(engine, reqs, schedule, routing)
    want = expected_for(config, state, reqs, dtype, routing)
    tn.compare(got, want, tol or tn.TOL[dtype], f"{what} [{dtype}]")
    assert engine.cache.free_pages() == engine.cache.total_pages()
    return got


# ------------------------------------------------------------------ kernels, each alone
def segments(lens, slots):
    """Step metadata of segments of ``lens`` tokens in state slots ``slots``."""
    q = [0]
    for n in lens:
        q.append(q[-1] + n)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    return seg, torch.tensor(slots, dtype=torch.int32).cuda(), torch.tensor(q, dtype=torch.int32).cuda()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("taps,bias", [(1, True), (2, False), (4, True), (5, False), (11, True)])
def test_conv_silu_carries_its_inputs(dtype, taps, bias):
    """Two requests fed in segments of 1 to 9 tokens that interleave, in slots 2 and 0 of rows that
    are wider than the convolution's state: every output equals the convolution over the whole
    sequence, and nothing outside the state's columns is touched."""
    from freetoken_b200.csrc import ops
    torch.manual_seed(taps)
    C, n = 37, 26
    u = {r: torch.randn(n, C).to(DTYPES[dtype]) for r in ("a", "b")}
    w = torch.randn(C, taps)
    b = torch.randn(C) if bias else None
    want = {r: plain.silu(plain.causal_conv(u[r].double(), w.double(), None if b is None else b.double())) for r in u}
    state = torch.zeros(4, (taps - 1) * C + 5, device="cuda")
    state[:, (taps - 1) * C:] = 7.0
    at = {"a": 0, "b": 0}
    got = {r: [] for r in u}
    for step, cut in enumerate([(1, 3), (2, 1), (9, 2), (1, 1), (5, 9), (8, 10)]):
        order = ("a", "b") if step % 2 == 0 else ("b", "a")
        lens = [cut[0] if r == "a" else cut[1] for r in order]
        x = torch.cat([u[r][at[r]:at[r] + n_] for r, n_ in zip(order, lens)])
        wide = torch.zeros(x.shape[0], C + 6, dtype=x.dtype)
        wide[:, 3:3 + C] = x                                           # a column range of a wider matrix
        seg, slot, q = segments(lens, [2 if r == "a" else 0 for r in order])
        out = torch.empty(x.shape[0], C, dtype=x.dtype, device="cuda")
        ops.conv_silu(wide.cuda()[:, 3:3 + C], out, w.cuda(), None if b is None else b.cuda(),
                      state[:, :(taps - 1) * C], seg, slot, q)
        o = out.cpu()
        for r, n_ in zip(order, lens):
            got[r].append(o[:n_])
            o = o[n_:]
            at[r] += n_
    tol = 1e-5 if dtype == "float32" else 2e-2
    for r in u:
        assert torch.allclose(torch.cat(got[r]).double(), want[r], atol=tol, rtol=tol), r
    assert torch.all(state[:, (taps - 1) * C:] == 7.0) and torch.all(state[[1, 3], :(taps - 1) * C] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads,P,N,G", [(3, 10, 12, 1), (4, 40, 70, 2), (2, 64, 128, 1), (4, 5, 200, 4)])
def test_ssd_scan_in_segments(dtype, heads, P, N, G):
    from freetoken_b200.csrc import ops
    torch.manual_seed(N)
    T = 45
    inner = heads * P
    xbc = (torch.randn(T, inner + 2 * G * N) * 0.7).to(DTYPES[dtype])
    dt = torch.randn(T, heads).to(DTYPES[dtype])
    dt_bias, a_log, d = torch.randn(heads) * 0.5 - 0.5, torch.randn(heads) * 0.5 - 0.5, torch.randn(heads)
    x64 = xbc.double()
    want = plain.ssd_recurrence(x64[:, :inner].view(T, heads, P), x64[:, inner:inner + G * N].view(T, G, N),
                                x64[:, inner + G * N:].view(T, G, N), dt.double(), dt_bias.double(),
                                a_log.double(), d.double()).reshape(T, inner)
    state = torch.zeros(3, heads * N * P + 3, device="cuda")
    got, at = [], 0
    for n in (1, 17, 2, 1, 16, 8):          # a chunk of the kernel is 16 tokens: below, at and above it
        seg, slot, q = segments([n], [1])
        y = torch.empty(n, inner, device="cuda")
        ops.ssd_scan(xbc[at:at + n].cuda(), dt[at:at + n].cuda(), dt_bias.cuda(), a_log.cuda(), d.cuda(),
                     state[:, 3:], y, slot, q, heads, P, N, G)
        got.append(y.cpu())
        at += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-3, rtol=3e-4)
    assert torch.all(state[[0, 2]] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads,G,D,P", [(4, 2, 12, 10), (2, 2, 40, 36), (4, 1, 128, 64), (3, 3, 8, 70), (2, 1, 200, 16)])
def test_delta_scan_in_segments(dtype, heads, G, D, P):
    from freetoken_b200.csrc import ops
    torch.manual_seed(D)
    T = 45
    qkv = torch.randn(T, 2 * G * D + heads * P).to(DTYPES[dtype])
    gates = torch.randn(T, 2 * heads + 1).to(DTYPES[dtype])
    dt_bias, a_log = torch.randn(heads) * 0.5 - 0.5, torch.randn(heads) * 0.5 - 1.0
    x64 = qkv.double()
    want = plain.delta_recurrence(x64[:, :G * D].view(T, G, D), x64[:, G * D:2 * G * D].view(T, G, D),
                                  x64[:, 2 * G * D:].view(T, heads, P), gates[:, :heads].double(),
                                  gates[:, heads:2 * heads].double(), dt_bias.double(), a_log.double()
                                  ).reshape(T, heads * P)
    state = torch.zeros(2, heads * D * P, device="cuda")
    got, at = [], 0
    for n in (2, 1, 16, 17, 1, 8):
        seg, slot, q = segments([n], [0])
        o = torch.empty(n, heads * P, device="cuda")
        gd = gates[at:at + n].cuda()
        ops.delta_scan(qkv[at:at + n].cuda(), gd[:, :heads], gd[:, heads:2 * heads], dt_bias.cuda(), a_log.cuda(),
                       state, o, slot, q, heads, G, D, P, 1e-6, D ** -0.5)
        got.append(o.cpu())
        at += n
    assert torch.allclose(torch.cat(got).double(), want, atol=2e-5, rtol=2e-4)
    assert torch.all(state[1] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("width,cases", [
    (60, ((4, 60, True), (1, 60, True), (5, 12, False))),            # parts of 15, 60, 12 values: a warp each
    (1536, ((1, 1536, True), (12, 128, False), (3, 1536, True))),    # a block a part; a warp a part
    (4100, ((1, 4100, True), (5, 820, False))),                      # rows kept in 16 pieces a thread
    (9004, ((1, 9004, True),)),                                      # longer than a thread block keeps
    (90, ((2, 45, False),)),                                         # an odd part: one value at a time
])
def test_gated_norm_both_orders(dtype, width, cases):
    from freetoken_b200.csrc import ops
    torch.manual_seed(5)
    T = 7
    y = torch.randn(T, width, device="cuda") * 3
    z = torch.randn(T, width + 8).to(DTYPES[dtype]).cuda()
    tol = 1e-5 if dtype == "float32" else 2e-2
    for groups, wlen, first in cases:
        w = (torch.rand(wlen) + 0.5).cuda()
        out = torch.empty(T, width, dtype=DTYPES[dtype], device="cuda")
        ops.gated_norm(y, z[:, 8:], w, out, groups, 1e-3, first)
        gate = plain.silu(z[:, 8:].double().cpu())
        v = y.double().cpu() * gate if first else y.double().cpu()
        v = plain.rms(v.view(T, groups, width // groups), 1e-3).reshape(T, width) * w.double().cpu().repeat(width // wlen)
        want = v if first else v * gate
        assert torch.allclose(out.double().cpu(), want, atol=tol, rtol=tol), (groups, first)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H", [44, 45, 2048 + 8])          # 16-byte pieces; one value at a time; several pieces a thread
def test_norm_add_scaled_sum_bias_glu(dtype, H):
    from freetoken_b200.csrc import ops
    torch.manual_seed(6)
    T, k = 5, 3
    tol = 1e-5 if dtype == "float32" else 2e-2
    branch = torch.randn(T, k, H).to(DTYPES[dtype]).cuda()
    res = torch.randn(T, H, device="cuda")
    w, w2 = (torch.randn(H) * 0.2).cuda(), (torch.randn(H) * 0.2).cuda()
    z = branch.double().cpu().sum(1)
    want_res = res.double().cpu() + 0.6 * plain.norm(z, w.double().cpu(), 1e-4)
    want_next = plain.norm(want_res, w2.double().cpu(), 1e-2)
    out = torch.empty(T, H, dtype=DTYPES[dtype], device="cuda")
    ops.norm_add(branch, res, w, 1e-4, True, 0.6, next_weight=w2, next_eps=1e-2, next_plus_one=True, next_out=out)
    assert torch.allclose(res.double().cpu(), want_res, atol=1e-5, rtol=1e-5)       # the residual is float32
    assert torch.allclose(out.double().cpu(), want_next, atol=tol, rtol=tol)
    res2 = torch.zeros(T, H, device="cuda")
    ops.norm_add(branch[:, 0].contiguous(), res2, w, 1e-4, False, 1.0)
    assert torch.allclose(res2.double().cpu(), plain.rms(branch[:, 0].double().cpu(), 1e-4) * w.double().cpu(),
                          atol=1e-5, rtol=1e-5)
    scale = torch.tensor([0.8, -1.5, 0.25]).cuda()
    ops.scaled_sum(branch, scale, out)
    assert torch.allclose(out.double().cpu(), (branch.double().cpu() * scale.double().cpu()[None, :, None]).sum(1),
                          atol=tol, rtol=tol)
    wide = torch.randn(T, H + 8).to(DTYPES[dtype]).cuda()
    before = wide.clone()
    bias = torch.randn(H).cuda()
    ops.bias_add(wide[:, 8:], bias)
    assert torch.allclose(wide[:, 8:].double().cpu(), before[:, 8:].double().cpu() + bias.double().cpu(), atol=tol, rtol=tol)
    assert torch.equal(wide[:, :8], before[:, :8])
    gu = torch.randn(T, 2 * 22).to(DTYPES[dtype]).cuda()
    mid = torch.empty(T, 22, dtype=DTYPES[dtype], device="cuda")
    ops.glu_rows(gu, mid, "gelu_tanh")
    want = plain.gelu_tanh(gu[:, :22].double().cpu()) * gu[:, 22:].double().cpu()
    assert torch.allclose(mid.double().cpu(), want, atol=tol, rtol=tol)


# ------------------------------------------------------------------- mechanisms, each alone
ALONE = {
    "window_attention": tn.one_layer(tn.parallel(tn.left(6, 3, 8, 8, 5, 4), tn.right(1, 4, 4, 1, 2, 1), 1.0, 0.0)),
    "window_attention_wider_values_one_key_head":
        tn.one_layer(tn.parallel(tn.left(4, 1, 12, 28, 9, 12, base=50.0), tn.right(1, 4, 4, 1, 2, 1), 1.7, 0.0)),
    "window_attention_wider_keys": tn.one_layer(tn.parallel(tn.left(2, 2, 20, 6, 300, 8), tn.right(1, 4, 4, 1, 2, 1), 1.0, 0.0)),
    "state_space": tn.one_layer(tn.parallel(tn.left(1, 1, 4, 4, 2, 2), tn.right(4, 10, 20, 2, 4, 2), 0.0, 1.0)),
    "state_space_one_group_wide_state": tn.one_layer(tn.parallel(tn.left(1, 1, 4, 4, 2, 2), tn.right(2, 33, 150, 1, 3, 1), 0.0, 0.7)),
    "both_halves": tn.one_layer(tn.parallel(tn.left(2, 1, 16, 16, 6, 8), tn.right(2, 8, 16, 1, 4, 1), 0.4, 1.6), mult=0.5),
    "delta": tn.one_layer(tn.delta(4, 2, 12, 10, 3)),
    "delta_one_key_head_no_memory_of_inputs": tn.one_layer(tn.delta(3, 1, 40, 7, 1)),
    "dense_feed_forward": tn.one_layer(tn.delta(1, 1, 4, 4, 2, tn.dense(40)), mult=0.5),
    "routed_feed_forward": tn.one_layer(tn.delta(1, 1, 4, 4, 2, tn.moe(7, 3, 16, 0.6))),
    "routed_feed_forward_top_one": tn.one_layer(tn.delta(1, 1, 4, 4, 2, tn.moe(4, 1, 16, 50.0))),
}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("what", list(ALONE))
def test_one_mechanism_alone(tmp_path, what, dtype):
    config = ALONE[what]
    state = tn.random_state(config, 31)
    folder = tn.write_model(str(tmp_path / "m"), config, tn.as_file(state))
    reqs = {"a": tn.tokens(1, 41, 90), "b": tn.tokens(2, 3, 90), "c": tn.tokens(3, 1, 90)}
    for cut in ("whole", "portions", "decode_tail"):
        run_and_compare(folder, config, state, reqs, CUTS[cut](reqs), dtype, 8, f"{what}, {cut}")


# --------------------------------------------------------------- whole models, every cut
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", list(tn.TN))
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(models, which, dtype, cut):
    """Exactly as many pages as the schedule's peak needs and (mixed) four slots for five requests:
    pages and state slots are used again; free pages hold NaN."""
    reqs = requests_of(which)
    state = tn.random_state(tn.TN[which], tn.SEEDS[which])
    run_and_compare(models[which], tn.TN[which], state, reqs, CUTS[cut](reqs), dtype, tn.PAGE[which], f"{which} {cut}")


def test_fast_attention_kernels_take_the_windows(models, monkeypatch):
    """Configuration B in bfloat16 (heads of 32, 64 and 128): decoded tokens take the split-KV
    tensor-core kernel, prompt portions the tiled one, both with windows."""
    from freetoken_b200.csrc import ops
    calls = {"prefill": 0, "decode": 0}
    real_p, real_d = ops.attn_prefill, ops.attn_decode
    monkeypatch.setattr(ops, "attn_prefill", lambda *a, **k: (calls.__setitem__("prefill", 1), real_p(*a, **k))[1])
    monkeypatch.setattr(ops, "attn_decode", lambda *a, **k: (calls.__setitem__("decode", 1), real_d(*a, **k))[1])
    reqs = requests_of("B")
    state = tn.random_state(tn.TN["B"], tn.SEEDS["B"])
    run_and_compare(models["B"], tn.TN["B"], state, reqs, rd.mixed(reqs), "bfloat16", 64, "B mixed, fast kernels")
    assert calls == {"prefill": 1, "decode": 1}


@pytest.mark.parametrize("which", ["A", "C"])
def test_float32_cuts_agree_bitwise(models, which):
    """In float32 the logits at a position depend neither on the cut nor on the batch: every
    token runs the same operations in the same order whatever else the step holds."""
    reqs = requests_of(which)
    results = {}
    for cut, fn in CUTS.items():
        schedule = fn(reqs)
        engine = tn.make_engine(models[which], "float32", tn.PAGE[which], rd.peak_tokens(schedule, tn.PAGE[which]))
        results[cut] = run_engine(engine, reqs, schedule)
    for cut in ("decode_tail", "portions", "mixed"):
        for rid in reqs:
            assert torch.equal(results[cut][rid], results["whole"][rid]), (cut, rid)


# ------------------------------------------------------------ a window's edge, sharp on purpose
def sharpen_left(config, state, asker, target, beta):
    """Rewrite the first layer's query projection so that token ``asker``'s query is ``beta`` times
    token ``target``'s key in every head (rotation off, biases of q and k zero): wherever
    ``target`` stands inside the window, ``asker`` puts nearly all its weight there."""
    a = config["layers"][0]["mixer"]["left"]
    H, G, d = a["heads"], a["kv_heads"], a["dim"]
    h = plain.norm(state["embed"][[asker, target]], state["l0.norm1"], config["norm"]["eps"])
    k = (state["l0.mix.left.k"] @ h[1]).view(G, d).repeat_interleave(H // G, dim=0)
    q = state["l0.mix.left.q"]
    q = q - (q @ h[0])[:, None] * h[0][None, :] / h[0].dot(h[0])
    q = q + beta * k.reshape(H * d, 1) * h[0][None, :] / h[0].dot(h[0])
    state["l0.mix.left.q"] = q.to(torch.bfloat16).double()
    state["l0.mix.left.q.b"].zero_()
    state["l0.mix.left.k.b"].zero_()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("dim,vdim,page,window", [(16, 24, 8, 24), (64, 64, 64, 70), (32, 32, 64, 64), (128, 128, 64, 129)])
def test_a_window_edge_decides(tmp_path, dim, vdim, page, window, dtype):
    """The asking token finds its target ``window - 1`` tokens back and must not find it ``window``
    back, inside a prompt portion and as a decoded token; windows shorter than, equal to and
    longer than a page; pages the window has passed are given back while the requests run (sizes
    16/24: the generic kernel, the others the tensor-core kernels in bfloat16)."""
    layer = tn.parallel(tn.left(2, 1, dim, vdim, window, 0, scale=0.25), tn.right(1, 4, 4, 1, 2, 1), 1.0, 0.05)
    config = tn.one_layer(layer, vocab=120, width=48)
    state = tn.random_state(config, 41)
    asker, target = 7, 11
    sharpen_left(config, state, asker, target, beta=128.0 / dim)
    n = 330
    reqs = {}
    for name, back in (("inside", window - 1), ("outside", window), ("next_to", 1), ("far_outside", 2 * window + 3)):
        toks = [t if t not in (asker, target) else 13 for t in tn.tokens(60 + back, n, 120)]
        for at in (n - 40, n - 1):            # asked from a prompt portion and by the last decoded token
            toks[at] = asker
            toks[at - back] = target
        reqs[name] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    blind = [t if t != target else 13 for t in reqs["inside"]]
    assert float(tn.position_errors(plain.forward(config, state, blind)[-1:], want["inside"][-1:])) > 0.2
    folder = tn.write_model(str(tmp_path / "m"), config, tn.as_file(state))
    tol = tn.TOL[dtype] * (1 if dtype == "float32" else 2)      # a sharp softmax: rounding of scores counts more
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = tn.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        tn.compare(run_engine(engine, reqs, schedule), want, tol, f"window {window}, {cut} [{dtype}]")
        assert engine.cache.free_pages() == engine.cache.total_pages()


# ------------------------------------------------------- a token far back, through the state
def only_the_target_writes(config, state, target, kind):
    """Rewrite the projection that sets how much a token writes into the state (the step size of
    the state space, the write strength of the delta rule) so that every token of the vocabulary
    writes next to nothing and ``target`` writes fully.  The vocabulary is smaller than the width,
    so a row with the wanted product for every token exists."""
    h = plain.norm(state["embed"], state["l0.norm1"], config["norm"]["eps"])            # [vocab, width]
    # (the delta rule's read-out is normed: a state that is all but empty would make the norm's
    # eps count, so its other tokens still write a little)
    y = torch.full((h.shape[0],), -7.0 if kind == "state_space" else -4.0, dtype=torch.float64)
    y[target] = 3.0
    row = torch.linalg.lstsq(h, y[:, None]).solution[:, 0]
    if kind == "state_space":
        r = config["layers"][0]["mixer"]["right"]
        w = state["l0.mix.right.in"]
        w[w.shape[0] - r["heads"]:] = row
        state["l0.mix.right.in"] = w.to(torch.bfloat16).double()
        state["l0.mix.right.dt_bias"].zero_()
    else:
        heads = config["layers"][0]["mixer"]["heads"]
        state["l0.mix.b"] = row.repeat(heads, 1).to(torch.bfloat16).double()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind", ["state_space", "delta"])
def test_a_far_token_reaches_through_the_state(tmp_path, kind, dtype):
    """States that forget slowly, and only one token that writes into them: it stands once, 250 to
    300 positions back - right before, on and right after a page border, and first of all - and
    reaches the last tokens only through the state carried from step to step.  Another token in
    its place changes their logits wholly."""
    if kind == "state_space":
        layer = tn.parallel(tn.left(1, 1, 4, 4, 3, 2), tn.right(3, 12, 24, 1, 3, 1), 0.05, 1.0)
    else:
        layer = tn.delta(3, 1, 24, 12, 3)
    config = tn.one_layer(layer, vocab=40, width=48)
    state = tn.random_state(config, 51, slow_decay=True)
    target, stand_in = 5, 6
    only_the_target_writes(config, state, target, kind)
    page, n = 16, 300
    reqs = {}
    for place in (15, 16, 17, 0, 49):
        toks = [t if t != target else stand_in for t in tn.tokens(70 + place, n, 40)]
        toks[place] = target
        reqs[f"t{place}"] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    other = list(reqs["t16"])
    other[16] = stand_in
    assert float(tn.position_errors(plain.forward(config, state, other)[-1:], want["t16"][-1:])) > 0.3
    folder = tn.write_model(str(tmp_path / "m"), config, tn.as_file(state))
    for cut in ("decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = tn.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        tn.compare(run_engine(engine, reqs, schedule), want, tn.TOL[dtype], f"far token, {kind}, {cut} [{dtype}]")


# --------------------------------------------------------- first tokens, long decoding
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_first_tokens_and_long_decoding(models, dtype):
    """A request that starts with a single token and is decoded one token at a time for 200 steps
    (windows pass, pages go back, decode steps are replayed from a graph in bfloat16), beside a
    second request that joins later two tokens a step; against the whole sequences."""
    from freetoken_b200.engine import StepEntry
    config = tn.TN["A"]
    state = tn.random_state(config, tn.SEEDS["A"])
    a, b = tn.tokens(5, 201, config["vocab"]), tn.tokens(6, 120, config["vocab"])
    engine = tn.make_engine(models["A"], dtype, 4, 204 + 120)
    got_a, got_b = [], []
    routed = len(tn.routed_layers(config))
    ids_a, ids_b = [], []
    for i in range(len(a)):
        entries = [StepEntry("a", [a[i]], [0])]
        j = i - 60
        if 0 <= j < len(b) // 2:
            entries.append(StepEntry("b", b[2 * j:2 * j + 2], [0, 1]))
        probe = {"router_ids": []}
        logits = engine.step(entries, probe=probe).float().cpu()
        got_a.append(logits[0])
        got_b.extend(logits[1:])
        ids_a.append([x[0].cpu().long() for x in probe["router_ids"]])
        if len(entries) > 1:
            ids_b.extend([x[r].cpu().long() for x in probe["router_ids"]] for r in (1, 2))
    assert routed == len(ids_a[0])
    want = {}
    for rid, toks, ids in (("a", a, ids_a), ("b", b, ids_b)):
        chosen = [torch.stack([step[j] for step in ids]) for j in range(routed)]     # per routed layer [T, top]
        want[rid] = plain.forward(config, state, toks, expert_ids=chosen if dtype == "bfloat16" else None)
    tn.compare({"a": torch.stack(got_a), "b": torch.stack(got_b)}, want, tn.TOL[dtype], f"long decoding [{dtype}]")


# ------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_scheduler(models, which, dtype):
    """``LLM.generate`` (scheduler, overlapped steps, graph replay of decode steps in bfloat16):
    every generated token is the plain model's own greedy choice for the sequence so far, unless
    its two best logits lie within rounding of each other."""
    from freetoken_b200 import LLM, SamplingParams
    config = tn.TN[which]
    state = tn.random_state(config, tn.SEEDS[which])
    llm = LLM(models[which], dtype, page_size=tn.PAGE[which], num_token_override=1024, max_running_req=3,
              max_extend_tokens=24)
    prompts = [tn.tokens(70 + i, n, config["vocab"]) for i, n in enumerate((3, 30, 11, 1, 47))]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    tie = 1e-4 if dtype == "float32" else 8e-2
    route_tie = 5e-2         # bfloat16: two router logits this close may be chosen the other way round
    ties = 0
    for prompt, result in zip(prompts, out):
        seq = list(prompt)
        assert len(result["token_ids"]) == 12
        for token in result["token_ids"]:
            margins = []
            logits = plain.forward(config, state, seq, margins=margins)[-1]
            if token != int(logits.argmax()):
                margin = min((float(m.min()) for m in margins), default=float("inf"))
                close = float(logits.max() - logits[token]) < tie or (dtype == "bfloat16" and margin < route_tie)
                assert close, (dtype, len(seq), token, int(logits.argmax()), float(logits.max() - logits[token]), margin)
                ties += 1
                if margin < route_tie:
                    break            # another expert somewhere in the sequence: what follows is another sequence
            seq.append(int(token))
    assert ties == 0 if dtype == "float32" else ties <= 4
    if dtype == "bfloat16":
        assert llm.engine.graph_replays > 0


# -------------------------------------------------------------------- the replay tool
def test_trace_replay_tool(models, tmp_path):
    """``bin/trace_run`` on a Tonapel folder: a mixed schedule with exactly the pages its peak needs."""
    which = "C"
    reqs = requests_of(which)
    state = tn.random_state(tn.TN[which], tn.SEEDS[which])
    schedule = rd.mixed(reqs)
    page = tn.PAGE[which]
    got = rd.run_trace_tool(models[which], "float32", reqs, schedule, str(tmp_path / "out"),
                            rd.peak_tokens(schedule, page), page, tn.TN[which]["vocab"])
    tn.compare(got, expected_for(tn.TN[which], state, reqs, "float32"), tn.TOL["float32"], "trace_run, mixed")
