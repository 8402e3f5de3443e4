"""Fazinex in the engine against the plain implementation: every kernel of its own alone,
every mixer alone, whole prompts against decoding, portions down to two tokens, mixed
batches with pages and slots used again, far keys and page borders with attention made
sharp on purpose, the first tokens, long decoding, three configurations that differ in
every size, greedy generation through the scheduler."""

import copy
import math

import pytest
import torch

import fazinex_tiny as fz
import plain_fazinex as plain
import replay_driver as rd

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 150, 66, 260, 21], "C": [2, 35, 77, 5]}
CUTS = {"whole": rd.whole, "decode_tail": rd.decode_tail, "portions": rd.portions, "mixed": rd.mixed}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def requests_of(which):
    vocab = fz.FZ[which]["vocab"]
    return {f"r{i}": fz.tokens(50 * i + len(which) + ord(which), n, vocab) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {which: fz.write_tiny(str(tmp_path_factory.mktemp(f"fz{which}")), which) for which in fz.FZ}


@pytest.fixture(scope="module")
def expected():
    cache = {}

    def get(which):
        if which not in cache:
            state = plain.random_state(fz.FZ[which], fz.SEEDS[which])
            cache[which] = {rid: plain.forward(fz.FZ[which], state, toks) for rid, toks in requests_of(which).items()}
        return cache[which]
    return get


# ------------------------------------------------------------------ kernels, each alone
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_embed_norm_kernel(dtype):
    from freetoken_b200.csrc import ops
    torch.manual_seed(1)
    table = torch.randn(50, 36).to(DTYPES[dtype]).cuda()
    g = (torch.rand(36) + 0.5).cuda()
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32).cuda()
    out = torch.empty(5, 36, device="cuda")
    ops.embed_norm(ids, table, g, out, 1e-3)
    want = plain.rms_norm(table.double().cpu()[ids.cpu().long()], g.double().cpu(), 1e-3)
    assert torch.allclose(out.cpu().double(), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("every,coef", [(1, 0.7), (4, 0.5), (48, 0.35), (5, 0.0)])
def test_key_store_temperature_and_pages(every, coef):
    """Queries times the temperature of their position - every position around every multiple
    of the period - and keys into the page and row of their position, two requests whose
    pages interleave."""
    from freetoken_b200.csrc import ops
    torch.manual_seed(2)
    H, G, d, P = 3, 2, 6, 4
    lens, starts = [70, 9], [0, 131]                    # the second request continues at 131
    T = sum(lens)
    src = torch.randn(T, 5 + (H + G) * d, device="cuda")      # rows wider than q | k, q at column 5
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int().cuda()
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    width = 40
    table = torch.zeros(2, width, dtype=torch.int32)
    table[0] = torch.arange(1, 2 * width, 2)            # request 0: odd pages, request 1: even pages
    table[1] = torch.arange(2, 2 * width + 1, 2)
    pages = torch.zeros(2 * width + 2, G, P, d, device="cuda")
    q_out = torch.empty(T, H * d, device="cuda")
    ops.key_store(src, q_out, pages, None, pos, seg, table.cuda(), q_off=5, k_off=5 + H * d, num_heads=H,
                  q_dim=d, num_kv_heads=G, k_dim=d, temp_coef=coef, temp_every=every)
    temp = plain.query_temperature(pos.cpu().long(), coef, every)
    want_q = src[:, 5:5 + H * d].cpu().double() * temp[:, None]
    assert torch.allclose(q_out.cpu().double(), want_q, atol=1e-6, rtol=2e-6)
    k = src[:, 5 + H * d:].cpu().view(T, G, d)
    seen = torch.zeros_like(pages.cpu())
    for t in range(T):
        p, s = int(pos[t]), int(seg[t])
        seen[table[s, p // P], :, p % P] = k[t]
    assert torch.equal(pages.cpu(), seen)               # nothing else was written, page 0 included


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_key_store_norms_the_latent(dtype):
    from freetoken_b200.csrc import ops
    torch.manual_seed(3)
    T, R, P = 11, 20, 4
    src = (torch.randn(T, 7 + R) * 3).to(DTYPES[dtype]).cuda()
    w = (torch.rand(R) + 0.5).cuda()
    pos = torch.arange(T).int().cuda()
    seg = torch.zeros(T, dtype=torch.int32).cuda()
    table = torch.tensor([[2, 1, 3]], dtype=torch.int32).cuda()
    pages = torch.zeros(4, 1, P, R, dtype=DTYPES[dtype], device="cuda")
    ops.key_store(src, None, pages, w, pos, seg, table, q_off=0, k_off=7, num_heads=1, q_dim=7,
                  num_kv_heads=1, k_dim=R, eps=1e-2)
    want = plain.rms_norm(src[:, 7:].double().cpu(), w.double().cpu(), 1e-2)
    got = torch.stack([pages[int(table[0, t // P]), 0, t % P] for t in range(T)]).double().cpu()
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol)


def test_gate_activation_softcap_kernels():
    from freetoken_b200.csrc import ops
    torch.manual_seed(4)
    T, H, d = 9, 3, 10
    o = torch.randn(T, H * d, device="cuda")
    z = torch.randn(T, 4 + H, device="cuda") * 3
    want = (o.cpu().double().view(T, H, d) * torch.sigmoid(z[:, 4:].cpu().double())[:, :, None]).view(T, H * d)
    ops.gate_heads(o, z[:, 4:], H, d)
    assert torch.allclose(o.cpu().double(), want, atol=1e-6)
    ob = torch.randn(T, H * 16, device="cuda").to(torch.bfloat16)        # 16-byte pieces of a head
    zb = (torch.randn(T, 4 + H, device="cuda") * 3).to(torch.bfloat16)
    want = (ob.float().cpu().double().view(T, H, 16) * torch.sigmoid(zb[:, 4:].float().cpu().double())[:, :, None])
    ops.gate_heads(ob, zb[:, 4:], H, 16)
    assert torch.allclose(ob.float().cpu().double(), want.view(T, H * 16), atol=1e-2, rtol=1e-2)
    x = torch.linspace(-6, 6, 203, device="cuda")
    for kind, f in (("relu2", lambda v: torch.relu(v) ** 2),
                    ("gelu_tanh", lambda v: 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))),
                    ("silu", lambda v: v * torch.sigmoid(v))):
        y = x.clone()
        ops.activation(y, kind)
        assert torch.allclose(y.cpu().double(), f(x.cpu().double()), atol=1e-5), kind
        yb = x.to(torch.bfloat16)[:200].clone()          # the 8-at-a-time bfloat16 form
        ops.activation(yb, kind)
        assert torch.allclose(yb.float().cpu().double(), f(x.to(torch.bfloat16)[:200].float().cpu().double()),
                              atol=1e-2, rtol=1e-2), kind
    logits = torch.linspace(-80, 80, 101, device="cuda").view(1, -1).contiguous()
    want = 12 * torch.tanh(logits.cpu().double() / 12)
    ops.softcap(logits, 12.0)
    assert torch.allclose(logits.cpu().double(), want, atol=1e-5)


@pytest.mark.parametrize("rows", [1, 8, 20])
@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
def test_activation_in_the_weight_streaming_product(rows, kind):
    """Few rows (decode): the up projection's activation is the product's epilogue, applied to
    the float32 accumulator; more rows take the library product and the activation kernel."""
    from freetoken_b200.parts import linear
    torch.manual_seed(6)
    K, N = 64, 40
    x = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.3).to(torch.bfloat16)
    f = {"relu2": lambda v: torch.relu(v) ** 2, "silu": lambda v: v * torch.sigmoid(v),
         "gelu_tanh": lambda v: 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))}[kind]
    want = f(x.float().cpu().double() @ w.float().cpu().double().T)
    for r in (rows, rows + 40):
        xx = x.repeat(-(-r // rows), 1)[:r].contiguous()
        out = torch.empty(r, N, device="cuda", dtype=torch.bfloat16)
        linear.linear(xx, w, out, activation=kind)
        ref = want.repeat(-(-r // rows), 1)[:r]
        assert torch.allclose(out.float().cpu().double(), ref, atol=3e-2, rtol=2e-2), (kind, r)


@pytest.mark.parametrize("T", [1, 5, 130])
def test_gemm_heads(T):
    """One product per head, on views with row strides of their own (both tile shapes)."""
    from freetoken_b200.csrc import ops
    torch.manual_seed(5)
    H, K, N = 3, 32, 20
    wide = torch.randn(T, 7 + H * K + 3, device="cuda")
    a = wide[:, 7:7 + H * K].view(T, H, K)
    w = torch.randn(H, N, K, device="cuda")
    c = torch.zeros(T, H * N, device="cuda")
    ops.gemm_heads(a, w, c.view(T, H, N))
    want = torch.einsum("thk,hnk->thn", a.cpu().double(), w.cpu().double()).reshape(T, H * N)
    assert torch.allclose(c.cpu().double(), want, atol=1e-4, rtol=1e-5)


# ------------------------------------------------------------------- mixers, each alone
def one_layer(layer, **top):
    cfg = {"architecture": "Fazinex", "vocab": 90, "width": 48, "norm": {"eps": 1e-6}, "layers": [layer]}
    cfg.update(top)
    return cfg


ALONE = {
    "attention": one_layer(fz.attn(6, 3, 8, 0.5, coef=0.9, every=2)),
    "attention_no_temperature_one_key_head": one_layer(fz.attn(4, 1, 12, 0.4)),
    "latent": one_layer(fz.latent(3, 8, 12, 20, 0.5)),
    "latent_wider_than_any_head": one_layer(fz.latent(2, 8, 8, 320, 0.3)),
    "feed_forward_beside_a_mixer": one_layer(fz.attn(1, 1, 8, 0.1, ff=40), logit_softcap=5.0),
}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("what", list(ALONE))
def test_one_mechanism_alone(tmp_path, what, dtype):
    config = ALONE[what]
    state = plain.random_state(config, 21)
    folder = fz.write_model(str(tmp_path / "m"), config, state)
    reqs = {"a": fz.tokens(1, 41, 90), "b": fz.tokens(2, 3, 90)}
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    for cut in ("whole", "portions"):
        schedule = CUTS[cut](reqs)
        engine = fz.make_engine(folder, dtype, 8, rd.peak_tokens(schedule, 8))
        fz.compare(rd.run_engine(engine, reqs, schedule), want, fz.TOL[dtype], f"{what}, {cut}")


# --------------------------------------------------------------- whole models, every cut
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", list(fz.FZ))
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(models, expected, which, dtype, cut):
    reqs = requests_of(which)
    schedule = CUTS[cut](reqs)
    page = fz.PAGE[which]
    # exactly as many pages as the schedule's peak needs, and (mixed) four slots for five
    # requests: pages and slots are used again
    engine = fz.make_engine(models[which], dtype, page, rd.peak_tokens(schedule, page), poison=True)
    fz.compare(rd.run_engine(engine, reqs, schedule), expected(which), fz.TOL[dtype], f"{which} {cut} [{dtype}]")
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_tensor_core_attention_reads_one_plane_twice(models, expected, monkeypatch):
    """Configuration B with the size threshold of the tcgen05 prefill kernel at 0: every prompt
    portion takes it, decoded tokens the TMA-fed decode kernel; both read the one cached plane
    as keys and as values.  Free pages hold NaN, so a read beyond a request's keys shows."""
    from freetoken_b200.csrc import ops
    calls = {"prefill_tc": 0, "decode": 0}
    real_p, real_d = ops.attn_prefill_tc, ops.attn_decode
    monkeypatch.setattr(ops, "PREFILL_TC_MIN_SCORES", 0)
    monkeypatch.setattr(ops, "attn_prefill_tc", lambda *a, **k: (calls.__setitem__("prefill_tc", 1), real_p(*a, **k))[1])
    monkeypatch.setattr(ops, "attn_decode", lambda *a, **k: (calls.__setitem__("decode", 1), real_d(*a, **k))[1])
    reqs = requests_of("B")
    for cut in ("portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = fz.make_engine(models["B"], "bfloat16", 64, rd.peak_tokens(schedule, 64), poison=True)
        got = rd.run_engine(engine, reqs, schedule)
        ops.check_tc_status(engine.device)
        fz.compare(got, expected("B"), fz.TOL["bfloat16"], f"B {cut}, tensor-core attention")
    assert calls == {"prefill_tc": 1, "decode": 1}


@pytest.mark.parametrize("which", ["A", "C"])
def test_float32_cuts_agree_bitwise(models, which):
    """In float32 the logits at a position depend neither on the cut nor on the batch."""
    reqs = requests_of(which)
    results = {}
    for cut, fn in CUTS.items():
        schedule = fn(reqs)
        engine = fz.make_engine(models[which], "float32", fz.PAGE[which], rd.peak_tokens(schedule, fz.PAGE[which]))
        results[cut] = rd.run_engine(engine, reqs, schedule)
    for cut in ("decode_tail", "portions", "mixed"):
        for rid in reqs:
            assert torch.equal(results[cut][rid], results["whole"][rid]), (cut, rid)


# ----------------------------------------------------- far keys, page borders, sharp on purpose
def sharpen(config, state, layer, asker, target, beta):
    """Rewrite layer ``layer``'s query matrix so that token ``asker``'s query (as the first
    layer sees it) is ``beta`` times token ``target``'s key in every head: wherever ``target``
    stands in the sequence, ``asker`` puts nearly all its weight there."""
    W = config["width"]
    eps = config["norm"]["eps"]
    E = state["embed"].double()
    x = plain.rms_norm(E[[asker, target]], state["embed.norm"].double(), eps)
    h = plain.rms_norm(x, state[f"l{layer}.norm1"].double(), eps)
    m = config["layers"][layer]["mixer"]
    H, d = m["heads"], m["dim"]
    if config["layers"][layer]["type"] == "attention":
        k = (state[f"l{layer}.mix.k"].double() @ h[1]).view(m["kv_heads"], d)
        k = k.repeat_interleave(H // m["kv_heads"], dim=0)                     # key of each query head
    else:
        c = plain.rms_norm(state[f"l{layer}.mix.dkv"].double() @ h[1], state[f"l{layer}.mix.dkv.norm"].double(), eps)
        k = (state[f"l{layer}.mix.uk"].double() @ c).view(H, d)
    q = state[f"l{layer}.mix.q"].double()
    q = q - (q @ h[0])[:, None] * h[0][None, :] / h[0].dot(h[0])               # forget what asker asked before
    q = q + beta * k.reshape(H * d, 1) * h[0][None, :] / h[0].dot(h[0])
    state[f"l{layer}.mix.q"] = q.to(torch.bfloat16)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_a_far_key_at_a_page_border_decides(tmp_path, kind, dtype):
    """One layer, attention made sharp: the asking token's output is the key (or value) of the
    target token, which stands once, hundreds of positions back, right before, on and right
    after a page border; asked from inside a prompt portion and from a decoded token.  A key
    that is not seen, or taken from a neighbouring row or page, changes the logits wholly."""
    layer = fz.attn(2, 1, 16, 0.25, coef=0.3, every=16) if kind == "attention" else fz.latent(2, 16, 16, 24, 0.25)
    config = one_layer(layer, vocab=120, width=48)
    state = plain.random_state(config, 31)
    asker, target = 7, 11
    sharpen(config, state, 0, asker, target, beta=8.0 if kind == "attention" else 20.0)
    page, n = 16, 300
    reqs = {}
    for place in (15, 16, 17, 0, 1, 255):
        toks = [t if t not in (asker, target) else 13 for t in fz.tokens(40 + place, n, 120)]
        toks[place] = target
        toks[n - 40] = asker                  # asked inside the prompt portion
        toks[n - 1] = asker                   # and by the last decoded token
        reqs[f"t{place}"] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    # the test is only worth something if losing the key shows
    blind = list(reqs["t16"])
    blind[16] = 13                            # (moving a key changes nothing: the design has no positions)
    other = plain.forward(config, state, blind)
    assert float(fz.position_errors(other[-1:], want["t16"][-1:])) > 0.3
    folder = fz.write_model(str(tmp_path / "m"), config, state)
    tol = fz.TOL[dtype] * (1 if dtype == "float32" else 3)      # sharp softmax: rounding of scores counts more
    for cut in ("decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = fz.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        fz.compare(rd.run_engine(engine, reqs, schedule), want, tol, f"far key, {kind}, {cut} [{dtype}]")


# --------------------------------------------------------- first tokens, long decoding
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_first_tokens_and_long_decoding(models, dtype):
    """A request that starts with a single token and is decoded one token at a time for 200
    steps (over many pages and several periods of the temperature), beside a second request
    that joins later; against the whole sequences."""
    from freetoken_b200.engine import StepEntry
    config = fz.FZ["A"]
    state = plain.random_state(config, fz.SEEDS["A"])
    a, b = fz.tokens(5, 201, config["vocab"]), fz.tokens(6, 120, config["vocab"])
    engine = fz.make_engine(models["A"], dtype, 4, 204 + 120)
    got_a, got_b = [], []
    for i in range(len(a)):
        entries = [StepEntry("a", [a[i]], [0])]
        j = i - 60
        if 0 <= j < len(b) // 2:
            entries.append(StepEntry("b", b[2 * j:2 * j + 2], [0, 1]))      # two tokens a step
        logits = engine.step(entries).float().cpu()
        got_a.append(logits[0])
        got_b.extend(logits[1:])
    fz.compare({"a": torch.stack(got_a), "b": torch.stack(got_b)},
               {"a": plain.forward(config, state, a), "b": plain.forward(config, state, b)},
               fz.TOL[dtype], f"long decoding [{dtype}]")


# ------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_scheduler(models, which, dtype):
    """``LLM.generate`` (scheduler, overlapped steps, graph replay of decode steps in
    bfloat16): every generated token is the plain model's own greedy choice for the sequence so
    far, unless its two best logits lie within rounding of each other."""
    from freetoken_b200 import LLM, SamplingParams
    config = fz.FZ[which]
    state = plain.random_state(config, fz.SEEDS[which])
    llm = LLM(models[which], dtype, page_size=fz.PAGE[which], num_token_override=1024, max_running_req=3,
              max_extend_tokens=24)
    prompts = [fz.tokens(70 + i, n, config["vocab"]) for i, n in enumerate((3, 30, 11, 1, 47))]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    tie = 1e-4 if dtype == "float32" else 5e-2
    ties = 0
    for prompt, result in zip(prompts, out):
        seq = list(prompt)
        assert len(result["token_ids"]) == 12
        for token in result["token_ids"]:
            logits = plain.forward(config, state, seq)[-1]
            if token != int(logits.argmax()):
                assert float(logits.max() - logits[token]) < tie, (dtype, len(seq), token, int(logits.argmax()))
                ties += 1
            seq.append(int(token))
    assert ties == 0 if dtype == "float32" else ties <= 3
    if dtype == "bfloat16":
        assert llm.engine.graph_replays > 0


def test_generate_command_and_sampling(models, capsys):
    """``ft generate`` on a Fazinex folder in float32: greedy tokens are the plain model's; with a
    temperature, a request's tokens depend on its seed and not on what else runs beside it."""
    import json

    from freetoken_b200 import LLM, SamplingParams, cli
    config = fz.FZ["C"]
    state = plain.random_state(config, fz.SEEDS["C"])
    prompt = fz.tokens(3, 9, config["vocab"])
    rc = cli.main(["generate", "--model-path", models["C"], "--dtype", "float32", "--page-size", "12",
                   "--num-tokens", "240", "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6",
                   "--ignore-eos"])
    assert rc == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    seq = list(prompt)
    for token in result["token_ids"]:
        assert token == int(plain.forward(config, state, seq)[-1].argmax())
        seq.append(token)
    llm = LLM(models["C"], "float32", page_size=12, num_token_override=480, max_running_req=3)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, max_tokens=8, ignore_eos=True, seed=5)
    alone = llm.generate([prompt], sp)[0]["token_ids"]
    beside = llm.generate([fz.tokens(4, 30, config["vocab"]), prompt, fz.tokens(5, 2, config["vocab"])],
                          [SamplingParams(temperature=1.0, max_tokens=8, ignore_eos=True, seed=1), sp,
                           SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)])[1]["token_ids"]
    assert alone == beside and len(alone) == 8


# ------------------------------------------- the mixer's window option (no Fazinex model sets it)
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("dim,page,window", [(16, 8, 24), (64, 64, 70)])
def test_shared_kv_attention_with_a_window(tmp_path, monkeypatch, dim, page, window, dtype):
    """``shared_kv_attention`` takes ``sliding_window`` like the engine's other attention mixer;
    a variant architecture registered here sets it.  Attention is made sharp: the asking token
    finds its target just inside the window (``window - 1`` back) and must not find it just
    outside (``window`` back), in a prompt portion and as a decoded token; pages the window has
    passed are given back while the requests run (head size 16: the generic kernel; 64: the
    TMA-fed ones)."""
    import dataclasses

    from freetoken_b200.config import fazinex as fzc
    from freetoken_b200.config.model_plan import PartSpec
    from freetoken_b200.registry import Architecture, register_architecture

    def build(cfg):
        plan = fzc.build_plan(cfg)
        layers = tuple(dataclasses.replace(l, mixer=PartSpec(l.mixer.kind, {**l.mixer.params, "sliding_window": window}))
                       for l in plan.layers)
        return dataclasses.replace(plan, layers=layers)
    register_architecture(Architecture(name="FazinexWindowedForTest", read_config=fzc.FazinexConfig.from_dict,
                                       build_plan=build, config_to_dict=lambda c: c.to_dict()))

    def windowed_softmax(scores):
        T = scores.shape[-1]
        seen = torch.ones(T, T, dtype=torch.bool).tril() & ~torch.ones(T, T, dtype=torch.bool).tril(-window)
        return torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)
    monkeypatch.setattr(plain, "causal_softmax", windowed_softmax)

    config = one_layer(fz.attn(2, 1, dim, 0.25, coef=0.2, every=32), vocab=120, width=48)
    state = plain.random_state(config, 41)
    asker, target = 7, 11
    sharpen(config, state, 0, asker, target, beta=8.0)
    n = 200
    reqs = {}
    for name, back in (("inside", window - 1), ("outside", window), ("far_outside", 3 * window)):
        toks = [t if t not in (asker, target) else 13 for t in fz.tokens(60 + back, n, 120)]
        for at in (n - 40, n - 1):            # asked from a prompt portion and by the last decoded token
            toks[at] = asker
            toks[at - back] = target
        reqs[name] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    blind = [t if t != target else 13 for t in reqs["inside"]]
    assert float(fz.position_errors(plain.forward(config, state, blind)[-1:], want["inside"][-1:])) > 0.3
    seen = [t if t != target else 13 for t in reqs["outside"]]
    assert float(fz.position_errors(plain.forward(config, state, seen)[-1:], want["outside"][-1:])) < 1e-9
    folder = fz.write_model(str(tmp_path / "m"), {**config, "architecture": "FazinexWindowedForTest"}, state)
    tol = fz.TOL[dtype] * (1 if dtype == "float32" else 3)
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = fz.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        fz.compare(rd.run_engine(engine, reqs, schedule), want, tol, f"window {window}, {cut} [{dtype}]")
        assert engine.cache.free_pages() == engine.cache.total_pages()
