"""The Fazinex architecture on the host: config.json reading and refusals, the run order of a
loop, the plan and its tensors, cache groups; and the plain implementation's own pieces."""

import copy
import math

import pytest
import torch

import fazinex_tiny as fz
import plain_fazinex as plain
from freetoken_b200.cache import CacheManager, PagedKeyNeed
from freetoken_b200.config.fazinex import FazinexConfig, build_plan
from freetoken_b200.config import ConfigError
from freetoken_b200.models import Model
from freetoken_b200.registry import architecture_of


def test_the_singular_architecture_key_picks_the_model():
    arch = architecture_of(fz.FZ_A)
    assert arch.name == "Fazinex"
    cfg = arch.read_config(fz.FZ_A)
    assert isinstance(cfg, FazinexConfig) and cfg.to_dict() == fz.FZ_A


@pytest.mark.parametrize("which", list(fz.FZ))
def test_run_order_is_the_plain_models(which):
    cfg = FazinexConfig.from_dict(fz.FZ[which])
    assert cfg.run_order() == plain.layer_order(fz.FZ[which])
    plan = build_plan(cfg)
    assert [s.layer for s in plan.schedule] == cfg.run_order()
    assert all(s.owns_cache for s in plan.schedule)          # every pass has a cache of its own


def test_loop_forms():
    base = copy.deepcopy(fz.FZ_A)
    for loop, want in (({"start": 0, "stop": 4, "times": 2}, [0, 1, 2, 3, 0, 1, 2, 3]),
                       ({"start": 3, "stop": 4, "times": 3}, [0, 1, 2, 3, 3, 3]),
                       ({"start": 2, "stop": 2, "times": 5}, [0, 1, 2, 3]),
                       ({"start": 0, "stop": 1, "times": 1}, [0, 1, 2, 3]),
                       (None, [0, 1, 2, 3])):
        base["loop"] = loop
        assert FazinexConfig.from_dict(base).run_order() == want == plain.layer_order(base)
    for bad in ({"start": 2, "stop": 1, "times": 2}, {"start": 0, "stop": 5, "times": 2},
                {"start": 0, "stop": 2, "times": 0}):
        base["loop"] = bad
        with pytest.raises(ConfigError):
            FazinexConfig.from_dict(base)


def test_every_constant_reaches_a_part():
    plan = build_plan(FazinexConfig.from_dict(fz.FZ_A))
    a, l, a2, l2 = (layer.mixer.params for layer in plan.layers)
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["sm_scale"]) == (4, 2, 16, 0.3)
    assert (a["q_temp_coef"], a["q_temp_every"]) == (0.25, 8)
    assert a2["q_temp_coef"] == 0.0                                  # no q_temp: no temperature
    assert (l["num_heads"], l["qk_dim"], l["v_dim"], l["rank"], l["sm_scale"]) == (3, 16, 24, 40, 0.2)
    assert l["norm_eps"] == 1e-5 and plan.layers[0].mixer_norm.params["eps"] == 1e-5
    assert plan.layers[3].feed_forward is None and plan.layers[1].feed_forward.params["intermediate_size"] == 80
    assert plan.head.params["softcap"] == 10.0 and plan.head.params["tied_to"] == "embed"
    assert build_plan(FazinexConfig.from_dict(fz.FZ_B)).head.params["softcap"] == 0.0


def test_refusals():
    def changed(path, value):
        cfg = copy.deepcopy(fz.FZ_A)
        node = cfg
        for key in path[:-1]:
            node = node[key]
        if value is None:
            node.pop(path[-1])
        else:
            node[path[-1]] = value
        return cfg
    for path, value in ((("vocab",), None), (("norm",), None), (("layers", 0, "type"), "mamba"),
                        (("layers", 0, "mixer", "kv_heads"), 3),
                        (("layers", 1, "mixer", "kv_rank"), None), (("layers", 0, "mlp", "kind"), "routed"),
                        (("layers", 0, "mixer", "scale"), None)):
        with pytest.raises(ConfigError):
            FazinexConfig.from_dict(changed(path, value))


@pytest.mark.parametrize("which", list(fz.FZ))
def test_the_models_tensors_are_the_files_tensors(which):
    """Names and shapes the model asks for are exactly what a checkpoint of the design holds
    (merged projections are assembled from the separate tensors)."""
    from freetoken_b200.weights.loader import plan_loading
    config = fz.FZ[which]
    model = Model(build_plan(FazinexConfig.from_dict(config)))
    state = plain.random_state(config, 0)
    chosen = plan_loading(model.tensor_specs(), {k: tuple(v.shape) for k, v in state.items()})
    assert len(chosen) == len(model.tensor_specs())
    state.pop("l0.norm1")
    state["l0.mix.extra"] = torch.zeros(1)
    from freetoken_b200.weights.loader import WeightError
    with pytest.raises(WeightError) as e:
        plan_loading(model.tensor_specs(), {k: tuple(v.shape) for k, v in state.items()})
    assert e.value.missing == ["l0.norm1"] and e.value.unexpected == ["l0.mix.extra"]


def test_cache_groups_follow_the_mixers():
    model = Model(build_plan(FazinexConfig.from_dict(fz.FZ_A)))
    needs = model.cache_needs()
    assert needs[0] == PagedKeyNeed(2, 16) and needs[1] == PagedKeyNeed(1, 40)
    assert len(needs) == 8                       # 1 + 3 x 2 + 1 stops
    manager = CacheManager(needs, 4, 16, 2, 64)
    assert [len(g.stops) for g in manager.paged_groups] == [1, 3, 3, 1]
    assert manager.paged_groups[1].need.layout(5, 4) == (5, 1, 4, 40)
    assert needs[1].elements_per_token() == 40   # one latent, not keys and values


# ---- the plain implementation's own pieces -----------------------------------------------
def test_plain_query_temperature():
    t = plain.query_temperature(torch.arange(20), 0.5, 4)
    assert t[0] == 1.0 and t[2] == 1.0                         # (p + 1) // 4 == 0
    assert math.isclose(float(t[3]), 1 + 0.5 * math.log(2))    # p + 1 == 4
    assert math.isclose(float(t[6]), 1 + 0.5 * math.log(2))
    assert math.isclose(float(t[7]), 1 + 0.5 * math.log(3))
    assert math.isclose(float(plain.query_temperature(torch.tensor([0]), 0.5, 1)[0]), 1 + 0.5 * math.log(2))


def test_plain_causal_softmax_and_norm():
    p = plain.causal_softmax(torch.zeros(3, 3, dtype=torch.float64))
    assert torch.allclose(p, torch.tensor([[1, 0, 0], [.5, .5, 0], [1 / 3, 1 / 3, 1 / 3]], dtype=torch.float64))
    v = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms(v, 0.0), v / math.sqrt(12.5))
    assert torch.allclose(plain.rms(v, 12.5), v / 5.0)           # eps inside the root


def test_plain_latent_attention_is_attention_over_the_latent():
    """The absorbed form (queries times Wuk^T, one shared head over c, Wuv afterwards)
    equals the written-out form: the identity the engine's mixer rests on."""
    torch.manual_seed(0)
    T, W, H, d, dv, R = 7, 12, 3, 4, 5, 6
    m = {"heads": H, "dim": d, "vdim": dv, "kv_rank": R, "scale": 0.3}
    w = {"q": torch.randn(H * d, W), "dkv": torch.randn(R, W), "dkv.norm": torch.rand(R) + 0.5,
         "uk": torch.randn(H * d, R), "uv": torch.randn(H * dv, R), "g": torch.randn(H, W),
         "o": torch.randn(W, H * dv)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    want = plain.latent_attention(h, w, m, 1e-6)
    c = plain.rms_norm(h @ w["dkv"].T, w["dkv.norm"], 1e-6)
    q = (h @ w["q"].T).view(T, H, d)
    out = []
    for i in range(H):
        qa = q[:, i] @ w["uk"].view(H, d, R)[i]
        p = plain.causal_softmax(qa @ c.T * 0.3)
        out.append((p @ c) @ w["uv"].view(H, dv, R)[i].T * torch.sigmoid(h @ w["g"][i])[:, None])
    got = torch.cat(out, dim=1) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-12)


def test_random_model_command_writes_the_designs_tensors(tmp_path):
    """``ft random-model`` on a Fazinex config: the folder holds the design's own tensor names
    (separate q / k / dkv / g, not the merged projections the engine keeps), the plain
    implementation runs on it, and norm weights are 1."""
    import json

    from freetoken_b200 import cli
    from plain_model import read_safetensors
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(fz.FZ_A))
    out = tmp_path / "model"
    assert cli.main(["random-model", "--config", str(cfg_path), "--out", str(out), "--seed", "3"]) == 0
    state = read_safetensors(str(out / "model.safetensors"))
    assert set(state) == set(plain.random_state(fz.FZ_A, 0))
    assert json.loads((out / "config.json").read_text()) == fz.FZ_A
    assert torch.all(state["l1.mix.dkv.norm"].float() == 1) and torch.all(state["embed.norm"].float() == 1)
    logits = plain.forward(fz.FZ_A, state, [1, 2, 3, 4])
    assert logits.shape == (4, 200) and torch.isfinite(logits).all()
