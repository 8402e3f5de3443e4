"""Host-side tests of the Tonapel configuration, its model plan, the tensors the plan asks for
and the cache a mixer made of two mixers gets (no GPU)."""

import copy

import pytest
import torch

import tonapel_tiny as tn
from freetoken_b200.cache import CacheManager, CompositeNeed, PagedKVNeed, StateNeed
from freetoken_b200.config.model_plan import ConfigError
from freetoken_b200.config.tonapel import TonapelConfig, build_plan
from freetoken_b200.models.model import Model
from freetoken_b200.registry import architecture_of
from freetoken_b200.weights.loader import WeightError, plan_loading


def test_registry_picks_the_design_by_its_singular_key():
    arch = architecture_of(tn.TN_A)
    assert arch.name == "Tonapel"
    cfg = arch.read_config(tn.TN_A)
    assert isinstance(cfg, TonapelConfig) and cfg.to_dict() == tn.TN_A


@pytest.mark.parametrize("which", list(tn.TN))
def test_plan_hands_every_constant_to_a_part(which):
    raw = tn.TN[which]
    plan = build_plan(TonapelConfig.from_dict(raw))
    assert [s.layer for s in plan.schedule] == list(range(len(raw["layers"])))
    for spec, layer in zip(plan.layers, raw["layers"]):
        assert spec.block.kind == "sandwich" and spec.block.params["residual_mult"] == raw["residual_mult"]
        assert (spec.feed_forward is None) == (layer["mlp"] is None)
        assert sorted(spec.all_norms()) == (["feed_forward", "feed_forward_out", "mixer", "mixer_out"]
                                            if layer["mlp"] else ["mixer", "mixer_out"])
        assert all(n.params["plus_one"] and n.params["eps"] == raw["norm"]["eps"] for n in spec.all_norms().values())
        m = layer["mixer"]
        if layer["type"] == "parallel":
            assert spec.mixer.kind == "mixer_sum"
            assert tuple(spec.mixer.params["scales"]) == (m["left_scale"], m["right_scale"])
            a, s = spec.mixer.params["members"]
            assert (a.kind, s.kind) == ("paged_attention", "ssd")
            assert a.params["sliding_window"] == m["left"]["mask"]["size"] and a.params["bias"]
            assert (a.params["head_dim"], a.params["value_dim"]) == (m["left"]["dim"], m["left"]["vdim"])
            assert a.params["sm_scale"] == m["left"]["scale"]
            assert a.params["position"].params["rotary_dim"] == m["left"]["rot"]["dims"]
            assert a.params["position"].params["theta"] == m["left"]["rot"]["base"]
            assert (s.params["state_dim"], s.params["groups"], s.params["conv_taps"], s.params["norm_groups"]) == \
                (m["right"]["state"], m["right"]["groups"], m["right"]["conv"], m["right"]["norm_groups"])
        else:
            assert spec.mixer.kind == "gated_delta"
            assert (spec.mixer.params["key_heads"], spec.mixer.params["key_dim"], spec.mixer.params["head_dim"],
                    spec.mixer.params["conv_taps"]) == (m["kv_heads"], m["dim"], m["vdim"], m["conv"])
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            f = spec.feed_forward.params
            assert (f["num_experts"], f["top_k"], f["act_limit"], f["intermediate_size"]) == \
                (layer["mlp"]["router"]["experts"], layer["mlp"]["router"]["top"], layer["mlp"]["expert"]["limit"],
                 layer["mlp"]["expert"]["ff"])
        elif layer["mlp"]:
            assert spec.feed_forward.params["gated"] and spec.feed_forward.params["activation"] == "gelu_tanh"


@pytest.mark.parametrize("which", list(tn.TN))
def test_the_model_asks_for_exactly_the_files_tensors(which):
    raw = tn.TN[which]
    model = Model(build_plan(TonapelConfig.from_dict(raw)))
    shapes = {k: tuple(v.shape) for k, v in tn.random_state(raw, 1).items()}
    plan_loading(model.tensor_specs(), shapes)
    shapes["l0.mix.left.extra"] = (3,)
    lost = next(k for k in shapes if k.endswith("norm1b"))
    del shapes[lost]
    with pytest.raises(WeightError) as e:
        plan_loading(model.tensor_specs(), shapes)
    assert e.value.missing == [lost] and e.value.unexpected == ["l0.mix.left.extra"]


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "hyena", "type"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "right", "groups"), 2, "groups"),
    (("layers", 0, "mixer", "right", "norm_groups"), 7, "norm_groups"),
    (("layers", 0, "mixer", "right", "state"), 300, "state"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("layers", 0, "mlp", "router", "top"), 6, "top"),
    (("layers", 0, "mlp", "expert", "limit"), 0.0, "limit"),
    (("norm",), None, "norm"),
    (("layers",), [], "layers"),
])
def test_refusals_name_the_key(path, value, word):
    raw = copy.deepcopy(tn.TN_A)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        TonapelConfig.from_dict(raw)
    assert word in str(e.value)


def test_a_mixer_of_two_mixers_gets_pages_and_state_slots():
    """The parallel layers' needs are composite: the attention members of equal shape and window
    share a page group whose window gives pages back, every state-space and delta mixer has a
    state row per request slot; a delta-only model has no pages at all."""
    model = Model(build_plan(TonapelConfig.from_dict(tn.TN_B)))
    needs = model.cache_needs()
    assert isinstance(needs[0], CompositeNeed) and isinstance(needs[1], StateNeed)
    kv, st = needs[0].parts
    assert kv == PagedKVNeed(2, 64, 100) and st.shape == ((4 - 1) * (4 * 32 + 2 * 2 * 64) + 4 * 64 * 32,)
    cache = CacheManager(needs, 64, 12, 2, 64 * 12)
    assert len(cache.paged_groups) == 3 and len(cache.state_groups) == 4
    assert cache.paged_index[(0, 0)] == (0, 0) and cache.state_index[(0, 1)][1] == 0 and 1 in cache.state_index
    cache.admit("a")
    cache.grow("a", 300)
    cache.advance("a", 300)
    assert cache.held_pages("a") == [2, 2, 3]        # windows of 100, 64 and 130 at 300 tokens, pages of 64
    cache.release("a")
    cache.check_integrity()
    only_delta = tn.model(50, 16, 1e-5, 1.0, [tn.delta(2, 1, 4, 4, 2), tn.delta(1, 1, 8, 4, 3, tn.dense(8))])
    needs = Model(build_plan(TonapelConfig.from_dict(only_delta))).cache_needs()
    cache = CacheManager(needs, 8, 4, 2, 32)
    assert cache.paged_groups == [] and len(cache.state_groups) == 2
    cache.admit("a")
    cache.grow("a", 20)
    cache.advance("a", 20)
    cache.release("a")
    cache.check_integrity()


def test_value_heads_of_another_size_are_filled_up_with_zeros():
    from freetoken_b200.config.model_plan import PartSpec
    from freetoken_b200.parts.attention import PagedAttention
    names = {"qkv": "qkv", "q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "qn", "k_norm": "kn", "qkv_bias": "qkv.b",
             "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b"}
    spec = PartSpec("paged_attention", {
        "hidden_size": 6, "num_heads": 2, "num_kv_heads": 1, "head_dim": 2, "value_dim": 3, "sm_scale": 1.0,
        "bias": True, "sliding_window": 4, "scope": "a", "checkpoint_names": names,
        "position": PartSpec("none", {})})
    part = PagedAttention(spec, "l0")
    assert part.cache_need() == PagedKVNeed(1, 3, 4)
    by_name = {s.name: s for s in part.tensor_specs()}
    assert by_name["l0.a.qkv"].shape == (2 * 2 + 2 + 3, 6) and by_name["l0.a.o"].shape == (6, 2 * 3)
    tensors = {n: torch.arange(1, 1 + torch.Size(s.shape).numel(), dtype=torch.float32).view(s.shape)
               for n, s in by_name.items()}
    part.bind(tensors, torch.float32)
    assert part.w_qkv.shape == (4 * 3, 6) and part.w_o.shape == (6, 6)
    q = tensors["l0.a.qkv"]
    assert torch.equal(part.w_qkv[0:2], q[0:2]) and torch.all(part.w_qkv[2] == 0)       # q head 0, filled up
    assert torch.equal(part.w_qkv[6:8], q[4:6]) and torch.all(part.w_qkv[8] == 0)       # the k head
    assert torch.equal(part.w_qkv[9:12], q[6:9])                                        # the v head as it is
    assert torch.equal(part.b_qkv[[0, 1, 3, 4, 6, 7, 9, 10, 11]], tensors["l0.a.qkv.b"]) and part.b_qkv[2] == 0
