"""Nizorax on the host: config.json keys and refusals, the plan it becomes (blocks with a norm before and after each
sublayer and a convolution part in front of it, a repeated run of layers), the tensors it expects and the caches its layers
ask for; and the plain implementation's own mechanisms where a fault would be silent.  Needs no GPU."""
import copy
import json
import math

import pytest
import torch

from imp_b200.cache.manager import CacheManager
from imp_b200.config.model_config import ConfigError, NizoraxConfig
from imp_b200.config.registry import config_from_dict, known_architectures, load_config, plan_for
from imp_b200.parts.registry import mixer_cache_spec
from plain import nizorax_plain as N

CFG = {
    "architecture": "Nizorax", "vocab": 101, "width": 72, "norm": {"eps": 2e-5}, "embedding": {"scale": 3.0}, "logit_scale": 0.5,
    "canon": {"taps": 3},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "diff": 0.3, "scale": 0.2, "mask": {"size": 10},
                   "rot": {"base": 100.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}},
         "mlp": {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 12, "top": 2, "scale": 2.5, "groups": {"count": 4, "keep": 2}},
                 "shared": {"ff": 36}}},
        {"type": "lightning", "mixer": {"heads": 3, "dim": 8, "vdim": 24, "decay": [0.5, 0.9, 0.99]}, "mlp": {"kind": "dense", "ff": 100}},
        {"type": "attention", "mixer": {"heads": 2, "dim": 16, "diff": 0.8}, "mlp": None},
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}


def test_architecture_is_known_and_round_trips(tmp_path):
    assert "Nizorax" in known_architectures()
    c = config_from_dict(CFG)
    assert isinstance(c, NizoraxConfig)
    assert (c.architecture, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Nizorax", 101, 72, 3)
    assert c.run_order() == [0, 1, 2, 1, 2]
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)) == c
    saved = json.load(open(tmp_path / "config.json"))
    assert saved["layers"][2]["mlp"] is None and saved["layers"][1]["mixer"]["decay"] == [0.5, 0.9, 0.99]


def test_plan_takes_every_size_and_constant_from_config():
    plan = plan_for(config_from_dict(CFG))
    assert [l.block for l in plan.layers] == ["sandwich"] * 3 and plan.order == [0, 1, 2, 1, 2]
    l0, l1, l2 = plan.layers
    assert list(l0.parts) == ["mixer_norm", "mixer_conv", "mixer", "mixer_post_norm", "ffn_norm", "ffn_conv", "feed_forward", "ffn_post_norm"]
    assert list(l2.parts) == ["mixer_norm", "mixer_conv", "mixer", "mixer_post_norm"]
    assert l0.block_params == {"has_ffn": True, "input_conv": True} and l2.block_params == {"has_ffn": False, "input_conv": True}
    a = l0.mixer
    assert a.kind == "differential_attention"
    assert (a.params["num_heads"], a.params["num_kv_heads"], a.params["head_dim"], a.params["value_dim"], a.params["scale"], a.params["lambda_init"],
            a.params["window"], a.params["rot_dims"], a.params["rot_base"], a.params["rot_pairing"], a.params["norm_eps"]) == \
        (6, 2, 24, 40, 0.2, 0.3, 10, 8, 100.0, "neighbours", 2e-5)
    assert a.params["rot_scaling"] == {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}
    assert a.tensors["lambda_k2"] == "l0.mix.lk2" and a.tensors["q_proj"] == "l0.mix.q"
    r = l1.mixer
    assert r.kind == "retention"
    assert (r.params["num_heads"], r.params["key_dim"], r.params["value_dim"], r.params["decay"], r.params["key_scale"], r.params["qkv_act"],
            r.params["gate_act"], r.params["norm_over"], r.params["out_norm"]) == (3, 8, 24, [0.5, 0.9, 0.99], 1.0, "silu", "sigmoid", "row", True)
    c = l0.parts["mixer_conv"]
    assert c.kind == "residual_conv" and c.params == {"hidden_size": 72, "taps": 3} and c.tensors == {"weight": "l0.canon1"}
    assert l0.parts["ffn_conv"].tensors == {"weight": "l0.canon2"}
    f = l0.feed_forward
    assert f.kind == "routed_experts"
    assert (f.params["num_experts"], f.params["top_k"], f.params["expert_size"], f.params["shared_size"], f.params["scores"], f.params["weight_scale"],
            f.params["num_groups"], f.params["keep_groups"], f.params["router_bias"], f.params["shared_gate"]) == (12, 2, 20, 36, "sigmoid", 2.5, 4, 2, False, False)
    d = l1.feed_forward
    assert d.kind == "polynorm_mlp" and (d.params["intermediate_size"], d.params["norm_eps"]) == (100, 2e-5) and d.tensors["coef"] == "l1.mlp.act"
    for n in (l0.mixer_norm, l0.parts["mixer_post_norm"], l1.parts["ffn_post_norm"], plan.final_norm):
        assert n.kind == "layernorm" and n.params["eps"] == 2e-5 and n.params["bias"] is True
    assert l0.parts["mixer_post_norm"].tensors == {"weight": "l0.norm1b", "bias": "l0.norm1b.b"}
    assert plan.embedding.params["scale"] == 3.0 and plan.head.params["scale"] == 0.5


def test_expected_tensors_are_the_checkpoint_names():
    exp = plan_for(config_from_dict(CFG)).expected_tensors()
    shapes = {k: tuple(v.shape) for k, v in exp.items()}
    assert shapes["embed"] == (101, 72) and shapes["head"] == (101, 72) and shapes["final.norm.b"] == (72,)
    assert shapes["l0.mix.q"] == (6 * 2 * 24, 72) and shapes["l0.mix.k"] == (2 * 2 * 24, 72) and shapes["l0.mix.v"] == (2 * 40, 72)
    assert shapes["l0.mix.lq1"] == (24,) and shapes["l0.mix.o"] == (72, 6 * 40)
    assert shapes["l0.canon1"] == (72, 3) and shapes["l0.canon2"] == (72, 3) and shapes["l0.norm2b.b"] == (72,)
    assert shapes["l0.mlp.router"] == (12, 72) and shapes["l0.mlp.e11.down"] == (72, 20) and shapes["l0.mlp.shared.gate"] == (36, 72)
    assert shapes["l1.mix.q"] == (24, 72) and shapes["l1.mix.v"] == (72, 72) and shapes["l1.mix.g"] == (72, 72) and shapes["l1.mix.norm"] == (72,)
    assert shapes["l1.mlp.up"] == (100, 72) and shapes["l1.mlp.down"] == (72, 100) and shapes["l1.mlp.act"] == (4,)
    assert shapes["l2.mix.q"] == (2 * 2 * 16, 72) and shapes["l2.mix.k"] == (2 * 2 * 16, 72) and shapes["l2.mix.v"] == (32, 72)
    for absent in ("l2.norm2", "l2.canon2", "l2.mlp.up", "l0.mlp.router.b", "l0.mlp.shared.sg", "l1.mix.lq1", "l0.mix.g"):
        assert absent not in exp


def test_options_that_config_leaves_out_do_not_exist():
    cfg = copy.deepcopy(CFG)
    del cfg["canon"], cfg["loop"], cfg["embedding"], cfg["logit_scale"]
    m = cfg["layers"][0]["mlp"]
    del m["router"]["groups"], m["router"]["scale"]
    m["shared"] = None
    plan = plan_for(config_from_dict(cfg))
    assert plan.order is None
    assert list(plan.layers[0].parts) == ["mixer_norm", "mixer", "mixer_post_norm", "ffn_norm", "feed_forward", "ffn_post_norm"]
    assert plan.layers[0].block_params["input_conv"] is False
    assert plan.embedding.params["scale"] == 1.0 and plan.head.params["scale"] == 1.0
    f = plan.layers[0].feed_forward
    assert (f.params["num_groups"], f.params["weight_scale"], f.params["shared_size"]) == (0, 1.0, 0)
    assert "shared_gate" not in f.tensors
    a = plan.layers[2].mixer           # neither mask nor rot nor kv_heads nor vdim nor scale
    assert (a.params["window"], a.params["rot_dims"], a.params["num_kv_heads"], a.params["value_dim"]) == (0, 0, 2, 16)
    assert a.params["scale"] == pytest.approx(0.25) and "rot_scaling" not in a.params


def test_every_run_of_a_layer_owns_its_caches():
    plan = plan_for(config_from_dict(CFG))
    att = mixer_cache_spec("differential_attention", plan.layers[0].mixer.params)
    assert att == {"kind": "paged", "num_kv_heads": 4, "head_dim": 48, "window": 10}      # two maps a key head; keys of 24 and values of 40 in rows of 48
    assert mixer_cache_spec("differential_attention", plan.layers[2].mixer.params) == {"kind": "paged", "num_kv_heads": 4, "head_dim": 16, "window": 0}
    conv = mixer_cache_spec("residual_conv", plan.layers[0].parts["mixer_conv"].params)
    assert conv["kind"] == "state" and [t["shape"] for t in conv["tensors"]] == [[2, 72]]
    ret = mixer_cache_spec("retention", plan.layers[1].mixer.params)
    assert [t["name"] for t in ret["tensors"]] == ["S"] and ret["tensors"][0]["shape"][0] >= 3 * 8 * 24
    one_tap = mixer_cache_spec("residual_conv", {"hidden_size": 72, "taps": 1})
    assert one_tap["tensors"][0]["shape"] == [1, 72]
    # a layer's caches in slot order (conv, mixer, conv); five layer runs
    per_layer = {0: [conv, att, conv], 1: [conv, ret, conv], 2: [conv, mixer_cache_spec("differential_attention", plan.layers[2].mixer.params)]}
    specs = [s for i in plan.order for s in per_layer[i]]
    mgr = CacheManager(specs, page_size=4, num_pages=32, num_state_slots=2)
    info = mgr.info()
    assert len(info["paged"]) == 2 and len(info["state"]) == 2        # two attention geometries; the convolutions' inputs and the lightning state
    for rid, n in ((1, 9), (2, 3)):
        mgr.add_request(rid)
        mgr.reserve(rid, n)
        mgr.commit(rid, n)
    mgr.check_invariants()
    mgr.release(1)
    mgr.release(2)
    assert mgr.free_pages() == 32


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][1].update(type="conv"), "unknown layer type 'conv'"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "unknown kind 'gated'"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.9]), "'decay' must list a number per head"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "6 heads are not a multiple of 4 kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims 7 must be even"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.5), "low < high"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=5), "count must divide the experts"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=12), "hold `top` experts"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=13), "top 13 exceeds the 12 experts"),
    (lambda c: c["layers"][2]["mixer"].pop("dim"), "dim"),
    (lambda c: c["canon"].update(taps=0), "taps"),
    (lambda c: c["loop"].update(stop=4), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals_name_the_key(edit, text):
    cfg = copy.deepcopy(CFG)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert text in str(e.value)


# ------------------------------------------------------------------ the plain implementation's own mechanisms
def test_plain_frequencies_keep_slow_and_blend():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    f = N.scaled_frequencies(100.0, 8, sc)
    raw = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    waves = [2 * math.pi / r for r in raw]
    assert waves[0] < 16 and f[0] == raw[0]                                   # short wavelength: kept
    assert waves[3] > 64 and f[3] == pytest.approx(raw[3] / 8.0)              # long: slowed down
    mid = [i for i in range(4) if 16 <= waves[i] <= 64]
    assert mid, "the case must hold a frequency between the two edges"
    for i in mid:
        s = (64 / waves[i] - 1.0) / 3.0
        assert float(f[i]) == pytest.approx((1 - s) * raw[i] / 8.0 + s * raw[i])
    assert torch.equal(N.scaled_frequencies(100.0, 8, None), torch.tensor(raw, dtype=torch.float64))


def test_plain_window_sees_itself_and_size_minus_one_before():
    T, D = 12, 4
    q = torch.zeros(T, D, dtype=torch.float64)
    k = torch.zeros(T, D, dtype=torch.float64)
    v = torch.eye(T, dtype=torch.float64)
    out = N.windowed_softmax_attention(q, k, v, 1.0, 5)           # equal scores: the output marks the keys that were seen
    for i in range(T):
        seen = torch.nonzero(out[i] > 0)[:, 0].tolist()
        assert seen == list(range(max(0, i - 4), i + 1))
    assert torch.nonzero(N.windowed_softmax_attention(q, k, v, 1.0, 0)[T - 1] > 0).numel() == T


def test_plain_route_keeps_groups_by_their_two_largest_scores():
    W = {"f.router": torch.eye(8, dtype=torch.float64)}
    c = {"router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 1}}}
    # group 0 holds the single largest score, group 2 the largest pair
    u = torch.tensor([[3.0, -5.0, 0.0, 0.0, 2.0, 2.5, 0.0, 0.0]], dtype=torch.float64)
    idx, w, s = N.route(u, W, "f.", c)
    assert sorted(idx[0].tolist()) == [4, 5]
    assert torch.allclose(w[0].sort().values, 1.5 * torch.sigmoid(torch.tensor([2.0, 2.5], dtype=torch.float64)))
    c["router"]["groups"] = None
    idx, _, _ = N.route(u, W, "f.", c)
    assert sorted(idx[0].tolist()) == [0, 5]
    assert float(N.route_margin(u, W, "f.", c)[0]) == pytest.approx(1 / (1 + math.exp(-2.5)) - 1 / (1 + math.exp(-2.0)))


def test_plain_convolution_ends_on_the_token_itself():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None].repeat(1, 2)
    w = torch.tensor([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]], dtype=torch.float64)
    out = N.add_causal_conv(u, w)
    assert out[:, 0].tolist() == [1 + 1, 2 + 10 + 2, 3 + 100 + 20 + 3, 4 + 200 + 30 + 4, 5 + 300 + 40 + 5]
    assert out[:, 1].tolist() == [3.0, 6.0, 9.0, 12.0, 15.0]
