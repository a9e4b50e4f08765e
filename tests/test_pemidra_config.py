"""Pemidra on the host: config.json keys and refusals, the plan it becomes (post-norm blocks with tensors of their own, a
pair of mixers with a cache each), the tensors it expects and the caches its layers ask for.  Needs no GPU."""
import copy
import json

import pytest

from imp_b200.cache.manager import CacheManager
from imp_b200.config.model_config import ConfigError, PemidraConfig
from imp_b200.config.registry import config_from_dict, known_architectures, load_config, plan_for
from imp_b200.parts.registry import mixer_cache_spec

CFG = {
    "architecture": "Pemidra", "vocab": 101, "width": 72, "norm": {"eps": 2e-5}, "postln_alpha": 1.7,
    "layers": [
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 1, "dim": 24, "vdim": 16, "scale": 0.3, "mask": {"size": 10}, "rot": {"base": 100.0, "dims": 8}},
                   "right": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 3}},
         "mlp": None},
        {"type": "retention", "mixer": {"heads": 3, "dim": 8, "vdim": 24, "decay": [0.5, 0.9, 0.99]}, "mlp": {"kind": "dense", "ff": 100}},
        {"type": "general_delta", "mixer": {"heads": 2, "dim": 20}, "mlp": None},
    ],
}


def test_architecture_is_known_and_round_trips(tmp_path):
    assert "Pemidra" in known_architectures()
    c = config_from_dict(CFG)
    assert isinstance(c, PemidraConfig)
    assert (c.architecture, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Pemidra", 101, 72, 3)
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)) == c
    saved = json.load(open(tmp_path / "config.json"))
    assert saved["layers"][0]["mlp"] is None and saved["layers"][1]["mixer"]["decay"] == [0.5, 0.9, 0.99]


def test_plan_takes_every_size_and_constant_from_config():
    plan = plan_for(config_from_dict(CFG))
    assert [l.block for l in plan.layers] == ["postnorm"] * 3 and plan.order is None
    l0, l1, l2 = plan.layers
    assert list(l0.parts) == ["mixer_norm", "left", "right"]
    assert list(l1.parts) == ["mixer_norm", "mixer", "ffn_norm", "feed_forward"] and list(l2.parts) == ["mixer_norm", "mixer"]
    assert l0.block_params == {"hidden_size": 72, "residual_mult": 1.7, "has_ffn": False, "pair": True, "pair_eps": 2e-5}
    assert l1.block_params["has_ffn"] is True and l1.block_params["pair"] is False
    assert l0.block_tensors == {"mixer_scale": "l0.ls1", "left_out": "l0.mix.left.out", "right_out": "l0.mix.right.out"}
    assert l1.block_tensors == {"mixer_scale": "l1.ls1", "ffn_scale": "l1.ls2"}
    a = l0.parts["left"]
    assert a.kind == "gated_head_attention"
    assert (a.params["num_heads"], a.params["num_kv_heads"], a.params["head_dim"], a.params["value_dim"], a.params["scale"], a.params["chunk"],
            a.params["rot_dims"], a.params["rot_base"], a.params["norm_eps"]) == (4, 1, 24, 16, 0.3, 10, 8, 100.0, 2e-5)
    assert all(a.params[k] is True for k in ("qk_norm", "value_norm", "head_temp", "sink", "head_gate"))
    b = l0.parts["right"]
    assert b.kind == "channel_delta_rule"
    assert (b.params["num_heads"], b.params["num_kv_heads"], b.params["key_dim"], b.params["value_dim"], b.params["conv_taps"]) == (4, 2, 12, 20, 3)
    r = l1.mixer
    assert r.kind == "retention" and (r.params["num_heads"], r.params["key_dim"], r.params["value_dim"], r.params["decay"]) == (3, 8, 24, [0.5, 0.9, 0.99])
    g = l2.mixer
    assert g.kind == "general_delta" and (g.params["num_heads"], g.params["head_dim"], g.params["norm_eps"]) == (2, 20, 2e-5)
    f = l1.feed_forward
    assert f.kind == "gated_mlp" and (f.params["intermediate_size"], f.params["activation"]) == (100, "gelu_tanh")
    for n in (l0.mixer_norm, l1.parts["ffn_norm"], plan.final_norm):
        assert n.kind == "layernorm" and n.params["eps"] == 2e-5 and n.params["bias"] is True
    assert plan.final_norm.tensors == {"weight": "final.norm", "bias": "final.norm.b"}


def test_expected_tensors_are_the_checkpoint_names():
    exp = plan_for(config_from_dict(CFG)).expected_tensors()
    shapes = {k: tuple(v.shape) for k, v in exp.items()}
    assert shapes["embed"] == (101, 72) and shapes["head"] == (101, 72) and shapes["final.norm.b"] == (72,)
    assert shapes["l0.mix.left.q"] == (96, 72) and shapes["l0.mix.left.k"] == (24, 72) and shapes["l0.mix.left.v"] == (16, 72)
    assert shapes["l0.mix.left.q.norm"] == (24,) and shapes["l0.mix.left.temp"] == (4,) and shapes["l0.mix.left.g"] == (4, 72)
    assert shapes["l0.mix.left.o"] == (72, 64) and shapes["l0.mix.left.out"] == (72,)
    assert shapes["l0.mix.right.q"] == (24, 72) and shapes["l0.mix.right.v"] == (80, 72) and shapes["l0.mix.right.v.conv"] == (80, 3)
    assert shapes["l0.mix.right.b"] == (4, 72) and shapes["l0.mix.right.A_log"] == (4,) and shapes["l0.mix.right.norm"] == (20,)
    assert shapes["l0.mix.right.a1"] == (-1, 72) and shapes["l0.mix.right.a2"] == (48, -1)         # the checkpoint gives the inner sizes
    assert shapes["l0.mix.right.g2"] == (80, -1) and shapes["l0.mix.right.dt_bias"] == (48,)
    assert shapes["l1.mix.q"] == (24, 72) and shapes["l1.mix.v"] == (72, 72) and shapes["l1.mix.g"] == (72, 72)
    assert shapes["l1.mlp.gate"] == (100, 72) and shapes["l1.mlp.down"] == (72, 100) and shapes["l1.norm2.b"] == (72,)
    assert shapes["l2.mix.a.b"] == (40,) and shapes["l2.mix.w0"] == (40,) and shapes["l2.mix.norm"] == (40,) and shapes["l2.mix.w2"] == (40, -1)
    assert "l0.norm2" not in exp and "l0.ls2" not in exp and "l2.mlp.gate" not in exp
    with_rank = copy.deepcopy(CFG)
    with_rank["layers"][2]["mixer"]["decay_rank"] = 12          # random weights need the sizes
    with_rank["layers"][0]["mixer"]["right"].update(decay_rank=5, gate_rank=9)
    exp = plan_for(config_from_dict(with_rank)).expected_tensors()
    assert tuple(exp["l2.mix.w1"].shape) == (12, 72) and tuple(exp["l0.mix.right.a1"].shape) == (5, 72) and tuple(exp["l0.mix.right.g2"].shape) == (80, 9)


def test_options_that_config_leaves_out_do_not_exist():
    cfg = copy.deepcopy(CFG)
    left = cfg["layers"][0]["mixer"]["left"]
    del left["mask"], left["rot"], left["kv_heads"], left["vdim"]
    a = plan_for(config_from_dict(cfg)).layers[0].parts["left"]
    assert (a.params["chunk"], a.params["rot_dims"], a.params["num_kv_heads"], a.params["value_dim"]) == (0, 0, 4, 24)


def test_a_pair_owns_a_paged_cache_and_a_state_the_others_a_state():
    plan = plan_for(config_from_dict(CFG))
    left = mixer_cache_spec("gated_head_attention", plan.layers[0].parts["left"].params)
    assert left == {"kind": "paged", "num_kv_heads": 1, "head_dim": 32, "window": 0}       # keys of 24 and values of 16 in rows of 32
    right = mixer_cache_spec("channel_delta_rule", plan.layers[0].parts["right"].params)
    assert [t["name"] for t in right["tensors"]] == ["S", "conv"] and right["tensors"][1]["shape"] == [2, 2 * 24 + 80]
    ret = mixer_cache_spec("retention", plan.layers[1].mixer.params)
    gd = mixer_cache_spec("general_delta", plan.layers[2].mixer.params)
    assert [t["name"] for t in ret["tensors"]] == ["S"] and ret["tensors"][0]["shape"][0] >= 3 * 8 * 24
    assert gd["tensors"][0]["shape"][0] >= 2 * 20 * 20
    mgr = CacheManager([left, right, ret, gd], page_size=4, num_pages=16, num_state_slots=2)
    info = mgr.info()
    assert len(info["paged"]) == 1 and len(info["state"]) == 3
    for rid, n in ((1, 9), (2, 3)):
        mgr.add_request(rid)
        mgr.reserve(rid, n)
        mgr.commit(rid, n)
    mgr.check_invariants()
    assert mgr.free_pages() == 16 - 3 - 1
    mgr.release(1)
    mgr.release(2)
    assert mgr.free_pages() == 16


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][1].update(type="conv"), "unknown layer type 'conv'"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "unknown kind 'moe'"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.9]), "'decay' must list a number per head (3)"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "heads 4 must be a multiple of kv_heads 3"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims 7 must be even"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "conv"),
    (lambda c: c["layers"][2]["mixer"].pop("dim"), "dim"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals_name_the_key(edit, text):
    cfg = copy.deepcopy(CFG)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert text in str(e.value)
