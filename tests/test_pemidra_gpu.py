"""Pemidra against the plain implementation (tests/plain/pemidra_plain.py): every mixer alone through the part bench
(whole prompts, portions beside decoded tokens, slots and pages that are freed and used again, long decoding), whole
models through the trace runner in every way of cutting with the stream compared after every layer, and greedy
generation through the engine's own entry point and the command line.  Weights are made here so that a fault shows:
decays spread over (0, 1), removal rates and step sizes away from 0 and 1, head factors that differ, and for the
attention one loud key that late queries look for, inside and outside their chunk."""
import json
import math
import os

import numpy as np
import pytest
import torch

from imp_b200.parts.bench import PartBench
from imp_b200.parts.plan import PartSpec
from imp_b200.parts.registry import mixer_cache_spec
from plain import pemidra_plain as P
from replay_helpers import collect, mixed, portions, round64, run_trace, tail_decode, whole
from safetensors_io import save_safetensors

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
EPS = 2e-5


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def uni(*shape, seed=0, lo=0.0, hi=1.0):
    g = torch.Generator().manual_seed(seed)
    return lo + (hi - lo) * torch.rand(*shape, generator=g)


def close(got, want, dtype, what="", loose=1.0):
    got, want = got.float().cpu(), want.float().cpu()
    scale = max(float(want.abs().max()), 1e-3)
    atol, rtol = (3e-5 * scale, 3e-5) if dtype == torch.float32 else (0.025 * scale * loose, 0.025 * loose)
    err = (got - want).abs()
    assert (err <= atol + rtol * want.abs()).all(), f"{what}: max error {err.max().item():.3g} (scale {scale:.3g})"


def run_part(bench, part, x, ctx, cache=None):
    torch.cuda.synchronize()
    out = part.forward(x.to(DEV), ctx, cache)
    bench.sync()
    return out.clone()


# ------------------------------------------------------------------ weights by checkpoint suffix
def retention_weights(d, c, seed):
    H, D, Dv = c["heads"], c["dim"], c.get("vdim", c["dim"])
    s = 1.0 / math.sqrt(d)
    return {"q": rnd(H * D, d, seed=seed, scale=s), "k": rnd(H * D, d, seed=seed + 1, scale=2 * s), "v": rnd(H * Dv, d, seed=seed + 2, scale=s),
            "g": rnd(H * Dv, d, seed=seed + 3, scale=2 * s), "o": rnd(d, H * Dv, seed=seed + 4, scale=1.0 / math.sqrt(H * Dv))}


def general_delta_weights(d, c, rank, seed):
    H, D = c["heads"], c["dim"]
    s = 1.0 / math.sqrt(d)
    w = {n: rnd(H * D, d, seed=seed + i, scale=s) for i, n in enumerate("rkvg")}
    w.update({"a": rnd(H * D, d, seed=seed + 4, scale=2 * s), "a.b": rnd(H * D, seed=seed + 5),            # removal rates over (0.1, 0.9)
              "w1": rnd(rank, d, seed=seed + 6, scale=s), "w2": rnd(H * D, rank, seed=seed + 7, scale=1.5),
              "w0": -1.0 + 2.0 * rnd(H * D, seed=seed + 8),                                                 # decays from 0.55 to 1
              "norm": 1 + 0.2 * rnd(H * D, seed=seed + 9), "o": rnd(d, H * D, seed=seed + 10, scale=1.0 / math.sqrt(H * D))})
    return w


def attention_weights(d, c, seed):
    H, G, D, Dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    s = 1.0 / math.sqrt(d)
    return {"q": rnd(H * D, d, seed=seed, scale=s), "k": rnd(G * D, d, seed=seed + 1, scale=s), "v": rnd(G * Dv, d, seed=seed + 2, scale=s),
            "q.norm": 1 + 0.3 * rnd(D, seed=seed + 3), "k.norm": 1 + 0.3 * rnd(D, seed=seed + 4), "temp": uni(H, seed=seed + 5, lo=0.5, hi=2.0),
            "g": rnd(H, d, seed=seed + 6, scale=3 * s), "o": rnd(d, H * Dv, seed=seed + 7, scale=1.0 / math.sqrt(H * Dv))}


def channel_delta_weights(d, c, ra, rg, seed):
    H, G, D, Dv, taps = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"]), c["conv"]
    s = 1.0 / math.sqrt(d)
    w = {"q": rnd(G * D, d, seed=seed, scale=2 * s), "k": rnd(G * D, d, seed=seed + 1, scale=2 * s), "v": rnd(H * Dv, d, seed=seed + 2, scale=2 * s)}
    for i, (n, rows) in enumerate((("q", G * D), ("k", G * D), ("v", H * Dv))):
        w[n + ".conv"] = rnd(rows, taps, seed=seed + 3 + i, scale=0.7)             # every tap weighs: a lost input shows
    w.update({"b": rnd(H, d, seed=seed + 6, scale=3 * s), "A_log": rnd(H, seed=seed + 7, scale=0.7), "norm": 1 + 0.2 * rnd(Dv, seed=seed + 8),
              "a1": rnd(ra, d, seed=seed + 9, scale=s), "a2": rnd(H * D, ra, seed=seed + 10, scale=1.5), "dt_bias": -1.5 + rnd(H * D, seed=seed + 11),
              "g1": rnd(rg, d, seed=seed + 12, scale=s), "g2": rnd(H * Dv, rg, seed=seed + 13, scale=1.5),
              "o": rnd(d, H * Dv, seed=seed + 14, scale=1.0 / math.sqrt(H * Dv))})
    return w


def mlp_weights(d, ff, seed):
    s = 1.0 / math.sqrt(d)
    return {"gate": rnd(ff, d, seed=seed, scale=2 * s), "up": rnd(ff, d, seed=seed + 1, scale=2 * s), "down": rnd(d, ff, seed=seed + 2, scale=1.0 / math.sqrt(ff))}


RETENTION_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "gate_proj", "o": "o_proj"}
GENERAL_DELTA_NAMES = {"r": "r_proj", "k": "k_proj", "v": "v_proj", "g": "gate_proj", "a": "a_proj", "a.b": "a_bias", "w1": "decay_down", "w2": "decay_up",
                       "w0": "decay_bias", "norm": "out_norm", "o": "o_proj"}
ATTENTION_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "q.norm": "q_norm", "k.norm": "k_norm", "temp": "head_temp", "g": "gate_proj", "o": "o_proj"}
CHANNEL_DELTA_NAMES = {"q": "q_proj", "q.conv": "q_conv", "k": "k_proj", "k.conv": "k_conv", "v": "v_proj", "v.conv": "v_conv", "b": "beta_proj",
                       "A_log": "a_log", "norm": "out_norm", "a1": "decay_down", "a2": "decay_up", "dt_bias": "dt_bias", "g1": "gate_down",
                       "g2": "gate_up", "o": "o_proj"}


# --------------------------------------------------------------------- layer norm with a bias
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [72, 5000])
def test_layer_norm_with_a_bias(dtype, d):
    bench = PartBench(NAME[dtype], [], max_tokens=64)
    w, b = (1 + 0.3 * rnd(d, seed=1)).to(dtype), rnd(d, seed=4).to(dtype)
    part = bench.build("norm", PartSpec("layernorm", {"size": d, "eps": EPS, "bias": True}), {"weight": w.to(DEV), "bias": b.to(DEV)})
    h = rnd(9, d, seed=2) + 3.0
    br = rnd(9, d, seed=3).to(dtype)
    ctx = bench.prepare([("a", [1] * 9, [])])
    hd = h.to(DEV).clone()
    out = part.add_norm(hd, br.to(DEV), ctx=ctx)
    bench.sync()
    total = h.double() + br.double()
    close(hd, total, torch.float32, "stream")
    close(out, P.layer_norm(total, w.double(), b.double(), EPS), dtype, "normalised")


# ------------------------------------------------------------- the three recurrent mixers alone
def recurrent_setup(dtype, kind, case, slots=4, seed=200):
    """(bench, part, the plain function of x) for one recurrent mixer; `case` holds the sizes under the configuration's keys."""
    d = case["d"]
    if kind == "retention":
        c = {k: case[k] for k in ("heads", "dim", "vdim", "decay")}
        params = {"hidden_size": d, "num_heads": c["heads"], "key_dim": c["dim"], "value_dim": c["vdim"], "decay": c["decay"], "norm_eps": EPS}
        w, names, fn = retention_weights(d, c, seed), RETENTION_NAMES, P.retention
    elif kind == "general_delta":
        c = {k: case[k] for k in ("heads", "dim")}
        params = {"hidden_size": d, "num_heads": c["heads"], "head_dim": c["dim"], "norm_eps": EPS}
        w, names, fn = general_delta_weights(d, c, case["rank"], seed), GENERAL_DELTA_NAMES, P.general_delta
    else:
        c = {k: case[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
        params = {"hidden_size": d, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"], "key_dim": c["dim"], "value_dim": c["vdim"],
                  "conv_taps": c["conv"], "norm_eps": EPS}
        w, names, fn = channel_delta_weights(d, c, case["ra"], case["rg"], seed), CHANNEL_DELTA_NAMES, P.channel_delta_rule
    bench = PartBench(NAME[dtype], [mixer_cache_spec(kind, params)], slots=slots, max_tokens=512, max_seq_len=512)
    w = {k: v.to(dtype) for k, v in w.items()}
    part = bench.build("mixer", PartSpec(kind, params), {names[k]: v.to(DEV) for k, v in w.items()})
    W = {"m." + k: v.double() for k, v in w.items()}
    return bench, part, (lambda x: fn(x.double(), W, "m.", c, EPS)), W, c


RECURRENT_CASES = [
    ("retention", dict(d=72, heads=3, dim=8, vdim=24, decay=[0.5, 0.9, 0.99])),
    ("retention", dict(d=40, heads=1, dim=70, vdim=20, decay=[0.97])),                  # one head; a key size that is no multiple of the lanes' rows
    ("retention", dict(d=64, heads=2, dim=128, vdim=40, decay=[0.999, 0.8])),           # value columns beyond one block of 32
    ("retention", dict(d=48, heads=5, dim=12, vdim=12, decay=[0.3, 0.6, 0.9, 0.95, 1.0])),
    ("general_delta", dict(d=72, heads=2, dim=20, rank=12)),
    ("general_delta", dict(d=40, heads=1, dim=70, rank=5)),                             # an odd inner size of the decay's two matrices
    ("general_delta", dict(d=64, heads=3, dim=128, rank=16)),
    ("general_delta", dict(d=24, heads=5, dim=8, rank=4)),
    ("channel_delta_rule", dict(d=72, heads=4, kv_heads=2, dim=12, vdim=20, conv=3, ra=5, rg=9)),
    ("channel_delta_rule", dict(d=40, heads=1, kv_heads=1, dim=70, vdim=36, conv=1, ra=8, rg=8)),      # one tap: no earlier input is kept
    ("channel_delta_rule", dict(d=64, heads=6, kv_heads=1, dim=16, vdim=8, conv=4, ra=12, rg=20)),      # six heads on one key head
    ("channel_delta_rule", dict(d=48, heads=2, kv_heads=2, dim=128, vdim=64, conv=6, ra=16, rg=4)),     # more taps than a short portion has tokens
]
IDS = [f"{k}-{i}" for i, (k, _) in enumerate(RECURRENT_CASES)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind, case", RECURRENT_CASES, ids=IDS)
def test_recurrent_mixer_whole_portions_decoding_and_reused_slots(dtype, kind, case):
    bench, part, plain, _, _ = recurrent_setup(dtype, kind, case, slots=2)
    d = case["d"]
    lengths = [75, 9]
    xs = [rnd(n, d, seed=40 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [plain(x) for x in xs]
    ctx = bench.prepare([(f"w{i}", [1] * n, []) for i, n in enumerate(lengths)])
    out = run_part(bench, part, torch.cat(xs), ctx, bench.cache_view(0))
    bench.commit()
    close(out[:75], want[0], dtype, "whole", loose=2.0)
    close(out[75:], want[1], dtype, "whole, second sequence", loose=2.0)
    # both slots go back and are used again: the new requests start from a zero state and zero earlier inputs
    bench.end("w0")
    bench.end("w1")
    done, outs, other = 0, [], 0
    for n in (10, 2, 1, 1, 20, 1, 4, 2, 2, 1, 17, 3, 1, 1, 1, 1, 1, 1, 2, 3):
        es, parts = [("p0", [1] * n, [])], [xs[0][done:done + n]]
        if other < lengths[1]:
            es.append(("p1", [1], []))
            parts.append(xs[1][other:other + 1])
        ctx = bench.prepare(es)
        o = run_part(bench, part, torch.cat(parts), ctx, bench.cache_view(0))
        bench.commit()
        outs.append(o[:n])
        if other < lengths[1]:
            close(o[n:], want[1][other:other + 1], dtype, f"decoded token {other}", loose=2.0)
            other += 1
        done += n
    assert done == 75
    close(torch.cat(outs), want[0], dtype, "portions", loose=2.0)


@pytest.mark.parametrize("kind, case", [RECURRENT_CASES[0], RECURRENT_CASES[4], RECURRENT_CASES[8], RECURRENT_CASES[11]])
def test_recurrent_mixer_pieces_change_no_bit(kind, case):
    """The order of every sum is fixed by the sizes alone: however a prompt is cut, float32 results are the same bits."""
    bench, part, plain, _, _ = recurrent_setup(torch.float32, kind, case)
    x = rnd(50, case["d"], seed=77)
    ctx = bench.prepare([("a", [1] * 50, [])])
    whole_out = run_part(bench, part, x, ctx, bench.cache_view(0))
    bench.commit()
    close(whole_out, plain(x), torch.float32, "whole")
    outs, done = [], 0
    for n in (3, 2, 1, 30, 1, 13):
        ctx = bench.prepare([("b", [1] * n, [])])
        outs.append(run_part(bench, part, x[done:done + n], ctx, bench.cache_view(0)))
        bench.commit()
        done += n
    assert torch.equal(torch.cat(outs), whole_out)


@pytest.mark.parametrize("kind, case", [RECURRENT_CASES[1], RECURRENT_CASES[5], RECURRENT_CASES[10]])
def test_recurrent_mixer_long_decoding_carries_the_state(kind, case):
    """300 tokens one by one: the state (and the convolution's earlier inputs) is the only memory."""
    bench, part, plain, _, _ = recurrent_setup(torch.float32, kind, case)
    x = rnd(300, case["d"], seed=78)
    want = plain(x)
    for t in range(300):
        ctx = bench.prepare([("a", [1], [])])
        o = run_part(bench, part, x[t:t + 1], ctx, bench.cache_view(0))
        bench.commit()
        if t < 6 or t > 290 or t % 37 == 0:
            close(o, want[t:t + 1], torch.float32, f"token {t}")


def test_what_the_recurrences_rest_on_shows_in_the_plain_results():
    """The weights above make each term matter: without it the plain result moves by far more than the tests' tolerance."""
    x = rnd(60, 72, seed=90).double()
    plain, W, c = recurrent_parts_plain("retention", RECURRENT_CASES[0][1])
    want = plain(x)
    slow = dict(c, decay=[0.6, 0.9, 0.99])
    assert (P.retention(x, W, "m.", slow, EPS) - want).abs().max() > 0.02 * want.abs().max(), "one head's decay"
    plain, W, c = recurrent_parts_plain("general_delta", RECURRENT_CASES[4][1])
    want = plain(x)
    for name, what in (("m.a.b", "removal rate"), ("m.w0", "decay")):
        other = dict(W)
        other[name] = W[name] + 1.0
        assert (P.general_delta(x, other, "m.", c, EPS) - want).abs().max() > 0.02 * want.abs().max(), what
    plain, W, c = recurrent_parts_plain("channel_delta_rule", RECURRENT_CASES[8][1])
    want = plain(x)
    for name, what in (("m.dt_bias", "decay"), ("m.A_log", "decay rate"), ("m.b", "step size")):
        other = dict(W)
        other[name] = W[name] + 1.0 if name != "m.b" else W[name] * 0.0
        assert (P.channel_delta_rule(x, other, "m.", c, EPS) - want).abs().max() > 0.02 * want.abs().max(), what
    first_tap = dict(W)
    first_tap["m.k.conv"] = W["m.k.conv"].clone()
    first_tap["m.k.conv"][:, 0] = 0
    assert (P.channel_delta_rule(x, first_tap, "m.", c, EPS) - want).abs().max() > 0.02 * want.abs().max(), "the oldest tap"


def recurrent_parts_plain(kind, case, seed=200):
    """The plain function, weights and sizes of recurrent_setup without a device."""
    d = case["d"]
    if kind == "retention":
        c = {k: case[k] for k in ("heads", "dim", "vdim", "decay")}
        w, fn = retention_weights(d, c, seed), P.retention
    elif kind == "general_delta":
        c = {k: case[k] for k in ("heads", "dim")}
        w, fn = general_delta_weights(d, c, case["rank"], seed), P.general_delta
    else:
        c = {k: case[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
        w, fn = channel_delta_weights(d, c, case["ra"], case["rg"], seed), P.channel_delta_rule
    W = {"m." + k: v.double() for k, v in w.items()}
    return (lambda x: fn(x.double(), W, "m.", c, EPS)), W, c


# ------------------------------------------------------------- attention with gated heads alone
ATTENTION_CASES = [
    dict(d=72, heads=4, kv_heads=1, dim=24, vdim=16, chunk=10, rot=8, base=100.0, page=4),          # keys of 24 and values of 16 in cached rows of 32
    dict(d=64, heads=6, kv_heads=2, dim=64, vdim=64, chunk=50, rot=64, base=10000.0, page=16),      # every entry rotated; the tensor-core kernels' head size
    dict(d=40, heads=2, kv_heads=2, dim=12, vdim=20, chunk=0, rot=0, base=1.0, page=8),             # neither mask nor rotation; values longer than keys
    dict(d=48, heads=3, kv_heads=3, dim=128, vdim=96, chunk=33, rot=32, base=500.0, page=16),       # a chunk that is no multiple of a page
    dict(d=48, heads=2, kv_heads=1, dim=40, vdim=40, chunk=1, rot=20, base=50.0, page=16),          # chunks of one: a token sees itself and the sink
    dict(d=32, heads=1, kv_heads=1, dim=16, vdim=16, chunk=64, rot=2, base=7.0, page=16),           # one head, one rotated pair, chunks of whole pages
]


def attention_setup(dtype, case, w=None, scale=None):
    c = {k: case[k] for k in ("heads", "kv_heads", "dim", "vdim")}
    c["scale"] = scale or 1.7 / math.sqrt(c["dim"])
    if case["chunk"]:
        c["mask"] = {"size": case["chunk"]}
    if case["rot"]:
        c["rot"] = {"base": case["base"], "dims": case["rot"]}
    params = {"hidden_size": case["d"], "num_heads": c["heads"], "num_kv_heads": c["kv_heads"], "head_dim": c["dim"], "value_dim": c["vdim"],
              "scale": c["scale"], "norm_eps": EPS, "qk_norm": True, "value_norm": True, "rot_dims": case["rot"], "rot_base": case["base"],
              "head_temp": True, "chunk": case["chunk"], "sink": True, "head_gate": True}
    bench = PartBench(NAME[dtype], [mixer_cache_spec("gated_head_attention", params)], page_size=case["page"], num_pages=2048 // case["page"],
                      max_tokens=1024, max_seq_len=1024)
    w = {k: v.to(dtype) for k, v in (w or attention_weights(case["d"], c, seed=100)).items()}
    part = bench.build("mixer", PartSpec("gated_head_attention", params), {ATTENTION_NAMES[k]: v.to(DEV) for k, v in w.items()})
    return bench, part, c, {"m." + k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_gated_head_attention_whole_portions_decoding_and_reused_pages(dtype, case):
    bench, part, c, W = attention_setup(dtype, case)
    d = case["d"]
    lengths = [93, 11]
    xs = [rnd(n, d, seed=20 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [P.gated_head_attention(x.double(), W, "m.", c, EPS) for x in xs]
    ctx = bench.prepare([(f"w{i}", [1] * n, []) for i, n in enumerate(lengths)])
    out = run_part(bench, part, torch.cat(xs), ctx, bench.cache_view(0))
    bench.commit()
    close(out[:93], want[0], dtype, "whole")
    close(out[93:], want[1], dtype, "whole, second sequence")
    bench.end("w0")
    bench.end("w1")                       # their pages come out first for the next requests
    done, outs, other = 0, [], 0
    for n in (10, 2, 20, 1, 4, 2, 33, 1, 1, 1, 2, 16):
        es, parts = [("p0", [1] * n, [])], [xs[0][done:done + n]]
        if other < lengths[1]:
            es.append(("p1", [1], []))
            parts.append(xs[1][other:other + 1])
        ctx = bench.prepare(es)
        o = run_part(bench, part, torch.cat(parts), ctx, bench.cache_view(0))
        bench.commit()
        outs.append(o[:n])
        if other < lengths[1]:
            close(o[n:], want[1][other:other + 1], dtype, f"decoded token {other}")
            other += 1
        done += n
    assert done == 93
    close(torch.cat(outs), want[0], dtype, "portions")
    # what the design adds to plain attention shows in these weights
    if dtype == torch.float32:
        x = xs[0].double()
        assert (P.gated_head_attention(x, W, "m.", c, EPS, sink=0.0) - want[0]).abs().max() > 0.05 * want[0].abs().max(), "the sink"
        if case["rot"]:
            odd = torch.arange(93)
            odd[10:] += 1
            moved = P.gated_head_attention(x, W, "m.", c, EPS, positions=odd)
            assert (moved[:10] - want[0][:10]).abs().max() < 1e-9
            if not case["chunk"]:
                assert (moved[40] - want[0][40]).abs().max() > 1e-3 * want[0][40].abs().max(), "positions"
        if case["heads"] > 1:
            same = dict(W)
            same["m.temp"] = torch.full_like(W["m.temp"], float(W["m.temp"][0]))
            assert (P.gated_head_attention(x, same, "m.", c, EPS) - want[0]).abs().max() > 0.01 * want[0].abs().max(), "a factor per head"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_loud_key_at_the_chunk_edge_is_seen_inside_and_not_outside(dtype):
    """Chunks of 200.  Tokens 199 and 200 carry a key that every later query looks for (one unrotated entry, large on both
    sides).  Queries 200 to 399 return token 200's value, 190 keys and a dozen pages away, in a prompt cut inside the chunk
    and decoded alone; query 400 does not see it any more, and no query from 200 on sees token 199."""
    case = dict(d=64, heads=2, kv_heads=1, dim=16, vdim=16, chunk=200, rot=8, base=1e4, page=16)
    c = {k: case[k] for k in ("heads", "kv_heads", "dim", "vdim")}
    w = attention_weights(64, c, seed=300)
    w["q.norm"].fill_(1.0)
    w["k.norm"].fill_(1.0)
    w["temp"] = torch.tensor([1.5, 2.0])
    w["k"][:, 5] = 0
    w["k"][:, 7] = 0
    w["k"][15] = 0
    w["k"][15, 5] = 1.0                                # key entry 15 (not rotated) reads x[5]
    for h in range(2):
        w["q"][h * 16 + 15] = 0
        w["q"][h * 16 + 15, 6] = 4.0                   # query entry 15 reads x[6]
    T = 440
    x = rnd(T, 64, seed=301, scale=0.3)
    x[:, 5] = 0
    for t in (199, 200):
        x[t] = 0
        x[t, 5] = 9.0
    x[199, 7] = 9.0                                    # another value than token 200's, the same key
    x[201:, 6] += 4.0
    x = x.to(dtype)
    bench, part, c, W = attention_setup(dtype, case, w=w, scale=0.5)
    want = P.gated_head_attention(x.double(), W, "m.", c, EPS)
    outs = []
    for a, b in ((0, 150), (150, 199), (199, 201), (201, 380)):
        ctx = bench.prepare([("a", [1] * (b - a), [])])
        outs.append(run_part(bench, part, x[a:b], ctx, bench.cache_view(0)))
        bench.commit()
    close(torch.cat(outs), want[:380], dtype, "prompt", loose=2.0)
    for t in range(380, T):
        ctx = bench.prepare([("a", [1], [])])
        o = run_part(bench, part, x[t:t + 1], ctx, bench.cache_view(0))
        bench.commit()
        close(o, want[t:t + 1], dtype, f"decoded {t}", loose=2.0)
    xd = x.double()
    no200, no199 = xd.clone(), xd.clone()
    no200[200] = 0
    no199[199] = 0
    gone = P.gated_head_attention(no200, W, "m.", c, EPS)
    for t in (201, 300, 379, 399):
        assert (gone[t] - want[t]).abs().max() > 0.3 * want[t].abs().max(), f"token 200 must carry query {t}'s output"
    assert torch.equal(gone[400:], want[400:]) and torch.equal(P.gated_head_attention(no199, W, "m.", c, EPS)[200:], want[200:])
    for size in (199, 201):                            # an edge that is one off shows at once
        off = P.gated_head_attention(xd, W, "m.", dict(c, mask={"size": size}), EPS)
        assert (off[395:403] - want[395:403]).abs().max() > 0.3 * want[395:403].abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim,chunk", [(64, 64, 200), (128, 128, 70), (128, 96, 128), (64, 48, 333)])
def test_gated_head_attention_long_portions_with_chunk_edges_inside_tiles(dtype, dim, vdim, chunk):
    """Portions of 64 tokens and more, which the tiled prefill kernels take, with chunk edges in the middle of a tile of keys
    and of a tile of queries, rows whose chunk begins after a tile's last key, a portion that starts at an edge and one
    that ends on it; beside a second sequence that brings single tokens."""
    case = dict(d=64, heads=4, kv_heads=2, dim=dim, vdim=vdim, chunk=chunk, rot=dim // 2, base=1e4, page=16)
    bench, part, c, W = attention_setup(dtype, case)
    T = chunk + 270
    x, y = rnd(T, 64, seed=70).to(dtype), rnd(5, 64, seed=71).to(dtype)
    want, want_y = P.gated_head_attention(x.double(), W, "m.", c, EPS), P.gated_head_attention(y.double(), W, "m.", c, EPS)
    ctx = bench.prepare([("w", [1] * T, [])])
    close(run_part(bench, part, x, ctx, bench.cache_view(0)), want, dtype, "whole")
    bench.commit()
    bench.end("w")
    done, outs = 0, []
    for i, n in enumerate((chunk, 64, 130, 3, T - chunk - 197)):
        es, parts = [("p", [1] * n, [])], [x[done:done + n]]
        if i < 5:
            es.insert(0, ("s", [1], []))               # the single token leads the step
            parts.insert(0, y[i:i + 1])
        ctx = bench.prepare(es)
        o = run_part(bench, part, torch.cat(parts), ctx, bench.cache_view(0))
        bench.commit()
        close(o[:1], want_y[i:i + 1], dtype, f"single token {i}")
        outs.append(o[1:])
        done += n
    assert done == T
    close(torch.cat(outs), want, dtype, "portions")


# --------------------------------------------------------------- whole models
def attn_cfg(heads, kv, dim, vdim, chunk, rot, base=10000.0, scale=None):
    c = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or 1.5 / math.sqrt(dim)}
    if chunk:
        c["mask"] = {"size": chunk}
    if rot:
        c["rot"] = {"base": base, "dims": rot}
    return c


def delta_cfg(heads, kv, dim, vdim, taps):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}


# M1: every mixer once, the pair first and without a feed-forward, feed-forwards behind the recurrences; chunks of 24 (one
# and a half pages).  M2: two pairs of different geometry (chunks of 7 and of 100, one without rotation and with values
# longer than keys, six value heads on one key head) around a retention layer whose key and value sizes differ; a width
# that is no power of two.  M3: no pair at all: the model owns no paged cache, only states.
MODELS = {
    "M1": ({"architecture": "Pemidra", "vocab": 97, "width": 64, "norm": {"eps": 3e-5}, "postln_alpha": 1.5,
            "layers": [{"type": "parallel", "mixer": {"left": attn_cfg(4, 2, 16, 24, 24, 8, base=100.0), "right": delta_cfg(4, 2, 12, 20, 3)}, "mlp": None},
                       {"type": "retention", "mixer": {"heads": 3, "dim": 8, "vdim": 24, "decay": [0.5, 0.9, 0.99]}, "mlp": {"kind": "dense", "ff": 100}},
                       {"type": "general_delta", "mixer": {"heads": 2, "dim": 20}, "mlp": {"kind": "dense", "ff": 72}}]}, 16, (5, 7, 9)),
    "M2": ({"architecture": "Pemidra", "vocab": 211, "width": 112, "norm": {"eps": 1e-6}, "postln_alpha": 4.0,
            "layers": [{"type": "parallel", "mixer": {"left": attn_cfg(3, 3, 64, 64, 7, 64), "right": delta_cfg(6, 1, 16, 8, 5)}, "mlp": {"kind": "dense", "ff": 130}},
                       {"type": "retention", "mixer": {"heads": 1, "dim": 40, "vdim": 56, "decay": [0.97]}, "mlp": None},
                       {"type": "general_delta", "mixer": {"heads": 5, "dim": 8}, "mlp": None},
                       {"type": "parallel", "mixer": {"left": attn_cfg(2, 1, 12, 40, 100, 0), "right": delta_cfg(1, 1, 36, 36, 1)}, "mlp": None}]}, 4, (12, 5, 8)),
    "M3": ({"architecture": "Pemidra", "vocab": 130, "width": 96, "norm": {"eps": 1e-5}, "postln_alpha": 1.0,
            "layers": [{"type": "general_delta", "mixer": {"heads": 3, "dim": 32}, "mlp": None},
                       {"type": "general_delta", "mixer": {"heads": 1, "dim": 64}, "mlp": {"kind": "dense", "ff": 64}},
                       {"type": "retention", "mixer": {"heads": 4, "dim": 16, "vdim": 16, "decay": [0.6, 0.8, 0.95, 0.995]}, "mlp": None}]}, 16, (6, 4, 4)),
}
LENGTHS = {"M1": (1, 23, 75, 40, 130, 64), "M2": (150, 2, 33, 201, 64, 97), "M3": (70, 5, 140, 31, 64, 2)}


def make_weights(cfg, ranks, seed):
    """ranks: the inner sizes of (the decay of general_delta, the decay of the delta rule, its gate)."""
    d = cfg["width"]
    rg = torch.Generator().manual_seed(seed)
    W = {"embed": rnd(cfg["vocab"], d, seed=seed), "final.norm": 1 + 0.2 * rnd(d, seed=seed + 1), "final.norm.b": 0.3 * rnd(d, seed=seed + 2),
         "head": rnd(cfg["vocab"], d, seed=seed + 3, scale=1.0 / math.sqrt(d))}
    for i, lay in enumerate(cfg["layers"]):
        p, s = f"l{i}.", seed + 1000 * (i + 1)
        W[p + "norm1"] = 1 + 0.2 * rnd(d, seed=s + 1)
        W[p + "norm1.b"] = 0.3 * rnd(d, seed=s + 2)
        W[p + "ls1"] = 1.0 + 1.5 * torch.rand(d, generator=rg)                      # a mixer weighs as much as the stream it joins
        m = lay["mixer"]
        if lay["type"] == "retention":
            mix = retention_weights(d, m, s + 10)
        elif lay["type"] == "general_delta":
            mix = general_delta_weights(d, m, ranks[0], s + 10)
        else:
            mix = {"left." + k: v for k, v in attention_weights(d, m["left"], s + 10).items()}
            mix.update({"right." + k: v for k, v in channel_delta_weights(d, m["right"], ranks[1], ranks[2], s + 40).items()})
            mix["left.out"] = 1 + 0.3 * rnd(d, seed=s + 70)
            mix["right.out"] = 1 + 0.3 * rnd(d, seed=s + 71)
        for k, v in mix.items():
            W[p + "mix." + k] = v
        if lay["mlp"]:
            W[p + "norm2"] = 1 + 0.2 * rnd(d, seed=s + 3)
            W[p + "norm2.b"] = 0.3 * rnd(d, seed=s + 4)
            W[p + "ls2"] = 1.0 + 1.5 * torch.rand(d, generator=rg)
            for k, v in mlp_weights(d, lay["mlp"]["ff"], s + 80).items():
                W[p + "mlp." + k] = v
    return {k: v.to(torch.bfloat16) for k, v in W.items()}


@pytest.fixture(scope="module")
def pemidra_folders(tmp_path_factory):
    out = {}
    for n, (name, (cfg, page, ranks)) in enumerate(MODELS.items()):
        folder = str(tmp_path_factory.mktemp(f"pemidra_{name}"))
        W = make_weights(cfg, ranks, seed=70 + n)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_safetensors(os.path.join(folder, "model.safetensors"), W)
        g = torch.Generator().manual_seed(n)
        reqs = {f"r{i}": torch.randint(0, cfg["vocab"], (m,), generator=g).tolist() for i, m in enumerate(LENGTHS[name])}
        Wd = {k: v.double() for k, v in W.items()}
        ref = {rid: P.forward(ids, Wd, cfg).float().numpy() for rid, ids in reqs.items()}
        out[name] = (folder, cfg, page, Wd, reqs, ref)
    return out


def check_rows(rows, reqs, ref, dtype, label=""):
    """float32: every logit to 1e-4 of the largest.  bfloat16: a row's root-mean-square error is at most 4 % of the root
    mean square of all logits for 95 of 100 rows and 15 % for every row."""
    scale = max(float(np.abs(r).max()) for r in ref.values())
    rms_all = float(np.sqrt(np.mean(np.concatenate([r.ravel() for r in ref.values()]) ** 2)))
    rel, n = [], 0
    for rid, ids in reqs.items():
        for p in range(len(ids)):
            got, want = rows[(rid, p)], ref[rid][p]
            err = np.abs(got - want)
            if dtype == "float32":
                assert not (err > 1e-4 * max(scale, 1.0) + 1e-4 * np.abs(want)).any(), \
                    f"{label}: request {rid} position {p}: max error {err.max():.3g} (largest logit {scale:.3g}) in {dtype}"
            else:
                rel.append(float(np.sqrt(np.mean(err ** 2))) / rms_all)
                assert rel[-1] <= 0.15, f"{label}: request {rid} position {p}: rms error {rel[-1]:.3g} of the logits' rms in {dtype}"
            n += 1
    assert n == sum(len(v) for v in reqs.values())
    if rel:
        assert float(np.quantile(rel, 0.95)) <= 0.04, f"{label}: 95th percentile of the rows' rms error {np.quantile(rel, 0.95):.3g} in {dtype}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M1", "M2", "M3"])
def test_replay_all_ways_of_cutting(name, dtype, pemidra_folders, tmp_path):
    folder, cfg, page, W, reqs, ref = pemidra_folders[name]
    V = cfg["vocab"]
    longest = round64(max(len(v) for v in reqs.values()))
    results = {}
    cuts = [("whole", whole(reqs), longest), ("tail", tail_decode(reqs), longest), ("portions", portions(reqs), longest),
            ("wide_portions", portions(reqs, sizes=(70, 2, 33, 64, 1, 100)), longest)]
    for label, steps, pool in cuts:
        out = run_trace(folder, dtype, steps, pool, str(tmp_path / label), V, page_size=page)
        rows = collect(steps, out)
        check_rows(rows, reqs, ref, dtype, label)
        results[label] = rows
    steps, peak = mixed(reqs)
    assert max(len(s["entries"]) for s in steps) == 4
    assert peak < sum(round64(len(v)) for v in reqs.values()), "the pool must be too small to avoid reuse"
    out = run_trace(folder, dtype, steps, peak, str(tmp_path / "mixed"), V, page_size=page)
    rows = collect(steps, out)
    check_rows(rows, reqs, ref, dtype, "mixed")
    results["mixed"] = rows
    if dtype == "float32":
        # every reduction of the float32 path has an order that depends on the row alone
        for label in [c[0] for c in cuts[1:]] + ["mixed"]:
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[label][key]), f"{label}: {key} differs from the whole run"


@pytest.mark.parametrize("name", ["M1", "M2"])
def test_the_stream_after_every_layer(name, pemidra_folders, tmp_path, monkeypatch):
    """The first layer that differs names the mechanism: the stream after every layer of one prompt, in float32."""
    folder, cfg, page, W, reqs, ref = pemidra_folders[name]
    ids = reqs["r2"]
    streams = []
    P.forward(ids, W, cfg, streams=streams)
    dump = tmp_path / "streams"
    dump.mkdir()
    monkeypatch.setenv("IMP_B200_DUMP_STREAM", str(dump))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids, "want": [len(ids) - 1]}], "end": ["a"]}]
    run_trace(folder, "float32", steps, round64(len(ids)), str(tmp_path / "out"), cfg["vocab"], page_size=page)
    for j, want in enumerate(streams):
        got = torch.from_numpy(np.fromfile(dump / f"step0_run{j}.f32", dtype="<f4").reshape(len(ids), cfg["width"]).copy())
        close(got, want, torch.float32, f"{name}: stream after layer {j} ({cfg['layers'][j]['type']})")


def test_greedy_generation_through_the_engine(pemidra_folders):
    """Prompts of unequal length through submit / schedule / step / sample with short prefill portions; the tokens are
    those of the plain model's argmax, and pages and slots all come back."""
    from imp_b200 import Engine, EngineConfig, GenerateParams
    folder, cfg, page, W, reqs, ref = pemidra_folders["M2"]
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 7, 30, 12, 3)]

    def plain_generate(ids, n):
        ids, out = list(ids), []
        for _ in range(n):
            tok = int(torch.argmax(P.forward(ids, W, cfg)[-1]))
            out.append(tok)
            ids.append(tok)
        return out

    want = [plain_generate(p, 8) for p in prompts]
    eng = Engine.from_folder(folder, EngineConfig(compute_dtype="float32", kv_block_size=page, max_batch_size=3, max_seq_len=256,
                                                  kv_cache_tokens=1024, max_batch_tokens=32, prefill_chunk_size=8))
    got = eng.generate(prompts, GenerateParams(max_tokens=8, temperature=0.0))
    assert got == want
    assert eng.free_pages() == eng.num_pages and not eng.has_work()
    info = eng.info()
    assert info["cache"]["free_slots"] == info["cache"]["slots"]
    # the same with CUDA graphs for the decode steps in bfloat16: first tokens from well separated logits agree
    eng16 = Engine.from_folder(folder, EngineConfig(compute_dtype="bfloat16", kv_block_size=page, max_batch_size=4, max_seq_len=256,
                                                    kv_cache_tokens=1024, max_batch_tokens=64))
    got16 = eng16.generate(prompts, GenerateParams(max_tokens=8, temperature=0.0))
    assert eng16.info()["model"]["graph_safe"]
    for p, g16, w in zip(prompts, got16, want):
        lg = P.forward(p, W, cfg)[-1]
        top2 = torch.topk(lg, 2).values
        if float(top2[0] - top2[1]) > 0.1 * float(lg.abs().max()):
            assert g16[0] == w[0]


def test_command_line_with_a_checkpoint_and_with_random_weights(pemidra_folders, tmp_path):
    import subprocess
    import sys
    cli = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "imp-cli")
    folder, cfg, page, W, reqs, ref = pemidra_folders["M1"]
    ids, want = [5, 17, 3], []
    for _ in range(6):
        want.append(int(torch.argmax(P.forward(ids + want, W, cfg)[-1])))
    p = subprocess.run([sys.executable, cli, "--model", folder, "--prompt", "5,17,3", "--max-tokens", "6", "--temperature", "0",
                        "--dtype", "fp32", "--page-size", str(page), "--kv-pages", "64", "--max-seq-len", "128"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()] == want
    only_config = tmp_path / "cfg"
    only_config.mkdir()
    with_rank = json.loads(json.dumps(cfg))
    for lay in with_rank["layers"]:                    # no checkpoint gives the inner sizes
        if lay["type"] == "general_delta":
            lay["mixer"]["decay_rank"] = 8
        if lay["type"] == "parallel":
            lay["mixer"]["right"].update(decay_rank=8, gate_rank=8)
    (only_config / "config.json").write_text(json.dumps(with_rank))
    b = subprocess.run([sys.executable, cli, "--model", str(only_config), "--random-weights", "--weights-seed", "3", "--kv-pages", "64",
                        "--max-seq-len", "256", "--bench", "--bench-pp", "48", "--max-tokens", "8", "--bench-reps", "2", "--bench-batch", "2"],
                       capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-2000:]
    assert "pp    96 tokens" in b.stderr and "tg    16 tokens" in b.stderr
