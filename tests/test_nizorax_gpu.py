"""Nizorax against the plain implementation (tests/plain/nizorax_plain.py): every mechanism alone through the part bench
(whole prompts, portions beside decoded tokens, slots and pages that are freed and used again, long decoding), whole
models through the trace runner in every way of cutting with the stream compared after every layer, and greedy
generation through the engine's own entry point and the command line.  Weights are made here so that a fault shows:
decays spread over (0, 1), every tap of a convolution weighing, and for the attention one loud key that late queries
look for, just inside and just outside their window and far away."""
import json
import math
import os

import numpy as np
import pytest
import torch

from imp_b200.parts.bench import PartBench
from imp_b200.parts.plan import PartSpec
from imp_b200.parts.registry import mixer_cache_spec
from plain import nizorax_plain as N
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


def pieces_beside_a_decoding_sequence(bench, part, xs, want, dtype, sizes, loose=1.0):
    """The first sequence in portions of `sizes`, the second one token at a time beside it."""
    done, outs, other = 0, [], 0
    for n in sizes:
        es, parts = [("p0", [1] * n, [])], [xs[0][done:done + n]]
        if other < xs[1].shape[0]:
            es.append(("p1", [1], []))
            parts.append(xs[1][other:other + 1])
        ctx = bench.prepare(es)
        o = run_part(bench, part, torch.cat(parts), ctx, bench.cache_view(0))
        bench.commit()
        outs.append(o[:n])
        if other < xs[1].shape[0]:
            close(o[n:], want[1][other:other + 1], dtype, f"decoded token {other}", loose=loose)
            other += 1
        done += n
    assert done == xs[0].shape[0]
    close(torch.cat(outs), want[0], dtype, "portions", loose=loose)


# ------------------------------------------------------------------ weights by checkpoint suffix
def attention_weights(d, c, seed):
    H, G, D, Dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    s = 1.0 / math.sqrt(d)
    return {"q": rnd(H * 2 * D, d, seed=seed, scale=s), "k": rnd(G * 2 * D, d, seed=seed + 1, scale=s), "v": rnd(G * Dv, d, seed=seed + 2, scale=s),
            "lq1": rnd(D, seed=seed + 3, scale=0.3), "lk1": rnd(D, seed=seed + 4, scale=0.3), "lq2": rnd(D, seed=seed + 5, scale=0.3),
            "lk2": rnd(D, seed=seed + 6, scale=0.3), "o": rnd(d, H * Dv, seed=seed + 7, scale=1.0 / math.sqrt(H * Dv))}


def lightning_weights(d, c, seed):
    H, D, Dv = c["heads"], c["dim"], c.get("vdim", c["dim"])
    s = 1.0 / math.sqrt(d)
    return {"q": rnd(H * D, d, seed=seed, scale=2 * s), "k": rnd(H * D, d, seed=seed + 1, scale=2 * s), "v": rnd(H * Dv, d, seed=seed + 2, scale=2 * s),
            "g": rnd(H * Dv, d, seed=seed + 3, scale=2 * s), "norm": 1 + 0.3 * rnd(H * Dv, seed=seed + 5),
            "o": rnd(d, H * Dv, seed=seed + 4, scale=1.0 / math.sqrt(H * Dv))}


def dense_weights(d, ff, seed):
    s = 1.0 / math.sqrt(d)
    return {"up": rnd(ff, d, seed=seed, scale=2 * s), "down": rnd(d, ff, seed=seed + 1, scale=1.0 / math.sqrt(ff)),
            "act": torch.tensor([0.9, 0.5, -0.3, 0.2]) + 0.1 * rnd(4, seed=seed + 2)}


def moe_weights(d, c, seed):
    E, F = c["router"]["experts"], c["expert"]["ff"]
    s = 1.0 / math.sqrt(d)
    w = {"router": rnd(E, d, seed=seed, scale=1.5 * s)}                     # scores spread over (0, 1) without saturating: choices rarely hang on rounding
    for e in range(E):
        w[f"e{e}.gate"] = rnd(F, d, seed=seed + 10 * e + 1, scale=2 * s)
        w[f"e{e}.up"] = rnd(F, d, seed=seed + 10 * e + 2, scale=2 * s)
        w[f"e{e}.down"] = rnd(d, F, seed=seed + 10 * e + 3, scale=1.0 / math.sqrt(F))
    if c.get("shared"):
        Fs = c["shared"]["ff"]
        w.update({"shared.gate": rnd(Fs, d, seed=seed + 7, scale=2 * s), "shared.up": rnd(Fs, d, seed=seed + 8, scale=2 * s),
                  "shared.down": rnd(d, Fs, seed=seed + 9, scale=1.0 / math.sqrt(Fs))})
    return w


ATTENTION_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2", "lk2": "lambda_k2", "o": "o_proj"}
LIGHTNING_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "gate_proj", "norm": "out_norm", "o": "o_proj"}


def moe_names(c):
    names = {"router": "router"}
    for e in range(c["router"]["experts"]):
        names.update({f"e{e}.gate": f"gate_{e}", f"e{e}.up": f"up_{e}", f"e{e}.down": f"down_{e}"})
    if c.get("shared"):
        names.update({"shared.gate": "shared_gate", "shared.up": "shared_up", "shared.down": "shared_down"})
    return names


def moe_params(d, c):
    r = c["router"]
    g = r.get("groups") or {}
    return {"hidden_size": d, "num_experts": r["experts"], "top_k": r["top"], "expert_size": c["expert"]["ff"],
            "shared_size": (c.get("shared") or {}).get("ff", 0), "router_bias": False, "shared_gate": False, "scores": "sigmoid",
            "weight_scale": r.get("scale", 1.0), "num_groups": g.get("count", 0), "keep_groups": g.get("keep", 0)}


# ------------------------------------------------- a branch with a norm of its own, the sum and the next norm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [70, 72, 4096, 8200, 9001])
def test_branch_norm_sum_and_next_norm_in_one_launch(dtype, d):
    """Widths that take each form of the kernel: rows in registers (multiples of 4 up to 8,192), rows in shared memory
    (the rest); rows with a large mean; a gather list that leaves the stream as it is; the branch's norm alone."""
    from imp_b200.ops import kernels as K
    n = 7
    bw, bb = (1 + 0.3 * rnd(d, seed=1)).to(dtype), rnd(d, seed=2).to(dtype)
    w, b = (1 + 0.3 * rnd(d, seed=3)).to(dtype), rnd(d, seed=4).to(dtype)
    h = rnd(n, d, seed=5) * 3 + 2.0
    br = (rnd(n, d, seed=6) * 2 + 5.0).to(dtype)
    normed = N.layer_norm(br.double(), bw.double(), bb.double(), 3e-5)
    total = h.double() + normed
    want = N.layer_norm(total, w.double(), b.double(), EPS)
    hd, out = h.to(DEV).clone(), torch.empty(n, d, dtype=dtype, device=DEV)
    K.add_normed_layernorm(hd, br.to(DEV), bw.to(DEV), bb.to(DEV), 3e-5, w.to(DEV), b.to(DEV), EPS, out)
    torch.cuda.synchronize()
    close(hd, total, torch.float32, "stream")
    close(out, want, dtype, "normalised")
    rows = torch.tensor([5, 0, 3], dtype=torch.int32, device=DEV)
    hd2, out3 = h.to(DEV).clone(), torch.empty(3, d, dtype=dtype, device=DEV)
    K.add_normed_layernorm(hd2, br.to(DEV), bw.to(DEV), bb.to(DEV), 3e-5, w.to(DEV), b.to(DEV), EPS, out3, rows=rows)
    torch.cuda.synchronize()
    assert torch.equal(hd2.cpu(), h), "a gather list leaves the stream as it is"
    assert torch.equal(out3, out[rows.long()]), "the gathered rows are the rows of the whole launch"
    alone = torch.empty(n, d, dtype=dtype, device=DEV)
    K.add_normed_layernorm(None, br.to(DEV), bw.to(DEV), bb.to(DEV), 3e-5, None, None, 0.0, alone)
    torch.cuda.synchronize()
    close(alone, normed, dtype, "the branch's norm alone")


# --------------------------------------------------------------- the convolution on a sublayer's input
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps, d", [(1, 40), (2, 72), (4, 300), (6, 64)])
def test_residual_conv_whole_portions_decoding_and_reused_slots(dtype, taps, d):
    params = {"hidden_size": d, "taps": taps}
    bench = PartBench(NAME[dtype], [mixer_cache_spec("residual_conv", params)], slots=2, max_tokens=256, max_seq_len=256)
    w = rnd(d, taps, seed=3, scale=0.7).to(dtype)                                   # every tap weighs: a lost input shows
    part = bench.build("mixer", PartSpec("residual_conv", params), {"weight": w.to(DEV)})
    lengths = [61, 9]
    xs = [rnd(n, d, seed=40 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [N.add_causal_conv(x.double(), w.double()) for x in xs]
    ctx = bench.prepare([(f"w{i}", [1] * n, []) for i, n in enumerate(lengths)])
    out = run_part(bench, part, torch.cat(xs), ctx, bench.cache_view(0))
    bench.commit()
    close(out[:61], want[0], dtype, "whole")
    close(out[61:], want[1], dtype, "whole, second sequence")
    bench.end("w0")
    bench.end("w1")            # both slots go back; the next requests start from zero inputs
    pieces_beside_a_decoding_sequence(bench, part, xs, want, dtype, (10, 2, 1, 1, 20, 1, 4, 2, 2, 1, 3, 1, 1, 1, 1, 2, 2, 6))
    if taps > 1:
        first_tap = w.double().clone()
        first_tap[:, 0] = 0
        assert (N.add_causal_conv(xs[0].double(), first_tap) - want[0]).abs().max() > 0.1 * want[0].abs().max(), "the oldest tap weighs"


# ------------------------------------------------------------------- differential attention alone
SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
ATTENTION_CASES = [
    dict(d=72, heads=6, kv_heads=2, dim=24, vdim=40, window=10, rot=8, base=100.0, scaling=SCALING, page=4),      # keys of 24 and values of 40 in cached rows of 48
    dict(d=64, heads=4, kv_heads=4, dim=64, vdim=64, window=50, rot=64, base=10000.0, scaling=None, page=16),     # a key head per head; every entry rotated
    dict(d=40, heads=2, kv_heads=1, dim=12, vdim=20, window=0, rot=0, base=1.0, scaling=None, page=8),            # neither window nor rotation
    dict(d=48, heads=3, kv_heads=1, dim=128, vdim=96, window=33, rot=32, base=500.0, scaling=SCALING, page=16),   # a window that is no multiple of a page
    dict(d=32, heads=1, kv_heads=1, dim=16, vdim=16, window=1, rot=2, base=7.0, scaling=None, page=16),           # a window of one: a token sees itself
    dict(d=48, heads=5, kv_heads=5, dim=20, vdim=8, window=64, rot=20, base=50.0, scaling=None, page=16),         # values shorter than keys; a window of whole pages
]


def attention_config(case, diff=0.4, scale=None):
    c = {k: case[k] for k in ("heads", "kv_heads", "dim", "vdim")}
    c["scale"] = scale or 1.7 / math.sqrt(c["dim"])
    c["diff"] = diff
    if case["window"]:
        c["mask"] = {"size": case["window"]}
    if case["rot"]:
        c["rot"] = {"base": case["base"], "dims": case["rot"]}
        if case["scaling"]:
            c["rot"]["scaling"] = case["scaling"]
    return c


def attention_setup(dtype, case, w=None, diff=0.4, scale=None):
    c = attention_config(case, diff, scale)
    params = {"hidden_size": case["d"], "num_heads": c["heads"], "num_kv_heads": c["kv_heads"], "head_dim": c["dim"], "value_dim": c["vdim"],
              "scale": c["scale"], "lambda_init": diff, "norm_eps": EPS, "window": case["window"], "rot_dims": case["rot"], "rot_base": case["base"],
              "rot_pairing": "neighbours"}
    if case["scaling"] and case["rot"]:
        params["rot_scaling"] = case["scaling"]
    bench = PartBench(NAME[dtype], [mixer_cache_spec("differential_attention", params)], page_size=case["page"], num_pages=2048 // case["page"],
                      max_tokens=1024, max_seq_len=1024)
    w = {k: v.to(dtype) for k, v in (w or attention_weights(case["d"], c, seed=100)).items()}
    part = bench.build("mixer", PartSpec("differential_attention", params), {ATTENTION_NAMES[k]: v.to(DEV) for k, v in w.items()})
    return bench, part, c, {"m." + k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_differential_attention_whole_portions_decoding_and_reused_pages(dtype, case):
    bench, part, c, W = attention_setup(dtype, case)
    d = case["d"]
    lengths = [93, 11]
    xs = [rnd(n, d, seed=20 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [N.differential_attention(x.double(), W, "m.", c, EPS) for x in xs]
    ctx = bench.prepare([(f"w{i}", [1] * n, []) for i, n in enumerate(lengths)])
    out = run_part(bench, part, torch.cat(xs), ctx, bench.cache_view(0))
    bench.commit()
    close(out[:93], want[0], dtype, "whole", loose=2.0)
    close(out[93:], want[1], dtype, "whole, second sequence", loose=2.0)
    bench.end("w0")
    bench.end("w1")                       # their pages come out first for the next requests
    pieces_beside_a_decoding_sequence(bench, part, xs, want, dtype, (10, 2, 20, 1, 4, 2, 33, 1, 1, 1, 2, 16), loose=2.0)


def test_what_differential_attention_rests_on_shows_in_the_plain_results():
    case = ATTENTION_CASES[0]
    c = attention_config(case)
    W = {"m." + k: v.double() for k, v in attention_weights(case["d"], c, seed=100).items()}
    x = rnd(60, case["d"], seed=20).double()
    want = N.differential_attention(x, W, "m.", c, EPS)
    far = lambda other: float((other - want).abs().max()) > 0.02 * float(want.abs().max())
    assert far(N.differential_attention(x, W, "m.", dict(c, diff=0.7), EPS)), "lambda's constant and the output's factor"
    assert far(N.differential_attention(x, W, "m.", dict(c, mask={"size": 11}), EPS)), "one more key in the window"
    assert far(N.differential_attention(x, W, "m.", dict(c, rot={"base": 100.0, "dims": 8}), EPS)), "the slowed wavelengths"
    assert far(N.differential_attention(x, W, "m.", c, EPS, positions=torch.arange(60) * 2)), "positions"
    swapped = dict(W)
    swapped["m.lq1"], swapped["m.lq2"] = W["m.lq2"], W["m.lq1"]
    assert far(N.differential_attention(x, swapped, "m.", c, EPS)), "lambda's vectors"


def loud_key_weights(case, c, seed):
    """Random weights plus one direction u of the input that every query's first map and every key's first map pick up in an
    entry that is not rotated: a token with much of u is a key that later tokens with some u look for."""
    d, D = case["d"], case["dim"]
    w = attention_weights(d, c, seed)
    u = torch.zeros(d)
    u[0] = 1.0
    at = D - 1                                       # beyond the rotated front
    assert at >= case["rot"]
    for h in range(c["heads"]):
        w["q"][(h * 2) * D + at] += 3.0 * u
    for g in range(c["kv_heads"]):
        w["k"][(g * 2) * D + at] += 3.0 * u
    return w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decoded", [False, True])
def test_a_loud_key_just_inside_and_just_outside_the_window_and_far_away(dtype, decoded):
    """The token at `at` is the key every later token looks for.  The query at at + window - 1 still sees it, the one at
    at + window does not; without a window a query 600 tokens later finds it among all the others.  In a prompt, and with
    the last tokens decoded one by one."""
    for case, T, at in ((dict(d=48, heads=3, kv_heads=1, dim=32, vdim=24, window=37, rot=8, base=100.0, scaling=SCALING, page=16), 120, 50),
                        (dict(d=48, heads=2, kv_heads=2, dim=16, vdim=16, window=64, rot=0, base=1.0, scaling=None, page=16), 150, 63),
                        (dict(d=40, heads=2, kv_heads=1, dim=16, vdim=32, window=0, rot=4, base=100.0, scaling=None, page=16), 640, 3)):
        c = attention_config(case, scale=1.0)
        bench, part, c, W = attention_setup(dtype, case, w=loud_key_weights(case, c, seed=300), scale=1.0)
        x = rnd(T, case["d"], seed=301, scale=0.5)
        x[:, 0] = 1.0                                  # some u in every token
        x[at, 0] = 6.0                                 # the loud one
        x = x.to(dtype)
        want = N.differential_attention(x.double(), W, "m.", c, EPS)
        quiet = x.clone()
        quiet[at, 0] = 1.0
        without = N.differential_attention(quiet.double(), W, "m.", c, EPS)
        moved = (want - without).abs().amax(dim=-1) / want.abs().max()
        win = case["window"]
        if win:
            assert moved[at + win - 1] > 0.2 and moved[at + win] < 1e-9, "the plain result hangs on the key exactly inside the window"
        else:
            assert moved[T - 1] > 0.2, "the plain result hangs on the far key"
        n_tail = 40 if decoded else 0
        cuts = [T - n_tail] + [1] * n_tail
        if decoded and win:
            assert T - n_tail <= at + win - 1, "the edge is passed while decoding"
        outs, done = [], 0
        for n in cuts:
            ctx = bench.prepare([("a", [1] * n, [])])
            outs.append(run_part(bench, part, x[done:done + n], ctx, bench.cache_view(0)))
            bench.commit()
            done += n
        out = torch.cat(outs)
        close(out, want, dtype, f"window {win}", loose=2.0)
        bench.end("a")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_with_window_edges_inside_the_kernels_tiles(dtype):
    """Portions of hundreds of tokens take the tiled kernels; the window's edge falls inside their tiles."""
    case = dict(d=64, heads=2, kv_heads=1, dim=64, vdim=64, window=150, rot=16, base=1000.0, scaling=SCALING, page=16)
    bench, part, c, W = attention_setup(dtype, case)
    T = 700
    x = rnd(T, case["d"], seed=21).to(dtype)
    want = N.differential_attention(x.double(), W, "m.", c, EPS)
    outs, done = [], 0
    for n in (300, 257, 2, 141):
        ctx = bench.prepare([("a", [1] * n, [])])
        outs.append(run_part(bench, part, x[done:done + n], ctx, bench.cache_view(0)))
        bench.commit()
        done += n
    close(torch.cat(outs), want, dtype, "long portions", loose=2.0)


# ------------------------------------------------------------------------------- lightning alone
LIGHTNING_CASES = [
    dict(d=72, heads=3, dim=8, vdim=24, decay=[0.5, 0.9, 0.99]),
    dict(d=40, heads=1, dim=70, vdim=20, decay=[0.97]),                     # one head; a key size that is no multiple of the lanes' rows
    dict(d=64, heads=2, dim=128, vdim=40, decay=[0.999, 0.8]),              # value columns beyond one block of 32
    dict(d=48, heads=5, dim=12, vdim=12, decay=[0.3, 0.6, 0.9, 0.95, 1.0]),
]


def lightning_setup(dtype, case, slots=4, seed=200):
    c = {k: case[k] for k in ("heads", "dim", "vdim", "decay")}
    d = case["d"]
    params = {"hidden_size": d, "num_heads": c["heads"], "key_dim": c["dim"], "value_dim": c["vdim"], "decay": c["decay"], "norm_eps": EPS,
              "key_scale": 1.0, "qkv_act": "silu", "gate_act": "sigmoid", "norm_over": "row", "out_norm": True}
    bench = PartBench(NAME[dtype], [mixer_cache_spec("retention", params)], slots=slots, max_tokens=512, max_seq_len=512)
    w = {k: v.to(dtype) for k, v in lightning_weights(d, c, seed).items()}
    part = bench.build("mixer", PartSpec("retention", params), {LIGHTNING_NAMES[k]: v.to(DEV) for k, v in w.items()})
    W = {"m." + k: v.double() for k, v in w.items()}
    return bench, part, (lambda x: N.lightning(x.double(), W, "m.", c, EPS)), W, c


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", LIGHTNING_CASES)
def test_lightning_whole_portions_decoding_and_reused_slots(dtype, case):
    bench, part, plain, _, _ = lightning_setup(dtype, case, slots=2)
    d = case["d"]
    lengths = [75, 9]
    xs = [rnd(n, d, seed=40 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [plain(x) for x in xs]
    ctx = bench.prepare([(f"w{i}", [1] * n, []) for i, n in enumerate(lengths)])
    out = run_part(bench, part, torch.cat(xs), ctx, bench.cache_view(0))
    bench.commit()
    close(out[:75], want[0], dtype, "whole", loose=2.0)
    close(out[75:], want[1], dtype, "whole, second sequence", loose=2.0)
    bench.end("w0")
    bench.end("w1")
    pieces_beside_a_decoding_sequence(bench, part, xs, want, dtype, (10, 2, 1, 1, 20, 1, 4, 2, 2, 1, 17, 3, 1, 1, 1, 1, 1, 1, 2, 3), loose=2.0)


def test_lightning_pieces_change_no_bit_and_long_decoding_carries_the_state():
    bench, part, plain, W, c = lightning_setup(torch.float32, LIGHTNING_CASES[0])
    x = rnd(50, 72, seed=77)
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
    want = plain(x)
    assert (N.lightning(x.double(), W, "m.", dict(c, decay=[0.6, 0.9, 0.99]), EPS) - want).abs().max() > 0.02 * want.abs().max(), "one head's decay"
    flat = dict(W)
    flat["m.norm"] = torch.ones_like(W["m.norm"])
    assert (N.lightning(x.double(), flat, "m.", c, EPS) - want).abs().max() > 0.02 * want.abs().max(), "the norm's weight"
    bench, part, plain, _, _ = lightning_setup(torch.float32, LIGHTNING_CASES[2])
    x = rnd(300, 64, seed=78)
    want = plain(x)
    for t in range(300):
        ctx = bench.prepare([("a", [1], [])])
        o = run_part(bench, part, x[t:t + 1], ctx, bench.cache_view(0))
        bench.commit()
        if t < 6 or t > 290 or t % 37 == 0:
            close(o, want[t:t + 1], torch.float32, f"token {t}")


# ------------------------------------------------------------------------------ feed-forwards alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, ff", [(72, 100), (64, 256), (40, 37)])
def test_polynorm_feed_forward(dtype, d, ff):
    bench = PartBench(NAME[dtype], [], max_tokens=256)
    w = {k: v.to(dtype) for k, v in dense_weights(d, ff, seed=600).items()}
    part = bench.build("feed_forward", PartSpec("polynorm_mlp", {"hidden_size": d, "intermediate_size": ff, "norm_eps": EPS}),
                       {"up_proj": w["up"].to(DEV), "down_proj": w["down"].to(DEV), "coef": w["act"].to(DEV)})
    W = {"f." + k: v.double() for k, v in w.items()}
    x = rnd(70, d, seed=601, scale=2.0).to(dtype)
    want = N.dense_ff(x.double(), W, "f.", EPS)
    ctx = bench.prepare([("a", [1] * 70, [])])
    out = run_part(bench, part, x, ctx)
    close(out, want, dtype, "whole", loose=2.0)
    for i, what in enumerate(("the first power", "the square", "the cube", "the constant")):
        other = dict(W)
        other["f.act"] = W["f.act"].clone()
        other["f.act"][i] += 0.5
        assert (N.dense_ff(x.double(), other, "f.", EPS) - want).abs().max() > 0.02 * want.abs().max(), what
    ctx = bench.prepare([("b", [1] * 2, [])])
    two = run_part(bench, part, x[5:7], ctx)
    if dtype == torch.float32:
        assert torch.equal(two, out[5:7]), "a token's result does not depend on its neighbours"


MOE_CASES = [
    dict(d=72, experts=12, top=2, ff=20, shared=36, scale=2.5, groups=(4, 2)),
    dict(d=64, experts=6, top=1, ff=32, shared=0, scale=1.0, groups=None),               # one expert a token, no groups, no shared expert
    dict(d=40, experts=16, top=3, ff=24, shared=24, scale=0.7, groups=(16, 5)),          # groups of one expert
    dict(d=48, experts=8, top=4, ff=16, shared=8, scale=1.5, groups=(2, 2)),             # every group kept
    dict(d=48, experts=70, top=6, ff=8, shared=0, scale=1.0, groups=(7, 3)),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", MOE_CASES)
def test_routed_experts_with_sigmoid_scores_and_groups(dtype, case):
    c = {"router": {"experts": case["experts"], "top": case["top"], "scale": case["scale"]}, "expert": {"ff": case["ff"]},
         "shared": {"ff": case["shared"]} if case["shared"] else None}
    if case["groups"]:
        c["router"]["groups"] = {"count": case["groups"][0], "keep": case["groups"][1]}
    d = case["d"]
    w = {k: v.to(dtype) for k, v in moe_weights(d, c, seed=500).items()}
    bench = PartBench(NAME[dtype], [], max_tokens=256)
    names = moe_names(c)
    part = bench.build("feed_forward", PartSpec("routed_experts", moe_params(d, c)), {names[k]: v.to(DEV) for k, v in w.items()})
    W = {"f." + k: v.double() for k, v in w.items()}
    x = rnd(150, d, seed=501).to(dtype)
    want = N.moe(x.double(), W, "f.", c)
    sure = N.route_margin(x.double(), W, "f.", c) > 1e-3           # rows whose choice hangs on less than rounding are not judged
    assert sure.sum() > 120
    ctx = bench.prepare([("a", [1] * 150, [])])
    out = run_part(bench, part, x, ctx)
    close(out[sure], want[sure], dtype, "whole", loose=2.0)
    outs, done = [], 0
    for n in (3, 1, 2, 64, 70, 10):
        ctx = bench.prepare([("b", [1] * n, [])])
        outs.append(run_part(bench, part, x[done:done + n], ctx))
        done += n
    pieces = torch.cat(outs)
    if dtype == torch.float32:
        assert torch.equal(pieces, out), "a token's result does not depend on its neighbours"
    else:
        close(pieces[sure], want[sure], dtype, "pieces", loose=2.0)
    if case["groups"] and case["groups"][1] < case["groups"][0] and case["experts"] > case["groups"][0]:
        free = dict(c, router=dict(c["router"], groups=None))
        assert (N.moe(x.double(), W, "f.", free) - want).abs().max() > 0.05 * want.abs().max(), "the groups decide"
    _, wt, _ = N.route(x.double(), W, "f.", c)
    assert float(wt.sum(-1).min()) < float(wt.sum(-1).max()) - 1e-3, "the weights are the scores themselves, not renormalised"


# --------------------------------------------------------------- whole models
def att(heads, kv, dim, vdim, window, rot, base=10000.0, scaling=None, diff=0.4, scale=None):
    c = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale or 1.5 / math.sqrt(dim)}
    if window:
        c["mask"] = {"size": window}
    if rot:
        c["rot"] = {"base": base, "dims": rot}
        if scaling:
            c["rot"]["scaling"] = scaling
    return c


def lig(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def moe_cfg(experts, top, ff, shared, scale=1.0, groups=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r, "shared": {"ff": shared} if shared else None}


# M1: layers 0-1 run twice before a third; three taps; windows of 24 (one and a half pages) and 7; grouped experts with a
# shared one.  M2: no convolution, no repeated run, neither embedding nor logit scale; an attention layer without window
# and rotation, a key head per head; experts one a token without groups; groups of one expert; a width that is no power
# of two; pages of 4.  M3: one tap; the middle layer runs three times between the others; a layer without feed-forward.
# M4: sizes that are multiples of nothing (a width of 70, maps of 10, values of 22, keys of 9, inner sizes 50, 12 and 10, three
# experts): the kernels' forms for single values, the plain products, experts whose gate and up rows are not interleaved.
MODELS = {
    "M1": ({"architecture": "Nizorax", "vocab": 97, "width": 64, "norm": {"eps": 3e-5}, "embedding": {"scale": 4.0}, "logit_scale": 0.5,
            "canon": {"taps": 3}, "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [{"type": "attention", "mixer": att(4, 2, 16, 24, 24, 8, base=100.0, scaling=SCALING), "mlp": moe_cfg(8, 2, 24, 40, 2.0, (4, 2))},
                       {"type": "lightning", "mixer": lig(3, 8, 24, [0.5, 0.9, 0.99]), "mlp": {"kind": "dense", "ff": 100}},
                       {"type": "attention", "mixer": att(2, 1, 32, 16, 7, 32, diff=0.7), "mlp": None}]}, 16),
    "M2": ({"architecture": "Nizorax", "vocab": 211, "width": 112, "norm": {"eps": 1e-6},
            "layers": [{"type": "lightning", "mixer": lig(1, 40, 56, [0.97]), "mlp": None},
                       {"type": "attention", "mixer": att(3, 3, 64, 64, 0, 0, diff=0.2), "mlp": moe_cfg(6, 1, 32, 0)},
                       {"type": "lightning", "mixer": lig(4, 16, 16, [0.6, 0.8, 0.95, 0.995]), "mlp": moe_cfg(16, 3, 24, 24, 0.7, (16, 5))},
                       {"type": "attention", "mixer": att(6, 1, 12, 40, 100, 12, base=50.0, scaling={"factor": 2.0, "low": 1.0, "high": 2.0, "original": 32}),
                        "mlp": {"kind": "dense", "ff": 130}}]}, 4),
    "M3": ({"architecture": "Nizorax", "vocab": 130, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5}, "logit_scale": 3.0,
            "canon": {"taps": 1}, "loop": {"start": 1, "stop": 2, "times": 3},
            "layers": [{"type": "attention", "mixer": att(2, 2, 48, 32, 40, 16), "mlp": {"kind": "dense", "ff": 64}},
                       {"type": "lightning", "mixer": lig(2, 32, 48, [0.9, 0.999]), "mlp": moe_cfg(4, 2, 32, 0, 1.5, (2, 1))},
                       {"type": "attention", "mixer": att(4, 2, 32, 32, 64, 32, base=1000.0), "mlp": None}]}, 16),
    "M4": ({"architecture": "Nizorax", "vocab": 83, "width": 70, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "canon": {"taps": 2},
            "layers": [{"type": "attention", "mixer": att(2, 1, 10, 22, 9, 4, base=30.0), "mlp": moe_cfg(3, 2, 12, 10, 1.2)},
                       {"type": "lightning", "mixer": lig(2, 9, 11, [0.8, 0.97]), "mlp": {"kind": "dense", "ff": 50}}]}, 8),
}
LENGTHS = {"M1": (1, 23, 75, 40, 130, 64), "M2": (150, 2, 33, 201, 64, 97), "M3": (70, 5, 140, 31, 64, 2), "M4": (45, 3, 70, 20, 64, 9)}


def make_weights(cfg, seed):
    d = cfg["width"]
    W = {"embed": rnd(cfg["vocab"], d, seed=seed), "final.norm": 1 + 0.2 * rnd(d, seed=seed + 1), "final.norm.b": 0.3 * rnd(d, seed=seed + 2),
         "head": rnd(cfg["vocab"], d, seed=seed + 3, scale=1.0 / math.sqrt(d))}
    taps = (cfg.get("canon") or {}).get("taps", 0)
    for i, lay in enumerate(cfg["layers"]):
        p, s = f"l{i}.", seed + 1000 * (i + 1)
        for j, n in enumerate(("norm1", "norm1b") + (("norm2", "norm2b") if lay["mlp"] else ())):
            W[p + n] = (1 + 0.2 * rnd(d, seed=s + 2 * j)) * (0.7 if n.endswith("b") else 1.0)
            W[p + n + ".b"] = 0.3 * rnd(d, seed=s + 2 * j + 1)
        if taps:
            W[p + "canon1"] = rnd(d, taps, seed=s + 20, scale=0.5)
            if lay["mlp"]:
                W[p + "canon2"] = rnd(d, taps, seed=s + 21, scale=0.5)
        m = lay["mixer"]
        mix = attention_weights(d, m, s + 30) if lay["type"] == "attention" else lightning_weights(d, m, s + 30)
        for k, v in mix.items():
            W[p + "mix." + k] = v
        if lay["mlp"]:
            f = dense_weights(d, lay["mlp"]["ff"], s + 80) if lay["mlp"]["kind"] == "dense" else moe_weights(d, lay["mlp"], s + 80)
            for k, v in f.items():
                W[p + "mlp." + k] = v
    return {k: v.to(torch.bfloat16) for k, v in W.items()}


@pytest.fixture(scope="module")
def nizorax_folders(tmp_path_factory):
    out = {}
    for n, (name, (cfg, page)) in enumerate(MODELS.items()):
        folder = str(tmp_path_factory.mktemp(f"nizorax_{name}"))
        W = make_weights(cfg, seed=70 + n)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_safetensors(os.path.join(folder, "model.safetensors"), W)
        g = torch.Generator().manual_seed(n)
        reqs = {f"r{i}": torch.randint(0, cfg["vocab"], (m,), generator=g).tolist() for i, m in enumerate(LENGTHS[name])}
        Wd = {k: v.double() for k, v in W.items()}
        ref, unsure = {}, set()
        for rid, ids in reqs.items():
            margins = []
            ref[rid] = N.forward(ids, Wd, cfg, margins=margins).float().numpy()
            if margins:
                # tokens whose choice of experts hangs on less than 16-bit rounding moves a router's score
                close_call = torch.stack(margins).min(dim=0).values < 0.008
                unsure.update((rid, int(p)) for p in torch.nonzero(close_call)[:, 0])
        out[name] = (folder, cfg, page, Wd, reqs, ref, unsure)
    return out


def check_rows(rows, reqs, ref, dtype, label="", unsure=()):
    """float32: every logit to 1e-4 of the largest.  bfloat16: a row's root-mean-square error against the root mean square
    of all logits is at most 5 % for 95 of 100 rows and 30 % for every row; rows in `unsure` (a router's choice for that
    token hangs on less than the rounding of its 16-bit input moves a score) are not judged."""
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
            elif (rid, p) not in unsure:
                rel.append(float(np.sqrt(np.mean(err ** 2))) / rms_all)
                assert rel[-1] <= 0.30, f"{label}: request {rid} position {p}: rms error {rel[-1]:.3g} of the logits' rms in {dtype}"
            n += 1
    assert n == sum(len(v) for v in reqs.values())
    if rel:
        assert float(np.quantile(rel, 0.95)) <= 0.05, f"{label}: 95th percentile of the rows' rms error {np.quantile(rel, 0.95):.3g} in {dtype}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M1", "M2", "M3", "M4"])
def test_replay_all_ways_of_cutting(name, dtype, nizorax_folders, tmp_path):
    folder, cfg, page, W, reqs, ref, unsure = nizorax_folders[name]
    assert len(unsure) < sum(len(v) for v in reqs.values()) // 3
    V = cfg["vocab"]
    longest = round64(max(len(v) for v in reqs.values()))
    results = {}
    cuts = [("whole", whole(reqs), longest), ("tail", tail_decode(reqs), longest), ("portions", portions(reqs), longest),
            ("wide_portions", portions(reqs, sizes=(70, 2, 33, 64, 1, 100)), longest)]
    for label, steps, pool in cuts:
        out = run_trace(folder, dtype, steps, pool, str(tmp_path / label), V, page_size=page)
        rows = collect(steps, out)
        check_rows(rows, reqs, ref, dtype, label, unsure)
        results[label] = rows
    steps, peak = mixed(reqs)
    assert max(len(s["entries"]) for s in steps) == 4
    assert peak < sum(round64(len(v)) for v in reqs.values()), "the pool must be too small to avoid reuse"
    out = run_trace(folder, dtype, steps, peak, str(tmp_path / "mixed"), V, page_size=page)
    rows = collect(steps, out)
    check_rows(rows, reqs, ref, dtype, "mixed", unsure)
    results["mixed"] = rows
    if dtype == "float32":
        # every reduction of the float32 path has an order that depends on the row alone
        for label in [c[0] for c in cuts[1:]] + ["mixed"]:
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[label][key]), f"{label}: {key} differs from the whole run"


@pytest.mark.parametrize("name", ["M1", "M2", "M3", "M4"])
def test_the_stream_after_every_layer(name, nizorax_folders, tmp_path, monkeypatch):
    """The first layer run that differs names the mechanism: the stream after every layer run of one prompt, in float32."""
    folder, cfg, page, W, reqs, ref, unsure = nizorax_folders[name]
    ids = reqs["r2"]
    streams = []
    N.forward(ids, W, cfg, streams=streams)
    order = N.run_order(cfg)
    assert len(streams) == len(order)
    dump = tmp_path / "streams"
    dump.mkdir()
    monkeypatch.setenv("IMP_B200_DUMP_STREAM", str(dump))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids, "want": [len(ids) - 1]}], "end": ["a"]}]
    run_trace(folder, "float32", steps, round64(len(ids)), str(tmp_path / "out"), cfg["vocab"], page_size=page)
    for j, want in enumerate(streams):
        got = torch.from_numpy(np.fromfile(dump / f"step0_run{j}.f32", dtype="<f4").reshape(len(ids), cfg["width"]).copy())
        close(got, want, torch.float32, f"{name}: stream after layer run {j} (layer {order[j]}, {cfg['layers'][order[j]]['type']})")


def test_greedy_generation_through_the_engine(nizorax_folders):
    """Prompts of unequal length through submit / schedule / step / sample with short prefill portions; the tokens are
    those of the plain model's argmax, and pages and slots all come back."""
    from imp_b200 import Engine, EngineConfig, GenerateParams
    folder, cfg, page, W, reqs, ref, unsure = nizorax_folders["M1"]
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 7, 30, 12, 3)]

    def plain_generate(ids, n):
        ids, out = list(ids), []
        for _ in range(n):
            tok = int(torch.argmax(N.forward(ids, W, cfg)[-1]))
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
        lg = N.forward(p, W, cfg)[-1]
        top2 = torch.topk(lg, 2).values
        if float(top2[0] - top2[1]) > 0.1 * float(lg.abs().max()):
            assert g16[0] == w[0]


def test_command_line_with_a_checkpoint_and_with_random_weights(nizorax_folders, tmp_path):
    import subprocess
    import sys
    cli = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "imp-cli")
    folder, cfg, page, W, reqs, ref, unsure = nizorax_folders["M3"]
    ids, want = [5, 17, 3], []
    for _ in range(6):
        want.append(int(torch.argmax(N.forward(ids + want, W, cfg)[-1])))
    p = subprocess.run([sys.executable, cli, "--model", folder, "--prompt", "5,17,3", "--max-tokens", "6", "--temperature", "0",
                        "--dtype", "fp32", "--page-size", str(page), "--kv-pages", "64", "--max-seq-len", "128"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()] == want
    only_config = tmp_path / "cfg"
    only_config.mkdir()
    (only_config / "config.json").write_text(json.dumps(MODELS["M1"][0]))
    b = subprocess.run([sys.executable, cli, "--model", str(only_config), "--random-weights", "--weights-seed", "3", "--kv-pages", "64",
                        "--max-seq-len", "256", "--bench", "--bench-pp", "48", "--max-tokens", "8", "--bench-reps", "2", "--bench-batch", "2"],
                       capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-2000:]
    assert "pp    96 tokens" in b.stderr and "tg    16 tokens" in b.stderr
