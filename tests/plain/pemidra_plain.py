"""A plain, slow implementation of the Pemidra decoder: whole sequences, no cache, one function per mechanism.

Pemidra is a post-norm decoder: the normalised sum is the stream, and both sublayers read the stream itself,

  x = ln1(m * x + s1 * mixer(x));  x = ln2(m * x + s2 * ffn(x))     (the second line only where the layer has a feed-forward)

with a layer norm that has a weight and a bias, learned factors per channel s1, s2 and one constant m.  The mixers:

  retention       a matrix state per head that fades by a fixed factor per head and collects k v^T; no softmax
  general_delta   a matrix state per head with a decay per key channel made from the input, from which a part along
                  the unit key is removed (at a rate per channel) before k v^T is added
  parallel        two mixers side by side, their outputs each RMS-normalised over the width and averaged:
                  softmax attention (heads normalised, rotated in part, scaled per head, masked by chunks, with a
                  sink in the denominator, gated per head) and a delta rule with short convolutions in front, a
                  decay per head and key channel and a step size beta

The feed-forward is gated with the tanh form of gelu.  Nothing here is shared with the engine; everything runs on
the CPU in the dtype of the caller's tensors (float64 in the tests).  Weights are a dictionary by checkpoint
tensor name; sizes and constants come from the configuration dictionary (the keys of config.json).
"""
from __future__ import annotations

import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z * z * z)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def unit_length(x, eps):
    """x / sqrt(sum(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b with the population variance."""
    mu = x.mean(dim=-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w + b


def rotate_front(x, positions, base, dims):
    """Rotate the first `dims` entries of the last axis of x [T, heads, size]: entry i pairs with i + dims/2 and turns
    by positions * base^(-2i/dims); the entries from `dims` on stay."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------ recurrences, one token at a time
def scan_fixed_decay(q, k, v, decay):
    """S <- decay S + k v^T;  o = S^T q.   q, k [T, D], v [T, Dv], decay a number."""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=v.dtype)
    out = []
    for t in range(k.shape[0]):
        S = decay * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out)


def scan_remove_along_key(r, k, v, w, a, unit_eps):
    """S <- diag(w) S - (a * u)(u^T S) + k v^T with u the unit key, both first terms over the old S;  o = S^T r."""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=v.dtype)
    out = []
    for t in range(k.shape[0]):
        u = unit_length(k[t], unit_eps)
        seen = u @ S                                   # what the old state returns for the unit key
        S = w[t][:, None] * S - (a[t] * u)[:, None] * seen[None, :] + k[t][:, None] * v[t][None, :]
        out.append(S.T @ r[t])
    return torch.stack(out)


def scan_delta(q, k, v, g, beta):
    """S <- diag(g) S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q (after the write)."""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=v.dtype)
    out = []
    for t in range(k.shape[0]):
        S = g[t][:, None] * S
        e = beta[t] * (v[t] - S.T @ k[t])
        S = S + k[t][:, None] * e[None, :]
        out.append(S.T @ q[t])
    return torch.stack(out)


# ------------------------------------------------------------------ mixers
def retention(x, W, p, c, eps):
    T = x.shape[0]
    H, D = c["heads"], c["dim"]
    Dv = c.get("vdim", D)
    q = (x @ W[p + "q"].T).view(T, H, D)
    k = (x @ W[p + "k"].T).view(T, H, D) / math.sqrt(D)
    v = (x @ W[p + "v"].T).view(T, H, Dv)
    o = torch.stack([scan_fixed_decay(q[:, h], k[:, h], v[:, h], c["decay"][h]) for h in range(H)], dim=1)
    y = unit_rms(o, eps).reshape(T, H * Dv) * silu(x @ W[p + "g"].T)
    return y @ W[p + "o"].T


def general_delta(x, W, p, c, eps):
    T = x.shape[0]
    H, D = c["heads"], c["dim"]
    r = (x @ W[p + "r"].T).view(T, H, D)
    k = (x @ W[p + "k"].T).view(T, H, D)
    v = (x @ W[p + "v"].T).view(T, H, D)
    z = torch.tanh(x @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(z)).view(T, H, D)
    a = torch.sigmoid(x @ W[p + "a"].T + W[p + "a.b"]).view(T, H, D)
    o = torch.stack([scan_remove_along_key(r[:, h], k[:, h], v[:, h], w[:, h], a[:, h], 1e-6) for h in range(H)], dim=1)
    y = unit_rms(o, eps).reshape(T, H * D) * W[p + "norm"] * torch.sigmoid(x @ W[p + "g"].T)
    return y @ W[p + "o"].T


def gated_head_attention(x, W, p, c, eps, positions=None, sink=1.0):
    """`sink` is what joins the softmax denominator beside the keys (exp of the sink's score 0; the design fixes 1)."""
    T = x.shape[0]
    H, G, D = c["heads"], c.get("kv_heads", c["heads"]), c["dim"]
    Dv = c.get("vdim", D)
    pos = torch.arange(T) if positions is None else positions
    q = unit_rms((x @ W[p + "q"].T).view(T, H, D), eps) * W[p + "q.norm"]
    k = unit_rms((x @ W[p + "k"].T).view(T, G, D), eps) * W[p + "k.norm"]
    v = unit_rms((x @ W[p + "v"].T).view(T, G, Dv), eps)
    if c.get("rot"):
        q = rotate_front(q, pos, c["rot"]["base"], c["rot"]["dims"])
        k = rotate_front(k, pos, c["rot"]["base"], c["rot"]["dims"])
    seen = pos[None, :] <= pos[:, None]
    if c.get("mask"):
        size = c["mask"]["size"]
        seen = seen & (torch.div(pos, size, rounding_mode="floor")[None, :] == torch.div(pos, size, rounding_mode="floor")[:, None])
    gate = torch.sigmoid(x @ W[p + "g"].T)                       # [T, H]
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * c["scale"] * W[p + "temp"][h]
        e = torch.where(seen, torch.exp(s), torch.zeros_like(s))
        prob = e / (sink + e.sum(dim=-1, keepdim=True))          # the sink has score 0 and no value
        heads.append((prob @ v[:, g]) * gate[:, h:h + 1])
    return torch.cat(heads, dim=-1) @ W[p + "o"].T


def short_conv_silu(z, w):
    """y[t, c] = silu(sum_j w[c, j] z[t - (taps - 1) + j, c]) with zeros before the start."""
    T, C = z.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=z.dtype), z], dim=0)
    y = torch.zeros_like(z)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j][None, :]
    return silu(y)


def channel_delta_rule(x, W, p, c, eps):
    T = x.shape[0]
    H, G, D = c["heads"], c.get("kv_heads", c["heads"]), c["dim"]
    Dv = c.get("vdim", D)
    q = short_conv_silu(x @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, D)
    k = short_conv_silu(x @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, D)
    v = short_conv_silu(x @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, Dv)
    q = unit_length(q, 1e-6) / math.sqrt(D)
    k = unit_length(k, 1e-6)
    beta = torch.sigmoid(x @ W[p + "b"].T)                       # [T, H]
    step = torch.nn.functional.softplus((x @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).view(T, H, D)
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * step)
    o = torch.stack([scan_delta(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], g[:, h], beta[:, h]) for h in range(H)], dim=1)
    gate = torch.sigmoid((x @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, Dv)
    y = unit_rms(o, eps) * W[p + "norm"] * gate
    return y.reshape(T, H * Dv) @ W[p + "o"].T


def pair(x, W, p, c, eps, positions=None):
    left = gated_head_attention(x, W, p + "left.", c["left"], eps, positions)
    right = channel_delta_rule(x, W, p + "right.", c["right"], eps)
    return 0.5 * (unit_rms(left, eps) * W[p + "left.out"] + unit_rms(right, eps) * W[p + "right.out"])


def gated_mlp(x, W, p):
    return (gelu_tanh(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


MIXERS = {"retention": retention, "general_delta": general_delta, "parallel": pair}


# ------------------------------------------------------------------ the model
def forward(ids, W, cfg, streams=None):
    """Logits [T, vocab] of one sequence; `streams` collects the stream after every layer."""
    eps, m = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = W["embed"][torch.as_tensor(ids, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](x, W, p + "mix.", layer["mixer"], eps)
        x = layer_norm(m * x + W[p + "ls1"] * y, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer.get("mlp"):
            y = gated_mlp(x, W, p + "mlp.")
            x = layer_norm(m * x + W[p + "ls2"] * y, W[p + "norm2"], W[p + "norm2.b"], eps)
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["head"].T
