"""A plain, slow implementation of the Nizorax decoder: whole sequences, no cache, one function per mechanism.

Nizorax wraps every sublayer in two layer norms (weight and bias) and adds a short causal convolution to what the
sublayer reads:

  u = ln1(x);  u = u + conv1(u);  x = x + ln1b(mixer(u))
  u = ln2(x);  u = u + conv2(u);  x = x + ln2b(ffn(u))          (the second line only where the layer has a feed-forward)

The mixers:

  lightning   linear attention: a matrix state per head that fades by a fixed factor per head and collects k v^T, read
              by q, with silu on q, k and v; the heads together are RMS-normalised with a weight and gated by a sigmoid
  attention   differential softmax attention: every head holds two score maps over the same values (grouped key/value
              heads, a sliding window, a rotation of neighbouring pairs in the front of each map with scaled
              frequencies); the second map's result is subtracted lambda times, the difference is RMS-normalised

The feed-forward is dense with a normalised polynomial as activation, or a mixture of gated experts whose router
scores are sigmoids, restricted to the best groups of experts, plus a shared expert.  A run of layers may be repeated
with the same weights.  Nothing here is shared with the engine; everything runs on the CPU in the dtype of the
caller's tensors (float64 in the tests).  Weights are a dictionary by checkpoint tensor name; sizes and constants come
from the configuration dictionary (the keys of config.json).
"""
from __future__ import annotations

import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b with the population variance."""
    mu = x.mean(dim=-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w + b


def add_causal_conv(u, w):
    """u [T, d] plus its causal convolution per channel: w [d, taps], the last tap on the token itself, zeros before
    the sequence's start."""
    T, taps = u.shape[0], w.shape[1]
    out = u.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def scaled_frequencies(base, dims, scaling):
    """base^(-2i/dims) for i < dims/2, long wavelengths slowed down: kept where the wavelength is below original/high,
    divided by `factor` above original/low, blended linearly in between."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wave = 2.0 * math.pi / f
            if wave < orig / hi:
                pass
            elif wave > orig / lo:
                f = f / fac
            else:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate_neighbours(x, positions, freqs):
    """Rotate the first 2 * len(freqs) entries of the last axis of x [T, heads, size]: entry 2i pairs with 2i + 1 and
    turns by positions * freqs[i]; the rest stays."""
    n = freqs.shape[0]
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = a * cos - b * sin
    out[..., 1:2 * n:2] = b * cos + a * sin
    return out


def windowed_softmax_attention(q, k, v, scale, window):
    """q, k [T, D], v [T, Dv] of one map of one head: position i sees j with 0 <= i - j < window (window 0: all earlier)."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if not window else ((j <= i) & (i - j < window))
    s = s.masked_fill(~seen, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def differential_attention(u, W, p, c, eps, positions=None):
    """u [T, d] -> [T, d]; W the weights, p the tensors' prefix ('l3.mix.'), c the mixer's configuration."""
    T = u.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    if positions is None:
        positions = torch.arange(T)
    q = (u @ W[p + "q"].T).view(T, H, 2, D)
    k = (u @ W[p + "k"].T).view(T, G, 2, D)
    v = (u @ W[p + "v"].T).view(T, G, Dv)
    rot = c.get("rot")
    if rot:
        f = scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q = rotate_neighbours(q.reshape(T, 2 * H, D), positions, f).view(T, H, 2, D)
        k = rotate_neighbours(k.reshape(T, 2 * G, D), positions, f).view(T, G, 2, D)
    window = (c.get("mask") or {}).get("size", 0)
    diff = c["diff"]
    lam = torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum()) + diff
    heads = []
    for h in range(H):
        g = h // (H // G)
        a1 = windowed_softmax_attention(q[:, h, 0], k[:, g, 0], v[:, g], c["scale"], window)
        a2 = windowed_softmax_attention(q[:, h, 1], k[:, g, 1], v[:, g], c["scale"], window)
        heads.append(unit_rms(a1 - lam * a2, eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1) @ W[p + "o"].T


def scan_fixed_decay(q, k, v, decay):
    """One head: S <- decay S + k v^T, o = S^T q, token by token from a zero state."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def lightning(u, W, p, c, eps):
    T = u.shape[0]
    H, D, Dv = c["heads"], c["dim"], c["vdim"]
    q = silu(u @ W[p + "q"].T).view(T, H, D)
    k = silu(u @ W[p + "k"].T).view(T, H, D)
    v = silu(u @ W[p + "v"].T).view(T, H, Dv)
    o = torch.cat([scan_fixed_decay(q[:, h], k[:, h], v[:, h], c["decay"][h]) for h in range(H)], dim=-1)
    y = unit_rms(o, eps) * W[p + "norm"] * torch.sigmoid(u @ W[p + "g"].T)
    return y @ W[p + "o"].T


def polynorm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, powers taken element by element, N dividing a row by its root mean square."""
    a, b, c3, e = [coef[i] for i in range(4)]
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c3 * unit_rms(z * z * z, eps) + e


def dense_ff(u, W, p, eps):
    return polynorm(u @ W[p + "up"].T, W[p + "act"], eps) @ W[p + "down"].T


def gated_expert(u, W, p):
    return (silu(u @ W[p + "gate"].T) * (u @ W[p + "up"].T)) @ W[p + "down"].T


def route(u, W, p, c):
    """Chosen experts and their weights for every row of u: sigmoid scores; experts in `count` equal groups of
    neighbours, a group scored by the sum of its two largest scores, the best `keep` groups stay; the `top` largest
    scores among those; weight = score * scale, not renormalised.  Returns (indices [T, top], weights [T, top], scores)."""
    r = c["router"]
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(u @ W[p + "router"].T)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        gs = s.view(-1, n, per)
        gscore = gs.topk(min(2, per), dim=-1).values.sum(dim=-1)
        best = gscore.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, best, True)
        allowed = gmask[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = s.masked_fill(~allowed, float("-inf"))
    idx = masked.topk(top, dim=-1).indices
    w = s.gather(1, idx) * r.get("scale", 1.0)
    return idx, w, s


def route_margin(u, W, p, c):
    """Per token, the smallest gap a choice hangs on: between the last kept and the first dropped group, and between the
    last chosen and the first refused score among the kept groups (infinite where nothing is refused)."""
    r = c["router"]
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(u @ W[p + "router"].T)
    inf = torch.full((u.shape[0],), float("inf"), dtype=u.dtype)
    margin = inf.clone()
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        gscore = s.view(-1, n, per).topk(min(2, per), dim=-1).values.sum(dim=-1)
        if keep < n:
            val = gscore.topk(keep + 1, dim=-1).values
            margin = torch.minimum(margin, val[:, keep - 1] - val[:, keep])
        best = gscore.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, best, True)
        allowed = gmask[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = s.masked_fill(~allowed, float("-inf"))
    if top < int(allowed[0].sum()):
        val = masked.topk(top + 1, dim=-1).values
        margin = torch.minimum(margin, val[:, top - 1] - val[:, top])
    return margin


def moe(u, W, p, c, margins=None):
    idx, w, _ = route(u, W, p, c)
    if margins is not None:
        margins.append(route_margin(u, W, p, c))
    out = torch.zeros(u.shape[0], W[p + "e0.down"].shape[0], dtype=u.dtype)
    for t in range(u.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += w[t, j] * gated_expert(u[t:t + 1], W, p + "e%d." % e)[0]
    if c.get("shared"):
        out = out + gated_expert(u, W, p + "shared.")
    return out


def run_order(cfg):
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(L))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], L))


def forward(ids, W, cfg, streams=None, margins=None):
    """ids: token ids of one sequence -> logits [T, vocab].  With `streams` (a list), the stream after every layer run; with
    `margins` (a list), every routed layer run's margins per token."""
    eps = cfg["norm"]["eps"]
    dtype = W["embed"].dtype
    x = W["embed"][torch.as_tensor(ids, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    has_conv = bool(cfg.get("canon"))
    for i in run_order(cfg):
        layer = cfg["layers"][i]
        p = "l%d." % i
        u = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if has_conv:
            u = add_causal_conv(u, W[p + "canon1"])
        if layer["type"] == "attention":
            m = differential_attention(u, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "lightning":
            m = lightning(u, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(m, W[p + "norm1b"], W[p + "norm1b.b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            u = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            if has_conv:
                u = add_causal_conv(u, W[p + "canon2"])
            f = dense_ff(u, W, p + "mlp.", eps) if mlp["kind"] == "dense" else moe(u, W, p + "mlp.", mlp, margins)
            x = x + layer_norm(f, W[p + "norm2b"], W[p + "norm2b.b"], eps)
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return (x @ W["head"].T * cfg.get("logit_scale", 1.0)).to(dtype)
