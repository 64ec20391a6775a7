"""Nevodra restated from its equations in plain tensor code: whole sequences, dense masks, one function per
mechanism, float64 on the CPU unless told otherwise.  Shares nothing with the package: it is what the package's
kernels are held to.

Weights are a dict name -> tensor with the checkpoint's names ('embed', 'loop.step', 'l<i>.norm1' / '.norm2',
'l<i>.canon1' / '.canon2', 'l<i>.mix.*', 'l<i>.mlp.*', 'final.norm', 'head'); the configuration is config.json's
dict.
"""
from __future__ import annotations

import torch


# ------------------------------------------------------------------------------------------------ small pieces

def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def input_conv(h, w):
    """h + causal convolution of h over time on each channel: h [T, C], w [C, taps], the last tap meets the current
    token, zeros before the sequence's start."""
    T, C = h.shape
    taps = w.shape[1]
    full = torch.cat([h.new_zeros(taps - 1, C), h], 0)
    y = h.clone()
    for j in range(taps):
        y = y + full[j:j + T] * w[:, j]
    return y


def rotate_interleaved(x, pos, base, dims):
    """Pairs (2i, 2i + 1) of the first `dims` entries of the last axis of x [T, ..., D] turned by pos[t] * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / dims)
    ang = pos.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def window_mask(T, size, keep_first):
    """[T, T] bool: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------------ mixers

def window_attention(h, W, p, m, eps):
    """Grouped-query softmax attention without rotation: q and k RMS-normed over their whole projection, scores
    soft-capped, a logarithmic distance penalty per head, a sliding window that also keeps the first tokens."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ W[p + "q"].T, W[p + "q.norm"], eps).view(T, H, D)
    k = rms_norm(h @ W[p + "k"].T, W[p + "k.norm"], eps).view(T, G, D)
    v = (h @ W[p + "v"].T).view(T, G, V)
    mask = m.get("mask")                      # no mask in the configuration: every earlier key
    ok = window_mask(T, mask["size"], mask.get("keep_first", 0)) if mask else window_mask(T, T, 0)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).to(h.dtype)
    cap = float(m.get("softcap") or 0.0)      # no cap when the configuration gives none
    out = h.new_zeros(T, H, V)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s - W[p + "r1"][hh] * torch.log(1 + W[p + "r2"][hh] * dist)
        s = s.masked_fill(~ok, float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * V) @ W[p + "o"].T


def latent_attention(h, W, p, m, eps):
    """Causal softmax attention through one latent per position: per-head keys [W_uk c | rotated shared part], values
    W_uv c, queries [unrotated | rotated] straight from W_q, and a per-head sink logit in the softmax denominator."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].T).view(T, H, D + R)
    dkv = h @ W[p + "dkv"].T
    c = rms_norm(dkv[:, :C], W[p + "dkv.norm"], eps)
    kr = rotate_interleaved(dkv[:, C:], pos, rot["base"], rot["dims"])                     # [T, R], shared by the heads
    qr = rotate_interleaved(q[..., D:], pos, rot["base"], rot["dims"])                     # [T, H, R]
    ku = (c @ W[p + "uk"].T).view(T, H, D)
    vv = (c @ W[p + "uv"].T).view(T, H, V)
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = h.new_zeros(T, H, V)
    for hh in range(H):
        s = (q[:, hh, :D] @ ku[:, hh].T + qr[:, hh] @ kr.T) * float(m["scale"])
        s = s.masked_fill(~causal, float("-inf"))
        sink = W[p + "sink"][hh]
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        out[:, hh] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))) @ vv[:, hh]
    return out.reshape(T, H * V) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forwards

def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N = division by the root mean square over the row."""
    a, b, c, e = coef
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, W, p, eps):
    return poly_norm(h @ W[p + "up"].T, W[p + "act"], eps) @ W[p + "down"].T


def gated_expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(z, correction, r):
    """Router of one token: z [n] logits -> (chosen ids, weights).  Scores sigmoid(z); the choice adds the correction;
    a group's score is the sum of its two largest choices; only the best `keep` groups can be chosen (the others count
    as minus infinity); the `top` largest choices win and are weighted by their scores times the router's scale."""
    n, top = z.shape[0], int(r["top"])
    groups = r.get("groups") or {}
    count = int(groups.get("count", 1))
    keep = int(groups.get("keep", count))
    s = torch.sigmoid(z)
    choice = s + correction
    if keep < count:
        per = choice.view(count, n // count)
        gs = per.topk(min(2, n // count), -1).values.sum(-1)
        best = gs.topk(keep).indices
        allowed = torch.zeros(count, dtype=torch.bool)
        allowed[best] = True
        choice = torch.where(allowed[:, None].expand(count, n // count).reshape(n), choice,
                             torch.full_like(choice, float("-inf")))
    ids = choice.topk(top).indices
    return ids, s[ids] * float(r["scale"])


def moe_ff(h, W, p, mlp):
    r = mlp["router"]
    z = h @ W[p + "router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        ids, wts = route(z[t], W[p + "correction"], r)
        for e, w in zip(ids.tolist(), wts):
            out[t] = out[t] + w * gated_expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W, p + "shared.")
    return out


# ------------------------------------------------------------------------------------------------ the model

def layer_runs(cfg):
    """[(layer index, pass number or None)] in the order the layers run: layers start .. stop-1 `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {}
    start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
    if stop <= start:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def layer(x, W, cfg, i):
    L = cfg["layers"][i]
    eps, p = float(cfg["norm"]["eps"]), f"l{i}."
    h1 = input_conv(rms_norm(x, W[p + "norm1"], eps), W[p + "canon1"])
    mix = (window_attention if L["type"] == "attention" else latent_attention)(h1, W, p + "mix.", L["mixer"], eps)
    mlp = L.get("mlp")
    if not mlp:
        return x + mix
    h2 = input_conv(rms_norm(x, W[p + "norm2"], eps), W[p + "canon2"])
    ff = dense_ff(h2, W, p + "mlp.", eps) if mlp["kind"] == "dense" else moe_ff(h2, W, p + "mlp.", mlp)
    return x + (mix + ff)


def forward(tokens, W, cfg, dtype=torch.float64, collect=None):
    """tokens [T] -> logits [T, vocab]; `collect`, if a list, receives the stream after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    x = W["embed"][tokens.long()] * float(cfg["embedding"]["scale"])
    loop = cfg.get("loop") or {}
    first = int(loop.get("start", 0))
    for i, t in layer_runs(cfg):
        if t is not None and i == first:
            x = x + W["loop.step"][t]
        x = layer(x, W, cfg, i)
        if collect is not None:
            collect.append(x.clone())
    return rms_norm(x, W["final.norm"], float(cfg["norm"]["eps"])) @ W["head"].T
