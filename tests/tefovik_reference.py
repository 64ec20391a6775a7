"""Tefovik restated from its equations in plain tensor code: whole sequences, dense masks, explicit token loops for
the recurrences, one function per mechanism, float64 on the CPU unless told otherwise.  Shares nothing with the
package: it is what the package's kernels are held to.

Weights are a dict name -> tensor with the checkpoint's names ('embed', 'embed.norm', 'l<i>.norm1', 'l<i>.ls1',
'l<i>.dwa', 'l<i>.mix.*', 'l<i>.mlp.up' / '.down', 'final.norm', 'head'); the configuration is config.json's dict.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ small pieces

def layer_norm(x, w, eps):
    """(x - mean) / sqrt(mean squared deviation + eps) * w over the last axis; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def short_conv(u, w, bias=None, before=None):
    """Causal per-channel convolution over time.  u [T, C], w [C, taps] whose last column meets the current token;
    `before` [taps - 1, C] = the inputs that came before u (zeros at a sequence's start).  Returns (y, last inputs)."""
    T, C = u.shape
    taps = w.shape[1]
    if before is None:
        before = u.new_zeros(taps - 1, C)
    full = torch.cat([before, u], 0)
    y = u.new_zeros(T, C)
    for j in range(taps):
        y = y + full[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return y, full[full.shape[0] - (taps - 1):]


def rotate_pairs(x, pos, base, dims, interleaved=True, sign=1.0):
    """Rotary turn of the first `dims` entries of the last axis of x [T, ..., D] by sign * pos[t] * base^(-2i/dims);
    pair i = (2i, 2i + 1) when interleaved, (i, i + dims/2) otherwise.  The rest passes unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / dims)
    ang = sign * pos.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def chunk_mask(pos_q, pos_k, size):
    """[Tq, Tk] bool: key j visible to query i iff j <= i and both lie in the same block of `size` positions."""
    i, j = pos_q[:, None], pos_k[None, :]
    ok = j <= i
    if size:
        ok = ok & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return ok


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def block_attention(q, k, v, pos_q, pos_k, scale, size):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, V]: softmax attention of every query over the keys chunk_mask lets it see."""
    rep = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~chunk_mask(pos_q, pos_k, size)[None], -math.inf)
    return torch.einsum("hij,jhv->ihv", torch.softmax(s, -1), v)


def state_space_scan(x, B, C, dt, a, D, S=None):
    """x [T, H, V], B / C [T, G, N], dt / a [T, H] (step size and decay), D [H]:  S <- a S + dt B x^T;  y = S^T C + D x.
    Returns (y, final states [H, N, V])."""
    T, H, V = x.shape
    N, rep = B.shape[-1], H // B.shape[1]
    S = x.new_zeros(H, N, V) if S is None else S.clone()
    y = x.new_zeros(T, H, V)
    for t in range(T):
        for h in range(H):
            g = h // rep
            S[h] = a[t, h] * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y, S


def delta_rule_scan(q, k, v, beta, decay, S=None):
    """q / k [T, G, D] (already normalised), v [T, H, V], beta [T, H], decay [T, H, D]:
    S <- diag(decay) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Returns (o, final states [H, D, V])."""
    T, H, V = v.shape
    D, rep = q.shape[-1], H // q.shape[1]
    S = v.new_zeros(H, D, V) if S is None else S.clone()
    o = v.new_zeros(T, H, V)
    for t in range(T):
        for h in range(H):
            g = h // rep
            S[h] = decay[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, g])
            S[h] = S[h] + torch.outer(k[t, g], u)
            o[t, h] = S[h].T @ q[t, g]
    return o, S


def unit_vectors(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def group_rms(y, parts, eps):
    T, W = y.shape
    y = y.view(T, parts, W // parts)
    return (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(T, W)


# ------------------------------------------------------------------------------------------------ mixers

def chunked_attention(h, W, p, m, eps, pos):
    """The left half of a parallel mixer.  h [T, E]; W/p: weights and the name prefix ('l3.mix.left.'); m: its sizes."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q, _ = short_conv(h @ W[p + "q"].T, W[p + "q.conv"])
    k, _ = short_conv(h @ W[p + "k"].T, W[p + "k.conv"])
    v, _ = short_conv(h @ W[p + "v"].T, W[p + "v.conv"])
    q = rms_norm(q.view(T, H, D), W[p + "q.norm"], eps)
    k = rms_norm(k.view(T, G, D), W[p + "k.norm"], eps)
    rot = m["rot"]
    q = rotate_pairs(q, pos, rot["base"], rot["dims"])
    k = rotate_pairs(k, pos, rot["base"], rot["dims"])
    v = rotate_pairs(v.view(T, G, V), pos, rot["base"], V)
    o = block_attention(q, k, v, pos, pos, m["scale"], (m.get("mask") or {}).get("size", 0))
    o = rotate_pairs(o, pos, rot["base"], V, sign=-1.0)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ W[p + "o"].T


def gated_delta_rule(h, W, p, m, eps):
    """The right half of a parallel mixer: a matrix state per head with a decay per key channel and a delta-rule
    write; the read-out sees the current token's write."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = F.silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])[0]).view(T, G, D)
    k = F.silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])[0]).view(T, G, D)
    v = F.silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])[0]).view(T, H, V)
    q, k = unit_vectors(q) * D ** -0.5, unit_vectors(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                            # [T, H]
    lam = torch.exp(W[p + "A_log"]).view(1, H, 1)
    decay = torch.exp(-lam * softplus((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).view(T, H, D))
    out = rms_norm(delta_rule_scan(q, k, v, beta, decay)[0], W[p + "norm"], eps)
    out = out * torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, V)
    return out.reshape(T, H * V) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps, pos):
    a = rms_norm(chunked_attention(h, W, p + "left.", m["left"], eps, pos), W[p + "left.out"], eps)
    b = rms_norm(gated_delta_rule(h, W, p + "right.", m["right"], eps), W[p + "right.out"], eps)
    return 0.5 * (a + b)


def mamba2_mixer(h, W, p, m, eps):
    """State-space mixer: input-dependent step size, one scalar decay per head, state [N, vdim] per head."""
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    T, inner = h.shape[0], m["heads"] * m["vdim"]
    zxbcdt = h @ W[p + "in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = F.silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"])[0])
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])                                              # [T, H]
    a = torch.exp(-torch.exp(W[p + "A_log"]) * dt)
    y = state_space_scan(x, B, C, dt, a, W[p + "D"])[0].reshape(T, inner) * F.silu(z)
    return group_rms(y, m.get("norm_groups", 1), eps) * W[p + "norm"] @ W[p + "o"].T


def squared_relu_mlp(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


# ------------------------------------------------------------------------------------------------ the model

def forward(cfg, W, tokens, dtype=torch.float64, collect=None):
    """Logits [T, vocab] of a whole sequence.  `collect`, if a list, receives the stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    pos = torch.arange(T)
    x = layer_norm(W["embed"][tokens], W["embed.norm"], eps)
    outs = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "mamba2":
            mixed = mamba2_mixer(x, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            mixed = parallel_mixer(x, W, p + "mix.", layer["mixer"], eps, pos)
        else:
            raise ValueError(layer["type"])
        x = layer_norm(alpha * x + W[p + "ls1"] * mixed, W[p + "norm1"], eps)
        if layer.get("mlp"):
            x = layer_norm(alpha * x + W[p + "ls2"] * squared_relu_mlp(x, W, p + "mlp."), W[p + "norm2"], eps)
        outs.append(x)
        x = sum(W[p + "dwa"][j] * outs[j] for j in range(i + 2))
        if collect is not None:
            collect.append(x.clone())
    x = layer_norm(x, W["final.norm"], eps)
    logits = x @ W["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
