"""PyTorch custom ops over the sequence-kernel C ABI (include/cc_b200_seq.h, libcc_b200_seq.so).

Registered in the same `torch.ops.cold_compress_b200` namespace as the compressed-KV ops (ops.py), with schemas that
declare the in-place writes.  CUDA tensors only: the CPU registrations raise.  Element types are taken from the
tensors: fp32 or bf16 for activations, tables and cache rows; the residual stream, q, sinks, biases, norm gains and
mixing coefficients are always fp32.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_library = torch.library.Library("cold_compress_b200", "FRAGMENT")

ATTN_CHUNK, ATTN_DECODE_APPEND, ATTN_APPEND_ONLY, ATTN_DECODE = 0, 1, 2, 3

_library.define("seq_embed(Tensor tokens, Tensor input_pos, Tensor(a!) prev_token, Tensor embed, Tensor? bigram, "
                "Tensor inv_freq, Tensor(b!) x, Tensor(c!)? x_act, float scale, int buckets, int mul_prev, int mul_cur) -> ()")
_library.define("seq_qkv_prepare(Tensor qkv, Tensor? bias, Tensor input_pos, Tensor? mix_lambda, Tensor? v_first, "
                "Tensor(a!) q, Tensor(b!) k, Tensor(c!) v, int H, int G, int Dk, int Dv, float eps, bool unit_norm, "
                "float gain_coef, int gain_every) -> ()")
_library.define("seq_attention(Tensor q, Tensor k_new, Tensor v_new, Tensor(a!) k_cache, Tensor(b!) v_cache, Tensor(c!) pos, "
                "Tensor(d!) mask, Tensor(e!) cache_cts, Tensor input_pos, Tensor(f!) y, Tensor? sink, int window, "
                "int sink_mode, float scale, int mode, Tensor(g!)? workspace, int block=0, int keep_first=0, "
                "float softcap=0.0, Tensor? dist_a=None, Tensor? dist_b=None) -> ()")
_library.define("seq_residual_norm(Tensor(a!) x, Tensor? y, Tensor w, float alpha, float eps, Tensor(b!)? x_act) -> ()")
_library.define("seq_clamped_glu(Tensor gu, Tensor(a!) out, float limit, float slope) -> ()")
_library.define("seq_gemv(Tensor x, Tensor? in_norm_w, Tensor w, Tensor? bias, Tensor? res, Tensor? res_norm_w, Tensor(a!) out, "
                "int mode, float alpha, float eps, float limit, float slope) -> ()")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.DT_F32
    if t.dtype == torch.bfloat16:
        return _lib.DT_BF16
    raise _lib.CcError(f"sequence kernels take fp32 or bf16 tensors, not {t.dtype}")


def _p(t):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(*pairs):
    for name, t, dtype in pairs:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.CcError("cold_compress_b200 sequence ops run on CUDA tensors only (no CPU fallback)")
        if not t.is_contiguous():
            raise _lib.CcError(f"{name}: expected a contiguous tensor")
        if dtype is not None and t.dtype != dtype:
            raise _lib.CcError(f"{name}: expected {dtype}, got {t.dtype}")


def _seq_embed(tokens, input_pos, prev_token, embed, bigram, inv_freq, x, x_act, scale, buckets, mul_prev, mul_cur):
    _need(("tokens", tokens, torch.int32), ("input_pos", input_pos, torch.int32), ("prev_token", prev_token, torch.int32),
          ("embed", embed, None), ("bigram", bigram, embed.dtype), ("inv_freq", inv_freq, torch.float32),
          ("x", x, torch.float32), ("x_act", x_act, None))
    T, E = tokens.numel(), embed.shape[1]
    assert x.shape[-1] == E and x.numel() == T * E and inv_freq.numel() >= (E + 1) // 2
    _lib.check_seq(_lib.load_seq().cc_seq_embed(
        _p(tokens), _p(input_pos), _p(prev_token), _p(embed), _p(bigram), _p(inv_freq), _p(x), _p(x_act), T, E,
        float(scale), int(buckets), int(mul_prev), int(mul_cur), _dt(embed), _dt(x_act) if x_act is not None else _lib.DT_F32,
        _stream()), "cc_seq_embed")


def _seq_qkv_prepare(qkv, bias, input_pos, mix_lambda, v_first, q, k, v, H, G, Dk, Dv, eps, unit_norm, gain_coef, gain_every):
    _need(("qkv", qkv, None), ("bias", bias, torch.float32), ("input_pos", input_pos, torch.int32),
          ("mix_lambda", mix_lambda, torch.float32), ("v_first", v_first, k.dtype), ("q", q, torch.float32), ("k", k, None),
          ("v", v, k.dtype))
    T = qkv.shape[0]
    assert qkv.shape[1] == (H + G) * Dk + G * Dv and q.numel() == T * H * Dk and k.numel() == T * G * Dk and v.numel() == T * G * Dv
    _lib.check_seq(_lib.load_seq().cc_seq_qkv_prepare(
        _p(qkv), _dt(qkv), _p(bias), _p(input_pos), _p(mix_lambda), _p(v_first), _p(q), _p(k), _p(v), _dt(k), T, H, G, Dk, Dv,
        float(eps), int(bool(unit_norm)), float(gain_coef), int(gain_every), _stream()), "cc_seq_qkv_prepare")


def _seq_attention(q, k_new, v_new, k_cache, v_cache, pos, mask, cache_cts, input_pos, y, sink, window, sink_mode, scale,
                   mode, workspace, block=0, keep_first=0, softcap=0.0, dist_a=None, dist_b=None):
    _need(("q", q, torch.float32), ("k_new", k_new, k_cache.dtype), ("v_new", v_new, k_cache.dtype), ("k_cache", k_cache, None),
          ("v_cache", v_cache, k_cache.dtype), ("pos", pos, torch.int32), ("mask", mask, torch.bool),
          ("cache_cts", cache_cts, torch.int32), ("input_pos", input_pos, torch.int32), ("y", y, None),
          ("sink", sink, torch.float32), ("workspace", workspace, None), ("dist_a", dist_a, torch.float32),
          ("dist_b", dist_b, torch.float32))
    a = _lib.CcSeqAttn()
    a.keep_first, a.softcap, a.dist_a, a.dist_b = int(keep_first), float(softcap), _p(dist_a), _p(dist_b)
    T, H, Dk = q.shape
    G, L = k_cache.shape[-3], k_cache.shape[-2]
    Dv = v_cache.shape[-1]
    assert k_cache.shape[-1] == Dk and k_new.shape == (T, G, Dk) and v_new.shape == (T, G, Dv) and y.shape == (T, H, Dv)
    assert pos.numel() == L and mask.numel() == G * L
    a.q, a.k_new, a.v_new, a.k_cache, a.v_cache = _p(q), _p(k_new), _p(v_new), _p(k_cache), _p(v_cache)
    a.pos, a.mask, a.cache_cts, a.input_pos, a.y, a.sink = _p(pos), _p(mask), _p(cache_cts), _p(input_pos), _p(y), _p(sink)
    a.T, a.H, a.G, a.Dk, a.Dv, a.L = T, H, G, Dk, Dv, L
    a.window, a.sink_mode, a.cache_dtype, a.y_dtype, a.scale = int(window), int(sink_mode), _dt(k_cache), _dt(y), float(scale)
    a.append = int(mode == ATTN_DECODE_APPEND)
    a.block = int(block)
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    lib = _lib.load_seq()
    if mode == ATTN_CHUNK:
        _lib.check_seq(lib.cc_seq_attention(C.byref(a), _stream()), "cc_seq_attention")
    elif mode in (ATTN_DECODE_APPEND, ATTN_DECODE):
        _lib.check_seq(lib.cc_seq_attention_decode(C.byref(a), _stream()), "cc_seq_attention_decode")
    elif mode == ATTN_APPEND_ONLY:
        _lib.check_seq(lib.cc_seq_cache_append(C.byref(a), _stream()), "cc_seq_cache_append")
    else:
        raise _lib.CcError(f"seq_attention: unknown mode {mode}")


def decode_workspace_bytes(H, G, Dv, L, window) -> int:
    return int(_lib.load_seq().cc_seq_decode_workspace(H, G, Dv, L, window))


def _seq_residual_norm(x, y, w, alpha, eps, x_act):
    _need(("x", x, torch.float32), ("y", y, None), ("w", w, torch.float32), ("x_act", x_act, None))
    E = x.shape[-1]
    T = x.numel() // E
    assert w.numel() == E and (y is None or y.numel() == x.numel()) and (x_act is None or x_act.numel() == x.numel())
    _lib.check_seq(_lib.load_seq().cc_seq_residual_norm(
        _p(x), _p(y), _dt(y) if y is not None else _lib.DT_F32, _p(w), float(alpha), float(eps), _p(x_act),
        _dt(x_act) if x_act is not None else _lib.DT_F32, T, E, _stream()), "cc_seq_residual_norm")


def _seq_clamped_glu(gu, out, limit, slope):
    _need(("gu", gu, None), ("out", out, None))
    F = out.shape[-1]
    T = out.numel() // F
    assert gu.numel() == 2 * T * F
    _lib.check_seq(_lib.load_seq().cc_seq_clamped_glu(_p(gu), _p(out), _dt(gu), _dt(out), float(limit), float(slope), T, F,
                                                      _stream()), "cc_seq_clamped_glu")


def _seq_gemv(x, in_norm_w, w, bias, res, res_norm_w, out, mode, alpha, eps, limit, slope):
    """One-token product with the post-sum norm folded into its prologue / epilogue (cc_seq_gemv)."""
    _need(("x", x, None), ("in_norm_w", in_norm_w, torch.float32), ("w", w, None), ("bias", bias, torch.float32),
          ("res", res, torch.float32), ("res_norm_w", res_norm_w, torch.float32), ("out", out, None))
    g = _lib.CcSeqGemv()
    rows, K = w.shape
    N = rows // 2 if mode == _lib.GEMV_GLU else rows
    assert x.numel() == K and out.numel() == N and (res is None or res.numel() == N) and (in_norm_w is None or in_norm_w.numel() == K)
    g.x, g.x_dtype, g.in_norm_w, g.W, g.w_dtype = _p(x), _dt(x), _p(in_norm_w), _p(w), _dt(w)
    g.bias, g.res, g.res_norm_w = _p(bias), _p(res), _p(res_norm_w)
    g.alpha, g.eps, g.limit, g.slope, g.mode = float(alpha), float(eps), float(limit), float(slope), int(mode)
    g.out, g.out_dtype, g.N, g.K = _p(out), _dt(out), N, K
    _lib.check_seq(_lib.load_seq().cc_seq_gemv(C.byref(g), _stream()), "cc_seq_gemv")


def _no_cpu(*_a, **_k):
    raise _lib.CcError("cold_compress_b200 sequence ops have no CPU implementation (sm_100a only)")


for _name, _fn in (("seq_embed", _seq_embed), ("seq_qkv_prepare", _seq_qkv_prepare), ("seq_attention", _seq_attention),
                   ("seq_residual_norm", _seq_residual_norm), ("seq_clamped_glu", _seq_clamped_glu), ("seq_gemv", _seq_gemv)):
    _library.impl(_name, _fn, "CUDA")
    _library.impl(_name, _no_cpu, "CPU")

seq_embed = torch.ops.cold_compress_b200.seq_embed
seq_qkv_prepare = torch.ops.cold_compress_b200.seq_qkv_prepare
seq_attention = torch.ops.cold_compress_b200.seq_attention
seq_residual_norm = torch.ops.cold_compress_b200.seq_residual_norm
seq_clamped_glu = torch.ops.cold_compress_b200.seq_clamped_glu
seq_gemv = torch.ops.cold_compress_b200.seq_gemv


# ------------------------------------------------------------------------------------------------------------------
# Second part of the C ABI (csrc/seq/mix_kernels.cu): state-carrying layers.  Plain functions over the same
# library: every call enqueues on the current stream and reads positions, expert ids and state from device memory.
# A "column range" argument is a 2-D fp32 view whose rows may be strided (a slice of a fused projection's output).

def _cols(t):
    """(pointer, row stride in elements) of a 2-D view with unit column stride."""
    if t is None:
        return None, 0
    if not t.is_cuda:
        raise _lib.CcError("cold_compress_b200 sequence ops run on CUDA tensors only (no CPU fallback)")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise _lib.CcError("expected a 2-D view with contiguous columns")
    return t.data_ptr(), t.stride(0)


def _f32(name, t):
    if t is not None and t.dtype != torch.float32:
        raise _lib.CcError(f"{name}: expected fp32, got {t.dtype}")
    return t


def embed_rows(tokens, embed, x, scale):
    _need(("tokens", tokens, torch.int32), ("embed", embed, None), ("x", x, torch.float32))
    T, E = tokens.numel(), embed.shape[1]
    assert x.shape == (T, E)
    _lib.check_seq(_lib.load_seq().cc_seq_embed_rows(_p(tokens), _p(embed), _dt(embed), _p(x), T, E, float(scale), _stream()),
                   "cc_seq_embed_rows")


def gated_group_norm(x, w, groups, eps, h=None, h_act=None, a=None, ga=None, ba=None, b=None, gb=None, bb=None, rows=None,
                     shift=None):
    """x (fp32 [*, E], in place) += a * sigmoid(ga + ba) + b * sigmoid(gb + bb); h / h_act = grouped RMS norm of it.
    shift (one token only) = (state, mu, hs_act, mix_state, mix_mu, mixes): the token shift of the normed row, and a
    second shift with several mixes on top of it, in the same launch (see cc_b200_seq.h)."""
    _need(("x", x, torch.float32), ("w", w, torch.float32), ("h", h, torch.float32), ("h_act", h_act, None),
          ("ba", ba, torch.float32), ("bb", bb, torch.float32), ("rows", rows, torch.int64))
    g = _lib.CcSeqGatedNorm()
    E = x.shape[-1]
    g.x, g.w, g.h, g.h_act = _p(x), _p(w), _p(h), _p(h_act)
    g.act_dtype = _dt(h_act) if h_act is not None else _lib.DT_F32
    g.a, g.lda = _cols(_f32("a", a))
    g.ga, g.ldga = _cols(_f32("ga", ga))
    g.b, g.ldb = _cols(_f32("b", b))
    g.gb, g.ldgb = _cols(_f32("gb", gb))
    g.ba, g.bb, g.rows = _p(ba), _p(bb), _p(rows)
    g.T = rows.numel() if rows is not None else x.numel() // E
    g.E, g.groups, g.eps = E, int(groups), float(eps)
    if shift is not None:
        state, mu, hs_act, mix_state, mix_mu, mixes = shift
        _need(("state", state, torch.float32), ("mu", mu, torch.float32), ("hs_act", hs_act, None), ("mix_state", mix_state, torch.float32),
              ("mix_mu", mix_mu, torch.float32), ("mixes", mixes, None))
        assert (hs_act is None or g.act_dtype == _dt(hs_act)) and (mixes is None or h_act is None or mixes.dtype == h_act.dtype)
        if h_act is None and (hs_act is not None or mixes is not None):
            g.act_dtype = _dt(hs_act if hs_act is not None else mixes)
        g.shift_state, g.shift_mu, g.hs_act = _p(state), _p(mu), _p(hs_act)
        g.mix_state, g.mix_mu, g.mixes = _p(mix_state), _p(mix_mu), _p(mixes)
        g.n_mix = mix_mu.numel() // E if mix_mu is not None else 0
    _lib.check_seq(_lib.load_seq().cc_seq_gated_group_norm(C.byref(g), _stream()), "cc_seq_gated_group_norm")


def token_shift(h, state, mu, out=None, outf=None):
    """out[s, t] = h[t] + (h[t-1] - h[t]) * mu[s] with h[-1] = state; state <- h[T-1]."""
    _need(("h", h, torch.float32), ("state", state, torch.float32), ("mu", mu, torch.float32), ("out", out, None),
          ("outf", outf, torch.float32))
    T, E = h.shape
    n = mu.numel() // E
    assert state.numel() == E and (out is None or out.numel() == n * T * E)
    _lib.check_seq(_lib.load_seq().cc_seq_token_shift(_p(h), _p(state), _p(mu), _p(out), _dt(out) if out is not None else _lib.DT_F32,
                                                      _p(outf), T, E, n, _stream()), "cc_seq_token_shift")


def gated_unit(src, off_gate, off_up, out, kind):
    """out[t, f] = act(src[t, off_gate + f]) * src[t, off_up + f]  (off_up < 0: activation only)."""
    _need(("out", out, None))
    ptr, ld = _cols(_f32("src", src))
    T, F = out.shape
    _lib.check_seq(_lib.load_seq().cc_seq_gated_unit(ptr, ld, int(off_gate), int(off_up), _p(out), _dt(out), T, F, int(kind),
                                                     _stream()), "cc_seq_gated_unit")


def latent_prepare(src, off_q, q_rank, off_kv, kv_rank, rot_dim, rot_dims, wq, wkv, inv_freq, input_pos, cq, krow, vrow, eps,
                   interleaved=False):
    _need(("wq", wq, torch.float32), ("wkv", wkv, torch.float32), ("inv_freq", inv_freq, torch.float32),
          ("input_pos", input_pos, torch.int32), ("cq", cq, krow.dtype), ("krow", krow, None), ("vrow", vrow, krow.dtype))
    a = _lib.CcSeqLatentPrep()
    a.inp, a.ld = _cols(_f32("src", src))
    a.off_q, a.q_rank, a.off_kv, a.kv_rank, a.rot_dim, a.rot_dims = int(off_q), int(q_rank), int(off_kv), int(kv_rank), int(rot_dim), int(rot_dims)
    a.wq, a.wkv, a.inv_freq, a.input_pos = _p(wq), _p(wkv), _p(inv_freq), _p(input_pos)
    a.cq, a.krow, a.vrow, a.dtype, a.T, a.eps = _p(cq), _p(krow), _p(vrow), _dt(krow), src.shape[0], float(eps)
    a.interleaved = int(bool(interleaved))
    _lib.check_seq(_lib.load_seq().cc_seq_latent_prepare(C.byref(a), _stream()), "cc_seq_latent_prepare")


def rope_heads(q, input_pos, inv_freq, H, head_w, off, seg, dims, tail=None, tail_off=0, interleaved=False):
    """Rotates the segment [off, off + seg) of each of the H heads of q (fp32 [T, >= H * head_w]) in place; pairs
    (i, i + dims / 2), or (2i, 2i + 1) when interleaved."""
    _need(("input_pos", input_pos, torch.int32), ("inv_freq", inv_freq, torch.float32), ("tail", tail, torch.float32))
    ptr, ld = _cols(_f32("q", q))
    _lib.check_seq(_lib.load_seq().cc_seq_rope_heads(ptr, ld, _p(input_pos), _p(inv_freq), q.shape[0], int(H), int(head_w), int(off),
                                                     int(seg), int(dims), _p(tail), tail.shape[-1] if tail is not None else 0,
                                                     int(tail_off), int(bool(interleaved)), _stream()), "cc_seq_rope_heads")


def latent_expand(kv_old, kv_new, lat_old, lat_new, k_old, v_old, k_new, v_new, H, D, V, R, kv_rank):
    a = _lib.CcSeqLatentExpand()
    a.kv_old, ld0 = _cols(_f32("kv_old", kv_old))
    a.kv_new, ld1 = _cols(_f32("kv_new", kv_new))
    a.ld_kv = ld1 or ld0
    assert kv_old is None or kv_new is None or ld0 == ld1
    a.lat_old, l0 = _cols(lat_old)
    a.lat_new, l1 = _cols(lat_new)
    a.ld_lat = l1 or l0
    assert lat_old is None or lat_new is None or l0 == l1
    ref = k_new if k_new is not None else k_old
    _need(("k_old", k_old, ref.dtype), ("v_old", v_old, ref.dtype), ("k_new", k_new, ref.dtype), ("v_new", v_new, ref.dtype))
    a.k_old, a.v_old, a.k_new, a.v_new, a.dtype = _p(k_old), _p(v_old), _p(k_new), _p(v_new), _dt(ref)
    a.n_old = kv_old.shape[0] if kv_old is not None else 0
    a.n_new = kv_new.shape[0] if kv_new is not None else 0
    a.H, a.D, a.V, a.R, a.kv_rank = int(H), int(D), int(V), int(R), int(kv_rank)
    _lib.check_seq(_lib.load_seq().cc_seq_latent_expand(C.byref(a), _stream()), "cc_seq_latent_expand")


def head_gate(y, g):
    """y [T, H, V] *= sigmoid(g[t, h]) (g: fp32 column range [T, H])."""
    _need(("y", y, None))
    ptr, ld = _cols(_f32("g", g))
    T, H, V = y.shape
    _lib.check_seq(_lib.load_seq().cc_seq_head_gate(_p(y), _dt(y), ptr, ld, T, H, V, _stream()), "cc_seq_head_gate")


def head_gemv(w, x, sx, out, so, gate=None):
    """out[h * so + n] = w[h, n, :] . x[h * sx : h * sx + K] (* sigmoid(gate[h])); one token."""
    _need(("w", w, None), ("gate", gate, torch.float32))
    H, N, K = w.shape
    _lib.check_seq(_lib.load_seq().cc_seq_head_gemv(_p(w), _dt(w), x.data_ptr(), _dt(x), int(sx), out.data_ptr(), _dt(out), int(so),
                                                    _p(gate), H, N, K, _stream()), "cc_seq_head_gemv")


def wkv(r, k, v, wraw, w0, u, state, o, H, D):
    _need(*[(n, t, torch.float32) for n, t in (("r", r), ("k", k), ("v", v), ("wraw", wraw), ("w0", w0), ("u", u),
                                               ("state", state), ("o", o))])
    a = _lib.CcSeqWkv()
    a.r, a.k, a.v, a.wraw, a.w0, a.u, a.state, a.o = _p(r), _p(k), _p(v), _p(wraw), _p(w0), _p(u), _p(state), _p(o)
    a.T, a.H, a.D = r.shape[0], int(H), int(D)
    assert r.shape[1] == H * D and state.numel() == H * D * D
    _lib.check_seq(_lib.load_seq().cc_seq_wkv(C.byref(a), _stream()), "cc_seq_wkv")


def head_norm_gate(o, graw, nw, out, H, D, eps):
    _need(("o", o, torch.float32), ("nw", nw, torch.float32), ("out", out, None))
    ptr, ld = _cols(_f32("graw", graw))
    _lib.check_seq(_lib.load_seq().cc_seq_head_norm_gate(_p(o), ptr, ld, _p(nw), _p(out), _dt(out), o.shape[0], int(H), int(D),
                                                         float(eps), _stream()), "cc_seq_head_norm_gate")


def moe_route(logits, correction, ids, wts, groups, keep, top, sigmoid_scores=False, group_top=1, renormalize=True,
              weight_scale=1.0):
    """Router: softmax (or sigmoid) scores, choice = score + correction, the `keep` best of `groups` groups by the sum of
    their `group_top` largest choices, `top` winners; weights = winners' scores (renormalised or not) * weight_scale."""
    _need(("correction", correction, torch.float32), ("ids", ids, torch.int32), ("wts", wts, torch.float32))
    ptr, ld = _cols(_f32("logits", logits))
    T, n = logits.shape
    _lib.check_seq(_lib.load_seq().cc_seq_moe_route(ptr, ld, _p(correction), _p(ids), _p(wts), T, n, int(groups), int(keep), int(top),
                                                    int(bool(sigmoid_scores)), int(group_top), int(bool(renormalize)),
                                                    float(weight_scale), _stream()), "cc_seq_moe_route")


def moe_group(ids, n_real, counts, slot, perm):
    _need(("ids", ids, torch.int32), ("counts", counts, torch.int32), ("slot", slot, torch.int32), ("perm", perm, torch.int32))
    _lib.check_seq(_lib.load_seq().cc_seq_moe_group(_p(ids), ids.numel(), ids.shape[-1], int(n_real), _p(counts), _p(slot), _p(perm),
                                                    _stream()), "cc_seq_moe_group")


def gather_rows(src, perm, dst, M):
    _need(("src", src, None), ("perm", perm, torch.int32), ("dst", dst, src.dtype))
    _lib.check_seq(_lib.load_seq().cc_seq_gather_rows(_p(src), _p(perm), _p(dst), _dt(src), int(M), src.shape[-1], _stream()),
                   "cc_seq_gather_rows")


def moe_expert_tokens(wgu, wd, h, ids, act, y, kind):
    """Experts of a few tokens, no grouping: wgu [n, 2F, E], wd [n, E, F], h [T, E], ids [T, top] -> y fp32 [T * top, E]."""
    _need(("wgu", wgu, None), ("wd", wd, wgu.dtype), ("h", h, wgu.dtype), ("ids", ids, torch.int32), ("act", act, wgu.dtype),
          ("y", y, torch.float32))
    n, F2, E = wgu.shape
    T, top = ids.shape
    _lib.check_seq(_lib.load_seq().cc_seq_moe_expert_tokens(_p(wgu), _p(wd), _p(h), _p(ids), _p(act), _p(y), _dt(wgu), T, top, n,
                                                            F2 // 2, E, int(kind), _stream()), "cc_seq_moe_expert_tokens")


def moe_combine(ids, wts, slot, y, h, shared, sg, out, n_real):
    _need(("ids", ids, torch.int32), ("wts", wts, torch.float32), ("slot", slot, torch.int32), ("y", y, torch.float32),
          ("h", h, torch.float32), ("shared", shared, torch.float32), ("out", out, torch.float32))
    a = _lib.CcSeqMoeCombine()
    a.ids, a.wts, a.slot, a.y, a.h, a.shared, a.out = _p(ids), _p(wts), _p(slot), _p(y), _p(h), _p(shared), _p(out)
    a.sg, a.ld_sg = _cols(_f32("sg", sg))
    a.T, a.top = ids.shape
    a.E, a.n_real = out.shape[-1], int(n_real)
    _lib.check_seq(_lib.load_seq().cc_seq_moe_combine(C.byref(a), _stream()), "cc_seq_moe_combine")


def cache_append(k_new, v_new, k_cache, v_cache, pos, mask, cache_cts, input_pos):
    """Rows k_new [T, G, Dk] / v_new [T, G, Dv] into slots (position mod L) of a cache, with pos / mask / cache_cts.
    v_new = None: the cache has key rows only."""
    _need(("k_new", k_new, k_cache.dtype), ("v_new", v_new, k_cache.dtype), ("k_cache", k_cache, None), ("v_cache", v_cache, k_cache.dtype),
          ("pos", pos, torch.int32), ("mask", mask, torch.bool), ("cache_cts", cache_cts, torch.int32), ("input_pos", input_pos, torch.int32))
    a = _lib.CcSeqAttn()
    a.k_new, a.k_cache = _p(k_new), _p(k_cache)
    a.v_new, a.v_cache = (_p(k_new), _p(k_cache)) if v_new is None else (_p(v_new), _p(v_cache))   # unused with Dv = 0
    a.pos, a.mask, a.cache_cts, a.input_pos = _p(pos), _p(mask), _p(cache_cts), _p(input_pos)
    a.T, a.G, a.Dk = k_new.shape
    a.Dv, a.L, a.H, a.cache_dtype = (0 if v_new is None else v_new.shape[-1]), k_cache.shape[-2], k_new.shape[1], _dt(k_cache)
    _lib.check_seq(_lib.load_seq().cc_seq_cache_append(C.byref(a), _stream()), "cc_seq_cache_append")


def attention_rows(q, k_new, v_new, k_old, v_old, pos_old, input_pos, y, scale, window=0, sink=None):
    """Causal attention of T new tokens over n_old earlier rows and themselves, none of it through a cache object:
    q fp32 [T, H, Dk], k_new [T, G, Dk], v_new [T, G, Dv]; k_old [G, n_old, Dk], v_old [G, n_old, Dv] with pos_old
    int32 [n_old] = the position each old row holds (row j must hold position j); n_old may be 0 (pass None)."""
    _need(("q", q, torch.float32), ("k_new", k_new, None), ("v_new", v_new, k_new.dtype), ("k_old", k_old, k_new.dtype),
          ("v_old", v_old, k_new.dtype), ("pos_old", pos_old, torch.int32), ("input_pos", input_pos, torch.int32), ("y", y, None),
          ("sink", sink, torch.float32))
    a = _lib.CcSeqAttn()
    T, H, Dk = q.shape
    G, Dv = k_new.shape[1], v_new.shape[-1]
    assert k_new.shape == (T, G, Dk) and v_new.shape == (T, G, Dv) and y.shape == (T, H, Dv)
    a.q, a.k_new, a.v_new, a.input_pos, a.y = _p(q), _p(k_new), _p(v_new), _p(input_pos), _p(y)
    if k_old is None:      # no earlier rows: one slot that holds no position
        a.k_cache, a.v_cache, a.pos, a.L = _p(k_new), _p(v_new), _p(_no_position(q.device)), 1
    else:
        assert k_old.shape[0] == G and v_old.shape[:2] == k_old.shape[:2] and pos_old.numel() == k_old.shape[1]
        a.k_cache, a.v_cache, a.pos, a.L = _p(k_old), _p(v_old), _p(pos_old), k_old.shape[1]
    a.T, a.H, a.G, a.Dk, a.Dv = T, H, G, Dk, Dv
    a.window, a.cache_dtype, a.y_dtype, a.scale = int(window), _dt(k_new), _dt(y), float(scale)
    a.sink, a.sink_mode = _p(sink), (_lib.SINK_NONE if sink is None else _lib.SINK_LEARNED)
    _lib.check_seq(_lib.load_seq().cc_seq_attention(C.byref(a), _stream()), "cc_seq_attention")


_NO_POSITION = {}


def _no_position(device):
    t = _NO_POSITION.get(device)
    if t is None:
        t = _NO_POSITION[device] = torch.full((1,), -1, dtype=torch.int32, device=device)
    return t


def latent_decode_workspace_bytes(H, C, L) -> int:
    return int(_lib.load_seq().cc_seq_latent_decode_workspace(int(H), int(C), int(L)))


def latent_decode(q, k_new, k_cache, pos, mask, cache_cts, input_pos, y, scale, workspace, append=True, sink=None):
    """Absorbed one-token latent attention: q fp32 [1, H, Dk] over rows k_cache [.., L, Dk] and k_new [.., Dk] (the newest
    key, appended when asked); y [1, H, C] = weighted sums of the rows' first C columns."""
    _need(("q", q, torch.float32), ("k_new", k_new, k_cache.dtype), ("k_cache", k_cache, None), ("pos", pos, torch.int32),
          ("mask", mask, torch.bool), ("cache_cts", cache_cts, torch.int32), ("input_pos", input_pos, torch.int32), ("y", y, None),
          ("workspace", workspace, None), ("sink", sink, torch.float32))
    a = _lib.CcSeqLatentDecode()
    a.sink = _p(sink)
    a.q, a.k_new, a.k_cache, a.pos, a.mask, a.cache_cts = _p(q), _p(k_new), _p(k_cache), _p(pos), _p(mask), _p(cache_cts)
    a.input_pos, a.y = _p(input_pos), _p(y)
    a.H, a.Dk, a.C, a.L = q.shape[-2], q.shape[-1], y.shape[-1], k_cache.shape[-2]
    assert k_cache.shape[-1] == a.Dk and k_new.numel() == a.Dk and y.numel() == a.H * a.C and pos.numel() == a.L
    a.cache_dtype, a.y_dtype, a.scale, a.append = _dt(k_cache), _dt(y), float(scale), int(bool(append))
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    _lib.check_seq(_lib.load_seq().cc_seq_latent_decode(C.byref(a), _stream()), "cc_seq_latent_decode")


def gemv_multi(jobs):
    """Up to six one-token products in one launch.  jobs: (x, w, out) or (src, w, out, kind, off_gate, off_up) where the
    input is built from the fp32 row `src` as act(src[off_gate + k]) * src[off_up + k]; out fp32 [1, N]."""
    g = _lib.CcSeqGemvMulti()
    g.n_jobs = len(jobs)
    assert 1 <= len(jobs) <= _lib.GEMV_MAX_JOBS
    g.w_dtype = _dt(jobs[0][1])
    for j, job in enumerate(jobs):
        x, w, out = job[:3]
        kind, off_gate, off_up = job[3:] if len(job) > 3 else (_lib.ACT_NONE, 0, -1)
        _need(("x", x, None), ("w", w, jobs[0][1].dtype), ("out", out, torch.float32))
        N, K = w.shape
        built = kind != _lib.ACT_NONE or off_up >= 0
        assert out.numel() == N and (x.numel() >= max(off_gate, off_up) + K if built else x.numel() == K)
        b = g.job[j]
        b.x, b.W, b.out = _p(x), _p(w), _p(out)
        b.x_dtype, b.kind, b.off_gate, b.off_up, b.N, b.K = _dt(x), int(kind), int(off_gate), int(off_up), N, K
    _lib.check_seq(_lib.load_seq().cc_seq_gemv_multi(C.byref(g), _stream()), "cc_seq_gemv_multi")


# ------------------------------------------------------------------------------------------------------------------
# Third part of the C ABI (csrc/seq/scan_kernels.cu): norms after the sum, short convolutions with a carried tail,
# matrix-state scans, gated group norms, rotations of heads, the logit soft cap.

def sum_norm(w, eps, x=None, y=None, y_norm_w=None, y2=None, y2_norm_w=None, y_coef=1.0, y_scale=None, alpha=1.0,
             center=True, gain_offset=0.0, out=None, out_act=None, stack=None, n_prev=0, coef=None, mix=None, rows=None):
    """n = norm(alpha * x + y_scale * y_coef * (y' + y2')) * (w + gain_offset), y' = y or its RMS norm times y_norm_w;
    out <- n; with coef: mix <- sum_j<n_prev coef[j] * stack[j] + coef[n_prev] * n; out_act <- mix (or n) in its dtype.
    `rows` (int64) selects input rows; outputs are compact."""
    _need(("w", w, torch.float32), ("x", x, torch.float32), ("y_norm_w", y_norm_w, torch.float32), ("y2_norm_w", y2_norm_w, torch.float32),
          ("y_scale", y_scale, torch.float32), ("out", out, torch.float32), ("out_act", out_act, None), ("stack", stack, torch.float32),
          ("coef", coef, torch.float32), ("mix", mix, torch.float32), ("rows", rows, torch.int64))
    a = _lib.CcSeqSumNorm()
    E = w.numel()
    ref = x if x is not None else y
    a.T = rows.numel() if rows is not None else ref.shape[0]
    a.E = E
    a.x, a.w, a.y_norm_w, a.y2_norm_w, a.y_scale = _p(x), _p(w), _p(y_norm_w), _p(y2_norm_w), _p(y_scale)
    a.y, a.ldy = _cols(_f32("y", y))
    a.y2, a.ldy2 = _cols(_f32("y2", y2))
    a.y_coef, a.alpha, a.eps, a.gain_offset, a.center = float(y_coef), float(alpha), float(eps), float(gain_offset), int(bool(center))
    a.out, a.out_act, a.rows = _p(out), _p(out_act), _p(rows)
    a.act_dtype = _dt(out_act) if out_act is not None else _lib.DT_F32
    if coef is not None:
        assert mix is not None and coef.numel() >= n_prev + 1 and (n_prev == 0 or stack is not None)
        a.stack, a.stack_stride, a.n_prev, a.coef, a.mix = _p(stack), (stack.stride(0) if stack is not None else 0), int(n_prev), _p(coef), _p(mix)
    _lib.check_seq(_lib.load_seq().cc_seq_sum_norm(C.byref(a), _stream()), "cc_seq_sum_norm")


def short_conv(u, w, bias, tail, out, act=_lib.ACT_NONE):
    """out[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]) with the inputs before this call in `tail`
    [taps - 1, C], which is then moved on.  u / out: fp32 column ranges [T, C]."""
    _need(("w", w, torch.float32), ("bias", bias, torch.float32), ("tail", tail, torch.float32))
    up, ldu = _cols(_f32("u", u))
    op, ldo = _cols(_f32("out", out))
    T, Cn = u.shape
    taps = w.shape[1]
    assert w.shape[0] == Cn and out.shape == u.shape and (taps == 1 or tail.shape == (taps - 1, Cn))
    _lib.check_seq(_lib.load_seq().cc_seq_short_conv(up, ldu, _p(w), _p(bias), _p(tail), op, ldo, T, Cn, taps, int(act), _stream()),
                   "cc_seq_short_conv")


def ssd_scan(x, B, Cm, dt_raw, dt_bias, A_log, D, state, y, H, G, N, V):
    """State-space scan over T tokens: x [T, H*V], B / Cm [T, G*N], dt_raw [T, H] (fp32 column ranges), state fp32
    [H, N, V] carried, y fp32 [T, H*V]."""
    _need(("dt_bias", dt_bias, torch.float32), ("A_log", A_log, torch.float32), ("D", D, torch.float32), ("state", state, torch.float32),
          ("y", y, torch.float32))
    a = _lib.CcSeqSsdScan()
    a.x, a.ldx = _cols(_f32("x", x))
    a.B, a.ldbc = _cols(_f32("B", B))
    a.C, ldc = _cols(_f32("C", Cm))
    a.dt_raw, a.lddt = _cols(_f32("dt_raw", dt_raw))
    assert ldc == a.ldbc and state.numel() == H * N * V and y.shape == (x.shape[0], H * V)
    a.dt_bias, a.A_log, a.D, a.state, a.y = _p(dt_bias), _p(A_log), _p(D), _p(state), _p(y)
    a.T, a.H, a.G, a.N, a.V = x.shape[0], int(H), int(G), int(N), int(V)
    _lib.check_seq(_lib.load_seq().cc_seq_ssd_scan(C.byref(a), _stream()), "cc_seq_ssd_scan")


def delta_scan(q, k, v, beta_raw, a_raw, dt_bias, A_log, state, o, H, G, D, V, q_scale, unit_eps=1e-6):
    """Delta rule with a decay per key channel over T tokens: q / k [T, G*D], v [T, H*V], beta_raw [T, H], a_raw
    [T, H*D] (fp32 column ranges), state fp32 [H, D, V] carried, o fp32 [T, H*V]."""
    _need(("dt_bias", dt_bias, torch.float32), ("A_log", A_log, torch.float32), ("state", state, torch.float32), ("o", o, torch.float32))
    a = _lib.CcSeqDeltaScan()
    a.q, a.ldqk = _cols(_f32("q", q))
    a.k, ldk = _cols(_f32("k", k))
    a.v, a.ldv = _cols(_f32("v", v))
    a.beta_raw, a.ldb = _cols(_f32("beta_raw", beta_raw))
    a.a_raw, a.lda = _cols(_f32("a_raw", a_raw))
    assert ldk == a.ldqk and state.numel() == H * D * V and o.shape == (q.shape[0], H * V) and dt_bias.numel() == H * D
    a.dt_bias, a.A_log, a.state, a.o = _p(dt_bias), _p(A_log), _p(state), _p(o)
    a.T, a.H, a.G, a.D, a.V = q.shape[0], int(H), int(G), int(D), int(V)
    a.q_scale, a.unit_eps = float(q_scale), float(unit_eps)
    lib = _lib.load_seq()
    if a.T >= DELTA_PREPARE_FROM:
        # long steps: the per-token preparation (unit vectors, decays, beta) in a launch of its own, spread over the GPU,
        # instead of once per column tile inside the scan; same arithmetic, same bits
        f32 = dict(dtype=torch.float32, device=o.device)
        qn, kn, gd = (torch.empty(a.T, H * D, **f32) for _ in range(3))
        bt, qk = torch.empty(a.T, H, **f32), torch.empty(a.T, H, **f32)
        _lib.check_seq(lib.cc_seq_delta_prepare(C.byref(a), _p(qn), _p(kn), _p(gd), _p(bt), _p(qk), _stream()), "cc_seq_delta_prepare")
        a.q, a.k, a.ldqk, a.a_raw, a.lda, a.beta_raw, a.ldb = _p(qn), _p(kn), H * D, _p(gd), H * D, _p(bt), H
        a.qk, a.G, a.prepared = _p(qk), int(H), 1
    _lib.check_seq(lib.cc_seq_delta_scan(C.byref(a), _stream()), "cc_seq_delta_scan")


DELTA_PREPARE_FROM = 64


def gated_rms_groups(y, gate, gate_act, gate_first, w, out, groups, eps):
    """out = group-wise RMS norm of y [T, W] times w[col mod len(w)], gated by act(gate) before or after the norm."""
    _need(("y", y, torch.float32), ("w", w, torch.float32), ("out", out, None))
    gp, ldg = _cols(_f32("gate", gate))
    T, W = y.shape
    _lib.check_seq(_lib.load_seq().cc_seq_gated_rms_groups(_p(y), gp, ldg, int(gate_act), int(bool(gate_first)), _p(w), w.numel(),
                                                           _p(out), _dt(out), T, W, int(groups), float(eps), _stream()),
                   "cc_seq_gated_rms_groups")


def qkv_rope(src, off_q, off_k, off_v, H, G, Dk, Dv, q_norm_w, k_norm_w, eps, rot_dims, interleaved, inv_freq, v_inv_freq,
             input_pos, q_out, k_out, v_out):
    _need(("q_norm_w", q_norm_w, torch.float32), ("k_norm_w", k_norm_w, torch.float32), ("inv_freq", inv_freq, torch.float32),
          ("v_inv_freq", v_inv_freq, torch.float32), ("input_pos", input_pos, torch.int32), ("q_out", q_out, torch.float32),
          ("k_out", k_out, None), ("v_out", v_out, k_out.dtype))
    a = _lib.CcSeqQkvRope()
    a.inp, a.ld = _cols(_f32("src", src))
    a.off_q, a.off_k, a.off_v, a.H, a.G, a.Dk, a.Dv = int(off_q), int(off_k), int(off_v), int(H), int(G), int(Dk), int(Dv)
    a.q_norm_w, a.k_norm_w, a.eps, a.rot_dims, a.interleaved = _p(q_norm_w), _p(k_norm_w), float(eps), int(rot_dims), int(bool(interleaved))
    assert (rot_dims == 0 or inv_freq.numel() >= rot_dims // 2) and (v_inv_freq is None or (Dv % 2 == 0 and v_inv_freq.numel() >= Dv // 2))
    a.inv_freq, a.v_inv_freq, a.input_pos = _p(inv_freq), _p(v_inv_freq), _p(input_pos)
    a.q_out, a.k_out, a.v_out, a.out_dtype, a.T = _p(q_out), _p(k_out), _p(v_out), _dt(k_out), src.shape[0]
    _lib.check_seq(_lib.load_seq().cc_seq_qkv_rope(C.byref(a), _stream()), "cc_seq_qkv_rope")


def turn_heads_gate(y, input_pos, inv_freq, dims, interleaved, sign, gate, out):
    """out[t, h] = turn(y[t, h], sign * position) * sigmoid(gate[t, h]); y fp32 [T, H, Dv]."""
    _need(("y", y, torch.float32), ("input_pos", input_pos, torch.int32), ("inv_freq", inv_freq, torch.float32), ("out", out, None))
    gp, ldg = _cols(_f32("gate", gate))
    T, H, Dv = y.shape
    _lib.check_seq(_lib.load_seq().cc_seq_turn_heads_gate(_p(y), _p(input_pos), _p(inv_freq), int(dims), int(bool(interleaved)),
                                                          float(sign), gp, ldg, _p(out), _dt(out), T, H, Dv, _stream()),
                   "cc_seq_turn_heads_gate")


def softcap(x, cap):
    _need(("x", x, torch.float32))
    _lib.check_seq(_lib.load_seq().cc_seq_softcap(_p(x), x.numel(), float(cap), _stream()), "cc_seq_softcap")


# ------------------------------------------------------------------------------------------------------------------
# Fourth part of the C ABI (csrc/seq/par_kernels.cu): sublayers that read norms of one stream through a short
# convolution added to its own input, whole-row query / key norms, the polynomial-of-unit-RMS activation.

def par_norm(x, outs, eps, a=None, b=None, add=None, tail=None, taps=1, rinv=None, x_out=None):
    """x (fp32 [T, E], in place) += a + b + add; then per entry (gain, conv_w, out) of `outs`: out = h + causal conv of h
    over time with h = unit_rms(x) * gain (conv_w fp32 [E, taps] or None).  `tail` fp32 [taps - 1, E] carries the
    unit-RMS rows before the step; `rinv` fp32 [T] is scratch for steps of several tokens.  `x_out` (one token): the
    summed row goes there instead of into x, and the launch spreads the row's channels over the GPU."""
    _need(("x", x, torch.float32), ("x_out", x_out, torch.float32), ("add", add, torch.float32), ("tail", tail, torch.float32), ("rinv", rinv, torch.float32))
    g = _lib.CcSeqParNorm()
    T, E = x.shape
    assert rinv is None or rinv.numel() >= T
    assert x_out is None or (x_out.shape == x.shape and x_out.data_ptr() != x.data_ptr())
    g.x, g.add, g.rinv, g.tail, g.x_out = _p(x), _p(add), _p(rinv), _p(tail), _p(x_out)
    g.a, g.lda = _cols(_f32("a", a))
    g.b, g.ldb = _cols(_f32("b", b))
    assert 1 <= len(outs) <= _lib.PAR_MAX_OUT and (taps == 1 or tail.shape == (taps - 1, E))
    for s, (gain, conv_w, out) in enumerate(outs):
        _need(("gain", gain, torch.float32), ("conv_w", conv_w, torch.float32), ("out", out, outs[0][2].dtype))
        assert gain.numel() == E and out.shape == (T, E) and (conv_w is None or conv_w.shape == (E, taps))
        g.gain[s], g.conv_w[s], g.out[s] = _p(gain), _p(conv_w), _p(out)
    g.n_out, g.act_dtype, g.T, g.E, g.taps, g.eps = len(outs), _dt(outs[0][2]), T, E, int(taps), float(eps)
    _lib.check_seq(_lib.load_seq().cc_seq_par_norm(C.byref(g), _stream()), "cc_seq_par_norm")


def qk_row_norm(src, off_q, nq, off_k, nk, off_v, nv, wq, wk, q_out, k_out, v_out, eps):
    """q and k column ranges of the fused projection `src` RMS-normed over their whole width (all heads at once) with
    gains wq / wk; v copied.  q_out fp32, k_out / v_out in the cache's type."""
    _need(("wq", wq, torch.float32), ("wk", wk, torch.float32), ("q_out", q_out, torch.float32), ("k_out", k_out, None),
          ("v_out", v_out, k_out.dtype))
    a = _lib.CcSeqQkRowNorm()
    a.inp, a.ld = _cols(_f32("src", src))
    a.off_q, a.nq, a.off_k, a.nk, a.off_v, a.nv = int(off_q), int(nq), int(off_k), int(nk), int(off_v), int(nv)
    T = src.shape[0]
    assert wq.numel() == nq and wk.numel() == nk and q_out.numel() == T * nq and k_out.numel() == T * nk and v_out.numel() == T * nv
    a.wq, a.wk, a.q_out, a.k_out, a.v_out, a.out_dtype, a.T, a.eps = _p(wq), _p(wk), _p(q_out), _p(k_out), _p(v_out), _dt(k_out), T, float(eps)
    _lib.check_seq(_lib.load_seq().cc_seq_qk_row_norm(C.byref(a), _stream()), "cc_seq_qk_row_norm")


def poly_norm(src, coef, out, eps):
    """out = coef[0] N(z) + coef[1] N(z^2) + coef[2] N(z^3) + coef[3] over the rows z of `src` (fp32 column range [T, F])."""
    _need(("coef", coef, torch.float32), ("out", out, None))
    ptr, ld = _cols(_f32("src", src))
    T, F = out.shape
    assert src.shape == (T, F) and coef.numel() == 4
    _lib.check_seq(_lib.load_seq().cc_seq_poly_norm(ptr, ld, _p(coef), _p(out), _dt(out), T, F, float(eps), _stream()), "cc_seq_poly_norm")
