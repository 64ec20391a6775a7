"""GPU tests of the Tefovik design: every mechanism's kernel against the plain restatement in tefovik_reference.py
(float64, CPU, whole sequences), then the model through the runtime: layer by layer, prompt against token-by-token
decoding, prompt portions down to two tokens, state and cache rows that are given back and used again, one key just
inside or just outside a block and one old token that decides the output, long decoding, other sizes, greedy
generation through generate() and the graph-captured decoder, and the trace replay command."""
import json

import pytest
import torch

import tefovik_reference as R
from tefovik_utils import (assert_rows_close, attention, build_model, default_layers, delta, dense, fp32_tolerance, make_config,
                           mamba_layer, parallel_layer, random_weights, row_error, run_portions)

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16_TOL = 6e-2
F64 = torch.float64


def _ops():
    from cold_compress_b200 import seq_ops
    return seq_ops


def _lib():
    from cold_compress_b200 import _lib
    return _lib


def _i32(*v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _tol(dtype, cfg, W, tokens, want):
    return BF16_TOL if dtype == torch.bfloat16 else fp32_tolerance(cfg, W, tokens, want)


def _close(got, want, rel):
    want = want.double()
    err = (got.detach().cpu().double() - want).abs().max().item()
    assert err <= rel * max(want.abs().max().item(), 1e-30), (err, want.abs().max().item())


# ----------------------------------------------------------------------------------------------- single mechanisms

@pytest.mark.parametrize("E", [1, 50, 640])
def test_norm_after_the_sum_kernel(E):
    ops = _ops()
    g = torch.Generator().manual_seed(E)
    T, eps, alpha = 6, 1e-5, 2.5
    x, w, ls, wa, wb = (torch.randn(T, E, generator=g) * 3 + 1.0, torch.randn(E, generator=g), torch.randn(E, generator=g),
                        torch.randn(E, generator=g), torch.randn(E, generator=g))
    wide = torch.randn(T, 2 * E + 3, generator=g)          # sublayer results as column ranges of wider rows
    y, y2 = wide[:, 1:1 + E], wide[:, 2 + E:2 + 2 * E]
    d = lambda t: t.double()
    xd, wd_, lsd, wided = x.to(DEV), w.to(DEV), ls.to(DEV), wide.to(DEV)
    yd, y2d = wided[:, 1:1 + E], wided[:, 2 + E:2 + 2 * E]
    # plain layer norm of a row; with the sum and the layer scale
    out = torch.empty(T, E, device=DEV)
    ops.sum_norm(wd_, eps, x=xd, out=out)
    _close(out, R.layer_norm(d(x), d(w), eps), 2e-5)
    act = torch.empty(T, E, device=DEV, dtype=torch.bfloat16)
    ops.sum_norm(wd_, eps, x=xd, y=yd, y_scale=lsd, alpha=alpha, out=out, out_act=act)
    want = R.layer_norm(alpha * d(x) + d(ls) * d(y), d(w), eps)
    _close(out, want, 2e-5)
    assert torch.equal(act, out.to(torch.bfloat16))
    # two sublayer results, each RMS-normed with its own gain, averaged
    ops.sum_norm(wd_, eps, x=xd, y=yd, y_norm_w=wa.to(DEV), y2=y2d, y2_norm_w=wb.to(DEV), y_coef=0.5, y_scale=lsd, alpha=alpha, out=out)
    pair = 0.5 * (R.rms_norm(d(y), d(wa), eps) + R.rms_norm(d(y2), d(wb), eps))
    _close(out, R.layer_norm(alpha * d(x) + d(ls) * pair, d(w), eps), 3e-5)
    # the depth average that follows: stack rows of three earlier results, the new one goes to its slot
    stack = torch.randn(4, T, E, generator=g).to(DEV)
    coef = torch.randn(4, generator=g)
    mix = torch.empty(T, E, device=DEV)
    ops.sum_norm(wd_, eps, x=xd, y=yd, alpha=alpha, out=stack[3], stack=stack, n_prev=3, coef=coef.to(DEV), mix=mix, out_act=act)
    n = R.layer_norm(alpha * d(x) + d(y), d(w), eps)
    _close(stack[3], n, 2e-5)
    want = sum(d(coef[j]) * d(stack[j].cpu()) for j in range(3)) + d(coef[3]) * n
    _close(mix, want, 3e-5)
    assert torch.equal(act, mix.to(torch.bfloat16))
    # the input may be overwritten by the average; rows can be selected; an RMS norm with a gain stored as an offset
    x2 = x.to(DEV)
    ops.sum_norm(wd_, eps, x=x2, y=yd, alpha=alpha, out=stack[3], stack=stack, n_prev=3, coef=coef.to(DEV), mix=x2)
    assert torch.equal(x2, mix)
    rows = torch.tensor([4, 0, 4], device=DEV)
    out3 = torch.empty(3, E, device=DEV)
    ops.sum_norm(wd_, eps, x=xd, rows=rows, out_act=out3)
    _close(out3, R.layer_norm(d(x), d(w), eps)[[4, 0, 4]], 2e-5)
    ops.sum_norm(wd_, eps, x=xd, center=False, gain_offset=1.0, out=out)
    _close(out, R.rms_norm(d(x), d(w) + 1.0, eps), 2e-5)


@pytest.mark.parametrize("taps,C,bias,act", [(1, 5, False, "none"), (2, 33, True, "silu"), (4, 300, False, "silu"), (7, 64, True, "none")])
def test_short_convolution_carries_its_tail_across_portions(taps, C, bias, act):
    ops, lib = _ops(), _lib()
    g = torch.Generator().manual_seed(taps)
    T = 23
    wide = torch.randn(T, C + 4, generator=g)
    u, w = wide[:, 2:2 + C], torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    want, last = R.short_conv(u.double(), w.double(), None if b is None else b.double())
    if act == "silu":
        want = torch.nn.functional.silu(want)
    tail = torch.zeros(max(taps - 1, 0), C, device=DEV)
    got, at = [], 0
    for n in (1, 1, 2, 9, 1, 5, 2, 2):
        src = wide[at:at + n].to(DEV)
        out = torch.empty(n, C + 1, device=DEV)
        ops.short_conv(src[:, 2:2 + C], w.to(DEV), None if b is None else b.to(DEV), tail if taps > 1 else None, out[:, 1:],
                       lib.ACT_SILU if act == "silu" else lib.ACT_NONE)
        got.append(out[:, 1:])
        at += n
        if taps > 1:   # the tail is the last taps - 1 inputs seen so far, zeros before the start
            seen = torch.cat([torch.zeros(taps - 1, C), u[:at]])[-(taps - 1):]
            assert torch.equal(tail.cpu(), seen)
    _close(torch.cat(got), want, 1e-6)
    assert taps == 1 or torch.equal(tail.cpu().double(), last)


def _ssd_inputs(T, H, G, N, V, seed, slow=False):
    g = torch.Generator().manual_seed(seed)
    x, B, C = torch.randn(T, H * V, generator=g), torch.randn(T, G * N, generator=g), torch.randn(T, G * N, generator=g)
    dt_raw = torch.randn(T, H, generator=g) - (4.0 if slow else 0.5)
    dt_bias, A_log, D = torch.randn(H, generator=g) * 0.3, torch.randn(H, generator=g) * 0.5 - (3.0 if slow else 0.3), torch.randn(H, generator=g)
    return x, B, C, dt_raw, dt_bias, A_log, D


def _ssd_want(x, B, C, dt_raw, dt_bias, A_log, D, H, G, N, V):
    d = lambda t: t.double()
    T = x.shape[0]
    dt = R.softplus(d(dt_raw) + d(dt_bias))
    return R.state_space_scan(d(x).view(T, H, V), d(B).view(T, G, N), d(C).view(T, G, N), dt, torch.exp(-torch.exp(d(A_log)) * dt), d(D))


@pytest.mark.parametrize("H,G,N,V", [(1, 1, 1, 1), (4, 2, 20, 12), (3, 1, 52, 40), (2, 2, 130, 70), (6, 3, 64, 32)])
def test_state_space_scan_kernel_in_portions(H, G, N, V):
    ops = _ops()
    T = 45
    x, B, C, dt_raw, dt_bias, A_log, D = _ssd_inputs(T, H, G, N, V, seed=H * 100 + N)
    want, S_want = _ssd_want(x, B, C, dt_raw, dt_bias, A_log, D, H, G, N, V)
    fused = torch.cat([x, B, C, dt_raw], 1).to(DEV)          # column ranges of one wide row, as the mixer passes them
    state = torch.zeros(H, N, V, device=DEV)
    got, at = [], 0
    for n in (1, 1, 2, 17, 1, 20, 3):
        f = fused[at:at + n]
        y = torch.empty(n, H * V, device=DEV)
        ops.ssd_scan(f[:, :H * V], f[:, H * V:H * V + G * N], f[:, H * V + G * N:H * V + 2 * G * N], f[:, H * V + 2 * G * N:],
                     dt_bias.to(DEV), A_log.to(DEV), D.to(DEV), state, y, H, G, N, V)
        got.append(y)
        at += n
    _close(torch.cat(got).view(T, H, V), want, 2e-5)
    _close(state, S_want, 2e-5)
    # the same bits whatever the portions
    state2 = torch.zeros(H, N, V, device=DEV)
    y2 = torch.empty(T, H * V, device=DEV)
    ops.ssd_scan(fused[:, :H * V], fused[:, H * V:H * V + G * N], fused[:, H * V + G * N:H * V + 2 * G * N], fused[:, H * V + 2 * G * N:],
                 dt_bias.to(DEV), A_log.to(DEV), D.to(DEV), state2, y2, H, G, N, V)
    assert torch.equal(y2, torch.cat(got)) and torch.equal(state2, state)


def test_state_space_scan_keeps_a_loud_token_600_steps():
    """Decays near one: the one loud input, 600 tokens back, is most of what the last token reads."""
    ops = _ops()
    H, G, N, V, T = 2, 1, 16, 8, 640
    x, B, C, dt_raw, dt_bias, A_log, D = _ssd_inputs(T, H, G, N, V, seed=7, slow=True)
    x = x * 0.01
    x[39] = 50.0
    dt_raw[39] = 3.0
    want, _ = _ssd_want(x, B, C, dt_raw, dt_bias, A_log, D, H, G, N, V)
    quiet = x.clone()
    quiet[39] = 0.0
    base, _ = _ssd_want(quiet, B, C, dt_raw, dt_bias, A_log, D, H, G, N, V)
    assert (want[-1] - base[-1]).abs().max() > 20 * base[-1].abs().max()          # the test's premise
    for portions in ((T,), (40, 599, 1), (300,) + (1,) * 340):
        state = torch.zeros(H, N, V, device=DEV)
        got, at = [], 0
        for n in portions:
            y = torch.empty(n, H * V, device=DEV)
            sl = slice(at, at + n)
            ops.ssd_scan(x[sl].to(DEV), B[sl].to(DEV), C[sl].to(DEV), dt_raw[sl].to(DEV), dt_bias.to(DEV), A_log.to(DEV), D.to(DEV),
                         state, y, H, G, N, V)
            got.append(y)
            at += n
        _close(torch.cat(got)[-1].view(H, V), want[-1], 1e-4)


def _delta_inputs(T, H, G, D, V, seed, slow=False):
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, G * D, generator=g), torch.randn(T, G * D, generator=g), torch.randn(T, H * V, generator=g)
    beta_raw, a_raw = torch.randn(T, H, generator=g), torch.randn(T, H * D, generator=g) - (5.0 if slow else 0.0)
    dt_bias, A_log = torch.randn(H * D, generator=g) * 0.3, torch.randn(H, generator=g) * 0.5 - (3.0 if slow else 0.5)
    return q, k, v, beta_raw, a_raw, dt_bias, A_log


def _delta_want(q, k, v, beta_raw, a_raw, dt_bias, A_log, H, G, D, V):
    d = lambda t: t.double()
    T = q.shape[0]
    decay = torch.exp(-torch.exp(d(A_log)).view(1, H, 1) * R.softplus(d(a_raw) + d(dt_bias)).view(T, H, D))
    return R.delta_rule_scan(R.unit_vectors(d(q).view(T, G, D)) * D ** -0.5, R.unit_vectors(d(k).view(T, G, D)), d(v).view(T, H, V),
                             torch.sigmoid(d(beta_raw)), decay)


@pytest.mark.parametrize("H,G,D,V", [(1, 1, 1, 1), (4, 2, 24, 10), (2, 2, 64, 32), (2, 1, 136, 40), (3, 3, 33, 70)])
def test_delta_rule_scan_kernel_in_portions(H, G, D, V):
    ops = _ops()
    T = 45
    q, k, v, beta_raw, a_raw, dt_bias, A_log = _delta_inputs(T, H, G, D, V, seed=H * 100 + D)
    want, S_want = _delta_want(q, k, v, beta_raw, a_raw, dt_bias, A_log, H, G, D, V)
    fused = torch.cat([q, k, v, beta_raw], 1).to(DEV)
    state = torch.zeros(H, D, V, device=DEV)

    def run(sl, st):
        f = fused[sl]
        o = torch.empty(f.shape[0], H * V, device=DEV)
        ops.delta_scan(f[:, :G * D], f[:, G * D:2 * G * D], f[:, 2 * G * D:2 * G * D + H * V], f[:, 2 * G * D + H * V:],
                       a_raw[sl].to(DEV), dt_bias.to(DEV), A_log.to(DEV), st, o, H, G, D, V, D ** -0.5)
        return o

    got, at = [], 0
    for n in (1, 1, 2, 17, 1, 20, 3):
        got.append(run(slice(at, at + n), state))
        at += n
    _close(torch.cat(got).view(T, H, V), want, 3e-5)
    _close(state, S_want, 3e-5)
    state2 = torch.zeros(H, D, V, device=DEV)
    assert torch.equal(run(slice(0, T), state2), torch.cat(got)) and torch.equal(state2, state)


def test_delta_rule_keeps_a_loud_token_600_steps():
    ops = _ops()
    H, G, D, V, T = 2, 2, 16, 8, 640
    q, k, v, beta_raw, a_raw, dt_bias, A_log = _delta_inputs(T, H, G, D, V, seed=9, slow=True)
    v = v * 0.01
    v[39] = 40.0
    beta_raw[39] = 6.0
    # the loud token's key is the first channel alone, which no other key touches (a delta rule erases what later keys
    # overlap); the last query asks for exactly that channel
    k.view(T, G, D)[:, :, 0] = 0.0
    k[39] = 0.0
    k.view(T, G, D)[39, :, 0] = 3.0
    q[-1] = k[39]
    want, _ = _delta_want(q, k, v, beta_raw, a_raw, dt_bias, A_log, H, G, D, V)
    quiet = v.clone()
    quiet[39] = 0.0
    base, _ = _delta_want(q, k, quiet, beta_raw, a_raw, dt_bias, A_log, H, G, D, V)
    assert (want[-1] - base[-1]).abs().max() > 20 * base[-1].abs().max()
    for portions in ((T,), (40, 599, 1), (300,) + (1,) * 340):
        state = torch.zeros(H, D, V, device=DEV)
        got, at = [], 0
        for n in portions:
            sl = slice(at, at + n)
            o = torch.empty(n, H * V, device=DEV)
            ops.delta_scan(q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), beta_raw[sl].to(DEV), a_raw[sl].to(DEV), dt_bias.to(DEV),
                           A_log.to(DEV), state, o, H, G, D, V, D ** -0.5)
            got.append(o)
            at += n
        _close(torch.cat(got)[-1].view(H, V), want[-1], 1e-4)


@pytest.mark.parametrize("first", [True, False])
@pytest.mark.parametrize("W_,groups,wlen", [(40, 1, 40), (96, 4, 96), (70, 7, 10), (4100, 1, 4100)])
def test_gated_group_norm_kernel(first, W_, groups, wlen):
    ops, lib = _ops(), _lib()
    g = torch.Generator().manual_seed(W_)
    T, eps = 5, 1e-5
    y, wide, w = torch.randn(T, W_, generator=g) * 2, torch.randn(T, W_ + 6, generator=g), torch.randn(wlen, generator=g)
    gate = wide[:, 3:3 + W_]
    d = lambda t: t.double()
    wfull = d(w).repeat(W_ // wlen)
    if first:
        want = R.group_rms(d(y) * torch.nn.functional.silu(d(gate)), groups, eps) * wfull
    else:
        want = R.group_rms(d(y), groups, eps) * wfull * torch.sigmoid(d(gate))
    out = torch.empty(T, W_, device=DEV)
    wd = wide.to(DEV)
    ops.gated_rms_groups(y.to(DEV), wd[:, 3:3 + W_], lib.ACT_SILU if first else lib.ACT_SIGMOID, first, w.to(DEV), out, groups, eps)
    _close(out, want, 2e-5)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("H,G,Dk,Dv,dims,p0", [(1, 1, 2, 2, 2, 0), (6, 2, 16, 20, 16, 5), (4, 4, 24, 8, 10, 90000), (5, 1, 70, 66, 0, 17)])
def test_head_rows_norm_and_rotation_kernels(interleaved, H, G, Dk, Dv, dims, p0):
    ops = _ops()
    from cold_compress_b200.tefovik import _inv_freq
    g = torch.Generator().manual_seed(H * 10 + Dk)
    T, eps, base = 9, 1e-5, 300.0
    nq, nk, nv = H * Dk, G * Dk, G * Dv
    wide = torch.randn(T, nq + nk + nv + 3, generator=g)
    qn, kn = torch.randn(Dk, generator=g), torch.randn(Dk, generator=g)
    d = lambda t: t.double()
    pos = torch.arange(p0, p0 + T)
    src = d(wide)[:, 2:]
    qw = R.rotate_pairs(R.rms_norm(src[:, :nq].reshape(T, H, Dk), d(qn), eps), pos, base, dims, interleaved) if dims else \
        R.rms_norm(src[:, :nq].reshape(T, H, Dk), d(qn), eps)
    kw = R.rotate_pairs(R.rms_norm(src[:, nq:nq + nk].reshape(T, G, Dk), d(kn), eps), pos, base, dims, interleaved) if dims else \
        R.rms_norm(src[:, nq:nq + nk].reshape(T, G, Dk), d(kn), eps)
    vw = R.rotate_pairs(src[:, nq + nk:nq + nk + nv].reshape(T, G, Dv), pos, base, Dv, interleaved)
    q = torch.empty(T, H, Dk, device=DEV)
    k, v = torch.empty(T, G, Dk, device=DEV), torch.empty(T, G, Dv, device=DEV)
    f, fv = _inv_freq(base, dims).to(DEV), _inv_freq(base, Dv).to(DEV)
    ops.qkv_rope(wide.to(DEV)[:, 2:], 0, nq, nq + nk, H, G, Dk, Dv, qn.to(DEV), kn.to(DEV), eps, dims, interleaved, f, fv, _i32(p0), q, k, v)
    tol = 2e-5 if p0 < 1000 else 2e-2        # an fp32 angle near 90000 rad carries up to 1e-2 rad of rounding (product and frequency)
    _close(q, qw, tol)
    _close(k, kw, tol)
    _close(v, vw, tol)
    # outputs of H heads turned back by the position and gated per head
    y, gates = torch.randn(T, H, Dv, generator=g), torch.randn(T, H + 2, generator=g)
    want = R.rotate_pairs(d(y), pos, base, Dv, interleaved, sign=-1.0) * torch.sigmoid(d(gates[:, 1:1 + H]))[:, :, None]
    out = torch.empty(T, H, Dv, device=DEV)
    ops.turn_heads_gate(y.to(DEV), _i32(p0), fv, Dv, interleaved, -1.0, gates.to(DEV)[:, 1:1 + H], out)
    _close(out, want, tol)


def test_soft_cap_kernel():
    x = torch.randn(3, 777, generator=torch.Generator().manual_seed(1)) * 40
    xd = x.to(DEV)
    _ops().softcap(xd, 25.0)
    _close(xd, 25.0 * torch.tanh(x.double() / 25.0), 1e-6)


# ----------------------------------------------------------------------------------------------- block-masked attention over the ring

def _ring(G, Dk, Dv, block, dtype):
    from cold_compress_b200.cache import get_cache_constructor
    ctor, _ = get_cache_constructor("recent_global")
    with torch.device(DEV):
        return ctor(1, G, Dk, dtype, v_head_dim=Dv, max_cache_length=block, max_seq_length=4096, global_tokens=0, cache_bits=None)


def _attend(cache, q, k, v, portions, block, scale, dtype):
    got, at = [], 0
    for n in portions:
        y = torch.empty(n, q.shape[1], v.shape[2], device=DEV)
        cache.sequence_step(q[at:at + n].to(DEV).contiguous(), k[at:at + n].to(DEV, dtype).contiguous(), v[at:at + n].to(DEV, dtype).contiguous(),
                            _i32(at), y, scale=scale, block=block)
        got.append(y)
        at += n
    return torch.cat(got).cpu().double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,Dk,Dv,block", [(6, 2, 16, 20, 9), (4, 4, 12, 8, 16), (10, 1, 56, 40, 70), (3, 1, 5, 3, 1), (17, 1, 8, 8, 33)])
def test_block_masked_attention_in_portions_and_single_tokens(dtype, H, G, Dk, Dv, block):
    g = torch.Generator().manual_seed(block)
    T = 150
    q, k, v = torch.randn(T, H, Dk, generator=g), torch.randn(T, G, Dk, generator=g), torch.randn(T, G, Dv, generator=g)
    if dtype == torch.bfloat16:
        k, v = k.bfloat16().float(), v.bfloat16().float()
    pos = torch.arange(T)
    want = R.block_attention(q.double(), k.double(), v.double(), pos, pos, 0.3, block)
    for portions in ((T,), (7, 2, 64, 33, 2, 40, 1, 1), (100,) + (1,) * 50, (1,) * T):
        cache = _ring(G, Dk, Dv, block, dtype)
        got = _attend(cache, q, k, v, portions, block, 0.3, dtype)
        assert (got - want).abs().max() < 2e-5 * max(1.0, want.abs().max()), (portions[:3], (got - want).abs().max())


@pytest.mark.parametrize("mode", ["prompt", "portions", "decode"])
@pytest.mark.parametrize("where", ["first_of_block", "last_of_previous_block", "own_position"])
def test_one_key_just_inside_or_outside_the_block_decides(mode, where):
    """One key's score stands far above the rest.  Inside the query's block it takes the whole softmax; one position
    earlier (the last of the block before) it must not be seen at all."""
    block, T, Dk, Dv = 44, 44 * 5 + 20, 16, 8
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(T, 2, Dk, generator=g) * 0.1, torch.randn(T, 1, Dk, generator=g) * 0.1, torch.randn(T, 1, Dv, generator=g)
    last = T - 1
    start = (last // block) * block
    j = {"first_of_block": start, "last_of_previous_block": start - 1, "own_position": last}[where]
    k[j, 0] = 0.0
    k[j, 0, 3] = 30.0
    q[last, :, 3] = 30.0          # score 900 x scale against |others| < 1
    v[j] = 100.0
    pos = torch.arange(T)
    want = R.block_attention(q.double(), k.double(), v.double(), pos, pos, 0.25, block)
    if where == "last_of_previous_block":
        assert want[last].abs().max() < 10
    else:
        assert (want[last] - 100.0).abs().max() < 1e-6
    portions = {"prompt": (T,), "portions": (start - 1, 2, T - start - 1), "decode": (start - 3,) + (1,) * (T - start + 3)}[mode]
    got = _attend(_ring(1, Dk, Dv, block, torch.float32), q, k, v, portions, block, 0.25, torch.float32)
    assert (got - want).abs().max() < 1e-4


def test_ring_rows_given_back_are_not_keys():
    """A second sequence after a longer one through the same ring: rows the first left behind must not be attended."""
    block, Dk, Dv = 20, 8, 6
    g = torch.Generator().manual_seed(4)
    cache = _ring(2, Dk, Dv, block, torch.float32)
    a = [torch.randn(57, h, d, generator=g) * 3 for h, d in ((4, Dk), (2, Dk), (2, Dv))]
    _attend(cache, *a, (57,), block, 0.5, torch.float32)
    cache.reset()
    b = [torch.randn(31, h, d, generator=g) for h, d in ((4, Dk), (2, Dk), (2, Dv))]
    pos = torch.arange(31)
    want = R.block_attention(*[t.double() for t in b], pos, pos, 0.5, block)
    got = _attend(cache, *b, (5, 1, 1, 17, 7), block, 0.5, torch.float32)
    assert (got - want).abs().max() < 2e-5
    assert int(cache.cache_cts.item()) == block


# ----------------------------------------------------------------------------------------------- the model in the runtime

def _reference_logits(cfg, W, tokens, collect=None):
    return R.forward(cfg, W, tokens, collect=collect)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_one_by_one_and_logits(dtype):
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=5)
    tokens = torch.randint(0, cfg["vocab"], (41,), generator=torch.Generator().manual_seed(6)).tolist()
    ref_layers = []
    want = _reference_logits(cfg, W, tokens, ref_layers)
    model = build_model(cfg, W, dtype, 41)
    got_layers = []
    x = torch.tensor(tokens, dtype=torch.int32, device=DEV).view(1, -1)
    got = model(x, torch.arange(41, dtype=torch.int32, device=DEV), is_prefill=True, logits_at=torch.arange(41, device=DEV),
                collect=got_layers)[0]
    assert len(got_layers) == len(ref_layers) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(got_layers, ref_layers)):
        assert_rows_close((a.cpu().double() - b).abs().max(-1).values / b.abs().max(), dtype, 6e-2 if dtype == torch.bfloat16 else 2e-5, i)
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portions", [(1,) * 70, (70,), (2,) * 35, (3, 11, 1, 1, 37, 2, 2, 12, 1), (8, 2, 6, 1, 53), (69, 1)],
                         ids=["token_by_token", "whole", "twos", "mixed", "around_block_edges", "last_alone"])
def test_prompt_portions_and_decoding_agree_with_the_whole(dtype, portions):
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=9)
    tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(10)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 70)
    got = run_portions(model, tokens, portions)
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_token_kernels_equal_the_portion_kernels(dtype):
    """A decode step through the one-token product kernels against the same step through library products."""
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=15)
    tokens = torch.randint(0, cfg["vocab"], (50,), generator=torch.Generator().manual_seed(16)).tolist()
    outs = []
    for fused in (True, False):
        model = build_model(cfg, W, dtype, 50)
        model.fused_decode = fused
        outs.append(run_portions(model, tokens, (30,) + (1,) * 20))
    assert_rows_close(row_error(outs[0], outs[1]), dtype, BF16_TOL if dtype == torch.bfloat16 else 1e-5)
    assert model.kernels_per_token() > 0


def test_sequences_one_after_another_reuse_state_and_rows():
    """Three sequences of unequal length through one model, caches and state given back in between: each equals
    itself alone."""
    from cold_compress_b200.generation_utils import reset_caches
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=11)
    g = torch.Generator().manual_seed(12)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (45, 90, 13)]
    model = build_model(cfg, W, torch.float32, 90)
    for s, portions in zip(seqs, [(40, 1, 1, 1, 1, 1), (17, 60, 13), (13,)]):
        got = run_portions(model, s, portions)
        want = _reference_logits(cfg, W, s)
        assert row_error(got, want).max() < fp32_tolerance(cfg, W, s, want)
        reset_caches(model)
        for l in model.layers:
            assert all(float(s_.vectors.abs().sum()) == 0 and float(s_.matrix.abs().sum()) == 0 for s_ in l.states)
            assert l.kv_cache is None or int(l.kv_cache.cache_cts.item()) == 0


def test_long_decoding_across_blocks():
    """150 prompt tokens, then 330 tokens one by one: the block of the attention passes several times over decoded
    tokens (its ring wraps), and the recurrent states go through hundreds of single steps."""
    cfg = make_config([mamba_layer(dense(40), heads=2, vdim=8, state=12, groups=1, norm_groups=1),
                       parallel_layer(None, left=attention(heads=2, kv_heads=1, dim=8, vdim=8, size=50), right=delta(heads=2, kv_heads=1, dim=16, vdim=8)),
                       parallel_layer(dense(24), left=attention(heads=2, kv_heads=2, dim=8, vdim=4, size=140, conv=3), right=delta(heads=1, kv_heads=1, dim=8, vdim=8))],
                      width=48, vocab=71)
    W = random_weights(cfg, seed=13)
    tokens = torch.randint(0, 71, (480,), generator=torch.Generator().manual_seed(14)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, torch.float32, 480)
    got = run_portions(model, tokens, (150,) + (1,) * 330)
    assert row_error(got, want).max() < fp32_tolerance(cfg, W, tokens, want)


OTHER = [
    # every size that can be one is one (value heads keep one pair)
    ([mamba_layer(dense(1), heads=1, vdim=1, state=1, groups=1, norm_groups=1, conv=1),
      parallel_layer(None, left=attention(heads=1, kv_heads=1, dim=2, vdim=2, conv=1, size=1, dims=2), right=delta(heads=1, kv_heads=1, dim=1, vdim=1, conv=1))],
     dict(width=4, vocab=5, alpha=1.0, softcap=0), (1, 1)),
    # no block mask (everything is kept), 17 query heads on one key head, long convolutions, no soft cap
    ([parallel_layer(dense(48), left=attention(heads=17, kv_heads=1, dim=8, vdim=8, conv=6, size=0, dims=4), right=delta(heads=6, kv_heads=2, dim=8, vdim=12, conv=5)),
      mamba_layer(None, heads=6, vdim=10, state=7, groups=3, norm_groups=5, conv=2)], dict(width=72, vocab=90, softcap=0), (3, 2)),
    # wide state rows (more than 128 per head), value tiles beyond 32 columns, odd sizes everywhere
    ([mamba_layer(dense(30), heads=2, vdim=70, state=136, groups=1, norm_groups=7, conv=4),
      parallel_layer(None, left=attention(heads=5, kv_heads=5, dim=66, vdim=34, conv=3, size=21, dims=30, base=77.0), right=delta(heads=3, kv_heads=1, dim=130, vdim=35, conv=3))],
     dict(width=70, vocab=60, alpha=0.5), (11, 1)),
    # only one kind of layer each
    ([mamba_layer(dense(64)), mamba_layer(None)], dict(width=96, vocab=33), (4, 4)),
    ([parallel_layer(dense(64)), parallel_layer(dense(32))], dict(width=96, vocab=33), (4, 4)),
]


@pytest.mark.parametrize("layers,kw,ranks", OTHER, ids=["ones", "unmasked_many_heads", "wide_odd", "state_space_only", "parallel_only"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_other_sizes(layers, kw, ranks, dtype):
    cfg = make_config(layers, **kw)
    W = random_weights(cfg, seed=21, ranks=ranks)
    tokens = torch.randint(0, cfg["vocab"], (48,), generator=torch.Generator().manual_seed(22)).tolist()
    want = _reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 48)
    got = run_portions(model, tokens, (5, 2, 30, 1, 1, 6, 1, 1, 1))
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


def test_checkpoint_folder_generate_and_graphed_decoder(tmp_path):
    """From a checkpoint folder through load_model, setup_caches and generate(): greedy tokens equal the restatement's
    arg-max continuation, with the prompt whole or in portions, eager or graph-captured."""
    from pathlib import Path
    from cold_compress_b200.checkpoint import write_safetensors
    from cold_compress_b200.generation_utils import compile_funcs, generate, load_model, reset_caches, setup_caches
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=17)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    prompt = torch.randint(0, cfg["vocab"], (33,), generator=torch.Generator().manual_seed(18)).tolist()
    new = 20
    seq, margins = list(prompt), []
    for _ in range(new):
        lg = _reference_logits(cfg, W, seq)[-1]
        top = torch.topk(lg, 2).values
        margins.append((top[0] - top[1]).item())
        seq.append(int(lg.argmax()))
    model = load_model(Path(tmp_path), DEV, torch.float32, use_tp=False)
    assert type(model).__name__ == "TefovikTransformer"
    setup_caches(model, None, DEV, len(prompt) + new, {})
    for compile_, chunk in ((False, None), (False, 7), (True, 2)):
        prefill, decode = compile_funcs(compile_)
        out, _, stats = generate(model, torch.tensor(prompt, dtype=torch.int32, device=DEV), prefill, decode,
                                 max_new_tokens=new, prefill_chunk=chunk)
        out = out.tolist()
        assert out[:len(prompt)] == prompt and len(out) == len(seq)
        for i, (a, b) in enumerate(zip(out[len(prompt):], seq[len(prompt):])):
            assert a == b or margins[i] < 1e-3, (compile_, chunk, i)
            if a != b:
                break
        assert stats["decode_tokens"] == new
        reset_caches(model)


def test_trace_replay_command(tmp_path):
    """bin/trace_run as a user runs it: a checkpoint folder, steps on standard input (a whole prompt, portions with the
    last tokens alone, a second sequence after the first has ended), logits files and `done` lines."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from cold_compress_b200.checkpoint import write_safetensors
    root = Path(__file__).resolve().parent.parent
    cfg = make_config([mamba_layer(dense(40)), parallel_layer(None), parallel_layer(dense(40), left=attention(size=32)), mamba_layer(None, heads=2, vdim=12)],
                      width=72, vocab=211)
    W = random_weights(cfg, seed=31)
    model_dir = tmp_path / "ckpt"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(model_dir / "model.safetensors", W)
    g = torch.Generator().manual_seed(32)
    a = torch.randint(0, 211, (75,), generator=g).tolist()
    b = torch.randint(0, 211, (41,), generator=g).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:73], "want": [5, 40]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[73:74], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": a[74:75], "want": [0]}], "end": ["a"]},
             {"step": 5, "entries": [{"id": "b", "tokens": b, "want": [0, 20, 40]}], "end": ["b"]}]
    want = {0: [0, 29], 2: [37, 72], 3: [73], 4: [74]}
    la, lb = _reference_logits(cfg, W, a), _reference_logits(cfg, W, b)
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 2 * BF16_TOL)):
        out = tmp_path / ("out_" + dtype)
        r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "75"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(6)]
        assert not (out / "1.f32").exists()
        for step, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), -1).copy())
            assert row_error(got, la[rows]).max() < tol, (dtype, step)
        got = torch.from_numpy(np.fromfile(out / "5.f32", dtype="<f4").reshape(3, -1).copy())
        assert row_error(got, lb[[0, 20, 40]]).max() < tol
