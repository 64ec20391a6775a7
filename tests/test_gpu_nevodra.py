"""GPU tests of the Nevodra design: every mechanism's kernel against the plain restatement in nevodra_reference.py
(float64, CPU, whole sequences), then the model through the runtime: layer by layer, prompt against token-by-token
decoding, prompt portions down to two tokens, cache rows and tails that are given back and used again, one key just
inside or just outside the window, among the kept first positions and far back, long decoding, other sizes, greedy
generation through generate() and the graph-captured decoder, and the trace replay command."""
import json

import pytest
import torch

import nevodra_reference as R
from nevodra_utils import (DEFAULT_LOOP, assert_rows_close, build_model, default_layers, dense, fp32_tolerance, latent_layer,
                           make_config, moe, random_weights, reference_logits, row_error, run_portions, window_layer)

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16_TOL = 6e-2
F64 = torch.float64


def _ops():
    from cold_compress_b200 import seq_ops
    return seq_ops


def _i32(*v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _tol(dtype, cfg, W, tokens, want):
    return BF16_TOL if dtype == torch.bfloat16 else fp32_tolerance(cfg, W, tokens, want)


def _close(got, want, rel):
    want = want.double()
    err = (got.detach().cpu().double() - want).abs().max().item()
    assert err <= rel * max(want.abs().max().item(), 1e-30), (err, want.abs().max().item())


# ----------------------------------------------------------------------------------------------- single mechanisms

@pytest.mark.parametrize("E,taps,n", [(1, 1, 1), (50, 2, 2), (640, 4, 2), (96, 7, 3)])
def test_sum_norms_and_input_convolution_carry_their_tail_across_portions(E, taps, n):
    ops = _ops()
    g = torch.Generator().manual_seed(E + taps)
    T, eps = 23, 1e-5
    x0 = torch.randn(T, E, generator=g) * 3 + 0.5
    wide = torch.randn(T, 2 * E + 3, generator=g)           # sublayer results as column ranges of wider rows
    add = torch.randn(E, generator=g)
    gains = [torch.randn(E, generator=g) for _ in range(n)]
    convs = [torch.randn(E, taps, generator=g) * 0.5 for _ in range(n)]
    xs = x0.double() + wide[:, 1:1 + E].double() + wide[:, 2 + E:2 + 2 * E].double() + add.double()
    want = [R.input_conv(R.rms_norm(xs, gains[s].double(), eps), convs[s].double()) for s in range(n)]
    for portions in ((T,), (1,) * T, (2, 5, 1, 1, 9, 2, 3), (taps + 1, T - taps - 1)):
        tail = torch.zeros(max(taps - 1, 1), E, device=DEV)
        at = 0
        for m in portions:
            x = x0[at:at + m].to(DEV).contiguous()
            wd = wide[at:at + m].to(DEV).contiguous()
            outs = [torch.empty(m, E, device=DEV) for _ in range(n)]
            spread = m == 1 and at % 2 == 1                 # one token: also the launch that spreads the row over the GPU
            x_out = torch.empty_like(x) if spread else None
            ops.par_norm(x, [(gains[s].to(DEV), convs[s].to(DEV), outs[s]) for s in range(n)], eps, a=wd[:, 1:1 + E],
                         b=wd[:, 2 + E:2 + 2 * E], add=add.to(DEV), tail=tail if taps > 1 else None, taps=taps,
                         rinv=torch.empty(m, device=DEV) if m > 1 else None, x_out=x_out)
            if spread:
                assert torch.equal(x.cpu(), x0[at:at + m])  # the input row is left as it was
                x = x_out
            _close(x, xs[at:at + m], 1e-6)                  # the stream after the sum
            for s in range(n):
                _close(outs[s], want[s][at:at + m], 3e-5)
            at += m
        if taps > 1:                                         # what the next step would read: the last unit-RMS rows
            _close(tail, R.unit_rms(xs, eps)[T - (taps - 1):] if T >= taps - 1 else tail.cpu(), 1e-5)


def test_norms_without_a_convolution_table_or_a_pending_sum():
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    x0, gain = torch.randn(5, 70, generator=g), torch.randn(70, generator=g)
    x, out = x0.to(DEV), torch.empty(5, 70, device=DEV, dtype=torch.bfloat16)
    ops.par_norm(x, [(gain.to(DEV), None, out)], 1e-6, taps=1, rinv=torch.empty(5, device=DEV))
    assert torch.equal(x.cpu(), x0)
    _close(out.float(), R.rms_norm(x0.double(), gain.double(), 1e-6), 1e-2)


@pytest.mark.parametrize("nq,nk,nv", [(1, 1, 1), (96, 32, 24), (300, 150, 75)])
def test_whole_row_query_and_key_norm_kernel(nq, nk, nv):
    ops = _ops()
    g = torch.Generator().manual_seed(nq)
    T = 7
    src = torch.randn(T, nq + nk + nv + 5, generator=g) * 2
    wq, wk = torch.randn(nq, generator=g), torch.randn(nk, generator=g)
    q, k, v = torch.empty(T, nq, device=DEV), torch.empty(T, nk, device=DEV), torch.empty(T, nv, device=DEV)
    ops.qk_row_norm(src.to(DEV), 0, nq, nq, nk, nq + nk, nv, wq.to(DEV), wk.to(DEV), q, k, v, 1e-5)
    d = src.double()
    _close(q, R.rms_norm(d[:, :nq], wq.double(), 1e-5), 1e-5)
    _close(k, R.rms_norm(d[:, nq:nq + nk], wk.double(), 1e-5), 1e-5)
    assert torch.equal(v.cpu(), src[:, nq + nk:nq + nk + nv])


@pytest.mark.parametrize("F", [1, 40, 1000])
def test_polynomial_activation_kernel(F):
    ops = _ops()
    g = torch.Generator().manual_seed(F)
    T = 6
    src = torch.randn(T, F + 3, generator=g) * 1.7
    coef = torch.tensor([0.8, -0.5, 0.3, 0.2])
    out = torch.empty(T, F, device=DEV)
    ops.poly_norm(src.to(DEV)[:, 2:2 + F], coef.to(DEV), out, 1e-5)
    _close(out, R.poly_norm(src[:, 2:2 + F].double(), coef.double(), 1e-5), 1e-5)


ROUTERS = [dict(experts=8, top=2, count=2, keep=1), dict(experts=6, top=3, count=3, keep=2), dict(experts=12, top=4, count=1, keep=1),
           dict(experts=9, top=2, count=9, keep=3), dict(experts=40, top=6, count=5, keep=2), dict(experts=4, top=1, count=2, keep=2)]


@pytest.mark.parametrize("r", ROUTERS, ids=lambda r: "-".join(str(v) for v in r.values()))
@pytest.mark.parametrize("negative", [False, True])
def test_router_follows_the_rules(r, negative):
    """Sigmoid scores, the correction for the choice only, groups ranked by the sum of their two best choices, losers
    at minus infinity (choice scores can all be negative), weights = scores times the scale, not renormalised."""
    ops = _ops()
    g = torch.Generator().manual_seed(r["experts"] + r["top"])
    n, T = r["experts"], 64
    z = torch.randn(T, n + 2, generator=g) * 2
    corr = torch.randn(n, generator=g) * 0.4 - (3.0 if negative else 0.0)
    ids = torch.empty(T, r["top"], dtype=torch.int32, device=DEV)
    wts = torch.empty(T, r["top"], device=DEV)
    ops.moe_route(z.to(DEV)[:, 1:1 + n], corr.to(DEV), ids, wts, r["count"], r["keep"], r["top"], sigmoid_scores=True,
                  group_top=2, renormalize=False, weight_scale=1.7)
    rr = {"top": r["top"], "scale": 1.7, "groups": {"count": r["count"], "keep": r["keep"]}}
    for t in range(T):
        wi, ww = R.route(z[t, 1:1 + n].float().double(), corr.double(), rr)
        assert sorted(ids[t].tolist()) == sorted(wi.tolist()), t
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        for e, w in zip(wi.tolist(), ww.tolist()):
            assert abs(got[e] - w) < 1e-5


# ----------------------------------------------------------------------------------------------- windowed attention

def _ring(G, Dk, Dv, window, keep, dtype):
    from cold_compress_b200.cache import get_cache_constructor
    ctor, _ = get_cache_constructor("recent_global" if window else "full")
    return ctor(1, G, Dk, dtype, max_cache_length=(window + keep) if window else 400, max_seq_length=400, global_tokens=keep,
                cache_bits=None, v_head_dim=Dv).to(DEV)


def _attend(cache, q, k, v, portions, window, scale, dtype, softcap, dist):
    got, at = [], 0
    dd = None if dist is None else (dist[0].to(DEV), dist[1].to(DEV))
    for n in portions:
        y = torch.empty(n, q.shape[1], v.shape[2], device=DEV)
        cache.sequence_step(q[at:at + n].to(DEV).contiguous(), k[at:at + n].to(DEV, dtype).contiguous(), v[at:at + n].to(DEV, dtype).contiguous(),
                            _i32(at), y, scale=scale, window=window, softcap=softcap, dist=dd)
        got.append(y)
        at += n
    return torch.cat(got).cpu().double()


def _window_reference(q, k, v, scale, window, keep, softcap, dist):
    """Dense restatement of the scores' path (cap, distance penalty, window with kept first positions)."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    ok = R.window_mask(T, window, keep) if window else R.window_mask(T, T, 0)
    dpos = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).double()
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if dist is not None:
            s = s - dist[0][h].double() * torch.log(1 + dist[1][h].double() * dpos)
        out[:, h] = torch.softmax(s.masked_fill(~ok, float("-inf")), -1) @ v[:, h // (H // G)]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,Dk,Dv,window,keep", [(6, 2, 16, 20, 9, 4), (4, 4, 12, 8, 16, 0), (10, 1, 56, 40, 70, 33), (3, 1, 5, 3, 1, 1),
                                                 (17, 1, 8, 8, 33, 2), (2, 2, 24, 24, 0, 0), (4, 2, 8, 8, 140, 130)])
def test_windowed_attention_in_portions_and_single_tokens(dtype, H, G, Dk, Dv, window, keep):
    g = torch.Generator().manual_seed(window + keep)
    T = 150
    q, k, v = torch.randn(T, H, Dk, generator=g), torch.randn(T, G, Dk, generator=g), torch.randn(T, G, Dv, generator=g)
    if dtype == torch.bfloat16:
        k, v = k.bfloat16().float(), v.bfloat16().float()
    dist = (torch.rand(H, generator=g) + 0.2, torch.rand(H, generator=g) * 2)
    want = _window_reference(q.double(), k.double(), v.double(), 0.3, window, keep, 5.0, dist)
    for portions in ((T,), (7, 2, 64, 33, 2, 40, 1, 1), (100,) + (1,) * 50, (1,) * T):
        cache = _ring(G, Dk, Dv, window, keep, dtype)
        got = _attend(cache, q, k, v, portions, window, 0.3, dtype, 5.0, dist)
        assert (got - want).abs().max() < 2e-5 * max(1.0, want.abs().max()), (portions[:3], (got - want).abs().max())


@pytest.mark.parametrize("mode", ["prompt", "portions", "decode"])
@pytest.mark.parametrize("where", ["oldest_in_window", "just_outside_window", "last_kept", "first_not_kept", "own_position", "position_0"])
def test_one_key_at_the_edges_of_window_and_kept_positions_decides(mode, where):
    """One key's score stands far above the rest (beyond what the cap and the distance penalty can undo).  Inside the
    window or among the kept first positions it takes the whole softmax; one position outside it must not be seen."""
    window, keep, T, Dk, Dv = 44, 7, 44 * 5 + 20, 16, 8
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(T, 2, Dk, generator=g) * 0.1, torch.randn(T, 1, Dk, generator=g) * 0.1, torch.randn(T, 1, Dv, generator=g)
    last = T - 1
    j = {"oldest_in_window": last - window + 1, "just_outside_window": last - window, "last_kept": keep - 1, "first_not_kept": keep,
         "own_position": last, "position_0": 0}[where]
    k[j, 0] = 0.0
    k[j, 0, 3] = 30.0
    q[last, :, 3] = 30.0          # score 900 x scale against |others| < 1; the cap leaves it at 60
    v[j] = 100.0
    dist = (torch.full((2,), 0.5), torch.full((2,), 1.0))
    want = _window_reference(q.double(), k.double(), v.double(), 0.25, window, keep, 60.0, dist)
    if where in ("just_outside_window", "first_not_kept"):
        assert want[last].abs().max() < 10
    else:
        assert (want[last] - 100.0).abs().max() < 1e-6
    cut = last - window
    portions = {"prompt": (T,), "portions": (keep - 1, 2, cut - keep, 2, T - cut - 3), "decode": (cut - 3,) + (1,) * (T - cut + 3)}[mode]
    got = _attend(_ring(1, Dk, Dv, window, keep, torch.float32), q, k, v, portions, window, 0.25, torch.float32, 60.0, dist)
    assert (got - want).abs().max() < 1e-4


def test_ring_and_kept_rows_given_back_are_not_keys():
    """A second sequence after a longer one through the same cache: rows the first left behind must not be attended."""
    window, keep, Dk, Dv = 20, 5, 8, 6
    g = torch.Generator().manual_seed(4)
    cache = _ring(2, Dk, Dv, window, keep, torch.float32)
    a = [torch.randn(57, h, d, generator=g) * 3 for h, d in ((4, Dk), (2, Dk), (2, Dv))]
    _attend(cache, *a, (57,), window, 0.5, torch.float32, 0.0, None)
    assert int(cache.cache_cts.item()) == window + keep
    cache.reset()
    b = [torch.randn(31, h, d, generator=g) for h, d in ((4, Dk), (2, Dk), (2, Dv))]
    want = _window_reference(*[t.double() for t in b], 0.5, window, keep, 0.0, None)
    got = _attend(cache, *b, (3, 1, 1, 19, 7), window, 0.5, torch.float32, 0.0, None)
    assert (got - want).abs().max() < 2e-5
    assert int(cache.cache_cts.item()) == window + keep
    assert sorted(cache.pos[0, 0].tolist()) == list(range(keep)) + list(range(31 - window, 31))


# ----------------------------------------------------------------------------------------------- latent attention

def _latent_setup(T, seed, heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, dims=None, width=48):
    layer = latent_layer(None, heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, dims=dims)
    cfg = make_config([layer], width=width, vocab=11, taps=1)
    W = {k: v.float() for k, v in random_weights(cfg, seed=seed).items()}
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(seed + 1))
    return layer["mixer"], cfg, W, h


def _latent_run(m, cfg, W, h, portions, dtype=torch.float32):
    from cold_compress_b200.cache import get_cache_constructor
    from cold_compress_b200.nevodra import NevodraBlock, NevodraArgs
    block = NevodraBlock(NevodraArgs.from_config(cfg), cfg["layers"][0], dtype)
    mix = block.mixer
    H, D, Rr, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rows = torch.cat([W["l0.mix.q"], W["l0.mix.dkv"]])
    mix.w_in.data[:rows.shape[0]] = rows.to(dtype)
    mix.kv_norm.data.copy_(W["l0.mix.dkv.norm"])
    mix.sink.data.copy_(W["l0.mix.sink"])
    mix.w_ukv.data.copy_(torch.cat([W["l0.mix.uk"], W["l0.mix.uv"]]).to(dtype))
    mix.w_uk_t.data.copy_(W["l0.mix.uk"].reshape(H, D, C).transpose(1, 2).to(dtype))
    mix.w_o.data.copy_(W["l0.mix.o"].to(dtype))
    mix = mix.to(DEV)
    ctor, _ = get_cache_constructor("latent")
    cache = ctor(1, 1, mix.row_width, dtype, max_cache_length=h.shape[0], max_seq_length=h.shape[0], global_tokens=0, cache_bits=None).to(DEV)
    out, at = [], 0
    for n in portions:
        out.append(mix(h[at:at + n].to(DEV, dtype).contiguous(), _i32(at), cache))
        at += n
    return torch.cat(out).cpu().double()


@pytest.mark.parametrize("kw", [dict(), dict(dims=4), dict(heads=17, dim=8, rot_dim=2, vdim=8, kv_rank=40), dict(heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1)],
                         ids=["default", "partly_rotated", "many_heads", "ones"])
def test_latent_attention_with_sink_and_interleaved_pairs(kw):
    T = 90
    m, cfg, W, h = _latent_setup(T, 5, **kw)
    want = R.latent_attention(h.double(), {k: v.double() for k, v in W.items()}, "l0.mix.", m, 1e-5)
    for portions in ((T,), (40, 2, 1, 1, 46), (1,) * T):
        got = _latent_run(m, cfg, W, h, portions)
        assert (got - want).abs().max() < 3e-5 * max(1.0, want.abs().max()), portions[:2]


@pytest.mark.parametrize("mode", ["prompt", "portions", "decode"])
def test_sink_takes_its_share_and_a_far_key_is_found(mode):
    """With a large sink logit the heads' outputs shrink by the sink's share; a key 600 positions back that the last
    query likes best (the scores are sharpened by the scale) still decides the output."""
    T = 640
    m, cfg, W, h = _latent_setup(T, 7)
    m = dict(m, scale=m["scale"] * 12)
    cfg["layers"][0]["mixer"] = m
    Wd = {k: v.double() for k, v in W.items()}
    base = R.latent_attention(h.double(), Wd, "l0.mix.", m, 1e-5)
    Wd2 = dict(Wd)
    Wd2["l0.mix.sink"] = Wd["l0.mix.sink"] + 6.0
    sunk = R.latent_attention(h.double(), Wd2, "l0.mix.", m, 1e-5)
    assert sunk.abs().sum() < base.abs().sum() and (sunk - base).abs().max() > 1e-3      # every head's output shrinks
    W2 = {k: v.float() for k, v in Wd2.items()}
    portions = {"prompt": (T,), "portions": (33, 2, 500, 105), "decode": (600,) + (1,) * 40}[mode]
    for weights, want in ((W, base), (W2, sunk)):
        got = _latent_run(m, cfg, weights, h, portions)
        assert (got - want).abs().max() < 5e-5 * max(1.0, want.abs().max())
    # the far key: among a few candidate inputs for position 39, the one that moves the last position's output most
    best, h2, want = 0.0, None, None
    for c in range(8):
        cand = h.clone()
        cand[39] = h[100 + c] * 4
        w = R.latent_attention(cand.double(), Wd, "l0.mix.", m, 1e-5)
        change = (w[-1] - base[-1]).abs().max().item()
        if change > best:
            best, h2, want = change, cand, w
    assert best > 1e-2
    got = _latent_run(m, cfg, W, h2, portions)
    assert (got[-1] - want[-1]).abs().max() < 5e-5 * max(1.0, want.abs().max())


# ----------------------------------------------------------------------------------------------- the model in the runtime

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_one_by_one_and_logits(dtype):
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=5, decisive=dtype == torch.bfloat16)
    tokens = torch.randint(0, cfg["vocab"], (41,), generator=torch.Generator().manual_seed(6)).tolist()
    ref_layers = []
    want = reference_logits(cfg, W, tokens, ref_layers)
    model = build_model(cfg, W, dtype, 41)
    got_layers = []
    x = torch.tensor(tokens, dtype=torch.int32, device=DEV).view(1, -1)
    got = model(x, torch.arange(41, dtype=torch.int32, device=DEV), is_prefill=True, logits_at=torch.arange(41, device=DEV),
                collect=got_layers)[0]
    assert len(got_layers) == len(ref_layers) == 9 == model.config.n_layer
    for i, (a, b) in enumerate(zip(got_layers, ref_layers)):
        assert_rows_close((a.cpu().double() - b).abs().max(-1).values / b.abs().max(), dtype, 6e-2 if dtype == torch.bfloat16 else 2e-5, i)
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portions", [(1,) * 70, (70,), (2,) * 35, (3, 11, 1, 1, 37, 2, 2, 12, 1), (8, 2, 3, 1, 56), (69, 1)],
                         ids=["token_by_token", "whole", "twos", "mixed", "around_window_edges", "last_alone"])
def test_prompt_portions_and_decoding_agree_with_the_whole(dtype, portions):
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=9, decisive=dtype == torch.bfloat16)
    tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(10)).tolist()
    want = reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 70)
    got = run_portions(model, tokens, portions)
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_token_kernels_equal_the_portion_kernels(dtype):
    """A decode step through the one-token product kernels against the same step through library products."""
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=15, decisive=dtype == torch.bfloat16)
    tokens = torch.randint(0, cfg["vocab"], (50,), generator=torch.Generator().manual_seed(16)).tolist()
    outs = []
    for fused in (True, False):
        model = build_model(cfg, W, dtype, 50)
        model.fused_decode = fused
        outs.append(run_portions(model, tokens, (30,) + (1,) * 20))
    assert_rows_close(row_error(outs[0], outs[1]), dtype, BF16_TOL if dtype == torch.bfloat16 else 1e-5)
    assert model.kernels_per_token() > 0


def test_sequences_one_after_another_reuse_tails_and_rows():
    """Three sequences of unequal length through one model, caches and tails given back in between: each equals
    itself alone."""
    from cold_compress_b200.generation_utils import reset_caches
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=11)
    g = torch.Generator().manual_seed(12)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (45, 90, 13)]
    model = build_model(cfg, W, torch.float32, 90)
    for s, portions in zip(seqs, [(40, 1, 1, 1, 1, 1), (17, 60, 13), (13,)]):
        got = run_portions(model, s, portions)
        want = reference_logits(cfg, W, s)
        assert row_error(got, want).max() < fp32_tolerance(cfg, W, s, want)
        reset_caches(model)
        for l in model.layers:
            assert float(l.state.vectors.abs().sum()) == 0 and int(l.kv_cache.cache_cts.item()) == 0


def test_long_decoding_across_windows():
    """150 prompt tokens, then 330 tokens one by one: the windows pass several times over decoded tokens (the rings wrap)
    while the kept first positions stay, and the latent rows grow past several key runs."""
    cfg = make_config([window_layer(dense(40), heads=2, kv_heads=1, dim=8, vdim=8, size=50, keep_first=6),
                       latent_layer(moe(experts=4, top=2, count=2, keep=1, ff=16, shared=24), heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16),
                       window_layer(None, heads=2, kv_heads=2, dim=8, vdim=4, size=140, keep_first=1)],
                      width=48, vocab=71, taps=3, loop=(0, 2, 2))
    W = random_weights(cfg, seed=13)
    tokens = torch.randint(0, 71, (480,), generator=torch.Generator().manual_seed(14)).tolist()
    want = reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, torch.float32, 480)
    got = run_portions(model, tokens, (150,) + (1,) * 330)
    assert row_error(got, want).max() < fp32_tolerance(cfg, W, tokens, want)


OTHER = [
    # every size that can be one is one (the rotated part keeps one pair); one tap, no loop
    ([window_layer(dense(1), heads=1, kv_heads=1, dim=1, vdim=1, size=1, keep_first=1),
      latent_layer(moe(experts=1, top=1, count=1, keep=1, ff=1, shared=1), heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1)],
     dict(width=4, vocab=5, taps=1, embed_scale=1.0)),
    # 17 query heads on one key head, no window (everything is kept), long convolutions, no cap, a loop over the last layers
    ([latent_layer(dense(48), heads=17, dim=6, rot_dim=2, vdim=6, kv_rank=40),
      window_layer(moe(experts=10, top=4, count=5, keep=3, shared=0), heads=17, kv_heads=1, dim=8, vdim=8, size=0, keep_first=0, softcap=0.0),
      window_layer(None, heads=5, kv_heads=5, dim=6, vdim=10, size=7, keep_first=9)], dict(width=72, vocab=90, taps=6, loop=(1, 3, 2))),
    # wide and odd sizes: heads beyond 64 columns, value rows of another width, a window larger than the sequence
    ([window_layer(dense(30), heads=3, kv_heads=1, dim=66, vdim=34, size=100, keep_first=2),
      latent_layer(moe(experts=9, top=2, count=3, keep=1, ff=10, shared=14), heads=5, dim=70, rot_dim=10, vdim=35, kv_rank=130, dims=6, base=77.0)],
     dict(width=70, vocab=60, taps=2, loop=(0, 2, 3))),
    # only one kind of layer each
    ([window_layer(dense(64)), window_layer(moe())], dict(width=96, vocab=33)),
    ([latent_layer(dense(64)), latent_layer(moe())], dict(width=96, vocab=33, loop=(0, 1, 4))),
]


@pytest.mark.parametrize("layers,kw", OTHER, ids=["ones", "unwindowed_many_heads", "wide_odd", "windowed_only", "latent_only"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_other_sizes(layers, kw, dtype):
    cfg = make_config(layers, **kw)
    W = random_weights(cfg, seed=21, decisive=dtype == torch.bfloat16)
    tokens = torch.randint(0, cfg["vocab"], (48,), generator=torch.Generator().manual_seed(22)).tolist()
    want = reference_logits(cfg, W, tokens)
    model = build_model(cfg, W, dtype, 48)
    got = run_portions(model, tokens, (5, 2, 30, 1, 1, 6, 1, 1, 1))
    assert_rows_close(row_error(got, want), dtype, _tol(dtype, cfg, W, tokens, want))


def test_checkpoint_folder_generate_and_graphed_decoder(tmp_path):
    """From a checkpoint folder through load_model, setup_caches and generate(): greedy tokens equal the restatement's
    arg-max continuation, with the prompt whole or in portions, eager or graph-captured."""
    from pathlib import Path
    from cold_compress_b200.checkpoint import write_safetensors
    from cold_compress_b200.generation_utils import compile_funcs, generate, load_model, reset_caches, setup_caches
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=17)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    prompt = torch.randint(0, cfg["vocab"], (33,), generator=torch.Generator().manual_seed(18)).tolist()
    new = 20
    seq, margins = list(prompt), []
    for _ in range(new):
        lg = reference_logits(cfg, W, seq)[-1]
        top = torch.topk(lg, 2).values
        margins.append((top[0] - top[1]).item())
        seq.append(int(lg.argmax()))
    model = load_model(Path(tmp_path), DEV, torch.float32, use_tp=False)
    assert type(model).__name__ == "NevodraTransformer"
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
    cfg = make_config([latent_layer(dense(40)), window_layer(moe(), size=32, keep_first=5), window_layer(None), latent_layer(moe(shared=0))],
                      width=72, vocab=211, loop=(1, 3, 2))
    W = random_weights(cfg, seed=31, decisive=True)
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
    la, lb = reference_logits(cfg, W, a), reference_logits(cfg, W, b)
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
