"""CPU tests of the Tefovik design's host side: registry, configuration and shape errors, weight loading and fusing,
the cache plan, and the plain restatement's own invariants (the GPU tests hold the kernels to that restatement)."""
import json

import pytest
import torch

import tefovik_reference as R
from tefovik_utils import attention, default_layers, delta, dense, make_config, mamba_layer, parallel_layer, random_weights

F64 = torch.float64


def test_registry_builds_the_class_from_a_checkpoint_folder(tmp_path):
    from cold_compress_b200.checkpoint import load_checkpoint_folder, write_safetensors
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=1)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    model = load_checkpoint_folder(tmp_path, "cpu", torch.bfloat16)
    assert type(model).__name__ == "TefovikTransformer" and model.config.n_layer == 5 and model.supports_prompt_portions
    m = model.layers[0].mixer            # fused projection: left rows, right rows, zero padding
    l, r = m.left, m.right
    assert m.w_in.shape[0] % 16 == 0 and m.w_in.shape[0] >= l.in_rows + r.in_rows
    nq = l.heads * l.head_dim
    assert torch.equal(m.w_in[:nq], W["l0.mix.left.q"]) and torch.equal(m.w_in[l.conv_width:l.conv_width + l.heads], W["l0.mix.left.g"])
    off = l.in_rows + r.conv_width + r.heads
    assert torch.equal(m.w_in[off:off + r.decay_rank], W["l0.mix.right.a1"]) and r.decay_rank == 5 and r.gate_rank == 7
    assert float(m.w_in[l.in_rows + r.in_rows:].abs().sum()) == 0
    assert torch.equal(l.conv.weight[nq:nq + l.kv_heads * l.head_dim], W["l0.mix.left.k.conv"].float())
    assert model.layers[3].depth_coef.numel() == 5 and model.layers[1].mlp is None and model.layers[1].norm2 is None


def test_configuration_and_shape_errors():
    from cold_compress_b200.tefovik import TefovikArgs, TefovikTransformer
    cfg = make_config(default_layers())
    bad = json.loads(json.dumps(cfg))
    bad["layers"][1]["type"] = "conv"
    with pytest.raises(ValueError, match="unknown mixer type"):
        TefovikArgs.from_config(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError, match="feed-forward"):
        TefovikArgs.from_config(bad)
    with pytest.raises(ValueError, match="kv heads"):
        TefovikTransformer.from_config(make_config([parallel_layer(None, left=attention(heads=5, kv_heads=2))]))
    with pytest.raises(ValueError, match="groups"):
        TefovikTransformer.from_config(make_config([mamba_layer(None, heads=3, groups=2)]))
    model = TefovikTransformer.from_config(cfg, torch.float32)
    W = random_weights(cfg, seed=2)
    short = dict(W)
    del short["l2.ls1"]
    with pytest.raises(KeyError, match="l2.ls1"):
        model.load_tensors(short)
    wrong = dict(W)
    wrong["l1.mix.conv"] = wrong["l1.mix.conv"][:, :2]
    with pytest.raises(ValueError, match="l1.mix.conv"):
        model.load_tensors(wrong)
    extra = dict(W)
    extra["l9.unused"] = torch.zeros(1)
    assert model.load_tensors(extra) == ["l9.unused"]


def test_cache_plan_and_state_shapes():
    from cold_compress_b200.generation_utils import reset_caches, setup_caches
    from cold_compress_b200.tefovik import TefovikTransformer
    layers = [parallel_layer(dense(), left=attention(size=9)), mamba_layer(), parallel_layer(None, left=attention(size=0))]
    model = TefovikTransformer.from_config(make_config(layers), torch.float32)
    ck = setup_caches(model, None, "cpu", 77, {})
    assert ck["cache_strategy"] == ["recent_global", "state", "full"] and ck["max_cache_length"] == [9, 0, 77]
    a, b, c = model.layers
    assert a.kv_cache.sequence_window() == 9 and c.kv_cache.sequence_window() == 0 and b.kv_cache is None
    assert a.kv_cache.k_cache.shape == (1, 2, 9, 16) and a.kv_cache.v_cache.shape == (1, 2, 9, 20)
    left, right = a.states
    assert left.vectors.shape == (1, (6 + 2) * 16 + 2 * 20) and left.matrix.numel() == 0
    assert right.vectors.shape == (3, 2 * 2 * 24 + 4 * 10) and right.matrix.shape == (4, 24, 10)
    assert b.states[0].vectors.shape == (2, 4 * 12 + 2 * 2 * 20) and b.states[0].matrix.shape == (4, 20, 12)
    assert model.min_cache_length() == 77 and model.prompt_cache_overflow(100) == [False, False, True]
    right.matrix.fill_(1.0)
    a.kv_cache.pos.fill_(3)
    reset_caches(model)
    assert float(right.matrix.sum()) == 0 and int(a.kv_cache.pos.max()) == -1
    assert model.get_cache_stats(10, 5)["cache_slots_0"] == 9.0 and model.kernels_per_token() > 0


def test_model_refuses_cpu_tensors():
    from cold_compress_b200._lib import CcError
    from cold_compress_b200.generation_utils import setup_caches
    from cold_compress_b200.tefovik import TefovikTransformer
    model = TefovikTransformer.from_config(make_config([mamba_layer()]), torch.float32)
    with pytest.raises(RuntimeError, match="Caches"):
        model(torch.zeros(1, 3, dtype=torch.int32), torch.arange(3))
    setup_caches(model, None, "cpu", 8, {})
    with pytest.raises(CcError, match="CUDA"):
        model(torch.zeros(1, 3, dtype=torch.int32), torch.arange(3))


# ----------------------------------------------------------------------------------------------- the restatement's own invariants

def test_restatement_is_causal_and_blocks_cut_the_attention():
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    b = list(a)
    b[30] = (b[30] + 1) % cfg["vocab"]
    la, lb = R.forward(cfg, W, a), R.forward(cfg, W, b)
    assert torch.equal(la[:30], lb[:30]) and (la[30:] - lb[30:]).abs().max() > 1e-6
    pos = torch.arange(20)
    m = R.chunk_mask(pos, pos, 8)
    assert m[7, 0] and not m[8, 7] and m[8, 8] and m[15, 8] and not m[16, 15] and not m[3, 4]
    assert R.chunk_mask(pos, pos, 0)[19, 0]


def test_restatement_scans_equal_their_unrolled_sums_and_hand_over_state():
    g = torch.Generator().manual_seed(5)
    T, H, G, N, V = 9, 2, 1, 3, 4
    x, B, C = torch.randn(T, H, V, generator=g, dtype=F64), torch.randn(T, G, N, generator=g, dtype=F64), torch.randn(T, G, N, generator=g, dtype=F64)
    dt, a = torch.rand(T, H, generator=g, dtype=F64), torch.rand(T, H, generator=g, dtype=F64)
    D = torch.randn(H, generator=g, dtype=F64)
    y, S = R.state_space_scan(x, B, C, dt, a, D)
    for h in range(H):     # y_t = sum_{s <= t} (prod_{s < r <= t} a_r) dt_s (C_t . B_s) x_s + D x_t
        for t in range(T):
            acc = D[h] * x[t, h]
            for s in range(t + 1):
                acc = acc + a[s + 1:t + 1, h].prod() * dt[s, h] * (C[t, 0] @ B[s, 0]) * x[s, h]
            assert (acc - y[t, h]).abs().max() < 1e-12
    y1, S1 = R.state_space_scan(x[:5], B[:5], C[:5], dt[:5], a[:5], D)
    y2, S2 = R.state_space_scan(x[5:], B[5:], C[5:], dt[5:], a[5:], D, S1)
    assert torch.allclose(torch.cat([y1, y2]), y, atol=1e-13) and torch.allclose(S2, S, atol=1e-13)
    # delta rule: with beta = 1 and unit decay, a key read back right after its write returns its value
    Dk = 6
    q, k, v = torch.randn(T, 1, Dk, generator=g, dtype=F64), torch.randn(T, 1, Dk, generator=g, dtype=F64), torch.randn(T, H, V, generator=g, dtype=F64)
    k = R.unit_vectors(k, 0.0)
    o, _ = R.delta_rule_scan(k, k, v, torch.ones(T, H, dtype=F64), torch.ones(T, H, Dk, dtype=F64))
    assert (o - v).abs().max() < 1e-12
    beta, decay = torch.rand(T, H, generator=g, dtype=F64), torch.rand(T, H, Dk, generator=g, dtype=F64)
    o, S = R.delta_rule_scan(q, k, v, beta, decay)
    o1, S1 = R.delta_rule_scan(q[:4], k[:4], v[:4], beta[:4], decay[:4])
    o2, S2 = R.delta_rule_scan(q[4:], k[4:], v[4:], beta[4:], decay[4:], S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-13) and torch.allclose(S2, S, atol=1e-13)


def test_restatement_convolution_and_rotation():
    g = torch.Generator().manual_seed(6)
    u, w = torch.randn(11, 5, generator=g, dtype=F64), torch.randn(5, 4, generator=g, dtype=F64)
    y, last = R.short_conv(u, w)
    assert torch.allclose(y[0], u[0] * w[:, 3]) and torch.allclose(y[3], (u[0:4] * w.T).sum(0)) and torch.equal(last, u[8:])
    y1, t1 = R.short_conv(u[:2], w)
    y2, t2 = R.short_conv(u[2:], w, before=t1)
    assert torch.allclose(torch.cat([y1, y2]), y) and torch.equal(t2, last)
    x = torch.randn(7, 3, 10, generator=g, dtype=F64)
    pos = torch.arange(100, 107)
    for inter in (True, False):
        r = R.rotate_pairs(x, pos, 50.0, 6, inter)
        assert torch.equal(r[..., 6:], x[..., 6:]) and torch.allclose(r.norm(dim=-1), x.norm(dim=-1))
        assert torch.allclose(R.rotate_pairs(r, pos, 50.0, 6, inter, sign=-1.0), x)
    # rotated values: what a query at i reads of the value at j depends on i - j only
    v = torch.randn(1, 1, 8, generator=g, dtype=F64)
    a = R.rotate_pairs(R.rotate_pairs(v, torch.tensor([5]), 50.0, 8), torch.tensor([9]), 50.0, 8, sign=-1.0)
    b = R.rotate_pairs(R.rotate_pairs(v, torch.tensor([105]), 50.0, 8), torch.tensor([109]), 50.0, 8, sign=-1.0)
    assert torch.allclose(a, b)
