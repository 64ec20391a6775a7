"""CPU tests of the Detatar design: registry and configuration, checkpoint loading, the cache plan, and invariants of
the plain restatement the GPU tests compare against."""
import json

import pytest
import torch

import detatar_reference as R
from detatar_utils import default_layers, dense, latent_layer, make_config, moe, random_weights, wkv_layer


def test_registry_builds_the_class_from_config(tmp_path):
    from cold_compress_b200.checkpoint import MODEL_REGISTRY, load_checkpoint_folder, write_safetensors
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=1)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    model = load_checkpoint_folder(tmp_path, "cpu", torch.float32)
    assert type(model).__name__ == "DetatarTransformer" and "Detatar" in MODEL_REGISTRY
    assert len(model.layers) == len(cfg["layers"])
    assert model.layers[5].block is model.layers[1].block and model.layers[6].block is model.layers[0].block
    # shared weights are registered once; the decay rank comes from the tensor's shape
    names = [n for n, _ in model.named_parameters()]
    assert len(names) == len(set(names)) and not any(n.startswith("layers.5.") or n.startswith("layers.6.") for n in names)
    assert model.layers[0].block.mixer.w_w1.shape == (6, cfg["width"])
    b = model.layers[1].block
    assert torch.equal(b.mixer.w_uk_t[1], W["l1.mix.uk"].float().reshape(3, 16, 40)[1].T)
    assert b.w_h.shape[0] == 288 and float(b.w_h[2 * 96 + 8 + 1 + 2 * 40:].abs().sum()) == 0     # 281 rows, padded to 16


def test_configuration_errors():
    from cold_compress_b200.detatar import DetatarArgs, DetatarTransformer
    with pytest.raises(ValueError, match="mixer type"):
        DetatarArgs.from_config(make_config([{"type": "conv", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError, match="feed-forward"):
        DetatarArgs.from_config(make_config([wkv_layer({"kind": "sparse"})]))
    with pytest.raises(ValueError, match="weights_of"):
        DetatarArgs.from_config(make_config([wkv_layer(None), latent_layer(None, weights_of=0)]))
    with pytest.raises(ValueError, match="groups"):
        DetatarArgs.from_config(make_config([wkv_layer(None)], width=50, groups=4))
    # a layer may name a layer that itself borrows its weights: all three run the first one's
    chain = DetatarTransformer.from_config(make_config([wkv_layer(None), wkv_layer(None, weights_of=0), wkv_layer(None, weights_of=1)]), torch.float32)
    assert chain.layers[2].block is chain.layers[0].block
    cfg = make_config([wkv_layer(dense())])
    W = random_weights(cfg)
    del W["l0.mix.u"]
    with pytest.raises(KeyError, match="l0.mix.u"):
        DetatarTransformer.from_config(cfg, torch.float32).load_tensors(W)
    W = random_weights(cfg)
    W["l0.rg1"] = W["l0.rg1"][:-1]
    with pytest.raises(ValueError, match="l0.rg1"):
        DetatarTransformer.from_config(cfg, torch.float32).load_tensors(W)


def test_cache_plan_and_state_sizes():
    from cold_compress_b200.detatar import DetatarTransformer
    from cold_compress_b200.generation_utils import reset_caches, setup_caches
    cfg = make_config(default_layers())
    model = DetatarTransformer.from_config(cfg, torch.float32)
    model.load_tensors(random_weights(cfg))
    ck = setup_caches(model, None, "cpu", 64, {})
    assert ck["cache_strategy"] == ["state", "latent", "latent", "state", "latent", "latent", "state"]
    l1, l5, l0, l6 = model.layers[1], model.layers[5], model.layers[0], model.layers[6]
    assert l1.kv_cache is not l5.kv_cache and l0.state is not l6.state        # shared weights, own cache and state
    assert l1.kv_cache.k_cache.shape == (1, 1, 64, 48) and l1.kv_cache.v_cache.numel() == 0
    assert l1.state.vectors.shape == (1, 96) and l0.state.vectors.shape == (2, 96) and l0.state.matrix.shape == (3, 24, 24)
    l0.state.matrix.fill_(1.0)
    l1.kv_cache.pos.fill_(3)
    reset_caches(model)
    assert float(l0.state.matrix.abs().sum()) == 0 and int(l1.kv_cache.pos.max()) == -1
    assert model.min_cache_length() == 64 and model.get_cache_stats(1, 1)["cache_memory_gb"] > 0


# ----------------------------------------------------------------------------------------------- the restatement itself

def test_restatement_is_causal_and_shifts_by_one_token():
    cfg = make_config(default_layers())
    W = random_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, cfg["vocab"], (20,), generator=g).tolist()
    b = a[:12] + torch.randint(0, cfg["vocab"], (8,), generator=g).tolist()
    la, lb = R.forward(cfg, W, a), R.forward(cfg, W, b)
    assert torch.allclose(la[:12], lb[:12], atol=1e-10) and not torch.allclose(la[12:], lb[12:], atol=1e-3)
    h = torch.randn(5, 7, dtype=torch.float64, generator=g)
    mu = torch.rand(7, dtype=torch.float64, generator=g)
    s = R.shift_mix(h, mu)
    assert torch.allclose(s[0], h[0] * (1 - mu)) and torch.allclose(s[3], h[3] + (h[2] - h[3]) * mu)


def test_restatement_recurrence_equals_its_unrolled_sum():
    """o_t = sum_{s<t} (r_t . (prod_{s<q<t} w_q) k_s) v_s + (r_t . u k_t) v_t, written out for one head."""
    g = torch.Generator().manual_seed(5)
    T, D = 9, 5
    r, k, v = (torch.randn(T, 1, D, dtype=torch.float64, generator=g) for _ in range(3))
    w = torch.rand(T, 1, D, dtype=torch.float64, generator=g)
    u = torch.randn(1, D, dtype=torch.float64, generator=g)
    out, S = R.wkv_recurrence(r, k, v, w, u)
    for t in range(T):
        want = (r[t, 0] * u[0] * k[t, 0]).sum() * v[t, 0]
        for s in range(t):
            decay = torch.ones(D, dtype=torch.float64)
            for q in range(s + 1, t):
                decay = decay * w[q, 0]
            want = want + (r[t, 0] * decay * k[s, 0]).sum() * v[s, 0]
        assert torch.allclose(out[t, 0], want, atol=1e-12)
    # a second call continues from the state the first left
    o2, _ = R.wkv_recurrence(r[5:], k[5:], v[5:], w[5:], u, R.wkv_recurrence(r[:5], k[:5], v[:5], w[:5], u)[1])
    assert torch.allclose(o2, out[5:], atol=1e-12)


def test_restatement_router_rules():
    g = torch.Generator().manual_seed(6)
    r = {"experts": 9, "identity": 3, "top": 4, "groups": {"count": 4, "keep": 2}}
    h = torch.randn(50, 16, dtype=torch.float64, generator=g)
    router = torch.randn(12, 16, dtype=torch.float64, generator=g)
    corr = torch.randn(12, dtype=torch.float64, generator=g) * 0.3 - 0.5       # every choice score negative
    ids, w = R.route(h, router, corr, r)
    assert torch.allclose(w.sum(-1), torch.ones(50, dtype=torch.float64)) and (w > 0).all()
    assert ((ids // 3).unsqueeze(-1) == (ids // 3).unsqueeze(-2)).sum(-1).min() >= 1
    assert all(len(set((row // 3).tolist())) <= 2 for row in ids)             # at most `keep` groups per token
    s = torch.softmax(h @ router.T, -1)
    assert torch.allclose(w, s.gather(1, ids) / s.gather(1, ids).sum(-1, keepdim=True))   # weights ignore the correction
    # with every group kept and no correction the choice is the plain top-k of the scores
    r2 = dict(r, groups={"count": 1, "keep": 1})
    ids2, _ = R.route(h, router, torch.zeros(12, dtype=torch.float64), r2)
    assert torch.equal(ids2.sort(-1).values, s.topk(4, -1).indices.sort(-1).values)


def test_restatement_identity_experts_and_rope():
    g = torch.Generator().manual_seed(7)
    mlp = moe(experts=2, identity=2, top=1, groups=1, keep=1, ff=4, shared=0)
    h = torch.randn(6, 8, dtype=torch.float64, generator=g)
    P = {"router": torch.tensor([[0.0] * 8] * 3 + [[0.0] * 8], dtype=torch.float64), "correction": torch.tensor([0., 0., 0., 1.], dtype=torch.float64)}
    for e in range(2):
        for n, shape in (("gate", (4, 8)), ("up", (4, 8)), ("down", (8, 4))):
            P[f"e{e}.{n}"] = torch.randn(*shape, dtype=torch.float64, generator=g)
    assert torch.allclose(R.moe(h, P, mlp), h)                                # the corrected choice is an identity expert, weight 1
    v = torch.randn(4, 2, 10, dtype=torch.float64, generator=g)
    out = R.rope(v, torch.tensor([0, 1, 2, 300]), 100.0, 6)
    assert torch.equal(out[0], v[0]) and torch.equal(out[..., 6:], v[..., 6:])
    assert torch.allclose(out[..., :6].pow(2).sum(-1), v[..., :6].pow(2).sum(-1))
    a = 300 * 100.0 ** (-2 / 6)
    assert torch.allclose(out[3, 0, 1], v[3, 0, 1] * torch.cos(torch.tensor(a, dtype=torch.float64)) - v[3, 0, 4] * torch.sin(torch.tensor(a, dtype=torch.float64)))


def test_new_entry_points_validate_their_arguments():
    """The binding's structures line up with the header: arguments are rejected by the field they are wrong in (no launch
    happens before validation, so this runs without a device)."""
    import ctypes as C
    from cold_compress_b200 import _lib
    lib = _lib.load_seq()
    err = lambda: lib.cc_seq_last_error().decode()
    fake = 0x1000
    g = _lib.CcSeqGatedNorm()
    g.x, g.w, g.T, g.E, g.groups = fake, fake, 2, 12, 5
    assert lib.cc_seq_gated_group_norm(C.byref(g), None) < 0 and "bad argument" in err()       # 5 groups do not divide 12
    g.groups, g.shift_state, g.shift_mu = 3, fake, fake
    assert lib.cc_seq_gated_group_norm(C.byref(g), None) < 0 and "one token" in err()          # the fused shift with T = 2
    d = _lib.CcSeqLatentDecode()
    for name in ("q", "k_new", "k_cache", "pos", "input_pos", "y"):
        setattr(d, name, fake)
    d.H, d.Dk, d.C, d.L = 4, 24, 32, 100
    assert lib.cc_seq_latent_decode(C.byref(d), None) < 0 and "bad argument" in err()          # value columns beyond the row
    d.C = 16
    assert lib.cc_seq_latent_decode(C.byref(d), None) < 0 and "workspace" in err()
    assert lib.cc_seq_latent_decode_workspace(4, 16, 100) == 4 * 4 * (2 + 16) * 4               # 4 runs of 32 keys
    m = _lib.CcSeqGemvMulti()
    assert lib.cc_seq_gemv_multi(C.byref(m), None) < 0 and "job count" in err()
    m.n_jobs = 2
    m.job[0].x = m.job[0].W = m.job[0].out = fake
    m.job[0].N = m.job[0].K = 8
    m.job[0].off_up = -1
    assert lib.cc_seq_gemv_multi(C.byref(m), None) < 0 and "bad job" in err()                   # the second job is empty
    w = _lib.CcSeqWkv()
    assert lib.cc_seq_wkv(C.byref(w), None) < 0 and "wkv" in err()
    for name in ("r", "k", "v", "wraw", "w0", "u", "state", "o"):
        setattr(w, name, fake)
    w.T, w.H, w.D = 1, 1, 300
    assert lib.cc_seq_wkv(C.byref(w), None) < 0 and "256" in err()
    assert lib.cc_seq_moe_route(fake, 8, None, fake, fake, 3, 8, 3, 1, 2, 0, 1, 1, 1.0, None) < 0 and "moe_route" in err()   # 3 groups of 8 outputs
