"""CPU tests of the Nevodra design's host side: registry, configuration and shape errors, weight loading and fusing,
layer runs of a loop, the cache plan, and the plain restatement's own invariants (the GPU tests hold the kernels to
that restatement)."""
import json

import pytest
import torch

import nevodra_reference as R
from nevodra_utils import DEFAULT_LOOP, default_layers, dense, latent_layer, make_config, moe, random_weights, reference_logits, window_layer

F64 = torch.float64


def test_registry_builds_the_class_from_a_checkpoint_folder(tmp_path):
    from cold_compress_b200.checkpoint import load_checkpoint_folder, write_safetensors
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=1)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    model = load_checkpoint_folder(tmp_path, "cpu", torch.bfloat16)
    assert type(model).__name__ == "NevodraTransformer" and model.config.n_layer == 9 and model.supports_prompt_portions
    assert [i for i, _ in model.config.runs()] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [l.step_row for l in model.layers] == [None, 0, None, 1, None, 2, None, None, None]
    assert model.layers[1].block is model.layers[3].block is model.layers[5].block and len(model.blocks()) == 5
    assert sum(p.numel() for p in model.parameters()) == sum(p.numel() for _, b in model.blocks() for p in b.parameters()) + \
        model.tok_embeddings.numel() + model.output.numel() + model.norm.weight.numel() + model.loop_step.numel()
    a = model.layers[0].block            # windowed layer: fused q | k | v rows, zero padding; dense up rows
    m = a.mixer
    assert m.w_in.shape[0] % 16 == 0 and torch.equal(m.w_in[:m.nq], W["l0.mix.q"]) and torch.equal(m.w_in[m.nq + m.nk:m.nq + m.nk + m.nv], W["l0.mix.v"])
    assert float(m.w_in[m.nq + m.nk + m.nv:].abs().sum()) == 0
    assert torch.equal(a.w_ff[:72], W["l0.mlp.up"]) and torch.equal(a.norms.conv[1], W["l0.canon2"].float())
    b = model.layers[1].block            # latent layer: q | dkv rows; router | shared gate | shared up rows
    m = b.mixer
    assert torch.equal(m.w_in[m.q_rows:m.q_rows + m.kv_rank + m.rot_dim], W["l1.mix.dkv"]) and m.q_rank == 0 and m.sink.numel() == 3
    assert torch.equal(b.w_ff[:6], W["l1.mlp.router"]) and torch.equal(b.w_ff[6:46], W["l1.mlp.shared.gate"])
    assert b.mlp.sigmoid_scores and b.mlp.group_top == 2 and not b.mlp.renormalize and b.mlp.sg_rows == 0
    assert model.layers[7].block.mlp is None and model.layers[7].block.norms.n == 1


def test_configuration_and_shape_errors():
    from cold_compress_b200.nevodra import NevodraArgs, NevodraTransformer
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][1]["type"] = "conv"
    with pytest.raises(ValueError, match="unknown mixer type"):
        NevodraArgs.from_config(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError, match="feed-forward"):
        NevodraArgs.from_config(bad)
    bad = json.loads(json.dumps(cfg))
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError, match="loop"):
        NevodraArgs.from_config(bad)
    with pytest.raises(ValueError, match="key/value heads"):
        NevodraTransformer.from_config(make_config([window_layer(None, heads=5, kv_heads=2)]))
    with pytest.raises(ValueError, match="equal groups"):
        NevodraTransformer.from_config(make_config([window_layer(moe(experts=7, count=3))]))
    model = NevodraTransformer.from_config(cfg, torch.float32)
    W = random_weights(cfg, seed=2)
    short = dict(W)
    del short["l2.canon2"]
    with pytest.raises(KeyError, match="l2.canon2"):
        model.load_tensors(short)
    wrong = dict(W)
    wrong["loop.step"] = wrong["loop.step"][:2]
    with pytest.raises(ValueError, match="loop.step"):
        model.load_tensors(wrong)
    extra = dict(W)
    extra["l9.unused"] = torch.zeros(1)
    assert model.load_tensors(extra) == ["l9.unused"]


def test_cache_plan_and_state_shapes():
    from cold_compress_b200.generation_utils import reset_caches, setup_caches
    from cold_compress_b200.nevodra import NevodraTransformer
    layers = [window_layer(dense(), size=9, keep_first=4), latent_layer(None), window_layer(None, size=0)]
    model = NevodraTransformer.from_config(make_config(layers, taps=4, loop=(0, 2, 2)), torch.float32)
    ck = setup_caches(model, None, "cpu", 77, {})
    assert ck["cache_strategy"] == ["recent_global", "latent", "recent_global", "latent", "full"]
    assert ck["max_cache_length"] == [13, 77, 13, 77, 77] and ck["global_tokens"] == [4, 0, 4, 0, 0]
    a, b, a2, b2, c = model.layers
    assert a.kv_cache is not a2.kv_cache and a.state is not a2.state and a.block is a2.block
    assert a.kv_cache.sequence_window() == 9 and a.kv_cache.sequence_kept() == 4 and c.kv_cache.sequence_window() == 0
    assert a.kv_cache.k_cache.shape == (1, 2, 13, 16) and a.kv_cache.v_cache.shape == (1, 2, 13, 12)
    assert b.kv_cache.k_cache.shape == (1, 1, 77, 24 + 8) and b.kv_cache.v_cache.numel() == 0
    assert a.state.vectors.shape == (3, 64) and a.state.matrix.numel() == 0
    assert model.min_cache_length() == 77 and model.prompt_cache_overflow(100) == [False, True, False, True, False]
    a.state.vectors.fill_(1.0)
    a.kv_cache.pos.fill_(3)
    reset_caches(model)
    assert float(a.state.vectors.abs().sum()) == 0 and int(a.kv_cache.pos.max()) == -1


# ----------------------------------------------------------------------------------------------- the restatement's own invariants

def test_restatement_is_causal_and_loops_share_weights():
    cfg = make_config(default_layers(), loop=DEFAULT_LOOP)
    W = random_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(4)
    tokens = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    full = reference_logits(cfg, W, tokens)
    assert (reference_logits(cfg, W, tokens[:25]) - full[:25]).abs().max() < 1e-9
    col = []
    reference_logits(cfg, W, tokens, col)
    assert len(col) == 9
    unrolled = make_config([cfg["layers"][i] for i in (0, 1, 2, 1, 2, 1, 2, 3, 4)])
    assert R.layer_runs(unrolled) == [(i, None) for i in range(9)]
    W2 = dict(W)
    W2["loop.step"] = torch.zeros_like(W["loop.step"])
    assert (reference_logits(cfg, W2, tokens) - full).abs().max() > 1e-6       # the pass vectors matter


def test_window_mask_reach():
    ok = R.window_mask(30, 5, 3)
    assert ok[20, 16] and not ok[20, 15] and ok[20, 2] and not ok[20, 3] and ok[20, 20] and not ok[20, 21]
    assert ok[4, 0] and ok[2, 0] and int(ok[29].sum()) == 5 + 3
    assert int(R.window_mask(30, 5, 0)[29].sum()) == 5


def test_input_convolution_and_polynomial_activation():
    g = torch.Generator().manual_seed(5)
    h, w = torch.randn(9, 4, generator=g, dtype=F64), torch.randn(4, 3, generator=g, dtype=F64)
    y = R.input_conv(h, w)
    assert torch.allclose(y[0], h[0] * (1 + w[:, 2])) and torch.allclose(y[5], h[5] * (1 + w[:, 2]) + h[4] * w[:, 1] + h[3] * w[:, 0])
    z = torch.randn(3, 50, generator=g, dtype=F64)
    out = R.poly_norm(z, torch.tensor([1.0, 0.0, 0.0, 0.0], dtype=F64), 0.0)
    assert torch.allclose((out * out).mean(-1), torch.ones(3, dtype=F64))
    assert torch.allclose(R.poly_norm(z, torch.tensor([0.0, 0.0, 0.0, 0.3], dtype=F64), 1e-5), torch.full((3, 50), 0.3, dtype=F64))


def test_router_rules():
    z = torch.tensor([2.0, 1.9, -3.0, -3.0, 3.0, -4.0, -4.0, -4.0], dtype=F64)
    corr = torch.zeros(8, dtype=F64)
    r = {"top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}}
    ids, wts = R.route(z, corr, r)            # the first group's two best outweigh the second group's single best
    assert sorted(ids.tolist()) == [0, 1] and torch.allclose(wts.sum(), 2.0 * (torch.sigmoid(z[0]) + torch.sigmoid(z[1])))
    corr2 = corr.clone()
    corr2[5] = 2.0                             # the correction moves the choice, not the weight
    ids, wts = R.route(z, corr2, r)
    assert sorted(ids.tolist()) == [4, 5] and abs(wts[ids.tolist().index(5)].item() - 2.0 * torch.sigmoid(z[5]).item()) < 1e-12
    ids, _ = R.route(z, corr - 5.0, r)        # all choice scores negative: losers are at minus infinity, not zero
    assert sorted(ids.tolist()) == [0, 1]


def test_sink_and_rotation():
    cfg = make_config([latent_layer(None)], taps=1)
    W = {k: v.double() for k, v in random_weights(cfg, seed=6).items()}
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(12, 64, generator=torch.Generator().manual_seed(7), dtype=F64)
    base = R.latent_attention(h, W, "l0.mix.", m, 1e-5)
    W2 = dict(W)
    W2["l0.mix.sink"] = W["l0.mix.sink"] - 50.0     # a sink that weighs nothing: ordinary softmax, first token = its own value
    free = R.latent_attention(h, W2, "l0.mix.", m, 1e-5)
    c = R.rms_norm((h @ W["l0.mix.dkv"].T)[:, :24], W["l0.mix.dkv.norm"], 1e-5)
    v0 = (c[0] @ W["l0.mix.uv"].T) @ W["l0.mix.o"].T.reshape(3 * 20, 64)
    assert torch.allclose(free[0], v0, atol=1e-9) and (free - base).abs().max() > 1e-4
    x = torch.randn(5, 2, 8, generator=torch.Generator().manual_seed(8), dtype=F64)
    pos = torch.arange(5)
    rot = R.rotate_interleaved(x, pos, 100.0, 4)
    assert torch.allclose(rot[0], x[0]) and torch.allclose(rot[..., 4:], x[..., 4:])
    assert torch.allclose((rot[..., 0:2] ** 2).sum(-1), (x[..., 0:2] ** 2).sum(-1))
    assert torch.allclose(rot[3, 1, 2], x[3, 1, 2] * torch.cos(torch.tensor(3 * 100.0 ** -0.5, dtype=F64)) - x[3, 1, 3] * torch.sin(torch.tensor(3 * 100.0 ** -0.5, dtype=F64)))
