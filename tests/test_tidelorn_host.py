"""CPU tests around the Tidelorn design: checkpoint folders and the model registry, configuration errors, the
per-layer cache plan, and sanity properties of the plain restatement the GPU tests compare against."""
import json

import pytest
import torch

import tidelorn_reference as R
from tidelorn_utils import as_double, default_layers, global_layer, make_config, random_weights, window_layer


def test_safetensors_round_trip(tmp_path):
    from cold_compress_b200.checkpoint import read_safetensors, write_safetensors
    t = {"a.b": torch.randn(3, 5).to(torch.bfloat16), "s": torch.tensor(0.25, dtype=torch.bfloat16),
         "i": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2)}
    write_safetensors(tmp_path / "m.safetensors", t)
    r = read_safetensors(tmp_path / "m.safetensors")
    assert set(r) == set(t)
    for k in t:
        assert r[k].dtype == t[k].dtype and r[k].shape == t[k].shape and torch.equal(r[k], t[k])


def test_registry_picks_the_class_from_config_json(tmp_path):
    from cold_compress_b200.checkpoint import load_checkpoint_folder, write_safetensors
    from cold_compress_b200.generation_utils import load_model
    from cold_compress_b200.tidelorn import TidelornTransformer
    cfg = make_config(default_layers())
    W = random_weights(cfg)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", W)
    model = load_model(tmp_path, "cpu", torch.bfloat16, use_tp=False)
    assert isinstance(model, TidelornTransformer) and model.config.n_layer == len(cfg["layers"])
    a = model.layers[1].attention
    nq = a.heads * a.head_dim
    assert torch.equal(a.wqkv[:nq], W["l1.mix.q"]) and torch.equal(a.wqkv[nq:nq + a.kv_heads * a.head_dim], W["l1.mix.k"])
    assert a.bqkv.dtype == torch.float32 and torch.equal(a.bqkv[:nq], W["l1.mix.q.b"].float())
    assert a.sink.dtype == torch.float32 and model.layers[0].attention.sink is None
    assert model.layers[4].feed_forward is None and model.layers[4].norm2 is None
    f = model.layers[0].feed_forward
    assert torch.equal(f.w13[f.ff:], W["l0.mlp.up"])
    (tmp_path / "config.json").write_text(json.dumps(dict(cfg, architecture="Nonesuch")))
    with pytest.raises(ValueError, match="unknown architecture"):
        load_checkpoint_folder(tmp_path, "cpu")


def test_configuration_and_weight_errors():
    from cold_compress_b200.tidelorn import TidelornArgs, TidelornTransformer
    cfg = make_config([global_layer()])
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "attention_9"
    with pytest.raises(ValueError, match="unknown mixer"):
        TidelornArgs.from_config(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError, match="feed-forward"):
        TidelornArgs.from_config(bad)
    with pytest.raises(ValueError, match="agree"):
        TidelornTransformer.from_config(make_config([global_layer(vdim=16), window_layer(3, vdim=24)]))
    W = random_weights(cfg)
    model = TidelornTransformer.from_config(cfg)
    W2 = dict(W)
    W2["l0.mix.k"] = W2["l0.mix.k"][:-1]
    with pytest.raises(ValueError, match="l0.mix.k"):
        model.load_tensors(W2)
    W2 = dict(W)
    del W2["l0.mix.sink"]
    with pytest.raises(KeyError, match="sink"):
        model.load_tensors(W2)
    assert model.load_tensors(dict(W, extra=torch.zeros(1))) == ["extra"]


def test_cache_plan_follows_the_layer_types():
    from cold_compress_b200.cache import KVCacheFull, KVCacheRecentGlobal
    from cold_compress_b200.generation_utils import setup_caches
    from cold_compress_b200.tidelorn import TidelornTransformer
    cfg = make_config(default_layers())
    model = TidelornTransformer.from_config(cfg, torch.float32)
    ck = setup_caches(model, None, "cpu", 100, {})
    assert ck["cache_strategy"][:3] == ["recent_global", "full", "full"]
    for block, layer in zip(model.layers, cfg["layers"]):
        c, m = block.attention.kv_cache, layer["mixer"]
        if layer["type"] == "attention_2":
            assert isinstance(c, KVCacheRecentGlobal) and c.max_cache_length == m["mask"]["size"] and c.sequence_window() == m["mask"]["size"]
        else:
            assert isinstance(c, KVCacheFull) and c.max_cache_length == 100 and c.sequence_window() == 0
        assert c.k_cache.shape == (1, m["kv_heads"], c.max_cache_length, m["dim"]) and c.k_cache.dtype == torch.float32
        assert c.v_cache.shape == (1, m["kv_heads"], c.max_cache_length, m["vdim"])
    assert model.min_cache_length() == 100
    # there is no CPU path: a step on CPU tensors raises instead of computing something else
    from cold_compress_b200._lib import CcError
    with pytest.raises(CcError):
        model(torch.zeros(1, 3, dtype=torch.int32), torch.arange(3), True)


def test_window_cache_with_global_tokens_keeps_them_and_scored_policies_refuse_position_addressing():
    from cold_compress_b200.cache import KVCacheHeavyHitter, KVCacheRecentGlobal
    c = KVCacheRecentGlobal(1, 2, 8, torch.float32, max_cache_length=16, global_tokens=4, max_seq_length=64, cache_bits=None)
    assert c.sequence_window() == 12 and c.sequence_kept() == 4      # the first four positions keep their slots, a ring of 12
    h = KVCacheHeavyHitter(1, 2, 8, torch.bfloat16, max_cache_length=16, global_tokens=1, max_seq_length=64, cache_bits=None,
                           history_window_size=1, recent_window=4, attn_thresholding=False)
    assert h.sequence_window() is None and h.v_head_dim == 8


# ----------------------------------------------------------------------------------------------- the restatement itself

def test_restatement_sink_softmax_and_masks():
    g = torch.Generator().manual_seed(0)
    s = torch.randn(3, 6, 6, generator=g, dtype=torch.float64)
    i, j = torch.arange(6)[:, None], torch.arange(6)[None, :]
    ok = (j <= i) & (i - j < 3)
    sink = torch.tensor([0.5, -1.0, 2.0], dtype=torch.float64)
    p = R.sink_softmax(s, ok, sink)
    assert (p[:, ~ok] == 0).all()
    share = torch.exp(sink)[:, None] / (torch.exp(s).masked_fill(~ok, 0).sum(-1) + torch.exp(sink)[:, None])
    assert torch.allclose(p.sum(-1) + share, torch.ones(3, 6, dtype=torch.float64))
    assert int(ok.sum(-1).max()) == 3 and int(ok[0].sum()) == 1


def test_restatement_bigram_rows_and_positions():
    rows = R.bigram_rows([4, 9, 2], buckets=7, mul_prev=5, mul_cur=3)
    assert rows.tolist() == [7, (4 * 5 + 9 * 3) % 7, (9 * 5 + 2 * 3) % 7]
    e = R.sinusoid(torch.tensor([0, 3]), 6, torch.float64)
    assert torch.allclose(e[0], torch.tensor([0.0, 1.0] * 3, dtype=torch.float64))
    w1 = 10000.0 ** (-2 / 6)
    assert abs(e[1, 2].item() - torch.sin(torch.tensor(3 * w1, dtype=torch.float64)).item()) < 1e-12
    t = R.query_temperature(10, 0.5, 4, torch.float64)
    assert t[2].item() == 1.0 and abs(t[3].item() - (1 + 0.5 * torch.log(torch.tensor(2.0, dtype=torch.float64)).item())) < 1e-12


def test_restatement_is_causal_and_windows_forget():
    cfg = make_config([window_layer(3, v_mix=False), window_layer(2, v_mix=False)], width=24, vocab=19)
    W = as_double(random_weights(cfg, seed=4))
    a = [1, 2, 3, 4, 5, 6, 7, 8]
    b = [9, 2, 3, 4, 5, 6, 7, 11]     # differs at the first and the last token
    la, lb = R.forward(a, W, cfg), R.forward(b, W, cfg)
    # two layers with windows 3 and 2 reach 3 tokens back; the bigram reaches one more
    assert torch.allclose(la[5:7], lb[5:7]) and not torch.allclose(la[3], lb[3]) and not torch.allclose(la[7], lb[7])
    cfg = make_config([global_layer()], width=24, vocab=19)
    W = as_double(random_weights(cfg, seed=5))
    la, lb = R.forward(a, W, cfg), R.forward(b, W, cfg)
    assert not torch.allclose(la[6], lb[6])
    assert torch.allclose(R.forward(a[:5], W, cfg), la[:5])


def test_sequence_library_exports_every_declared_symbol():
    """Every function include/cc_b200_seq.h declares is bound in _lib.SEQ_EXPORTS and exported by the built library."""
    import re
    from pathlib import Path
    from cold_compress_b200 import _lib
    from cold_compress_b200.build import build_seq_extension
    header = (Path(__file__).resolve().parent.parent / "include" / "cc_b200_seq.h").read_text()
    declared = set(re.findall(r"\b(cc_seq_\w+)\s*\(", header))
    assert declared == set(_lib.SEQ_EXPORTS), declared ^ set(_lib.SEQ_EXPORTS)
    build_seq_extension()
    lib = _lib.load_seq()
    assert lib.cc_seq_abi_version() == _lib.SEQ_ABI_VERSION
    assert lib.cc_seq_decode_workspace(8, 2, 64, 1000, 0) > 0
    # argument checks come back as error codes with a message, not as faults
    a = _lib.CcSeqAttn()
    assert lib.cc_seq_attention(a, None) < 0 and b"NULL" in lib.cc_seq_last_error()
    g = _lib.CcSeqGemv()
    assert lib.cc_seq_gemv(g, None) < 0 and b"gemv" in lib.cc_seq_last_error()
