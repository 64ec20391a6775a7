"""Small random Nevodra checkpoints for the tests: configurations, weights under the checkpoint's tensor names, and
helpers to run the runtime.  The sizes here are the tests' own."""
from __future__ import annotations

import copy

import torch

from tidelorn_utils import row_error  # noqa: F401  (same error measure for all designs)


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, count=3, keep=2, scale=1.3, shared=40):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def window_layer(mlp=None, heads=4, kv_heads=2, dim=16, vdim=12, size=13, keep_first=3, scale=None, softcap=8.0):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5}
    if size:
        mixer["mask"] = {"size": size, "keep_first": keep_first}
    if softcap:
        mixer["softcap"] = softcap
    return {"type": "attention", "mlp": mlp, "mixer": mixer}


def latent_layer(mlp=None, heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, base=300.0, dims=None, scale=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def make_config(layers, width=64, vocab=131, eps=1e-5, taps=4, embed_scale=0.7, loop=None):
    cfg = {"architecture": "Nevodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
           "embedding": {"scale": embed_scale}, "layers": copy.deepcopy(layers)}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def default_layers():
    """Both mixers and both feed-forwards, one layer without a feed-forward."""
    return [window_layer(dense()), latent_layer(moe()), window_layer(moe(experts=8, top=3, count=4, keep=2, shared=0), heads=6, kv_heads=2, size=9, keep_first=0),
            latent_layer(None, dims=4), latent_layer(dense(40), heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16)]


DEFAULT_LOOP = (1, 3, 3)     # layers 1 and 2 run three times in a row


def random_weights(cfg, seed=0, decisive=False):
    """bf16 tensors under the checkpoint's names; gains and coefficients away from their neutral values.  `decisive`
    spaces the routers' corrections further apart than the scores can vary, so that no choice (of an expert or of a
    group) is a close call: with
    random corrections a few tokens sit where two choice scores differ by less than the bf16 error of the router's
    input, either choice is a correct bf16 result, and the tokens after such a one see it too.  The bf16 runs of the
    model use decisive weights and are held to a bar for every position; the fp32 runs route by the scores."""
    g = torch.Generator().manual_seed(seed)
    E, V = cfg["width"], cfg["vocab"]
    taps = cfg["canon"]["taps"]

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16)

    W = {"embed": rnd(V, E, s=1.5), "final.norm": rnd(E, s=0.2, mean=1.0), "head": rnd(V, E, s=E ** -0.5 * 3.0)}
    loop = cfg.get("loop")
    if loop:
        W["loop.step"] = rnd(loop["times"], E, s=0.5)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        W[p + "norm1"], W[p + "canon1"] = rnd(E, s=0.2, mean=1.0), rnd(E, taps, s=0.4)
        q = p + "mix."
        if layer["type"] == "attention":
            H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[q + "q"], W[q + "k"], W[q + "v"] = rnd(H * D, E, s=E ** -0.5), rnd(G * D, E, s=E ** -0.5), rnd(G * Vd, E, s=E ** -0.5)
            W[q + "q.norm"], W[q + "k.norm"] = rnd(H * D, s=0.3, mean=1.5), rnd(G * D, s=0.3, mean=1.5)
            W[q + "r1"], W[q + "r2"] = rnd(H, s=0.2, mean=0.6).abs(), rnd(H, s=0.3, mean=0.8).abs()
            W[q + "o"] = rnd(E, H * Vd, s=(H * Vd) ** -0.5)
        else:
            H, D, R, Vd, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            W[q + "q"], W[q + "dkv"] = rnd(H * (D + R), E, s=E ** -0.5 * 2.0), rnd(C + R, E, s=E ** -0.5 * 2.0)
            W[q + "dkv.norm"] = rnd(C, s=0.2, mean=1.0)
            W[q + "uk"], W[q + "uv"] = rnd(H * D, C, s=C ** -0.5 * 1.5), rnd(H * Vd, C, s=C ** -0.5)
            W[q + "sink"] = rnd(H, s=1.0, mean=0.5)
            W[q + "o"] = rnd(E, H * Vd, s=(H * Vd) ** -0.5)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        W[p + "norm2"], W[p + "canon2"] = rnd(E, s=0.2, mean=1.0), rnd(E, taps, s=0.4)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            W[q + "up"], W[q + "down"] = rnd(F, E, s=E ** -0.5 * 1.5), rnd(E, F, s=F ** -0.5)
            W[q + "act"] = torch.tensor([0.9, 0.4, -0.3, 0.1]).to(torch.bfloat16) + rnd(4, s=0.05)
        else:
            n, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            W[q + "router"] = rnd(n, E, s=E ** -0.5 * 2.0)
            if decisive:      # 1.5 * 2^k in a random order: single choices and sums of a group's two best are all 1.5 or more apart
                perm = torch.randperm(n, generator=g).double()
                W[q + "correction"] = (1.5 * torch.pow(2.0, perm) if n <= 16 else 1.5 * perm).to(torch.bfloat16)
            else:
                W[q + "correction"] = rnd(n, s=0.3)
            names = [f"e{e}." for e in range(n)] + (["shared."] if mlp.get("shared") else [])
            for name in names:
                Fe = mlp["shared"]["ff"] if name == "shared." else F
                W[q + name + "gate"], W[q + name + "up"] = rnd(Fe, E, s=E ** -0.5 * 1.5), rnd(Fe, E, s=E ** -0.5 * 1.5)
                W[q + name + "down"] = rnd(E, Fe, s=Fe ** -0.5)
    return W


def build_model(cfg, W, dtype, max_seq_length, device="cuda"):
    from cold_compress_b200.generation_utils import setup_caches
    from cold_compress_b200.nevodra import NevodraTransformer
    model = NevodraTransformer.from_config(cfg, dtype)
    model.load_tensors(W)
    model = model.to(device).eval()
    setup_caches(model, None, device, max_seq_length, {})
    return model


def reference_logits(cfg, W, tokens, collect=None, dtype=torch.float64):
    import nevodra_reference as R
    return R.forward(torch.as_tensor(tokens), W, cfg, dtype=dtype, collect=collect)


def fp32_tolerance(cfg, W, tokens, want):
    """Three times the row error that fp32 rounding alone causes in the restatement itself (float32 against float64
    on the CPU): the bar for the fp32 kernels."""
    return max(3.0 * row_error(reference_logits(cfg, W, tokens, dtype=torch.float32), want).max().item(), 5e-6)


def run_portions(model, tokens, portions, device="cuda"):
    """Feeds `tokens` in consecutive portions through the runtime's step function; logits of every position."""
    from cold_compress_b200.generation_utils import model_step
    assert sum(portions) == len(tokens)
    out, at = [], 0
    for n in portions:
        x = torch.tensor(tokens[at:at + n], dtype=torch.int32, device=device).view(1, -1)
        ip = torch.arange(at, at + n, dtype=torch.int32, device=device)
        lg = model_step(model, x, ip, is_prefill=not (n == 1 and at > 0), logits_at=torch.arange(n, device=device))
        out.append(lg[0].float())
        at += n
    return torch.cat(out, 0)


def assert_rows_close(err, dtype, tol, what=""):
    """err: one error per position.  fp32: every position within `tol`.  bf16: the median within a third of `tol` and no
    position beyond it."""
    err = torch.as_tensor(err).double().reshape(-1)
    if dtype == torch.bfloat16:
        assert err.max() < tol and err.median() < tol / 3, (what, err.median().item(), err.max().item())
    else:
        assert err.max() < tol, (what, err.max().item(), int(err.argmax()))
