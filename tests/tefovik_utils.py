"""Small random Tefovik checkpoints for the tests: configurations, weights under the checkpoint's tensor names, and
helpers to run the runtime.  The sizes here are the tests' own."""
from __future__ import annotations

import copy

import torch

from tidelorn_utils import row_error  # noqa: F401  (same error measure for all designs)


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def mamba_layer(mlp=None, heads=4, vdim=12, state=20, groups=2, norm_groups=2, conv=3):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}


def attention(heads=6, kv_heads=2, dim=16, vdim=20, conv=2, size=9, base=500.0, dims=None, scale=None):
    cfg = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
           "rot": {"base": base, "dims": dim if dims is None else dims}, "scale": scale or dim ** -0.5}
    if size:
        cfg["mask"] = {"size": size}
    return cfg


def delta(heads=4, kv_heads=2, dim=24, vdim=10, conv=4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel_layer(mlp=None, left=None, right=None):
    return {"type": "parallel", "mlp": mlp, "mixer": {"left": left or attention(), "right": right or delta()}}


def make_config(layers, width=64, vocab=131, eps=1e-5, alpha=2.0, softcap=12.0):
    cfg = {"architecture": "Tefovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
           "layers": copy.deepcopy(layers)}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def default_layers():
    """Both mixers with and without a feed-forward; grouped heads on every side; a partly rotated attention."""
    return [parallel_layer(dense()), mamba_layer(), parallel_layer(None, left=attention(heads=4, kv_heads=4, dim=12, vdim=8, conv=4, size=16, dims=8)),
            mamba_layer(dense(40), heads=3, vdim=16, state=9, groups=1, norm_groups=1, conv=4),
            parallel_layer(dense(56), right=delta(heads=2, kv_heads=2, dim=40, vdim=36, conv=2))]


def random_weights(cfg, seed=0, ranks=(5, 7)):
    """bf16 tensors under the checkpoint's names; gains, scales and depth coefficients away from their neutral values."""
    g = torch.Generator().manual_seed(seed)
    E, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16)

    def conv(name, channels, taps):
        W[name] = rnd(channels, taps, s=taps ** -0.5, mean=0.3)

    W = {"embed": rnd(V, E, s=0.8), "embed.norm": rnd(E, s=0.2, mean=1.0), "final.norm": rnd(E, s=0.2, mean=1.0),
         "head": rnd(V, E, s=E ** -0.5 * 3.0)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        W[p + "norm1"], W[p + "ls1"] = rnd(E, s=0.2, mean=1.0), rnd(E, s=0.3, mean=1.0)
        W[p + "dwa"] = rnd(i + 2, s=0.3, mean=1.0 / (i + 2))
        if layer["type"] == "mamba2":
            H, Vd, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, q = H * Vd, p + "mix."
            W[q + "in"] = rnd(2 * inner + 2 * G * N + H, E, s=E ** -0.5)
            conv(q + "conv", inner + 2 * G * N, m["conv"])
            W[q + "conv.b"] = rnd(inner + 2 * G * N, s=0.2)
            W[q + "dt_bias"], W[q + "A_log"], W[q + "D"] = rnd(H, s=0.5, mean=-1.0), rnd(H, s=0.5, mean=-0.5), rnd(H, s=0.5, mean=1.0)
            W[q + "norm"], W[q + "o"] = rnd(inner, s=0.2, mean=1.0), rnd(E, inner, s=inner ** -0.5 * 2.0)
        else:
            l, r = m["left"], m["right"]
            q = p + "mix.left."
            H, G, D, Vd = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            for name, rows in (("q", H * D), ("k", G * D), ("v", G * Vd)):
                W[q + name] = rnd(rows, E, s=E ** -0.5 * 1.5)
                conv(q + name + ".conv", rows, l["conv"])
            W[q + "q.norm"], W[q + "k.norm"] = rnd(D, s=0.3, mean=1.5), rnd(D, s=0.3, mean=1.5)
            W[q + "g"], W[q + "o"], W[q + "out"] = rnd(H, E, s=E ** -0.5 * 2.0), rnd(E, H * Vd, s=(H * Vd) ** -0.5), rnd(E, s=0.2, mean=1.0)
            q = p + "mix.right."
            H, G, D, Vd = r["heads"], r["kv_heads"], r["dim"], r["vdim"]
            for name, rows in (("q", G * D), ("k", G * D), ("v", H * Vd)):
                W[q + name] = rnd(rows, E, s=E ** -0.5 * 1.5)
                conv(q + name + ".conv", rows, r["conv"])
            W[q + "b"], W[q + "A_log"] = rnd(H, E, s=E ** -0.5 * 2.0), rnd(H, s=0.5, mean=-1.0)
            W[q + "a1"], W[q + "a2"], W[q + "dt_bias"] = rnd(ranks[0], E, s=E ** -0.5), rnd(H * D, ranks[0], s=0.5), rnd(H * D, s=0.5, mean=-1.0)
            W[q + "g1"], W[q + "g2"] = rnd(ranks[1], E, s=E ** -0.5), rnd(H * Vd, ranks[1], s=0.7)
            W[q + "norm"], W[q + "o"], W[q + "out"] = rnd(Vd, s=0.2, mean=1.0), rnd(E, H * Vd, s=(H * Vd) ** -0.5), rnd(E, s=0.2, mean=1.0)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            W[p + "norm2"], W[p + "ls2"] = rnd(E, s=0.2, mean=1.0), rnd(E, s=0.3, mean=1.0)
            W[p + "mlp.up"], W[p + "mlp.down"] = rnd(F, E, s=E ** -0.5 * 1.5), rnd(E, F, s=F ** -0.5)
    return W


def build_model(cfg, W, dtype, max_seq_length, device="cuda"):
    from cold_compress_b200.generation_utils import setup_caches
    from cold_compress_b200.tefovik import TefovikTransformer
    model = TefovikTransformer.from_config(cfg, dtype)
    model.load_tensors(W)
    model = model.to(device).eval()
    setup_caches(model, None, device, max_seq_length, {})
    return model


def fp32_tolerance(cfg, W, tokens, want):
    """Three times the row error that fp32 rounding alone causes in the restatement itself (float32 against float64
    on the CPU): the bar for the fp32 kernels."""
    import tefovik_reference as R
    return max(3.0 * row_error(R.forward(cfg, W, tokens, dtype=torch.float32), want).max().item(), 5e-6)


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
