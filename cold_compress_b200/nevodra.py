"""Nevodra: a decoder-only design whose layers run a mixer and a feed-forward side by side, each on its own RMS norm
of the same stream (`x <- x + mixer(c1(norm1(x))) + ff(c2(norm2(x)))`), where `c(h) = h + conv(h)` adds a short causal
per-channel convolution over time to the sublayer's input.  Two kinds of mixer: grouped-query softmax attention without
rotation (query and key RMS-normed over their whole projection, tanh soft cap on the scores, a penalty
`a_h ln(1 + b_h (i - j))` on the distance, a sliding window that also keeps the first tokens) and attention through
low-rank latents (full-rank queries, interleaved rotary pairs on a key part shared by all heads, a learned sink logit in
the softmax denominator).  Two kinds of feed-forward: dense with a polynomial-of-unit-RMS activation, and a mixture of
experts (sigmoid scores, a correction for the choice only, groups ranked by the sum of their two best choices, weights
not renormalised but scaled, an ungated shared expert).  A run of consecutive layers can be repeated with the same
weights: every pass has caches and state of its own and starts by adding a learned vector to the stream.

The model plugs into the same runtime as the package's other models: `setup_caches` builds each layer run's cache and
state through `cache.get_cache_constructor` ("recent_global" = kept first positions + a ring for windowed layers,
"latent" rows for latent layers, "state" for the convolution tails), `forward(idx, input_pos, is_prefill)` is what
`generation_utils.prefill` / `decode_one_token` / `GraphedDecoder` call, and a step of any length continues from what
the earlier steps left.  Matrix products of prompt portions are cuBLAS (torch.mm, fp32 accumulation and output);
one-token steps use this package's product kernels; everything between products is a kernel of csrc/seq.  There is no
CPU path.

Precision: weights, cache rows and product inputs are in the compute dtype (bf16 or fp32); the residual stream,
norms, convolutions, angles, attention scores and weights and router scores are fp32 in both.

`ParallelNorms`, `WindowAttention` and `PolyNormMLP` take their sizes and constants as arguments so that another design
can use them; the latent attention and the routed experts are the ones of `detatar` with other options.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import _lib, seq_ops
from .cache import get_cache_constructor
from .detatar import GroupRMSNorm, LatentAttention, RoutedExperts, _out, _pad16, _padded_rows, _proj, _zeros

MIXERS = ("attention", "latent_attention")
FEED_FORWARDS = ("dense", "moe")


# --------------------------------------------------------------------------------------------- configuration

@dataclass
class NevodraArgs:
    vocab_size: int
    dim: int
    layers: List[Dict[str, Any]]
    norm_eps: float
    embedding_scale: float
    canon_taps: int
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    block_size: int = 1 << 20      # angles and distances are computed from the position: no table limits the length
    n_layer: int = field(init=False)

    def __post_init__(self):
        if self.canon_taps < 1:
            raise ValueError("the input convolution needs at least one tap")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ValueError("loop: start <= stop must lie within the layers and times must be positive")
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        self.n_layer = len(self.runs())

    def runs(self):
        """[(layer index, pass number or None)] in running order: layers start .. stop-1 `times` times in a row."""
        n = len(self.layers)
        if self.loop_stop <= self.loop_start:
            return [(i, None) for i in range(n)]
        out = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            out += [(i, t) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, None) for i in range(self.loop_stop, n)]

    @classmethod
    def from_config(cls, cfg: Dict[str, Any]):
        loop = cfg.get("loop") or {}
        return cls(vocab_size=int(cfg["vocab"]), dim=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float(cfg["norm"]["eps"]), embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                   canon_taps=int((cfg.get("canon") or {}).get("taps", 1)), loop_start=int(loop.get("start", 0)),
                   loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)))


# --------------------------------------------------------------------------------------------- mechanisms

class ParallelNorms(nn.Module):
    """n RMS norms of the same row (one pass gives the unit-RMS row, each norm its gain), each followed by the input
    convolution `h + sum_j w[:, j] h_(t - taps + 1 + j)` with its own taps table.  The kernel also performs the residual
    sum that precedes the norms (`pending`: the sublayer results of the layer before, and a vector for the whole
    step), so the stream is read and written once per layer.  State per sequence: the last taps - 1 unit-RMS rows."""

    def __init__(self, dim: int, n: int, taps: int, eps: float):
        super().__init__()
        self.n, self.taps, self.eps = int(n), int(taps), float(eps)
        self.weight = _zeros(self.n, dim, dtype=torch.float32)
        self.conv = _zeros(self.n, dim, self.taps, dtype=torch.float32)

    def forward(self, x: Tensor, outs: List[Tensor], tail: Tensor, pending: Optional[dict] = None, add: Optional[Tensor] = None) -> Tensor:
        """Returns the stream after the sum: x itself (updated in place) for steps of several tokens, a new row for one
        token (the launch spreads the row over the GPU, and the CTAs that still read the old row must not see it change)."""
        T = x.shape[0]
        rinv = torch.empty(T, dtype=torch.float32, device=x.device) if T > 1 else None
        x_out = torch.empty_like(x) if T == 1 else None
        seq_ops.par_norm(x, [(self.weight[s], self.conv[s], outs[s]) for s in range(self.n)], self.eps, add=add,
                         tail=tail if self.taps > 1 else None, taps=self.taps, rinv=rinv, x_out=x_out, **(pending or {}))
        return x if x_out is None else x_out


class WindowAttention(nn.Module):
    """Grouped-query softmax attention without rotation.  q and k are RMS-normed over their whole projection (all heads
    at once, a gain per column); scaled scores pass `cap * tanh(s / cap)` and lose `a_h ln(1 + b_h (i - j))`; query i
    sees key j <= i when `i - j < window` or `j < keep_first` (window 0: every earlier key).  The cache keeps the first
    `keep_first` positions in slots of their own and the last `window` in a ring."""

    def __init__(self, dim: int, heads: int, kv_heads: int, head_dim: int, v_dim: int, scale: float, softcap: float,
                 window: int, keep_first: int, eps: float, dtype):
        super().__init__()
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        self.dim, self.heads, self.kv_heads, self.head_dim, self.v_dim = dim, int(heads), int(kv_heads), int(head_dim), int(v_dim)
        self.scale, self.softcap, self.window, self.eps = float(scale), float(softcap), int(window), float(eps)
        self.keep_first = int(keep_first) if self.window else 0
        self.nq, self.nk, self.nv = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_dim
        self.w_in = _zeros(_pad16(self.nq + self.nk + self.nv), dim, dtype=dtype)      # rows: q | k | v | padding
        self.q_norm = _zeros(self.nq, dtype=torch.float32)
        self.k_norm = _zeros(self.nk, dtype=torch.float32)
        self.dist_a = _zeros(self.heads, dtype=torch.float32)
        self.dist_b = _zeros(self.heads, dtype=torch.float32)
        self.w_o = _zeros(dim, self.heads * self.v_dim, dtype=dtype)

    def first_jobs(self, h_act: Tensor):
        a = _out(self.w_in)
        return [(h_act, self.w_in, a)], [a]

    def _attend(self, a: Tensor, ip: Tensor, cache) -> Tensor:
        T, dev, dt = a.shape[0], a.device, self.w_in.dtype
        H, G, D, V = self.heads, self.kv_heads, self.head_dim, self.v_dim
        q = torch.empty(T, H, D, dtype=torch.float32, device=dev)
        k = torch.empty(T, G, D, dtype=dt, device=dev)
        v = torch.empty(T, G, V, dtype=dt, device=dev)
        seq_ops.qk_row_norm(a, 0, self.nq, self.nq, self.nk, self.nq + self.nk, self.nv, self.q_norm, self.k_norm, q, k, v, self.eps)
        y = torch.empty(T, H, V, dtype=dt, device=dev)
        cache.sequence_step(q, k, v, ip, y, window=self.window, scale=self.scale, softcap=self.softcap,
                            dist=(self.dist_a, self.dist_b))
        return y.view(T, H * V)

    def finish(self, outs, ip: Tensor, cache) -> Tensor:
        return self._attend(outs[0], ip, cache)

    def forward(self, h_act: Tensor, ip: Tensor, cache, one_token_kernel: bool = True) -> Tensor:
        return _proj(self._attend(_proj(h_act, self.w_in), ip, cache), self.w_o)

    def one_token_fits(self) -> bool:
        return True


class PolyNormMLP(nn.Module):
    """down(act(up h)), act(z) = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with powers element by element and N = division
    by the root mean square over the token's ff values.  Its up rows are the layer's feed-forward input projection."""

    def __init__(self, dim: int, ff: int, eps: float, dtype):
        super().__init__()
        self.ff, self.eps = int(ff), float(eps)
        self.coef = _zeros(4, dtype=torch.float32)
        self.w_down = _zeros(dim, self.ff, dtype=dtype)

    def n_rows(self):
        return self.ff

    def _act(self, hp: Tensor, off: int) -> Tensor:
        act = torch.empty(hp.shape[0], self.ff, dtype=self.w_down.dtype, device=hp.device)
        seq_ops.poly_norm(hp[:, off:off + self.ff], self.coef, act, self.eps)
        return act

    def forward(self, hp: Tensor, off: int, h, h_act, one_token_kernel: bool = True) -> Tensor:
        return _proj(self._act(hp, off), self.w_down)

    def one_token(self, hp: Tensor, off: int, h, h_act):
        out = _out(self.w_down)
        return [(self._act(hp, off), self.w_down, out)], lambda: out


# --------------------------------------------------------------------------------------------- a layer

class NevodraBlock(nn.Module):
    """The weights of one layer: both norms with their convolutions, the mixer, the feed-forward and its input
    projection (router / shared rows, or the dense up rows)."""

    def __init__(self, cfg: NevodraArgs, layer: Dict[str, Any], dtype):
        super().__init__()
        E, m, mlp = cfg.dim, layer["mixer"], layer.get("mlp")
        self.kind = layer["type"]
        if self.kind == "attention":
            mask = m.get("mask") or {}
            self.mixer = WindowAttention(E, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])),
                                         float(m["scale"]), float(m.get("softcap", 0.0)), int(mask.get("size", 0)),
                                         int(mask.get("keep_first", 0)), cfg.norm_eps, dtype)
        else:
            rot = m.get("rot") or {}
            self.mixer = LatentAttention(E, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), 0, int(m["kv_rank"]),
                                         float(m["scale"]), float(rot.get("base", 10000.0)), int(rot.get("dims", m["rot_dim"])),
                                         cfg.norm_eps, dtype, gated=False, sink=True, interleaved=True)
        if not mlp:
            self.mlp = None
        elif mlp["kind"] == "dense":
            self.mlp = PolyNormMLP(E, int(mlp["ff"]), cfg.norm_eps, dtype)
        else:
            r, shared = mlp["router"], mlp.get("shared") or {}
            g = r.get("groups") or {}
            self.mlp = RoutedExperts(E, int(r["experts"]), 0, int(mlp["expert"]["ff"]), int(r["top"]), int(g.get("count", 1)),
                                     int(g.get("keep", g.get("count", 1))), int(shared.get("ff", 0)), _lib.ACT_SILU, dtype,
                                     scoring="sigmoid", group_top=2, renormalize=False, weight_scale=float(r.get("scale", 1.0)),
                                     shared_gate=False)
        self.norms = ParallelNorms(E, 2 if self.mlp is not None else 1, cfg.canon_taps, cfg.norm_eps)
        self.w_ff = _zeros(_pad16(self.mlp.n_rows()), E, dtype=dtype) if self.mlp is not None else None

    def _inputs(self, x: Tensor, state, pending, add):
        T, E = x.shape
        dt = self.mixer.w_in.dtype
        hs = [torch.empty(T, E, dtype=dt, device=x.device) for _ in range(self.norms.n)]
        return hs, self.norms(x, hs, state.vectors, pending, add)

    def forward(self, x: Tensor, ip: Tensor, state, kv_cache, pending: Optional[dict], add: Optional[Tensor],
                one_token_kernel: bool):
        """Applies the pending sum of the layer before (and the pass's vector), runs this layer's sublayers on the two
        norms of the result and returns (the stream after the sum, the sublayer results as the next pending sum)."""
        hs, x = self._inputs(x, state, pending, add)
        out = dict(a=self.mixer(hs[0], ip, kv_cache, one_token_kernel))
        if self.mlp is not None:
            out["b"] = self.mlp(_proj(hs[1], self.w_ff), 0, None, hs[1], one_token_kernel)
        return x, out

    def step_one_token(self, x: Tensor, ip: Tensor, state, kv_cache, pending: Optional[dict], add: Optional[Tensor]):
        """The same layer for one token: sum + norms + convolutions in one launch; every product that reads a sublayer
        input in one launch; the mixer's core; the products that close the sublayers in one launch."""
        hs, x = self._inputs(x, state, pending, add)
        jobs, outs = self.mixer.first_jobs(hs[0])
        hp = None
        if self.mlp is not None:
            hp = _out(self.w_ff)
            jobs = jobs + [(hs[1], self.w_ff, hp)]
        seq_ops.gemv_multi(jobs)
        core = self.mixer.finish(outs, ip, kv_cache)
        mixed = _out(self.mixer.w_o)
        closing, result = [(core, self.mixer.w_o, mixed)], None
        if self.mlp is not None:
            more, result = self.mlp.one_token(hp, 0, None, hs[1])
            closing += more
        seq_ops.gemv_multi(closing)
        out = dict(a=mixed)
        if result is not None:
            out["b"] = result()
        return x, out

    def one_token_fits(self) -> bool:
        return self.kind == "attention" or self.mixer.absorbed_fits()


class NevodraLayer(nn.Module):
    """One run of a block: the (possibly shared) weights with this run's own cache and state, and for the first layer
    of a pass the row of the step table that is added to the stream before it."""

    def __init__(self, block: NevodraBlock, shares_weights: bool, step_row: Optional[int]):
        super().__init__()
        if shares_weights:
            object.__setattr__(self, "block", block)    # not registered twice
        else:
            self.block = block
        self.step_row = step_row
        self.state = None
        self.kv_cache = None


# --------------------------------------------------------------------------------------------- the model

class NevodraTransformer(nn.Module):
    """Same runtime surface as `model.Transformer`: setup_caches / reset_caches / forward / min_cache_length /
    get_cache_stats / prompt_cache_overflow, `config.block_size`, `config.n_layer` (the number of layer runs)."""

    supports_prompt_portions = True

    def __init__(self, config: NevodraArgs, dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32)
        self.config, self.dtype = config, dtype
        self.tok_embeddings = _zeros(config.vocab_size, config.dim, dtype=dtype)
        looped = config.loop_stop > config.loop_start
        self.loop_step = _zeros(config.loop_times, config.dim, dtype=torch.float32) if looped else None
        blocks: Dict[int, NevodraBlock] = {}
        layers = []
        for i, t in config.runs():
            fresh = i not in blocks
            if fresh:
                blocks[i] = NevodraBlock(config, config.layers[i], dtype)
            layers.append(NevodraLayer(blocks[i], not fresh, t if (t is not None and i == config.loop_start) else None))
        self.layers = nn.ModuleList(layers)
        self.norm = GroupRMSNorm(config.dim, 1, config.norm_eps)
        self.output = _zeros(config.vocab_size, config.dim, dtype=dtype)
        self.max_batch_size = 1
        self.max_seq_length = 0
        # one-token steps through this package's product kernels and the one-token attention kernels; False = the
        # kernels of a prompt portion of one token (library products), used by A/B tests
        self.fused_decode = True

    def blocks(self):
        """(layer index in the configuration, block) of every distinct block, in running order."""
        seen, out = set(), []
        for (i, _), layer in zip(self.config.runs(), self.layers):
            if i not in seen:
                seen.add(i)
                out.append((i, layer.block))
        return out

    # ---- caches and state -------------------------------------------------------------------------
    def layer_cache_plan(self, cache_kwargs: Dict[str, Any], max_seq_length: int) -> Dict[str, Any]:
        """Per layer run: a windowed layer keeps its first positions and a ring of one window ("recent_global" with the
        kept positions as global tokens; "full" without a window), a latent layer one row per position ("latent"); every
        run also carries the convolution tail ("state")."""
        ck = dict(cache_kwargs or {})
        ck["max_seq_length"] = max_seq_length
        strategies, lengths, kept = [], [], []
        for layer in self.layers:
            m = layer.block.mixer
            if layer.block.kind == "latent_attention":
                strategies.append("latent"); lengths.append(max_seq_length); kept.append(0)
            elif m.window:
                strategies.append("recent_global"); lengths.append(m.window + m.keep_first); kept.append(m.keep_first)
            else:
                strategies.append("full"); lengths.append(max_seq_length); kept.append(0)
        ck["cache_strategy"], ck["max_cache_length"], ck["global_tokens"] = strategies, lengths, kept
        ck["cache_bits"] = None
        ck["prompt_compression_strategy"] = ["none"] * len(self.layers)
        return ck

    def setup_caches(self, **kwargs):
        lengths, kept = kwargs["max_cache_length"], kwargs["global_tokens"]
        state_ctor, _ = get_cache_constructor("state")
        for i, layer in enumerate(self.layers):
            m = layer.block.mixer
            ctor, _ = get_cache_constructor(kwargs["cache_strategy"][i])
            if layer.block.kind == "latent_attention":
                layer.kv_cache = ctor(self.max_batch_size, 1, m.row_width, self.dtype, max_cache_length=int(lengths[i]),
                                      max_seq_length=kwargs.get("max_seq_length"), global_tokens=0, cache_bits=None)
            else:
                layer.kv_cache = ctor(self.max_batch_size, m.kv_heads, m.head_dim, self.dtype, max_cache_length=int(lengths[i]),
                                      max_seq_length=kwargs.get("max_seq_length"), global_tokens=int(kept[i]), cache_bits=None,
                                      v_head_dim=m.v_dim)
            layer.state = state_ctor(self.max_batch_size, 0, 0, state_vectors=max(self.config.canon_taps - 1, 1),
                                     state_width=self.config.dim)
        self.max_seq_length = int(kwargs.get("max_seq_length") or max(lengths))

    def reset_caches(self):
        """Gives back what the finished sequence held: every slot empty, every tail zero."""
        for layer in self.layers:
            layer.state.reset()
            layer.kv_cache.reset()

    def prompt_cache_overflow(self, prompt_length: int):
        return [l.block.kind == "latent_attention" and prompt_length > l.kv_cache.max_cache_length for l in self.layers]

    def min_cache_length(self):
        full = [l.kv_cache.max_cache_length for l in self.layers if l.block.kind == "latent_attention" or not l.block.mixer.window]
        return min(full) if full else self.max_seq_length

    def get_cache_stats(self, prompt_len, gen_len):
        stats, mem = {}, 0.0
        for i, layer in enumerate(self.layers):
            stats[f"cache_slots_{i}"] = float(layer.kv_cache.max_cache_length)
            mem += layer.state.memory_usage() + layer.kv_cache.memory_usage()
        stats["cache_memory_gb"] = mem
        return stats

    # ---- one step: a whole prompt, a portion of it, or one token ----------------------------------
    @torch.no_grad()
    def forward(self, idx: Tensor, input_pos: Tensor, is_prefill: bool = True, mask: Optional[Tensor] = None,
                attn_top_k: Optional[float] = 1.0, logits_at: Optional[Tensor] = None,
                collect: Optional[list] = None) -> Tensor:
        """idx [1, T] token ids, input_pos [T] (or [1]) positions with input_pos[0] the first token's; returns fp32
        logits [1, n, vocab] for the rows `logits_at` (default: the last).  The step continues from the caches and
        state that earlier steps left.  `collect`, if a list, receives the residual stream after every layer run."""
        assert attn_top_k in (None, 1, 1.0), "top-k attention is not part of this design"
        if self.layers[0].state is None:
            raise RuntimeError("Caches must be initialized first")
        tokens = idx.reshape(-1)
        if not tokens.is_cuda:
            raise _lib.CcError("this model runs on CUDA tensors only (no CPU fallback)")
        tokens = tokens if tokens.dtype == torch.int32 else tokens.to(torch.int32)
        ip = input_pos.reshape(-1)[:1]
        ip = ip if ip.dtype == torch.int32 else ip.to(torch.int32)
        T, E, dev = tokens.numel(), self.config.dim, tokens.device
        x = torch.empty(T, E, dtype=torch.float32, device=dev)
        seq_ops.embed_rows(tokens, self.tok_embeddings, x, self.config.embedding_scale)
        pending = None
        one = T == 1 and self.fused_decode and collect is None
        for layer in self.layers:
            add = self.loop_step[layer.step_row] if layer.step_row is not None else None
            if one and layer.block.one_token_fits():
                x, pending = layer.block.step_one_token(x, ip, layer.state, layer.kv_cache, pending, add)
            else:
                x, pending = layer.block(x, ip, layer.state, layer.kv_cache, pending, add, self.fused_decode)
            if collect is not None:
                seq_ops.gated_group_norm(x, None, 1, 0.0, **pending)
                pending = None
                collect.append(x.clone())
        rows = None if logits_at is None else logits_at.to(device=dev, dtype=torch.int64).contiguous()
        if rows is None:
            rows = torch.full((1,), T - 1, dtype=torch.int64, device=dev)
        n = rows.numel()
        xs = torch.empty(n, E, dtype=torch.float32, device=dev)
        xs_act = xs if self.dtype == torch.float32 else torch.empty(n, E, dtype=self.dtype, device=dev)
        self.norm(x, xs, None if xs_act is xs else xs_act, pending, rows=rows)
        if one:
            logits = _out(self.output)
            seq_ops.gemv_multi([(xs_act, self.output, logits)])
            return logits.view(1, 1, -1)
        return _proj(xs_act, self.output).view(1, n, -1)

    def kernels_per_token(self) -> int:
        """Launches of this package's kernels in one decode step (fused_decode)."""
        n = 3   # embedding, last norm, output product
        for layer in self.layers:
            b = layer.block
            n += 3      # sum + norms + convolutions; products of the sublayer inputs; closing products
            # windowed: q/k norm, attention; latent: rows, rotation, 2 per-head products, attention (2 launches)
            n += 2 if b.kind == "attention" else 6
            if isinstance(b.mlp, RoutedExperts):
                n += 4      # router, experts up and down, combination
            elif b.mlp is not None:
                n += 1      # activation
        return n

    # ---- weights --------------------------------------------------------------------------------
    def load_tensors(self, tensors: Dict[str, Tensor]):
        """Fills the parameters from the checkpoint's tensor names ('embed', 'loop.step', 'l<i>.norm1' / '.norm2',
        'l<i>.canon1' / '.canon2', 'l<i>.mix.*', 'l<i>.mlp.*', 'final.norm', 'head'), fusing the rows that read the
        same input."""
        used = set()

        def get(name, shape=None):
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = tensors[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)} does not fit the configuration {tuple(shape)}")
            return t

        def put(param, value):
            param.data.copy_(value.to(param.dtype).reshape(param.shape))

        cfg = self.config
        E, taps = cfg.dim, cfg.canon_taps
        put(self.tok_embeddings, get("embed", (cfg.vocab_size, E)))
        if self.loop_step is not None:
            put(self.loop_step, get("loop.step", (cfg.loop_times, E)).float())
        for i, b in self.blocks():
            p = f"l{i}."
            n = b.norms.n
            put(b.norms.weight, torch.stack([get(f"{p}norm{s + 1}", (E,)).float() for s in range(n)]))
            put(b.norms.conv, torch.stack([get(f"{p}canon{s + 1}", (E, taps)).float() for s in range(n)]))
            m = b.mixer
            if b.kind == "attention":
                put(m.w_in, _padded_rows([get(p + "mix.q", (m.nq, E)), get(p + "mix.k", (m.nk, E)), get(p + "mix.v", (m.nv, E))],
                                         m.w_in.shape[0]))
                put(m.q_norm, get(p + "mix.q.norm", (m.nq,)).float())
                put(m.k_norm, get(p + "mix.k.norm", (m.nk,)).float())
                put(m.dist_a, get(p + "mix.r1", (m.heads,)).float())
                put(m.dist_b, get(p + "mix.r2", (m.heads,)).float())
                put(m.w_o, get(p + "mix.o", (E, m.heads * m.v_dim)))
            else:
                H, D, R, V, C = m.heads, m.head_dim, m.rot_dim, m.v_dim, m.kv_rank
                put(m.w_in, _padded_rows([get(p + "mix.q", (H * (D + R), E)), get(p + "mix.dkv", (C + R, E))], m.w_in.shape[0]))
                put(m.kv_norm, get(p + "mix.dkv.norm", (C,)).float())
                put(m.sink, get(p + "mix.sink", (H,)).float())
                uk, uv = get(p + "mix.uk", (H * D, C)), get(p + "mix.uv", (H * V, C))
                put(m.w_ukv, torch.cat([uk, uv]))
                put(m.w_uk_t, uk.reshape(H, D, C).transpose(1, 2))
                put(m.w_o, get(p + "mix.o", (E, H * V)))
            f = b.mlp
            if isinstance(f, PolyNormMLP):
                put(b.w_ff, _padded_rows([get(p + "mlp.up", (f.ff, E))], b.w_ff.shape[0]))
                put(f.coef, get(p + "mlp.act", (4,)).float())
                put(f.w_down, get(p + "mlp.down", (E, f.ff)))
            elif isinstance(f, RoutedExperts):
                rows = [get(p + "mlp.router", (f.n_real, E))]
                put(f.correction, get(p + "mlp.correction", (f.n_real,)).float())
                if f.shared_ff:
                    rows += [get(p + "mlp.shared.gate", (f.shared_ff, E)), get(p + "mlp.shared.up", (f.shared_ff, E))]
                    put(f.w_shared_down, get(p + "mlp.shared.down", (E, f.shared_ff)))
                put(f.w_gu, torch.stack([torch.cat([get(f"{p}mlp.e{e}.gate", (f.ff, E)), get(f"{p}mlp.e{e}.up", (f.ff, E))])
                                         for e in range(f.n_real)]))
                put(f.w_d, torch.stack([get(f"{p}mlp.e{e}.down", (E, f.ff)) for e in range(f.n_real)]))
                put(b.w_ff, _padded_rows(rows, b.w_ff.shape[0]))
        put(self.norm.weight, get("final.norm", (E,)).float())
        put(self.output, get("head", (cfg.vocab_size, E)))
        return sorted(set(tensors) - used)

    @classmethod
    def from_config(cls, cfg: Dict[str, Any], dtype=torch.bfloat16):
        return cls(NevodraArgs.from_config(cfg), dtype)
