"""Detatar: a decoder-only design whose layers run a mixer and a feed-forward side by side on one grouped RMS norm
(`x <- x + gate1 * mixer(shift(h)) + gate2 * ff(h)`, `h = norm(x)`, gates = sigmoid of a projection of `h`), with a
per-layer token shift in front of the mixer, two kinds of mixer (a matrix-state linear recurrence with per-channel
decay, "wkv", and causal softmax attention through low-rank latents, "latent_attention") and two kinds of
feed-forward (dense gated, and a mixture of experts with grouped top-k routing, identity experts and a gated shared
expert).  A layer may reuse the weights of an earlier layer while keeping a cache and state of its own.

The model plugs into the same runtime as `model.Transformer` and `tidelorn.TidelornTransformer`: `setup_caches`
builds each layer's cache and state through `cache.get_cache_constructor` ("latent" rows for attention layers,
"state" for what every layer carries from token to token), `forward(idx, input_pos, is_prefill)` is what
`generation_utils.prefill` / `decode_one_token` / `GraphedDecoder` call, and a step of any length continues from
what the earlier steps left.  Matrix products of prompt portions are cuBLAS (torch.mm, fp32 accumulation and output);
one-token steps use this package's product kernels; everything between products is a kernel of csrc/seq.  There is
no CPU path.

Precision: weights, cache rows and product inputs are in the compute dtype (bf16 or fp32); the residual stream,
norms, gates, angles, attention scores and weights, router scores, decays and the recurrent state are fp32 in both.

The mechanisms (`GroupRMSNorm`, `TokenShift`, `WkvMixer`, `LatentAttention`, `GatedMLP`, `RoutedExperts`) take their
sizes and constants as arguments so that another design can use them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import _lib, seq_ops
from .cache import get_cache_constructor
from .tidelorn import _mm


def _proj(x: Tensor, w: Tensor) -> Tensor:
    """x [T, K] (compute dtype) times w[N, K]^T -> fp32 [T, N] through cuBLAS (prompt portions; one-token steps batch
    their products through seq_ops.gemv_multi instead)."""
    return _mm(x, w)


def _out(w: Tensor) -> Tensor:
    return torch.empty(1, w.shape[0], dtype=torch.float32, device=w.device)


def _zeros(*shape, dtype):
    return nn.Parameter(torch.zeros(*shape, dtype=dtype), requires_grad=False)


def _pad16(n: int) -> int:
    """Rows of a fused projection are padded to a multiple of 16: the library's fast product kernels want the fp32
    output's row stride aligned, and a router's row count (plus one gate row) is often odd."""
    return (n + 15) // 16 * 16


def _padded_rows(rows, total: int) -> Tensor:
    t = torch.cat(rows)
    return t if t.shape[0] == total else torch.cat([t, t.new_zeros(total - t.shape[0], t.shape[1])])


# --------------------------------------------------------------------------------------------- configuration

MIXERS = ("wkv", "latent_attention")
FEED_FORWARDS = ("dense", "moe")


@dataclass
class DetatarArgs:
    vocab_size: int
    dim: int
    layers: List[Dict[str, Any]]
    norm_eps: float
    norm_groups: int
    embedding_scale: float
    block_size: int = 1 << 20      # rotary angles are computed from the position: no table limits the length
    n_layer: int = field(init=False)

    def __post_init__(self):
        self.n_layer = len(self.layers)
        if self.dim % self.norm_groups:
            raise ValueError(f"norm groups ({self.norm_groups}) must divide the width ({self.dim})")
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            j = layer.get("weights_of")
            if j is not None and not (0 <= int(j) < i and self.layers[int(j)]["type"] == layer["type"]):
                raise ValueError(f"layer {i}: weights_of must name an earlier layer of the same kind")

    @classmethod
    def from_config(cls, cfg: Dict[str, Any]):
        norm = cfg["norm"]
        return cls(vocab_size=int(cfg["vocab"]), dim=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float(norm["eps"]), norm_groups=int(norm.get("groups", 1)),
                   embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)))


# --------------------------------------------------------------------------------------------- mechanisms

class GroupRMSNorm(nn.Module):
    """The vector in `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times a plain weight.
    The kernel also performs the gated residual sum that precedes the norm (`pending`: the sublayer results of the layer
    before with their gate logits and biases), so the stream is read and written once per layer."""

    def __init__(self, dim: int, groups: int, eps: float):
        super().__init__()
        self.groups, self.eps = int(groups), float(eps)
        self.weight = _zeros(dim, dtype=torch.float32)

    def forward(self, x: Tensor, h: Optional[Tensor], h_act: Optional[Tensor], pending: Optional[dict] = None,
                rows: Optional[Tensor] = None):
        seq_ops.gated_group_norm(x, self.weight, self.groups, self.eps, h, h_act, rows=rows, **(pending or {}))


def apply_pending(x: Tensor, pending: Optional[dict]):
    """x += the pending gated sublayer results, without a norm."""
    if pending:
        seq_ops.gated_group_norm(x, None, 1, 0.0, **pending)


class TokenShift(nn.Module):
    """n mixes of each row with the row of the previous token: h + (h_prev - h) * mu[s].  The previous row of a step's
    first token is the sequence's state vector, which the step then replaces by its last row."""

    def __init__(self, dim: int, n: int = 1):
        super().__init__()
        self.n = n
        self.mu = _zeros(n, dim, dtype=torch.float32)

    def forward(self, h: Tensor, state: Tensor, out: Optional[Tensor], outf: Optional[Tensor] = None):
        seq_ops.token_shift(h, state, self.mu, out, outf)


class WkvMixer(nn.Module):
    """Matrix-state linear recurrence: five token-shift mixes feed the receptance, key, value, gate and decay
    projections; per head `o_t = (S + diag(u) k_t v_t^T)^T r_t`, `S <- diag(w_t) S + k_t v_t^T` with
    `w_t = exp(-exp(W2 tanh(W1 mix_w) + w0))`; each head's output is divided by its RMS, scaled, gated by silu(g) and
    projected.  State per sequence: the previous input row and S (fp32)."""

    state_vectors = 2          # [0] the layer's shift, [1] this mixer's

    def __init__(self, dim: int, heads: int, head_dim: int, decay_rank: int, eps: float, dtype):
        super().__init__()
        self.dim, self.heads, self.head_dim, self.eps = dim, heads, head_dim, eps
        hd = heads * head_dim
        self.shift = TokenShift(dim, 5)                      # r, k, v, g, w
        self.w_r, self.w_k, self.w_v, self.w_g = (_zeros(hd, dim, dtype=dtype) for _ in range(4))
        self.w_w1 = _zeros(decay_rank, dim, dtype=dtype)
        self.w_w2 = _zeros(hd, decay_rank, dtype=dtype)
        self.w0 = _zeros(hd, dtype=torch.float32)
        self.u = _zeros(hd, dtype=torch.float32)
        self.norm_w = _zeros(hd, dtype=torch.float32)
        self.w_o = _zeros(dim, hd, dtype=dtype)

    def first_jobs(self, mixes: Tensor):
        """One token: the five input products as jobs of one launch; returns (jobs, their outputs)."""
        ws = (self.w_r, self.w_k, self.w_v, self.w_g, self.w_w1)
        outs = [_out(w) for w in ws]
        return [(mixes[i], w, o) for i, (w, o) in enumerate(zip(ws, outs))], outs

    def finish(self, outs, state) -> Tensor:
        """One token, after the input products: decay product (tanh applied while its input is staged), recurrence, head
        norm and gate; returns the input of the output product."""
        r, k, v, g, low = outs
        H, D = self.heads, self.head_dim
        wraw = _out(self.w_w2)
        seq_ops.gemv_multi([(low, self.w_w2, wraw, _lib.ACT_TANH, 0, -1)])
        o = torch.empty(1, H * D, dtype=torch.float32, device=r.device)
        seq_ops.wkv(r, k, v, wraw, self.w0, self.u, state.matrix, o, H, D)
        on = torch.empty(1, H * D, dtype=self.w_o.dtype, device=r.device)
        seq_ops.head_norm_gate(o, g, self.norm_w, on, H, D, self.eps)
        return on

    def forward(self, hs: Tensor, state, one_token_kernel: bool = True) -> Tensor:
        """hs fp32 [T, dim] (the shifted layer input) -> fp32 [T, dim]."""
        T, dev, dt = hs.shape[0], hs.device, self.w_r.dtype
        H, D = self.heads, self.head_dim
        mixes = torch.empty(5, T, self.dim, dtype=dt, device=dev)
        self.shift(hs, state.vectors[1], mixes)
        r, k, v, g = (_proj(mixes[i], w) for i, w in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)))
        low = _proj(mixes[4], self.w_w1)
        low_act = torch.empty(T, low.shape[1], dtype=dt, device=dev)
        seq_ops.gated_unit(low, 0, -1, low_act, _lib.ACT_TANH)
        wraw = _proj(low_act, self.w_w2)
        o = torch.empty(T, H * D, dtype=torch.float32, device=dev)
        seq_ops.wkv(r, k, v, wraw, self.w0, self.u, state.matrix, o, H, D)
        on = torch.empty(T, H * D, dtype=dt, device=dev)
        seq_ops.head_norm_gate(o, g, self.norm_w, on, H, D, self.eps)
        return _proj(on, self.w_o)


class LatentAttention(nn.Module):
    """Causal softmax attention whose keys and values are up-projections of one cached latent per position.
    Queries: `q = W_uq rms_norm(W_dq h)` (or, with `q_rank == 0`, one full-rank projection `q = W_q h`), per head
    [dim unrotated | rot_dim rotated].  Keys: per head `[W_uk c | rot(k_r)]` with `c = rms_norm(first kv_rank rows of
    W_dkv h)` and `k_r` the last rot_dim rows, shared by all heads; values `W_uv c`.  Options: `gated` multiplies each
    head's output by sigmoid of one row of `W_g h`; `sink` adds exp of a learned logit per head to the softmax
    denominator; `interleaved` pairs rotary dimensions (2i, 2i + 1) instead of (i, i + dims / 2).

    Only `[c | rot(k_r)]` is cached.  A prompt portion up-projects the cached latents of the earlier positions
    (tensor-core product) and attends over per-head rows; a single token uses the absorbed form instead: the query
    is carried through `W_uk^T` so that all heads attend over the latent rows themselves, and `W_uv` is applied to
    the attention-weighted latent."""

    def __init__(self, dim: int, heads: int, head_dim: int, rot_dim: int, v_dim: int, q_rank: int, kv_rank: int,
                 scale: float, rot_base: float, rot_dims: int, eps: float, dtype, gated: bool = True, sink: bool = False,
                 interleaved: bool = False):
        super().__init__()
        if rot_dims > rot_dim or rot_dims % 2:
            raise ValueError("rotary dims must be even and at most the rotated width")
        self.dim, self.heads, self.head_dim, self.rot_dim, self.v_dim = dim, heads, head_dim, rot_dim, v_dim
        self.q_rank, self.kv_rank, self.scale, self.rot_dims, self.eps = q_rank, kv_rank, float(scale), rot_dims, eps
        self.gated, self.interleaved = bool(gated), bool(interleaved)
        # rows of the fused input projection: query part (down-projection, or all query heads when q_rank == 0) | dkv | g | padding
        self.q_rows = q_rank if q_rank else heads * (head_dim + rot_dim)
        self.w_in = _zeros(_pad16(self.q_rows + kv_rank + rot_dim + (heads if gated else 0)), dim, dtype=dtype)
        self.q_norm = _zeros(q_rank, dtype=torch.float32) if q_rank else None
        self.kv_norm = _zeros(kv_rank, dtype=torch.float32)
        self.sink = _zeros(heads, dtype=torch.float32) if sink else None
        self.w_uq = _zeros(heads * (head_dim + rot_dim), q_rank, dtype=dtype) if q_rank else None
        self.w_ukv = _zeros(heads * (head_dim + v_dim), kv_rank, dtype=dtype)           # rows: uk (H * dim) | uv (H * vdim)
        self.w_uk_t = _zeros(heads, kv_rank, head_dim, dtype=dtype)                    # per head W_uk^T, for the absorbed query
        self.w_o = _zeros(dim, heads * v_dim, dtype=dtype)
        i = torch.arange(0, max(rot_dims // 2, 1), dtype=torch.float64)
        self.register_buffer("inv_freq", torch.pow(torch.tensor(float(rot_base), dtype=torch.float64),
                                                   -2.0 * i / max(rot_dims, 1)).to(torch.float32), persistent=False)

    @property
    def row_width(self):
        return self.kv_rank + self.rot_dim

    def absorbed_fits(self) -> bool:
        """The one-token kernel stages 40 rows in shared memory: rows of up to 1280 columns."""
        return self.row_width <= 1280 and self.kv_rank <= 1024

    def first_jobs(self, hs_act: Tensor):
        a = _out(self.w_in)
        return [(hs_act, self.w_in, a)], [a]

    def finish(self, outs, ip: Tensor, cache) -> Tensor:
        """One token, absorbed form, after the down-projections: rows, query up-projection, rotation, the query through
        W_uk^T, attention over the latent rows (the new row is stored), W_uv and the head gates on the weighted latent;
        returns the input of the output product."""
        (a,) = outs
        dev, dt = a.device, self.w_in.dtype
        H, D, R, V, C, Q = self.heads, self.head_dim, self.rot_dim, self.v_dim, self.kv_rank, self.q_rows
        cq = torch.empty(1, self.q_rank, dtype=dt, device=dev) if self.q_rank else None
        krow = torch.empty(1, 1, C + R, dtype=dt, device=dev)
        seq_ops.latent_prepare(a, 0, self.q_rank, Q, C, R, self.rot_dims, self.q_norm, self.kv_norm,
                               self.inv_freq, ip, cq, krow, None, self.eps, self.interleaved)
        if self.q_rank:
            q = _out(self.w_uq)
            seq_ops.gemv_multi([(cq, self.w_uq, q)])
        else:
            q = a[:, :Q]      # the query heads are columns of the fused projection (fp32), rotated in place
        qf = torch.empty(1, H, C + R, dtype=torch.float32, device=dev)
        seq_ops.rope_heads(q, ip, self.inv_freq, H, D + R, D, R, self.rot_dims, tail=qf, tail_off=C, interleaved=self.interleaved)
        seq_ops.head_gemv(self.w_uk_t, q, D + R, qf, C + R)
        ctx = torch.empty(1, H, C, dtype=dt, device=dev)
        cache.latent_step(qf, krow, ip, ctx, self.scale, sink=self.sink)
        y = torch.empty(1, H * V, dtype=dt, device=dev)
        seq_ops.head_gemv(self.w_ukv[H * D:].view(H, V, C), ctx, C, y, V,
                          gate=a[0, Q + C + R:Q + C + R + H] if self.gated else None)
        return y

    def forward(self, hs_act: Tensor, ip: Tensor, cache, one_token_kernel: bool = True) -> Tensor:
        T, dev, dt = hs_act.shape[0], hs_act.device, self.w_in.dtype
        H, D, R, V, C = self.heads, self.head_dim, self.rot_dim, self.v_dim, self.kv_rank
        if T == 1 and one_token_kernel and self.absorbed_fits():
            jobs, outs = self.first_jobs(hs_act)
            seq_ops.gemv_multi(jobs)
            y, out = self.finish(outs, ip, cache), _out(self.w_o)
            seq_ops.gemv_multi([(y, self.w_o, out)])
            return out
        Q = self.q_rows
        a = _proj(hs_act, self.w_in)
        cq = torch.empty(T, self.q_rank, dtype=dt, device=dev) if self.q_rank else None
        krow = torch.empty(T, 1, C + R, dtype=dt, device=dev)
        lat_new = torch.empty(T, C, dtype=dt, device=dev)     # contiguous latents for the up-projection
        seq_ops.latent_prepare(a, 0, self.q_rank, Q, C, R, self.rot_dims, self.q_norm, self.kv_norm,
                               self.inv_freq, ip, cq, krow, lat_new, self.eps, self.interleaved)
        q = _proj(cq, self.w_uq) if self.q_rank else a[:, :Q].contiguous()             # fp32 [T, H * (D + R)]
        gate = a[:, Q + C + R:Q + C + R + H]
        p0 = int(ip.item())      # a prompt portion sizes its expanded rows on the host (one read per layer step)
        seq_ops.rope_heads(q, ip, self.inv_freq, H, D + R, D, R, self.rot_dims, interleaved=self.interleaved)
        kv_new = _mm(lat_new, self.w_ukv)
        k_new = torch.empty(T, H, D + R, dtype=dt, device=dev)
        v_new = torch.empty(T, H, V, dtype=dt, device=dev)
        if p0 > 0:
            lat_old = cache.latent_rows(p0)
            kv_old = _mm(lat_old[:, :C].contiguous(), self.w_ukv)
            k_old = torch.empty(H, p0, D + R, dtype=dt, device=dev)
            v_old = torch.empty(H, p0, V, dtype=dt, device=dev)
            pos_old = cache.pos[0, 0, :p0]
        else:
            lat_old = kv_old = k_old = v_old = pos_old = None
        seq_ops.latent_expand(kv_old, kv_new, lat_old, krow.view(T, C + R), k_old, v_old, k_new, v_new, H, D, V, R, C)
        y = torch.empty(T, H, V, dtype=dt, device=dev)
        seq_ops.attention_rows(q.view(T, H, D + R), k_new, v_new, k_old, v_old, pos_old, ip, y, self.scale, sink=self.sink)
        cache.sequence_append(krow, ip)
        if self.gated:
            seq_ops.head_gate(y, gate)
        return _proj(y.view(T, H * V), self.w_o)


class GatedMLP(nn.Module):
    """down(act(gate h) * (up h)).  Its gate and up rows are part of the layer's fused projection of h."""

    def __init__(self, dim: int, ff: int, act: int, dtype):
        super().__init__()
        self.ff, self.act = int(ff), int(act)
        self.w_down = _zeros(dim, self.ff, dtype=dtype)

    def n_rows(self):
        return 2 * self.ff

    def forward(self, hp: Tensor, off: int, h: Tensor, h_act: Tensor, one_token_kernel: bool = True) -> Tensor:
        act = torch.empty(hp.shape[0], self.ff, dtype=self.w_down.dtype, device=hp.device)
        seq_ops.gated_unit(hp, off, off + self.ff, act, self.act)
        return _proj(act, self.w_down)

    def one_token(self, hp: Tensor, off: int, h: Tensor, h_act: Tensor):
        """-> (jobs for the layer's closing launch, function that returns the result after it): the gated unit is applied
        while the down-projection stages its input."""
        out = _out(self.w_down)
        return [(hp, self.w_down, out, self.act, off, off + self.ff)], lambda: out


class RoutedExperts(nn.Module):
    """Mixture of experts.  Router scores = softmax over all router outputs; the choice adds a correction to the score;
    outputs form equal groups of neighbours of which only the best `keep` (by their largest choice) can be chosen; the
    `top` largest choices win and are weighted by their scores divided by their sum.  The last `identity` outputs are
    identity experts (the input itself).  A shared expert runs for every token, times sigmoid of one projection row.
    Its router, shared-gate and shared gate/up rows are part of the layer's fused projection of h.  Options: `scoring`
    "sigmoid" scores every output on its own instead of the softmax; `group_top` makes a group's score the sum of its
    that many largest choices instead of the largest; `renormalize=False` keeps the chosen scores as weights;
    `weight_scale` multiplies the weights; `shared_gate=False` adds the shared expert without a gate.

    Steps of up to `small_t` tokens run the chosen experts through a kernel that reads the ids on the device (no host
    round trip: a decode step stays capturable); longer portions group the (token, choice) pairs by expert, read the
    group sizes once and run one product pair per expert."""

    small_t = 4

    def __init__(self, dim: int, n_experts: int, n_identity: int, ff: int, top: int, groups: int, keep: int,
                 shared_ff: int, act: int, dtype, scoring: str = "softmax", group_top: int = 1, renormalize: bool = True,
                 weight_scale: float = 1.0, shared_gate: bool = True):
        super().__init__()
        self.dim, self.n_real, self.n_identity, self.ff, self.top = dim, int(n_experts), int(n_identity), int(ff), int(top)
        self.groups, self.keep, self.shared_ff, self.act = int(groups), int(keep), int(shared_ff), int(act)
        if (self.n_real + self.n_identity) % self.groups:
            raise ValueError("router outputs must split into equal groups")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown router scoring {scoring!r}")
        self.sigmoid_scores, self.group_top, self.renormalize = scoring == "sigmoid", int(group_top), bool(renormalize)
        self.weight_scale, self.sg_rows = float(weight_scale), (1 if shared_gate and self.shared_ff else 0)
        self.correction = _zeros(self.n_real + self.n_identity, dtype=torch.float32)
        self.w_gu = _zeros(self.n_real, 2 * self.ff, dim, dtype=dtype)      # per expert: gate rows | up rows
        self.w_d = _zeros(self.n_real, dim, self.ff, dtype=dtype)
        self.w_shared_down = _zeros(dim, self.shared_ff, dtype=dtype) if self.shared_ff else None

    def n_rows(self):
        return self.n_real + self.n_identity + ((self.sg_rows + 2 * self.shared_ff) if self.shared_ff else 0)

    def _route(self, hp: Tensor, off: int):
        T, dev = hp.shape[0], hp.device
        n = self.n_real + self.n_identity
        ids = torch.empty(T, self.top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, self.top, dtype=torch.float32, device=dev)
        seq_ops.moe_route(hp[:, off:off + n], self.correction, ids, wts, self.groups, self.keep, self.top,
                          self.sigmoid_scores, self.group_top, self.renormalize, self.weight_scale)
        return ids, wts

    def _few_tokens(self, h_act: Tensor, ids: Tensor):
        M = ids.numel()
        act = torch.empty(M, self.ff, dtype=self.w_gu.dtype, device=ids.device)
        y = torch.empty(M, self.dim, dtype=torch.float32, device=ids.device)
        seq_ops.moe_expert_tokens(self.w_gu, self.w_d, h_act, ids, act, y, self.act)
        return y

    def _combine(self, ids, wts, slot, y, h, shared, sg):
        out = torch.empty(ids.shape[0], self.dim, dtype=torch.float32, device=ids.device)
        seq_ops.moe_combine(ids, wts, slot, y, h, shared, sg, out, self.n_real)
        return out

    def one_token(self, hp: Tensor, off: int, h: Tensor, h_act: Tensor):
        """-> (jobs for the layer's closing launch, function that returns the result after it)."""
        n = self.n_real + self.n_identity
        ids, wts = self._route(hp, off)
        y = self._few_tokens(h_act, ids)
        jobs, shared, sg = [], None, None
        if self.shared_ff:
            g0 = off + n + self.sg_rows
            shared, sg = _out(self.w_shared_down), (hp[:, off + n:off + n + 1] if self.sg_rows else None)
            jobs.append((hp, self.w_shared_down, shared, self.act, g0, g0 + self.shared_ff))
        return jobs, lambda: self._combine(ids, wts, None, y, h, shared, sg)

    def forward(self, hp: Tensor, off: int, h: Tensor, h_act: Tensor, one_token_kernel: bool = True) -> Tensor:
        T, dev, dt = hp.shape[0], hp.device, self.w_gu.dtype
        n, E, F, top = self.n_real + self.n_identity, self.dim, self.ff, self.top
        ids, wts = self._route(hp, off)
        shared = sg = None
        if self.shared_ff:
            g0 = off + n + self.sg_rows
            sg = hp[:, off + n:off + n + 1] if self.sg_rows else None
            act = torch.empty(T, self.shared_ff, dtype=dt, device=dev)
            seq_ops.gated_unit(hp, g0, g0 + self.shared_ff, act, self.act)
            shared = _proj(act, self.w_shared_down)
        M = T * top
        if T <= self.small_t:
            y, slot = self._few_tokens(h_act, ids), None
        else:
            counts = torch.empty(self.n_real, dtype=torch.int32, device=dev)
            slot = torch.empty(M, dtype=torch.int32, device=dev)
            perm = torch.empty(M, dtype=torch.int32, device=dev)
            seq_ops.moe_group(ids, self.n_real, counts, slot, perm)
            sizes = counts.tolist()
            rows = sum(sizes)
            y = torch.empty(max(rows, 1), E, dtype=torch.float32, device=dev)
            if rows:
                xs = torch.empty(rows, E, dtype=dt, device=dev)
                seq_ops.gather_rows(h_act, perm, xs, rows)
                lo = 0
                for e, cnt in enumerate(sizes):
                    if cnt:
                        gu = _mm(xs[lo:lo + cnt], self.w_gu[e])
                        act = torch.empty(cnt, F, dtype=dt, device=dev)
                        seq_ops.gated_unit(gu, 0, F, act, self.act)
                        y[lo:lo + cnt] = _mm(act, self.w_d[e])
                        lo += cnt
        return self._combine(ids, wts, slot, y, h, shared, sg)


# --------------------------------------------------------------------------------------------- a layer

class DetatarBlock(nn.Module):
    """The weights of one layer: norm, shift, the fused projection of h (residual gates and the feed-forward's input
    rows), the mixer and the feed-forward."""

    def __init__(self, cfg: DetatarArgs, layer: Dict[str, Any], dtype):
        super().__init__()
        E, m, mlp = cfg.dim, layer["mixer"], layer.get("mlp")
        self.kind = layer["type"]
        self.norm1 = GroupRMSNorm(E, cfg.norm_groups, cfg.norm_eps)
        self.shift = TokenShift(E, 1)
        if self.kind == "wkv":
            # the rank of the decay's low-rank projection is a tensor shape: load_tensors sizes those two parameters
            self.mixer = WkvMixer(E, int(m["heads"]), int(m["dim"]), int(m.get("decay_rank", 0)), cfg.norm_eps, dtype)
        else:
            rot = m.get("rot") or {}
            self.mixer = LatentAttention(E, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["q_rank"]),
                                         int(m["kv_rank"]), float(m["scale"]), float(rot.get("base", 10000.0)),
                                         int(rot.get("dims", m["rot_dim"])), cfg.norm_eps, dtype)
        if not mlp:
            self.mlp = None
        elif mlp["kind"] == "dense":
            self.mlp = GatedMLP(E, int(mlp["ff"]), _lib.ACT_GELU_TANH, dtype)
        else:
            r, shared = mlp["router"], mlp.get("shared") or {}
            g = r.get("groups") or {}
            self.mlp = RoutedExperts(E, int(r["experts"]), int(r.get("identity", 0)), int(mlp["expert"]["ff"]), int(r["top"]),
                                     int(g.get("count", 1)), int(g.get("keep", g.get("count", 1))), int(shared.get("ff", 0)),
                                     _lib.ACT_SILU, dtype)
        n_gate = 2 * E if self.mlp is not None else E
        self.w_h = _zeros(_pad16(n_gate + (self.mlp.n_rows() if self.mlp is not None else 0)), E, dtype=dtype)   # rg1 | rg2 | mlp rows | padding
        self.rg1_b = _zeros(E, dtype=torch.float32)
        self.rg2_b = _zeros(E, dtype=torch.float32) if self.mlp is not None else None

    def forward(self, x: Tensor, ip: Tensor, state, kv_cache, pending: Optional[dict], one_token_kernel: bool) -> dict:
        """Applies the pending sum of the layer before, runs this layer's sublayers on the norm of the result and
        returns them as the next pending sum (the stream itself is updated by whoever norms it next)."""
        T, E = x.shape
        dev, dt = x.device, self.w_h.dtype
        h = torch.empty(T, E, dtype=torch.float32, device=dev)
        h_act = h if dt == torch.float32 else torch.empty(T, E, dtype=dt, device=dev)
        self.norm1(x, h, None if h_act is h else h_act, pending)
        if self.kind == "wkv":
            hs = torch.empty(T, E, dtype=torch.float32, device=dev)
            self.shift(h, state.vectors[0], None, hs)
            mixed = self.mixer(hs, state, one_token_kernel)
        else:
            hs_act = torch.empty(T, E, dtype=dt, device=dev)
            self.shift(h, state.vectors[0], hs_act)
            mixed = self.mixer(hs_act, ip, kv_cache, one_token_kernel)
        hp = _proj(h_act, self.w_h)
        out = dict(a=mixed, ga=hp[:, :E], ba=self.rg1_b)
        if self.mlp is not None:
            out.update(b=self.mlp(hp, 2 * E, h, h_act, one_token_kernel), gb=hp[:, E:2 * E], bb=self.rg2_b)
        return out


    def step_one_token(self, x: Tensor, ip: Tensor, state, kv_cache, pending: Optional[dict]) -> dict:
        """The same layer for one token in four kinds of launch: norm with both token shifts; all products that read the
        normed row or its shifted copies; the mixer's core; the products that close the sublayers."""
        E, dev, dt = x.shape[1], x.device, self.w_h.dtype
        h = torch.empty(1, E, dtype=torch.float32, device=dev)
        h_act = h if dt == torch.float32 else torch.empty(1, E, dtype=dt, device=dev)
        if self.kind == "wkv":
            shifted = torch.empty(5, 1, E, dtype=dt, device=dev)
            shift = (state.vectors[0], self.shift.mu, None, state.vectors[1], self.mixer.shift.mu, shifted)
        else:
            shifted = torch.empty(1, E, dtype=dt, device=dev)
            shift = (state.vectors[0], self.shift.mu, shifted, None, None, None)
        seq_ops.gated_group_norm(x, self.norm1.weight, self.norm1.groups, self.norm1.eps, h, None if h_act is h else h_act,
                                 shift=shift, **(pending or {}))
        hp = _out(self.w_h)
        jobs, outs = self.mixer.first_jobs(shifted)
        seq_ops.gemv_multi([(h_act, self.w_h, hp)] + jobs)
        core = self.mixer.finish(outs, state) if self.kind == "wkv" else self.mixer.finish(outs, ip, kv_cache)
        mixed = _out(self.mixer.w_o)
        closing, result = [(core, self.mixer.w_o, mixed)], None
        if self.mlp is not None:
            more, result = self.mlp.one_token(hp, 2 * E, h, h_act)
            closing += more
        seq_ops.gemv_multi(closing)
        out = dict(a=mixed, ga=hp[:, :E], ba=self.rg1_b)
        if result is not None:
            out.update(b=result(), gb=hp[:, E:2 * E], bb=self.rg2_b)
        return out

    def one_token_fits(self) -> bool:
        return self.kind == "wkv" or self.mixer.absorbed_fits()


class DetatarLayer(nn.Module):
    """One run of a block: the (possibly shared) weights with this layer's own cache and state."""

    def __init__(self, block: DetatarBlock, shares_weights: bool):
        super().__init__()
        if shares_weights:
            object.__setattr__(self, "block", block)    # not registered twice
        else:
            self.block = block
        self.state = None
        self.kv_cache = None


# --------------------------------------------------------------------------------------------- the model

class DetatarTransformer(nn.Module):
    """Same runtime surface as `model.Transformer`: setup_caches / reset_caches / forward / min_cache_length /
    get_cache_stats / prompt_cache_overflow, `config.block_size`, `config.n_layer`."""

    supports_prompt_portions = True

    def __init__(self, config: DetatarArgs, dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32)
        self.config, self.dtype = config, dtype
        self.tok_embeddings = _zeros(config.vocab_size, config.dim, dtype=dtype)
        layers = []
        for i, layer in enumerate(config.layers):
            j = layer.get("weights_of")
            layers.append(DetatarLayer(layers[int(j)].block, True) if j is not None
                          else DetatarLayer(DetatarBlock(config, layer, dtype), False))
        self.layers = nn.ModuleList(layers)
        self.norm = GroupRMSNorm(config.dim, config.norm_groups, config.norm_eps)
        self.output = _zeros(config.vocab_size, config.dim, dtype=dtype)
        self.max_batch_size = 1
        self.max_seq_length = 0
        # one-token steps through this package's product kernels and the absorbed attention; False = the kernels of a
        # prompt portion of one token (library products, expanded attention rows), used by A/B tests
        self.fused_decode = True

    # ---- caches and state -------------------------------------------------------------------------
    def layer_cache_plan(self, cache_kwargs: Dict[str, Any], max_seq_length: int) -> Dict[str, Any]:
        """An attention layer keeps one latent row per position ("latent", max_seq_length slots); every layer carries
        fixed-size state ("state"): its token-shift row, and for a recurrent mixer a second row and the matrix."""
        ck = dict(cache_kwargs or {})
        ck["max_seq_length"] = max_seq_length
        ck["cache_strategy"] = ["latent" if l.block.kind == "latent_attention" else "state" for l in self.layers]
        ck["max_cache_length"] = [max_seq_length if l.block.kind == "latent_attention" else 0 for l in self.layers]
        ck["global_tokens"] = 0
        ck["cache_bits"] = None
        ck["prompt_compression_strategy"] = ["none"] * len(self.layers)
        return ck

    def setup_caches(self, **kwargs):
        lengths = kwargs["max_cache_length"]
        state_ctor, _ = get_cache_constructor("state")
        for i, layer in enumerate(self.layers):
            mixer = layer.block.mixer
            if layer.block.kind == "latent_attention":
                ctor, _ = get_cache_constructor(kwargs["cache_strategy"][i])
                layer.kv_cache = ctor(self.max_batch_size, 1, mixer.row_width, self.dtype,
                                      max_cache_length=int(lengths[i]), max_seq_length=kwargs.get("max_seq_length"),
                                      global_tokens=0, cache_bits=None)
                layer.state = state_ctor(self.max_batch_size, 0, 0, state_vectors=1, state_width=self.config.dim)
            else:
                layer.kv_cache = None
                layer.state = state_ctor(self.max_batch_size, mixer.heads, mixer.head_dim, state_vectors=mixer.state_vectors,
                                         state_width=self.config.dim)
        self.max_seq_length = int(kwargs.get("max_seq_length") or max(lengths))

    def reset_caches(self):
        """Gives back what the finished sequence held: every slot empty, every state zero."""
        for layer in self.layers:
            layer.state.reset()
            if layer.kv_cache is not None:
                layer.kv_cache.reset()

    def prompt_cache_overflow(self, prompt_length: int):
        return [l.kv_cache is not None and prompt_length > l.kv_cache.max_cache_length for l in self.layers]

    def min_cache_length(self):
        full = [l.kv_cache.max_cache_length for l in self.layers if l.kv_cache is not None]
        return min(full) if full else self.max_seq_length

    def get_cache_stats(self, prompt_len, gen_len):
        stats, mem = {}, 0.0
        for i, layer in enumerate(self.layers):
            stats[f"cache_slots_{i}"] = float(layer.kv_cache.max_cache_length if layer.kv_cache is not None else 0)
            mem += layer.state.memory_usage() + (layer.kv_cache.memory_usage() if layer.kv_cache is not None else 0.0)
        stats["cache_memory_gb"] = mem
        return stats

    # ---- one step: a whole prompt, a portion of it, or one token ----------------------------------
    @torch.no_grad()
    def forward(self, idx: Tensor, input_pos: Tensor, is_prefill: bool = True, mask: Optional[Tensor] = None,
                attn_top_k: Optional[float] = 1.0, logits_at: Optional[Tensor] = None,
                collect: Optional[list] = None) -> Tensor:
        """idx [1, T] token ids, input_pos [T] (or [1]) positions with input_pos[0] the first token's; returns fp32
        logits [1, n, vocab] for the rows `logits_at` (default: the last).  The step continues from the caches and
        state that earlier steps left.  `collect`, if a list, receives the residual stream after every layer."""
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
        fused = self.fused_decode
        x = torch.empty(T, E, dtype=torch.float32, device=dev)
        seq_ops.embed_rows(tokens, self.tok_embeddings, x, self.config.embedding_scale)
        pending = None
        one = T == 1 and fused and collect is None
        for layer in self.layers:
            if one and layer.block.one_token_fits():
                pending = layer.block.step_one_token(x, ip, layer.state, layer.kv_cache, pending)
            else:
                pending = layer.block(x, ip, layer.state, layer.kv_cache, pending, fused)
            if collect is not None:
                apply_pending(x, pending)
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
            n += 3      # norm with the token shifts; products of the normed row and its copies; closing products
            # recurrent: decay product, recurrence, head norm; latent: rows, query product, rotation, 2 per-head
            # products, attention (2 launches)
            n += 3 if b.kind == "wkv" else 7
            if isinstance(b.mlp, RoutedExperts):
                n += 4      # router, experts up and down, combination
        return n

    # ---- weights --------------------------------------------------------------------------------
    def load_tensors(self, tensors: Dict[str, Tensor]):
        """Fills the parameters from the checkpoint's tensor names ('embed', 'l<i>.norm1', '.shift', '.rg1' (+ '.b'),
        '.rg2', 'l<i>.mix.*', 'l<i>.mlp.*', 'final.norm', 'head'), fusing the rows that read the same input."""
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
        E = cfg.dim
        put(self.tok_embeddings, get("embed", (cfg.vocab_size, E)))
        for i, layer in enumerate(self.layers):
            if cfg.layers[i].get("weights_of") is not None:
                continue
            b, p = layer.block, f"l{i}."
            put(b.norm1.weight, get(p + "norm1", (E,)).float())
            put(b.shift.mu, get(p + "shift", (E,)).float())
            put(b.rg1_b, get(p + "rg1.b", (E,)).float())
            rows_h = [get(p + "rg1", (E, E))]
            m = b.mixer
            if b.kind == "wkv":
                hd = m.heads * m.head_dim
                put(m.shift.mu, torch.stack([get(p + "mix.mu." + s, (E,)).float() for s in "rkvgw"]))
                for s in "rkvg":
                    put(getattr(m, "w_" + s), get(p + "mix." + s, (hd, E)))
                rank = get(p + "mix.w1").shape[0]
                if m.w_w1.shape[0] != rank:
                    m.w_w1 = _zeros(rank, E, dtype=m.w_w1.dtype).to(m.w_w1.device)
                    m.w_w2 = _zeros(hd, rank, dtype=m.w_w2.dtype).to(m.w_w2.device)
                put(m.w_w1, get(p + "mix.w1", (rank, E)))
                put(m.w_w2, get(p + "mix.w2", (hd, rank)))
                put(m.w0, get(p + "mix.w0", (hd,)).float())
                put(m.u, get(p + "mix.u").float().reshape(-1))
                put(m.norm_w, get(p + "mix.norm", (hd,)).float())
                put(m.w_o, get(p + "mix.o", (E, hd)))
            else:
                H, D, R, V, C = m.heads, m.head_dim, m.rot_dim, m.v_dim, m.kv_rank
                put(m.w_in, _padded_rows([get(p + "mix.dq", (m.q_rank, E)), get(p + "mix.dkv", (C + R, E)), get(p + "mix.g", (H, E))],
                                         m.w_in.shape[0]))
                put(m.q_norm, get(p + "mix.dq.norm", (m.q_rank,)).float())
                put(m.kv_norm, get(p + "mix.dkv.norm", (C,)).float())
                put(m.w_uq, get(p + "mix.uq", (H * (D + R), m.q_rank)))
                uk, uv = get(p + "mix.uk", (H * D, C)), get(p + "mix.uv", (H * V, C))
                put(m.w_ukv, torch.cat([uk, uv]))
                put(m.w_uk_t, uk.reshape(H, D, C).transpose(1, 2))
                put(m.w_o, get(p + "mix.o", (E, H * V)))
            f = b.mlp
            if f is not None:
                put(b.rg2_b, get(p + "rg2.b", (E,)).float())
                rows_h.append(get(p + "rg2", (E, E)))
            if isinstance(f, GatedMLP):
                rows_h += [get(p + "mlp.gate", (f.ff, E)), get(p + "mlp.up", (f.ff, E))]
                put(f.w_down, get(p + "mlp.down", (E, f.ff)))
            elif isinstance(f, RoutedExperts):
                n = f.n_real + f.n_identity
                rows_h.append(get(p + "mlp.router", (n, E)))
                put(f.correction, get(p + "mlp.correction", (n,)).float())
                if f.shared_ff:
                    rows_h += [get(p + "mlp.shared.sg", (1, E)), get(p + "mlp.shared.gate", (f.shared_ff, E)),
                               get(p + "mlp.shared.up", (f.shared_ff, E))]
                    put(f.w_shared_down, get(p + "mlp.shared.down", (E, f.shared_ff)))
                put(f.w_gu, torch.stack([torch.cat([get(f"{p}mlp.e{e}.gate", (f.ff, E)), get(f"{p}mlp.e{e}.up", (f.ff, E))])
                                         for e in range(f.n_real)]))
                put(f.w_d, torch.stack([get(f"{p}mlp.e{e}.down", (E, f.ff)) for e in range(f.n_real)]))
            put(b.w_h, _padded_rows(rows_h, b.w_h.shape[0]))
        put(self.norm.weight, get("final.norm", (E,)).float())
        put(self.output, get("head", (cfg.vocab_size, E)))
        return sorted(set(tensors) - used)

    @classmethod
    def from_config(cls, cfg: Dict[str, Any], dtype=torch.bfloat16):
        return cls(DetatarArgs.from_config(cfg), dtype)
