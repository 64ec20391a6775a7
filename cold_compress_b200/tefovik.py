"""Tefovik: a decoder-only design whose layers norm AFTER the sum (`x <- LN(alpha * x + scale * f(x))`, a layer norm
with a gain and no bias, a per-channel layer scale on every sublayer) and whose next-layer input is a learned
weighted average over the outputs of ALL layers so far (and of the embedding).  Two mixers:

* `mamba2`: a state-space mixer.  One input projection gives a gate z, the inputs x, B, C (through a short causal
  convolution and silu) and a step size per head; per head `S <- exp(-exp(A) dt) S + dt B x^T`, `y = S^T C + D x`;
  `y * silu(z)` is RMS-normed in groups and projected out.
* `parallel`: two mixers read the same input and their outputs, each RMS-normed over the model width, are averaged.
  Left: grouped-query softmax attention inside blocks of positions (a query sees the earlier keys of its own block
  only), with a short convolution on q, k and v, per-head RMS norm of q and k, rotary positions on part of q / k,
  values rotated by their position before caching and the head outputs rotated back by the query's position, and a
  sigmoid gate per head.  Right: a delta rule with a decay per key channel (`S <- diag(g) S; u = beta (v - S^T k);
  S <- S + k u^T; o = S^T q`), short convolutions with silu, unit-length q and k, low-rank projections for the decay
  and the output gate, RMS norm per head.

Feed-forward: `down(relu(up x)^2)`.  Output: layer norm, head, `cap * tanh(logits / cap)`.

The model plugs into the same runtime as `model.Transformer`, `tidelorn.TidelornTransformer` and
`detatar.DetatarTransformer`: `setup_caches` builds every layer's cache and state through
`cache.get_cache_constructor` (a ring of one block of positions for a block-masked attention, "state" for the
convolution tails and the matrix states), `forward(idx, input_pos, is_prefill)` is what `generation_utils.prefill` /
`decode_one_token` / `GraphedDecoder` call, and a step of any length continues from what earlier steps left.  Matrix
products of prompt portions are cuBLAS (torch.mm, fp32 accumulation and output); one-token steps use this package's
product kernels; everything between products is a kernel of csrc/seq.  There is no CPU path.

Precision: weights, cache rows and product inputs are in the compute dtype (bf16 or fp32); the residual stream, all
norms, convolutions, angles, attention scores and weights, step sizes, decays, gates of the recurrences and the
recurrent states are fp32 in both.

The mechanisms (`SumLayerNorm`, `ShortConv`, `StateSpaceMixer`, `BlockRotaryAttention`, `GatedDeltaRule`,
`ParallelMixer`, `SquaredReluMLP`) take their sizes and constants as arguments so that another design can use them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import _lib, seq_ops
from .cache import get_cache_constructor
from .detatar import _out, _pad16, _padded_rows, _zeros
from .tidelorn import _mm

MIXERS = ("mamba2", "parallel")


def _product(x: Tensor, w: Tensor, one_token: bool) -> Tensor:
    """x [T, K] times w[N, K]^T -> fp32 [T, N]: this package's product kernel for one token, cuBLAS otherwise."""
    if one_token and x.shape[0] == 1:
        out = _out(w)
        seq_ops.gemv_multi([(x, w, out)])
        return out
    return _mm(x, w)


def _inv_freq(base: float, dims: int) -> Tensor:
    """base^(-2i / dims) for i < dims / 2, computed in float64 and rounded once."""
    i = torch.arange(0, max(dims // 2, 1), dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / max(dims, 1)).to(torch.float32)


# --------------------------------------------------------------------------------------------- configuration

@dataclass
class TefovikArgs:
    vocab_size: int
    dim: int
    layers: List[Dict[str, Any]]
    norm_eps: float
    postln_alpha: float
    logit_softcap: float = 0.0
    block_size: int = 1 << 20      # angles are computed from the position: no table limits the length
    n_layer: int = field(init=False)

    def __post_init__(self):
        self.n_layer = len(self.layers)
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {layer.get('type')!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")

    @classmethod
    def from_config(cls, cfg: Dict[str, Any]):
        return cls(vocab_size=int(cfg["vocab"]), dim=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float(cfg["norm"]["eps"]), postln_alpha=float(cfg.get("postln_alpha", 1.0)),
                   logit_softcap=float(cfg.get("logit_softcap") or 0.0))


# --------------------------------------------------------------------------------------------- mechanisms

class SumLayerNorm(nn.Module):
    """n = LN(alpha * x + scale * y) * weight: a layer norm (mean and variance over the row, no bias) after the residual
    sum, with an optional per-channel `scale` on the sublayer's result.  The kernel can also take two sublayer results
    that are RMS-normed with their own gains and averaged first, write the depth average that follows the layer, and
    select rows (`seq_ops.sum_norm`); `center=False` makes it an RMS norm."""

    def __init__(self, dim: int, eps: float, alpha: float = 1.0, layer_scale: bool = False, center: bool = True):
        super().__init__()
        self.eps, self.alpha, self.center = float(eps), float(alpha), bool(center)
        self.weight = _zeros(dim, dtype=torch.float32)
        self.scale = _zeros(dim, dtype=torch.float32) if layer_scale else None

    def forward(self, x: Optional[Tensor], y: Optional[Tensor] = None, **kw):
        seq_ops.sum_norm(self.weight, self.eps, x=x, y=y, y_scale=self.scale if y is not None else None,
                         alpha=self.alpha, center=self.center, **kw)


class ShortConv(nn.Module):
    """Causal convolution over time on every channel, `taps` wide, optional bias and activation.  The last taps - 1
    inputs of a sequence are its state (`tail`, fp32 [taps - 1, channels]), carried from step to step."""

    def __init__(self, channels: int, taps: int, bias: bool = False, act: int = _lib.ACT_NONE):
        super().__init__()
        self.channels, self.taps, self.act = int(channels), int(taps), int(act)
        self.weight = _zeros(self.channels, self.taps, dtype=torch.float32)
        self.bias = _zeros(self.channels, dtype=torch.float32) if bias else None

    def forward(self, u: Tensor, tail: Tensor) -> Tensor:
        out = torch.empty(u.shape[0], self.channels, dtype=torch.float32, device=u.device)
        seq_ops.short_conv(u, self.weight, self.bias, tail if self.taps > 1 else None, out, self.act)
        return out


class StateSpaceMixer(nn.Module):
    """Input projection rows [z: inner | x: inner | B: G*N | C: G*N | dt: H] (inner = H * V); x, B, C through one short
    convolution with bias and silu; `dt = softplus(dt + dt_bias)`, per head `S <- exp(-exp(A_log) dt) S + dt B x^T`
    ([N, V]), `y = S^T C + D x`; `y * silu(z)` RMS-normed in `norm_groups` parts, times a gain, projected out.
    State per sequence: the convolution tail and S (fp32)."""

    def __init__(self, dim: int, heads: int, v_dim: int, state: int, groups: int, norm_groups: int, taps: int, eps: float, dtype):
        super().__init__()
        if heads % groups or (heads * v_dim) % norm_groups:
            raise ValueError("groups must divide the heads, norm groups the inner width")
        self.dim, self.heads, self.v_dim, self.state, self.groups = dim, int(heads), int(v_dim), int(state), int(groups)
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        self.inner = self.heads * self.v_dim
        self.conv_width = self.inner + 2 * self.groups * self.state
        self.w_in = _zeros(_pad16(self.inner + self.conv_width + self.heads), dim, dtype=dtype)
        self.conv = ShortConv(self.conv_width, taps, bias=True, act=_lib.ACT_SILU)
        self.dt_bias, self.A_log, self.D = (_zeros(self.heads, dtype=torch.float32) for _ in range(3))
        self.norm_w = _zeros(self.inner, dtype=torch.float32)
        self.w_o = _zeros(dim, self.inner, dtype=dtype)

    def state_spec(self):
        return dict(n_heads=self.heads, head_dim=self.state, state_cols=self.v_dim, state_vectors=self.conv.taps - 1,
                    state_width=self.conv_width)

    def forward(self, h_act: Tensor, ip: Tensor, state, one_token: bool = True):
        """h_act [T, dim] (compute dtype) -> the sublayer result as keyword arguments of the norm that sums it."""
        T, dev = h_act.shape[0], h_act.device
        H, V, N, G, inner, GN = self.heads, self.v_dim, self.state, self.groups, self.inner, self.groups * self.state
        zx = _product(h_act, self.w_in, one_token)
        c = self.conv(zx[:, inner:inner + self.conv_width], state.vectors)
        y = torch.empty(T, inner, dtype=torch.float32, device=dev)
        seq_ops.ssd_scan(c[:, :inner], c[:, inner:inner + GN], c[:, inner + GN:], zx[:, inner + self.conv_width:inner + self.conv_width + H],
                         self.dt_bias, self.A_log, self.D, state.matrix, y, H, G, N, V)
        yn = torch.empty(T, inner, dtype=self.w_o.dtype, device=dev)
        seq_ops.gated_rms_groups(y, zx[:, :inner], _lib.ACT_SILU, True, self.norm_w, yn, self.norm_groups, self.eps)
        return dict(y=_product(yn, self.w_o, one_token))

    def kernels_per_token(self):
        return 6   # input product, convolution, scan, gated norm, output product, the norm after the sum


class BlockRotaryAttention(nn.Module):
    """Grouped-query softmax attention with fp32 scores, over a position-addressed cache.  q, k, v pass a short
    convolution; q and k heads are RMS-normed with a gain shared by the heads and the first `rot_dims` of their entries
    are turned by the position; values are turned by their position over their whole width before they are cached, and
    each head's output is turned back by the query's position; `block` > 0 limits a query to the keys of its own block
    of positions (counted from the sequence's start); a sigmoid gate per head multiplies the output.  Its input rows
    [q | k | v | gate] are part of the fused projection of whoever owns it (`in_rows`, read at column `off`)."""

    def __init__(self, dim: int, heads: int, kv_heads: int, head_dim: int, v_dim: int, scale: float, taps: int, block: int,
                 rot_base: float, rot_dims: int, eps: float, dtype, interleaved: bool = True):
        super().__init__()
        if heads % kv_heads or rot_dims % 2 or rot_dims > head_dim or v_dim % 2:
            raise ValueError("kv heads must divide the heads; rotary dims must be even and at most the head size; values have pairs")
        self.dim, self.heads, self.kv_heads, self.head_dim, self.v_dim = dim, int(heads), int(kv_heads), int(head_dim), int(v_dim)
        self.scale, self.block, self.rot_dims, self.eps, self.interleaved = float(scale), int(block), int(rot_dims), float(eps), interleaved
        self.conv_width = (self.heads + self.kv_heads) * self.head_dim + self.kv_heads * self.v_dim
        self.in_rows = self.conv_width + self.heads
        self.conv = ShortConv(self.conv_width, taps)
        self.q_norm = _zeros(self.head_dim, dtype=torch.float32)
        self.k_norm = _zeros(self.head_dim, dtype=torch.float32)
        self.w_o = _zeros(dim, self.heads * self.v_dim, dtype=dtype)
        self.register_buffer("inv_freq", _inv_freq(rot_base, self.rot_dims), persistent=False)
        self.register_buffer("v_inv_freq", _inv_freq(rot_base, self.v_dim), persistent=False)

    def state_spec(self):
        return dict(n_heads=0, head_dim=0, state_vectors=self.conv.taps - 1, state_width=self.conv_width)

    def core(self, hp: Tensor, off: int, ip: Tensor, state, kv_cache) -> Tensor:
        """From the fused projection's fp32 rows to the input of the output projection [T, heads * v_dim]."""
        T, dev, dt = hp.shape[0], hp.device, self.w_o.dtype
        H, G, Dk, Dv = self.heads, self.kv_heads, self.head_dim, self.v_dim
        c = self.conv(hp[:, off:off + self.conv_width], state.vectors)
        q = torch.empty(T, H, Dk, dtype=torch.float32, device=dev)
        k = torch.empty(T, G, Dk, dtype=dt, device=dev)
        v = torch.empty(T, G, Dv, dtype=dt, device=dev)
        seq_ops.qkv_rope(c, 0, H * Dk, (H + G) * Dk, H, G, Dk, Dv, self.q_norm, self.k_norm, self.eps, self.rot_dims,
                         self.interleaved, self.inv_freq, self.v_inv_freq, ip, q, k, v)
        y = torch.empty(T, H, Dv, dtype=torch.float32, device=dev)
        kv_cache.sequence_step(q, k, v, ip, y, scale=self.scale, block=self.block)
        ya = torch.empty(T, H * Dv, dtype=dt, device=dev)
        seq_ops.turn_heads_gate(y, ip, self.v_inv_freq, Dv, self.interleaved, -1.0,
                                hp[:, off + self.conv_width:off + self.conv_width + H], ya.view(T, H, Dv))
        return ya


class GatedDeltaRule(nn.Module):
    """Delta rule with a decay per key channel.  q, k (kv_heads x dim) and v (heads x v_dim) pass short convolutions with
    silu; q and k become unit vectors per head (q also times dim^-1/2); `beta = sigmoid(W_b h)` per head; decay
    `g = exp(-exp(A_log) * softplus(W_a2 W_a1 h + dt_bias))` per head and key channel; per head `S <- diag(g) S;
    u = beta (v - S^T k); S <- S + k u^T; o = S^T q`; o is RMS-normed per head with a gain shared by the heads and
    multiplied by `sigmoid(W_g2 W_g1 h)`.  Input rows [q | k | v | b | a1 | g1] are part of the owner's fused projection.
    State per sequence: the convolution tail and S [heads, dim, v_dim] (fp32)."""

    unit_eps = 1e-6

    def __init__(self, dim: int, heads: int, kv_heads: int, head_dim: int, v_dim: int, taps: int, decay_rank: int, gate_rank: int,
                 eps: float, dtype):
        super().__init__()
        if heads % kv_heads:
            raise ValueError("kv heads must divide the heads")
        self.dim, self.heads, self.kv_heads, self.head_dim, self.v_dim = dim, int(heads), int(kv_heads), int(head_dim), int(v_dim)
        self.decay_rank, self.gate_rank, self.eps = int(decay_rank), int(gate_rank), float(eps)
        self.conv_width = 2 * self.kv_heads * self.head_dim + self.heads * self.v_dim
        self.in_rows = self.conv_width + self.heads + self.decay_rank + self.gate_rank
        self.conv = ShortConv(self.conv_width, taps, act=_lib.ACT_SILU)
        self.w_a2 = _zeros(self.heads * self.head_dim, self.decay_rank, dtype=dtype)
        self.w_g2 = _zeros(self.heads * self.v_dim, self.gate_rank, dtype=dtype)
        self.dt_bias = _zeros(self.heads * self.head_dim, dtype=torch.float32)
        self.A_log = _zeros(self.heads, dtype=torch.float32)
        self.norm_w = _zeros(self.v_dim, dtype=torch.float32)
        self.w_o = _zeros(dim, self.heads * self.v_dim, dtype=dtype)

    def state_spec(self):
        return dict(n_heads=self.heads, head_dim=self.head_dim, state_cols=self.v_dim, state_vectors=self.conv.taps - 1,
                    state_width=self.conv_width)

    def core(self, hp: Tensor, off: int, ip: Tensor, state, one_token: bool) -> Tensor:
        T, dev, dt = hp.shape[0], hp.device, self.w_o.dtype
        H, G, D, V = self.heads, self.kv_heads, self.head_dim, self.v_dim
        ob = off + self.conv_width
        oa, og = ob + H, ob + H + self.decay_rank
        c = self.conv(hp[:, off:off + self.conv_width], state.vectors)
        if one_token and T == 1:
            a_raw, g_raw = _out(self.w_a2), _out(self.w_g2)
            seq_ops.gemv_multi([(hp[:, oa:oa + self.decay_rank], self.w_a2, a_raw), (hp[:, og:og + self.gate_rank], self.w_g2, g_raw)])
        else:
            low_a = torch.empty(T, self.decay_rank, dtype=dt, device=dev)
            low_g = torch.empty(T, self.gate_rank, dtype=dt, device=dev)
            seq_ops.gated_unit(hp, oa, -1, low_a, _lib.ACT_NONE)
            seq_ops.gated_unit(hp, og, -1, low_g, _lib.ACT_NONE)
            a_raw, g_raw = _mm(low_a, self.w_a2), _mm(low_g, self.w_g2)
        o = torch.empty(T, H * V, dtype=torch.float32, device=dev)
        seq_ops.delta_scan(c[:, :G * D], c[:, G * D:2 * G * D], c[:, 2 * G * D:], hp[:, ob:ob + H], a_raw, self.dt_bias, self.A_log,
                           state.matrix, o, H, G, D, V, D ** -0.5, self.unit_eps)
        on = torch.empty(T, H * V, dtype=dt, device=dev)
        seq_ops.gated_rms_groups(o, g_raw, _lib.ACT_SIGMOID, False, self.norm_w, on, H, self.eps)
        return on


class ParallelMixer(nn.Module):
    """Two mixers on the same input; the result is the mean of their outputs, each first RMS-normed over the model
    width with its own gain.  One fused projection serves both ([left rows | right rows], padded to 16); the mean of
    the normed outputs is formed by the norm that sums the sublayer into the stream."""

    def __init__(self, dim: int, left: BlockRotaryAttention, right: GatedDeltaRule, dtype):
        super().__init__()
        self.left, self.right = left, right
        self.w_in = _zeros(_pad16(left.in_rows + right.in_rows), dim, dtype=dtype)
        self.left_out = _zeros(dim, dtype=torch.float32)
        self.right_out = _zeros(dim, dtype=torch.float32)

    def forward(self, h_act: Tensor, ip: Tensor, states, kv_cache, one_token: bool = True):
        hp = _product(h_act, self.w_in, one_token)
        ya = self.left.core(hp, 0, ip, states[0], kv_cache)
        on = self.right.core(hp, self.left.in_rows, ip, states[1], one_token)
        if one_token and h_act.shape[0] == 1:
            a, b = _out(self.left.w_o), _out(self.right.w_o)
            seq_ops.gemv_multi([(ya, self.left.w_o, a), (on, self.right.w_o, b)])
        else:
            a, b = _mm(ya, self.left.w_o), _mm(on, self.right.w_o)
        return dict(y=a, y_norm_w=self.left_out, y2=b, y2_norm_w=self.right_out, y_coef=0.5)

    def kernels_per_token(self):
        # fused product; left: convolution, q/k/v rows, attention + append, turn + gate; right: convolution, low-rank
        # products, scan, gated norm; both output products; the norm after the sum
        return 1 + 4 + 4 + 1 + 1


class SquaredReluMLP(nn.Module):
    """down(relu(up x)^2)."""

    def __init__(self, dim: int, ff: int, dtype):
        super().__init__()
        self.ff = int(ff)
        self.w_up = _zeros(self.ff, dim, dtype=dtype)
        self.w_down = _zeros(dim, self.ff, dtype=dtype)

    def forward(self, x_act: Tensor, one_token: bool = True) -> Tensor:
        if one_token and x_act.shape[0] == 1:     # the activation is applied while the second product stages its input
            up, out = _out(self.w_up), _out(self.w_down)
            seq_ops.gemv_multi([(x_act, self.w_up, up)])
            seq_ops.gemv_multi([(up, self.w_down, out, _lib.ACT_RELU_SQ, 0, -1)])
            return out
        up = _mm(x_act, self.w_up)
        act = torch.empty(x_act.shape[0], self.ff, dtype=self.w_down.dtype, device=x_act.device)
        seq_ops.gated_unit(up, 0, -1, act, _lib.ACT_RELU_SQ)
        return _mm(act, self.w_down)


# --------------------------------------------------------------------------------------------- a layer

class TefovikBlock(nn.Module):
    """Mixer sublayer, optional feed-forward sublayer (each `x <- LN(alpha * x + scale * f(x))`), then the depth
    average `sum_j coef[j] * X_j` over the embedding output and the results of the layers so far."""

    def __init__(self, cfg: TefovikArgs, index: int, layer: Dict[str, Any], dtype):
        super().__init__()
        E, m, mlp = cfg.dim, layer["mixer"], layer.get("mlp")
        self.kind, self.index = layer["type"], index
        if self.kind == "mamba2":
            self.mixer = StateSpaceMixer(E, int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m.get("groups", 1)),
                                         int(m.get("norm_groups", 1)), int(m["conv"]), cfg.norm_eps, dtype)
        else:
            l, r = m["left"], m["right"]
            rot = l.get("rot") or {}
            left = BlockRotaryAttention(E, int(l["heads"]), int(l["kv_heads"]), int(l["dim"]), int(l["vdim"]), float(l["scale"]),
                                        int(l.get("conv", 1)), int((l.get("mask") or {}).get("size", 0)), float(rot.get("base", 10000.0)),
                                        int(rot.get("dims", 0)), cfg.norm_eps, dtype)
            # the ranks of the two low-rank projections are tensor shapes: load_tensors sizes those parameters
            right = GatedDeltaRule(E, int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"]), int(r.get("conv", 1)),
                                   int(r.get("decay_rank", 0)), int(r.get("gate_rank", 0)), cfg.norm_eps, dtype)
            self.mixer = ParallelMixer(E, left, right, dtype)
        self.norm1 = SumLayerNorm(E, cfg.norm_eps, cfg.postln_alpha, layer_scale=True)
        self.mlp = SquaredReluMLP(E, int(mlp["ff"]), dtype) if mlp else None
        self.norm2 = SumLayerNorm(E, cfg.norm_eps, cfg.postln_alpha, layer_scale=True) if mlp else None
        self.depth_coef = _zeros(index + 2, dtype=torch.float32)
        self.states = None      # list of cache.RecurrentState (one per mixer that carries state)
        self.kv_cache = None

    def forward(self, x: Tensor, x_act: Tensor, stack: Tensor, ip: Tensor, one_token: bool):
        """x fp32 [T, E] and its copy in the compute dtype are this layer's input and, on return, the next layer's;
        stack[j] holds X_j, this layer's own result goes to stack[index + 1]."""
        i = self.index
        side = None if x_act is x else x_act
        average = dict(out=stack[i + 1], stack=stack, n_prev=i + 1, coef=self.depth_coef, mix=x, out_act=side)
        if self.kind == "mamba2":
            mixed = self.mixer(x_act, ip, self.states[0], one_token)
        else:
            mixed = self.mixer(x_act, ip, self.states, self.kv_cache, one_token)
        if self.mlp is None:
            self.norm1(x, **mixed, **average)
            return
        x1 = torch.empty_like(x)
        x1_act = x1 if x_act is x else torch.empty_like(x_act)
        self.norm1(x, **mixed, out=x1, out_act=None if x1_act is x1 else x1_act)
        self.norm2(x1, self.mlp(x1_act, one_token), **average)

    def kernels_per_token(self):
        return self.mixer.kernels_per_token() + (3 if self.mlp is not None else 0)


# --------------------------------------------------------------------------------------------- the model

class TefovikTransformer(nn.Module):
    """Same runtime surface as `model.Transformer`: setup_caches / reset_caches / forward / min_cache_length /
    get_cache_stats / prompt_cache_overflow, `config.block_size`, `config.n_layer`."""

    supports_prompt_portions = True

    def __init__(self, config: TefovikArgs, dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32)
        self.config, self.dtype = config, dtype
        self.tok_embeddings = _zeros(config.vocab_size, config.dim, dtype=dtype)
        self.embed_norm = SumLayerNorm(config.dim, config.norm_eps)
        self.layers = nn.ModuleList(TefovikBlock(config, i, layer, dtype) for i, layer in enumerate(config.layers))
        self.norm = SumLayerNorm(config.dim, config.norm_eps)
        self.output = _zeros(config.vocab_size, config.dim, dtype=dtype)
        self.max_batch_size = 1
        self.max_seq_length = 0
        # one-token steps through this package's product kernels; False = library products as in a prompt portion of
        # one token (used by A/B tests)
        self.fused_decode = True

    # ---- caches and state -------------------------------------------------------------------------
    def layer_cache_plan(self, cache_kwargs: Dict[str, Any], max_seq_length: int) -> Dict[str, Any]:
        """A block-masked attention keeps a ring of one block of positions ("recent_global" without global tokens; the
        keys a query may see never leave it), an unmasked one keeps everything ("full"); a layer without attention only
        carries fixed-size state ("state": convolution tails and matrix states, which every layer has)."""
        ck = dict(cache_kwargs or {})
        ck["max_seq_length"] = max_seq_length
        strategies, lengths = [], []
        for layer in self.layers:
            if layer.kind == "parallel":
                block = layer.mixer.left.block
                strategies.append("recent_global" if block else "full")
                lengths.append(block if block else max_seq_length)
            else:
                strategies.append("state")
                lengths.append(0)
        ck["cache_strategy"], ck["max_cache_length"] = strategies, lengths
        ck["global_tokens"] = 0
        ck["cache_bits"] = None
        ck["prompt_compression_strategy"] = ["none"] * len(self.layers)
        return ck

    def setup_caches(self, **kwargs):
        strategies, lengths = kwargs["cache_strategy"], kwargs["max_cache_length"]
        state_ctor, _ = get_cache_constructor("state")
        for i, layer in enumerate(self.layers):
            if layer.kind == "parallel":
                att = layer.mixer.left
                ctor, _ = get_cache_constructor(strategies[i])
                layer.kv_cache = ctor(self.max_batch_size, att.kv_heads, att.head_dim, self.dtype, v_head_dim=att.v_dim,
                                      max_cache_length=int(lengths[i]), max_seq_length=kwargs.get("max_seq_length"),
                                      global_tokens=0, cache_bits=None)
                layer.states = nn.ModuleList([state_ctor(self.max_batch_size, **att.state_spec()),
                                              state_ctor(self.max_batch_size, **layer.mixer.right.state_spec())])
            else:
                layer.kv_cache = None
                layer.states = nn.ModuleList([state_ctor(self.max_batch_size, **layer.mixer.state_spec())])
        self.max_seq_length = int(kwargs.get("max_seq_length") or max(lengths))

    def reset_caches(self):
        """Gives back what the finished sequence held: every slot empty, every state zero."""
        for layer in self.layers:
            for s in layer.states:
                s.reset()
            if layer.kv_cache is not None:
                layer.kv_cache.reset()

    def prompt_cache_overflow(self, prompt_length: int):
        return [l.kv_cache is not None and not l.mixer.left.block and prompt_length > l.kv_cache.max_cache_length for l in self.layers]

    def min_cache_length(self):
        full = [l.kv_cache.max_cache_length for l in self.layers if l.kv_cache is not None and not l.mixer.left.block]
        return min(full) if full else self.max_seq_length

    def get_cache_stats(self, prompt_len, gen_len):
        stats, mem = {}, 0.0
        for i, layer in enumerate(self.layers):
            stats[f"cache_slots_{i}"] = float(layer.kv_cache.max_cache_length if layer.kv_cache is not None else 0)
            mem += sum(s.memory_usage() for s in layer.states) + (layer.kv_cache.memory_usage() if layer.kv_cache is not None else 0.0)
        stats["cache_memory_gb"] = mem
        return stats

    # ---- one step: a whole prompt, a portion of it, or one token ----------------------------------
    @torch.no_grad()
    def forward(self, idx: Tensor, input_pos: Tensor, is_prefill: bool = True, mask: Optional[Tensor] = None,
                attn_top_k: Optional[float] = 1.0, logits_at: Optional[Tensor] = None,
                collect: Optional[list] = None) -> Tensor:
        """idx [1, T] token ids, input_pos [T] (or [1]) positions with input_pos[0] the first token's; returns fp32
        logits [1, n, vocab] for the rows `logits_at` (default: the last).  The step continues from the caches and
        state that earlier steps left.  `collect`, if a list, receives the next layer's input after every layer."""
        assert attn_top_k in (None, 1, 1.0), "top-k attention is not part of this design"
        if self.layers[0].states is None:
            raise RuntimeError("Caches must be initialized first")
        tokens = idx.reshape(-1)
        if not tokens.is_cuda:
            raise _lib.CcError("this model runs on CUDA tensors only (no CPU fallback)")
        tokens = tokens if tokens.dtype == torch.int32 else tokens.to(torch.int32)
        ip = input_pos.reshape(-1)[:1]
        ip = ip if ip.dtype == torch.int32 else ip.to(torch.int32)
        T, E, dev, dt = tokens.numel(), self.config.dim, tokens.device, self.dtype
        one = T == 1 and self.fused_decode
        stack = torch.empty(len(self.layers) + 1, T, E, dtype=torch.float32, device=dev)
        x = torch.empty(T, E, dtype=torch.float32, device=dev)
        x_act = x if dt == torch.float32 else torch.empty(T, E, dtype=dt, device=dev)
        seq_ops.embed_rows(tokens, self.tok_embeddings, x, 1.0)
        self.embed_norm(x, out=stack[0], out_act=None if x_act is x else x_act)
        x.copy_(stack[0])
        for layer in self.layers:
            layer(x, x_act, stack, ip, one)
            if collect is not None:
                collect.append(x.clone())
        rows = None if logits_at is None else logits_at.to(device=dev, dtype=torch.int64).contiguous()
        if rows is None:
            rows = torch.full((1,), T - 1, dtype=torch.int64, device=dev)
        xs_act = torch.empty(rows.numel(), E, dtype=dt, device=dev)
        self.norm(x, rows=rows, out_act=xs_act)
        logits = _product(xs_act, self.output, one)
        if self.config.logit_softcap > 0:
            seq_ops.softcap(logits, self.config.logit_softcap)
        return logits.view(1, rows.numel(), -1)

    def kernels_per_token(self) -> int:
        """Launches of this package's kernels in one decode step (fused_decode)."""
        return 3 + 3 + sum(l.kernels_per_token() for l in self.layers)   # embedding rows, its norm, copy; last norm, head, cap

    # ---- weights --------------------------------------------------------------------------------
    def load_tensors(self, tensors: Dict[str, Tensor]):
        """Fills the parameters from the checkpoint's tensor names ('embed', 'embed.norm', 'l<i>.norm1' / '.norm2',
        '.ls1' / '.ls2', '.dwa', 'l<i>.mix.*', 'l<i>.mlp.up' / '.down', 'final.norm', 'head'), fusing the projection
        rows that read the same input."""
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

        def conv_rows(conv: ShortConv, names, widths):
            # a checkpoint may leave out the table of a one-tap convolution: that is the identity
            put(conv.weight, torch.cat([get(n, (w, conv.taps)).float() if conv.taps > 1 or n in tensors else torch.ones(w, 1)
                                        for n, w in zip(names, widths)]))

        cfg = self.config
        E = cfg.dim
        put(self.tok_embeddings, get("embed", (cfg.vocab_size, E)))
        put(self.embed_norm.weight, get("embed.norm", (E,)).float())
        for i, b in enumerate(self.layers):
            p = f"l{i}."
            put(b.norm1.weight, get(p + "norm1", (E,)).float())
            put(b.norm1.scale, get(p + "ls1", (E,)).float())
            put(b.depth_coef, get(p + "dwa", (i + 2,)).float())
            m = b.mixer
            if b.kind == "mamba2":
                q = p + "mix."
                put(m.w_in, _padded_rows([get(q + "in", (m.inner + m.conv_width + m.heads, E))], m.w_in.shape[0]))
                conv_rows(m.conv, [q + "conv"], [m.conv_width])
                put(m.conv.bias, get(q + "conv.b", (m.conv_width,)).float())
                for name in ("dt_bias", "A_log", "D"):
                    put(getattr(m, name), get(q + name, (m.heads,)).float())
                put(m.norm_w, get(q + "norm", (m.inner,)).float())
                put(m.w_o, get(q + "o", (E, m.inner)))
            else:
                l, r = m.left, m.right
                ql, qr = p + "mix.left.", p + "mix.right."
                nq, nk, nv = l.heads * l.head_dim, l.kv_heads * l.head_dim, l.kv_heads * l.v_dim
                rq, rv = r.kv_heads * r.head_dim, r.heads * r.v_dim
                ra, rg = get(qr + "a1").shape[0], get(qr + "g1").shape[0]
                if (r.decay_rank, r.gate_rank) != (ra, rg):     # the ranks come from the tensors
                    dev, dt = r.w_a2.device, r.w_a2.dtype
                    r.decay_rank, r.gate_rank = ra, rg
                    r.in_rows = r.conv_width + r.heads + ra + rg
                    r.w_a2 = _zeros(r.heads * r.head_dim, ra, dtype=dt).to(dev)
                    r.w_g2 = _zeros(rv, rg, dtype=dt).to(dev)
                    m.w_in = _zeros(_pad16(l.in_rows + r.in_rows), E, dtype=dt).to(dev)
                put(m.w_in, _padded_rows([get(ql + "q", (nq, E)), get(ql + "k", (nk, E)), get(ql + "v", (nv, E)), get(ql + "g", (l.heads, E)),
                                          get(qr + "q", (rq, E)), get(qr + "k", (rq, E)), get(qr + "v", (rv, E)), get(qr + "b", (r.heads, E)),
                                          get(qr + "a1", (ra, E)), get(qr + "g1", (rg, E))], m.w_in.shape[0]))
                conv_rows(l.conv, [ql + "q.conv", ql + "k.conv", ql + "v.conv"], [nq, nk, nv])
                put(l.q_norm, get(ql + "q.norm", (l.head_dim,)).float())
                put(l.k_norm, get(ql + "k.norm", (l.head_dim,)).float())
                put(l.w_o, get(ql + "o", (E, l.heads * l.v_dim)))
                conv_rows(r.conv, [qr + "q.conv", qr + "k.conv", qr + "v.conv"], [rq, rq, rv])
                put(r.w_a2, get(qr + "a2", (r.heads * r.head_dim, ra)))
                put(r.w_g2, get(qr + "g2", (rv, rg)))
                put(r.dt_bias, get(qr + "dt_bias", (r.heads * r.head_dim,)).float())
                put(r.A_log, get(qr + "A_log", (r.heads,)).float())
                put(r.norm_w, get(qr + "norm", (r.v_dim,)).float())
                put(r.w_o, get(qr + "o", (E, rv)))
                put(m.left_out, get(ql + "out", (E,)).float())
                put(m.right_out, get(qr + "out", (E,)).float())
            if b.mlp is not None:
                put(b.norm2.weight, get(p + "norm2", (E,)).float())
                put(b.norm2.scale, get(p + "ls2", (E,)).float())
                put(b.mlp.w_up, get(p + "mlp.up", (b.mlp.ff, E)))
                put(b.mlp.w_down, get(p + "mlp.down", (E, b.mlp.ff)))
        put(self.norm.weight, get("final.norm", (E,)).float())
        put(self.output, get("head", (cfg.vocab_size, E)))
        return sorted(set(tensors) - used)

    @classmethod
    def from_config(cls, cfg: Dict[str, Any], dtype=torch.bfloat16):
        return cls(TefovikArgs.from_config(cfg), dtype)
