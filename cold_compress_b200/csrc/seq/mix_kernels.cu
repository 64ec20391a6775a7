// mix_kernels.cu -- sequence kernels for layers that carry per-sequence state besides a key/value cache
// (include/cc_b200_seq.h, second part): grouped RMS norm fused with a gated residual sum, token shift, a
// matrix-state linear recurrence with per-channel decay and a current-token bonus, the row preparation of latent
// (low-rank) attention, per-head products for its absorbed one-token form, gated units, and the routing, dispatch and
// combination of a mixture of experts.
//
// Arithmetic rule (as in seq_kernels.cu): norms, gates, angles, decays, the recurrent state, router scores and the
// residual stream are fp32 whatever the storage type; expf / tanhf / sincosf are the accurate versions.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include "../../../include/cc_b200_seq.h"

namespace ccs {
int fail(int code, const char* msg);
int cuda_check(const char* where);
}  // namespace ccs

namespace ccm {
using ccs::cuda_check;
using ccs::fail;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float ldf(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const bf16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Sum over the block in a fixed order (warp shuffles, then the warps' partial sums one after another).
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];
    return s;
}

__device__ __forceinline__ void load8(const float* p, float* o) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* o) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const bf16* e = reinterpret_cast<const bf16*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __bfloat162float(e[i]);
}
// One weight row against one input row, by a warp: eight elements per lane and load when both rows allow it.
template <typename WT, typename XT>
__device__ __forceinline__ float warp_dot(const WT* __restrict__ w, const XT* __restrict__ x, int K, int lane) {
    float acc = 0.f;
    if (K % 8 == 0 && (((uintptr_t)w | (uintptr_t)x) & 15) == 0) {
#pragma unroll 2
        for (int k = lane * 8; k < K; k += 256) {
            float a[8], b[8];
            load8(w + k, a);
            load8(x + k, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(ldf(w, k), ldf(x, k), acc);
    }
    return warp_sum(acc);
}

__device__ __forceinline__ float unit_act(float z, int kind) {
    switch (kind) {
        case CC_ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        case CC_ACT_SILU: return z * sigmoidf_(z);
        case CC_ACT_TANH: return tanhf(z);
        case CC_ACT_SIGMOID: return sigmoidf_(z);
        case CC_ACT_RELU_SQ: { const float r = fmaxf(z, 0.f); return r * r; }
        default: return z;
    }
}

// ------------------------------------------------------------------------------------------------ embedding rows
template <typename ST>
__global__ void embed_rows_kernel(const int32_t* __restrict__ tokens, const ST* __restrict__ embed, float* __restrict__ x,
                                  int E, float scale) {
    const int t = blockIdx.x;
    const size_t row = (size_t)tokens[t] * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) x[(size_t)t * E + e] = ldf(embed, row + e) * scale;
}

// ------------------------------------------------------------------------------------------------ gated sum + grouped norm
// One (token, norm group) per CTA: x += a * sigmoid(ga + ba) + b * sigmoid(gb + bb) on the group's part of the row, then
// h = x / rms(part) * w.  Groups are independent, so a single token still spreads over `groups` CTAs.
template <typename ST>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const CcSeqGatedNorm g) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int i = blockIdx.x, E = g.E, tid = threadIdx.x;
    const int gs = E / g.groups, c0 = blockIdx.y * gs;
    const size_t t = g.rows ? (size_t)g.rows[i] : (size_t)i;
    float* x = g.x + t * E;
    float ss = 0.f;
    for (int e = tid; e < gs; e += blockDim.x) {
        const int c = c0 + e;
        float v = x[c];
        if (g.a != nullptr) {
            const float gate = g.ga ? sigmoidf_(g.ga[t * g.ldga + c] + (g.ba ? g.ba[c] : 0.f)) : 1.f;
            v += g.a[t * g.lda + c] * gate;
        }
        if (g.b != nullptr) {
            const float gate = g.gb ? sigmoidf_(g.gb[t * g.ldgb + c] + (g.bb ? g.bb[c] : 0.f)) : 1.f;
            v += g.b[t * g.ldb + c] * gate;
        }
        row[e] = v;
        ss += v * v;
        if (g.a != nullptr || g.b != nullptr) x[c] = v;
    }
    if (g.w == nullptr) return;
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)gs + g.eps);
    for (int e = tid; e < gs; e += blockDim.x) {      // thread e reads back only what it wrote
        const int c = c0 + e;
        const float h = row[e] * rinv * g.w[c];
        if (g.h != nullptr) g.h[(size_t)i * E + c] = h;
        if (g.h_act != nullptr) stf((ST*)g.h_act, (size_t)i * E + c, h);
        if (g.shift_state != nullptr) {      // one token: its shifted copies in the same pass (thread owns element c)
            const float hs = h + (g.shift_state[c] - h) * g.shift_mu[c];
            g.shift_state[c] = h;
            if (g.hs_act != nullptr) stf((ST*)g.hs_act, c, hs);
            if (g.n_mix > 0) {
                const float prev = g.mix_state[c];
                for (int m = 0; m < g.n_mix; ++m) stf((ST*)g.mixes, (size_t)m * E + c, hs + (prev - hs) * g.mix_mu[(size_t)m * E + c]);
                g.mix_state[c] = hs;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ token shift
// out[s][t] = h[t] + (h[t-1] - h[t]) * mu[s]; the row before the first one is the sequence's state, which then
// becomes the last row.  Thread e alone reads and writes state[e].
template <typename ST>
__global__ void token_shift_kernel(const float* __restrict__ h, float* state, const float* __restrict__ mu,
                                   ST* __restrict__ out, float* __restrict__ outf, int T, int E, int n) {
    const int t = blockIdx.x;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float cur = h[(size_t)t * E + e];
        const float prev = t > 0 ? h[(size_t)(t - 1) * E + e] : state[e];
        for (int s = 0; s < n; ++s) {
            const float m = cur + (prev - cur) * mu[(size_t)s * E + e];
            if (out != nullptr) stf(out, ((size_t)s * T + t) * E + e, m);
            if (outf != nullptr && s == 0) outf[(size_t)t * E + e] = m;
        }
        if (t == 0) state[e] = h[(size_t)(T - 1) * E + e];
    }
}

// ------------------------------------------------------------------------------------------------ gated unit
template <typename ST>
__global__ void gated_unit_kernel(const float* __restrict__ in, int64_t ld, int off_gate, int off_up, ST* __restrict__ out,
                                  int T, int F, int kind) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;      // column; rows stride over gridDim.y (no division per element)
    if (f >= F) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float* row = in + (size_t)t * ld;
        float v = unit_act(row[off_gate + f], kind);
        if (off_up >= 0) v *= row[off_up + f];
        stf(out, (size_t)t * F + f, v);
    }
}

// ------------------------------------------------------------------------------------------------ latent attention rows
// One token per CTA.  From the fused down-projection row: the query latent and the key/value latent are RMS-normed
// (plain weights); the trailing `rot_dim` columns are the key part shared by all heads, rotated by the position.
template <typename ST>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const CcSeqLatentPrep a) {
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* in = a.in + (size_t)t * a.ld;
    const int Dk = a.kv_rank + a.rot_dim;
    if (a.q_rank > 0) {
        float ss = 0.f;
        for (int e = tid; e < a.q_rank; e += blockDim.x) { const float v = in[a.off_q + e]; ss += v * v; }
        const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)a.q_rank + a.eps);
        for (int e = tid; e < a.q_rank; e += blockDim.x)
            stf((ST*)a.cq, (size_t)t * a.q_rank + e, in[a.off_q + e] * rinv * a.wq[e]);
    }
    float ss = 0.f;
    for (int e = tid; e < a.kv_rank; e += blockDim.x) { const float v = in[a.off_kv + e]; ss += v * v; }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)a.kv_rank + a.eps);
    for (int e = tid; e < a.kv_rank; e += blockDim.x) {
        const float c = in[a.off_kv + e] * rinv * a.wkv[e];
        stf((ST*)a.krow, (size_t)t * Dk + e, c);
        if (a.vrow != nullptr) stf((ST*)a.vrow, (size_t)t * a.kv_rank + e, c);
    }
    const float p = (float)(a.input_pos[0] + t);
    const float* tail = in + a.off_kv + a.kv_rank;
    const int half = a.rot_dims / 2;
    ST* kr = (ST*)a.krow + (size_t)t * Dk + a.kv_rank;
    for (int e = tid; e < half; e += blockDim.x) {
        float sn, cs;
        sincosf(p * a.inv_freq[e], &sn, &cs);
        const int i0 = a.interleaved ? 2 * e : e, i1 = a.interleaved ? 2 * e + 1 : e + half;
        const float u = tail[i0], v = tail[i1];
        stf(kr, i0, u * cs - v * sn);
        stf(kr, i1, v * cs + u * sn);
    }
    for (int e = 2 * half + tid; e < a.rot_dim; e += blockDim.x) stf(kr, e, tail[e]);
}

// Rotation of one segment of every head of a fused query row, in place; optionally the rotated segment is also
// copied to `tail` (the absorbed query layout [H, tail_ld] at column tail_off).
__global__ void rope_heads_kernel(float* __restrict__ q, int64_t ld, const int32_t* __restrict__ input_pos,
                                  const float* __restrict__ inv_freq, int H, int head_w, int off, int seg, int dims,
                                  float* __restrict__ tail, int64_t tail_ld, int tail_off, int T, int interleaved) {
    const int t = blockIdx.x, half = dims / 2;
    const float p = (float)(input_pos[0] + t);
    float* row = q + (size_t)t * ld;
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, e = idx - h * half;
        float* s = row + (size_t)h * head_w + off;
        float sn, cs;
        sincosf(p * inv_freq[e], &sn, &cs);
        const int i0 = interleaved ? 2 * e : e, i1 = interleaved ? 2 * e + 1 : e + half;
        const float u = s[i0], v = s[i1];
        s[i0] = u * cs - v * sn;
        s[i1] = v * cs + u * sn;
    }
    if (tail == nullptr) return;
    __syncthreads();
    for (int idx = threadIdx.x; idx < H * seg; idx += blockDim.x) {
        const int h = idx / seg, e = idx - h * seg;
        tail[((size_t)t * H + h) * tail_ld + tail_off + e] = row[(size_t)h * head_w + off + e];
    }
}

// Per-head key and value rows from the up-projection of the latents: row n < n_old goes into the head-major
// "old" buffers [H, n_old, *], the others into the token-major "new" buffers [T, H, *].  The key row of head h is
// [up-projected part | shared rotated part of the latent row].
template <typename ST>
__global__ void latent_expand_kernel(const CcSeqLatentExpand a) {
    const int n = blockIdx.x, H = a.H, D = a.D, V = a.V, R = a.R, Dk = D + R;
    const bool old = n < a.n_old;
    const int r = old ? n : n - a.n_old;
    const float* kv = old ? a.kv_old + (size_t)r * a.ld_kv : a.kv_new + (size_t)r * a.ld_kv;
    const ST* lat = old ? (const ST*)a.lat_old + (size_t)r * a.ld_lat : (const ST*)a.lat_new + (size_t)r * a.ld_lat;
    for (int idx = threadIdx.x; idx < H * Dk; idx += blockDim.x) {
        const int h = idx / Dk, e = idx - h * Dk;
        const float v = e < D ? kv[(size_t)h * D + e] : ldf(lat, a.kv_rank + e - D);
        if (old) stf((ST*)a.k_old, ((size_t)h * a.n_old + r) * Dk + e, v);
        else stf((ST*)a.k_new, ((size_t)r * H + h) * Dk + e, v);
    }
    for (int idx = threadIdx.x; idx < H * V; idx += blockDim.x) {
        const int h = idx / V, e = idx - h * V;
        const float v = kv[(size_t)H * D + (size_t)h * V + e];
        if (old) stf((ST*)a.v_old, ((size_t)h * a.n_old + r) * V + e, v);
        else stf((ST*)a.v_new, ((size_t)r * H + h) * V + e, v);
    }
}

// y [T, H, V] *= sigmoid(g[t, h]); a CTA per token
template <typename ST>
__global__ void head_gate_kernel(ST* __restrict__ y, const float* __restrict__ g, int64_t ldg, int T, int H, int V) {
    const size_t t = blockIdx.x;
    for (int h = threadIdx.y; h < H; h += blockDim.y) {
        const float gate = sigmoidf_(g[t * ldg + h]);
        ST* row = y + (t * H + h) * V;
        for (int v = threadIdx.x; v < V; v += blockDim.x) stf(row, v, ldf(row, v) * gate);
    }
}

// out[h, n] = W[h, n, :] . x[h, :]  (* sigmoid(gate[h])): a block-diagonal one-token product, a warp per row.
template <typename WT, typename XT, typename OT>
__global__ void __launch_bounds__(256) head_gemv_kernel(const WT* __restrict__ W, const XT* __restrict__ x, int64_t sx,
                                                        OT* __restrict__ out, int64_t so, const float* __restrict__ gate,
                                                        int H, int N, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    if (row >= H * N) return;
    const int h = row / N, n = row - h * N;
    float acc = warp_dot<WT, XT>(W + ((size_t)h * N + n) * K, x + (size_t)h * sx, K, lane);
    if (lane == 0) {
        if (gate != nullptr) acc *= sigmoidf_(gate[h]);
        stf(out, (size_t)h * so + n, acc);
    }
}

// ------------------------------------------------------------------------------------------------ matrix-state recurrence
// Per head a state S [D, D] (key channel i, value channel j):  o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j]),
// then S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j], with w_t = exp(-exp(wraw_t + w0)).  A CTA owns WKV_J value
// channels of one head; thread (part, j) keeps WKV_CH rows of column j in registers.  Tokens are staged WKV_TB at a
// time; the parts' partial outputs meet in shared memory after each batch, summed in part order, so the arithmetic of
// a token does not depend on how the sequence was cut into launches.
constexpr int WKV_J = 32;   // template: TB tokens per staged batch (fewer when a wide head would not fit), CH state rows per thread

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Shared memory: two buffers of [r | k | w | v] for WKV_TB tokens (the next batch is copied in asynchronously while
// this one is computed; rows are padded to a multiple of 4 floats so that a thread reads its 16 key channels with
// 16-byte loads), then the parts' partial outputs.
template <int TB, int CH>
__global__ void __launch_bounds__(512) wkv_kernel(const CcSeqWkv a) {
    extern __shared__ float4 smw4[];
    float* sm = reinterpret_cast<float*>(smw4);
    const int D = a.D, P = (D + CH - 1) / CH, Dp = P * CH;
    const int buf_floats = TB * (3 * Dp + WKV_J);
    float* __restrict__ part = sm + 2 * buf_floats;    // [TB][P][J]
    const int h = blockIdx.x, j0 = blockIdx.y * WKV_J;
    const int tid = threadIdx.x, nth = blockDim.x, jl = tid % WKV_J, p = tid / WKV_J, j = j0 + jl;
    const int i0 = p * CH;
    const size_t HD = (size_t)a.H * D;
    float* S = a.state + (size_t)h * D * D;
    float st[CH], u[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const bool in = i0 + c < D && j < D;
        st[c] = in ? S[(size_t)(i0 + c) * D + j] : 0.f;
        u[c] = i0 + c < D ? a.u[(size_t)h * D + i0 + c] : 0.f;
    }
    // staging layout: with more threads than channels, thread = (token lane t0, channel ich)
    const int tstep = nth > D ? nth / D : 1, istep = nth > D ? D : nth;
    int t0 = nth > D ? tid / D : 0;
    const int ich = nth > D ? tid - t0 * D : tid;
    if (t0 >= tstep) t0 = 1 << 20;      // threads beyond the last whole token lane do not stage
    for (int idx = tid; idx < 2 * buf_floats; idx += nth) sm[idx] = 0.f;    // padding channels stay zero
    __syncthreads();
    auto fetch = [&](int tb, float* buf) {
        const int nt = min(TB, a.T - tb);
        // thread -> (token t0 + n * tstep, channel i): every thread copies, with one division per batch
        for (int t = t0; t < nt; t += tstep) {
            const size_t row = (size_t)(tb + t) * HD + (size_t)h * D;
            for (int i = ich; i < D; i += istep) {
                cp_async4(buf + t * Dp + i, a.r + row + i);
                cp_async4(buf + TB * Dp + t * Dp + i, a.k + row + i);
                cp_async4(buf + 2 * TB * Dp + t * Dp + i, a.wraw + row + i);
            }
        }
        for (int idx = tid; idx < nt * WKV_J; idx += nth) {
            const int t = idx / WKV_J, c = idx - t * WKV_J;
            if (j0 + c < D) cp_async4(buf + 3 * TB * Dp + idx, a.v + (size_t)(tb + t) * HD + (size_t)h * D + j0 + c);
        }
        cp_async_commit();
    };
    fetch(0, sm);
    int cur = 0;
    for (int tb = 0; tb < a.T; tb += TB, cur ^= 1) {
        float* buf = sm + cur * buf_floats;
        const int nt = min(TB, a.T - tb);
        if (tb + TB < a.T) { fetch(tb + TB, sm + (cur ^ 1) * buf_floats); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        float* ws = buf + 2 * TB * Dp;
        for (int i = ich; i < D; i += istep) {      // decay from its raw form, in place
            const float w0 = a.w0[(size_t)h * D + i];
            for (int t = t0; t < nt; t += tstep) ws[t * Dp + i] = expf(-expf(ws[t * Dp + i] + w0));
        }
        __syncthreads();
        const float* __restrict__ vs = buf + 3 * TB * Dp;
        const float* __restrict__ rb = buf + i0;
        const float* __restrict__ kb = buf + TB * Dp + i0;
        const float* __restrict__ wb = ws + i0;
#pragma unroll 4
        for (int t = 0; t < nt; ++t) {
            const float v = vs[t * WKV_J + jl];
            const float4* r4 = reinterpret_cast<const float4*>(rb + t * Dp);
            const float4* k4 = reinterpret_cast<const float4*>(kb + t * Dp);
            const float4* w4 = reinterpret_cast<const float4*>(wb + t * Dp);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c4 = 0; c4 < CH / 4; ++c4) {
                const float4 rv = r4[c4], kv4 = k4[c4], wv = w4[c4];
                const float rr[4] = {rv.x, rv.y, rv.z, rv.w}, kk[4] = {kv4.x, kv4.y, kv4.z, kv4.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int c = 4 * c4 + e;
                    const float kv = kk[e] * v;
                    acc[e] = fmaf(rr[e], fmaf(u[c], kv, st[c]), acc[e]);
                    st[c] = fmaf(ww[e], st[c], kv);
                }
            }
            part[(t * P + p) * WKV_J + jl] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * WKV_J; idx += nth) {
            const int t = idx / WKV_J, c = idx - t * WKV_J;
            if (j0 + c >= D) continue;
            float o = 0.f;
            for (int q = 0; q < P; ++q) o += part[(t * P + q) * WKV_J + c];
            a.o[(size_t)(tb + t) * HD + (size_t)h * D + j0 + c] = o;
        }
    }
#pragma unroll
    for (int c = 0; c < CH; ++c)
        if (i0 + c < D && j < D) S[(size_t)(i0 + c) * D + j] = st[c];
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * nw[h, :] * silu(graw[t, h, :]); a warp per (token, head).
template <typename ST>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ graw, int64_t ldg,
                                      const float* __restrict__ nw, ST* __restrict__ out, int T, int H, int D, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t th = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (th >= (size_t)T * H) return;
    const size_t t = th / H, h = th - t * H;
    const float* row = o + th * D;
    float ss = 0.f;
    for (int e = lane; e < D; e += 32) ss += row[e] * row[e];
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
    for (int e = lane; e < D; e += 32) {
        const float g = graw[t * ldg + h * D + e];
        stf(out, th * D + e, row[e] * rinv * nw[h * D + e] * (g * sigmoidf_(g)));
    }
}

// ------------------------------------------------------------------------------------------------ mixture of experts
// A warp per token.  Scores = softmax of the router logits over all outputs; choice = score + correction; experts
// outside the `keep` best groups (group score = its largest choice) cannot be chosen; the `top` largest choices win
// (the lower index on a tie); weights = the winners' scores divided by their sum.
__global__ void moe_route_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ correction,
                                 int32_t* __restrict__ ids, float* __restrict__ wts, int T, int n, int groups, int keep, int top,
                                 int sigmoid_scores, int group_top, int renormalize, float weight_scale) {
    extern __shared__ float smr[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int t = blockIdx.x * nw + warp;
    float* s = smr + (size_t)warp * (2 * n + groups);
    float* c = s + n;
    float* gm = c + n;
    if (t >= T) return;
    const float* z = logits + (size_t)t * ld;
    if (sigmoid_scores) {
        for (int i = lane; i < n; i += 32) { s[i] = sigmoidf_(z[i]); c[i] = s[i] + (correction ? correction[i] : 0.f); }
    } else {
        float mx = -INFINITY;
        for (int i = lane; i < n; i += 32) mx = fmaxf(mx, z[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int i = lane; i < n; i += 32) { const float e = expf(z[i] - mx); s[i] = e; sum += e; }
        sum = warp_sum(sum);
        for (int i = lane; i < n; i += 32) { s[i] = s[i] / sum; c[i] = s[i] + (correction ? correction[i] : 0.f); }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int gs = n / groups;
        for (int g = lane; g < groups; g += 32) {
            float m;
            if (group_top <= 1) {
                m = -INFINITY;
                for (int i = 0; i < gs; ++i) m = fmaxf(m, c[g * gs + i]);
            } else {   // the sum of the group's group_top largest choices, largest first
                m = 0.f;
                float last = INFINITY;
                int last_i = -1;
                for (int kk = 0; kk < group_top && kk < gs; ++kk) {
                    float bv = -INFINITY;
                    int bi = -1;
                    for (int i = 0; i < gs; ++i) {
                        const float v = c[g * gs + i];
                        const bool below = v < last || (v == last && i > last_i);
                        if (below && (bi < 0 || v > bv)) { bv = v; bi = i; }
                    }
                    m += bv;
                    last = bv;
                    last_i = bi;
                }
            }
            gm[g] = m;
        }
        __syncwarp();
        if (lane == 0) {   // the `keep` best groups are marked with NaN-free +inf, the others stay
            for (int kk = 0; kk < keep; ++kk) {
                int best = -1;
                float bv = -INFINITY;
                for (int g = 0; g < groups; ++g)
                    if (gm[g] != INFINITY && (best < 0 || gm[g] > bv)) { best = g; bv = gm[g]; }
                if (best >= 0) gm[best] = INFINITY;
            }
        }
        __syncwarp();
        for (int i = lane; i < n; i += 32)
            if (gm[i / gs] != INFINITY) c[i] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int kk = 0; kk < top; ++kk) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float v = c[i];
            if (v > bv || (v == bv && i < bi && v != -INFINITY)) { bv = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= n) bi = 0;   // fewer choosable experts than `top`: a configuration error, kept harmless
        if (lane == 0) {
            ids[(size_t)t * top + kk] = bi;
            wts[(size_t)t * top + kk] = s[bi];
            c[bi] = -INFINITY;
        }
        wsum += s[bi];
        __syncwarp();
    }
    __syncwarp();
    const float div = renormalize ? wsum + 1e-20f : 1.f;
    for (int kk = lane; kk < top; kk += 32) wts[(size_t)t * top + kk] = wts[(size_t)t * top + kk] / div * weight_scale;
}

// Groups the (token, choice) pairs of the real experts by expert: counts[e], and for every pair its row `slot` in the
// grouped order (-1 for an identity expert) with the row's token in perm[slot].  One CTA.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t* __restrict__ ids, int M, int top, int n_real,
                                                         int32_t* __restrict__ counts, int32_t* __restrict__ slot,
                                                         int32_t* __restrict__ perm) {
    extern __shared__ int smi[];
    int* cnt = smi;             // [n_real]
    int* off = cnt + n_real;    // [n_real]
    for (int e = threadIdx.x; e < n_real; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        const int e = ids[m];
        if (e < n_real) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_real; ++e) { off[e] = run; run += cnt[e]; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_real; e += blockDim.x) { counts[e] = cnt[e]; cnt[e] = 0; }
    __syncthreads();
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        const int e = ids[m];
        if (e < n_real) {
            const int s = off[e] + atomicAdd(&cnt[e], 1);
            slot[m] = s;
            perm[s] = m / top;
        } else {
            slot[m] = -1;
        }
    }
}

template <typename ST>
__global__ void gather_rows_kernel(const ST* __restrict__ src, const int32_t* __restrict__ perm, ST* __restrict__ dst, int E) {
    const size_t m = blockIdx.x;
    const ST* s = src + (size_t)perm[m] * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst[m * E + e] = s[e];
}

// One-token form of the experts: a block of 8 warps takes 8 rows of the chosen expert's gate and up matrices for
// one (token, choice) pair: act = silu(gate . h) * (up . h).  Pairs that chose an identity expert are skipped.
template <typename ST>
__global__ void __launch_bounds__(256) moe_expert_up_kernel(const ST* __restrict__ Wgu, const ST* __restrict__ h,
                                                            const int32_t* __restrict__ ids, ST* __restrict__ act,
                                                            int n_real, int F, int E, int kind, int top) {
    const int m = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = ids[m];
    const int f = blockIdx.x * 8 + warp;
    if (e >= n_real || f >= F) return;
    const int t = m / top;
    const ST* x = h + (size_t)t * E;
    const ST* wg = Wgu + ((size_t)e * 2 * F + f) * E;
    const float g = warp_dot<ST, ST>(wg, x, E, lane);
    const float u = warp_dot<ST, ST>(wg + (size_t)F * E, x, E, lane);
    if (lane == 0) stf(act, (size_t)m * F + f, unit_act(g, kind) * u);
}

template <typename ST>
__global__ void __launch_bounds__(256) moe_expert_down_kernel(const ST* __restrict__ Wd, const ST* __restrict__ act,
                                                              const int32_t* __restrict__ ids, float* __restrict__ y,
                                                              int n_real, int F, int E) {
    const int m = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = ids[m];
    const int n = blockIdx.x * 8 + warp;
    if (e >= n_real || n >= E) return;
    const float v = warp_dot<ST, ST>(Wd + ((size_t)e * E + n) * F, act + (size_t)m * F, F, lane);
    if (lane == 0) y[(size_t)m * E + n] = v;
}

// out[t] = sum_k w[t,k] * (expert row | h[t] for an identity expert) + sigmoid(sg[t]) * shared[t]
__global__ void moe_combine_kernel(const CcSeqMoeCombine a) {
    const int t = blockIdx.x, E = a.E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < a.top; ++k) {
            const size_t m = (size_t)t * a.top + k;
            const float w = a.wts[m];
            if (a.ids[m] >= a.n_real) acc += a.h != nullptr ? w * a.h[(size_t)t * E + e] : 0.f;
            else acc += w * a.y[(size_t)(a.slot ? a.slot[m] : (int)m) * E + e];
        }
        if (a.shared != nullptr) {
            const float g = a.sg ? sigmoidf_(a.sg[(size_t)t * a.ld_sg]) : 1.f;
            acc += g * a.shared[(size_t)t * E + e];
        }
        a.out[(size_t)t * E + e] = acc;
    }
}


// ------------------------------------------------------------------------------------------------ absorbed latent attention
// One token, all query heads over one shared row per position ([latent | rotated key part], Dk columns), whose first
// C columns are also the value row: a key tile is staged once and serves scores and values.  Grid = (runs of keys,
// groups of LD_HG heads); a warp owns one head, a lane one key of the 32-key tile (scores) and value columns
// lane, lane + 32, ... (weighted sum).  Keys are addressed by position (slot = position mod L, counted only if the
// slot records that position); the newest key comes from k_new.  Every run leaves (max, sum, weighted values) per
// head in the workspace; latent_combine_kernel merges the live runs in run order and appends the new row.
constexpr int LD_TK = 32, LD_HG = 8, LD_THREADS = 256;

__host__ __device__ inline int ld_stride(int width) {   // floats; a multiple of 4 whose quarter is odd
    const int w4 = (width + 3) / 4;
    return 4 * (w4 | 1);
}
__host__ __device__ inline int ld_keys_per_run(int L) { return LD_TK * ((L + LD_TK * 128 - 1) / (LD_TK * 128)); }   // at most 128 runs

template <typename CT, int NC>
__global__ void __launch_bounds__(LD_THREADS) latent_decode_kernel(const CcSeqLatentDecode a) {
    extern __shared__ float4 sml4[];
    float* sm = reinterpret_cast<float*>(sml4);
    const int Dk = a.Dk, C = a.C, Dkp = ld_stride(Dk), Dk4 = (Dk + 3) / 4;
    float* Qs = sm;                         // [LD_HG][Dkp]
    float* Ks = Qs + LD_HG * Dkp;           // [LD_TK][Dkp]
    float* Ps = Ks + LD_TK * Dkp;           // [LD_HG][LD_TK]
    int* src = (int*)(Ps + LD_HG * LD_TK);  // [LD_TK] slot, -1 = not a key, -2 = the new row
    const int p = a.input_pos[0], kpr = ld_keys_per_run(a.L);
    const int j_begin = blockIdx.x * kpr;
    if (j_begin > p) return;
    const int j_end = min(p, j_begin + kpr - 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h0 = blockIdx.y * LD_HG, nh = min(LD_HG, a.H - h0);
    const CT* kc = (const CT*)a.k_cache;
    const CT* kn = (const CT*)a.k_new;
    for (int idx = tid; idx < LD_HG * Dkp; idx += LD_THREADS) {
        const int h = idx / Dkp, d = idx - h * Dkp;
        Qs[idx] = (h < nh && d < Dk) ? a.q[(size_t)(h0 + h) * Dk + d] : 0.f;
    }
    for (int idx = tid; idx < LD_TK * (Dkp - Dk); idx += LD_THREADS) {   // padding columns stay zero
        const int r = idx / (Dkp - Dk), d = Dk + idx - r * (Dkp - Dk);
        Ks[r * Dkp + d] = 0.f;
    }
    float m = -INFINITY, l = 0.f, o[NC];
#pragma unroll
    for (int i = 0; i < NC; ++i) o[i] = 0.f;
    constexpr int VEC = 16 / (int)sizeof(CT);
    const bool vec = Dk % VEC == 0;
    for (int jt = j_begin; jt <= j_end; jt += LD_TK) {
        __syncthreads();
        if (tid < LD_TK) {
            const int j = jt + tid;
            int sl = -1;
            if (j <= j_end) {
                if (j == p) sl = -2;
                else { const int slot = j % a.L; sl = a.pos[slot] == j ? slot : -1; }
            }
            src[tid] = sl;
        }
        __syncthreads();
        if (vec) {
            const int per_row = Dk / VEC;
            for (int idx = tid; idx < LD_TK * per_row; idx += LD_THREADS) {
                const int r = idx / per_row, c = (idx - r * per_row) * VEC, sl = src[r];
                float* d = Ks + r * Dkp + c;
                if (sl == -1) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) d[e] = 0.f;
                } else {
                    const CT* row = sl == -2 ? kn : kc + (size_t)sl * Dk;
                    const uint4 u = __ldg(reinterpret_cast<const uint4*>(row + c));
                    const CT* e8 = reinterpret_cast<const CT*>(&u);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) d[e] = ldf(e8, e);
                }
            }
        } else {
            for (int idx = tid; idx < LD_TK * Dk; idx += LD_THREADS) {
                const int r = idx / Dk, c = idx - r * Dk, sl = src[r];
                Ks[r * Dkp + c] = sl == -1 ? 0.f : ldf(sl == -2 ? kn : kc + (size_t)sl * Dk, c);
            }
        }
        __syncthreads();
        if (warp < nh) {
            const float4* q4 = reinterpret_cast<const float4*>(Qs + warp * Dkp);
            const float4* k4 = reinterpret_cast<const float4*>(Ks + lane * Dkp);
            float s = 0.f;
#pragma unroll 4
            for (int d = 0; d < Dk4; ++d) {
                const float4 qv = q4[d], kv = k4[d];
                s = fmaf(qv.x, kv.x, s); s = fmaf(qv.y, kv.y, s); s = fmaf(qv.z, kv.z, s); s = fmaf(qv.w, kv.w, s);
            }
            const bool valid = src[lane] != -1;
            s = valid ? s * a.scale : -INFINITY;
            float mt = s;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, off));
            const float m_new = fmaxf(m, mt);
            if (m_new != -INFINITY) {
                const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
                const float pj = valid ? expf(s - m_new) : 0.f;
                l = l * corr + warp_sum(pj);
                Ps[warp * LD_TK + lane] = pj;
                __syncwarp();
#pragma unroll
                for (int i = 0; i < NC; ++i) o[i] *= corr;
                for (int j = 0; j < LD_TK; ++j) {
                    const float pw = Ps[warp * LD_TK + j];
                    const float* kr = Ks + j * Dkp + lane;
#pragma unroll
                    for (int i = 0; i < NC; ++i)
                        if (lane + 32 * i < C) o[i] = fmaf(pw, kr[32 * i], o[i]);
                }
                m = m_new;
                __syncwarp();
            }
        }
    }
    if (warp < nh) {
        float* w = (float*)a.workspace + ((size_t)blockIdx.x * a.H + h0 + warp) * (2 + C);
        if (lane == 0) { w[0] = m; w[1] = l; }
#pragma unroll
        for (int i = 0; i < NC; ++i)
            if (lane + 32 * i < C) w[2 + lane + 32 * i] = o[i];
    }
}

// One CTA per head: the global maximum over the live runs, then warp w sums runs w, w + 8, ... for value columns
// lane, lane + 32, ... and the eight partial sums meet in shared memory in warp order.
constexpr int LC_WARPS = 8;
template <typename CT, typename YT, int NC>
__global__ void __launch_bounds__(LC_WARPS * 32) latent_combine_kernel(const CcSeqLatentDecode a) {
    extern __shared__ float smc[];          // [LC_WARPS][C + 1]
    __shared__ float red[LC_WARPS];
    const int h = blockIdx.x, C = a.C, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = a.input_pos[0], kpr = ld_keys_per_run(a.L);
    const int runs = min(p / kpr + 1, (a.L + kpr - 1) / kpr);   // never more runs than the tile kernel has
    const float* ws = (const float*)a.workspace;
    const size_t stride = (size_t)a.H * (2 + C);
    const float* mine = ws + (size_t)h * (2 + C);
    float mx = -INFINITY;
    for (int r = tid; r < runs; r += LC_WARPS * 32) mx = fmaxf(mx, mine[r * stride]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < LC_WARPS; ++i) mx = fmaxf(mx, red[i]);
    if (a.sink != nullptr) mx = fmaxf(mx, a.sink[h]);   // the sink: a term of the denominator without key or value
    float l = 0.f, acc[NC];
#pragma unroll
    for (int i = 0; i < NC; ++i) acc[i] = 0.f;
    for (int r = warp; r < runs; r += LC_WARPS) {
        const float* w = mine + r * stride;
        const float mr = w[0];
        const float wt = mr == -INFINITY ? 0.f : expf(mr - mx);
        l = fmaf(wt, w[1], l);
#pragma unroll
        for (int i = 0; i < NC; ++i)
            if (lane + 32 * i < C) acc[i] = fmaf(wt, w[2 + lane + 32 * i], acc[i]);
    }
    float* out = smc + warp * (C + 1);
    if (lane == 0) out[C] = l;
#pragma unroll
    for (int i = 0; i < NC; ++i)
        if (lane + 32 * i < C) out[lane + 32 * i] = acc[i];
    __syncthreads();
    float lt = a.sink != nullptr ? expf(a.sink[h] - mx) : 0.f;
    for (int i = 0; i < LC_WARPS; ++i) lt += smc[i * (C + 1) + C];
    for (int c = tid; c < C; c += LC_WARPS * 32) {
        float v = 0.f;
        for (int i = 0; i < LC_WARPS; ++i) v += smc[i * (C + 1) + c];
        stf((YT*)a.y, (size_t)h * C + c, v / lt);
    }
    if (h == 0 && a.append) {   // the tile kernel took the newest key from k_new; nothing reads the cache here
        const int slot = p % a.L;
        CT* kc = (CT*)a.k_cache;
        const CT* kn = (const CT*)a.k_new;
        for (int d = tid; d < a.Dk; d += LC_WARPS * 32) kc[(size_t)slot * a.Dk + d] = kn[d];
        if (tid == 0) {
            if (a.mask != nullptr) a.mask[slot] = 1;
            const int old = a.pos[slot];
            a.pos[slot] = p;
            if (old < 0 && a.cache_cts != nullptr) atomicAdd(a.cache_cts, 1);
        }
    }
}

template <typename CT, typename YT, int NC>
static int launch_latent_decode(const CcSeqLatentDecode* a, cudaStream_t st) {
    const int Dkp = ld_stride(a->Dk);
    const size_t smem = sizeof(float) * ((size_t)(LD_HG + LD_TK) * Dkp + LD_HG * LD_TK) + sizeof(int) * LD_TK;
    auto kern = latent_decode_kernel<CT, NC>;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        configured = smem;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return cuda_check("latent_decode: shared memory");
    }
    const int kpr = ld_keys_per_run(a->L);
    dim3 grid((a->L + kpr - 1) / kpr, (a->H + LD_HG - 1) / LD_HG);
    kern<<<grid, LD_THREADS, smem, st>>>(*a);
    latent_combine_kernel<CT, YT, NC><<<a->H, LC_WARPS * 32, sizeof(float) * LC_WARPS * (a->C + 1), st>>>(*a);
    return cuda_check("latent_decode kernels");
}

template <typename CT, typename YT>
static int dispatch_latent_decode(const CcSeqLatentDecode* a, cudaStream_t st) {
    const int nc = (a->C + 31) / 32;
    if (nc <= 2) return launch_latent_decode<CT, YT, 2>(a, st);
    if (nc <= 4) return launch_latent_decode<CT, YT, 4>(a, st);
    if (nc <= 8) return launch_latent_decode<CT, YT, 8>(a, st);
    if (nc <= 16) return launch_latent_decode<CT, YT, 16>(a, st);
    if (nc <= 32) return launch_latent_decode<CT, YT, 32>(a, st);
    return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "latent_decode: value rows wider than 1024");
}

// ------------------------------------------------------------------------------------------------ one-token products
// Several independent matrix-vector products in one launch: job j is out_j = W_j xin_j with xin_j either the given
// vector or, read from an fp32 row, act(src[off_gate + k]) * src[off_up + k] (the input side of a gated unit, or an
// activation alone when off_up < 0).  The input is staged in shared memory rounded to the weights' type, as the
// prompt path rounds what it hands to a product.  8 rows per CTA, a warp per row, 16-byte weight loads.
__device__ __forceinline__ float round_to(float v, const float*) { return v; }
__device__ __forceinline__ float round_to(float v, const bf16*) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename WT>
__global__ void __launch_bounds__(256) gemv_multi_kernel(const CcSeqGemvMulti g) {
    extern __shared__ float4 smg4[];
    float* xs = reinterpret_cast<float*>(smg4);
    int j = 0, first = 0;
    while (j + 1 < g.n_jobs && (int)blockIdx.x >= first + (g.job[j].N + 7) / 8) { first += (g.job[j].N + 7) / 8; ++j; }
    const CcSeqGemvJob& jb = g.job[j];
    const int K = jb.K, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const WT* W = (const WT*)jb.W;
    if (jb.kind != CC_ACT_NONE || jb.off_up >= 0) {
        const float* src = (const float*)jb.x;
        for (int k = tid; k < K; k += 256) {
            float v = unit_act(src[jb.off_gate + k], jb.kind);
            if (jb.off_up >= 0) v *= src[jb.off_up + k];
            xs[k] = round_to(v, W);
        }
    } else if (jb.x_dtype == CC_DT_F32) {
        for (int k = tid; k < K; k += 256) xs[k] = round_to(((const float*)jb.x)[k], W);
    } else {
        for (int k = tid; k < K; k += 256) xs[k] = __bfloat162float(((const bf16*)jb.x)[k]);
    }
    __syncthreads();
    const int n = ((int)blockIdx.x - first) * 8 + warp;
    if (n >= jb.N) return;
    const WT* w = W + (size_t)n * K;
    constexpr int VEC = 16 / (int)sizeof(WT);
    float acc = 0.f;
    if (K % VEC == 0) {
        const uint4* w16 = reinterpret_cast<const uint4*>(w);
        const int nv = K / VEC;
#pragma unroll 4
        for (int i = lane; i < nv; i += 32) {
            const uint4 u = __ldg(w16 + i);
            const WT* e = reinterpret_cast<const WT*>(&u);
            const float4* x4 = reinterpret_cast<const float4*>(xs + i * VEC);
#pragma unroll
            for (int q = 0; q < VEC / 4; ++q) {
                const float4 xv = x4[q];
                acc = fmaf(ldf(e, 4 * q + 0), xv.x, acc);
                acc = fmaf(ldf(e, 4 * q + 1), xv.y, acc);
                acc = fmaf(ldf(e, 4 * q + 2), xv.z, acc);
                acc = fmaf(ldf(e, 4 * q + 3), xv.w, acc);
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(ldf(w, k), xs[k], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) ((float*)jb.out)[n] = acc;
}

template <int TB, int CH>
static int launch_wkv(const CcSeqWkv* a, cudaStream_t st) {
    const int P = (a->D + CH - 1) / CH;
    const size_t smem = sizeof(float) * (2 * (size_t)TB * (3 * P * CH + WKV_J) + (size_t)TB * P * WKV_J);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        configured = smem;
        if (cudaFuncSetAttribute(wkv_kernel<TB, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return cuda_check("wkv: shared memory");
    }
    dim3 grid(a->H, (a->D + WKV_J - 1) / WKV_J);
    wkv_kernel<TB, CH><<<grid, P * WKV_J, smem, st>>>(*a);
    return cuda_check("wkv_kernel");
}

// 8 state rows per thread up to 128-wide heads (at most 512 threads), 16 above; the token batch shrinks until two
// staging buffers and the partial outputs fit in 160 KB.
template <int CH>
static int dispatch_wkv(const CcSeqWkv* a, cudaStream_t st) {
    const int P = (a->D + CH - 1) / CH;
    auto bytes = [&](int tb) { return sizeof(float) * (2 * (size_t)tb * (3 * P * CH + WKV_J) + (size_t)tb * P * WKV_J); };
    if (bytes(32) <= 160 * 1024) return launch_wkv<32, CH>(a, st);
    if (bytes(16) <= 160 * 1024) return launch_wkv<16, CH>(a, st);
    return launch_wkv<8, CH>(a, st);
}


}  // namespace ccm

using namespace ccm;

#define CCM_ST(dt, CALL)                                                \
    do {                                                                \
        if ((dt) == CC_DT_F32) { CALL(float); }                         \
        else if ((dt) == CC_DT_BF16) { CALL(bf16); }                    \
        else return fail(CC_SEQ_ERR_INVALID_ARG, "unknown element type"); \
    } while (0)

extern "C" {

int cc_seq_embed_rows(const int32_t* tokens, const void* embed, int32_t table_dtype, float* x, int32_t T, int32_t E,
                      float scale, void* stream) {
    if (!tokens || !embed || !x || T < 1 || E < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "embed_rows: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST) embed_rows_kernel<ST><<<T, 256, 0, st>>>(tokens, (const ST*)embed, x, E, scale)
    CCM_ST(table_dtype, CALL);
#undef CALL
    return cuda_check("embed_rows_kernel");
}

int cc_seq_gated_group_norm(const CcSeqGatedNorm* g, void* stream) {
    if (!g || !g->x || g->T < 1 || g->E < 1 || g->groups < 1 || g->E % g->groups)
        return fail(CC_SEQ_ERR_INVALID_ARG, "gated_group_norm: bad argument");
    if (g->shift_state && (g->T != 1 || g->rows || !g->w || !g->shift_mu || (g->n_mix > 0 && (!g->mix_state || !g->mix_mu || !g->mixes))))
        return fail(CC_SEQ_ERR_INVALID_ARG, "gated_group_norm: the fused token shift serves one token");
    const size_t smem = sizeof(float) * (size_t)(g->E / g->groups);
    if (smem > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "gated_group_norm: groups longer than 51200");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST)                                                                                                     \
    {                                                                                                                \
        auto kern = gated_group_norm_kernel<ST>;                                                                     \
        static size_t configured = 48 * 1024;                                                                        \
        if (smem > configured) {                                                                                     \
            configured = smem;                                                                                       \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)   \
                return cuda_check("gated_group_norm: shared memory");                                                \
        }                                                                                                            \
        kern<<<dim3(g->T, g->groups), 256, smem, st>>>(*g);                                                          \
    }
    CCM_ST(g->act_dtype, CALL);
#undef CALL
    return cuda_check("gated_group_norm_kernel");
}

int cc_seq_token_shift(const float* h, float* state, const float* mu, void* out, int32_t out_dtype, float* outf,
                       int32_t T, int32_t E, int32_t n, void* stream) {
    if (!h || !state || !mu || T < 1 || E < 1 || n < 1 || (!out && !outf))
        return fail(CC_SEQ_ERR_INVALID_ARG, "token_shift: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST) token_shift_kernel<ST><<<T, 256, 0, st>>>(h, state, mu, (ST*)out, outf, T, E, n)
    CCM_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("token_shift_kernel");
}

int cc_seq_gated_unit(const float* in, int64_t ld, int32_t off_gate, int32_t off_up, void* out, int32_t out_dtype,
                      int32_t T, int32_t F, int32_t kind, void* stream) {
    if (!in || !out || T < 1 || F < 1 || kind < CC_ACT_NONE || kind > CC_ACT_LAST)
        return fail(CC_SEQ_ERR_INVALID_ARG, "gated_unit: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 nb((F + 255) / 256, T < 4096 ? T : 4096);
#define CALL(ST) gated_unit_kernel<ST><<<nb, 256, 0, st>>>(in, ld, off_gate, off_up, (ST*)out, T, F, kind)
    CCM_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("gated_unit_kernel");
}

int cc_seq_latent_prepare(const CcSeqLatentPrep* a, void* stream) {
    if (!a || !a->in || !a->krow || !a->wkv || !a->input_pos || a->T < 1 || a->kv_rank < 1 || a->rot_dim < 0 ||
        a->rot_dims < 0 || a->rot_dims > a->rot_dim || (a->rot_dims & 1) || (a->rot_dims && !a->inv_freq) ||
        (a->q_rank > 0 && (!a->cq || !a->wq)))
        return fail(CC_SEQ_ERR_INVALID_ARG, "latent_prepare: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST) latent_prepare_kernel<ST><<<a->T, 256, 0, st>>>(*a)
    CCM_ST(a->dtype, CALL);
#undef CALL
    return cuda_check("latent_prepare_kernel");
}

int cc_seq_rope_heads(float* q, int64_t ld, const int32_t* input_pos, const float* inv_freq, int32_t T, int32_t H,
                      int32_t head_w, int32_t off, int32_t seg, int32_t dims, float* tail, int64_t tail_ld,
                      int32_t tail_off, int32_t interleaved, void* stream) {
    if (!q || !input_pos || T < 1 || H < 1 || dims < 0 || (dims & 1) || dims > seg || off + seg > head_w ||
        (dims && !inv_freq))
        return fail(CC_SEQ_ERR_INVALID_ARG, "rope_heads: bad argument");
    rope_heads_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(q, ld, input_pos, inv_freq, H, head_w, off, seg, dims, tail,
                                                           tail_ld, tail_off, T, interleaved);
    return cuda_check("rope_heads_kernel");
}

int cc_seq_latent_expand(const CcSeqLatentExpand* a, void* stream) {
    if (!a || a->n_old < 0 || a->n_new < 0 || a->n_old + a->n_new < 1 || a->H < 1 || a->D < 0 || a->V < 1 || a->R < 0 ||
        (a->n_old && (!a->kv_old || !a->lat_old || !a->k_old || !a->v_old)) ||
        (a->n_new && (!a->kv_new || !a->lat_new || !a->k_new || !a->v_new)))
        return fail(CC_SEQ_ERR_INVALID_ARG, "latent_expand: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST) latent_expand_kernel<ST><<<a->n_old + a->n_new, 256, 0, st>>>(*a)
    CCM_ST(a->dtype, CALL);
#undef CALL
    return cuda_check("latent_expand_kernel");
}

int cc_seq_head_gate(void* y, int32_t dtype, const float* g, int64_t ldg, int32_t T, int32_t H, int32_t V, void* stream) {
    if (!y || !g || T < 1 || H < 1 || V < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "head_gate: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST) head_gate_kernel<ST><<<T, dim3(32, 8), 0, st>>>((ST*)y, g, ldg, T, H, V)
    CCM_ST(dtype, CALL);
#undef CALL
    return cuda_check("head_gate_kernel");
}

int cc_seq_head_gemv(const void* W, int32_t w_dtype, const void* x, int32_t x_dtype, int64_t sx, void* out,
                     int32_t out_dtype, int64_t so, const float* gate, int32_t H, int32_t N, int32_t K, void* stream) {
    if (!W || !x || !out || H < 1 || N < 1 || K < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "head_gemv: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const int nb = (H * N + 7) / 8;
    const bool wb = w_dtype == CC_DT_BF16, xb = x_dtype == CC_DT_BF16, ob = out_dtype == CC_DT_BF16;
#define HG(WT, XT, OT) head_gemv_kernel<WT, XT, OT><<<nb, 256, 0, st>>>((const WT*)W, (const XT*)x, sx, (OT*)out, so, gate, H, N, K)
    if (wb && xb && ob) HG(bf16, bf16, bf16);
    else if (wb && xb && !ob) HG(bf16, bf16, float);
    else if (wb && !xb && ob) HG(bf16, float, bf16);
    else if (wb && !xb && !ob) HG(bf16, float, float);
    else if (!wb && !xb && !ob) HG(float, float, float);
    else return fail(CC_SEQ_ERR_INVALID_ARG, "head_gemv: unsupported combination of element types");
#undef HG
    return cuda_check("head_gemv_kernel");
}

int cc_seq_wkv(const CcSeqWkv* a, void* stream) {
    if (!a || !a->r || !a->k || !a->v || !a->wraw || !a->w0 || !a->u || !a->state || !a->o || a->T < 1 || a->H < 1 || a->D < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "wkv: bad argument");
    if (a->D > 256) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "wkv: head size above 256");
    cudaStream_t st = (cudaStream_t)stream;
    return a->D <= 128 ? dispatch_wkv<8>(a, st) : dispatch_wkv<16>(a, st);
}

int cc_seq_head_norm_gate(const float* o, const float* graw, int64_t ldg, const float* nw, void* out, int32_t out_dtype,
                          int32_t T, int32_t H, int32_t D, float eps, void* stream) {
    if (!o || !graw || !nw || !out || T < 1 || H < 1 || D < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "head_norm_gate: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const int nb = (int)(((size_t)T * H + 7) / 8);
#define CALL(ST) head_norm_gate_kernel<ST><<<nb, 256, 0, st>>>(o, graw, ldg, nw, (ST*)out, T, H, D, eps)
    CCM_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("head_norm_gate_kernel");
}

int cc_seq_moe_route(const float* logits, int64_t ld, const float* correction, int32_t* ids, float* wts, int32_t T,
                     int32_t n, int32_t groups, int32_t keep, int32_t top, int32_t sigmoid_scores, int32_t group_top,
                     int32_t renormalize, float weight_scale, void* stream) {
    if (!logits || !ids || !wts || T < 1 || n < 1 || groups < 1 || n % groups || keep < 1 || top < 1 || top > n || group_top < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "moe_route: bad argument");
    const int warps = 4;
    const size_t smem = sizeof(float) * (size_t)warps * (2 * n + groups);
    if (smem > 48 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "moe_route: too many experts");
    moe_route_kernel<<<(T + warps - 1) / warps, warps * 32, smem, (cudaStream_t)stream>>>(logits, ld, correction, ids, wts, T,
                                                                                        n, groups, keep, top, sigmoid_scores,
                                                                                        group_top, renormalize, weight_scale);
    return cuda_check("moe_route_kernel");
}

int cc_seq_moe_group(const int32_t* ids, int32_t M, int32_t top, int32_t n_real, int32_t* counts, int32_t* slot,
                     int32_t* perm, void* stream) {
    if (!ids || !counts || !slot || !perm || M < 1 || top < 1 || n_real < 1 || n_real > 4096)
        return fail(CC_SEQ_ERR_INVALID_ARG, "moe_group: bad argument");
    moe_group_kernel<<<1, 1024, sizeof(int) * 2 * n_real, (cudaStream_t)stream>>>(ids, M, top, n_real, counts, slot, perm);
    return cuda_check("moe_group_kernel");
}

int cc_seq_gather_rows(const void* src, const int32_t* perm, void* dst, int32_t dtype, int32_t M, int32_t E, void* stream) {
    if (!src || !perm || !dst || M < 1 || E < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "gather_rows: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST) gather_rows_kernel<ST><<<M, 256, 0, st>>>((const ST*)src, perm, (ST*)dst, E)
    CCM_ST(dtype, CALL);
#undef CALL
    return cuda_check("gather_rows_kernel");
}

int cc_seq_moe_expert_tokens(const void* Wgu, const void* Wd, const void* h, const int32_t* ids, void* act, float* y,
                             int32_t dtype, int32_t T, int32_t top, int32_t n_real, int32_t F, int32_t E, int32_t kind,
                             void* stream) {
    if (!Wgu || !Wd || !h || !ids || !act || !y || T < 1 || top < 1 || F < 1 || E < 1 || (size_t)T * top > 65535)
        return fail(CC_SEQ_ERR_INVALID_ARG, "moe_expert_tokens: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 gu((F + 7) / 8, T * top, 1), gd((E + 7) / 8, T * top, 1);
#define CALL(ST)                                                                                                       \
    {                                                                                                                  \
        moe_expert_up_kernel<ST><<<gu, 256, 0, st>>>((const ST*)Wgu, (const ST*)h, ids, (ST*)act, n_real, F, E, kind, top); \
        moe_expert_down_kernel<ST><<<gd, 256, 0, st>>>((const ST*)Wd, (const ST*)act, ids, y, n_real, F, E);           \
    }
    CCM_ST(dtype, CALL);
#undef CALL
    return cuda_check("moe_expert kernels");
}

uint64_t cc_seq_latent_decode_workspace(int32_t H, int32_t C, int32_t L) {
    const int kpr = ld_keys_per_run(L);
    return sizeof(float) * (uint64_t)((L + kpr - 1) / kpr) * (uint64_t)H * (2 + (uint64_t)C);
}

int cc_seq_latent_decode(const CcSeqLatentDecode* a, void* stream) {
    if (!a || !a->q || !a->k_new || !a->k_cache || !a->pos || !a->input_pos || !a->y || a->H < 1 || a->Dk < 1 || a->C < 1 ||
        a->C > a->Dk || a->L < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "latent_decode: bad argument");
    if (!a->workspace || a->workspace_bytes < cc_seq_latent_decode_workspace(a->H, a->C, a->L))
        return fail(CC_SEQ_ERR_INVALID_ARG, "latent_decode: workspace missing or too small");
    if ((size_t)(LD_HG + LD_TK) * ld_stride(a->Dk) * 4 > 200 * 1024)
        return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "latent_decode: rows wider than 1280");
    cudaStream_t st = (cudaStream_t)stream;
    const bool cb = a->cache_dtype == CC_DT_BF16, yb = a->y_dtype == CC_DT_BF16;
    if (a->cache_dtype != CC_DT_BF16 && a->cache_dtype != CC_DT_F32) return fail(CC_SEQ_ERR_INVALID_ARG, "unknown element type");
    if (cb && yb) return dispatch_latent_decode<bf16, bf16>(a, st);
    if (cb && !yb) return dispatch_latent_decode<bf16, float>(a, st);
    if (!cb && yb) return dispatch_latent_decode<float, bf16>(a, st);
    return dispatch_latent_decode<float, float>(a, st);
}

int cc_seq_gemv_multi(const CcSeqGemvMulti* g, void* stream) {
    if (!g || g->n_jobs < 1 || g->n_jobs > CC_GEMV_MAX_JOBS) return fail(CC_SEQ_ERR_INVALID_ARG, "gemv_multi: bad job count");
    int blocks = 0, kmax = 0;
    for (int j = 0; j < g->n_jobs; ++j) {
        const CcSeqGemvJob& b = g->job[j];
        if (!b.x || !b.W || !b.out || b.N < 1 || b.K < 1 || b.kind < CC_ACT_NONE || b.kind > CC_ACT_LAST ||
            ((b.kind != CC_ACT_NONE || b.off_up >= 0) && b.x_dtype != CC_DT_F32))
            return fail(CC_SEQ_ERR_INVALID_ARG, "gemv_multi: bad job");
        blocks += (b.N + 7) / 8;
        kmax = b.K > kmax ? b.K : kmax;
    }
    const size_t smem = sizeof(float) * (size_t)((kmax + 3) & ~3);
    if (smem > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "gemv_multi: input longer than 51200");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(ST)                                                                                                   \
    {                                                                                                              \
        auto kern = gemv_multi_kernel<ST>;                                                                         \
        static size_t configured = 48 * 1024;                                                                      \
        if (smem > configured) {                                                                                   \
            configured = smem;                                                                                     \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
                return cuda_check("gemv_multi: shared memory");                                                    \
        }                                                                                                          \
        kern<<<blocks, 256, smem, st>>>(*g);                                                                       \
    }
    CCM_ST(g->w_dtype, CALL);
#undef CALL
    return cuda_check("gemv_multi_kernel");
}

int cc_seq_moe_combine(const CcSeqMoeCombine* a, void* stream) {
    if (!a || !a->ids || !a->wts || !a->y || !a->out || a->T < 1 || a->E < 1 || a->top < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "moe_combine: bad argument");   // h may be NULL when no id reaches n_real
    moe_combine_kernel<<<a->T, 256, 0, (cudaStream_t)stream>>>(*a);
    return cuda_check("moe_combine_kernel");
}

}  // extern "C"
