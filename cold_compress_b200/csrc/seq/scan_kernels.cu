// scan_kernels.cu -- sequence kernels, third part of include/cc_b200_seq.h: norms after the sum with layer scale, a
// second (pre-normed) sublayer input and a weighted average over the depth; short causal convolutions whose tail is
// carried from step to step; a state-space scan (scalar decay per head) and a delta-rule scan (decay per key channel),
// both with the state of a (head, 32 value columns) tile in registers; gated group norms; rotations of query, key and
// value heads; the logit soft cap.
//
// Arithmetic rule (as in seq_kernels.cu): everything here is fp32 whatever the storage type of the neighbours; expf /
// tanhf / sincosf / log1pf are the accurate versions.  Both scans are exactly sequential over tokens and sum in a
// fixed order, so a sequence gives the same bits however it is cut into steps.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../../include/cc_b200_seq.h"

namespace ccs {
int fail(int code, const char* msg);
int cuda_check(const char* where);
}  // namespace ccs

namespace ccn {
using ccs::cuda_check;
using ccs::fail;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }

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

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// ------------------------------------------------------------------------------------------------ norm after the sum
// One CTA per row.  The sum is kept in shared memory so that the variance is the mean of the squared deviations from
// the mean (two passes), not a difference of two large numbers.  Every pass is a chain of dependent loads, so a step
// of few rows runs 1024 threads per row (few loads per thread) and a long one 256 (more rows per SM).
template <typename AT>
__global__ void __launch_bounds__(1024) sum_norm_kernel(const CcSeqSumNorm a) {
    extern __shared__ float sn_s[];
    __shared__ float red[32];
    const int t = blockIdx.x, E = a.E, tid = threadIdx.x, nth = blockDim.x;
    const size_t src = a.rows != nullptr ? (size_t)a.rows[t] : (size_t)t;
    const float* x = a.x != nullptr ? a.x + src * E : nullptr;
    const float* y = a.y != nullptr ? a.y + src * a.ldy : nullptr;
    const float* y2 = a.y2 != nullptr ? a.y2 + src * a.ldy2 : nullptr;
    float ry = 1.f, ry2 = 1.f;
    if (y != nullptr && a.y_norm_w != nullptr) {
        float ss = 0.f;
        for (int e = tid; e < E; e += nth) ss = fmaf(y[e], y[e], ss);
        ry = 1.0f / sqrtf(block_sum(ss, red) / (float)E + a.eps);
    }
    if (y2 != nullptr && a.y2_norm_w != nullptr) {
        float ss = 0.f;
        for (int e = tid; e < E; e += nth) ss = fmaf(y2[e], y2[e], ss);
        ry2 = 1.0f / sqrtf(block_sum(ss, red) / (float)E + a.eps);
    }
    float sum = 0.f;
    for (int e = tid; e < E; e += nth) {
        float v = x != nullptr ? a.alpha * x[e] : 0.f;
        if (y != nullptr) {
            float r = y[e] * ry;
            if (a.y_norm_w != nullptr) r *= a.y_norm_w[e];
            if (y2 != nullptr) {
                float r2 = y2[e] * ry2;
                if (a.y2_norm_w != nullptr) r2 *= a.y2_norm_w[e];
                r += r2;
            }
            r *= a.y_coef;
            if (a.y_scale != nullptr) r *= a.y_scale[e];
            v += r;
        }
        sn_s[e] = v;
        sum += v;
    }
    const float mean = a.center ? block_sum(sum, red) / (float)E : 0.f;
    float ss = 0.f;
    for (int e = tid; e < E; e += nth) {
        const float d = sn_s[e] - mean;
        ss = fmaf(d, d, ss);
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)E + a.eps);
    AT* act = (AT*)a.out_act;
    for (int e = tid; e < E; e += nth) {
        float r = (sn_s[e] - mean) * rinv * (a.w[e] + a.gain_offset);
        const size_t o = (size_t)t * E + e;
        if (a.out != nullptr) a.out[o] = r;
        if (a.coef != nullptr) {
            float m = 0.f;
            for (int j = 0; j < a.n_prev; ++j) m = fmaf(a.coef[j], a.stack[(size_t)j * a.stack_stride + o], m);
            r = fmaf(a.coef[a.n_prev], r, m);
            a.mix[o] = r;
        }
        if (act != nullptr) stf(act, o, r);
    }
}

// ------------------------------------------------------------------------------------------------ short convolution
// A thread per (token, channel); the taps are read through L1 (each input is read `taps` times).  With `tail_too`
// (one token per channel column, i.e. gridDim.x == 1 and T == 1) the same thread then moves the tail on.
__device__ __forceinline__ float conv_input(const float* u, int64_t ldu, const float* tail, int C, int taps, int t, int c) {
    return t >= 0 ? u[(size_t)t * ldu + c] : tail[(size_t)(taps - 1 + t) * C + c];
}

__device__ __forceinline__ void conv_move_tail(const float* u, int64_t ldu, float* tail, int T, int C, int taps, int c) {
    // new tail[s] = input at time T - (taps - 1) + s.  Entry s reads old entry s + T (> s): ascending s is safe in place.
    for (int s = 0; s < taps - 1; ++s) tail[(size_t)s * C + c] = conv_input(u, ldu, tail, C, taps, T - (taps - 1) + s, c);
}

__global__ void short_conv_kernel(const float* __restrict__ u, int64_t ldu, const float* __restrict__ w,
                                  const float* __restrict__ bias, float* tail, float* __restrict__ out, int64_t ldo, int T,
                                  int C, int taps, int act, int tail_too) {
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float acc = bias != nullptr ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) acc = fmaf(w[(size_t)c * taps + j], conv_input(u, ldu, tail, C, taps, t - taps + 1 + j, c), acc);
    out[(size_t)t * ldo + c] = unit_act(acc, act);
    if (tail_too) conv_move_tail(u, ldu, tail, T, C, taps, c);
}

__global__ void conv_tail_kernel(const float* __restrict__ u, int64_t ldu, float* tail, int T, int C, int taps) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) conv_move_tail(u, ldu, tail, T, C, taps, c);
}

// ------------------------------------------------------------------------------------------------ state-space scan
// CTA = one head x 32 value columns; warp p keeps state rows p * CH .. p * CH + CH - 1 of its lane's column in
// registers.  Tokens are staged TB at a time through two cp.async buffers (B and C rows, the 32 x values, the raw step
// size); the step size and the decay of a token are computed once per batch; the warps' partial read-outs go to shared
// memory and are summed in warp order after the batch.
constexpr int SCAN_J = 32;

template <int CH, int TB>
__global__ void __launch_bounds__(512) ssd_scan_kernel(const CcSeqSsdScan a) {
    extern __shared__ float4 sm_ssd4[];
    float* sm = reinterpret_cast<float*>(sm_ssd4);
    const int N = a.N, P = (N + CH - 1) / CH, Np = P * CH;
    const int buf_floats = TB * (2 * Np + SCAN_J + 2);
    float* __restrict__ part = sm + 2 * buf_floats;   // [TB][P][32]
    const int h = blockIdx.x, j0 = blockIdx.y * SCAN_J, g = h / (a.H / a.G);
    const int tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, p = tid >> 5, j = j0 + lane;
    const int n0 = p * CH;
    float* S = a.state + (size_t)h * N * a.V;
    float st[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) st[c] = (n0 + c < N && j < a.V) ? S[(size_t)(n0 + c) * a.V + j] : 0.f;
    for (int idx = tid; idx < 2 * buf_floats; idx += nth) sm[idx] = 0.f;   // padding rows and columns stay zero
    __syncthreads();
    const float lam = expf(a.A_log[h]), bias = a.dt_bias[h], skip = a.D != nullptr ? a.D[h] : 0.f;
    auto fetch = [&](int tb, float* buf) {
        const int nt = min(TB, a.T - tb);
        for (int idx = tid; idx < nt * N; idx += nth) {
            const int t = idx / N, n = idx - t * N;
            const size_t row = (size_t)(tb + t) * a.ldbc + (size_t)g * N + n;
            cp_async4(buf + t * Np + n, a.B + row);
            cp_async4(buf + TB * Np + t * Np + n, a.C + row);
        }
        for (int idx = tid; idx < nt * SCAN_J; idx += nth) {
            const int t = idx / SCAN_J, c = idx - t * SCAN_J;
            if (j0 + c < a.V) cp_async4(buf + 2 * TB * Np + idx, a.x + (size_t)(tb + t) * a.ldx + (size_t)h * a.V + j0 + c);
        }
        if (tid < nt) cp_async4(buf + 2 * TB * Np + TB * SCAN_J + tid, a.dt_raw + (size_t)(tb + tid) * a.lddt + h);
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
        float* dts = buf + 2 * TB * Np + TB * SCAN_J;
        float* decs = dts + TB;
        if (tid < nt) {
            const float dt = softplusf_(dts[tid] + bias);
            dts[tid] = dt;
            decs[tid] = expf(-lam * dt);
        }
        __syncthreads();
        const float* __restrict__ Bs = buf + n0;
        const float* __restrict__ Cs = buf + TB * Np + n0;
        const float* __restrict__ xs = buf + 2 * TB * Np;
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            const float xv = xs[t * SCAN_J + lane], dec = decs[t];
            const float dtx = dts[t] * xv;
            float acc = p == 0 ? skip * xv : 0.f;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                st[c] = fmaf(dec, st[c], Bs[t * Np + c] * dtx);
                acc = fmaf(Cs[t * Np + c], st[c], acc);
            }
            part[(t * P + p) * SCAN_J + lane] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < nt * SCAN_J; idx += nth) {
            const int t = idx / SCAN_J, c = idx - t * SCAN_J;
            if (j0 + c >= a.V) continue;
            float y = 0.f;
            for (int q = 0; q < P; ++q) y += part[(t * P + q) * SCAN_J + c];
            a.y[(size_t)(tb + t) * a.H * a.V + (size_t)h * a.V + j0 + c] = y;
        }
    }
#pragma unroll
    for (int c = 0; c < CH; ++c)
        if (n0 + c < N && j < a.V) S[(size_t)(n0 + c) * a.V + j] = st[c];
}

// ------------------------------------------------------------------------------------------------ delta-rule scan
// CTA = one head x 32 value columns.  A warp owns 4 NC columns; 8 lanes share NC columns and each keeps CH consecutive
// state rows of them in registers, so the two sums over the rows that a token needs (S^T k and S^T q over the decayed state)
// are three shuffle steps inside the warp: no shared-memory partials and no barrier per token, the warps run
// independently through a batch.  Per batch of TB tokens (two cp.async buffers) a warp per token turns the staged rows
// (unless a separate launch has prepared them: a.prepared) into what the recurrence reads: q and k as unit vectors (q also times q_scale), their dot product, the decays
// exp(-exp(A_log) softplus(.)) and beta.  Per token: decay the rows, the two sums, u = beta (v - S^T k), S += k u^T,
// and o = S^T q + (q . k) u, which is the read-out of the state after the write.  The q / k / decay vectors lie in
// shared memory in runs of CH with 4 floats of padding, so that the 8 lanes' 16-byte loads fall into different banks.
#ifndef CC_DELTA_NC
#define CC_DELTA_NC 1
#endif
// lanes per column, columns per lane.  Two columns per lane halve the shared-memory reads per column but leave half
// as many warps to overlap the per-token chain of dependent steps: measured slower (2.04 against 1.69 ms for 4096
// tokens of 8 heads x 128 x 128), so one column per lane is the default.
constexpr int DL_PARTS = 8, DL_NC = CC_DELTA_NC;

// One token's rows turned into what the recurrence reads, by one warp: q and k as unit vectors (q times q_scale), the
// decays, and (returned) q . k.  The same code serves the scan's own batches and the separate launch that long steps
// use, so both give the same bits.
template <typename LQ, typename LK, typename LA, typename SQ, typename SK, typename SG>
__device__ __forceinline__ float delta_prepare_rows(int D, int lane, float q_scale, float unit_eps, float lam,
                                                    const float* __restrict__ dt_bias, LQ ldq, LK ldk, LA lda, SQ stq, SK stk, SG stg) {
    float sq = 0.f, sk = 0.f;
    for (int n = lane; n < D; n += 32) { const float qv = ldq(n), kv = ldk(n); sq = fmaf(qv, qv, sq); sk = fmaf(kv, kv, sk); }
    const float rq = q_scale / sqrtf(warp_sum(sq) + unit_eps), rk = 1.0f / sqrtf(warp_sum(sk) + unit_eps);
    float dot = 0.f;
    for (int n = lane; n < D; n += 32) {
        const float qn = ldq(n) * rq, kn = ldk(n) * rk;
        stq(n, qn);
        stk(n, kn);
        dot = fmaf(qn, kn, dot);
        stg(n, expf(-lam * softplusf_(lda(n) + dt_bias[n])));
    }
    return warp_sum(dot);
}

// The preparation alone, a warp per (token, head), for steps long enough that it pays to spread it over the GPU
// instead of repeating it in every column tile of the scan: qn, kn, gd [T, H * D], beta, qk [T, H].
__global__ void delta_prepare_kernel(const CcSeqDeltaScan a, float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ gd,
                                     float* __restrict__ beta, float* __restrict__ qk) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t th = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (th >= (size_t)a.T * a.H) return;
    const size_t t = th / a.H;
    const int h = (int)(th - t * a.H), g = h / (a.H / a.G), D = a.D;
    const float* q = a.q + t * a.ldqk + (size_t)g * D;
    const float* k = a.k + t * a.ldqk + (size_t)g * D;
    const float* ar = a.a_raw + t * a.lda + (size_t)h * D;
    float* qo = qn + th * D;
    float* ko = kn + th * D;
    float* go = gd + th * D;
    const float dot = delta_prepare_rows(D, lane, a.q_scale, a.unit_eps, expf(a.A_log[h]), a.dt_bias + (size_t)h * D,
                                         [&](int n) { return q[n]; }, [&](int n) { return k[n]; }, [&](int n) { return ar[n]; },
                                         [&](int n, float v) { qo[n] = v; }, [&](int n, float v) { ko[n] = v; }, [&](int n, float v) { go[n] = v; });
    if (lane == 0) { qk[th] = dot; beta[th] = sigmoidf_(a.beta_raw[t * a.ldb + h]); }
}

template <int CH, int NC, int TB>
__global__ void __launch_bounds__(SCAN_J / (4 * NC) * 32, 2) delta_scan_kernel(const CcSeqDeltaScan a) {
    extern __shared__ float4 sm_dl4[];
    float* sm = reinterpret_cast<float*>(sm_dl4);
    constexpr int NW = SCAN_J / (4 * NC), RUN = CH + 4, Dp = DL_PARTS * RUN, NTH = NW * 32;
    constexpr int buf_floats = TB * (3 * Dp + SCAN_J + 2);
    const int D = a.D;
    const int h = blockIdx.x, j0 = blockIdx.y * SCAN_J, g = h / (a.H / a.G);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int jl = (warp * 4 + (lane >> 3)) * NC, p = lane & 7, j = j0 + jl;      // this lane's first column
    const int n0 = p * CH;
    float* S = a.state + (size_t)h * D * a.V;
    float st[NC][CH];
#pragma unroll
    for (int e = 0; e < NC; ++e)
#pragma unroll
        for (int c = 0; c < CH; ++c) st[e][c] = (n0 + c < D && j + e < a.V) ? S[(size_t)(n0 + c) * a.V + j + e] : 0.f;
    for (int idx = tid; idx < 2 * buf_floats; idx += NTH) sm[idx] = 0.f;   // rows beyond D and padding stay zero
    __syncthreads();
    const float lam = expf(a.A_log[h]);
    auto at = [](int n) { return (n / CH) * RUN + (n % CH); };
    auto fetch = [&](int tb, float* buf) {
        const int nt = min(TB, a.T - tb);
        // thread -> (token lane, channel): no division per copy
        const int lanes_t = D <= NTH / 2 ? NTH / ((D + 31) / 32 * 32) : 1, width = NTH / lanes_t;
        const int t0 = tid / width, nb = tid - t0 * width;
        for (int t = t0; t < nt; t += lanes_t)
            for (int n = nb; n < D; n += width) {
                const int o = t * Dp + at(n);
                const size_t row = (size_t)(tb + t) * a.ldqk + (size_t)g * D + n;
                cp_async4(buf + o, a.q + row);
                cp_async4(buf + TB * Dp + o, a.k + row);
                cp_async4(buf + 2 * TB * Dp + o, a.a_raw + (size_t)(tb + t) * a.lda + (size_t)h * D + n);
            }
        for (int idx = tid; idx < nt * SCAN_J; idx += NTH) {
            const int t = idx / SCAN_J, c = idx - t * SCAN_J;
            if (j0 + c < a.V) cp_async4(buf + 3 * TB * Dp + idx, a.v + (size_t)(tb + t) * a.ldv + (size_t)h * a.V + j0 + c);
        }
        if (tid < nt) {
            cp_async4(buf + 3 * TB * Dp + TB * SCAN_J + tid, a.beta_raw + (size_t)(tb + tid) * a.ldb + h);
            if (a.prepared) cp_async4(buf + 3 * TB * Dp + TB * SCAN_J + TB + tid, a.qk + (size_t)(tb + tid) * a.H + h);
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
        float* betas = buf + 3 * TB * Dp + TB * SCAN_J;
        float* qks = betas + TB;
        if (!a.prepared) {
            for (int t = warp; t < nt; t += NW) {     // a warp per token
                float* q = buf + t * Dp;
                float* k = buf + TB * Dp + t * Dp;
                float* gd = buf + 2 * TB * Dp + t * Dp;
                const float dot = delta_prepare_rows(D, lane, a.q_scale, a.unit_eps, lam, a.dt_bias + (size_t)h * D,
                                                     [&](int n) { return q[at(n)]; }, [&](int n) { return k[at(n)]; }, [&](int n) { return gd[at(n)]; },
                                                     [&](int n, float v) { q[at(n)] = v; }, [&](int n, float v) { k[at(n)] = v; },
                                                     [&](int n, float v) { gd[at(n)] = v; });
                if (lane == 0) { qks[t] = dot; betas[t] = sigmoidf_(betas[t]); }
            }
            __syncthreads();
        }
        const float4* __restrict__ q4 = reinterpret_cast<const float4*>(buf + p * RUN);
        const float4* __restrict__ k4 = reinterpret_cast<const float4*>(buf + TB * Dp + p * RUN);
        const float4* __restrict__ g4 = reinterpret_cast<const float4*>(buf + 2 * TB * Dp + p * RUN);
        const float* __restrict__ vs = buf + 3 * TB * Dp;
        float* orow = a.o + (size_t)tb * a.H * a.V + (size_t)h * a.V + j;
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            float kk[CH], rk[NC], rq[NC];
#pragma unroll
            for (int e = 0; e < NC; ++e) rk[e] = rq[e] = 0.f;
#pragma unroll
            for (int c4 = 0; c4 < CH / 4; ++c4) {
                const float4 gv = g4[t * (Dp / 4) + c4], kv = k4[t * (Dp / 4) + c4], qv = q4[t * (Dp / 4) + c4];
                const float g_[4] = {gv.x, gv.y, gv.z, gv.w}, k_[4] = {kv.x, kv.y, kv.z, kv.w}, q_[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    kk[4 * c4 + i] = k_[i];
#pragma unroll
                    for (int e = 0; e < NC; ++e) {
                        st[e][4 * c4 + i] *= g_[i];
                        rk[e] = fmaf(k_[i], st[e][4 * c4 + i], rk[e]);
                        rq[e] = fmaf(q_[i], st[e][4 * c4 + i], rq[e]);
                    }
                }
            }
#pragma unroll
            for (int o = 1; o < DL_PARTS; o <<= 1)
#pragma unroll
                for (int e = 0; e < NC; ++e) {
                    rk[e] += __shfl_xor_sync(0xffffffffu, rk[e], o);
                    rq[e] += __shfl_xor_sync(0xffffffffu, rq[e], o);
                }
            const float bt = betas[t], dot = qks[t];
#pragma unroll
            for (int e = 0; e < NC; ++e) {
                const float u = bt * (vs[t * SCAN_J + jl + e] - rk[e]);
#pragma unroll
                for (int c = 0; c < CH; ++c) st[e][c] = fmaf(kk[c], u, st[e][c]);
                if (p == 0 && j + e < a.V) orow[(size_t)t * a.H * a.V + e] = fmaf(dot, u, rq[e]);
            }
        }
        __syncthreads();   // the batch's buffer is free for the fetch after next
    }
#pragma unroll
    for (int e = 0; e < NC; ++e)
#pragma unroll
        for (int c = 0; c < CH; ++c)
            if (n0 + c < D && j + e < a.V) S[(size_t)(n0 + c) * a.V + j + e] = st[e][c];
}

// ------------------------------------------------------------------------------------------------ gated group norm
// A warp per (token, group).
template <typename OT>
__global__ void gated_rms_groups_kernel(const float* __restrict__ y, const float* __restrict__ gate, int64_t ldg, int gate_act,
                                        int gate_first, const float* __restrict__ w, int w_len, OT* __restrict__ out, int T, int W,
                                        int groups, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t tg = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (tg >= (size_t)T * groups) return;
    const size_t t = tg / groups;
    const int grp = (int)(tg - t * groups), Wg = W / groups, base = grp * Wg;
    const float* row = y + t * W + base;
    const float* grow = gate != nullptr ? gate + t * ldg + base : nullptr;
    const bool pre = grow != nullptr && gate_first;
    float ss = 0.f;
    for (int e = lane; e < Wg; e += 32) {
        const float v = pre ? row[e] * unit_act(grow[e], gate_act) : row[e];
        ss = fmaf(v, v, ss);
    }
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)Wg + eps);
    for (int e = lane; e < Wg; e += 32) {
        float v = row[e];
        const float ga = grow != nullptr ? unit_act(grow[e], gate_act) : 1.f;
        if (pre) v *= ga;
        v = v * rinv * w[(base + e) % w_len];
        if (!pre) v *= ga;
        stf(out, t * W + base + e, v);
    }
}

// The same with a CTA per (token, group), for wide groups.
template <typename OT>
__global__ void __launch_bounds__(1024) gated_rms_groups_wide_kernel(const float* __restrict__ y, const float* __restrict__ gate, int64_t ldg,
                                                                      int gate_act, int gate_first, const float* __restrict__ w, int w_len,
                                                                      OT* __restrict__ out, int W, int groups, float eps) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    const int grp = blockIdx.y, Wg = W / groups, base = grp * Wg, tid = threadIdx.x, nth = blockDim.x;
    const float* row = y + t * W + base;
    const float* grow = gate != nullptr ? gate + t * ldg + base : nullptr;
    const bool pre = grow != nullptr && gate_first;
    float ss = 0.f;
    for (int e = tid; e < Wg; e += nth) {
        const float v = pre ? row[e] * unit_act(grow[e], gate_act) : row[e];
        ss = fmaf(v, v, ss);
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)Wg + eps);
    for (int e = tid; e < Wg; e += nth) {
        float v = row[e];
        const float ga = grow != nullptr ? unit_act(grow[e], gate_act) : 1.f;
        if (pre) v *= ga;
        v = v * rinv * w[(base + e) % w_len];
        if (!pre) v *= ga;
        stf(out, t * W + base + e, v);
    }
}

// ------------------------------------------------------------------------------------------------ rotations
__device__ __forceinline__ void pair_index(int i, int dims, int interleaved, int& d0, int& d1) {
    if (interleaved) { d0 = 2 * i; d1 = 2 * i + 1; }
    else { d0 = i; d1 = i + dims / 2; }
}

// A warp per (token, head) over the H query heads, the G key heads and the G value heads.
template <typename OT>
__global__ void qkv_rope_kernel(const CcSeqQkvRope a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.H + 2 * a.G;
    const size_t th = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (th >= (size_t)a.T * heads) return;
    const size_t t = th / heads;
    const int hh = (int)(th - t * heads);
    const float pos = (float)(a.input_pos[0] + (int)t);
    const float* in = a.in + t * a.ld;
    if (hh < a.H + a.G) {
        const bool isq = hh < a.H;
        const int Dk = a.Dk, head = isq ? hh : hh - a.H;
        const float* row = in + (isq ? a.off_q : a.off_k) + (size_t)head * Dk;
        const float* nw = isq ? a.q_norm_w : a.k_norm_w;
        float rinv = 1.f;
        if (nw != nullptr) {
            float ss = 0.f;
            for (int d = lane; d < Dk; d += 32) ss = fmaf(row[d], row[d], ss);
            rinv = 1.0f / sqrtf(warp_sum(ss) / (float)Dk + a.eps);
        }
        float* qo = isq ? a.q_out + (t * a.H + head) * Dk : nullptr;
        OT* ko = isq ? nullptr : (OT*)a.k_out + (t * a.G + head) * Dk;
        auto val = [&](int d) { return nw != nullptr ? row[d] * rinv * nw[d] : row[d]; };
        auto put = [&](int d, float v) { if (isq) qo[d] = v; else stf(ko, d, v); };
        for (int i = lane; i < a.rot_dims / 2; i += 32) {
            int d0, d1;
            pair_index(i, a.rot_dims, a.interleaved, d0, d1);
            float s, c;
            sincosf(pos * a.inv_freq[i], &s, &c);
            const float u = val(d0), v = val(d1);
            put(d0, u * c - v * s);
            put(d1, v * c + u * s);
        }
        for (int d = a.rot_dims + lane; d < Dk; d += 32) put(d, val(d));
    } else {
        const int head = hh - a.H - a.G, Dv = a.Dv;
        const float* row = in + a.off_v + (size_t)head * Dv;
        OT* vo = (OT*)a.v_out + (t * a.G + head) * Dv;
        if (a.v_inv_freq != nullptr) {
            for (int i = lane; i < Dv / 2; i += 32) {
                int d0, d1;
                pair_index(i, Dv, a.interleaved, d0, d1);
                float s, c;
                sincosf(pos * a.v_inv_freq[i], &s, &c);
                const float u = row[d0], v = row[d1];
                stf(vo, d0, u * c - v * s);
                stf(vo, d1, v * c + u * s);
            }
            if ((Dv & 1) && lane == 0) stf(vo, Dv - 1, row[Dv - 1]);
        } else {
            for (int d = lane; d < Dv; d += 32) stf(vo, d, row[d]);
        }
    }
}

template <typename OT>
__global__ void turn_heads_gate_kernel(const float* __restrict__ y, const int32_t* __restrict__ input_pos,
                                       const float* __restrict__ inv_freq, int dims, int interleaved, float sign,
                                       const float* __restrict__ gate, int64_t ldg, OT* __restrict__ out, int T, int H, int Dv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t th = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (th >= (size_t)T * H) return;
    const size_t t = th / H;
    const int h = (int)(th - t * H);
    const float pos = sign * (float)(input_pos[0] + (int)t);
    const float gv = gate != nullptr ? sigmoidf_(gate[t * ldg + h]) : 1.f;
    const float* row = y + th * Dv;
    for (int i = lane; i < dims / 2; i += 32) {
        int d0, d1;
        pair_index(i, dims, interleaved, d0, d1);
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        const float u = row[d0], v = row[d1];
        stf(out, th * Dv + d0, (u * c - v * s) * gv);
        stf(out, th * Dv + d1, (v * c + u * s) * gv);
    }
    for (int d = dims + lane; d < Dv; d += 32) stf(out, th * Dv + d, row[d] * gv);
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t n, float cap) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

// ------------------------------------------------------------------------------------------------ host side
template <typename K>
static int set_smem(K kern, size_t smem, size_t& configured) {
    if (smem > configured) {
        configured = smem;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return cuda_check("shared memory size");
    }
    return CC_SEQ_OK;
}

template <int CH, int TB>
static int launch_ssd(const CcSeqSsdScan* a, cudaStream_t st) {
    const int P = (a->N + CH - 1) / CH;
    const size_t smem = sizeof(float) * (2 * (size_t)TB * (2 * P * CH + SCAN_J + 2) + (size_t)TB * P * SCAN_J);
    static size_t configured = 48 * 1024;
    if (int rc = set_smem(ssd_scan_kernel<CH, TB>, smem, configured)) return rc;
    dim3 grid(a->H, (a->V + SCAN_J - 1) / SCAN_J);
    ssd_scan_kernel<CH, TB><<<grid, P * 32, smem, st>>>(*a);
    return cuda_check("ssd_scan_kernel");
}

template <int CH, int NC, int TB>
static int launch_delta(const CcSeqDeltaScan* a, cudaStream_t st) {
    const size_t smem = sizeof(float) * 2 * (size_t)TB * (3 * DL_PARTS * (CH + 4) + SCAN_J + 2);
    static size_t configured = 48 * 1024;
    if (int rc = set_smem(delta_scan_kernel<CH, NC, TB>, smem, configured)) return rc;
    dim3 grid(a->H, (a->V + SCAN_J - 1) / SCAN_J);
    delta_scan_kernel<CH, NC, TB><<<grid, SCAN_J / (4 * NC) * 32, smem, st>>>(*a);
    return cuda_check("delta_scan_kernel");
}

}  // namespace ccn

using namespace ccn;

#define CCN_ST(dt, CALL)                                                  \
    do {                                                                  \
        if ((dt) == CC_DT_F32) { CALL(float); }                           \
        else if ((dt) == CC_DT_BF16) { CALL(bf16); }                      \
        else return fail(CC_SEQ_ERR_INVALID_ARG, "unknown element type"); \
    } while (0)

extern "C" {

int cc_seq_sum_norm(const CcSeqSumNorm* a, void* stream) {
    if (!a || !a->w || a->T < 1 || a->E < 1 || (!a->x && !a->y) || (a->y2 && !a->y) || (!a->out && !a->out_act && !a->coef))
        return fail(CC_SEQ_ERR_INVALID_ARG, "sum_norm: bad argument");
    if (a->coef && (!a->mix || a->n_prev < 0 || (a->n_prev > 0 && !a->stack) || a->rows))
        return fail(CC_SEQ_ERR_INVALID_ARG, "sum_norm: the depth average needs its stack and output, and no row selection");
    const size_t smem = sizeof(float) * (size_t)a->E;
    if (smem > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "sum_norm: rows longer than 51200");
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = a->T < 64 ? (a->E >= 1024 ? 1024 : ((a->E + 31) / 32) * 32) : 256;
#define CALL(AT)                                                                 \
    {                                                                            \
        static size_t configured = 48 * 1024;                                    \
        if (int rc = set_smem(sum_norm_kernel<AT>, smem, configured)) return rc; \
        sum_norm_kernel<AT><<<a->T, threads, smem, st>>>(*a);                    \
    }
    CCN_ST(a->out_act ? a->act_dtype : CC_DT_F32, CALL);
#undef CALL
    return cuda_check("sum_norm_kernel");
}

int cc_seq_short_conv(const float* u, int64_t ldu, const float* w, const float* bias, float* tail, float* out,
                      int64_t ldo, int32_t T, int32_t C, int32_t taps, int32_t act, void* stream) {
    if (!u || !w || !out || T < 1 || C < 1 || taps < 1 || (taps > 1 && !tail) || act < CC_ACT_NONE || act > CC_ACT_LAST)
        return fail(CC_SEQ_ERR_INVALID_ARG, "short_conv: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = 128, cb = (C + threads - 1) / threads;
    const int fused = T == 1 && taps > 1;
    short_conv_kernel<<<dim3(T, cb), threads, 0, st>>>(u, ldu, w, bias, tail, out, ldo, T, C, taps, act, fused);
    if (!fused && taps > 1) conv_tail_kernel<<<cb, threads, 0, st>>>(u, ldu, tail, T, C, taps);
    return cuda_check("short_conv_kernel");
}

int cc_seq_ssd_scan(const CcSeqSsdScan* a, void* stream) {
    if (!a || !a->x || !a->B || !a->C || !a->dt_raw || !a->dt_bias || !a->A_log || !a->state || !a->y || a->T < 1 ||
        a->H < 1 || a->G < 1 || a->H % a->G || a->N < 1 || a->V < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "ssd_scan: bad argument");
    if (a->N > 256) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "ssd_scan: more than 256 state rows per head");
    cudaStream_t st = (cudaStream_t)stream;
    if (a->N <= 128) return launch_ssd<8, 16>(a, st);
    return launch_ssd<16, 16>(a, st);
}

int cc_seq_delta_prepare(const CcSeqDeltaScan* a, float* qn, float* kn, float* gd, float* beta, float* qk, void* stream) {
    if (!a || !a->q || !a->k || !a->beta_raw || !a->a_raw || !a->dt_bias || !a->A_log || !qn || !kn || !gd || !beta || !qk ||
        a->T < 1 || a->H < 1 || a->G < 1 || a->H % a->G || a->D < 1 || a->prepared)
        return fail(CC_SEQ_ERR_INVALID_ARG, "delta_prepare: bad argument");
    const size_t warps = (size_t)a->T * a->H;
    delta_prepare_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(*a, qn, kn, gd, beta, qk);
    return cuda_check("delta_prepare_kernel");
}

int cc_seq_delta_scan(const CcSeqDeltaScan* a, void* stream) {
    if (!a || !a->q || !a->k || !a->v || !a->beta_raw || !a->a_raw || !a->dt_bias || !a->A_log || !a->state || !a->o ||
        a->T < 1 || a->H < 1 || a->G < 1 || a->H % a->G || a->D < 1 || a->V < 1 || (a->prepared && (!a->qk || a->G != a->H)))
        return fail(CC_SEQ_ERR_INVALID_ARG, "delta_scan: bad argument");
    if (a->D > 256) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "delta_scan: key heads wider than 256");
    cudaStream_t st = (cudaStream_t)stream;
    // rows per lane (8 lanes share a column's rows) x columns per lane
    if (a->D <= 64) return launch_delta<8, DL_NC, 16>(a, st);
    if (a->D <= 128) return launch_delta<16, DL_NC, 16>(a, st);
    return launch_delta<32, DL_NC, 16>(a, st);
}

int cc_seq_gated_rms_groups(const float* y, const float* gate, int64_t ldg, int32_t gate_act, int32_t gate_first,
                            const float* w, int32_t w_len, void* out, int32_t out_dtype, int32_t T, int32_t W,
                            int32_t groups, float eps, void* stream) {
    if (!y || !w || !out || T < 1 || W < 1 || groups < 1 || W % groups || w_len < 1 || gate_act < CC_ACT_NONE || gate_act > CC_ACT_LAST)
        return fail(CC_SEQ_ERR_INVALID_ARG, "gated_rms_groups: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t warps = (size_t)T * groups;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    const int Wg = W / groups;
    if (Wg >= 512 && groups <= 65535) {     // wide groups: a CTA each, 4 elements per thread when the step has few rows
        const int per = T < 64 ? 4 : 16;
        int threads = ((Wg + per - 1) / per + 31) / 32 * 32;
        threads = threads > 1024 ? 1024 : threads;
#define CALL(OT) gated_rms_groups_wide_kernel<OT><<<dim3(T, groups), threads, 0, st>>>(y, gate, ldg, gate_act, gate_first, w, w_len, (OT*)out, W, groups, eps)
        CCN_ST(out_dtype, CALL);
#undef CALL
        return cuda_check("gated_rms_groups_wide_kernel");
    }
#define CALL(OT) gated_rms_groups_kernel<OT><<<blocks, 256, 0, st>>>(y, gate, ldg, gate_act, gate_first, w, w_len, (OT*)out, T, W, groups, eps)
    CCN_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("gated_rms_groups_kernel");
}

int cc_seq_qkv_rope(const CcSeqQkvRope* a, void* stream) {
    if (!a || !a->in || !a->input_pos || !a->q_out || !a->k_out || !a->v_out || a->T < 1 || a->H < 1 || a->G < 1 ||
        a->Dk < 1 || a->Dv < 1 || a->rot_dims < 0 || a->rot_dims > a->Dk || (a->rot_dims & 1) || (a->rot_dims > 0 && !a->inv_freq))
        return fail(CC_SEQ_ERR_INVALID_ARG, "qkv_rope: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t warps = (size_t)a->T * (a->H + 2 * a->G);
    const unsigned blocks = (unsigned)((warps + 7) / 8);
#define CALL(OT) qkv_rope_kernel<OT><<<blocks, 256, 0, st>>>(*a)
    CCN_ST(a->out_dtype, CALL);
#undef CALL
    return cuda_check("qkv_rope_kernel");
}

int cc_seq_turn_heads_gate(const float* y, const int32_t* input_pos, const float* inv_freq, int32_t dims,
                           int32_t interleaved, float sign, const float* gate, int64_t ldg, void* out,
                           int32_t out_dtype, int32_t T, int32_t H, int32_t Dv, void* stream) {
    if (!y || !input_pos || !out || T < 1 || H < 1 || Dv < 1 || dims < 0 || dims > Dv || (dims & 1) || (dims > 0 && !inv_freq))
        return fail(CC_SEQ_ERR_INVALID_ARG, "turn_heads_gate: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t warps = (size_t)T * H;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
#define CALL(OT) turn_heads_gate_kernel<OT><<<blocks, 256, 0, st>>>(y, input_pos, inv_freq, dims, interleaved, sign, gate, ldg, (OT*)out, T, H, Dv)
    CCN_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("turn_heads_gate_kernel");
}

int cc_seq_softcap(float* x, int64_t n, float cap, void* stream) {
    if (!x || n < 1 || !(cap > 0.f)) return fail(CC_SEQ_ERR_INVALID_ARG, "softcap: bad argument");
    const int64_t blocks = (n + 255) / 256;
    softcap_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, (cudaStream_t)stream>>>(x, n, cap);
    return cuda_check("softcap_kernel");
}

}  // extern "C"
