// par_kernels.cu -- sequence kernels, fourth part of include/cc_b200_seq.h: layers whose sublayers all read norms of
// the same stream.  The residual sum of the layer before, one unit-RMS pass over the row and, per sublayer, a gain and
// a short causal convolution added to its own input (h + conv(h)) with the tail carried from step to step; the
// whole-row RMS norm of a fused query / key / value projection; the polynomial-of-unit-RMS activation.
//
// Arithmetic rule (as in seq_kernels.cu): everything here is fp32 whatever the storage type of the neighbours.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../../include/cc_b200_seq.h"

namespace ccs {
int fail(int code, const char* msg);
int cuda_check(const char* where);
}  // namespace ccs

namespace ccp {
using ccs::cuda_check;
using ccs::fail;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

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

// Three sums over the block at once, in the same fixed order.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*red)[32]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    if (lane == 0) { red[0][warp] = a; red[1][warp] = b; red[2][warp] = c; }
    __syncthreads();
    a = b = c = 0.f;
    for (int i = 0; i < nw; ++i) { a += red[0][i]; b += red[1][i]; c += red[2][i]; }
}

// ------------------------------------------------------------------------------------------------ sum + unit RMS (+ canon)
// The unit-RMS value of channel c at token t of the step: x * rinv for t >= 0, the carried tail (row taps - 1 + t) for
// the tokens before the step's first.
__device__ __forceinline__ float canon_input(const float* __restrict__ x, const float* __restrict__ rinv,
                                             const float* __restrict__ tail, int E, int taps, int t, int c) {
    return t >= 0 ? x[(size_t)t * E + c] * rinv[t] : tail[(size_t)(taps - 1 + t) * E + c];
}

// CTA per token: x += a + b + add (each optional), rinv[t] = 1 / sqrt(mean(x^2) + eps).  With one token (fused != 0)
// the sublayer inputs and the tail's move happen in the same launch, and everything they need besides the row's own
// statistics (gains, taps, tail rows) is loaded before the reduction: out_s = A_s * xh + B_s with
// A_s = g + w_last g and B_s = sum_{j < taps - 1} w_j (tail_j g) kept in shared memory.  Thread c alone touches
// channel c of the tail.
template <typename ST>
__global__ void __launch_bounds__(1024) par_norm_kernel(const CcSeqParNorm g, int fused) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int t = blockIdx.x, E = g.E, tid = threadIdx.x, taps = g.taps;
    float* x = g.x + (size_t)t * E;
    float* AB = row + E;      // fused: [n_out][2][E]
    float ss = 0.f;
    for (int c = tid; c < E; c += blockDim.x) {
        float v = x[c];
        if (g.a != nullptr) v += g.a[(size_t)t * g.lda + c];
        if (g.b != nullptr) v += g.b[(size_t)t * g.ldb + c];
        if (g.add != nullptr) v += g.add[c];
        if (fused) {
            for (int s = 0; s < g.n_out; ++s) {
                const float gn = g.gain[s][c];
                const float* cw = g.conv_w[s];
                float A = gn, B = 0.f;
                if (cw != nullptr) {
                    A = fmaf(cw[(size_t)c * taps + taps - 1], gn, gn);
                    for (int j = 0; j < taps - 1; ++j) B = fmaf(cw[(size_t)c * taps + j], g.tail[(size_t)j * E + c] * gn, B);
                }
                AB[(size_t)(2 * s) * E + c] = A;
                AB[(size_t)(2 * s + 1) * E + c] = B;
            }
            for (int k = 0; k + 1 < taps - 1; ++k) g.tail[(size_t)k * E + c] = g.tail[(size_t)(k + 1) * E + c];
        }
        row[c] = v;
        ss += v * v;
        if (g.a != nullptr || g.b != nullptr || g.add != nullptr) x[c] = v;
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)E + g.eps);
    if (!fused) {
        if (tid == 0) g.rinv[t] = rinv;
        return;
    }
    for (int c = tid; c < E; c += blockDim.x) {      // thread c reads back only what it wrote
        const float xh = row[c] * rinv;
        for (int s = 0; s < g.n_out; ++s) stf((ST*)g.out[s], c, fmaf(AB[(size_t)(2 * s) * E + c], xh, AB[(size_t)(2 * s + 1) * E + c]));
        if (taps > 1) g.tail[(size_t)(taps - 2) * E + c] = xh;
    }
}

// One token, spread over the GPU: CTA = 256 channels.  Every CTA computes the row's statistic itself (the sums of the
// whole row: reads only, so the loads pipeline), after the loads its own channels need (gains, taps, tail rows) are
// in flight.  The summed row goes to x_out, a buffer of its own: other CTAs still read x for their statistic.
constexpr int TOKEN_THREADS = 256;
template <typename ST>
__global__ void __launch_bounds__(TOKEN_THREADS) par_norm_token_kernel(const CcSeqParNorm g) {
    __shared__ float red[32];
    const int E = g.E, tid = threadIdx.x, taps = g.taps, c = blockIdx.x * TOKEN_THREADS + tid;
    const float* __restrict__ x = g.x;
    const float* __restrict__ pa = g.a;
    const float* __restrict__ pb = g.b;
    const float* __restrict__ padd = g.add;
    float own = 0.f, A[CC_PAR_MAX_OUT], B[CC_PAR_MAX_OUT];
    if (c < E) {
        own = x[c];
        if (pa != nullptr) own += pa[c];
        if (pb != nullptr) own += pb[c];
        if (padd != nullptr) own += padd[c];
#pragma unroll
        for (int s = 0; s < CC_PAR_MAX_OUT; ++s) {
            A[s] = B[s] = 0.f;
            if (s >= g.n_out) continue;
            const float gn = g.gain[s][c];
            const float* cw = g.conv_w[s];
            A[s] = gn;
            if (cw != nullptr) {
                A[s] = fmaf(cw[(size_t)c * taps + taps - 1], gn, gn);
                for (int j = 0; j < taps - 1; ++j) B[s] = fmaf(cw[(size_t)c * taps + j], g.tail[(size_t)j * E + c] * gn, B[s]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll 4
    for (int i = tid; i < E; i += TOKEN_THREADS) {
        float v = x[i];
        if (pa != nullptr) v += pa[i];
        if (pb != nullptr) v += pb[i];
        if (padd != nullptr) v += padd[i];
        ss += v * v;
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)E + g.eps);
    if (c >= E) return;
    const float xh = own * rinv;
    g.x_out[c] = own;
#pragma unroll
    for (int s = 0; s < CC_PAR_MAX_OUT; ++s)
        if (s < g.n_out) stf((ST*)g.out[s], c, fmaf(A[s], xh, B[s]));
    for (int k = 0; k + 1 < taps - 1; ++k) g.tail[(size_t)k * E + c] = g.tail[(size_t)(k + 1) * E + c];
    if (taps > 1) g.tail[(size_t)(taps - 2) * E + c] = xh;
}

// Steps of several tokens: thread = one channel over a run of TT tokens, with the last TAPS - 1 unit-RMS values of the
// channel in registers, so that every value is read once (coalesced across the channels) and serves all sublayers.
// out_s = h + sum_j w_s[c, j] h(t - TAPS + 1 + j), h = xh * gain_s.  TAPS == 0: any number of taps, values re-read.
constexpr int CANON_TT = 16;
template <typename ST, int TAPS>
__global__ void __launch_bounds__(128) par_canon_kernel(const CcSeqParNorm g) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x, E = g.E;
    if (c >= E) return;
    const int t0 = blockIdx.x * CANON_TT, t1 = min(g.T, t0 + CANON_TT);
    if (TAPS == 0) {
        const int taps = g.taps;
        for (int t = t0; t < t1; ++t) {
            const float cur = g.x[(size_t)t * E + c] * g.rinv[t];
            for (int s = 0; s < g.n_out; ++s) {
                const float gn = g.gain[s][c];
                const float* cw = g.conv_w[s];
                float acc = cur * gn;
                if (cw != nullptr)
                    for (int j = 0; j < taps; ++j)
                        acc = fmaf(cw[(size_t)c * taps + j], (j == taps - 1 ? cur : canon_input(g.x, g.rinv, g.tail, E, taps, t - taps + 1 + j, c)) * gn, acc);
                stf((ST*)g.out[s], (size_t)t * E + c, acc);
            }
        }
        return;
    }
    constexpr int NW = TAPS > 1 ? TAPS - 1 : 1, NT = TAPS > 0 ? TAPS : 1;
    float win[NW], gn[CC_PAR_MAX_OUT], cw[CC_PAR_MAX_OUT][NT];
#pragma unroll
    for (int j = 0; j < NW; ++j) win[j] = TAPS > 1 ? canon_input(g.x, g.rinv, g.tail, E, TAPS, t0 - (TAPS - 1) + j, c) : 0.f;
#pragma unroll
    for (int s = 0; s < CC_PAR_MAX_OUT; ++s) {
        gn[s] = s < g.n_out ? g.gain[s][c] : 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j) cw[s][j] = (s < g.n_out && g.conv_w[s] != nullptr) ? g.conv_w[s][(size_t)c * TAPS + j] : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
        const float cur = g.x[(size_t)t * E + c] * g.rinv[t];
#pragma unroll
        for (int s = 0; s < CC_PAR_MAX_OUT; ++s) {
            if (s >= g.n_out) break;
            float acc = cur * gn[s];
#pragma unroll
            for (int j = 0; j < NT - 1; ++j) acc = fmaf(cw[s][j], win[j] * gn[s], acc);
            acc = fmaf(cw[s][NT - 1], cur * gn[s], acc);
            stf((ST*)g.out[s], (size_t)t * E + c, acc);
        }
#pragma unroll
        for (int j = 0; j + 1 < NW; ++j) win[j] = win[j + 1];
        if (TAPS > 1) win[NW - 1] = cur;
    }
}

// After every token of the step has read it: the tail becomes the step's last taps - 1 unit-RMS rows (rows that the
// step did not bring move up from the old tail; ascending order reads each old row before it is overwritten).
__global__ void par_tail_kernel(const CcSeqParNorm g) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= g.E) return;
    for (int k = 0; k < g.taps - 1; ++k)
        g.tail[(size_t)k * g.E + c] = canon_input(g.x, g.rinv, g.tail, g.E, g.taps, g.T - (g.taps - 1) + k, c);
}

// ------------------------------------------------------------------------------------------------ whole-row q / k norm
// CTA per token: q and k are each divided by the root mean square of their WHOLE projection row (all heads at once)
// and multiplied by a gain per column; v is copied.  q in fp32, k and v in the cache's type.
// With few tokens the outputs of a row are cut into gridDim.y slices; every CTA computes both statistics itself.
template <typename ST>
__global__ void __launch_bounds__(256) qk_row_norm_kernel(const CcSeqQkRowNorm a) {
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* __restrict__ in = a.in + (size_t)t * a.ld;
    float sq = 0.f, sk = 0.f;
#pragma unroll 4
    for (int e = tid; e < a.nq; e += blockDim.x) { const float v = in[a.off_q + e]; sq += v * v; }
#pragma unroll 4
    for (int e = tid; e < a.nk; e += blockDim.x) { const float v = in[a.off_k + e]; sk += v * v; }
    const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)a.nq + a.eps);
    const float rk = 1.0f / sqrtf(block_sum(sk, red) / (float)a.nk + a.eps);
    const int total = a.nq + a.nk + a.nv, per = (total + gridDim.y - 1) / gridDim.y;
    const int lo = blockIdx.y * per, hi = min(total, lo + per);
    for (int i = lo + tid; i < hi; i += blockDim.x) {
        if (i < a.nq) a.q_out[(size_t)t * a.nq + i] = in[a.off_q + i] * rq * a.wq[i];
        else if (i < a.nq + a.nk) { const int e = i - a.nq; stf((ST*)a.k_out, (size_t)t * a.nk + e, in[a.off_k + e] * rk * a.wk[e]); }
        else { const int e = i - a.nq - a.nk; stf((ST*)a.v_out, (size_t)t * a.nv + e, in[a.off_v + e]); }
    }
}

// ------------------------------------------------------------------------------------------------ polynomial of unit RMS
// CTA per token: out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with N(u) = u / sqrt(mean(u^2) + eps) over the row and the
// powers taken element by element.  Rows that allow it are read with 16-byte loads; steps of few tokens run 1024
// threads per row, so that a thread's loads are few and all in flight at once.
template <typename ST>
__global__ void __launch_bounds__(1024) poly_norm_kernel(const float* __restrict__ in, int64_t ld, const float* __restrict__ coef,
                                                         ST* __restrict__ out, int F, float eps, int vec) {
    __shared__ float red3[3][32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* __restrict__ z = in + (size_t)t * ld;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    auto add = [&](float v) {
        const float v2 = v * v, v3 = v2 * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v3 * v3;
    };
    if (vec) {
        const float4* __restrict__ z4 = reinterpret_cast<const float4*>(z);
#pragma unroll 4
        for (int f = tid; f < F / 4; f += blockDim.x) { const float4 v = z4[f]; add(v.x); add(v.y); add(v.z); add(v.w); }
    } else {
#pragma unroll 8
        for (int f = tid; f < F; f += blockDim.x) add(z[f]);
    }
    block_sum3(s1, s2, s3, red3);
    const float r1 = coef[0] / sqrtf(s1 / (float)F + eps);
    const float r2 = coef[1] / sqrtf(s2 / (float)F + eps);
    const float r3 = coef[2] / sqrtf(s3 / (float)F + eps);
    const float c3 = coef[3];
    auto act = [&](float v) { const float v2 = v * v; return v * r1 + v2 * r2 + v2 * v * r3 + c3; };
    ST* __restrict__ o = out + (size_t)t * F;
    if (vec) {
        const float4* __restrict__ z4 = reinterpret_cast<const float4*>(z);
#pragma unroll 4
        for (int f = tid; f < F / 4; f += blockDim.x) {
            const float4 v = z4[f];
            stf(o, 4 * f, act(v.x)); stf(o, 4 * f + 1, act(v.y)); stf(o, 4 * f + 2, act(v.z)); stf(o, 4 * f + 3, act(v.w));
        }
    } else {
#pragma unroll 8
        for (int f = tid; f < F; f += blockDim.x) stf(o, f, act(z[f]));
    }
}

#define CCP_ST(dt, CALL)                                                 \
    do {                                                                 \
        if ((dt) == CC_DT_F32) { CALL(float); }                          \
        else if ((dt) == CC_DT_BF16) { CALL(bf16); }                     \
        else return fail(CC_SEQ_ERR_INVALID_ARG, "unknown element type"); \
    } while (0)

}  // namespace ccp

using namespace ccp;

extern "C" {

int cc_seq_par_norm(const CcSeqParNorm* g, void* stream) {
    if (!g || !g->x || g->T < 1 || g->E < 1 || g->n_out < 0 || g->n_out > CC_PAR_MAX_OUT || g->taps < 1 ||
        (g->taps > 1 && g->n_out > 0 && !g->tail) || (g->T > 1 && g->n_out > 0 && !g->rinv))
        return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: bad argument");
    for (int s = 0; s < g->n_out; ++s)
        if (!g->out[s] || !g->gain[s]) return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: output or gain missing");
    if ((size_t)g->E * sizeof(float) > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "par_norm: row too wide");
    cudaStream_t st = (cudaStream_t)stream;
    if (g->x_out != nullptr) {      // one token, spread over the GPU; the sum goes to a buffer of its own
        if (g->T != 1 || g->n_out < 1 || g->x_out == g->x) return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: x_out is for one token and may not be x");
#define CALL(ST) par_norm_token_kernel<ST><<<(g->E + TOKEN_THREADS - 1) / TOKEN_THREADS, TOKEN_THREADS, 0, st>>>(*g)
        CCP_ST(g->act_dtype, CALL);
#undef CALL
        return cuda_check("par_norm_token_kernel");
    }
    const int fused = g->T == 1 && g->n_out > 0;
    const int threads = g->T <= 4 ? 1024 : 256;      // few rows: every pass is a chain of dependent loads
    const size_t smem = sizeof(float) * (size_t)g->E * (fused ? 1 + 2 * g->n_out : 1);
    if (smem > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "par_norm: row too wide");
    if (smem > 48 * 1024) {
        static size_t configured = 48 * 1024;
        if (smem > configured) {
            configured = smem;
            cudaFuncSetAttribute(par_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            cudaFuncSetAttribute(par_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        }
    }
    if (g->n_out == 0 && !g->rinv) return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: nothing to write");
#define CALL(ST) par_norm_kernel<ST><<<g->T, threads, smem, st>>>(*g, fused)
    CCP_ST(g->act_dtype, CALL);
#undef CALL
    if (!fused && g->n_out > 0) {
        const int th = 128, cb = (g->E + th - 1) / th;
        const dim3 grid((g->T + CANON_TT - 1) / CANON_TT, cb);
#define CALL(ST)                                                                  \
    switch (g->taps) {                                                            \
        case 1: par_canon_kernel<ST, 1><<<grid, th, 0, st>>>(*g); break;          \
        case 2: par_canon_kernel<ST, 2><<<grid, th, 0, st>>>(*g); break;          \
        case 3: par_canon_kernel<ST, 3><<<grid, th, 0, st>>>(*g); break;          \
        case 4: par_canon_kernel<ST, 4><<<grid, th, 0, st>>>(*g); break;          \
        default: par_canon_kernel<ST, 0><<<grid, th, 0, st>>>(*g); break;         \
    }
        CCP_ST(g->act_dtype, CALL);
#undef CALL
        if (g->taps > 1) par_tail_kernel<<<cb, th, 0, st>>>(*g);
    }
    return cuda_check("par_norm kernels");
}

int cc_seq_qk_row_norm(const CcSeqQkRowNorm* a, void* stream) {
    if (!a || !a->in || !a->q_out || !a->k_out || !a->v_out || !a->wq || !a->wk || a->T < 1 || a->nq < 1 || a->nk < 1 || a->nv < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "qk_row_norm: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const int total = a->nq + a->nk + a->nv;
    const dim3 grid(a->T, a->T <= 4 ? (total + 511) / 512 : 1);
#define CALL(ST) qk_row_norm_kernel<ST><<<grid, 256, 0, st>>>(*a)
    CCP_ST(a->out_dtype, CALL);
#undef CALL
    return cuda_check("qk_row_norm_kernel");
}

int cc_seq_poly_norm(const float* in, int64_t ld, const float* coef, void* out, int32_t out_dtype, int32_t T, int32_t F,
                     float eps, void* stream) {
    if (!in || !coef || !out || T < 1 || F < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "poly_norm: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = T <= 4 ? 1024 : 256;
    const int vec = F % 4 == 0 && ld % 4 == 0 && ((uintptr_t)in & 15) == 0;
#define CALL(ST) poly_norm_kernel<ST><<<T, threads, 0, st>>>(in, ld, coef, (ST*)out, F, eps, vec)
    CCP_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("poly_norm_kernel");
}

}  // extern "C"
