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

// ------------------------------------------------------------------------------------------------ sum + unit RMS (+ canon)
// The unit-RMS row `pos` steps back from the end of the rows the convolution of token t reaches: from xhat for t >= 0,
// from the carried tail (row taps - 1 + t, t < 0) before the step's first token.
__device__ __forceinline__ float canon_input(const float* __restrict__ xhat, const float* __restrict__ tail, int E, int taps,
                                             int t, int c) {
    return t >= 0 ? xhat[(size_t)t * E + c] : tail[(size_t)(taps - 1 + t) * E + c];
}

// One sublayer input for channel c of token t: h + sum_j cw[c, j] * h(t - taps + 1 + j), h = xhat * gain.
__device__ __forceinline__ float canon_value(const float* __restrict__ xhat, const float* __restrict__ tail,
                                             const float* __restrict__ gain, const float* __restrict__ cw, int E, int taps,
                                             int t, int c, float cur) {
    const float g = gain[c];
    float acc = cur * g;
    if (cw != nullptr)
        for (int j = 0; j < taps; ++j) {
            const float prev = j == taps - 1 ? cur : canon_input(xhat, tail, E, taps, t - taps + 1 + j, c);
            acc = fmaf(cw[(size_t)c * taps + j], prev * g, acc);
        }
    return acc;
}

// CTA per token: x += a + b + add (each optional), xhat = x / rms(x).  With one token (fused != 0) the sublayer inputs
// and the tail's move happen in the same launch: thread c alone touches channel c of the tail.
template <typename ST>
__global__ void __launch_bounds__(1024) par_norm_kernel(const CcSeqParNorm g, int fused) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int t = blockIdx.x, E = g.E, tid = threadIdx.x;
    float* x = g.x + (size_t)t * E;
    float ss = 0.f;
    for (int c = tid; c < E; c += blockDim.x) {
        float v = x[c];
        if (g.a != nullptr) v += g.a[(size_t)t * g.lda + c];
        if (g.b != nullptr) v += g.b[(size_t)t * g.ldb + c];
        if (g.add != nullptr) v += g.add[c];
        row[c] = v;
        ss += v * v;
        if (g.a != nullptr || g.b != nullptr || g.add != nullptr) x[c] = v;
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)E + g.eps);
    for (int c = tid; c < E; c += blockDim.x) {      // thread c reads back only what it wrote
        const float xh = row[c] * rinv;
        if (!fused) { g.xhat[(size_t)t * E + c] = xh; continue; }
        for (int s = 0; s < g.n_out; ++s)
            stf((ST*)g.out[s], c, canon_value(nullptr, g.tail, g.gain[s], g.conv_w[s], E, g.taps, 0, c, xh));
        for (int k = 0; k + 1 < g.taps - 1; ++k) g.tail[(size_t)k * E + c] = g.tail[(size_t)(k + 1) * E + c];
        if (g.taps > 1) g.tail[(size_t)(g.taps - 2) * E + c] = xh;
    }
}

template <typename ST>
__global__ void par_canon_kernel(const CcSeqParNorm g) {
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= g.E) return;
    const float cur = g.xhat[(size_t)t * g.E + c];
    for (int s = 0; s < g.n_out; ++s)
        stf((ST*)g.out[s], (size_t)t * g.E + c, canon_value(g.xhat, g.tail, g.gain[s], g.conv_w[s], g.E, g.taps, t, c, cur));
}

// After every token of the step has read it: the tail becomes the step's last taps - 1 unit-RMS rows (rows that the
// step did not bring move up from the old tail; ascending order reads each old row before it is overwritten).
__global__ void par_tail_kernel(const CcSeqParNorm g) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= g.E) return;
    for (int k = 0; k < g.taps - 1; ++k)
        g.tail[(size_t)k * g.E + c] = canon_input(g.xhat, g.tail, g.E, g.taps, g.T - (g.taps - 1) + k, c);
}

// ------------------------------------------------------------------------------------------------ whole-row q / k norm
// CTA per token: q and k are each divided by the root mean square of their WHOLE projection row (all heads at once)
// and multiplied by a gain per column; v is copied.  q in fp32, k and v in the cache's type.
template <typename ST>
__global__ void __launch_bounds__(256) qk_row_norm_kernel(const CcSeqQkRowNorm a) {
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* in = a.in + (size_t)t * a.ld;
    float sq = 0.f, sk = 0.f;
    for (int e = tid; e < a.nq; e += blockDim.x) { const float v = in[a.off_q + e]; sq += v * v; }
    for (int e = tid; e < a.nk; e += blockDim.x) { const float v = in[a.off_k + e]; sk += v * v; }
    const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)a.nq + a.eps);
    const float rk = 1.0f / sqrtf(block_sum(sk, red) / (float)a.nk + a.eps);
    for (int e = tid; e < a.nq; e += blockDim.x) a.q_out[(size_t)t * a.nq + e] = in[a.off_q + e] * rq * a.wq[e];
    for (int e = tid; e < a.nk; e += blockDim.x) stf((ST*)a.k_out, (size_t)t * a.nk + e, in[a.off_k + e] * rk * a.wk[e]);
    for (int e = tid; e < a.nv; e += blockDim.x) stf((ST*)a.v_out, (size_t)t * a.nv + e, in[a.off_v + e]);
}

// ------------------------------------------------------------------------------------------------ polynomial of unit RMS
// CTA per token: out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with N(u) = u / sqrt(mean(u^2) + eps) over the row and the
// powers taken element by element.
template <typename ST>
__global__ void __launch_bounds__(512) poly_norm_kernel(const float* __restrict__ in, int64_t ld, const float* __restrict__ coef,
                                                        ST* __restrict__ out, int F, float eps) {
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* z = in + (size_t)t * ld;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int f = tid; f < F; f += blockDim.x) {
        const float v = z[f], v2 = v * v, v3 = v2 * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v3 * v3;
    }
    const float r1 = coef[0] / sqrtf(block_sum(s1, red) / (float)F + eps);
    const float r2 = coef[1] / sqrtf(block_sum(s2, red) / (float)F + eps);
    const float r3 = coef[2] / sqrtf(block_sum(s3, red) / (float)F + eps);
    const float c3 = coef[3];
    for (int f = tid; f < F; f += blockDim.x) {
        const float v = z[f], v2 = v * v;
        stf(out, (size_t)t * F + f, v * r1 + v2 * r2 + v2 * v * r3 + c3);
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
        (g->taps > 1 && g->n_out > 0 && !g->tail) || (g->T > 1 && g->n_out > 0 && !g->xhat))
        return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: bad argument");
    for (int s = 0; s < g->n_out; ++s)
        if (!g->out[s] || !g->gain[s]) return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: output or gain missing");
    if ((size_t)g->E * sizeof(float) > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "par_norm: row too wide");
    cudaStream_t st = (cudaStream_t)stream;
    const int fused = g->T == 1 && g->n_out > 0;
    const int threads = g->T <= 4 ? 1024 : 256;      // few rows: every pass is a chain of dependent loads
    const size_t smem = sizeof(float) * (size_t)g->E;
    if (smem > 48 * 1024) {
        static size_t configured = 48 * 1024;
        if (smem > configured) {
            configured = smem;
            cudaFuncSetAttribute(par_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            cudaFuncSetAttribute(par_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        }
    }
    if (g->n_out == 0 && !g->xhat) return fail(CC_SEQ_ERR_INVALID_ARG, "par_norm: nothing to write");
#define CALL(ST) par_norm_kernel<ST><<<g->T, threads, smem, st>>>(*g, fused)
    CCP_ST(g->act_dtype, CALL);
#undef CALL
    if (!fused && g->n_out > 0) {
        const int th = 128, cb = (g->E + th - 1) / th;
#define CALL(ST) par_canon_kernel<ST><<<dim3(g->T, cb), th, 0, st>>>(*g)
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
#define CALL(ST) qk_row_norm_kernel<ST><<<a->T, 256, 0, st>>>(*a)
    CCP_ST(a->out_dtype, CALL);
#undef CALL
    return cuda_check("qk_row_norm_kernel");
}

int cc_seq_poly_norm(const float* in, int64_t ld, const float* coef, void* out, int32_t out_dtype, int32_t T, int32_t F,
                     float eps, void* stream) {
    if (!in || !coef || !out || T < 1 || F < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "poly_norm: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = T <= 4 ? 512 : 256;
#define CALL(ST) poly_norm_kernel<ST><<<T, threads, 0, st>>>(in, ld, coef, (ST*)out, F, eps)
    CCP_ST(out_dtype, CALL);
#undef CALL
    return cuda_check("poly_norm_kernel");
}

}  // extern "C"
