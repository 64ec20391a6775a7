// seq_kernels.cu -- position-addressed sequence kernels behind include/cc_b200_seq.h (libcc_b200_seq.so).
//
// Arithmetic rule of this file: positions, angles, norms, attention scores, softmax weights, the weighted value sum
// and the residual stream are fp32 whatever the storage type of activations, weights and cache rows (fp32 or bf16);
// expf / logf / sinf / cosf / sqrtf are the accurate versions (no fast-math).  Results of the attention kernels depend on
// the key positions a query sees, never on which launch, chunk or slot brought a key: keys are addressed by
// position (slot = position mod capacity, checked against the slot's recorded position).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include "../../../include/cc_b200_seq.h"

namespace ccs {

static thread_local char g_err[512] = "";
// fail() and cuda_check() are shared with the other files of this library (declared there by hand)
int fail(int code, const char* msg) {
    strncpy(g_err, msg, sizeof(g_err) - 1);
    g_err[sizeof(g_err) - 1] = 0;
    return code;
}
int cuda_check(const char* where) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return CC_SEQ_OK;
    snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
    return CC_SEQ_ERR_CUDA;
}

__device__ __forceinline__ float ldf(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------------------------------------ embedding
template <typename WT, typename AT>
__global__ void embed_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ input_pos,
                             int32_t* prev_token, const WT* __restrict__ embed, const WT* __restrict__ bigram,
                             const float* __restrict__ inv_freq, float* __restrict__ x, AT* __restrict__ x_act, int T,
                             int E, float scale, int buckets, int mul_prev, int mul_cur) {
    const int t = blockIdx.x;
    const int p = input_pos[0] + t;
    const int tok = tokens[t];
    long long row = -1;
    if (bigram != nullptr) {
        if (p == 0) {
            row = buckets;
        } else {
            const long long prev = t > 0 ? tokens[t - 1] : prev_token[0];
            row = (prev * (long long)mul_prev + (long long)tok * (long long)mul_cur) % (long long)buckets;
            if (row < 0) row += buckets;
        }
    }
    const float pf = (float)p;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float v = ldf(embed, (size_t)tok * E + e) * scale;
        if (row >= 0) v += ldf(bigram, (size_t)row * E + e);
        const float ang = pf * inv_freq[e >> 1];
        v += (e & 1) ? cosf(ang) : sinf(ang);
        x[(size_t)t * E + e] = v;
        if (x_act != nullptr) stf(x_act, (size_t)t * E + e, v);
    }
    if (t == 0) {  // every thread of this block has read the old state above
        __syncthreads();
        if (threadIdx.x == 0) prev_token[0] = tokens[T - 1];
    }
}

// ------------------------------------------------------------------------------------------------ q/k/v preparation
template <typename IT, typename OT>
__global__ void qkv_prepare_kernel(const IT* __restrict__ qkv, const float* __restrict__ bias,
                                   const int32_t* __restrict__ input_pos, const float* __restrict__ mix_lambda,
                                   const OT* __restrict__ v_first, float* __restrict__ q_out, OT* __restrict__ k_out,
                                   OT* __restrict__ v_out, int T, int H, int G, int Dk, int Dv, float eps, int unit_norm,
                                   float gain_coef, int gain_every) {
    const int t = blockIdx.x;
    const int N = (H + G) * Dk + G * Dv;
    const IT* row = qkv + (size_t)t * N;
    const int p = input_pos[0] + t;
    float gain = 1.0f;
    if (gain_every > 0) gain = 1.0f + gain_coef * logf((float)((p + 1) / gain_every + 1));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    for (int hh = warp; hh < H + G; hh += nwarp) {
        const int off = hh * Dk;
        float ss = 0.f;
        for (int d = lane; d < Dk; d += 32) {
            float v = ldf(row, off + d);
            if (bias != nullptr) v += bias[off + d];
            ss += v * v;
        }
        ss = warp_sum(ss);
        const float r = unit_norm ? 1.0f / sqrtf(ss / (float)Dk + eps) : 1.0f;
        for (int d = lane; d < Dk; d += 32) {
            float v = ldf(row, off + d);
            if (bias != nullptr) v += bias[off + d];
            if (hh < H) q_out[((size_t)t * H + hh) * Dk + d] = v * r * gain;
            else stf(k_out, ((size_t)t * G + (hh - H)) * Dk + d, v * r);
        }
    }
    const int voff = (H + G) * Dk, NV = G * Dv;
    const float lam = v_first != nullptr ? mix_lambda[0] : 0.f;
    for (int i = threadIdx.x; i < NV; i += blockDim.x) {
        float v = ldf(row, voff + i);
        if (bias != nullptr) v += bias[voff + i];
        if (v_first != nullptr) v = (1.0f - lam) * v + lam * ldf(v_first, (size_t)t * NV + i);
        stf(v_out, (size_t)t * NV + i, v);
    }
}

// ------------------------------------------------------------------------------------------------ chunk attention
constexpr int BQ = 64, BK = 32, ATT_THREADS = 256;

// Slot of position j: the first keep_first positions own the first slots for good, the others share a ring over the
// rest of the cache (keep_first == 0: slot = j mod L).
__device__ __forceinline__ int slot_of(const CcSeqAttn& a, int j) {
    return j < a.keep_first ? j : a.keep_first + (j - a.keep_first) % (a.L - a.keep_first);
}

__device__ __forceinline__ int key_source(const CcSeqAttn& a, int j, int p0) {
    // >= 0: cache slot, -1: not a key, <= -2: row -(s + 2) of the chunk
    if (j >= p0) return -(j - p0) - 2;
    const int slot = slot_of(a, j);
    return a.pos[slot] == j ? slot : -1;
}

// What the design does to a scaled score before the softmax: a tanh soft cap, then a penalty that grows with the
// logarithm of the distance between query i and key j, with two numbers per query head.
__device__ __forceinline__ float shape_score(const CcSeqAttn& a, float s, int h, int dist) {
    if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
    if (a.dist_a != nullptr) s -= a.dist_a[h] * log1pf(a.dist_b[h] * (float)dist);
    return s;
}

// Stages `rows` rows of `width` elements (global, row r at src(r), or zeros when src(r) == nullptr) into fp32 shared
// memory rows of `stride` floats (a multiple of 4, dst 16-byte aligned).  16-byte loads and stores when the rows allow
// it, element loads otherwise.
template <typename CT, typename SrcFn>
__device__ __forceinline__ void stage_rows(float* dst, int stride, int rows, int width, SrcFn src, int tid, int nthreads) {
    constexpr int VEC = 16 / (int)sizeof(CT);
    if (width % VEC == 0) {
        constexpr int U = 4;   // loads in flight per thread
        const int per_row = width / VEC, total = rows * per_row;
        for (int base = tid; base < total; base += nthreads * U) {
            uint4 u[U];
            int off[U];
#pragma unroll
            for (int e = 0; e < U; ++e) {
                const int idx = base + e * nthreads;
                off[e] = -1;
                u[e] = make_uint4(0u, 0u, 0u, 0u);
                if (idx < total) {
                    const int r = idx / per_row, c = (idx - r * per_row) * VEC;
                    off[e] = r * stride + c;
                    const CT* p = src(r);
                    if (p != nullptr) u[e] = __ldg(reinterpret_cast<const uint4*>(p + c));
                }
            }
#pragma unroll
            for (int e = 0; e < U; ++e) {
                if (off[e] < 0) continue;
                const CT* e8 = reinterpret_cast<const CT*>(&u[e]);
                float4* d4 = reinterpret_cast<float4*>(dst + off[e]);   // stride and column are multiples of 4 floats
#pragma unroll
                for (int i = 0; i < VEC / 4; ++i)
                    d4[i] = make_float4(ldf(e8, 4 * i), ldf(e8, 4 * i + 1), ldf(e8, 4 * i + 2), ldf(e8, 4 * i + 3));
            }
        }
    } else {
        for (int idx = tid; idx < rows * width; idx += nthreads) {
            const int r = idx / width, c = idx - r * width;
            const CT* p = src(r);
            dst[r * stride + c] = p == nullptr ? 0.f : ldf(p, c);
        }
    }
}


// Row stride (floats) of a shared-memory tile read with 16-byte loads by lanes that hold different rows: a multiple
// of 4 whose quarter is odd, so that eight rows fall into eight different 16-byte bank groups.
__host__ __device__ inline int vec_stride(int width) {
    const int w4 = (width + 3) / 4;
    return 4 * (w4 | 1);
}

// CTA = 64 consecutive queries of one query head; key tiles of 32 positions.  Thread (ty, tx) of the 16 x 16 grid owns
// score rows 4 ty .. 4 ty + 3 x columns tx, tx + 16 and output rows 4 ty .. x value columns 64 c + 4 tx .. 4 tx + 3.
// All shared-memory operands are read with 16-byte loads: q, k along the head dimension, P along the keys, V along
// the value columns; 32 (scores) and 64 DV4 (values) FMAs per 6 and 4 + 4 DV4 loads.
template <typename CT, typename YT, int DV4>
__global__ void __launch_bounds__(ATT_THREADS) attn_chunk_kernel(const CcSeqAttn a) {
    extern __shared__ float4 sm4[];
    float* sm = reinterpret_cast<float*>(sm4);
    const int Dk = a.Dk, Dv = a.Dv, Dkp = vec_stride(Dk), Dk4 = (Dk + 3) / 4;
    constexpr int DVW = 64 * DV4, SP = BK + 4;
    float* Qs = sm;
    float* Ks = Qs + BQ * Dkp;
    float* Vs = Ks + BK * Dkp;
    float* Ss = Vs + BK * DVW;
    int* ksrc = (int*)(Ss + BQ * SP);
    int* kpos = ksrc + BK;

    const int qb = blockIdx.x, h = blockIdx.y, g = h / (a.H / a.G);
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int p0 = a.input_pos[0];
    const int i0 = qb * BQ;
    const int nq = min(BQ, a.T - i0);
    const CT* kc = (const CT*)a.k_cache;
    const CT* vc = (const CT*)a.v_cache;
    const CT* kn = (const CT*)a.k_new;
    const CT* vn = (const CT*)a.v_new;

    // padding columns are zero for the whole kernel (the tile loads below never touch them)
    for (int idx = tid; idx < (BQ + BK) * (Dkp - Dk); idx += ATT_THREADS) {
        const int r = idx / (Dkp - Dk), c = Dk + idx - r * (Dkp - Dk);
        Qs[r * Dkp + c] = 0.f;   // Ks follows Qs with the same stride
    }
    for (int idx = tid; idx < BK * (DVW - Dv); idx += ATT_THREADS) {
        const int r = idx / (DVW - Dv), c = Dv + idx - r * (DVW - Dv);
        Vs[r * DVW + c] = 0.f;
    }
    stage_rows<float>(Qs, Dkp, BQ, Dk, [&](int r) -> const float* {
        return r < nq ? a.q + ((size_t)(i0 + r) * a.H + h) * Dk : nullptr;
    }, tid, ATT_THREADS);
    const int j_hi = p0 + i0 + nq - 1;
    const int j_lo = a.block > 0 ? ((p0 + i0) / a.block) * a.block : (a.window > 0 ? max(0, p0 + i0 - a.window + 1) : 0);

    float m[4], l[4], O[4][4 * DV4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        if (a.sink_mode == CC_SINK_LEARNED) { m[r] = a.sink[h]; l[r] = 1.f; }
        else if (a.sink_mode == CC_SINK_ZERO) { m[r] = 0.f; l[r] = 1.f; }
        else { m[r] = -INFINITY; l[r] = 0.f; }
#pragma unroll
        for (int c = 0; c < 4 * DV4; ++c) O[r][c] = 0.f;
    }

    // the keys of this CTA in order: the kept first positions that lie below the window, then j_lo .. j_hi
    const int kx = a.window > 0 ? min(a.keep_first, j_lo) : 0;
    const int n_keys = kx + (j_hi - j_lo + 1);
    for (int ut = 0; ut < n_keys; ut += BK) {
        __syncthreads();  // the previous tile is consumed
        const int nk = min(BK, n_keys - ut);
        if (tid < BK) {
            const int u = ut + tid, j = u < kx ? u : j_lo + (u - kx);
            kpos[tid] = j;
            ksrc[tid] = tid < nk ? key_source(a, j, p0) : -1;
        }
        __syncthreads();
        stage_rows<CT>(Ks, Dkp, BK, Dk, [&](int r) -> const CT* {
            const int s = ksrc[r];
            return s >= 0 ? kc + ((size_t)g * a.L + s) * Dk : (s <= -2 ? kn + ((size_t)(-s - 2) * a.G + g) * Dk : nullptr);
        }, tid, ATT_THREADS);
        stage_rows<CT>(Vs, DVW, BK, Dv, [&](int r) -> const CT* {
            const int s = ksrc[r];
            return s >= 0 ? vc + ((size_t)g * a.L + s) * Dv : (s <= -2 ? vn + ((size_t)(-s - 2) * a.G + g) * Dv : nullptr);
        }, tid, ATT_THREADS);
        __syncthreads();

        float s[4][2];
#pragma unroll
        for (int r = 0; r < 4; ++r) s[r][0] = s[r][1] = 0.f;
        const float4* q4 = reinterpret_cast<const float4*>(Qs + (ty * 4) * Dkp);
        const float4* k4 = reinterpret_cast<const float4*>(Ks + tx * Dkp);
        const int rs4 = Dkp / 4;
#pragma unroll 2
        for (int d = 0; d < Dk4; ++d) {
            float4 qv[4], kv[2];
#pragma unroll
            for (int r = 0; r < 4; ++r) qv[r] = q4[r * rs4 + d];
            kv[0] = k4[d];
            kv[1] = k4[16 * rs4 + d];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    s[r][c] = fmaf(qv[r].x, kv[c].x, s[r][c]);
                    s[r][c] = fmaf(qv[r].y, kv[c].y, s[r][c]);
                    s[r][c] = fmaf(qv[r].z, kv[c].z, s[r][c]);
                    s[r][c] = fmaf(qv[r].w, kv[c].w, s[r][c]);
                }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int qi = ty * 4 + r;
            const int i = p0 + i0 + qi;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int col = tx + 16 * c;
                const int j = kpos[col];
                const bool ok = qi < nq && col < nk && ksrc[col] != -1 && j <= i &&
                                (a.window == 0 || i - j < a.window || j < a.keep_first) &&
                                (a.block == 0 || j >= (i / a.block) * a.block);
                s[r][c] = ok ? shape_score(a, s[r][c] * a.scale, h, i - j) : -INFINITY;
                mx = fmaxf(mx, s[r][c]);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_new = fmaxf(m[r], mx);
            const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
            float rsum = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float pr = (s[r][c] == -INFINITY) ? 0.f : expf(s[r][c] - m_new);
                rsum += pr;
                Ss[qi * SP + tx + 16 * c] = pr;
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, o);
            l[r] = l[r] * corr + rsum;
            m[r] = m_new;
#pragma unroll
            for (int c = 0; c < 4 * DV4; ++c) O[r][c] *= corr;
        }
        __syncwarp();
        const float4* p4 = reinterpret_cast<const float4*>(Ss + (ty * 4) * SP);
        const float4* v4 = reinterpret_cast<const float4*>(Vs) + tx;
#pragma unroll 2
        for (int kq = 0; kq < BK / 4; ++kq) {
            float4 pv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) pv[r] = p4[r * (SP / 4) + kq];
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int c = 0; c < DV4; ++c) {
                    const float4 vv = v4[(kq * 4 + kk) * (DVW / 4) + 16 * c];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float pk = kk == 0 ? pv[r].x : kk == 1 ? pv[r].y : kk == 2 ? pv[r].z : pv[r].w;
                        O[r][4 * c + 0] = fmaf(pk, vv.x, O[r][4 * c + 0]);
                        O[r][4 * c + 1] = fmaf(pk, vv.y, O[r][4 * c + 1]);
                        O[r][4 * c + 2] = fmaf(pk, vv.z, O[r][4 * c + 2]);
                        O[r][4 * c + 3] = fmaf(pk, vv.w, O[r][4 * c + 3]);
                    }
                }
            }
        }
    }
    YT* y = (YT*)a.y;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int qi = ty * 4 + r;
        if (qi >= nq) continue;
        const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
#pragma unroll
        for (int c = 0; c < 4 * DV4; ++c) {
            const int col = 64 * (c / 4) + 4 * tx + (c & 3);
            if (col < Dv) stf(y, ((size_t)(i0 + qi) * a.H + h) * Dv + col, O[r][c] * inv);
        }
    }
}

// ------------------------------------------------------------------------------------------------ decode attention
constexpr int KS = 128;           // keys per tile of the one-token kernel
constexpr int DEC_THREADS = 128;  // one thread per key
#ifndef CC_DEC_MAX_SPLITS
#define CC_DEC_MAX_SPLITS 64
#endif
constexpr int DEC_MAX_SPLITS = CC_DEC_MAX_SPLITS;  // runs of tiles per key/value head: bounds the partials the last CTA combines

__host__ __device__ inline int dec_k_stride(int Dk) {
    const int d4 = (Dk + 3) & ~3;
    return d4 + ((8 - (d4 & 31)) & 31);
}

__host__ __device__ inline int decode_max_splits(int L, int window) {
    const long long maxkeys = window > 0 ? (window < L + 1 ? window : L + 1) : (long long)L + 1;
    const long long tiles = (maxkeys + KS - 1) / KS;
    return (int)(tiles < DEC_MAX_SPLITS ? tiles : DEC_MAX_SPLITS);
}

// the most keys a query can see besides the limit of the cache: its window, or its block
__host__ __device__ inline int attn_reach(const CcSeqAttn& a) {
    return a.block > 0 ? a.block : (a.window > 0 ? a.window + a.keep_first : 0);
}

template <typename CT>
__device__ __forceinline__ void append_row(const CcSeqAttn& a, int g, int t, int p, int tid, int nthreads) {
    const int slot = slot_of(a, p);
    CT* kc = (CT*)a.k_cache;
    CT* vc = (CT*)a.v_cache;
    const CT* kn = (const CT*)a.k_new;
    const CT* vn = (const CT*)a.v_new;
    for (int d = tid; d < a.Dk; d += nthreads) kc[((size_t)g * a.L + slot) * a.Dk + d] = kn[((size_t)t * a.G + g) * a.Dk + d];
    for (int d = tid; d < a.Dv; d += nthreads) vc[((size_t)g * a.L + slot) * a.Dv + d] = vn[((size_t)t * a.G + g) * a.Dv + d];
    if (tid == 0) {
        if (a.mask != nullptr) a.mask[(size_t)g * a.L + slot] = 1;
        if (g == 0) {
            const int old = a.pos[slot];
            a.pos[slot] = p;
            if (old < 0 && a.cache_cts != nullptr) atomicAdd(a.cache_cts, 1);
        }
    }
}

// One CTA = a run of KS-key tiles of one key/value head, all R = H / G query heads of the group.  Per tile: one thread
// per key reads its K row straight from global memory with 16-byte loads (all in flight at once; consecutive keys are
// consecutive rows, so a warp's loads cover whole lines) and dots it with the R query rows held in shared memory
// (broadcast float4 reads); online softmax per query head; then one thread per value column walks the tile's V rows
// (coalesced across the columns).  A head's keys are cut into at most DEC_MAX_SPLITS runs; partial (max, sum, weighted
// values) go to the workspace; the last CTA of the head to arrive combines them in split order and, when asked,
// appends the new row.
template <typename CT, typename YT, int RMAX>
__global__ void __launch_bounds__(DEC_THREADS) attn_decode_kernel(const CcSeqAttn a) {
    extern __shared__ float4 smd4[];
    float* sm = reinterpret_cast<float*>(smd4);
    constexpr int VEC = 16 / (int)sizeof(CT);
    const int R = a.H / a.G, Dk = a.Dk, Dv = a.Dv;
    const int Dq = (Dk + 7) & ~7;   // q rows zero-padded to whole vectors
    float* qs = sm;               // [R, Dq]
    float* Ps = qs + R * Dq;      // [R, KS]
    int* ksrc = (int*)(Ps + R * KS);
    __shared__ int s_last;
    __shared__ float s_M[16], s_L[16], s_corr[16];

    const int sp = blockIdx.x, g = blockIdx.y, tid = threadIdx.x;
    const int p = a.input_pos[0];
    const int j_lo = a.block > 0 ? (p / a.block) * a.block : (a.window > 0 ? max(0, p - a.window + 1) : 0);
    const int kx = a.window > 0 ? min(a.keep_first, j_lo) : 0;   // kept first positions below the window
    const int n = kx + (p - j_lo + 1);
    const int n_tiles = (n + KS - 1) / KS;
    const int tiles_per = (n_tiles + DEC_MAX_SPLITS - 1) / DEC_MAX_SPLITS;
    const int nsplit = (n_tiles + tiles_per - 1) / tiles_per;
    if (sp >= nsplit) return;
    const int NS = decode_max_splits(a.L, attn_reach(a));
    int* counters = (int*)a.workspace;
    float* part_m = (float*)(counters + ((a.G + 3) & ~3));
    float* part_l = part_m + (size_t)a.G * NS * R;
    float* part_o = part_l + (size_t)a.G * NS * R;

    const CT* kc = (const CT*)a.k_cache;
    const CT* vc = (const CT*)a.v_cache;
    const CT* kn = (const CT*)a.k_new;
    const CT* vn = (const CT*)a.v_new;
    for (int i = tid; i < R * Dq; i += DEC_THREADS) {
        const int r = i / Dq, d = i - r * Dq;
        qs[i] = d < Dk ? a.q[((size_t)g * R + r) * Dk + d] : 0.f;
    }
    if (tid < 16) { s_M[tid] = -INFINITY; s_L[tid] = 0.f; }
    const int warp = tid >> 5, lane = tid & 31;
    float oacc[2][RMAX];   // value columns tid and tid + DEC_THREADS
#pragma unroll
    for (int r = 0; r < RMAX; ++r) oacc[0][r] = oacc[1][r] = 0.f;
    const bool vec_rows = (Dk % VEC) == 0;
    // value phase with 16-byte loads when the rows allow it and R x VEC accumulators fit in registers
    constexpr int VR = RMAX * VEC <= 64 ? RMAX : 1;
    const int ncg = Dv / VEC;
    const bool vec_values = RMAX * VEC <= 64 && Dv % VEC == 0 && ncg <= DEC_THREADS;
    const int nkg = vec_values ? DEC_THREADS / ncg : 1;
    const int kg = vec_values ? tid / ncg : 0, cg = vec_values ? tid - kg * ncg : 0;
    float vacc[VR][VEC];
#pragma unroll
    for (int r = 0; r < VR; ++r)
#pragma unroll
        for (int x = 0; x < VEC; ++x) vacc[r][x] = 0.f;

    const int tile_end = min(n_tiles, (sp + 1) * tiles_per);
    for (int tile = sp * tiles_per; tile < tile_end; ++tile) {
        const int u0 = tile * KS;
        const int nk = min(KS, n - u0);
        __syncthreads();   // the previous tile is consumed (first pass: qs and the running maxima are written)
        const int jk = u0 + tid < kx ? u0 + tid : j_lo + (u0 + tid - kx);
        const int src = tid < nk ? key_source(a, jk, p) : -1;
        ksrc[tid] = src;
        {   // scores: one thread per key
            float acc[RMAX];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) acc[r] = 0.f;
            if (src != -1) {
                const CT* krow = src >= 0 ? kc + ((size_t)g * a.L + src) * Dk : kn + (size_t)g * Dk;
                if (vec_rows) {
                    const uint4* k16 = reinterpret_cast<const uint4*>(krow);
                    const float4* q4 = reinterpret_cast<const float4*>(qs);
                    const int nv = Dk / VEC, q4_row = Dq / 4;
#pragma unroll 8
                    for (int i = 0; i < nv; ++i) {
                        const uint4 u = __ldg(k16 + i);
                        const CT* e = reinterpret_cast<const CT*>(&u);
                        float kf[VEC];
#pragma unroll
                        for (int x = 0; x < VEC; ++x) kf[x] = ldf(e, x);
#pragma unroll
                        for (int r = 0; r < RMAX; ++r)
                            if (r < R) {
#pragma unroll
                                for (int x4 = 0; x4 < VEC / 4; ++x4) {
                                    const float4 qv = q4[r * q4_row + i * (VEC / 4) + x4];
                                    acc[r] = fmaf(qv.x, kf[4 * x4 + 0], acc[r]);
                                    acc[r] = fmaf(qv.y, kf[4 * x4 + 1], acc[r]);
                                    acc[r] = fmaf(qv.z, kf[4 * x4 + 2], acc[r]);
                                    acc[r] = fmaf(qv.w, kf[4 * x4 + 3], acc[r]);
                                }
                            }
                    }
                } else {
                    for (int d = 0; d < Dk; ++d) {
                        const float kv = ldf(krow, d);
#pragma unroll
                        for (int r = 0; r < RMAX; ++r)
                            if (r < R) acc[r] = fmaf(qs[r * Dq + d], kv, acc[r]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                if (r < R) Ps[r * KS + tid] = src != -1 ? shape_score(a, acc[r] * a.scale, g * R + r, p - jk) : -INFINITY;
        }
        __syncthreads();
        for (int r = warp; r < R; r += DEC_THREADS / 32) {
            float mx = -INFINITY;
            for (int k = lane; k < KS; k += 32) mx = fmaxf(mx, Ps[r * KS + k]);
            mx = warp_max(mx);
            const float m_old = s_M[r];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int k = lane; k < KS; k += 32) {
                const float sv = Ps[r * KS + k];
                const float pr = sv == -INFINITY ? 0.f : expf(sv - m_new);
                Ps[r * KS + k] = pr;
                sum += pr;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                s_corr[r] = corr;
                s_L[r] = s_L[r] * corr + sum;
                s_M[r] = m_new;
            }
        }
        __syncthreads();
        if (vec_values) {
            // thread (kg, cg): keys kg, kg + nkg, ... of the tile x the VEC value columns of group cg, 16-byte loads
            if (kg < nkg) {
#pragma unroll
                for (int r = 0; r < VR; ++r)
                    if (r < R) {
                        const float cr = s_corr[r];
#pragma unroll
                        for (int x = 0; x < VEC; ++x) vacc[r][x] *= cr;
                    }
                const CT* vbase = vc + (size_t)g * a.L * Dv + cg * VEC;
                const CT* vnew = vn + (size_t)g * Dv + cg * VEC;
#pragma unroll 4
                for (int k = kg; k < nk; k += nkg) {
                    const int s = ksrc[k];
                    if (s == -1) continue;
                    const uint4 u = __ldg(reinterpret_cast<const uint4*>(s >= 0 ? vbase + (size_t)s * Dv : vnew));
                    const CT* e = reinterpret_cast<const CT*>(&u);
                    float vf[VEC];
#pragma unroll
                    for (int x = 0; x < VEC; ++x) vf[x] = ldf(e, x);
#pragma unroll
                    for (int r = 0; r < VR; ++r)
                        if (r < R) {
                            const float pw = Ps[r * KS + k];
#pragma unroll
                            for (int x = 0; x < VEC; ++x) vacc[r][x] = fmaf(pw, vf[x], vacc[r][x]);
                        }
                }
            }
        } else {
    #pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = tid + cc * DEC_THREADS;
                if (c >= Dv) break;
    #pragma unroll
                for (int r = 0; r < RMAX; ++r)
                    if (r < R) oacc[cc][r] *= s_corr[r];
                const CT* vbase = vc + (size_t)g * a.L * Dv + c;
                const CT* vnew = vn + (size_t)g * Dv + c;
    #pragma unroll 2
                for (int k = 0; k < KS; k += 4) {
                    if (k >= nk) break;
                    float v[4];
    #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int s = ksrc[k + i];   // -1 beyond nk as well
                        v[i] = s >= 0 ? ldf(vbase, (size_t)s * Dv) : (s <= -2 ? ldf(vnew, 0) : 0.f);
                    }
    #pragma unroll
                    for (int r = 0; r < RMAX; ++r)
                        if (r < R) {
                            const float4 pw = *reinterpret_cast<const float4*>(Ps + r * KS + k);
                            oacc[cc][r] = fmaf(pw.x, v[0], oacc[cc][r]);
                            oacc[cc][r] = fmaf(pw.y, v[1], oacc[cc][r]);
                            oacc[cc][r] = fmaf(pw.z, v[2], oacc[cc][r]);
                            oacc[cc][r] = fmaf(pw.w, v[3], oacc[cc][r]);
                        }
                }
            }
    
        }
    }
    if (vec_values) {   // sum the key groups' partial value sums: red[kg][r][c] -> column c of this thread
        __syncthreads();
        float* red = Ps + R * KS + KS;   // behind the key sources
        if (kg < nkg) {
#pragma unroll
            for (int r = 0; r < VR; ++r)
                if (r < R) {
#pragma unroll
                    for (int x = 0; x < VEC; ++x) red[((size_t)kg * R + r) * Dv + cg * VEC + x] = vacc[r][x];
                }
        }
        __syncthreads();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            const int c = tid + cc * DEC_THREADS;
            if (c >= Dv) break;
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                if (r < R) {
                    float t = 0.f;
                    for (int q = 0; q < nkg; ++q) t += red[((size_t)q * R + r) * Dv + c];
                    oacc[cc][r] = t;
                }
        }
    }
    const size_t pbase = ((size_t)g * NS + sp) * R;
    if (tid < R) { part_m[pbase + tid] = s_M[tid]; part_l[pbase + tid] = s_L[tid]; }
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int c = tid + cc * DEC_THREADS;
        if (c >= Dv) break;
#pragma unroll
        for (int r = 0; r < RMAX; ++r)
            if (r < R) part_o[(pbase + r) * Dv + c] = oacc[cc][r];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&counters[g], 1) == nsplit - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the last CTA of this head: every other CTA of the head has finished reading; combine in split order
    // (partials are read with ld.global.cg: other SMs wrote them, so L1 is bypassed)
    YT* y = (YT*)a.y;
    __shared__ float s_inv[16], s_max[16];
    float* wgt = Ps;   // [R, KS] weights of up to KS splits at a time (reuses the probability tile)
    for (int r = warp; r < R; r += DEC_THREADS / 32) {
        const int h = g * R + r;
        float M = -INFINITY;
        if (a.sink_mode == CC_SINK_LEARNED) M = a.sink[h];
        else if (a.sink_mode == CC_SINK_ZERO) M = 0.f;
        const float sinkv = M;
        for (int s = lane; s < nsplit; s += 32) M = fmaxf(M, __ldcg(part_m + ((size_t)g * NS + s) * R + r));
        M = warp_max(M);
        float Lsum = 0.f;
        for (int s = lane; s < nsplit; s += 32) {
            const size_t b = ((size_t)g * NS + s) * R + r;
            const float ms = __ldcg(part_m + b);
            Lsum += __ldcg(part_l + b) * (ms == -INFINITY ? 0.f : expf(ms - M));
        }
        Lsum = warp_sum(Lsum);
        if (a.sink_mode != CC_SINK_NONE) Lsum += expf(sinkv - M);
        if (lane == 0) { s_inv[r] = Lsum > 0.f ? 1.0f / Lsum : 0.f; s_max[r] = M; }
    }
    for (int c0 = 0; c0 < Dv; c0 += DEC_THREADS) {
        const int c = c0 + tid;
        float acc[RMAX];
#pragma unroll
        for (int r = 0; r < RMAX; ++r) acc[r] = 0.f;
        for (int s0 = 0; s0 < nsplit; s0 += KS) {   // splits in order, KS at a time
            const int ns = min(KS, nsplit - s0);
            __syncthreads();
            for (int i = tid; i < R * ns; i += DEC_THREADS) {
                const int r = i / ns, s = i - r * ns;
                const float ms = __ldcg(part_m + ((size_t)g * NS + s0 + s) * R + r);
                wgt[r * KS + s] = ms == -INFINITY ? 0.f : expf(ms - s_max[r]);
            }
            __syncthreads();
            if (c < Dv) {
#pragma unroll 8
                for (int s = 0; s < ns; ++s) {
                    const float* po = part_o + (((size_t)g * NS + s0 + s) * R) * Dv + c;
#pragma unroll
                    for (int r = 0; r < RMAX; ++r)
                        if (r < R) acc[r] = fmaf(__ldcg(po + (size_t)r * Dv), wgt[r * KS + s], acc[r]);
                }
            }
        }
        if (c < Dv) {
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                if (r < R) stf(y, (size_t)(g * R + r) * Dv + c, acc[r] * s_inv[r]);
        }
    }
    if (tid == 0) counters[g] = 0;
    if (a.append) append_row<CT>(a, g, 0, p, tid, DEC_THREADS);
}

template <typename CT>
__global__ void cache_append_kernel(const CcSeqAttn a, int t_first) {
    const int t = t_first + blockIdx.x, g = blockIdx.y;
    const int p = a.input_pos[0] + t;
    // a row whose slot a later row of the same chunk takes is not written (kept first positions never are)
    if (p >= a.keep_first && p + (a.L - a.keep_first) <= a.input_pos[0] + a.T - 1) return;
    append_row<CT>(a, g, t, p, threadIdx.x, blockDim.x);
}

// ------------------------------------------------------------------------------------------------ post-sum norm
template <typename YT, typename AT>
__global__ void residual_norm_kernel(float* __restrict__ x, const YT* __restrict__ y, const float* __restrict__ w,
                                     float alpha, float eps, AT* __restrict__ x_act, int E) {
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * E;
    float ss = 0.f;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float s = alpha * x[base + e];
        if (y != nullptr) s += ldf(y, base + e);
        ss += s * s;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const float r = 1.0f / sqrtf(red[0] / (float)E + eps);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float s = alpha * x[base + e];
        if (y != nullptr) s += ldf(y, base + e);
        const float v = s * r * (1.0f + w[e]);
        x[base + e] = v;
        if (x_act != nullptr) stf(x_act, base + e, v);
    }
}

// ------------------------------------------------------------------------------------------------ clamped gated unit
template <typename IT, typename OT>
__global__ void clamped_glu_kernel(const IT* __restrict__ gu, OT* __restrict__ out, float limit, float slope, int T,
                                   int F) {
    const size_t n = (size_t)T * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F, f = i - t * F;
        const float g = fminf(ldf(gu, t * 2 * F + f), limit);
        const float u = fminf(fmaxf(ldf(gu, t * 2 * F + F + f), -limit), limit);
        stf(out, i, g * (1.0f / (1.0f + expf(-slope * g))) * (u + 1.0f));
    }
}

// ------------------------------------------------------------------------------------------------ one-token products
constexpr int GEMV_THREADS = 256, GEMV_ROWS = 8;   // one row per warp: small CTAs, many row streams in flight per SM
// (measured on a B200 at widths 2048 / 4096: 8 rows per CTA 0.435 / 0.801 ms per token, 16: 0.456 / 0.796, 32: 0.58 / 0.96;
// requesting a row's first vectors before the input is staged did not pay: 0.427 / 0.830)

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
        t = warp_sum(t);
        if (threadIdx.x == 0) red[0] = t;
    }
    __syncthreads();
    t = red[0];
    __syncthreads();
    return t;
}

__device__ __forceinline__ float round_like(float v, const float*) { return v; }
__device__ __forceinline__ float round_like(float v, const __nv_bfloat16*) { return __bfloat162float(__float2bfloat16_rn(v)); }

// One row of W against the staged input: 16-byte loads, four in flight per lane.
template <typename WT>
__device__ __forceinline__ float row_dot(const WT* __restrict__ w, const float* __restrict__ xs, int K, int lane) {
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
    return warp_sum(acc);
}

template <typename WT, typename XT, typename OT>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const CcSeqGemv g) {
    extern __shared__ float4 smg4[];
    float* xs = reinterpret_cast<float*>(smg4);   // [K] the product's input, rounded as the weights are
    __shared__ float red[32];
    const int K = g.K, N = g.N, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const XT* x = (const XT*)g.x;
    const WT* W = (const WT*)g.W;
    float rin = 1.f;
    if (g.in_norm_w != nullptr) {
        float ss = 0.f;
        for (int k = tid; k < K; k += GEMV_THREADS) { const float v = ldf(x, k); ss += v * v; }
        rin = 1.0f / sqrtf(block_sum(ss, red) / (float)K + g.eps);
    }
    for (int k = tid; k < K; k += GEMV_THREADS) {
        float v = ldf(x, k);
        if (g.in_norm_w != nullptr) v = v * rin * (1.0f + g.in_norm_w[k]);
        xs[k] = round_like(v, W);
    }
    float rres = 1.f;
    if (g.mode == CC_GEMV_RESIDUAL && g.res_norm_w != nullptr) {
        float ss = 0.f;
        for (int n = tid; n < N; n += GEMV_THREADS) { const float v = g.res[n]; ss += v * v; }
        rres = 1.0f / sqrtf(block_sum(ss, red) / (float)N + g.eps);
    }
    __syncthreads();
    for (int i = 0; i < GEMV_ROWS / (GEMV_THREADS / 32); ++i) {
        const int n = blockIdx.x * GEMV_ROWS + i * (GEMV_THREADS / 32) + warp;
        if (n >= N) break;
        float acc = row_dot<WT>(W + (size_t)n * K, xs, K, lane);
        if (g.mode == CC_GEMV_GLU) {
            const float up = row_dot<WT>(W + (size_t)(N + n) * K, xs, K, lane);
            if (lane == 0) {
                const float gt = fminf(acc, g.limit);
                const float u = fminf(fmaxf(up, -g.limit), g.limit);
                stf((OT*)g.out, n, gt * (1.0f / (1.0f + expf(-g.slope * gt))) * (u + 1.0f));
            }
            continue;
        }
        if (lane != 0) continue;
        if (g.bias != nullptr) acc += g.bias[n];
        if (g.mode == CC_GEMV_RESIDUAL) {
            float r = g.res[n];
            if (g.res_norm_w != nullptr) r = r * rres * (1.0f + g.res_norm_w[n]);
            acc = g.alpha * r + acc;
        }
        stf((OT*)g.out, n, acc);
    }
}

template <typename WT, typename XT, typename OT>
static int launch_gemv(const CcSeqGemv* g, cudaStream_t st) {
    const size_t smem = sizeof(float) * (size_t)((g->K + 3) & ~3);
    auto kern = gemv_kernel<WT, XT, OT>;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        configured = smem;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(CC_SEQ_ERR_CUDA, cudaGetErrorString(e));
    }
    kern<<<(g->N + GEMV_ROWS - 1) / GEMV_ROWS, GEMV_THREADS, smem, st>>>(*g);
    return cuda_check("gemv_kernel");
}

// ------------------------------------------------------------------------------------------------ host side
static int check_attn(const CcSeqAttn* a) {
    if (!a || !a->q || !a->k_new || !a->v_new || !a->k_cache || !a->v_cache || !a->pos || !a->input_pos || !a->y)
        return fail(CC_SEQ_ERR_INVALID_ARG, "attention: NULL pointer");
    if (a->T < 1 || a->H < 1 || a->G < 1 || a->H % a->G || a->Dk < 1 || a->Dv < 1 || a->L < 1 || a->window < 0)
        return fail(CC_SEQ_ERR_INVALID_ARG, "attention: bad sizes");
    if (a->Dk > 256 || a->Dv > 256) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "attention: head sizes above 256");
    if (a->keep_first < 0 || (a->keep_first > 0 && a->L <= a->keep_first) || a->softcap < 0.f || (a->dist_a && !a->dist_b))
        return fail(CC_SEQ_ERR_INVALID_ARG, "attention: bad kept-first count, soft cap or distance penalty");
    if (a->window > 0 && a->L < a->window + a->keep_first)
        return fail(CC_SEQ_ERR_INVALID_ARG, "attention: cache capacity below the window plus the kept first positions");
    if (a->block < 0 || (a->block > 0 && (a->window > 0 || a->L < a->block)))
        return fail(CC_SEQ_ERR_INVALID_ARG, "attention: a block mask needs a cache of at least one block and no window");
    if (a->sink_mode == CC_SINK_LEARNED && !a->sink) return fail(CC_SEQ_ERR_INVALID_ARG, "attention: sink missing");
    return CC_SEQ_OK;
}

template <typename CT, typename YT, int DV4>
static int launch_chunk(const CcSeqAttn* a, cudaStream_t st) {
    const int Dkp = vec_stride(a->Dk);
    const size_t smem = sizeof(float) * ((size_t)(BQ + BK) * Dkp + (size_t)BK * 64 * DV4 + (size_t)BQ * (BK + 4)) + sizeof(int) * 2 * BK;
    auto kern = attn_chunk_kernel<CT, YT, DV4>;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        configured = smem;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(CC_SEQ_ERR_CUDA, cudaGetErrorString(e));
    }
    dim3 grid((a->T + BQ - 1) / BQ, a->H);
    kern<<<grid, ATT_THREADS, smem, st>>>(*a);
    return cuda_check("attn_chunk_kernel");
}

template <typename CT, typename YT>
static int dispatch_chunk(const CcSeqAttn* a, cudaStream_t st) {
    const int need = (a->Dv + 63) / 64;
    if (need <= 1) return launch_chunk<CT, YT, 1>(a, st);
    if (need <= 2) return launch_chunk<CT, YT, 2>(a, st);
    if (need <= 3) return launch_chunk<CT, YT, 3>(a, st);
    return launch_chunk<CT, YT, 4>(a, st);
}

template <typename CT, typename YT, int RMAX>
static int launch_decode_r(const CcSeqAttn* a, cudaStream_t st) {
    const int R = a->H / a->G;
    const int vecw = 16 / (int)sizeof(CT);
    const size_t red = (RMAX * vecw <= 64 && a->Dv % vecw == 0 && a->Dv / vecw <= DEC_THREADS) ? (size_t)(DEC_THREADS / (a->Dv / vecw)) * R * a->Dv : 0;
    const size_t smem = sizeof(float) * ((size_t)R * ((a->Dk + 7) & ~7) + (size_t)R * KS + red) + sizeof(int) * KS;
    auto kern = attn_decode_kernel<CT, YT, RMAX>;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        configured = smem;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(CC_SEQ_ERR_CUDA, cudaGetErrorString(e));
    }
    dim3 grid(decode_max_splits(a->L, attn_reach(*a)), a->G);
    kern<<<grid, DEC_THREADS, smem, st>>>(*a);
    return cuda_check("attn_decode_kernel");
}

template <typename CT, typename YT>
static int launch_decode(const CcSeqAttn* a, cudaStream_t st) {
    const int R = a->H / a->G;
    if (R <= 1) return launch_decode_r<CT, YT, 1>(a, st);
    if (R <= 2) return launch_decode_r<CT, YT, 2>(a, st);
    if (R <= 4) return launch_decode_r<CT, YT, 4>(a, st);
    if (R <= 8) return launch_decode_r<CT, YT, 8>(a, st);
    if (R <= 16) return launch_decode_r<CT, YT, 16>(a, st);
    return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "attention_decode: more than 16 query heads per key/value head");
}

#define CCS_DISPATCH2(d0, d1, CALL)                                                              \
    do {                                                                                         \
        if ((d0) == CC_DT_F32 && (d1) == CC_DT_F32) return CALL(float, float);                   \
        if ((d0) == CC_DT_F32 && (d1) == CC_DT_BF16) return CALL(float, __nv_bfloat16);          \
        if ((d0) == CC_DT_BF16 && (d1) == CC_DT_F32) return CALL(__nv_bfloat16, float);          \
        if ((d0) == CC_DT_BF16 && (d1) == CC_DT_BF16) return CALL(__nv_bfloat16, __nv_bfloat16); \
        return fail(CC_SEQ_ERR_INVALID_ARG, "unknown element type");                             \
    } while (0)

}  // namespace ccs

using namespace ccs;

extern "C" {

int cc_seq_abi_version(void) { return CC_SEQ_ABI_VERSION; }
const char* cc_seq_last_error(void) { return g_err; }

int cc_seq_embed(const int32_t* tokens, const int32_t* input_pos, int32_t* prev_token, const void* embed,
                 const void* bigram, const float* inv_freq, float* x, void* x_act, int32_t T, int32_t E, float scale,
                 int32_t buckets, int32_t mul_prev, int32_t mul_cur, int32_t table_dtype, int32_t act_dtype, void* stream) {
    if (!tokens || !input_pos || !prev_token || !embed || !inv_freq || !x || T < 1 || E < 1 || (bigram && buckets < 1))
        return fail(CC_SEQ_ERR_INVALID_ARG, "embed: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(WT, AT)                                                                                                  \
    (embed_kernel<WT, AT><<<T, 128, 0, st>>>(tokens, input_pos, prev_token, (const WT*)embed, (const WT*)bigram,      \
                                             inv_freq, x, (AT*)x_act, T, E, scale, buckets, mul_prev, mul_cur),       \
     cuda_check("embed_kernel"))
    CCS_DISPATCH2(table_dtype, act_dtype, CALL);
#undef CALL
}

int cc_seq_qkv_prepare(const void* qkv, int32_t in_dtype, const float* bias, const int32_t* input_pos,
                       const float* mix_lambda, const void* v_first, float* q_out, void* k_out, void* v_out,
                       int32_t out_dtype, int32_t T, int32_t H, int32_t G, int32_t Dk, int32_t Dv, float eps,
                       int32_t unit_norm, float gain_coef, int32_t gain_every, void* stream) {
    if (!qkv || !input_pos || !q_out || !k_out || !v_out || T < 1 || H < 1 || G < 1 || Dk < 1 || Dv < 1 ||
        (v_first && !mix_lambda))
        return fail(CC_SEQ_ERR_INVALID_ARG, "qkv_prepare: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(IT, OT)                                                                                                   \
    (qkv_prepare_kernel<IT, OT><<<T, 128, 0, st>>>((const IT*)qkv, bias, input_pos, mix_lambda, (const OT*)v_first,    \
                                                   q_out, (OT*)k_out, (OT*)v_out, T, H, G, Dk, Dv, eps, unit_norm,     \
                                                   gain_coef, gain_every),                                             \
     cuda_check("qkv_prepare_kernel"))
    CCS_DISPATCH2(in_dtype, out_dtype, CALL);
#undef CALL
}

int cc_seq_attention(const CcSeqAttn* a, void* stream) {
    int rc = check_attn(a);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(CT, YT) dispatch_chunk<CT, YT>(a, st)
    CCS_DISPATCH2(a->cache_dtype, a->y_dtype, CALL);
#undef CALL
}

uint64_t cc_seq_decode_workspace(int32_t H, int32_t G, int32_t Dv, int32_t L, int32_t window) {
    const uint64_t NS = (uint64_t)decode_max_splits(L, window);
    return sizeof(int) * (uint64_t)((G + 3) & ~3) + sizeof(float) * NS * (uint64_t)H * (2 + (uint64_t)Dv);
}

int cc_seq_attention_decode(const CcSeqAttn* a, void* stream) {
    int rc = check_attn(a);
    if (rc) return rc;
    if (a->T != 1) return fail(CC_SEQ_ERR_INVALID_ARG, "attention_decode: one token per call");
    if (!a->workspace || a->workspace_bytes < cc_seq_decode_workspace(a->H, a->G, a->Dv, a->L, attn_reach(*a)))
        return fail(CC_SEQ_ERR_INVALID_ARG, "attention_decode: workspace missing or too small");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(CT, YT) launch_decode<CT, YT>(a, st)
    CCS_DISPATCH2(a->cache_dtype, a->y_dtype, CALL);
#undef CALL
}

int cc_seq_cache_append(const CcSeqAttn* a, void* stream) {
    if (!a || !a->k_new || !a->v_new || !a->k_cache || !a->v_cache || !a->pos || !a->input_pos || a->T < 1 || a->L < 1)
        return fail(CC_SEQ_ERR_INVALID_ARG, "cache_append: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    if (a->keep_first < 0 || a->L <= a->keep_first) return fail(CC_SEQ_ERR_INVALID_ARG, "cache_append: bad kept-first count");
    const int t_first = (a->keep_first == 0 && a->T > a->L) ? a->T - a->L : 0;   // with kept positions every row's CTA decides
    dim3 grid(a->T - t_first, a->G);
    if (a->cache_dtype == CC_DT_F32) cache_append_kernel<float><<<grid, 64, 0, st>>>(*a, t_first);
    else if (a->cache_dtype == CC_DT_BF16) cache_append_kernel<__nv_bfloat16><<<grid, 64, 0, st>>>(*a, t_first);
    else return fail(CC_SEQ_ERR_INVALID_ARG, "cache_append: unknown element type");
    return cuda_check("cache_append_kernel");
}

int cc_seq_residual_norm(float* x, const void* y, int32_t y_dtype, const float* w, float alpha, float eps, void* x_act,
                         int32_t act_dtype, int32_t T, int32_t E, void* stream) {
    if (!x || !w || T < 1 || E < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "residual_norm: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(YT, AT)                                                                                                \
    (residual_norm_kernel<YT, AT><<<T, 256, 0, st>>>(x, (const YT*)y, w, alpha, eps, (AT*)x_act, E),                \
     cuda_check("residual_norm_kernel"))
    CCS_DISPATCH2(y_dtype, act_dtype, CALL);
#undef CALL
}

int cc_seq_clamped_glu(const void* gu, void* out, int32_t io_dtype, int32_t out_dtype, float limit, float slope,
                       int32_t T, int32_t F, void* stream) {
    if (!gu || !out || T < 1 || F < 1) return fail(CC_SEQ_ERR_INVALID_ARG, "clamped_glu: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = (size_t)T * F;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
#define CALL(IT, OT)                                                                                    \
    (clamped_glu_kernel<IT, OT><<<blocks, 256, 0, st>>>((const IT*)gu, (OT*)out, limit, slope, T, F),   \
     cuda_check("clamped_glu_kernel"))
    CCS_DISPATCH2(io_dtype, out_dtype, CALL);
#undef CALL
}

int cc_seq_gemv(const CcSeqGemv* g, void* stream) {
    if (!g || !g->x || !g->W || !g->out || g->N < 1 || g->K < 1 || (g->mode == CC_GEMV_RESIDUAL && !g->res) ||
        g->mode < CC_GEMV_PLAIN || g->mode > CC_GEMV_GLU)
        return fail(CC_SEQ_ERR_INVALID_ARG, "gemv: bad argument");
    if (g->in_norm_w && g->x_dtype != CC_DT_F32) return fail(CC_SEQ_ERR_INVALID_ARG, "gemv: a normed input is an fp32 sum");
    if (g->mode != CC_GEMV_GLU && g->out_dtype != CC_DT_F32) return fail(CC_SEQ_ERR_INVALID_ARG, "gemv: fp32 output expected");
    if ((size_t)g->K * 4 > 200 * 1024) return fail(CC_SEQ_ERR_UNSUPPORTED_SHAPE, "gemv: input longer than 51200");
    cudaStream_t st = (cudaStream_t)stream;
    const bool wb = g->w_dtype == CC_DT_BF16, xb = g->x_dtype == CC_DT_BF16, ob = g->out_dtype == CC_DT_BF16;
    if (wb && xb && ob) return launch_gemv<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(g, st);
    if (wb && xb && !ob) return launch_gemv<__nv_bfloat16, __nv_bfloat16, float>(g, st);
    if (wb && !xb && ob) return launch_gemv<__nv_bfloat16, float, __nv_bfloat16>(g, st);
    if (wb && !xb && !ob) return launch_gemv<__nv_bfloat16, float, float>(g, st);
    if (!wb && !xb && !ob) return launch_gemv<float, float, float>(g, st);
    return fail(CC_SEQ_ERR_INVALID_ARG, "gemv: unsupported combination of element types");
}

}  // extern "C"
