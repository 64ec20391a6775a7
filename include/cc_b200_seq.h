/*
 * cc_b200_seq.h -- C ABI of the position-addressed sequence kernels (libcc_b200_seq.so).
 *
 * These serve decoder designs that append every token to a slot cache in order (slot = position mod capacity:
 * a full cache while capacity >= sequence length, a ring for sliding-window layers) and need their attention
 * arithmetic in fp32: softmax with a sink term in the denominator, optional sliding window, unit-RMS q/k with a
 * position-dependent query gain, value mixing across layers, post-sum normalisation, a clamped gated feed-forward,
 * and a token + hashed-bigram + sinusoid embedding.
 *
 * Plain pointers and sizes only.  Every function returns 0 on success and a negative CC_ERR_* code (cc_b200.h
 * values) on failure; cc_seq_last_error() gives the message.  All pointers are DEVICE pointers owned by the caller.
 * Every call enqueues work on the caller's stream and never synchronises; positions are read from device memory,
 * so a decode step can be captured in a CUDA graph.
 */
#ifndef CC_B200_SEQ_H
#define CC_B200_SEQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CC_SEQ_ABI_VERSION 4

#define CC_SEQ_OK                     0
#define CC_SEQ_ERR_INVALID_ARG       -1
#define CC_SEQ_ERR_UNSUPPORTED_SHAPE -2
#define CC_SEQ_ERR_CUDA              -3

/* element types of activations, weights and cache rows */
#define CC_DT_F32   0
#define CC_DT_BF16  1

/* what the softmax denominator contains besides the keys */
#define CC_SINK_NONE     0
#define CC_SINK_LEARNED  1  /* exp(sink[h]), one fp32 logit per query head */
#define CC_SINK_ZERO     2  /* exp(0) = 1                                  */

/*
 * One attention layer's step over a chunk of T consecutive tokens whose first position is *input_pos.
 * Query i (position p = *input_pos + i) sees key position j when j <= p and (window == 0 or p - j < window or
 * j < keep_first) and (block == 0 or floor(p / block) == floor(j / block)): blocks are counted from position 0 of the
 * sequence.  Keys j >= *input_pos are rows of k_new / v_new; older keys are read from the cache slot of j and count
 * only if pos[slot] == j (an empty, stale or overwritten slot is not a key).  Slot of j: j itself for j < keep_first,
 * keep_first + (j - keep_first) mod (L - keep_first) otherwise (j mod L without kept positions).
 * A scaled score s becomes softcap * tanh(s / softcap) (softcap > 0), then s - dist_a[h] * ln(1 + dist_b[h] * (p - j))
 * (dist_a set), before the softmax.
 */
typedef struct CcSeqAttn {
    const float* q;            /* [T, H, Dk] fp32, already normalised and scaled by the query gain */
    const void* k_new;         /* [T, G, Dk] cache dtype */
    const void* v_new;         /* [T, G, Dv] cache dtype */
    void* k_cache;             /* [G, L, Dk] cache dtype */
    void* v_cache;             /* [G, L, Dv] cache dtype */
    int32_t* pos;              /* [L] position held by each slot, -1 = empty */
    uint8_t* mask;             /* [G, L] 1 = slot filled (may be NULL) */
    int32_t* cache_cts;        /* [1] number of filled slots (may be NULL) */
    const int32_t* input_pos;  /* [1] */
    void* y;                   /* [T, H, Dv] y dtype */
    const float* sink;         /* [H] fp32 for CC_SINK_LEARNED, else NULL */
    int32_t T, H, G, Dk, Dv, L;
    int32_t window;            /* 0 = every earlier key */
    int32_t sink_mode;
    int32_t cache_dtype, y_dtype;
    float scale;               /* multiplies q.k */
    int32_t append;            /* decode only (T == 1): also write the new row into its slot */
    void* workspace;           /* decode only: cc_seq_decode_workspace() bytes, zeroed once by the caller */
    uint64_t workspace_bytes;
    int32_t block;             /* 0 = none; else keys of the query's own block of `block` positions only (L >= block) */
    int32_t keep_first;        /* with a window: the first keep_first positions stay visible and keep their slots (L >= window + keep_first) */
    float softcap;             /* 0 = none */
    const float* dist_a;       /* [H] fp32 or NULL: the distance penalty's factor ... */
    const float* dist_b;       /* [H] fp32: ... and the slope inside its logarithm */
} CcSeqAttn;

int cc_seq_abi_version(void);
const char* cc_seq_last_error(void);

/* x[t] = embed[tok[t]] * scale + bigram[row(t)] + sinusoid(pos(t)), fp32 [T, E] (and a copy in act dtype if x_act).
 * row(t) = (prev * mul_prev + tok * mul_cur) mod buckets with prev the token before (from *prev_token for t = 0),
 * row = buckets for position 0.  bigram may be NULL.  *prev_token is updated to tok[T-1].
 * inv_freq [ceil(E/2)] fp32: entry 2i = sin(p * inv_freq[i]), 2i+1 = cos(same). */
int cc_seq_embed(const int32_t* tokens, const int32_t* input_pos, int32_t* prev_token, const void* embed,
                 const void* bigram, const float* inv_freq, float* x, void* x_act, int32_t T, int32_t E, float scale,
                 int32_t buckets, int32_t mul_prev, int32_t mul_cur, int32_t table_dtype, int32_t act_dtype, void* stream);

/* Splits a fused projection row [H*Dk | G*Dk | G*Dv] (in_dtype, plus the fp32 bias row when given) per token: q and k heads divided by their root mean
 * square (when unit_norm), q multiplied by 1 + gain_coef * ln(floor((p + 1) / gain_every) + 1) (when gain_every > 0),
 * v <- (1 - *mix_lambda) v + *mix_lambda v_first (when v_first).  q_out fp32, k_out / v_out in out_dtype. */
int cc_seq_qkv_prepare(const void* qkv, int32_t in_dtype, const float* bias, const int32_t* input_pos,
                       const float* mix_lambda, const void* v_first, float* q_out, void* k_out, void* v_out,
                       int32_t out_dtype, int32_t T, int32_t H, int32_t G, int32_t Dk, int32_t Dv, float eps,
                       int32_t unit_norm, float gain_coef, int32_t gain_every, void* stream);

/* Attention of a chunk (any T >= 1) over cache + chunk; the cache is not written. */
int cc_seq_attention(const CcSeqAttn* a, void* stream);
/* T == 1: keys split over CTAs, partial results combined in split order by the last CTA of a head; with
 * a->append the new row is written to slot p mod L (k, v, pos, mask, cache_cts) by the same launch. */
int cc_seq_attention_decode(const CcSeqAttn* a, void* stream);
/* `window`: the layer's window plus its kept first positions, or its block size when it has one (the most keys a token
 * can see; 0 = all) */
uint64_t cc_seq_decode_workspace(int32_t H, int32_t G, int32_t Dv, int32_t L, int32_t window);
/* Writes rows of k_new / v_new into their slots; of a chunk longer than the ring only the rows that stay. */
int cc_seq_cache_append(const CcSeqAttn* a, void* stream);

/* x <- unit_rms(alpha * x + y) * (1 + w), fp32 [T, E] in place; y (y_dtype) may be NULL; a copy in act dtype goes to
 * x_act when given. */
int cc_seq_residual_norm(float* x, const void* y, int32_t y_dtype, const float* w, float alpha, float eps, void* x_act,
                         int32_t act_dtype, int32_t T, int32_t E, void* stream);

/* gu [T, 2F] = [gate | up] (io dtype): g = min(gate, limit), u = clamp(up, -limit, limit),
 * out [T, F] = g * sigmoid(slope * g) * (u + 1). */
int cc_seq_clamped_glu(const void* gu, void* out, int32_t io_dtype, int32_t out_dtype, float limit, float slope,
                       int32_t T, int32_t F, void* stream);

/*
 * One-token matrix-vector product out = epilogue(W xin) for the decode step, with the post-sum norm folded in:
 *   xin[k] = x[k]                                    (in_norm_w == NULL; x in x_dtype)
 *          = x[k] * rinv(x) * (1 + in_norm_w[k])      (x fp32 = a pre-norm sum; rinv = 1/sqrt(mean(x^2) + eps)),
 *            rounded to the weights' type, as the prompt path rounds its product inputs
 * epilogues (acc = W xin + bias in fp32):
 *   CC_GEMV_PLAIN     out[n] = acc                                             (fp32)
 *   CC_GEMV_RESIDUAL  out[n] = alpha * r[n] + acc, r = res or res * rinv(res) * (1 + res_norm_w)   (fp32 pre-norm sum)
 *   CC_GEMV_GLU       rows n and N + n of W: g = min(acc_n, limit), u = clamp(acc_{N+n}, +-limit),
 *                     out[n] = g * sigmoid(slope * g) * (u + 1)                 (out_dtype)
 * Every CTA recomputes the row statistics it needs (K and N floats from L2) instead of waiting for a norm kernel.
 */
#define CC_GEMV_PLAIN     0
#define CC_GEMV_RESIDUAL  1
#define CC_GEMV_GLU       2

typedef struct CcSeqGemv {
    const void* x;  int32_t x_dtype;
    const float* in_norm_w;
    const void* W;  int32_t w_dtype;      /* [N (2N for GLU), K] row-major */
    const float* bias;                    /* [N] or NULL (not with GLU) */
    const float* res;                     /* [N] fp32, RESIDUAL only */
    const float* res_norm_w;              /* [N] or NULL */
    float alpha, eps, limit, slope;
    int32_t mode;
    void* out;      int32_t out_dtype;
    int32_t N, K;
} CcSeqGemv;

int cc_seq_gemv(const CcSeqGemv* g, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Second part (csrc/seq/mix_kernels.cu): layers that carry per-sequence state besides a key/value cache.
 * Inputs named "fp32 [T, ld]" are usually column ranges of a fused projection's output: a pointer to the first
 * column and the row stride in elements.
 * ------------------------------------------------------------------------------------------------------------------ */

/* activations of cc_seq_gated_unit and of the expert kernels */
#define CC_ACT_NONE       0
#define CC_ACT_GELU_TANH  1  /* 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) */
#define CC_ACT_SILU       2  /* z sigmoid(z) */
#define CC_ACT_TANH       3
#define CC_ACT_SIGMOID    4
#define CC_ACT_RELU_SQ    5  /* max(z, 0)^2 */
#define CC_ACT_LAST       5

/* x[t] = embed[tok[t]] * scale, fp32 [T, E] */
int cc_seq_embed_rows(const int32_t* tokens, const void* embed, int32_t table_dtype, float* x, int32_t T, int32_t E,
                      float scale, void* stream);

/*
 * Gated residual sum fused with the grouped RMS norm that reads it.  Per row t (row rows[i] when `rows` is given):
 *   x[t] += a[t] * sigmoid(ga[t] + ba) + b[t] * sigmoid(gb[t] + bb)      (each term only if its pointer is set;
 *                                                                         no gate when ga / gb is NULL)
 *   h[i]  = x[t] split into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times w
 * h (fp32) and h_act (act_dtype) are optional outputs, compact in i; w == NULL stops after the sum.
 */
typedef struct CcSeqGatedNorm {
    float* x;                                   /* [*, E] fp32 residual stream, updated in place */
    const float* a;  int64_t lda;  const float* ga;  int64_t ldga;  const float* ba;
    const float* b;  int64_t ldb;  const float* gb;  int64_t ldgb;  const float* bb;
    const float* w;                             /* [E] */
    float* h;  void* h_act;  int32_t act_dtype;
    const int64_t* rows;                        /* [T] or NULL */
    int32_t T, E, groups;
    float eps;
    /* one token only (T == 1, no rows): the token shift of the normed row in the same pass.  hs = h + (shift_state - h)
     * * shift_mu, shift_state <- h; then mixes[m] = hs + (mix_state - hs) * mix_mu[m] for m < n_mix, mix_state <- hs. */
    float* shift_state;  const float* shift_mu;  void* hs_act;
    float* mix_state;  const float* mix_mu;  void* mixes;  int32_t n_mix;
} CcSeqGatedNorm;
int cc_seq_gated_group_norm(const CcSeqGatedNorm* g, void* stream);

/* Token shift: out[s][t] = h[t] + (h[t-1] - h[t]) * mu[s] for s < n, with h[-1] = state (fp32 [E]); afterwards
 * state = h[T-1].  out [n, T, E] in out_dtype and / or outf fp32 [T, E] (mix 0 only). */
int cc_seq_token_shift(const float* h, float* state, const float* mu, void* out, int32_t out_dtype, float* outf,
                       int32_t T, int32_t E, int32_t n, void* stream);

/* out[t, f] = act(in[t, off_gate + f]) * in[t, off_up + f]   (off_up < 0: no second factor); in fp32 [T, ld] */
int cc_seq_gated_unit(const float* in, int64_t ld, int32_t off_gate, int32_t off_up, void* out, int32_t out_dtype,
                      int32_t T, int32_t F, int32_t kind, void* stream);

/*
 * Rows of latent (low-rank) attention from the fused down-projection `in` fp32 [T, ld]:
 *   cq[t]   = rms_norm(in[t, off_q : off_q + q_rank]) * wq                          (dtype, skipped when q_rank == 0)
 *   krow[t] = [ rms_norm(in[t, off_kv : off_kv + kv_rank]) * wkv | rot(in[t, off_kv + kv_rank : + rot_dim]) ]
 *   vrow[t] = the first kv_rank columns of krow[t] again                            (optional)
 * rot() turns pairs (i, i + rot_dims/2) -- or (2i, 2i + 1) when `interleaved` -- of the first rot_dims entries by the
 * angle p * inv_freq[i], p = *input_pos + t.
 */
typedef struct CcSeqLatentPrep {
    const float* in;  int64_t ld;
    int32_t off_q, q_rank, off_kv, kv_rank, rot_dim, rot_dims;
    const float* wq;  const float* wkv;  const float* inv_freq;
    const int32_t* input_pos;
    void* cq;  void* krow;  void* vrow;  int32_t dtype;
    int32_t T;
    float eps;
    int32_t interleaved;
} CcSeqLatentPrep;
int cc_seq_latent_prepare(const CcSeqLatentPrep* a, void* stream);

/* In place on q fp32 [T, ld] = H heads of head_w columns: the segment [off, off + seg) of every head is rotated
 * (first `dims` entries, pairs (i, i + dims/2) or, when `interleaved`, (2i, 2i + 1), angle p * inv_freq[i]).  With
 * `tail`, the segment is also copied to tail[(t * H + h) * tail_ld + tail_off ...]. */
int cc_seq_rope_heads(float* q, int64_t ld, const int32_t* input_pos, const float* inv_freq, int32_t T, int32_t H,
                      int32_t head_w, int32_t off, int32_t seg, int32_t dims, float* tail, int64_t tail_ld,
                      int32_t tail_off, int32_t interleaved, void* stream);

/*
 * Per-head key / value rows from up-projected latents: kv_* fp32 [n, ld_kv] = [H*D key part | H*V values], lat_*
 * [n, ld_lat] (dtype) = latent rows whose columns kv_rank .. kv_rank + R are the shared rotated key part.
 * Old rows go to k_old [H, n_old, D + R] / v_old [H, n_old, V], new rows to k_new [n_new, H, D + R] / v_new [n_new, H, V].
 */
typedef struct CcSeqLatentExpand {
    const float* kv_old;  const float* kv_new;  int64_t ld_kv;
    const void* lat_old;  const void* lat_new;  int64_t ld_lat;
    void* k_old;  void* v_old;  void* k_new;  void* v_new;
    int32_t dtype, n_old, n_new, H, D, V, R, kv_rank;
} CcSeqLatentExpand;
int cc_seq_latent_expand(const CcSeqLatentExpand* a, void* stream);

/*
 * Absorbed one-token step of latent attention: all H query heads attend over one shared row per position.
 * q fp32 [H, Dk] (the query carried through the key up-projection | its rotated part), rows [L, Dk] in cache dtype
 * whose first C columns are also the value row, k_new [Dk] the row of this token (position *input_pos), which is the
 * newest key and, with `append`, is stored in slot position mod L (pos / mask / cache_cts as in CcSeqAttn).
 * y [H, C] = softmax(scale * q . row) weighted sum of the rows' first C columns.  Keys are addressed by position.
 * With `sink` (fp32 [H]) the softmax denominator also holds exp(sink[h]): a term without key or value.
 */
typedef struct CcSeqLatentDecode {
    const float* q;  const void* k_new;  void* k_cache;
    int32_t* pos;  uint8_t* mask;  int32_t* cache_cts;  const int32_t* input_pos;
    void* y;
    int32_t H, Dk, C, L, cache_dtype, y_dtype;
    float scale;
    int32_t append;
    void* workspace;  uint64_t workspace_bytes;   /* cc_seq_latent_decode_workspace() bytes; needs no clearing */
    const float* sink;
} CcSeqLatentDecode;
uint64_t cc_seq_latent_decode_workspace(int32_t H, int32_t C, int32_t L);
int cc_seq_latent_decode(const CcSeqLatentDecode* a, void* stream);

/*
 * Several one-token products in one launch (job j: out_j fp32 [N] = W_j [N, K] xin_j).  xin_j = x (x_dtype: fp32 or
 * the weights' type), or, with kind != CC_ACT_NONE or off_up >= 0, built from the fp32 row x as
 * act(x[off_gate + k]) * x[off_up + k] (no second factor when off_up < 0): the input side of a gated unit.
 */
#define CC_GEMV_MAX_JOBS 6
typedef struct CcSeqGemvJob {
    const void* x;  const void* W;  void* out;
    int32_t x_dtype, kind, off_gate, off_up, N, K;
} CcSeqGemvJob;
typedef struct CcSeqGemvMulti {
    CcSeqGemvJob job[CC_GEMV_MAX_JOBS];
    int32_t n_jobs, w_dtype;
} CcSeqGemvMulti;
int cc_seq_gemv_multi(const CcSeqGemvMulti* g, void* stream);

/* y [T, H, V] (dtype) *= sigmoid(g[t * ldg + h]) */
int cc_seq_head_gate(void* y, int32_t dtype, const float* g, int64_t ldg, int32_t T, int32_t H, int32_t V, void* stream);

/* One-token block-diagonal product: out[h * so + n] = W[h, n, :] . x[h * sx : h * sx + K]  (* sigmoid(gate[h])) */
int cc_seq_head_gemv(const void* W, int32_t w_dtype, const void* x, int32_t x_dtype, int64_t sx, void* out,
                     int32_t out_dtype, int64_t so, const float* gate, int32_t H, int32_t N, int32_t K, void* stream);

/*
 * Linear recurrence with a matrix state per head, fp32 throughout.  For t = 0 .. T-1, head h, with D-vectors
 * r, k, v and the decay w_t = exp(-exp(wraw_t + w0)):
 *   o_t[j]  = sum_i r_t[i] * (S[i][j] + u[i] * k_t[i] * v_t[j])
 *   S[i][j] = w_t[i] * S[i][j] + k_t[i] * v_t[j]
 * r, k, v, wraw, o: fp32 [T, H * D] contiguous; w0, u: [H * D]; state [H, D, D] is read and written.
 */
typedef struct CcSeqWkv {
    const float* r;  const float* k;  const float* v;  const float* wraw;
    const float* w0;  const float* u;
    float* state;  float* o;
    int32_t T, H, D;
} CcSeqWkv;
int cc_seq_wkv(const CcSeqWkv* a, void* stream);

/* out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * nw[h, :] * silu(graw[t, h, :])   (graw fp32 [T, ldg]) */
int cc_seq_head_norm_gate(const float* o, const float* graw, int64_t ldg, const float* nw, void* out, int32_t out_dtype,
                          int32_t T, int32_t H, int32_t D, float eps, void* stream);

/*
 * Router of a mixture of experts over n outputs (real and identity experts alike), logits fp32 [T, ld]:
 * scores s = softmax(logits) over all outputs, or sigmoid(logits) each on its own (`sigmoid_scores`); choice = s +
 * correction; the outputs form `groups` equal groups of neighbours and only those of the `keep` groups with the largest
 * group score can be chosen (the others count as minus infinity), a group's score being the sum of its `group_top`
 * largest choices (1 = its maximum); the `top` largest choices win (the lower index on a tie);
 * wts = s of the winners / (their sum + 1e-20) when `renormalize`, else s; both times weight_scale.
 * ids int32 [T, top], wts fp32 [T, top].
 */
int cc_seq_moe_route(const float* logits, int64_t ld, const float* correction, int32_t* ids, float* wts, int32_t T,
                     int32_t n, int32_t groups, int32_t keep, int32_t top, int32_t sigmoid_scores, int32_t group_top,
                     int32_t renormalize, float weight_scale, void* stream);

/* Groups the M = T * top (token, choice) pairs by real expert (id < n_real): counts [n_real], slot [M] = row of the
 * pair in expert order (-1 for an identity expert), perm [M] = token of each row. */
int cc_seq_moe_group(const int32_t* ids, int32_t M, int32_t top, int32_t n_real, int32_t* counts, int32_t* slot,
                     int32_t* perm, void* stream);
int cc_seq_gather_rows(const void* src, const int32_t* perm, void* dst, int32_t dtype, int32_t M, int32_t E, void* stream);

/* Experts for a few tokens without grouping: pair m = t * top + k with expert e = ids[m] < n_real:
 * act[m] = act(Wgu[e, 0:F] h[t]) * (Wgu[e, F:2F] h[t]),  y[m] = Wd[e] act[m]  (fp32 [M, E]).  Weights, h and act in dtype. */
int cc_seq_moe_expert_tokens(const void* Wgu, const void* Wd, const void* h, const int32_t* ids, void* act, float* y,
                             int32_t dtype, int32_t T, int32_t top, int32_t n_real, int32_t F, int32_t E, int32_t kind,
                             void* stream);

/* out[t] = sum_k wts[t, k] * (ids[t, k] < n_real ? y[slot[t, k]] : h[t]) + sigmoid(sg[t * ld_sg]) * shared[t];
 * slot == NULL means row t * top + k; shared may be NULL; sg == NULL means no gate on it; h may be NULL when there are
 * no identity experts. */
typedef struct CcSeqMoeCombine {
    const int32_t* ids;  const float* wts;  const int32_t* slot;
    const float* y;  const float* h;  const float* shared;  const float* sg;  int64_t ld_sg;
    float* out;
    int32_t T, E, top, n_real;
} CcSeqMoeCombine;
int cc_seq_moe_combine(const CcSeqMoeCombine* a, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Third part (csrc/seq/scan_kernels.cu): post-sum norms with layer scale and a weighted average over the depth,
 * short causal convolutions with a carried tail, two matrix-state recurrences (a state-space scan with a scalar decay
 * per head, and a delta rule with a decay per key channel), gated group norms, and rotations of query, key and value
 * heads.  fp32 arithmetic throughout; inputs named "fp32 [T, ld]" are column ranges of wider rows.
 * ------------------------------------------------------------------------------------------------------------------ */

/*
 * Norm after the sum.  Per row t (row rows[t] of x / y / y2 when `rows` is given; outputs are compact in t):
 *   r = y                                   (plain)     or  y / sqrt(mean(y^2) + eps) * y_norm_w   (y_norm_w set)
 *   r = y_coef * (r + the same of y2)        (y2 set; y_coef multiplies also without y2)
 *   s = alpha * x + y_scale * r              (x, y, y_scale each optional)
 *   n = (s - mean(s)) / sqrt(mean((s - mean(s))^2) + eps) * (w + gain_offset)     (center != 0)
 *     =  s / sqrt(mean(s^2) + eps) * (w + gain_offset)                             (center == 0)
 *   out[t] = n;  with coef:  mix[t] = sum_{j < n_prev} coef[j] * stack[j * stack_stride + t * E ...] + coef[n_prev] * n
 *   out_act[t] = mix[t] if coef else n, in act_dtype.
 */
typedef struct CcSeqSumNorm {
    const float* x;
    const float* y;   int64_t ldy;   const float* y_norm_w;
    const float* y2;  int64_t ldy2;  const float* y2_norm_w;
    float y_coef;
    const float* y_scale;
    const float* w;
    float alpha, eps, gain_offset;
    int32_t center;
    float* out;
    const float* stack;  int64_t stack_stride;  int32_t n_prev;  const float* coef;  float* mix;
    void* out_act;  int32_t act_dtype;
    const int64_t* rows;
    int32_t T, E;
} CcSeqSumNorm;
int cc_seq_sum_norm(const CcSeqSumNorm* a, void* stream);

/*
 * Causal convolution over time on each of C channels: out[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]),
 * where u[-k] for k = 1 .. taps-1 is tail[taps - 1 - k, c] (the inputs that came before this call; zeros at a
 * sequence's start).  Afterwards tail holds the last taps - 1 inputs.  u fp32 [T, ldu], w fp32 [C, taps], out fp32
 * [T, ldo], tail fp32 [taps - 1, C]; bias may be NULL; act is a CC_ACT_* kind.  taps >= 1.
 */
int cc_seq_short_conv(const float* u, int64_t ldu, const float* w, const float* bias, float* tail, float* out,
                      int64_t ldo, int32_t T, int32_t C, int32_t taps, int32_t act, void* stream);

/*
 * State-space scan, one state S [N, V] per head (head h reads group h / (H / G) of B and C):
 *   dt = softplus(dt_raw + dt_bias[h]);  a = exp(-exp(A_log[h]) * dt)
 *   S <- a * S + dt * B_t x_t^T;   y_t = S^T C_t + D[h] * x_t
 * x fp32 [T, ldx] (H * V columns), B, C fp32 [T, ldbc] (G * N columns each), dt_raw fp32 [T, lddt] (H columns),
 * y fp32 [T, H * V] contiguous, state fp32 [H, N, V] read and written.  Exactly sequential in t.
 */
typedef struct CcSeqSsdScan {
    const float* x;  int64_t ldx;
    const float* B;  const float* C;  int64_t ldbc;
    const float* dt_raw;  int64_t lddt;
    const float* dt_bias;  const float* A_log;  const float* D;
    float* state;  float* y;
    int32_t T, H, G, N, V;
} CcSeqSsdScan;
int cc_seq_ssd_scan(const CcSeqSsdScan* a, void* stream);

/*
 * Delta rule with a decay per key channel, one state S [D, V] per head (head h reads q / k head h / (H / G)):
 *   qn = q / sqrt(sum(q^2) + unit_eps) * q_scale;  kn = k / sqrt(sum(k^2) + unit_eps);  beta = sigmoid(beta_raw)
 *   g[i] = exp(-exp(A_log[h]) * softplus(a_raw[h * D + i] + dt_bias[h * D + i]))
 *   S <- diag(g) S;  u = beta * (v - S^T kn);  S <- S + kn u^T;  o = S^T qn
 * q, k fp32 [T, ldqk] (G * D columns), v fp32 [T, ldv] (H * V), beta_raw fp32 [T, ldb] (H), a_raw fp32 [T, lda]
 * (H * D), o fp32 [T, H * V] contiguous, state fp32 [H, D, V] read and written.  Exactly sequential in t.
 */
typedef struct CcSeqDeltaScan {
    const float* q;  const float* k;  int64_t ldqk;
    const float* v;  int64_t ldv;
    const float* beta_raw;  int64_t ldb;
    const float* a_raw;  int64_t lda;
    const float* dt_bias;  const float* A_log;
    float* state;  float* o;
    int32_t T, H, G, D, V;
    float q_scale, unit_eps;
    /* prepared != 0: q, k hold qn, kn per head ([T, H * D], G == H), a_raw holds the decays g, beta_raw holds beta, and
     * qk [T, H] holds qn . kn, all as cc_seq_delta_prepare writes them; the scan then only runs the recurrence. */
    const float* qk;
    int32_t prepared;
} CcSeqDeltaScan;
int cc_seq_delta_scan(const CcSeqDeltaScan* a, void* stream);
/* The per-token preparation of cc_seq_delta_scan alone, spread over the GPU: qn, kn, gd fp32 [T, H * D], beta, qk fp32
 * [T, H], from an unprepared argument block.  Worth its launch for long steps; gives the same bits as the scan's own. */
int cc_seq_delta_prepare(const CcSeqDeltaScan* a, float* qn, float* kn, float* gd, float* beta, float* qk, void* stream);

/*
 * Rows y fp32 [T, W] in `groups` equal consecutive parts, each divided by its root mean square, times w[col mod
 * w_len], with a gate act(gate[t, col]) applied before the norm (gate_first != 0: the norm sees the gated values) or
 * after it.  gate fp32 [T, ldg] or NULL; out [T, W] in out_dtype.
 */
int cc_seq_gated_rms_groups(const float* y, const float* gate, int64_t ldg, int32_t gate_act, int32_t gate_first,
                            const float* w, int32_t w_len, void* out, int32_t out_dtype, int32_t T, int32_t W,
                            int32_t groups, float eps, void* stream);

/*
 * Query, key and value heads of T tokens from fp32 rows `in` [T, ld] (q at off_q: H heads of Dk, k at off_k: G heads
 * of Dk, v at off_v: G heads of Dv).  q and k heads: divided by their root mean square times q_norm_w / k_norm_w
 * ([Dk], when set), then the first rot_dims entries turned by the angle p * inv_freq[i] for pair i, p = *input_pos + t;
 * v heads: all Dv entries turned by p * v_inv_freq[m] (when set).  Pairs are (2i, 2i + 1) when interleaved, else
 * (i, i + dims / 2).  A pair (a, b) becomes (a cos - b sin, b cos + a sin).  q_out fp32, k_out / v_out in out_dtype.
 */
typedef struct CcSeqQkvRope {
    const float* in;  int64_t ld;
    int32_t off_q, off_k, off_v, H, G, Dk, Dv;
    const float* q_norm_w;  const float* k_norm_w;  float eps;
    int32_t rot_dims, interleaved;
    const float* inv_freq;  const float* v_inv_freq;
    const int32_t* input_pos;
    float* q_out;  void* k_out;  void* v_out;  int32_t out_dtype;
    int32_t T;
} CcSeqQkvRope;
int cc_seq_qkv_rope(const CcSeqQkvRope* a, void* stream);

/* out[t, h, :] = turn(y[t, h, :], sign * p * inv_freq) * sigmoid(gate[t * ldg + h]): the first `dims` entries of each
 * head are turned (pairs as above), p = *input_pos + t; gate may be NULL.  y fp32 [T, H, Dv], out in out_dtype. */
int cc_seq_turn_heads_gate(const float* y, const int32_t* input_pos, const float* inv_freq, int32_t dims,
                           int32_t interleaved, float sign, const float* gate, int64_t ldg, void* out,
                           int32_t out_dtype, int32_t T, int32_t H, int32_t Dv, void* stream);

/* x <- cap * tanh(x / cap), fp32, n elements, in place */
int cc_seq_softcap(float* x, int64_t n, float cap, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Fourth part (csrc/seq/par_kernels.cu): layers whose sublayers read norms of the same stream, each through a short
 * causal convolution added to its own input; whole-row query / key norms; the polynomial-of-unit-RMS activation.
 * ------------------------------------------------------------------------------------------------------------------ */

/*
 * Residual sum + one unit-RMS pass + up to CC_PAR_MAX_OUT sublayer inputs.  Per row t of the fp32 stream x [T, E]:
 *   x[t] += a[t] + b[t] + add              (each optional: the sublayer results of the layer before, a vector per pass)
 *   xh[t] = x[t] / sqrt(mean(x[t]^2) + eps)
 *   h_s[t] = xh[t] * gain_s;   out_s[t] = h_s[t] + sum_j conv_w_s[c, j] * h_s[t - taps + 1 + j]    (conv_w_s NULL: h_s[t])
 * The rows before the step's first token come from `tail` fp32 [taps - 1, E] (unit-RMS rows xh, oldest first; zeros
 * at a sequence's start), which afterwards holds the step's last taps - 1 rows.  conv_w_s fp32 [E, taps], the last
 * tap meets the current token.  out_s [T, E] in act_dtype.  rinv fp32 [T] is scratch (needed when T > 1): the rows'
 * 1 / sqrt(mean + eps), handed from the launch that sums to the launch that convolves.
 */
#define CC_PAR_MAX_OUT 4
typedef struct CcSeqParNorm {
    float* x;
    const float* a;  int64_t lda;
    const float* b;  int64_t ldb;
    const float* add;
    float* rinv;
    float* x_out;              /* one token only (T == 1), may be NULL: the summed row goes here instead of x (a buffer of
                                * its own), and the row's channels are spread over the GPU */
    float* tail;
    const float* gain[CC_PAR_MAX_OUT];
    const float* conv_w[CC_PAR_MAX_OUT];
    void* out[CC_PAR_MAX_OUT];
    int32_t n_out, act_dtype, T, E, taps;
    float eps;
} CcSeqParNorm;
int cc_seq_par_norm(const CcSeqParNorm* g, void* stream);

/*
 * From fp32 rows `in` [T, ld]: q (nq columns at off_q) and k (nk columns at off_k) are each divided by the root mean
 * square of the whole range (all heads at once) and multiplied by wq [nq] / wk [nk]; v (nv columns at off_v) is copied.
 * q_out fp32 [T, nq]; k_out [T, nk] and v_out [T, nv] in out_dtype.
 */
typedef struct CcSeqQkRowNorm {
    const float* in;  int64_t ld;
    int32_t off_q, nq, off_k, nk, off_v, nv;
    const float* wq;  const float* wk;
    float* q_out;  void* k_out;  void* v_out;
    int32_t out_dtype, T;
    float eps;
} CcSeqQkRowNorm;
int cc_seq_qk_row_norm(const CcSeqQkRowNorm* a, void* stream);

/* out[t] = coef[0] N(z) + coef[1] N(z^2) + coef[2] N(z^3) + coef[3], z = in[t, 0:F] (fp32 [T, ld]), powers element by
 * element, N(u) = u / sqrt(mean(u^2) + eps) over the F columns; coef fp32 [4] on the device; out [T, F] in out_dtype. */
int cc_seq_poly_norm(const float* in, int64_t ld, const float* coef, void* out, int32_t out_dtype, int32_t T, int32_t F,
                     float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CC_B200_SEQ_H */
