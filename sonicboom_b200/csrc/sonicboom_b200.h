/* Public C interface of the sonicboom_b200 kernel libraries (sm_100a).
 *
 * Two kinds of shared library are built from this folder:
 *   libsonicboom_b200.so              the core library: everything under "core library" below;
 *   libsonicboom_b200_attn_hd<N>.so   one per head size N (16 ... 256 in steps of 16): the
 *                                     tensor-core attention kernels, under "attention library".
 * Every library also exports sb_last_error, sb_pdl_enabled and sb_set_pdl (its own copies).
 *
 * Conventions.  Every entry point takes raw device pointers and a CUDA stream, checks its
 * arguments on the host before anything is launched and returns an SbStatus; on a non-zero
 * status sb_last_error() of the same library describes what was refused.  Nothing here
 * allocates device memory: scratch is passed in by the caller (or, for
 * sb_attention_decode_static, lives in the library: see no_alloc.h).  Tensors are contiguous and
 * row-major; dtype arguments are SbDtype codes.  The header compiles as C and as C++.
 */
#ifndef SONICBOOM_B200_H
#define SONICBOOM_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__) || defined(__CUDA_RUNTIME_API_H__) || defined(__DRIVER_TYPES_H__)
#include <cuda_runtime_api.h>
typedef cudaStream_t sb_stream_t;
#else
typedef struct CUstream_st* sb_stream_t;       /* the type cuda_runtime_api.h calls cudaStream_t */
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum SbDtype { SB_F32 = 0, SB_BF16 = 1 };
enum SbStatus { SB_OK = 0, SB_ERR_ARG = 1, SB_ERR_UNSUPPORTED = 2, SB_ERR_CUDA = 3 };
/* What a product does with its finished rows.  SB_EPI_SWIGLU: the weight's rows alternate in
 * blocks of 8 (8 gate rows, the 8 up rows of the same outputs); out[m, o] = silu(gate) * up and
 * has N / 2 columns. */
enum SbEpilogue { SB_EPI_NONE = 0, SB_EPI_BIAS = 1, SB_EPI_RESIDUAL = 2, SB_EPI_SWIGLU = 3 };
/* The activation of a gated feed-forward: act(gate) * up. */
enum SbGate { SB_GATE_SILU = 0, SB_GATE_CLAMPED = 1, SB_GATE_GELU_TANH = 2 };
/* Kernel classes: bits of the mask that says which kernels are launched with programmatic
 * dependent launch (sb_set_pdl). */
enum SbKernelClass {
  SB_K_TC5 = 1,          /* tcgen05 products */
  SB_K_SKINNY = 2,       /* weight-streaming and tiled mma.sync products */
  SB_K_ATTENTION = 4,
  SB_K_ELEMENTWISE = 8,  /* embedding, norms, rotation, casts, small adds */
  SB_K_REDUCE = 16,      /* the split-K reduce of the tcgen05 product */
  SB_K_OTHER = 32        /* sampler, plain kernels */
};

/* The rotation and cache write that may finish a fused q|k|v product (the arguments of
 * sb_rope_store without the input row, which the product supplies). */
typedef struct SbRopeStore {
  int n_q_heads, n_kv_heads, hd, rot;
  const float* inv_freq;
  const int32_t* row_seq;
  const int32_t* row_pos;
  const int32_t* page_off;
  const int32_t* page_ids;
  int page_size;
  void* cache;                 /* bfloat16 pages of the schedule entry; null: queries only */
  void* q_out;                 /* bfloat16 [rows, n_q_heads, hd] */
} SbRopeStore;

/* What may accompany a product (all optional): the RMSNorm of its finished rows, memory to ask
 * into L2 for a later kernel, and the rotation + cache write of a q|k|v product's rows (then the
 * product's own output is not written: `out` may be null). */
typedef struct SbLinearExtras {
  const void* norm_weight;     /* null: no norm */
  int norm_weight_dtype;
  float norm_eps;
  void* norm_out;
  int norm_out_dtype;
  const void* warm;            /* null: nothing; else bytes a later kernel will stream */
  size_t warm_bytes;
  const SbRopeStore* rope;     /* null: none; only where sb_gemm_tc5_fuses_rope says so */
  float gate_limit;            /* SB_EPI_SWIGLU only: > 0 makes the gated epilogue a sigmoid(gate_slope a) (b + 1), */
  float gate_slope;            /* a = min(gate, limit), b = clamp(up, -limit, limit); 0: silu(gate) * up */
  int gate_kind;               /* SB_EPI_SWIGLU only: SB_GATE_GELU_TANH makes it gelu(gate) * up; else by gate_limit */
} SbLinearExtras;

/* One row's sampling record (sb_sample reads an array of them from device memory). */
typedef struct SbSampleParams {
  float temperature, top_p, min_p, repeat_penalty, presence_penalty, frequency_penalty;
  uint32_t top_k;
  int32_t history_len;         /* tokens of this row in `history` (already cut to the window) */
  uint64_t seed;
  uint64_t position;           /* absolute position of the token being produced */
} SbSampleParams;

/* ------------------------------------------------------------------ every library */
const char* sb_last_error(void);
int sb_pdl_enabled(void);                 /* the mask of SbKernelClass bits in force */
void sb_set_pdl(int mask);

/* ------------------------------------------------------------------ core library */
int sb_abi_version(void);

/* out[t, :] = table[tokens[t], :] * scale as float32; an id outside the table gives NaN. */
int sb_embed(const int32_t* tokens, int n_rows, const void* table, int table_dtype, int vocab,
             int width, float scale, float* out, sb_stream_t stream);
/* out[r] = x[rows ? rows[r] : r] / sqrt(mean(x^2) + eps) * weight */
int sb_rmsnorm(const float* x, const int32_t* rows, int n_rows, int width, const void* weight,
               int weight_dtype, float eps, void* out, int out_dtype, sb_stream_t stream);
/* The same over the first `width` values of input rows that lie x_ld values apart. */
int sb_rmsnorm_ld(const float* x, int x_ld, const int32_t* rows, int n_rows, int width, const void* weight,
                  int weight_dtype, float eps, void* out, int out_dtype, sb_stream_t stream);
int sb_softcap(float* x, size_t n, float cap, sb_stream_t stream);     /* x = cap tanh(x / cap) */
int sb_add_bias(float* x, const void* bias, int bias_dtype, int rows, int width, sb_stream_t stream);   /* x[m, n] += bias[n] */
int sb_cast(const void* in, int in_dtype, void* out, int out_dtype, size_t n, sb_stream_t stream);
/* Rotates q and k of the fused row [q | k | v], writes q to q_out and k, v into the pages of
 * each row's sequence; a position without a page in its own sequence's list writes nothing. */
int sb_rope_store(const float* qkv, int n_rows, int n_q_heads, int n_kv_heads, int hd, int rot,
                  const float* inv_freq, const int32_t* row_seq, const int32_t* row_pos,
                  const int32_t* page_off, const int32_t* page_ids, int page_size, void* cache,
                  int cache_dtype, void* q_out, int q_dtype, int has_kv, sb_stream_t stream);

/* out[M, N] = A[M, K] . W[N, K]^T with an SbEpilogue; float32 accumulation. */
int sb_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                  int epilogue, const void* bias, int bias_dtype, const float* residual,
                  void* out, int out_dtype, sb_stream_t stream);
int sb_gemm_skinny(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                   int epilogue, const void* bias, int bias_dtype, const float* residual,
                   void* out, int out_dtype, sb_stream_t stream);
/* sb_gemm_skinny with SB_EPI_SWIGLU's layout and the gated activation gate_kind names (SB_GATE_CLAMPED
 * with its limit and slope, or SB_GATE_GELU_TANH; see SbLinearExtras). */
int sb_gemm_skinny_gated(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                         void* out, int out_dtype, float gate_limit, float gate_slope, int gate_kind,
                         sb_stream_t stream);
int sb_gemm_tiled(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                  int epilogue, const void* bias, int bias_dtype, const float* residual,
                  void* out, int out_dtype, sb_stream_t stream);
/* TMA + tcgen05.  form: 0 by the number of rows, 1 the normal form, 2 the swapped (decode) form. */
int sb_gemm_tc5(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                int epilogue, const void* bias, int bias_dtype, const float* residual, void* out,
                int out_dtype, void* scratch, size_t scratch_bytes, int n_sms, int form,
                sb_stream_t stream);
int sb_gemm_tc5_ex(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                   int epilogue, const void* bias, int bias_dtype, const float* residual,
                   void* out, int out_dtype, void* scratch, size_t scratch_bytes, int n_sms,
                   int form, const SbLinearExtras* extras, sb_stream_t stream);
size_t sb_gemm_tc5_scratch_bytes(int M, int N, int K, int n_sms);
int sb_gemm_tc5_fuses_norm(int M, int N, int K, int n_sms, int epilogue, int out_dtype, int form);
/* Whether sb_gemm_tc5_ex can finish a q|k|v product of these sizes with the rotation and the
 * cache write (the split-K decode form, bfloat16 queries and cache, head sizes in steps of 8). */
int sb_gemm_tc5_fuses_rope(int M, int N, int K, int n_sms, int n_q_heads, int n_kv_heads, int hd,
                           int rot, int has_kv);
int sb_tc5_status(void);      /* 0, or the code of a bounded wait that gave up; clears it */
void sb_gemm_tc5_pairs(int mode);   /* products of more than 128 rows on pairs of SMs: 1 yes, 0 no, -1 by SB_TC5_PAIR */
void sb_gemm_tc5_force_width(int bn);   /* 256, 240, 224, 208 or 192 for every many-rows product; else by the sizes */
int sb_gemm_tc5_tile_width(int M, int N, int n_sms);   /* tile width of the many-rows form; 0: that form does not run */

/* ---- residual-stream rows ----
 * out[r] = x[r] + y[r] / sqrt(mean(y[r]^2) + eps) * w (w has `width` values): a sublayer's result,
 * normed, joins the stream.  With `normed` non-null the RMS norm of the finished row (weight
 * next_w, next_eps) is written too, in normed_dtype.  out may be x. */
int sb_norm_add(const float* y, const float* x, int n_rows, int width, const void* w, int w_dtype,
                float eps, float* out, const void* next_w, int next_w_dtype, float next_eps,
                void* normed, int normed_dtype, sb_stream_t stream);
/* out[r] = sum over j < n_inputs of coef[j] * planes[j * plane + r * width ...], j ascending; the
 * optional norm of the finished row as in sb_norm_add.  With join_y non-null the last plane is made
 * first, as sb_norm_add would: planes[n_inputs - 1][r] = join_x[r] + norm(join_y[r]) * join_w
 * (join_w in the coefficients' dtype; join_x may be that plane). */
int sb_depth_mix(float* planes, size_t plane, int n_inputs, const void* coef, int coef_dtype,
                 int n_rows, int width, float* out, const void* next_w, int next_w_dtype,
                 float next_eps, void* normed, int normed_dtype, const float* join_y,
                 const float* join_x, const void* join_w, int join_w_dtype, float join_eps,
                 sb_stream_t stream);
/* gu[r] = [gate (ff) | up (ff)], or with `interleaved` blocks of 8 gates followed by the 8 up values of
 * the same outputs (ff a multiple of 8); out[r, c] = a sigmoid(alpha a) (b + 1), a = min(gate, limit),
 * b = clamp(up, -limit, limit). */
int sb_glu_clamped(const float* gu, int n_rows, int ff, float limit, float alpha, int interleaved,
                   void* out, int out_dtype, sb_stream_t stream);
/* The same rows with the activation named by `kind` (SbGate): silu(gate) * up, the clamped form of
 * sb_glu_clamped, or gelu(gate) * up with gelu(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))). */
int sb_gated_act(const float* gu, int n_rows, int ff, int kind, float limit, float alpha, int interleaved,
                 void* out, int out_dtype, sb_stream_t stream);
int sb_scale(float* x, size_t n, float c, sb_stream_t stream);          /* x *= c */

/* ---- attention over a cached latent ----
 * proj[r] = [n_heads x (dim | rd) | rank | rd] (the last two only with has_kv).  Rotates the first
 * `rot` values of every rd part in interleaved pairs (2i, 2i + 1) by float(pos) * inv_freq[i];
 * writes each head's rotated part to q_wide[r, h, rank : rank + rd] (q_wide lies [head group][row][head
 * in group][rank + rd] with groups of q_group heads; q_group = n_heads is [row][head]); with has_kv, RMS-norms the
 * latent (weight cnorm, eps) and writes the page row of the position: key plane [latent | rotated
 * key part], value plane [latent | zeros].  The cache entry has one head of size rank + rd.
 * `kv` (or null): rows [rank | rd] of their own, kv_ld values apart, instead of the tail of proj's rows.
 * interleaved = 0: the pairs are (i, i + rot/2).  rot_scale multiplies every cosine and sine. */
int sb_latent_prep(const float* proj, int n_rows, int n_heads, int dim, int rd, int rank, int rot,
                   const float* inv_freq, const int32_t* row_seq, const int32_t* row_pos,
                   const int32_t* page_off, const int32_t* page_ids, int page_size, const void* cnorm,
                   int cnorm_dtype, float eps, void* cache, int cache_dtype, void* q_wide, int q_dtype,
                   int q_group, int has_kv, const float* kv, int kv_ld, int interleaved, float rot_scale,
                   sb_stream_t stream);
/* out[r * out_ld + h * out_hs + n] = sum_k in[r * in_ld + h * in_hs + k] * W[(h * N + n) * K + k] */
int sb_head_linear(const void* in, int in_dtype, size_t in_ld, size_t in_hs, const void* W, int w_dtype,
                   int n_rows, int n_heads, int N, int K, void* out, int out_dtype, size_t out_ld,
                   size_t out_hs, sb_stream_t stream);

/* ---- matrix-memory recurrence (mLSTM) ----
 * proj[r] = [q heads*dim | k heads*dim | v heads*vdim | g heads*vdim | x_i heads | x_f heads] float32.
 * state: float32 [slot, heads, vdim + 1, col_stride] with col_stride >= dim + 1 (column vdim is the
 * normalizer; after a column's dim values comes its copy of the running maximum).  sb_mlstm_scan walks every sequence's rows in order from its slot's state and leaves the
 * state after the last row; num [rows, heads, vdim + 1] and m_row [rows, heads] receive the
 * numerators and maxima; max_new is an upper bound of any sequence's rows in the step.  sb_mlstm_out divides, norms each head (eps), applies norm_w
 * [heads*vdim] and the gate sigmoid(g): out [rows, heads*vdim]. */
int sb_mlstm_scan(const float* proj, int n_seqs, const int32_t* seq_row0, const int32_t* seq_slot,
                  int n_heads, int dim, int vdim, const void* i_bias, const void* f_bias, int bias_dtype,
                  float cap, float q_scale, int max_new, float* state, int col_stride, float* num,
                  float* m_row, sb_stream_t stream);
int sb_mlstm_out(const float* num, const float* m_row, const float* proj, int n_rows, int n_heads,
                 int dim, int vdim, const void* norm_w, int norm_w_dtype, float eps, void* out,
                 int out_dtype, sb_stream_t stream);

/* Plain attention over the paged cache (float32 arithmetic, any head size up to 1024).  sink: null,
 * or one float32 per query head whose exponential joins that head's softmax denominator. */
int sb_attention_plain(const void* q, void* out, int act_dtype, int n_rows, const int32_t* row_seq,
                       const int32_t* row_pos, const int32_t* page_off, const int32_t* page_ids,
                       int page_size, const void* cache, int cache_dtype, int n_q_heads,
                       int n_kv_heads, int hd, int window, float scale, const float* sink,
                       float softcap, sb_stream_t stream);

/* ---- the stream, the feed-forward and mixers with projections of their own kind ----
 * out[r] = x[r] + add[r] + vec (add [rows, width] float32 and vec [width] are optional; out may be
 * x); the optional norm of the finished row as in sb_norm_add. */
int sb_stream_add(const float* x, const float* add, const void* vec, int vec_dtype, int n_rows,
                  int width, float* out, const void* next_w, int next_w_dtype, float next_eps,
                  void* normed, int normed_dtype, sb_stream_t stream);
/* out[r] = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with N(u) = u / sqrt(mean(u^2) + eps) over the row's
 * ff values, powers element by element; coef holds the four numbers. */
int sb_polynorm(const float* z, int n_rows, int ff, const void* coef, int coef_dtype, float eps,
                void* out, int out_dtype, sb_stream_t stream);
/* Projection rows (float32, row stride ld; queries at q_off [n_q_heads x dim], keys at k_off
 * [n_kv_heads x dim], values at v_off [n_kv_heads x vdim], or v_off < 0: the values are the key
 * projection as it is) to queries q_out [rows, n_q_heads, hd] and the cache rows of each
 * position (one entry's pages, heads of size hd >= dim, vdim; the padding is zeros).  With
 * q_norm / k_norm the whole q (k) projection of a row is RMS-normed with that weight first.  The
 * first `rot` values of every q and k head turn by float(pos) * inv_freq[i], in pairs
 * (i, i + rot/2), or (2i, 2i + 1) with `interleaved`; with v_inv_freq [vdim/2] every value head turns
 * the same way over all vdim.  has_kv = 0: queries only.
 * head_norm 1: every q and k head is RMS-normed by itself before the rotation, q_norm / k_norm being
 * one weight [dim] for all heads; head_norm 2: every head is divided by its root mean square after the
 * rotation (no weights).  rot_scale multiplies every cosine and sine of the q and k rotation. */
int sb_attn_prep(const float* proj, int n_rows, int ld, int q_off, int k_off, int v_off,
                 int n_q_heads, int n_kv_heads, int dim, int vdim, int hd, int rot, int interleaved,
                 const float* inv_freq, const float* v_inv_freq, const void* q_norm,
                 const void* k_norm, int norm_dtype, int head_norm, float rot_scale, float eps,
                 const int32_t* row_seq, const int32_t* row_pos, const int32_t* page_off,
                 const int32_t* page_ids, int page_size, void* cache, int cache_dtype, void* q_out,
                 int q_dtype, int has_kv, sb_stream_t stream);
/* out [rows, n_heads * vdim] = the first vdim values of every head of in [rows, n_heads, hd], turned
 * by -float(pos) * v_inv_freq[i] in the same pairs (v_inv_freq null: copied).  With `gate`, head h of
 * row r is multiplied by sigmoid(gate[r * gate_ld + h]). */
int sb_attn_unrotate(const void* in, void* out, int dtype, int n_rows, int n_heads, int hd, int vdim,
                     int interleaved, const float* v_inv_freq, const int32_t* row_pos,
                     const float* gate, int gate_ld, sb_stream_t stream);
/* In place on projection rows: q (at q_off) and k (at k_off), [n_heads x dim] each, are rotated
 * (the first `rot` of every head, pairs as in sb_attn_prep) and multiplied by q_scale / k_scale; z
 * [rows, n_heads * dim], if given, becomes exp(logsigmoid(z) * inv_tau).  With a2 [n_heads * dim,
 * rank] and a2_bias the logits are made here first: z = a2 . proj[row, a1_off : a1_off + rank] + a2_bias
 * (z is then written only). */
int sb_linrec_prep(float* proj, int n_rows, int ld, int q_off, int k_off, int n_heads, int dim,
                   float q_scale, float k_scale, int rot, int interleaved, const float* inv_freq,
                   const int32_t* row_pos, float* z, float inv_tau, const void* a2, const void* a2_bias,
                   int a2_dtype, int rank, int a1_off, sb_stream_t stream);
/* S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head and sequence, token by token, from
 * and to state [slot, n_heads, vdim, dim] float32; a_t from decay [rows, n_heads * dim], or one
 * fixed value per head from head_decay [n_heads], or one value per token and head from
 * token_decay [rows, n_heads] (exactly one of the three).  heads_per_qk neighbouring heads read the
 * same q and k (q and k then hold n_heads / heads_per_qk heads).  out [rows, n_heads, vdim]. */
int sb_linrec_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay,
                   const float* head_decay, const float* token_decay, int heads_per_qk, int n_seqs,
                   const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim, int vdim,
                   float* state, float* out, sb_stream_t stream);
void sb_linrec_force_columns(int cpt);   /* 1 or 2 columns per thread in sb_linrec_scan; 0: by the sizes */
/* out [rows, n_heads * vdim] = o / sqrt(mean over vdim of o^2 + eps) * norm_w (optional: [vdim] for
 * all heads, or [n_heads * vdim] with w_per_head) * gate(g), g at g_off of the projection row;
 * the gate is silu, or the logistic function with gate_sigmoid. */
int sb_linrec_out(const float* o, const float* proj, int n_rows, int ld, int g_off, int n_heads,
                  int vdim, const void* norm_w, int norm_w_dtype, int w_per_head, int gate_sigmoid,
                  float eps, void* out, int out_dtype, sb_stream_t stream);

/* ---- rows that look at their neighbours in the sequence; the layer norm ----
 * out[r] = table[tokens[r]] * scale + pair[i], i = (previous token * mul_prev + token * mul_cur) mod
 * buckets, or i = buckets for a sequence's first token (pair has buckets + 1 rows).  The token before
 * a step's first row comes from prev_token[slot]; sb_keep_last_token stores a step's last tokens there. */
int sb_embed_pair(const int32_t* tokens, int n_rows, const int32_t* row_seq, const int32_t* row_pos,
                  const int32_t* seq_row0, const int32_t* seq_slot, const int32_t* prev_token,
                  const void* table, int table_dtype, int vocab, const void* pair, int buckets,
                  int mul_prev, int mul_cur, int width, float scale, float* out, sb_stream_t stream);
int sb_keep_last_token(const int32_t* tokens, const int32_t* seq_row0, const int32_t* seq_slot,
                       int n_seqs, int32_t* prev_token, sb_stream_t stream);
/* out[r] = (x - mean) / sqrt(var + eps) * weight over the row x[rows ? rows[r] : r] */
int sb_layernorm(const float* x, const int32_t* rows, int n_rows, int width, const void* weight,
                 int weight_dtype, float eps, void* out, int out_dtype, sb_stream_t stream);
/* out[r, out_off + c] = act([x_t +] [bias +] sum_j w[c, j] x_(t - taps + 1 + j)) over the `channels`
 * columns of x at x_off; taps before a step's first row of a sequence come from state [slot,
 * taps - 1, channels] (float32), which then receives the step's last taps - 1 inputs; act 1: silu. */
int sb_causal_conv(const float* x, int n_rows, int ld, int x_off, int channels, int taps, const void* w,
                   const void* bias, int w_dtype, int act, int add_input, int n_seqs,
                   const int32_t* row_seq, const int32_t* row_pos, const int32_t* seq_row0,
                   const int32_t* seq_pos0, const int32_t* seq_slot, float* state, void* out,
                   int out_dtype, int ld_out, int out_off, sb_stream_t stream);

/* ---- the generalized delta rule ----
 * aux [rows, 3, n_heads * dim] = decays exp(-decay_scale * sigmoid(w2 . tanh(proj[z_off : z_off + rank])
 * + w0)) | sigmoid(proj[a_off ...] + a_bias) * u | u, u = k / sqrt(sum over the head of k^2 + key_eps). */
int sb_delta_prep(const float* proj, int n_rows, int ld, int k_off, int a_off, int z_off, int n_heads,
                  int dim, int rank, const void* w2, const void* w0, const void* a_bias, int w_dtype,
                  float decay_scale, float key_eps, float* aux, sb_stream_t stream);
/* S_t = diag(w) S_(t-1) - (a u)(u^T S_(t-1)) + k v^T, o_t = S_t^T r, from and to state [slot, n_heads,
 * dim, dim] float32 (value channel by value channel); out [rows, n_heads, dim]. */
int sb_delta_scan(const float* proj, int ld, int r_off, int k_off, int v_off, const float* aux, int n_seqs,
                  const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim, float* state,
                  float* out, sb_stream_t stream);

/* ---- the state-space mixer's rows ----
 * decay [rows, n_heads] = exp(-exp(a_log) dt), dt = softplus(proj[dt_off + h] + dt_bias); the row
 * buffer's columns at xdt_off receive dt * (its columns at x_off). */
int sb_ssd_prep(const float* proj, int n_rows, int ld_proj, int dt_off, float* xbc, int ld, int x_off,
                int xdt_off, int n_heads, int vdim, const void* dt_bias, const void* a_log, int w_dtype,
                float* decay, sb_stream_t stream);
/* out [rows, n_heads * vdim] = rms over each of norm_groups equal parts of ((o + d_skip[h] x) silu(z)),
 * times norm_w. */
int sb_ssd_out(const float* o, const float* xbc, int n_rows, int ld, int x_off, const float* proj,
               int ld_proj, int z_off, int n_heads, int vdim, int norm_groups, const void* d_skip,
               const void* norm_w, int w_dtype, float eps, void* out, int out_dtype, sb_stream_t stream);

/* ---- attention with logistic weights (see attn_sigmoid.cu) ---- */
int sb_attention_sigmoid(const void* q, void* out, int act_dtype, int n_rows, const int32_t* row_seq,
                         const int32_t* row_pos, int n_seqs, int max_new, const int32_t* seq_row0,
                         const int32_t* seq_pos0, const int32_t* page_off, const int32_t* page_ids,
                         int page_size, const void* cache, int cache_dtype, int n_q_heads,
                         int n_kv_heads, int hd, int window, int keep_first, float scale, float softcap,
                         const float* head_bias, sb_stream_t stream);

/* ---- mixture of experts (see moe.cu) ----
 * ids, weights [rows, top]; order [pairs]; meta [1 + 3 * sb_moe_max_tiles]; w of sb_moe_up [experts, 2
 * (gate, up), ff, width], of sb_moe_down [experts, width, ff]; act [pairs, ff] in the activation dtype
 * (in grouped order); pair_out [pairs, width] float32 (in pair order). */
int sb_moe_route(const float* logits, int n_rows, int n_experts, int top, int32_t* ids, float* weights,
                 sb_stream_t stream);
/* Scores s = sigmoid(logits); choice scores s + correction (float32 [experts], or null); the experts
 * lie in n_groups equal groups of neighbours, a group's score is the sum of its group_top largest
 * choice scores, and only experts of the keep_groups best groups can be chosen; the `top` largest
 * choice scores win (the lower index on a tie); weights s * scale, over the chosen ones' sum of s
 * first when `renormalize`. */
int sb_moe_route_scored(const float* logits, const float* correction, int n_rows, int n_experts, int top,
                        int n_groups, int keep_groups, int group_top, float scale, int renormalize,
                        int32_t* ids, float* weights, sb_stream_t stream);
/* Pairs of a tile of one expert (32, 64 or 128) that group, up and down of one step share. */
int sb_moe_tile_rows(int dtype, int n_pairs, int n_experts, int ff, int width);
int sb_moe_max_tiles(int n_pairs, int n_experts, int tile_rows);
int sb_moe_group(const int32_t* ids, int n_pairs, int n_experts, int tile_rows, int32_t* order, int32_t* meta,
                 sb_stream_t stream);
int sb_moe_up(const void* a, int a_dtype, const void* w, int w_dtype, const int32_t* order,
              const int32_t* meta, int n_pairs, int n_experts, int tile_rows, int top, int ff, int width,
              float limit, float slope, void* act, sb_stream_t stream);
int sb_moe_down(const void* act, int a_dtype, const void* w, int w_dtype, const int32_t* order,
                const int32_t* meta, int n_pairs, int n_experts, int tile_rows, int top, int width, int ff,
                float* pair_out, sb_stream_t stream);
int sb_moe_combine(float* x, const float* pair_out, const float* weights, int n_rows, int top, int width,
                   sb_stream_t stream);

int sb_sample_params_size(void);
int sb_sample(float* logits, int n_rows, int vocab, const void* params, const int32_t* history,
              int history_stride, const int32_t* fed_pos, int32_t* out_tokens, sb_stream_t stream);
int sb_add_i32(int32_t* x, int n, int delta, sb_stream_t stream);
/* x[i] = min(x[i] + 1, last[i]) */
int sb_advance_rows(int32_t* x, const int32_t* last, int n, sb_stream_t stream);
/* out[e] = mean + std * z_e, z standard normal, a function of (key0, key1, e) only. */
int sb_random_normal(void* out, int out_dtype, size_t n, uint32_t key0, uint32_t key1, float mean,
                     float std, sb_stream_t stream);

/* ------------------------------------------------------------------ attention library */
int sb_attention_head_dim(void);
void sb_attention_force_mma(int mode);    /* 0 by size; 1 the mma.sync kernels; 2 the TMA decode kernel always */
int sb_attention_status(void);            /* as sb_tc5_status; -1: no tensor-memory kernel */
int sb_attention_last_launches(void);     /* kernels the last sb_attention call launched */
size_t sb_attention_scratch_bytes(int n_rows, int n_q_heads, int n_kv_heads, int max_new,
                                  int max_len);
/* Causal grouped-query attention of a step's rows over one cache entry's pages (bfloat16).
 * sink: as in sb_attention_plain. */
int sb_attention(const void* q, void* out, int n_rows, int n_seqs, int max_new,
                 const int32_t* seq_row0, const int32_t* seq_pos0, const int32_t* page_off,
                 const int32_t* page_ids, int page_size, const void* cache, int n_q_heads,
                 int n_kv_heads, int hd, int window, float scale, void* scratch,
                 size_t scratch_bytes, int* counters, int n_counters, int max_len, int n_pages,
                 int n_sms, const void* warm, size_t warm_bytes, const float* sink, float softcap,
                 sb_stream_t stream);

#ifdef __cplusplus
}
#endif

#include "no_alloc.h"        /* sb_attention_decode_static (attention library) */

#endif /* SONICBOOM_B200_H */
