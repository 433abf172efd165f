// Attention whose weights are not normalised over the keys: the weight of a visible key is
// sigmoid(cap(q . k * scale) + bias_h), cap(s) = softcap * tanh(s / softcap) (softcap 0: none), a
// number per query head added to the score, and out = sum_j weight_j v_j.  Visible for the query
// at absolute position i: key j <= i with i - j < window (window 0: every earlier key) or
// j < keep_first, the first tokens of a sequence that a window keeps.
//
// The plain kernel: one block per (row, query head), float32 arithmetic, keys in ascending order
// in chunks at absolute positions, so a sum depends on the positions only, not on the batch or on
// where the pages lie.  It reads the same paged cache as the softmax kernels.
#include <math.h>

#include "common.cuh"

int sb_check_attention_args(const char* who, int n_rows, int n_q_heads, int n_kv_heads, int hd,
                            int window, int page_size);

namespace {

constexpr int CHUNK = 128;
constexpr int THREADS = 128;
constexpr int MAX_HD = 1024;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(THREADS)
attn_sigmoid_kernel(const TQ* q, TQ* out, const int32_t* row_seq, const int32_t* row_pos,
                    const int32_t* page_off, const int32_t* page_ids, int page_size, const TC* cache,
                    int n_q_heads, int n_kv_heads, int hd, int window, int keep_first, float scale,
                    float softcap, const float* __restrict__ head_bias) {
  __shared__ float qs[MAX_HD];
  __shared__ float wts[CHUNK];
  sb_pdl_launch();
  sb_pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = h / (n_q_heads / n_kv_heads);
  const int pos = row_pos[t];
  const int seq = row_seq[t];
  const int32_t* pages = page_ids + page_off[seq];
  if (pos < 0 || pos / page_size >= page_off[seq + 1] - page_off[seq]) {
    for (int d = tid; d < hd; d += THREADS) out[((size_t)t * n_q_heads + h) * hd + d] = sb_from_f32<TQ>(0.0f);
    return;
  }
  for (int d = tid; d < hd; d += THREADS) qs[d] = sb_to_f32<TQ>(q[((size_t)t * n_q_heads + h) * hd + d]);
  __syncthreads();
  const float pb = head_bias ? head_bias[h] : 0.0f;
  const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;        // the window's first key
  const int kept = min(keep_first, lo);                             // keys [0, kept) are seen besides
  float acc[MAX_HD / THREADS] = {};
  // two stretches of keys, both in ascending order: the kept first tokens, then the window
  for (int part = 0; part < 2; ++part) {
    const int from = part == 0 ? 0 : lo, to = part == 0 ? kept : pos + 1;
    for (int cs = (from / CHUNK) * CHUNK; cs < to; cs += CHUNK) {
      const int j0 = max(cs, from), j1 = min(cs + CHUNK, to);
      for (int j = j0 + warp; j < j1; j += THREADS / 32) {
        const TC* krow = cache + ((((size_t)pages[j / page_size] * 2) * n_kv_heads + kvh) * page_size + j % page_size) * hd;
        float dot = 0.0f;
        for (int d = lane; d < hd; d += 32) dot = fmaf(qs[d], sb_to_f32<TC>(krow[d]), dot);
        float s = sb_warp_sum(dot) * scale;
        if (softcap > 0.0f) s = softcap * tanhf(s * inv_cap);
        if (lane == 0) wts[j - cs] = 1.0f / (1.0f + expf(-(s + pb)));
      }
      __syncthreads();
      for (int j = j0; j < j1; ++j) {
        const float p = wts[j - cs];
        const TC* vrow = cache + ((((size_t)pages[j / page_size] * 2 + 1) * n_kv_heads + kvh) * page_size + j % page_size) * hd;
#pragma unroll
        for (int i = 0; i < MAX_HD / THREADS; ++i) {
          const int d = tid + i * THREADS;
          if (d < hd) acc[i] = fmaf(p, sb_to_f32<TC>(vrow[d]), acc[i]);
        }
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_HD / THREADS; ++i) {
    const int d = tid + i * THREADS;
    if (d < hd) out[((size_t)t * n_q_heads + h) * hd + d] = sb_from_f32<TQ>(acc[i]);
  }
}

}  // namespace

extern "C" int sb_attention_sigmoid(const void* q, void* out, int act_dtype, int n_rows, const int32_t* row_seq,
                                    const int32_t* row_pos, const int32_t* page_off, const int32_t* page_ids,
                                    int page_size, const void* cache, int cache_dtype, int n_q_heads,
                                    int n_kv_heads, int hd, int window, int keep_first, float scale, float softcap,
                                    const float* head_bias, cudaStream_t stream) {
  if (int rc = sb_check_attention_args("sb_attention_sigmoid", n_rows, n_q_heads, n_kv_heads, hd, window, page_size))
    return rc;
  if (keep_first < 0 || softcap < 0.0f) SB_FAIL(SB_ERR_ARG, "sb_attention_sigmoid: keep_first=%d softcap=%g", keep_first, softcap);
  if (hd > MAX_HD) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention_sigmoid: head dim %d is above %d", hd, MAX_HD);
  if (!sb_valid_dtype(act_dtype) || !sb_valid_dtype(cache_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_attention_sigmoid: dtype codes %d %d", act_dtype, cache_dtype);
  if (n_q_heads > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention_sigmoid: %d heads", n_q_heads);
  const dim3 grid(n_rows, n_q_heads);
  SB_DISPATCH_DTYPE(act_dtype, TQ, {
    SB_DISPATCH_DTYPE(cache_dtype, TC, {
      sb_launch(attn_sigmoid_kernel<TQ, TC>, grid, dim3(THREADS), 0, stream, (const TQ*)q, (TQ*)out, row_seq, row_pos,
                page_off, page_ids, page_size, (const TC*)cache, n_q_heads, n_kv_heads, hd, window, keep_first, scale,
                softcap, head_bias);
    });
  });
  SB_CHECK_LAUNCH("sb_attention_sigmoid");
  return SB_OK;
}
