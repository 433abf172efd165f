// Row kernels that look at a row's neighbours in its own sequence, and the layer norm:
//
//   sb_embed_pair:      embedding row plus a row of a second table chosen by a hash of the
//                       previous and the current token (the previous token of a step's first
//                       row comes from per-slot state)
//   sb_keep_last_token: a step's last token of every sequence into that state
//   sb_layernorm:       (x - mean) / sqrt(var + eps) * w, no bias
//   sb_causal_conv:     a short causal convolution over time on every channel, reading the
//                       taps before a step's first row from per-slot state
//   sb_conv_state:      a step's last taps - 1 inputs of every sequence into that state
//
// All arithmetic is float32; sums over a row are fixed trees.
#include <math.h>

#include "common.cuh"

namespace {

template <int NT>
__device__ __forceinline__ float block_sum(float s, float* red) {
  s = sb_warp_sum(s);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int i = 0; i < NT / 32; ++i) total += red[i];
    red[NT / 32] = total;
  }
  __syncthreads();
  return red[NT / 32];
}

template <typename T>
__global__ void embed_pair_kernel(const int32_t* tokens, const int32_t* row_seq, const int32_t* row_pos,
                                  const int32_t* seq_row0, const int32_t* seq_slot, const int32_t* prev_token,
                                  const T* __restrict__ table, int vocab, const T* __restrict__ pair, int buckets,
                                  int mul_prev, int mul_cur, int width, float scale, float* out) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int r = blockIdx.x;
  const int tok = tokens[r];
  float* o = out + (size_t)r * width;
  if (tok < 0 || tok >= vocab) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = NAN;
    return;
  }
  const int s = row_seq[r];
  long long idx = buckets;                       // a sequence's first token: the table's last row
  if (row_pos[r] > 0) {
    const int prev = r > seq_row0[s] ? tokens[r - 1] : prev_token[seq_slot[s]];
    idx = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (idx < 0) idx += buckets;
  }
  const T* a = table + (size_t)tok * width;
  const T* b = pair + (size_t)idx * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = sb_to_f32<T>(a[i]) * scale + sb_to_f32<T>(b[i]);
}

__global__ void keep_last_token_kernel(const int32_t* tokens, const int32_t* seq_row0, const int32_t* seq_slot,
                                       int n_seqs, int32_t* prev_token) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < n_seqs) prev_token[seq_slot[s]] = tokens[seq_row0[s + 1] - 1];
}

template <int NT, typename TW, typename TO>
__global__ void __launch_bounds__(NT)
layernorm_kernel(const float* x, const int32_t* rows, int width, const TW* __restrict__ w, float eps, TO* out) {
  __shared__ float red[NT / 32 + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* xr = x + r * width;
  float s = 0.0f;
  for (int i = threadIdx.x; i < width; i += NT) s += xr[i];
  const float mean = block_sum<NT>(s, red) / (float)width;
  float q = 0.0f;
  for (int i = threadIdx.x; i < width; i += NT) {
    const float d = xr[i] - mean;
    q = fmaf(d, d, q);
  }
  const float inv = 1.0f / sqrtf(block_sum<NT>(q, red) / (float)width + eps);
  TO* o = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += NT)
    o[i] = sb_from_f32<TO>(((xr[i] - mean) * inv) * sb_to_f32<TW>(w[i]));
}

// y_t = [x_t +] [bias +] sum_j w[c, j] x_(t - taps + 1 + j), optionally through silu.  A tap before
// the step's first row of the sequence is read from state[slot, taps - 1, channels] (the inputs at
// the taps - 1 positions before the step), one before the sequence's start is zero.  OWN: every
// sequence brings exactly one row, and the thread that computes a channel also shifts its state.
template <typename TW, typename TO, bool OWN>
__global__ void causal_conv_kernel(const float* x, int ld, int x_off, int channels, int taps,
                                   const TW* __restrict__ w, const TW* __restrict__ bias, int act, int add_input,
                                   const int32_t* row_seq, const int32_t* row_pos, const int32_t* seq_row0,
                                   const int32_t* seq_pos0, const int32_t* seq_slot, float* state, TO* out,
                                   int ld_out, int out_off) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = row_seq[r], pos = row_pos[r];
  const int pos0 = OWN ? pos : seq_pos0[s], r0 = OWN ? r : seq_row0[s];
  float* st = state ? state + (size_t)seq_slot[s] * (taps - 1) * channels + c : nullptr;
  const float cur = x[(size_t)r * ld + x_off + c];
  float acc = bias ? sb_to_f32<TW>(bias[c]) : 0.0f;
  for (int j = 0; j < taps; ++j) {
    const int p = pos - (taps - 1) + j;
    float v = 0.0f;
    if (p >= pos0) v = x[(size_t)(r0 + (p - pos0)) * ld + x_off + c];
    else if (p >= 0) v = st[(size_t)(p - pos0 + taps - 1) * channels];
    acc = fmaf(sb_to_f32<TW>(w[(size_t)c * taps + j]), v, acc);
  }
  if (add_input) acc += cur;
  if (act) acc = sb_silu(acc);
  out[(size_t)r * ld_out + out_off + c] = sb_from_f32<TO>(acc);
  if (OWN) {
    for (int i = 0; i + 1 < taps - 1; ++i) st[(size_t)i * channels] = st[(size_t)(i + 1) * channels];
    if (taps > 1) st[(size_t)(taps - 2) * channels] = cur;
  }
}

// The same sums for a step with several rows a sequence and at most CONV_MAXT taps: a thread walks
// CONV_RUN consecutive rows of its channel and keeps the last taps - 1 inputs in registers, so a row
// is read once instead of once per tap.  Every sum has the order of the kernel above.
constexpr int CONV_MAXT = 8, CONV_RUN = 8;
template <typename TW, typename TO>
__global__ void causal_conv_run_kernel(const float* x, int n_rows, int ld, int x_off, int channels, int taps,
                                       const TW* __restrict__ w, const TW* __restrict__ bias, int act, int add_input,
                                       const int32_t* row_seq, const int32_t* row_pos, const int32_t* seq_pos0,
                                       const int32_t* seq_slot, const float* state, TO* out, int ld_out, int out_off) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int r_begin = blockIdx.x * CONV_RUN, r_end = min(n_rows, r_begin + CONV_RUN);
  float wd[CONV_MAXT], hist[CONV_MAXT];     // by distance d: the weight of x_(t - d); hist[d] = x of the row d before
#pragma unroll
  for (int d = 0; d < CONV_MAXT; ++d) {
    wd[d] = d < taps ? sb_to_f32<TW>(w[(size_t)c * taps + (taps - 1 - d)]) : 0.0f;
    hist[d] = (d >= 1 && d < taps && r_begin - d >= 0) ? x[(size_t)(r_begin - d) * ld + x_off + c] : 0.0f;
  }
  const float b = bias ? sb_to_f32<TW>(bias[c]) : 0.0f;
  for (int r = r_begin; r < r_end; ++r) {
    const int s = row_seq[r], pos = row_pos[r], pos0 = seq_pos0[s];
    const float* st = state ? state + (size_t)seq_slot[s] * (taps - 1) * channels + c : nullptr;
    const float cur = x[(size_t)r * ld + x_off + c];
    hist[0] = cur;
    float acc = b;
#pragma unroll
    for (int d = CONV_MAXT - 1; d >= 0; --d) {
      if (d < taps) {
        const int p = pos - d;
        float v = 0.0f;
        if (p >= pos0) v = hist[d];
        else if (p >= 0) v = st[(size_t)(p - pos0 + taps - 1) * channels];
        acc = fmaf(wd[d], v, acc);
      }
    }
    if (add_input) acc += cur;
    if (act) acc = sb_silu(acc);
    out[(size_t)r * ld_out + out_off + c] = sb_from_f32<TO>(acc);
#pragma unroll
    for (int d = CONV_MAXT - 1; d >= 1; --d) hist[d] = hist[d - 1];
  }
}

__global__ void conv_state_kernel(const float* x, int ld, int x_off, int channels, int taps,
                                  const int32_t* seq_row0, const int32_t* seq_slot, float* state) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int r0 = seq_row0[s], n = seq_row0[s + 1] - r0;
  float* st = state + (size_t)seq_slot[s] * (taps - 1) * channels + c;
  for (int i = 0; i < taps - 1; ++i) {
    const int rel = n - (taps - 1) + i;              // the position kept at i, counted from the step's first
    st[(size_t)i * channels] = rel >= 0 ? x[(size_t)(r0 + rel) * ld + x_off + c]
                                        : st[(size_t)(i + n) * channels];      // i + n > i: not yet overwritten
  }
}

}  // namespace

extern "C" int sb_embed_pair(const int32_t* tokens, int n_rows, const int32_t* row_seq, const int32_t* row_pos,
                             const int32_t* seq_row0, const int32_t* seq_slot, const int32_t* prev_token,
                             const void* table, int table_dtype, int vocab, const void* pair, int buckets,
                             int mul_prev, int mul_cur, int width, float scale, float* out, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || vocab <= 0 || buckets <= 0 || !tokens || !table || !pair || !out || !prev_token)
    SB_FAIL(SB_ERR_ARG, "sb_embed_pair: rows=%d width=%d vocab=%d buckets=%d", n_rows, width, vocab, buckets);
  if (!sb_valid_dtype(table_dtype)) SB_FAIL(SB_ERR_ARG, "sb_embed_pair: dtype code %d", table_dtype);
  SB_DISPATCH_DTYPE(table_dtype, T, {
    sb_launch<SB_K_ELEMENTWISE>(embed_pair_kernel<T>, dim3(n_rows), dim3(width >= 1024 ? 256 : 128), 0, stream, tokens,
                                row_seq, row_pos, seq_row0, seq_slot, prev_token, (const T*)table, vocab,
                                (const T*)pair, buckets, mul_prev, mul_cur, width, scale, out);
  });
  SB_CHECK_LAUNCH("sb_embed_pair");
  return SB_OK;
}

extern "C" int sb_keep_last_token(const int32_t* tokens, const int32_t* seq_row0, const int32_t* seq_slot,
                                  int n_seqs, int32_t* prev_token, cudaStream_t stream) {
  if (n_seqs <= 0 || !tokens || !seq_row0 || !seq_slot || !prev_token)
    SB_FAIL(SB_ERR_ARG, "sb_keep_last_token: seqs=%d", n_seqs);
  sb_launch<SB_K_ELEMENTWISE>(keep_last_token_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, tokens, seq_row0,
                              seq_slot, n_seqs, prev_token);
  SB_CHECK_LAUNCH("sb_keep_last_token");
  return SB_OK;
}

extern "C" int sb_layernorm(const float* x, const int32_t* rows, int n_rows, int width, const void* weight,
                            int weight_dtype, float eps, void* out, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || !x || !weight || !out) SB_FAIL(SB_ERR_ARG, "sb_layernorm: rows=%d width=%d", n_rows, width);
  if (!sb_valid_dtype(weight_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_layernorm: dtype codes %d %d", weight_dtype, out_dtype);
  SB_DISPATCH_DTYPE(weight_dtype, TW, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      if (n_rows >= 512 || width <= 1024)
        sb_launch<SB_K_ELEMENTWISE>(layernorm_kernel<256, TW, TO>, dim3(n_rows), dim3(256), 0, stream, x, rows, width,
                                    (const TW*)weight, eps, (TO*)out);
      else
        sb_launch<SB_K_ELEMENTWISE>(layernorm_kernel<1024, TW, TO>, dim3(n_rows), dim3(1024), 0, stream, x, rows, width,
                                    (const TW*)weight, eps, (TO*)out);
    });
  });
  SB_CHECK_LAUNCH("sb_layernorm");
  return SB_OK;
}

extern "C" int sb_causal_conv(const float* x, int n_rows, int ld, int x_off, int channels, int taps, const void* w,
                              const void* bias, int w_dtype, int act, int add_input, int n_seqs,
                              const int32_t* row_seq, const int32_t* row_pos, const int32_t* seq_row0,
                              const int32_t* seq_pos0, const int32_t* seq_slot, float* state, void* out,
                              int out_dtype, int ld_out, int out_off, cudaStream_t stream) {
  if (n_rows <= 0 || channels <= 0 || taps <= 0 || n_seqs <= 0 || !x || !w || !out || (taps > 1 && !state))
    SB_FAIL(SB_ERR_ARG, "sb_causal_conv: rows=%d channels=%d taps=%d seqs=%d", n_rows, channels, taps, n_seqs);
  if (x_off < 0 || x_off + channels > ld || out_off < 0 || out_off + channels > ld_out)
    SB_FAIL(SB_ERR_ARG, "sb_causal_conv: %d channels at %d of %d, out at %d of %d", channels, x_off, ld, out_off, ld_out);
  if (!sb_valid_dtype(w_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_causal_conv: dtype codes %d %d", w_dtype, out_dtype);
  if ((const void*)x == (const void*)out) SB_FAIL(SB_ERR_ARG, "sb_causal_conv: in place");
  const int nt = channels >= 256 ? 256 : 128;
  const dim3 grid(n_rows, (channels + nt - 1) / nt);
  const bool own = n_rows == n_seqs;        // one row a sequence: the row's threads shift the state themselves
  SB_DISPATCH_DTYPE(w_dtype, TW, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      if (!own && taps <= CONV_MAXT)
        sb_launch<SB_K_ELEMENTWISE>(causal_conv_run_kernel<TW, TO>, dim3((n_rows + CONV_RUN - 1) / CONV_RUN, grid.y), dim3(nt),
                                    0, stream, x, n_rows, ld, x_off, channels, taps, (const TW*)w, (const TW*)bias, act,
                                    add_input, row_seq, row_pos, seq_pos0, seq_slot, (const float*)state, (TO*)out, ld_out,
                                    out_off);
      else if (own)
        sb_launch<SB_K_ELEMENTWISE>(causal_conv_kernel<TW, TO, true>, grid, dim3(nt), 0, stream, x, ld, x_off, channels,
                                    taps, (const TW*)w, (const TW*)bias, act, add_input, row_seq, row_pos, seq_row0,
                                    seq_pos0, seq_slot, state, (TO*)out, ld_out, out_off);
      else
        sb_launch<SB_K_ELEMENTWISE>(causal_conv_kernel<TW, TO, false>, grid, dim3(nt), 0, stream, x, ld, x_off, channels,
                                    taps, (const TW*)w, (const TW*)bias, act, add_input, row_seq, row_pos, seq_row0,
                                    seq_pos0, seq_slot, state, (TO*)out, ld_out, out_off);
    });
  });
  SB_CHECK_LAUNCH("sb_causal_conv");
  if (!own && taps > 1) {
    sb_launch<SB_K_ELEMENTWISE>(conv_state_kernel, dim3(n_seqs, (channels + nt - 1) / nt), dim3(nt), 0, stream, x, ld,
                                x_off, channels, taps, seq_row0, seq_slot, state);
    SB_CHECK_LAUNCH("sb_causal_conv (state)");
  }
  return SB_OK;
}
