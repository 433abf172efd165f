// Row kernels around attention and linear-recurrence mixers whose projections need more than
// a half-split rotation, and two kernels of the residual stream and the feed-forward.
//
//   sb_stream_add:     out[r] = x[r] + add[r] + vec            (a vector joins every row)
//   sb_polynorm:       out[r] = a N(z) + b N(z^2) + c N(z^3) + e, N(u) = u / sqrt(mean(u^2) + eps)
//   sb_attn_prep:      projection rows -> queries and cache rows: optional RMS norm over the whole
//                      q (k) projection, rotation of a prefix of every head in pairs (i, i + n/2) or
//                      (2i, 2i + 1), values that are the raw key projection, values rotated by their
//                      own position, heads padded with zeros to the cache's head size
//   sb_attn_unrotate:  attention results turned back by the query's position, padding dropped
//   sb_linrec_prep:    rotation and scaling of a recurrence's q and k in place; decay logits to
//                      decays exp(logsigmoid(z) / tau) in place
//   sb_linrec_out:     RMS norm of every head's recurrence output, optional weight, gate silu(g)
//
// All arithmetic is float32; angles are float(position) * table entry with the accurate
// sincosf; the rotation itself is sb_rot_lo / sb_rot_hi as everywhere.  Sums are fixed trees.
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

// ------------------------------------------------------------------------------ stream add
template <int NT, typename TV, typename TN, typename TO>
__global__ void __launch_bounds__(NT)
stream_add_kernel(const float* x, const float* add, const TV* __restrict__ vec, int width, float* out,
                  const TN* __restrict__ next_w, float next_eps, TO* normed) {
  __shared__ float red[NT / 32 + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < width; i += NT) {
    float v = x[r * width + i];
    if (add) v += add[r * width + i];
    if (vec) v += sb_to_f32<TV>(vec[i]);
    out[r * width + i] = v;
    sq = fmaf(v, v, sq);
  }
  if (!normed) return;
  const float inv = 1.0f / sqrtf(block_sum<NT>(sq, red) / (float)width + next_eps);
  for (int i = threadIdx.x; i < width; i += NT)
    normed[r * width + i] = sb_from_f32<TO>((out[r * width + i] * inv) * sb_to_f32<TN>(next_w[i]));
}

// -------------------------------------------------------------------------------- polynorm
template <int NT, typename TC, typename TO>
__global__ void __launch_bounds__(NT)
polynorm_kernel(const float* z, int ff, const TC* __restrict__ coef, float eps, TO* out) {
  __shared__ float red[NT / 32 + 1];
  sb_pdl_launch();
  const float a = sb_to_f32<TC>(coef[0]), b = sb_to_f32<TC>(coef[1]), c = sb_to_f32<TC>(coef[2]),
              e = sb_to_f32<TC>(coef[3]);
  sb_pdl_wait();
  const float* zr = z + (size_t)blockIdx.x * ff;
  float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
  for (int i = threadIdx.x; i < ff; i += NT) {
    const float u = zr[i], u2 = u * u, u3 = u2 * u;
    s2 += u2;
    s4 = fmaf(u2, u2, s4);
    s6 = fmaf(u3, u3, s6);
  }
  const float n = (float)ff;
  const float i1 = 1.0f / sqrtf(block_sum<NT>(s2, red) / n + eps);
  const float i2 = 1.0f / sqrtf(block_sum<NT>(s4, red) / n + eps);
  const float i3 = 1.0f / sqrtf(block_sum<NT>(s6, red) / n + eps);
  const float ka = a * i1, kb = b * i2, kc = c * i3;
  TO* o = out + (size_t)blockIdx.x * ff;
  for (int i = threadIdx.x; i < ff; i += NT) {
    const float u = zr[i], u2 = u * u;
    o[i] = sb_from_f32<TO>(ka * u + kb * u2 + kc * (u2 * u) + e);
  }
}

// ------------------------------------------------------------------------------- rotations
// Element c of a head whose first `rot` values turn: its pair number and whether it is the
// pair's first member; `other` is the partner's index.
__device__ __forceinline__ void pair_of(int c, int rot, int interleaved, int& i, bool& first, int& other) {
  if (interleaved) {
    i = c >> 1;
    first = !(c & 1);
    other = c ^ 1;
  } else {
    const int half = rot >> 1;
    first = c < half;
    i = first ? c : c - half;
    other = first ? c + half : c - half;
  }
}

__device__ __forceinline__ int page_of(const int32_t* page_off, const int32_t* page_ids, int seq, int pos,
                                       int page_size) {
  const int first = page_off[seq], n = page_off[seq + 1] - first;
  const int i = pos / page_size;
  return (pos >= 0 && i < n) ? page_ids[first + i] : -1;
}

struct PrepArgs {
  const float* proj;
  int ld, q_off, k_off, v_off;         // v_off < 0: the values are the key projection as it is
  int n_q_heads, n_kv_heads, dim, vdim, hd;
  int rot, interleaved;
  const float* inv_freq;               // [rot / 2]
  const float* v_inv_freq;             // [vdim / 2], or null: values are not rotated
  const void* q_norm;                  // [n_q_heads * dim] or null ([dim] with head_norm 1)
  const void* k_norm;                  // [n_kv_heads * dim] or null ([dim] with head_norm 1)
  int head_norm;                       // 0: the norm, if any, is over the whole projection; 1: every head by itself
                                       // before the rotation, one weight [dim] for all heads; 2: every head by
                                       // itself after the rotation, no weight
  float rot_scale;                     // multiplies every cosine and sine (1: a pure rotation)
  float eps;
  const int32_t* row_seq;
  const int32_t* row_pos;
  const int32_t* page_off;
  const int32_t* page_ids;
  int page_size, has_kv;
  void* cache;
  void* q_out;
};

// Rotates the first `rot` values of `heads` vectors of `n_in` values each (read through `get(head,
// c)`) by the angles fpos * inv_freq[i] and hands every finished value to `put(head, c, value)`;
// values from `rot` on pass as they are, and values from n_in up to n_out are zeros.  A thread keeps
// to one pair and walks over the heads, so the pair's sine and cosine are worked out once.
template <int NT, typename Get, typename Put>
__device__ __forceinline__ void turn_heads(int heads, int n_in, int n_out, int rot, int interleaved,
                                           const float* __restrict__ inv_freq, float fpos, Get get, Put put,
                                           float rot_scale = 1.0f) {
  const int n_pairs = rot >> 1;
  if (n_pairs > 0) {
    const int groups = NT / n_pairs > 0 ? NT / n_pairs : 1;      // thread groups that take heads in turn
    const int i = threadIdx.x % n_pairs, first_head = threadIdx.x / n_pairs;
    if (n_pairs <= NT) {
      if (first_head < groups) {
        float sn, cs;
        sincosf(fpos * inv_freq[i], &sn, &cs);
        sn *= rot_scale;
        cs *= rot_scale;
        const int lo = interleaved ? 2 * i : i, hi = interleaved ? 2 * i + 1 : i + n_pairs;
        for (int h = first_head; h < heads; h += groups) {
          const float a = get(h, lo), b = get(h, hi);
          put(h, lo, sb_rot_lo(a, b, cs, sn));
          put(h, hi, sb_rot_hi(a, b, cs, sn));
        }
      }
    } else {
      for (int j = threadIdx.x; j < n_pairs; j += NT) {          // more pairs than threads
        float sn, cs;
        sincosf(fpos * inv_freq[j], &sn, &cs);
        sn *= rot_scale;
        cs *= rot_scale;
        const int lo = interleaved ? 2 * j : j, hi = interleaved ? 2 * j + 1 : j + n_pairs;
        for (int h = 0; h < heads; ++h) {
          const float a = get(h, lo), b = get(h, hi);
          put(h, lo, sb_rot_lo(a, b, cs, sn));
          put(h, hi, sb_rot_hi(a, b, cs, sn));
        }
      }
    }
  }
  const int rest = n_out - rot;
  for (int e = threadIdx.x; e < heads * rest; e += NT) {
    const int h = e / rest, c = rot + e % rest;
    put(h, c, c < n_in ? get(h, c) : 0.0f);
  }
}

// blockIdx.y: 0 queries, 1 keys, 2 values.
template <int NT, typename TW, typename TQ, typename TC>
__global__ void __launch_bounds__(NT) attn_prep_kernel(const PrepArgs p) {
  __shared__ float red[NT / 32 + 1];
  sb_pdl_launch();
  const int t = blockIdx.x, what = blockIdx.y;
  const int pos = p.row_pos[t];
  const float fpos = (float)pos;
  int page = 0;
  if (what > 0) {
    page = page_of(p.page_off, p.page_ids, p.row_seq[t], pos, p.page_size);
    if (page < 0) return;              // no page of its own there: nothing is written
  }
  sb_pdl_wait();
  const float* row = p.proj + (size_t)t * p.ld;
  if (what == 2) {
    // values: the v section, or the raw key projection; rotated over all vdim when a table is given
    const float* src = row + (p.v_off >= 0 ? p.v_off : p.k_off);
    TC* dst = reinterpret_cast<TC*>(p.cache) +
              ((((size_t)page * 2 + 1) * p.n_kv_heads) * p.page_size + pos % p.page_size) * p.hd;
    const size_t head_step = (size_t)p.page_size * p.hd;
    const int vdim = p.vdim;
    turn_heads<NT>(p.n_kv_heads, vdim, p.hd, p.v_inv_freq ? vdim : 0, p.interleaved, p.v_inv_freq, fpos,
                   [&](int h, int c) { return src[h * vdim + c]; },
                   [&](int h, int c, float v) { dst[h * head_step + c] = sb_from_f32<TC>(v); });
    return;
  }
  const int heads = what == 0 ? p.n_q_heads : p.n_kv_heads;
  const float* src = row + (what == 0 ? p.q_off : p.k_off);
  const TW* nw = reinterpret_cast<const TW*>(what == 0 ? p.q_norm : p.k_norm);
  const int dim = p.dim;
  if (p.head_norm) {
    // Every head is normed by itself: before the rotation with one weight for all heads (1), or
    // after it without a weight (2).  The turned heads wait in shared memory ([heads, dim], then
    // one inverse root mean square per head) until the head's sum is known; a warp sums a head.
    extern __shared__ float staged[];
    float* hinv = staged + heads * dim;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (p.head_norm == 1) {
      for (int h = warp; h < heads; h += NT / 32) {
        float s = 0.0f;
        for (int c = lane; c < dim; c += 32) s = fmaf(src[h * dim + c], src[h * dim + c], s);
        s = sb_warp_sum(s);
        if (lane == 0) hinv[h] = 1.0f / sqrtf(s / (float)dim + p.eps);
      }
      __syncthreads();
    }
    const bool pre = p.head_norm == 1;
    turn_heads<NT>(heads, dim, dim, p.rot, p.interleaved, p.inv_freq, fpos,
                   [&](int h, int c) {
                     const float v = src[h * dim + c];
                     return pre ? (v * hinv[h]) * sb_to_f32<TW>(nw[c]) : v;
                   },
                   [&](int h, int c, float v) { staged[h * dim + c] = v; }, p.rot_scale);
    __syncthreads();
    if (!pre) {
      for (int h = warp; h < heads; h += NT / 32) {
        float s = 0.0f;
        for (int c = lane; c < dim; c += 32) s = fmaf(staged[h * dim + c], staged[h * dim + c], s);
        s = sb_warp_sum(s);
        if (lane == 0) hinv[h] = 1.0f / sqrtf(s / (float)dim + p.eps);
      }
      __syncthreads();
    }
    const int hd = p.hd;
    if (what == 0) {
      TQ* dst = reinterpret_cast<TQ*>(p.q_out) + (size_t)t * p.n_q_heads * hd;
      for (int e = threadIdx.x; e < heads * hd; e += NT) {
        const int h = e / hd, c = e % hd;
        dst[e] = sb_from_f32<TQ>(c < dim ? (pre ? staged[h * dim + c] : staged[h * dim + c] * hinv[h]) : 0.0f);
      }
    } else {
      TC* dst = reinterpret_cast<TC*>(p.cache) +
                ((((size_t)page * 2) * p.n_kv_heads) * p.page_size + pos % p.page_size) * hd;
      const size_t head_step = (size_t)p.page_size * hd;
      for (int e = threadIdx.x; e < heads * hd; e += NT) {
        const int h = e / hd, c = e % hd;
        dst[h * head_step + c] =
            sb_from_f32<TC>(c < dim ? (pre ? staged[h * dim + c] : staged[h * dim + c] * hinv[h]) : 0.0f);
      }
    }
    return;
  }
  float inv = 1.0f;
  if (nw) {
    float s = 0.0f;
    for (int e = threadIdx.x; e < heads * dim; e += NT) s = fmaf(src[e], src[e], s);
    inv = 1.0f / sqrtf(block_sum<NT>(s, red) / (float)(heads * dim) + p.eps);
  }
  auto get = [&](int h, int c) {
    const float v = src[h * dim + c];
    return nw ? (v * inv) * sb_to_f32<TW>(nw[h * dim + c]) : v;
  };
  if (what == 0) {
    TQ* dst = reinterpret_cast<TQ*>(p.q_out) + (size_t)t * p.n_q_heads * p.hd;
    const int hd = p.hd;
    turn_heads<NT>(heads, dim, hd, p.rot, p.interleaved, p.inv_freq, fpos, get,
                   [&](int h, int c, float v) { dst[h * hd + c] = sb_from_f32<TQ>(v); }, p.rot_scale);
  } else {
    TC* dst = reinterpret_cast<TC*>(p.cache) +
              ((((size_t)page * 2) * p.n_kv_heads) * p.page_size + pos % p.page_size) * p.hd;
    const size_t head_step = (size_t)p.page_size * p.hd;
    turn_heads<NT>(heads, dim, p.hd, p.rot, p.interleaved, p.inv_freq, fpos, get,
                   [&](int h, int c, float v) { dst[h * head_step + c] = sb_from_f32<TC>(v); }, p.rot_scale);
  }
}

// One block per row: the first vdim values of every head, turned back by the row's position.
template <int NT, typename T>
__global__ void __launch_bounds__(NT)
attn_unrotate_kernel(const T* in, T* out, int n_heads, int hd, int vdim, int interleaved,
                     const float* __restrict__ v_inv_freq, const int32_t* row_pos, const float* gate, int gate_ld) {
  sb_pdl_launch();
  const size_t t = blockIdx.x;
  const float fpos = v_inv_freq ? -(float)row_pos[t] : 0.0f;
  sb_pdl_wait();
  const T* src = in + t * n_heads * hd;
  T* dst = out + t * n_heads * vdim;
  if constexpr (sizeof(T) == 2) {
    // neighbouring pairs of 16-bit values: a pair is one 4-byte access
    const int n_pairs = vdim >> 1;
    if (v_inv_freq && !gate && interleaved && !(hd & 1) && !(vdim & 1) && n_pairs <= NT) {
      const int groups = NT / n_pairs, i = threadIdx.x % n_pairs, first_head = threadIdx.x / n_pairs;
      if (first_head >= groups) return;
      float sn, cs;
      sincosf(fpos * v_inv_freq[i], &sn, &cs);
      const __nv_bfloat162* src2 = reinterpret_cast<const __nv_bfloat162*>(src);
      __nv_bfloat162* dst2 = reinterpret_cast<__nv_bfloat162*>(dst);
      for (int h = first_head; h < n_heads; h += groups) {
        const float2 ab = __bfloat1622float2(src2[h * (hd >> 1) + i]);
        dst2[h * n_pairs + i] = __floats2bfloat162_rn(sb_rot_lo(ab.x, ab.y, cs, sn), sb_rot_hi(ab.x, ab.y, cs, sn));
      }
      return;
    }
  }
  turn_heads<NT>(n_heads, vdim, vdim, v_inv_freq ? vdim : 0, interleaved, v_inv_freq, fpos,
                 [&](int h, int c) { return sb_to_f32<T>(src[h * hd + c]); },
                 [&](int h, int c, float v) {
                   // a gate: the head's result times the logistic function of the row's number for that head
                   if (gate) v = v / (1.0f + expf(-gate[t * gate_ld + h]));
                   dst[h * vdim + c] = sb_from_f32<T>(v);
                 });
}

// ---------------------------------------------------------------------- linear recurrence
// With `a2` the decay logits are worked out here: z[t, c] = bias[c] + sum_r a2[c, r] * proj[t, a1_off + r]
// (r ascending, float32), the second half of a low-rank map whose first half came with the projection.
template <typename TA>
__global__ void linrec_prep_kernel(float* proj, int ld, int q_off, int k_off, int n_heads, int dim,
                                   float q_scale, float k_scale, int rot, int interleaved,
                                   const float* __restrict__ inv_freq, const int32_t* row_pos, size_t n_rows,
                                   float* z, float inv_tau, const TA* __restrict__ a2, const TA* __restrict__ a2_bias,
                                   int rank, int a1_off) {
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t per_row = (size_t)n_heads * dim;
  const size_t n = n_rows * per_row;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t t = e / per_row;
    const int at = (int)(e % per_row), c = at % dim;
    if (z) {
      float u;
      if (a2) {
        const float* low = proj + t * ld + a1_off;
        const TA* w = a2 + (size_t)at * rank;
        u = sb_to_f32<TA>(a2_bias[at]);
        for (int r = 0; r < rank; ++r) u = fmaf(sb_to_f32<TA>(w[r]), low[r], u);
      } else {
        u = z[e];
      }
      const float ls = fminf(u, 0.0f) - log1pf(expf(-fabsf(u)));      // log sigmoid(u)
      z[e] = expf(ls * inv_tau);
    }
    float* q = proj + t * ld + q_off;
    float* k = proj + t * ld + k_off;
    if (c < rot) {
      int i, other;
      bool first;
      pair_of(c, rot, interleaved, i, first, other);
      if (!first) continue;                           // the pair's first member writes both
      const int bt = at - c + other;
      float s, co;
      sincosf((float)row_pos[t] * inv_freq[i], &s, &co);
      const float qa = q[at], qb = q[bt], ka = k[at], kb = k[bt];
      q[at] = sb_rot_lo(qa, qb, co, s) * q_scale;
      q[bt] = sb_rot_hi(qa, qb, co, s) * q_scale;
      k[at] = sb_rot_lo(ka, kb, co, s) * k_scale;
      k[bt] = sb_rot_hi(ka, kb, co, s) * k_scale;
    } else {
      q[at] *= q_scale;
      k[at] *= k_scale;
    }
  }
}

// One warp per (row, head).
template <typename TW, typename TO>
__global__ void linrec_out_kernel(const float* o, const float* proj, int ld, int g_off, size_t n_items,
                                  int n_heads, int vdim, const TW* __restrict__ norm_w, int w_per_head,
                                  int gate_sigmoid, float eps, TO* out) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const size_t t = item / n_heads;
  const int h = (int)(item % n_heads);
  const float* src = o + item * vdim;
  float s = 0.0f;
  for (int j = lane; j < vdim; j += 32) s = fmaf(src[j], src[j], s);
  const float inv = 1.0f / sqrtf(sb_warp_sum(s) / (float)vdim + eps);
  const float* g = proj + t * ld + g_off + (size_t)h * vdim;
  for (int j = lane; j < vdim; j += 32) {
    float v = src[j] * inv;
    if (norm_w) v *= sb_to_f32<TW>(norm_w[(w_per_head ? (size_t)h * vdim : 0) + j]);
    out[item * vdim + j] = sb_from_f32<TO>(gate_sigmoid ? v / (1.0f + expf(-g[j])) : v * sb_silu(g[j]));
  }
}

inline int grid_for(size_t n, int threads) {
  const size_t b = (n + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > 8192 ? 8192 : b));
}

}  // namespace

extern "C" int sb_stream_add(const float* x, const float* add, const void* vec, int vec_dtype, int n_rows,
                             int width, float* out, const void* next_w, int next_w_dtype, float next_eps,
                             void* normed, int normed_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || !x || !out) SB_FAIL(SB_ERR_ARG, "sb_stream_add: rows=%d width=%d", n_rows, width);
  if ((vec && !sb_valid_dtype(vec_dtype)) || (normed && (!next_w || !sb_valid_dtype(next_w_dtype) || !sb_valid_dtype(normed_dtype))))
    SB_FAIL(SB_ERR_ARG, "sb_stream_add: dtype codes %d %d %d", vec_dtype, next_w_dtype, normed_dtype);
  // few rows (decode): more threads a row, so that a row's loads are in flight together
  SB_DISPATCH_DTYPE(vec ? vec_dtype : SB_F32, TV, {
    SB_DISPATCH_DTYPE(normed ? next_w_dtype : SB_F32, TN, {
      SB_DISPATCH_DTYPE(normed ? normed_dtype : SB_F32, TO, {
        if (n_rows >= 512 || width <= 1024)
          sb_launch<SB_K_ELEMENTWISE>(stream_add_kernel<256, TV, TN, TO>, dim3(n_rows), dim3(256), 0, stream, x, add,
                                      (const TV*)vec, width, out, (const TN*)next_w, next_eps, (TO*)normed);
        else
          sb_launch<SB_K_ELEMENTWISE>(stream_add_kernel<1024, TV, TN, TO>, dim3(n_rows), dim3(1024), 0, stream, x, add,
                                      (const TV*)vec, width, out, (const TN*)next_w, next_eps, (TO*)normed);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_stream_add");
  return SB_OK;
}

extern "C" int sb_polynorm(const float* z, int n_rows, int ff, const void* coef, int coef_dtype, float eps,
                           void* out, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || ff <= 0 || !z || !coef || !out) SB_FAIL(SB_ERR_ARG, "sb_polynorm: rows=%d ff=%d", n_rows, ff);
  if (!sb_valid_dtype(coef_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_polynorm: dtype codes %d %d", coef_dtype, out_dtype);
  SB_DISPATCH_DTYPE(coef_dtype, TC, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      if (n_rows >= 512 || ff <= 1024)
        sb_launch<SB_K_ELEMENTWISE>(polynorm_kernel<256, TC, TO>, dim3(n_rows), dim3(256), 0, stream, z, ff,
                                    (const TC*)coef, eps, (TO*)out);
      else
        sb_launch<SB_K_ELEMENTWISE>(polynorm_kernel<1024, TC, TO>, dim3(n_rows), dim3(1024), 0, stream, z, ff,
                                    (const TC*)coef, eps, (TO*)out);
    });
  });
  SB_CHECK_LAUNCH("sb_polynorm");
  return SB_OK;
}

extern "C" int sb_attn_prep(const float* proj, int n_rows, int ld, int q_off, int k_off, int v_off,
                            int n_q_heads, int n_kv_heads, int dim, int vdim, int hd, int rot, int interleaved,
                            const float* inv_freq, const float* v_inv_freq, const void* q_norm,
                            const void* k_norm, int norm_dtype, int head_norm, float rot_scale, float eps,
                            const int32_t* row_seq, const int32_t* row_pos, const int32_t* page_off,
                            const int32_t* page_ids, int page_size, void* cache, int cache_dtype, void* q_out,
                            int q_dtype, int has_kv, cudaStream_t stream) {
  if (n_rows <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || dim <= 0 || vdim <= 0 || hd < dim || hd < vdim)
    SB_FAIL(SB_ERR_ARG, "sb_attn_prep: rows=%d heads=%d/%d dim=%d vdim=%d hd=%d", n_rows, n_q_heads, n_kv_heads,
            dim, vdim, hd);
  if (rot < 0 || rot % 2 || rot > dim || (rot > 0 && !inv_freq))
    SB_FAIL(SB_ERR_ARG, "sb_attn_prep: %d rotated of %d dimensions (even, at most dim, with a table)", rot, dim);
  if (v_inv_freq && vdim % 2) SB_FAIL(SB_ERR_ARG, "sb_attn_prep: rotated values need an even vdim, not %d", vdim);
  if (v_off < 0 && vdim != dim) SB_FAIL(SB_ERR_ARG, "sb_attn_prep: keys as values need vdim == dim (%d, %d)", vdim, dim);
  if (!sb_valid_dtype(cache_dtype) || !sb_valid_dtype(q_dtype) || ((q_norm || k_norm) && !sb_valid_dtype(norm_dtype)))
    SB_FAIL(SB_ERR_ARG, "sb_attn_prep: dtype codes %d %d %d", cache_dtype, q_dtype, norm_dtype);
  if (!proj || !q_out || !row_pos || (has_kv && (!cache || !row_seq || !page_off || !page_ids || page_size <= 0)))
    SB_FAIL(SB_ERR_ARG, "sb_attn_prep: arguments missing");
  if ((q_norm == nullptr) != (k_norm == nullptr)) SB_FAIL(SB_ERR_ARG, "sb_attn_prep: one of the two norms is missing");
  if (head_norm < 0 || head_norm > 2 || (head_norm == 1 && !q_norm) || (head_norm == 2 && q_norm))
    SB_FAIL(SB_ERR_ARG, "sb_attn_prep: head_norm %d (1 needs the two weights, 2 takes none)", head_norm);
  const int most_heads = n_q_heads > n_kv_heads ? n_q_heads : n_kv_heads;
  const size_t staged = head_norm ? ((size_t)most_heads * dim + most_heads) * sizeof(float) : 0;
  if (staged > 200 * 1024)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attn_prep: %d heads of %d values do not fit shared memory for per-head norms",
            most_heads, dim);
  PrepArgs p;
  p.head_norm = head_norm; p.rot_scale = rot_scale;
  p.proj = proj; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.dim = dim; p.vdim = vdim; p.hd = hd;
  p.rot = rot; p.interleaved = interleaved; p.inv_freq = inv_freq; p.v_inv_freq = v_inv_freq;
  p.q_norm = q_norm; p.k_norm = k_norm; p.eps = eps; p.row_seq = row_seq; p.row_pos = row_pos;
  p.page_off = page_off; p.page_ids = page_ids; p.page_size = page_size; p.has_kv = has_kv;
  p.cache = cache; p.q_out = q_out;
  constexpr int NT = 256;
  const dim3 grid(n_rows, has_kv ? 3 : 1);
  SB_DISPATCH_DTYPE(q_norm ? norm_dtype : SB_F32, TW, {
    SB_DISPATCH_DTYPE(q_dtype, TQ, {
      SB_DISPATCH_DTYPE(has_kv ? cache_dtype : SB_F32, TC, {
        if (staged > 48 * 1024 &&
            cudaFuncSetAttribute(attn_prep_kernel<NT, TW, TQ, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)staged) != cudaSuccess)
          SB_FAIL(SB_ERR_CUDA, "sb_attn_prep: shared memory opt-in failed");
        sb_launch<SB_K_ELEMENTWISE>(attn_prep_kernel<NT, TW, TQ, TC>, grid, dim3(NT), staged, stream, p);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_attn_prep");
  return SB_OK;
}

extern "C" int sb_attn_unrotate(const void* in, void* out, int dtype, int n_rows, int n_heads, int hd, int vdim,
                                int interleaved, const float* v_inv_freq, const int32_t* row_pos,
                                const float* gate, int gate_ld, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || vdim <= 0 || hd < vdim || !in || !out || !sb_valid_dtype(dtype))
    SB_FAIL(SB_ERR_ARG, "sb_attn_unrotate: rows=%d heads=%d hd=%d vdim=%d dtype=%d", n_rows, n_heads, hd, vdim, dtype);
  if (v_inv_freq && (vdim % 2 || !row_pos)) SB_FAIL(SB_ERR_ARG, "sb_attn_unrotate: rotation needs an even vdim and positions");
  SB_DISPATCH_DTYPE(dtype, T, {
    sb_launch<SB_K_ELEMENTWISE>(attn_unrotate_kernel<256, T>, dim3(n_rows), dim3(256), 0, stream, (const T*)in, (T*)out,
                                n_heads, hd, vdim, interleaved, v_inv_freq, row_pos, gate, gate_ld);
  });
  SB_CHECK_LAUNCH("sb_attn_unrotate");
  return SB_OK;
}

extern "C" int sb_linrec_prep(float* proj, int n_rows, int ld, int q_off, int k_off, int n_heads, int dim,
                              float q_scale, float k_scale, int rot, int interleaved, const float* inv_freq,
                              const int32_t* row_pos, float* z, float inv_tau, const void* a2,
                              const void* a2_bias, int a2_dtype, int rank, int a1_off, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || dim <= 0 || !proj) SB_FAIL(SB_ERR_ARG, "sb_linrec_prep: rows=%d heads=%d dim=%d", n_rows, n_heads, dim);
  if (rot < 0 || rot % 2 || rot > dim || (rot > 0 && (!inv_freq || !row_pos)))
    SB_FAIL(SB_ERR_ARG, "sb_linrec_prep: %d rotated of %d dimensions (even, at most dim, with a table)", rot, dim);
  if (a2 && (!z || !a2_bias || rank <= 0 || a1_off < 0 || !sb_valid_dtype(a2_dtype)))
    SB_FAIL(SB_ERR_ARG, "sb_linrec_prep: the decay map needs z, its bias, a rank and a valid dtype (rank=%d dtype=%d)", rank, a2_dtype);
  const size_t n = (size_t)n_rows * n_heads * dim;
  SB_DISPATCH_DTYPE(a2 ? a2_dtype : SB_F32, TA, {
    sb_launch<SB_K_ELEMENTWISE>(linrec_prep_kernel<TA>, dim3(grid_for(n, 256)), dim3(256), 0, stream, proj, ld, q_off,
                                k_off, n_heads, dim, q_scale, k_scale, rot, interleaved, inv_freq, row_pos,
                                (size_t)n_rows, z, inv_tau, (const TA*)a2, (const TA*)a2_bias, rank, a1_off);
  });
  SB_CHECK_LAUNCH("sb_linrec_prep");
  return SB_OK;
}

extern "C" int sb_linrec_out(const float* o, const float* proj, int n_rows, int ld, int g_off, int n_heads,
                             int vdim, const void* norm_w, int norm_w_dtype, int w_per_head, int gate_sigmoid,
                             float eps, void* out, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || vdim <= 0 || !o || !proj || !out)
    SB_FAIL(SB_ERR_ARG, "sb_linrec_out: rows=%d heads=%d vdim=%d", n_rows, n_heads, vdim);
  if (!sb_valid_dtype(out_dtype) || (norm_w && !sb_valid_dtype(norm_w_dtype)))
    SB_FAIL(SB_ERR_ARG, "sb_linrec_out: dtype codes %d %d", out_dtype, norm_w_dtype);
  const size_t items = (size_t)n_rows * n_heads;
  const int blocks = (int)((items + 7) / 8);
  SB_DISPATCH_DTYPE(norm_w ? norm_w_dtype : SB_F32, TW, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      sb_launch<SB_K_ELEMENTWISE>(linrec_out_kernel<TW, TO>, dim3(blocks), dim3(256), 0, stream, o, proj, ld, g_off,
                                  items, n_heads, vdim, (const TW*)norm_w, w_per_head, gate_sigmoid, eps, (TO*)out);
    });
  });
  SB_CHECK_LAUNCH("sb_linrec_out");
  return SB_OK;
}
