// Row kernels of the residual stream for blocks that norm a sublayer's result before they add
// it, and for models that feed each layer a weighted sum of everything before it.
//
//   sb_norm_add:   out[r] = x[r] + y[r] / sqrt(mean(y[r]^2) + eps) * w
//   sb_gated_act:  out = act(gate) * up over [gate | up] rows: silu, the clamped form, or the tanh form of gelu
//   sb_scale:      x *= c
//   sb_depth_mix:  out[r] = sum_j c[j] * planes[j][r]           (j ascending, float32)
//
// Both can also deliver the RMS norm of the row they have just finished (the first norm of
// whatever runs next) in the activation dtype, so that the row is read once.  One block per
// row; sums are fixed trees (thread-strided partial sums, warp shuffles, the warps in order), so
// a row's result does not depend on the other rows of the launch.  All arithmetic is float32.
#include "common.cuh"

namespace {

// A row is walked in groups of V values (V = 4: 16-byte accesses, for widths that are multiples
// of 4 and aligned rows) by NT threads: 256 when the launch has rows enough to fill the GPU, 1024
// when it has few (decode), so that a row's loads are in flight together.
template <int V>
struct Vec {
  float v[V];
};
template <int V>
__device__ __forceinline__ Vec<V> ld(const float* p) {
  Vec<V> r;
  if (V == 4) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    r.v[0] = f.x; r.v[1 % V] = f.y; r.v[2 % V] = f.z; r.v[3 % V] = f.w;
  } else {
    r.v[0] = *p;
  }
  return r;
}
template <int V>
__device__ __forceinline__ void st(float* p, const Vec<V>& r) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1 % V], r.v[2 % V], r.v[3 % V]);
  else *p = r.v[0];
}

// Sum over the block, the same value in every thread.  `red` holds NT / 32 + 1 floats.
template <int NT>
__device__ __forceinline__ float block_sum(float s, float* red) {
  s = sb_warp_sum(s);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();                       // `red` may still be read from an earlier sum
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

// Writes normed[i] = out[i] * inv * next_w[i] for the thread's own elements of the row it wrote.
template <int NT, int V, typename TN, typename TO>
__device__ __forceinline__ void write_normed(const float* o, int width, float sq, float next_eps,
                                             const TN* __restrict__ next_w, TO* nrm, float* red) {
  const float total = block_sum<NT>(sq, red);
  const float inv = 1.0f / sqrtf(total / (float)width + next_eps);
  for (int i = threadIdx.x * V; i < width; i += NT * V) {
    const Vec<V> x = ld<V>(o + i);
#pragma unroll
    for (int j = 0; j < V; ++j) nrm[i + j] = sb_from_f32<TO>((x.v[j] * inv) * sb_to_f32<TN>(next_w[i + j]));
  }
}

template <int NT, int V, typename TW, typename TN, typename TO>
__global__ void __launch_bounds__(NT)
norm_add_kernel(const float* y, const float* x, int width, const TW* __restrict__ w, float eps,
                float* out, const TN* __restrict__ next_w, float next_eps, TO* normed) {
  __shared__ float red[NT / 32 + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  const float* yr = y + r * width;
  const float* xr = x + r * width;
  float* o = out + r * width;
  float s = 0.0f;
  for (int i = threadIdx.x * V; i < width; i += NT * V) {
    const Vec<V> a = ld<V>(yr + i);
#pragma unroll
    for (int j = 0; j < V; ++j) s = fmaf(a.v[j], a.v[j], s);
  }
  const float inv = 1.0f / sqrtf(block_sum<NT>(s, red) / (float)width + eps);
  float sq = 0.0f;
  for (int i = threadIdx.x * V; i < width; i += NT * V) {
    const Vec<V> a = ld<V>(yr + i), b = ld<V>(xr + i);
    Vec<V> v;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      v.v[j] = b.v[j] + (a.v[j] * inv) * sb_to_f32<TW>(w[i + j]);
      sq = fmaf(v.v[j], v.v[j], sq);
    }
    st<V>(o + i, v);
    if (normed && !next_w) {             // no norm named: the finished row as it is, in the other dtype
#pragma unroll
      for (int j = 0; j < V; ++j) normed[r * width + i + j] = sb_from_f32<TO>(v.v[j]);
    }
  }
  if (normed && next_w) write_normed<NT, V, TN, TO>(o, width, sq, next_eps, next_w, normed + r * width, red);
}

constexpr int MIX_MAX = 256;       // most planes one depth mix adds up

// With `join_y` the last plane is made here first: planes[n - 1][r] = join_x[r] + join_y[r] /
// sqrt(mean(join_y[r]^2) + join_eps) * join_w (join_x may be that plane itself), so that the
// block's last residual add and the mix that follows it are one pass over the row.
template <int NT, int V, typename TC, typename TN, typename TO>
__global__ void __launch_bounds__(NT)
depth_mix_kernel(float* planes, size_t plane, int n_inputs, const TC* __restrict__ coef, int width, float* out,
                 const TN* __restrict__ next_w, float next_eps, TO* normed, const float* join_y,
                 const float* join_x, const TC* __restrict__ join_w, float join_eps) {
  __shared__ float red[NT / 32 + 1];
  __shared__ float c[MIX_MAX];
  sb_pdl_launch();
  for (int j = threadIdx.x; j < n_inputs; j += NT) c[j] = sb_to_f32<TC>(coef[j]);
  __syncthreads();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  float* o = out + r * width;
  float inv = 0.0f;
  if (join_y) {
    float s = 0.0f;
    for (int i = threadIdx.x * V; i < width; i += NT * V) {
      const Vec<V> a = ld<V>(join_y + r * width + i);
#pragma unroll
      for (int j = 0; j < V; ++j) s = fmaf(a.v[j], a.v[j], s);
    }
    inv = 1.0f / sqrtf(block_sum<NT>(s, red) / (float)width + join_eps);
  }
  const int n_read = join_y ? n_inputs - 1 : n_inputs;
  float sq = 0.0f;
  for (int i = threadIdx.x * V; i < width; i += NT * V) {
    float* p = planes + r * width + i;
    Vec<V> v;
#pragma unroll
    for (int j = 0; j < V; ++j) v.v[j] = 0.0f;
#pragma unroll 4
    for (int k = 0; k < n_read; ++k) {
      const Vec<V> a = ld<V>(p + (size_t)k * plane);
#pragma unroll
      for (int j = 0; j < V; ++j) v.v[j] = fmaf(c[k], a.v[j], v.v[j]);
    }
    if (join_y) {
      const Vec<V> a = ld<V>(join_y + r * width + i), b = ld<V>(join_x + r * width + i);
      Vec<V> last;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        last.v[j] = b.v[j] + (a.v[j] * inv) * sb_to_f32<TC>(join_w[i + j]);
        v.v[j] = fmaf(c[n_read], last.v[j], v.v[j]);
      }
      st<V>(p + (size_t)n_read * plane, last);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) sq = fmaf(v.v[j], v.v[j], sq);
    st<V>(o + i, v);
  }
  if (normed) write_normed<NT, V, TN, TO>(o, width, sq, next_eps, next_w, normed + r * width, red);
}

// y = a * sigmoid(alpha a) * (b + 1) with a = min(gate, limit), b = clamp(up, -limit, limit);
// the input row is [gate (ff) | up (ff)] in float32.
// With `interleaved` the row is blocks of SB_SWIGLU_BLOCK gates followed by the up values of the same
// outputs, as the products with a gated epilogue want their weights.
template <typename TO>
__global__ void glu_clamped_kernel(const float* gu, size_t n, int ff, float limit, float alpha,
                                   int interleaved, TO* out) {
  sb_pdl_launch();
  sb_pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / ff, c = e % ff;
    const size_t g = interleaved ? (c / SB_SWIGLU_BLOCK) * 2 * SB_SWIGLU_BLOCK + c % SB_SWIGLU_BLOCK : c;
    const size_t u = interleaved ? g + SB_SWIGLU_BLOCK : ff + c;
    out[e] = sb_from_f32<TO>(sb_glu_clamped(gu[r * 2 * ff + g], gu[r * 2 * ff + u], limit, alpha));
  }
}

// The same row layouts with the activation chosen by `kind`: 0 silu(gate) * up, 1 the clamped form
// above, 2 gelu(gate) * up in gelu's tanh form, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
template <typename TO>
__global__ void gated_act_kernel(const float* gu, size_t n, int ff, int kind, float limit, float alpha,
                                 int interleaved, TO* out) {
  sb_pdl_launch();
  sb_pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / ff, c = e % ff;
    const size_t g = interleaved ? (c / SB_SWIGLU_BLOCK) * 2 * SB_SWIGLU_BLOCK + c % SB_SWIGLU_BLOCK : c;
    const size_t u = interleaved ? g + SB_SWIGLU_BLOCK : ff + c;
    const float gate = gu[r * 2 * ff + g], up = gu[r * 2 * ff + u];
    out[e] = sb_from_f32<TO>(kind == 1 ? sb_glu_clamped(gate, up, limit, alpha)
                                       : kind == 2 ? sb_gelu_tanh(gate) * up : sb_silu(gate) * up);
  }
}

__global__ void scale_kernel(float* x, size_t n, float c) {
  sb_pdl_launch();
  sb_pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) x[e] *= c;
}

}  // namespace

#define SB_DISPATCH_NEXT(has, code, TN, ...)  \
  do {                                         \
    if (!(has) || (code) == SB_F32) {          \
      using TN = float;                        \
      __VA_ARGS__                              \
    } else {                                   \
      using TN = __nv_bfloat16;                \
      __VA_ARGS__                              \
    }                                          \
  } while (0)

// Launches KERNEL<NT, V, T1, TN, TO> over n_rows blocks: 16-byte accesses when `vec`, 1024 threads
// a row when the launch has few rows of a wide stream.
#define SB_ROW_LAUNCH(KERNEL, T1, ...)                                                                        \
  do {                                                                                                        \
    if (vec && wide)                                                                                          \
      sb_launch<SB_K_ELEMENTWISE>(KERNEL<1024, 4, T1, TN, TO>, dim3(n_rows), dim3(1024), 0, stream, __VA_ARGS__); \
    else if (vec)                                                                                             \
      sb_launch<SB_K_ELEMENTWISE>(KERNEL<256, 4, T1, TN, TO>, dim3(n_rows), dim3(256), 0, stream, __VA_ARGS__);   \
    else                                                                                                      \
      sb_launch<SB_K_ELEMENTWISE>(KERNEL<256, 1, T1, TN, TO>, dim3(n_rows), dim3(256), 0, stream, __VA_ARGS__);   \
  } while (0)

extern "C" int sb_norm_add(const float* y, const float* x, int n_rows, int width, const void* w,
                           int w_dtype, float eps, float* out, const void* next_w, int next_w_dtype,
                           float next_eps, void* normed, int normed_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || !y || !x || !w || !out)
    SB_FAIL(SB_ERR_ARG, "sb_norm_add: rows=%d width=%d", n_rows, width);
  if (!sb_valid_dtype(w_dtype) || (normed && ((next_w && !sb_valid_dtype(next_w_dtype)) || !sb_valid_dtype(normed_dtype))))
    SB_FAIL(SB_ERR_ARG, "sb_norm_add: dtype codes %d %d %d", w_dtype, next_w_dtype, normed_dtype);
  if (!(eps >= 0.0f) || (normed && next_w && !(next_eps >= 0.0f))) SB_FAIL(SB_ERR_ARG, "sb_norm_add: eps %g %g", eps, next_eps);
  const bool vec = width % 4 == 0 && (((uintptr_t)y | (uintptr_t)x | (uintptr_t)out) & 15) == 0;
  const bool wide = n_rows <= 256 && width >= 2048;
  SB_DISPATCH_DTYPE(w_dtype, TW, {
    SB_DISPATCH_NEXT(normed && next_w, next_w_dtype, TN, {
      SB_DISPATCH_NEXT(normed, normed_dtype, TO, {
        SB_ROW_LAUNCH(norm_add_kernel, TW, y, x, width, (const TW*)w, eps, out, (const TN*)next_w, next_eps, (TO*)normed);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_norm_add");
  return SB_OK;
}

extern "C" int sb_depth_mix(float* planes, size_t plane, int n_inputs, const void* coef,
                            int coef_dtype, int n_rows, int width, float* out, const void* next_w,
                            int next_w_dtype, float next_eps, void* normed, int normed_dtype,
                            const float* join_y, const float* join_x, const void* join_w, int join_w_dtype,
                            float join_eps, cudaStream_t stream) {
  if (join_y && (!join_x || !join_w || join_w_dtype != coef_dtype || !(join_eps >= 0.0f)))
    SB_FAIL(SB_ERR_ARG, "sb_depth_mix: a joined last plane needs its stream, a norm weight of the coefficients' dtype and eps");
  if (n_rows <= 0 || width <= 0 || !planes || !coef || !out)
    SB_FAIL(SB_ERR_ARG, "sb_depth_mix: rows=%d width=%d", n_rows, width);
  if (n_inputs < 1 || n_inputs > MIX_MAX)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_depth_mix: %d inputs (1 to %d)", n_inputs, MIX_MAX);
  if (plane < (size_t)n_rows * width) SB_FAIL(SB_ERR_ARG, "sb_depth_mix: planes overlap");
  const bool vec = width % 4 == 0 && plane % 4 == 0 &&
                   (((uintptr_t)planes | (uintptr_t)out | (uintptr_t)join_y | (uintptr_t)join_x) & 15) == 0;
  const bool wide = n_rows <= 256 && width >= 2048;
  if (!sb_valid_dtype(coef_dtype) || (normed && (!next_w || !sb_valid_dtype(next_w_dtype) || !sb_valid_dtype(normed_dtype))))
    SB_FAIL(SB_ERR_ARG, "sb_depth_mix: dtype codes %d %d %d", coef_dtype, next_w_dtype, normed_dtype);
  SB_DISPATCH_DTYPE(coef_dtype, TC, {
    SB_DISPATCH_NEXT(normed, next_w_dtype, TN, {
      SB_DISPATCH_NEXT(normed, normed_dtype, TO, {
        SB_ROW_LAUNCH(depth_mix_kernel, TC, planes, plane, n_inputs, (const TC*)coef, width, out, (const TN*)next_w,
                      next_eps, (TO*)normed, join_y, join_x, (const TC*)join_w, join_eps);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_depth_mix");
  return SB_OK;
}

extern "C" int sb_glu_clamped(const float* gu, int n_rows, int ff, float limit, float alpha, int interleaved,
                              void* out, int out_dtype, cudaStream_t stream) {
  if (interleaved && ff % SB_SWIGLU_BLOCK)
    SB_FAIL(SB_ERR_ARG, "sb_glu_clamped: %d outputs are no multiple of %d", ff, SB_SWIGLU_BLOCK);
  if (n_rows <= 0 || ff <= 0 || !gu || !out) SB_FAIL(SB_ERR_ARG, "sb_glu_clamped: rows=%d ff=%d", n_rows, ff);
  if (!sb_valid_dtype(out_dtype)) SB_FAIL(SB_ERR_ARG, "sb_glu_clamped: dtype code %d", out_dtype);
  if (!(limit > 0.0f)) SB_FAIL(SB_ERR_ARG, "sb_glu_clamped: limit %g must be positive", limit);
  const size_t n = (size_t)n_rows * ff;
  const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
  SB_DISPATCH_DTYPE(out_dtype, TO, {
    sb_launch<SB_K_ELEMENTWISE>(glu_clamped_kernel<TO>, dim3(blocks), dim3(256), 0, stream, gu, n, ff, limit, alpha,
                                interleaved, (TO*)out);
  });
  SB_CHECK_LAUNCH("sb_glu_clamped");
  return SB_OK;
}

extern "C" int sb_gated_act(const float* gu, int n_rows, int ff, int kind, float limit, float alpha, int interleaved,
                            void* out, int out_dtype, cudaStream_t stream) {
  if (interleaved && ff % SB_SWIGLU_BLOCK)
    SB_FAIL(SB_ERR_ARG, "sb_gated_act: %d outputs are no multiple of %d", ff, SB_SWIGLU_BLOCK);
  if (n_rows <= 0 || ff <= 0 || !gu || !out) SB_FAIL(SB_ERR_ARG, "sb_gated_act: rows=%d ff=%d", n_rows, ff);
  if (!sb_valid_dtype(out_dtype)) SB_FAIL(SB_ERR_ARG, "sb_gated_act: dtype code %d", out_dtype);
  if (kind < SB_GATE_SILU || kind > SB_GATE_GELU_TANH || (kind == SB_GATE_CLAMPED && !(limit > 0.0f)))
    SB_FAIL(SB_ERR_ARG, "sb_gated_act: kind %d, limit %g", kind, limit);
  const size_t n = (size_t)n_rows * ff;
  const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
  SB_DISPATCH_DTYPE(out_dtype, TO, {
    sb_launch<SB_K_ELEMENTWISE>(gated_act_kernel<TO>, dim3(blocks), dim3(256), 0, stream, gu, n, ff, kind, limit, alpha,
                                interleaved, (TO*)out);
  });
  SB_CHECK_LAUNCH("sb_gated_act");
  return SB_OK;
}

extern "C" int sb_scale(float* x, size_t n, float c, cudaStream_t stream) {
  if (!x || n == 0) SB_FAIL(SB_ERR_ARG, "sb_scale: nothing to scale");
  const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
  sb_launch<SB_K_ELEMENTWISE>(scale_kernel, dim3(blocks), dim3(256), 0, stream, x, n, c);
  SB_CHECK_LAUNCH("sb_scale");
  return SB_OK;
}
