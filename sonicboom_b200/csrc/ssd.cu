// Row kernels of the state-space mixer (a scalar decay per token and head over a matrix state):
//
//   sb_ssd_prep: step sizes dt = softplus(raw + bias) per head, decays exp(-exp(A_log) dt) into
//                decay [rows, heads], and the inputs times their step size, dt * x, into columns
//                of the row buffer of their own (what the recurrence adds to the state)
//   sb_ssd_out:  y = o + D x per head, times silu(z), then the RMS norm of every one of
//                `norm_groups` equal parts of the row, times a weight
//
// The recurrence itself is sb_linrec_scan with a decay per token and head and q (C) and k (B)
// shared by the heads of a group.  All arithmetic is float32.
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

__device__ __forceinline__ float softplus(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

template <typename TW>
__global__ void ssd_prep_kernel(const float* proj, int ld_proj, int dt_off, float* xbc, int ld, int x_off, int xdt_off,
                                int n_heads, int vdim, int per, const TW* __restrict__ dt_bias,
                                const TW* __restrict__ a_log, float* decay) {
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  const int inner = n_heads * vdim;
  // a thread takes `per` channels, a block's apart: one at few rows, where the blocks are few
  for (int i = 0, c = blockIdx.y * blockDim.x * per + threadIdx.x; i < per && c < inner; ++i, c += blockDim.x) {
    const int h = c / vdim;
    const float dt = softplus(proj[r * ld_proj + dt_off + h] + sb_to_f32<TW>(dt_bias[h]));
    xbc[r * ld + xdt_off + c] = dt * xbc[r * ld + x_off + c];
    if (c == h * vdim) decay[r * n_heads + h] = expf(-expf(sb_to_f32<TW>(a_log[h])) * dt);
  }
}

// One block per (row, norm group).
template <int NT, typename TW, typename TO>
__global__ void __launch_bounds__(NT)
ssd_out_kernel(const float* o, const float* xbc, int ld, int x_off, const float* proj, int ld_proj, int z_off,
               int n_heads, int vdim, int group, const TW* __restrict__ d_skip, const TW* __restrict__ norm_w,
               float eps, TO* out) {
  __shared__ float red[NT / 32 + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  const int inner = n_heads * vdim, c0 = blockIdx.y * group;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < group; i += NT) {
    const int c = c0 + i;
    const float y = (o[r * inner + c] + sb_to_f32<TW>(d_skip[c / vdim]) * xbc[r * ld + x_off + c]) *
                    sb_silu(proj[r * ld_proj + z_off + c]);
    sq = fmaf(y, y, sq);
  }
  const float inv = 1.0f / sqrtf(block_sum<NT>(sq, red) / (float)group + eps);
  for (int i = threadIdx.x; i < group; i += NT) {
    const int c = c0 + i;
    const float y = (o[r * inner + c] + sb_to_f32<TW>(d_skip[c / vdim]) * xbc[r * ld + x_off + c]) *
                    sb_silu(proj[r * ld_proj + z_off + c]);
    out[r * inner + c] = sb_from_f32<TO>((y * inv) * sb_to_f32<TW>(norm_w[c]));
  }
}

}  // namespace

extern "C" int sb_ssd_prep(const float* proj, int n_rows, int ld_proj, int dt_off, float* xbc, int ld, int x_off,
                           int xdt_off, int n_heads, int vdim, const void* dt_bias, const void* a_log, int w_dtype,
                           float* decay, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || vdim <= 0 || !proj || !xbc || !dt_bias || !a_log || !decay)
    SB_FAIL(SB_ERR_ARG, "sb_ssd_prep: rows=%d heads=%d vdim=%d", n_rows, n_heads, vdim);
  const int inner = n_heads * vdim;
  if (dt_off < 0 || dt_off + n_heads > ld_proj || x_off < 0 || xdt_off < 0 || x_off + inner > ld || xdt_off + inner > ld ||
      (x_off < xdt_off + inner && xdt_off < x_off + inner))
    SB_FAIL(SB_ERR_ARG, "sb_ssd_prep: offsets %d of %d; %d, %d of %d", dt_off, ld_proj, x_off, xdt_off, ld);
  if (!sb_valid_dtype(w_dtype)) SB_FAIL(SB_ERR_ARG, "sb_ssd_prep: dtype code %d", w_dtype);
  const int per = n_rows >= 256 ? 8 : 1;
  const int by = (inner + 256 * per - 1) / (256 * per);
  if (by > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_ssd_prep: %d values a row", inner);
  SB_DISPATCH_DTYPE(w_dtype, TW, {
    sb_launch<SB_K_ELEMENTWISE>(ssd_prep_kernel<TW>, dim3(n_rows, by), dim3(256), 0, stream, proj, ld_proj, dt_off, xbc, ld,
                                x_off, xdt_off, n_heads, vdim, per, (const TW*)dt_bias, (const TW*)a_log, decay);
  });
  SB_CHECK_LAUNCH("sb_ssd_prep");
  return SB_OK;
}

extern "C" int sb_ssd_out(const float* o, const float* xbc, int n_rows, int ld, int x_off, const float* proj,
                          int ld_proj, int z_off, int n_heads, int vdim, int norm_groups, const void* d_skip,
                          const void* norm_w, int w_dtype, float eps, void* out, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || vdim <= 0 || norm_groups <= 0 || !o || !xbc || !proj || !d_skip || !norm_w || !out)
    SB_FAIL(SB_ERR_ARG, "sb_ssd_out: rows=%d heads=%d vdim=%d groups=%d", n_rows, n_heads, vdim, norm_groups);
  const int inner = n_heads * vdim;
  if (inner % norm_groups || norm_groups > 65535)
    SB_FAIL(SB_ERR_ARG, "sb_ssd_out: %d values do not split into %d equal parts", inner, norm_groups);
  if (x_off < 0 || x_off + inner > ld || z_off < 0 || z_off + inner > ld_proj)
    SB_FAIL(SB_ERR_ARG, "sb_ssd_out: offsets %d of %d, %d of %d", x_off, ld, z_off, ld_proj);
  if (!sb_valid_dtype(w_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_ssd_out: dtype codes %d %d", w_dtype, out_dtype);
  const int group = inner / norm_groups;
  SB_DISPATCH_DTYPE(w_dtype, TW, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      if (group <= 1024 || n_rows * norm_groups >= 512)
        sb_launch<SB_K_ELEMENTWISE>(ssd_out_kernel<256, TW, TO>, dim3(n_rows, norm_groups), dim3(256), 0, stream, o, xbc,
                                    ld, x_off, proj, ld_proj, z_off, n_heads, vdim, group, (const TW*)d_skip,
                                    (const TW*)norm_w, eps, (TO*)out);
      else
        sb_launch<SB_K_ELEMENTWISE>(ssd_out_kernel<1024, TW, TO>, dim3(n_rows, norm_groups), dim3(1024), 0, stream, o, xbc,
                                    ld, x_off, proj, ld_proj, z_off, n_heads, vdim, group, (const TW*)d_skip,
                                    (const TW*)norm_w, eps, (TO*)out);
    });
  });
  SB_CHECK_LAUNCH("sb_ssd_out");
  return SB_OK;
}
