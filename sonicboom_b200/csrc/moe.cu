// Mixture of experts: every row goes through the `top` experts whose router logits are largest.
//
//   sb_moe_route:   per row, the `top` largest logits (the lower index wins a tie), their softmax
//                   over the chosen ones only; expert ids and weights per (row, choice) pair
//   sb_moe_group:   the pairs grouped by expert, and the tiles of up to 32 pairs of one expert that
//                   the products walk (one block; everything stays on the device)
//   sb_moe_up:      for every tile, gate and up products of the expert with the clamped gated
//                   activation a * sigmoid(slope a) * (b + 1) in the epilogue
//   sb_moe_down:    for every tile, the expert's down product, one float32 row per pair
//   sb_moe_combine: x[row] += sum over the row's choices, in the order of the choices, of
//                   weight * that pair's row
//
// A pair's result is a function of its own row and expert only (every output is one dot product
// summed in a fixed order), so results do not depend on what else a step holds or on the order in
// which pairs were grouped.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int BM = 32, BN = 64, BK = 32;      // pairs, outputs, inner values of a tile
constexpr int GEMM_THREADS = 256;

__global__ void moe_route_kernel(const float* logits, int n_rows, int n_experts, int top, int32_t* ids,
                                 float* weights) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  const float* z = logits + (size_t)r * n_experts;
  int32_t* id = ids + (size_t)r * top;
  float* w = weights + (size_t)r * top;
  for (int k = 0; k < top; ++k) {
    int best = -1;
    float bv = 0.0f;
    for (int e = 0; e < n_experts; ++e) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= id[j] == e;
      const float v = z[e];
      if (!taken && (best < 0 || v > bv)) best = e, bv = v;
    }
    id[k] = best;
    w[k] = bv;
  }
  const float m = w[0];                        // the largest chosen logit
  float sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    w[k] = expf(w[k] - m);
    sum += w[k];
  }
  for (int k = 0; k < top; ++k) w[k] /= sum;
}

// meta: [0] number of tiles; then per tile (expert, first place in `order`, pairs).
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* ids, int n_pairs, int n_experts, int32_t* order, int32_t* meta) {
  extern __shared__ int32_t sh[];               // counts, then starts, then cursors
  int32_t* count = sh;
  int32_t* start = sh + n_experts;
  int32_t* cursor = sh + 2 * n_experts;
  sb_pdl_launch();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  sb_pdl_wait();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < n_experts; ++e) {
      start[e] = at;
      for (int o = 0; o < count[e]; o += BM) {
        meta[1 + 3 * tiles] = e;
        meta[2 + 3 * tiles] = at + o;
        meta[3 + 3 * tiles] = min(BM, count[e] - o);
        ++tiles;
      }
      at += count[e];
    }
    meta[0] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    order[start[e] + atomicAdd(&cursor[e], 1)] = p;
  }
}

// One tile of pairs of one expert times BN outputs.  GATED: a[pair's row] . (gate | up)^T with
// the activation, written at the pair's place in `order`; else act[place] . down^T, written at the
// pair's own index.
template <typename TA, typename TW, bool GATED>
__global__ void __launch_bounds__(GEMM_THREADS)
moe_gemm_kernel(const TA* a, const TW* __restrict__ w, const int32_t* order, const int32_t* meta, int top,
                int n_out, int n_in, float limit, float slope, void* out_) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[GATED ? 2 : 1][BK][BN + 1];
  __shared__ int32_t src_row[BM];
  sb_pdl_launch();
  sb_pdl_wait();
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int e = meta[1 + 3 * tile], first = meta[2 + 3 * tile], cnt = meta[3 + 3 * tile];
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;       // 4 outputs x 2 pairs a thread
  if (tid < BM) src_row[tid] = tid < cnt ? (GATED ? order[first + tid] / top : first + tid) : -1;
  __syncthreads();
  const TW* we = w + (size_t)e * (GATED ? 2 : 1) * n_out * n_in;
  float acc[GATED ? 2 : 1][2][4] = {};
  for (int k0 = 0; k0 < n_in; k0 += BK) {
    for (int i = tid; i < BM * BK; i += GEMM_THREADS) {
      const int m = i / BK, k = i % BK;
      const int row = src_row[m];
      As[k][m] = (row >= 0 && k0 + k < n_in) ? sb_to_f32<TA>(a[(size_t)row * n_in + k0 + k]) : 0.0f;
    }
    for (int i = tid; i < BN * BK; i += GEMM_THREADS) {
      const int n = i / BK, k = i % BK;
      const bool ok = n0 + n < n_out && k0 + k < n_in;
      Ws[0][k][n] = ok ? sb_to_f32<TW>(we[(size_t)(n0 + n) * n_in + k0 + k]) : 0.0f;
      if (GATED) Ws[1][k][n] = ok ? sb_to_f32<TW>(we[(size_t)(n_out + n0 + n) * n_in + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < BK; ++k) {
      const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float b = Ws[g][k][tx * 4 + j];
          acc[g][0][j] = fmaf(a0, b, acc[g][0][j]);
          acc[g][1][j] = fmaf(a1, b, acc[g][1][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = ty * 2 + i;
    if (m >= cnt) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= n_out) continue;
      if (GATED) {
        TA* out = (TA*)out_;
        out[(size_t)(first + m) * n_out + n] = sb_from_f32<TA>(sb_glu_clamped(acc[0][i][j], acc[GATED ? 1 : 0][i][j], limit, slope));
      } else {
        float* out = (float*)out_;
        out[(size_t)order[first + m] * n_out + n] = acc[0][i][j];
      }
    }
  }
}

__global__ void moe_combine_kernel(float* x, const float* pair_out, const float* weights, int top, int width) {
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < top; ++k) s = fmaf(weights[r * top + k], pair_out[(r * top + k) * width + c], s);
    x[r * width + c] += s;
  }
}

}  // namespace

extern "C" int sb_moe_route(const float* logits, int n_rows, int n_experts, int top, int32_t* ids, float* weights,
                            cudaStream_t stream) {
  if (n_rows <= 0 || n_experts <= 0 || top <= 0 || top > n_experts || !logits || !ids || !weights)
    SB_FAIL(SB_ERR_ARG, "sb_moe_route: rows=%d experts=%d top=%d", n_rows, n_experts, top);
  sb_launch<SB_K_ELEMENTWISE>(moe_route_kernel, dim3((n_rows + 127) / 128), dim3(128), 0, stream, logits, n_rows, n_experts,
                              top, ids, weights);
  SB_CHECK_LAUNCH("sb_moe_route");
  return SB_OK;
}

extern "C" int sb_moe_max_tiles(int n_pairs, int n_experts) { return (n_pairs + BM - 1) / BM + n_experts; }

extern "C" int sb_moe_group(const int32_t* ids, int n_pairs, int n_experts, int32_t* order, int32_t* meta,
                            cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0 || !ids || !order || !meta)
    SB_FAIL(SB_ERR_ARG, "sb_moe_group: pairs=%d experts=%d", n_pairs, n_experts);
  const size_t smem = (size_t)3 * n_experts * sizeof(int32_t);
  if (smem > 48 * 1024) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_moe_group: %d experts", n_experts);
  sb_launch<SB_K_ELEMENTWISE>(moe_group_kernel, dim3(1), dim3(1024), smem, stream, ids, n_pairs, n_experts, order, meta);
  SB_CHECK_LAUNCH("sb_moe_group");
  return SB_OK;
}

extern "C" int sb_moe_up(const void* a, int a_dtype, const void* w, int w_dtype, const int32_t* order,
                         const int32_t* meta, int n_pairs, int n_experts, int top, int ff, int width, float limit,
                         float slope, void* act, cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0 || top <= 0 || ff <= 0 || width <= 0 || !a || !w || !order || !meta || !act)
    SB_FAIL(SB_ERR_ARG, "sb_moe_up: pairs=%d experts=%d top=%d ff=%d width=%d", n_pairs, n_experts, top, ff, width);
  if (!sb_valid_dtype(a_dtype) || a_dtype != w_dtype) SB_FAIL(SB_ERR_ARG, "sb_moe_up: dtype codes %d %d", a_dtype, w_dtype);
  const dim3 grid(sb_moe_max_tiles(n_pairs, n_experts), (ff + BN - 1) / BN);
  SB_DISPATCH_DTYPE(a_dtype, T, {
    sb_launch<SB_K_OTHER>(moe_gemm_kernel<T, T, true>, grid, dim3(GEMM_THREADS), 0, stream, (const T*)a, (const T*)w, order,
                          meta, top, ff, width, limit, slope, act);
  });
  SB_CHECK_LAUNCH("sb_moe_up");
  return SB_OK;
}

extern "C" int sb_moe_down(const void* act, int a_dtype, const void* w, int w_dtype, const int32_t* order,
                           const int32_t* meta, int n_pairs, int n_experts, int top, int width, int ff,
                           float* pair_out, cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0 || top <= 0 || ff <= 0 || width <= 0 || !act || !w || !order || !meta || !pair_out)
    SB_FAIL(SB_ERR_ARG, "sb_moe_down: pairs=%d experts=%d top=%d ff=%d width=%d", n_pairs, n_experts, top, ff, width);
  if (!sb_valid_dtype(a_dtype) || a_dtype != w_dtype) SB_FAIL(SB_ERR_ARG, "sb_moe_down: dtype codes %d %d", a_dtype, w_dtype);
  const dim3 grid(sb_moe_max_tiles(n_pairs, n_experts), (width + BN - 1) / BN);
  SB_DISPATCH_DTYPE(a_dtype, T, {
    sb_launch<SB_K_OTHER>(moe_gemm_kernel<T, T, false>, grid, dim3(GEMM_THREADS), 0, stream, (const T*)act, (const T*)w, order,
                          meta, top, width, ff, 0.0f, 0.0f, (void*)pair_out);
  });
  SB_CHECK_LAUNCH("sb_moe_down");
  return SB_OK;
}

extern "C" int sb_moe_combine(float* x, const float* pair_out, const float* weights, int n_rows, int top, int width,
                              cudaStream_t stream) {
  if (n_rows <= 0 || top <= 0 || width <= 0 || !x || !pair_out || !weights)
    SB_FAIL(SB_ERR_ARG, "sb_moe_combine: rows=%d top=%d width=%d", n_rows, top, width);
  const int by = n_rows >= 256 ? 1 : (width + 255) / 256;
  sb_launch<SB_K_ELEMENTWISE>(moe_combine_kernel, dim3(n_rows, by < 64 ? by : 64), dim3(256), 0, stream, x, pair_out, weights,
                              top, width);
  SB_CHECK_LAUNCH("sb_moe_combine");
  return SB_OK;
}
