// Mixture of experts: every row goes through the `top` experts whose router logits are largest.
//
//   sb_moe_route:   per row, the `top` largest logits (the lower index wins a tie), their softmax
//                   over the chosen ones only; expert ids and weights per (row, choice) pair
//   sb_moe_group:   the pairs grouped by expert, and the tiles of up to `tile_rows` pairs of one expert
//                   that the products walk (one block; everything stays on the device)
//   sb_moe_up:      for every tile, gate and up products of the expert with the clamped gated
//                   activation a * sigmoid(slope a) * (b + 1) in the epilogue.  bfloat16 with inner
//                   sizes in multiples of 8 runs on tensor cores (mma.sync m16n8k16, tiles of 64 or
//                   128 pairs x 128 weight rows x 64 inner values, a cp.async pipeline of 3 or 4 stages whose
//                   16-byte copies also stream an expert's weights when a step has few pairs); the
//                   rest runs the plain float32 tiles of 32 pairs
//   sb_moe_down:    for every tile, the expert's down product, one float32 row per pair
//   sb_moe_combine: x[row] += sum over the row's choices, in the order of the choices, of
//                   weight * that pair's row
//
// A pair's result is a function of its own row and expert only (every output is one dot product
// summed in a fixed order), so results do not depend on what else a step holds or on the order in
// which pairs were grouped.
#include <limits.h>
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

// The same choice with a warp per row (up to 1024 experts): a lane looks at experts lane, lane + 32, ...,
// the lanes' best are compared by shuffles (the larger logit, then the lower index), and lane 0
// finishes the softmax over the chosen logits in the order they were chosen.
__global__ void __launch_bounds__(128)
moe_route_warp_kernel(const float* logits, int n_rows, int n_experts, int top, int32_t* ids, float* weights) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float* z = logits + (size_t)r * n_experts;
  int32_t* id = ids + (size_t)r * top;
  float* w = weights + (size_t)r * top;
  uint32_t taken = 0;
  for (int k = 0; k < top; ++k) {
    int best = INT_MAX;
    float bv = 0.0f;
    for (int i = 0, e = lane; e < n_experts; ++i, e += 32) {
      const float v = z[e];
      if (!((taken >> i) & 1u) && (best == INT_MAX || v > bv)) best = e, bv = v;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
      const int oe = __shfl_xor_sync(0xffffffffu, best, off);
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      if (oe != INT_MAX && (best == INT_MAX || ov > bv || (ov == bv && oe < best))) best = oe, bv = ov;
    }
    if ((best & 31) == lane) taken |= 1u << (best >> 5);
    if (lane == 0) id[k] = best, w[k] = bv;
  }
  if (lane == 0) {
    const float m = w[0];                      // the largest chosen logit
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
      w[k] = expf(w[k] - m);
      sum += w[k];
    }
    for (int k = 0; k < top; ++k) w[k] /= sum;
  }
}

// The choice with scores that are logistic functions of the logits (a warp per row, up to 1024
// experts).  s_e = sigmoid(z_e); the choice score is s_e + correction_e.  The experts lie in
// `n_groups` equal groups of neighbours; a group's score is the sum of its `group_top` largest
// choice scores, and only experts of the `keep_groups` best groups can be chosen (n_groups 1:
// every expert can).  The `top` experts with the largest choice scores are chosen (the lower
// index wins a tie); their weights are s_e * scale, divided by the chosen ones' sum of s when
// `renormalize`.  All float32.  `sc` holds a warp's choice scores (minus infinity once an expert
// is chosen or its group is out), `gs` its group scores.
constexpr int ROUTE_WARPS = 4, ROUTE_MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_scored_kernel(const float* logits, const float* __restrict__ correction, int n_rows, int n_experts,
                        int top, int n_groups, int keep_groups, int group_top, float scale, int renormalize,
                        int32_t* ids, float* weights) {
  __shared__ float sc_all[ROUTE_WARPS][ROUTE_MAX_EXPERTS];
  __shared__ float gs_all[ROUTE_WARPS][ROUTE_MAX_EXPERTS];
  sb_pdl_launch();
  sb_pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x * ROUTE_WARPS + warp;
  if (r >= n_rows) return;
  float* sc = sc_all[warp];
  float* gs = gs_all[warp];
  const float* z = logits + (size_t)r * n_experts;
  for (int e = lane; e < n_experts; e += 32) {
    const float s = 1.0f / (1.0f + expf(-z[e]));
    sc[e] = s + (correction ? correction[e] : 0.0f);
  }
  __syncwarp();
  if (n_groups > 1) {
    const int per = n_experts / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      // the sum of the group's `group_top` largest choice scores, largest first
      float sum = 0.0f, bound = INFINITY;
      int bound_at = -1;
      for (int k = 0; k < group_top && k < per; ++k) {
        float bv = -INFINITY;
        int best = -1;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = sc[e];
          const bool below = v < bound || (v == bound && e > bound_at);     // not taken yet
          if (below && (best < 0 || v > bv)) best = e, bv = v;
        }
        sum += bv;
        bound = bv;
        bound_at = best;
      }
      gs[g] = sum;
    }
    __syncwarp();
    // the best groups keep their score's sign bit out of the way: mark the kept ones, then close the rest
    for (int k = 0; k < keep_groups; ++k) {
      int best = INT_MAX;
      float bv = -INFINITY;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (best == INT_MAX || v > bv)) best = g, bv = v;
      }
#pragma unroll
      for (int off = 16; off; off >>= 1) {
        const int og = __shfl_xor_sync(0xffffffffu, best, off);
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        if (og != INT_MAX && (best == INT_MAX || ov > bv || (ov == bv && og < best))) best = og, bv = ov;
      }
      if (lane == 0 && best != INT_MAX) gs[best] = INFINITY;              // kept
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gs[e / per] != INFINITY) sc[e] = -INFINITY;
    __syncwarp();
  }
  int32_t* id = ids + (size_t)r * top;
  float* w = weights + (size_t)r * top;
  float total = 0.0f;
  for (int k = 0; k < top; ++k) {
    int best = INT_MAX;
    float bv = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = sc[e];
      if (v != -INFINITY && (best == INT_MAX || v > bv)) best = e, bv = v;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
      const int oe = __shfl_xor_sync(0xffffffffu, best, off);
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      if (oe != INT_MAX && (best == INT_MAX || ov > bv || (ov == bv && oe < best))) best = oe, bv = ov;
    }
    // fewer experts in the kept groups than `top`: the rest of the choices repeat nothing, they
    // point at expert 0 with weight 0
    if (lane == 0) {
      if (best == INT_MAX) {
        id[k] = 0;
        w[k] = 0.0f;
      } else {
        const float s = 1.0f / (1.0f + expf(-z[best]));
        id[k] = best;
        w[k] = s;
        total += s;
        sc[best] = -INFINITY;
      }
    }
    __syncwarp();
  }
  if (lane == 0)
    for (int k = 0; k < top; ++k) w[k] = renormalize ? w[k] / total * scale : w[k] * scale;
}

// meta: [0] number of tiles; then per tile (expert, first place in `order`, pairs).
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* ids, int n_pairs, int n_experts, int tile_rows, int32_t* order, int32_t* meta) {
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
      for (int o = 0; o < count[e]; o += tile_rows) {
        meta[1 + 3 * tiles] = e;
        meta[2 + 3 * tiles] = at + o;
        meta[3 + 3 * tiles] = min(tile_rows, count[e] - o);
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

// ------------------------------------------------------------------------------ tensor cores
typedef __nv_bfloat16 bf16;
constexpr int TN = 128, TK = 64, MMA_THREADS = 256;   // weight rows, inner values of a tile
// cp.async stages: four for the tiles of 64 pairs (24 KiB a stage, two blocks an SM), which also stream an
// expert's weights when a step has few pairs; three for the tiles of 128 pairs (32 KiB a stage)
constexpr int stages_for(int mi) { return mi <= 2 ? 4 : 3; }

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;                            // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// A tile row holds TK = 64 values = 8 chunks of 16 bytes; chunk c of row r is stored at chunk
// c ^ (r & 7): the cp.async stores and the ldmatrix reads are free of bank conflicts.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return (uint32_t)(row * (TK * 2) + ((chunk ^ (row & 7)) << 4));
}

constexpr int mma_smem(int mi) { return stages_for(mi) * (mi * 32 + TN) * TK * 2; }

// One tile of up to MI * 32 pairs of one expert.  2 x 4 warps, MI * 16 pairs x 32 weight rows each.
// GATED: the 128 weight rows of a block are, for each of its four warp columns, 16 gate rows and
// the 16 up rows of the same outputs, so a thread holds gate and up of an output side by side;
// a block finishes 64 outputs.  Else 128 outputs of the down product.  Every output is summed over
// the inner values in the same order whatever the tile, the pair's place in it, or MI.
template <int MI, bool GATED>
__global__ void __launch_bounds__(MMA_THREADS, 2)
moe_gemm_mma_kernel(const bf16* a, const bf16* __restrict__ w, const int32_t* order, const int32_t* meta, int top,
                    int n_out, int n_in, float limit, float slope, void* out_) {
  constexpr int TM = MI * 32, STAGES = stages_for(MI);
  constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int32_t src_row[TM];
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
  sb_pdl_launch();
  sb_pdl_wait();
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int e = meta[1 + 3 * tile], first = meta[2 + 3 * tile], cnt = meta[3 + 3 * tile];
  const int n0 = blockIdx.y * (GATED ? TN / 2 : TN);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp >> 2, warp_n = warp & 3;
  for (int m = tid; m < TM; m += MMA_THREADS) src_row[m] = m < cnt ? (GATED ? order[first + m] / top : first + m) : -1;
  __syncthreads();
  const bf16* we = w + (size_t)e * (GATED ? 2 : 1) * n_out * n_in;
  // what this thread copies of every stage: MI chunks of the pairs' rows, 4 chunks of weight rows
  const int chunk = tid & 7;
  const bf16* a_src[MI];
  const bf16* b_src[4];
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    const int r = src_row[(tid >> 3) + i * 32];
    a_src[i] = r >= 0 ? a + (size_t)r * n_in + chunk * 8 : nullptr;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = (tid >> 3) + i * 32;
    int n;
    if (GATED) {
      n = n0 + (rr >> 5) * 16 + (rr & 15);
      n = n < n_out ? ((rr & 16) ? n_out + n : n) : -1;
    } else {
      n = n0 + rr < n_out ? n0 + rr : -1;
    }
    b_src[i] = n >= 0 ? we + (size_t)n * n_in + chunk * 8 : nullptr;
  }
  const int n_k = (n_in + TK - 1) / TK;
  auto load_stage = [&](int stage, int kt) {
    const int k0 = kt * TK;
    const bool kv = k0 + chunk * 8 + 8 <= n_in;
    const uint32_t a_base = smem_base + stage * (A_BYTES + B_BYTES), b_base = a_base + A_BYTES;
#pragma unroll
    for (int i = 0; i < MI; ++i) {
      const bool ok = kv && a_src[i] != nullptr;
      cp_async16(a_base + tile_offset((tid >> 3) + i * 32, chunk), ok ? a_src[i] + k0 : a, ok);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = kv && b_src[i] != nullptr;
      cp_async16(b_base + tile_offset((tid >> 3) + i * 32, chunk), ok ? b_src[i] + k0 : w, ok);
    }
  };
  float acc[MI][4][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;
  // whether any of this warp's rows holds a pair (the upper half of a ragged tile's warps often has none)
  const int mi_n = cnt > warp_m * (MI * 16) ? 1 : 0;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_k) load_stage(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < n_k; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (kt + STAGES - 1 < n_k) load_stage((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
    cp_async_commit();
    const uint32_t a_base = smem_base + (kt % STAGES) * (A_BYTES + B_BYTES), b_base = a_base + A_BYTES;
    if (mi_n == 0) continue;                       // none of the warp's rows holds a pair: it only copies
#pragma unroll
    for (int ks = 0; ks < TK / 16; ++ks) {
      uint32_t af[MI][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < MI; ++i) {
        const int row = warp_m * (MI * 16) + i * 16 + (lane & 15), ch = ks * 2 + (lane >> 4);
        ldmatrix_x4(a_base + tile_offset(row, ch), af[i][0], af[i][1], af[i][2], af[i][3]);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int row = warp_n * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int ch = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b_base + tile_offset(row, ch), bfr[2 * j][0], bfr[2 * j][1], bfr[2 * j + 1][0], bfr[2 * j + 1][1]);
      }
#pragma unroll
      for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bfr[j][0], bfr[j][1]);
    }
  }
  cp_async_wait<0>();
  // a thread holds pairs g and g + 8 and columns 2t, 2t + 1 of every 16 x 8 tile
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int i = 0; i < MI; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = warp_m * (MI * 16) + i * 16 + g + half * 8;
      if (m >= cnt) continue;
      if (GATED) {
        bf16* out = (bf16*)out_ + (size_t)(first + m) * n_out;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int n = n0 + warp_n * 16 + j * 8 + 2 * t + c;
            if (n < n_out)
              out[n] = __float2bfloat16(sb_glu_clamped(acc[i][j][half * 2 + c], acc[i][j + 2][half * 2 + c], limit, slope));
          }
      } else {
        float* out = (float*)out_ + (size_t)order[first + m] * n_out;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int n = n0 + warp_n * 32 + j * 8 + 2 * t + c;
            if (n < n_out) out[n] = acc[i][j][half * 2 + c];
          }
      }
    }
  }
}

template <int MI, bool GATED>
int launch_mma(const void* a, const void* w, const int32_t* order, const int32_t* meta, int tiles, int top, int n_out,
               int n_in, float limit, float slope, void* out, cudaStream_t stream) {
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_mma_kernel<MI, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         mma_smem(MI));
    if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "mixture of experts: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  const dim3 grid(tiles, (n_out + (GATED ? TN / 2 : TN) - 1) / (GATED ? TN / 2 : TN));
  sb_launch<SB_K_OTHER>(moe_gemm_mma_kernel<MI, GATED>, grid, dim3(MMA_THREADS), (size_t)mma_smem(MI), stream,
                        (const bf16*)a, (const bf16*)w, order, meta, top, n_out, n_in, limit, slope, out);
  return SB_OK;
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
  if (n_experts <= 1024)
    sb_launch<SB_K_ELEMENTWISE>(moe_route_warp_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, stream, logits, n_rows,
                                n_experts, top, ids, weights);
  else
    sb_launch<SB_K_ELEMENTWISE>(moe_route_kernel, dim3((n_rows + 127) / 128), dim3(128), 0, stream, logits, n_rows,
                                n_experts, top, ids, weights);
  SB_CHECK_LAUNCH("sb_moe_route");
  return SB_OK;
}

extern "C" int sb_moe_route_scored(const float* logits, const float* correction, int n_rows, int n_experts, int top,
                                   int n_groups, int keep_groups, int group_top, float scale, int renormalize,
                                   int32_t* ids, float* weights, cudaStream_t stream) {
  if (n_rows <= 0 || n_experts <= 0 || top <= 0 || top > n_experts || !logits || !ids || !weights)
    SB_FAIL(SB_ERR_ARG, "sb_moe_route_scored: rows=%d experts=%d top=%d", n_rows, n_experts, top);
  if (n_experts > ROUTE_MAX_EXPERTS)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_moe_route_scored: %d experts (at most %d)", n_experts, ROUTE_MAX_EXPERTS);
  if (n_groups < 1 || n_experts % n_groups || keep_groups < 1 || keep_groups > n_groups || group_top < 1)
    SB_FAIL(SB_ERR_ARG, "sb_moe_route_scored: %d groups of %d experts, %d kept, %d scores a group", n_groups, n_experts,
            keep_groups, group_top);
  if ((long long)keep_groups * (n_experts / n_groups) < top)
    SB_FAIL(SB_ERR_ARG, "sb_moe_route_scored: %d kept groups of %d experts cannot give %d choices", keep_groups,
            n_experts / n_groups, top);
  sb_launch<SB_K_ELEMENTWISE>(moe_route_scored_kernel, dim3((n_rows + ROUTE_WARPS - 1) / ROUTE_WARPS),
                              dim3(ROUTE_WARPS * 32), 0, stream, logits, correction, n_rows, n_experts, top, n_groups,
                              keep_groups, group_top, scale, renormalize, ids, weights);
  SB_CHECK_LAUNCH("sb_moe_route_scored");
  return SB_OK;
}

// Pairs of a tile for these sizes: 32 on the plain path; on tensor cores 128 when the experts
// get about a tile of that size each, else 64.  A choice of speed only: results are the same.
extern "C" int sb_moe_tile_rows(int dtype, int n_pairs, int n_experts, int ff, int width) {
  if (dtype != SB_BF16 || ff % 8 || width % 8) return BM;
  return n_pairs >= 96 * (long long)n_experts ? 128 : 64;
}

extern "C" int sb_moe_max_tiles(int n_pairs, int n_experts, int tile_rows) {
  return (n_pairs + tile_rows - 1) / tile_rows + n_experts;
}

extern "C" int sb_moe_group(const int32_t* ids, int n_pairs, int n_experts, int tile_rows, int32_t* order,
                            int32_t* meta, cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0 || !ids || !order || !meta || (tile_rows != BM && tile_rows != 64 && tile_rows != 128))
    SB_FAIL(SB_ERR_ARG, "sb_moe_group: pairs=%d experts=%d tile_rows=%d", n_pairs, n_experts, tile_rows);
  const size_t smem = (size_t)3 * n_experts * sizeof(int32_t);
  if (smem > 48 * 1024) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_moe_group: %d experts", n_experts);
  sb_launch<SB_K_ELEMENTWISE>(moe_group_kernel, dim3(1), dim3(1024), smem, stream, ids, n_pairs, n_experts, tile_rows,
                              order, meta);
  SB_CHECK_LAUNCH("sb_moe_group");
  return SB_OK;
}

extern "C" int sb_moe_up(const void* a, int a_dtype, const void* w, int w_dtype, const int32_t* order,
                         const int32_t* meta, int n_pairs, int n_experts, int tile_rows, int top, int ff, int width,
                         float limit, float slope, void* act, cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0 || top <= 0 || ff <= 0 || width <= 0 || !a || !w || !order || !meta || !act)
    SB_FAIL(SB_ERR_ARG, "sb_moe_up: pairs=%d experts=%d top=%d ff=%d width=%d", n_pairs, n_experts, top, ff, width);
  if (!sb_valid_dtype(a_dtype) || a_dtype != w_dtype) SB_FAIL(SB_ERR_ARG, "sb_moe_up: dtype codes %d %d", a_dtype, w_dtype);
  if (tile_rows != sb_moe_tile_rows(a_dtype, n_pairs, n_experts, ff, width))
    SB_FAIL(SB_ERR_ARG, "sb_moe_up: tiles of %d pairs are not what sb_moe_tile_rows gives", tile_rows);
  const int tiles = sb_moe_max_tiles(n_pairs, n_experts, tile_rows);
  if (tile_rows != BM) {
    if (((uintptr_t)a | (uintptr_t)w) & 15) SB_FAIL(SB_ERR_ARG, "sb_moe_up: operands must be 16-byte aligned");
    const int rc = tile_rows == 128 ? launch_mma<4, true>(a, w, order, meta, tiles, top, ff, width, limit, slope, act, stream)
                                    : launch_mma<2, true>(a, w, order, meta, tiles, top, ff, width, limit, slope, act, stream);
    if (rc) return rc;
    SB_CHECK_LAUNCH("sb_moe_up");
    return SB_OK;
  }
  const dim3 grid(tiles, (ff + BN - 1) / BN);
  SB_DISPATCH_DTYPE(a_dtype, T, {
    sb_launch<SB_K_OTHER>(moe_gemm_kernel<T, T, true>, grid, dim3(GEMM_THREADS), 0, stream, (const T*)a, (const T*)w, order,
                          meta, top, ff, width, limit, slope, act);
  });
  SB_CHECK_LAUNCH("sb_moe_up");
  return SB_OK;
}

extern "C" int sb_moe_down(const void* act, int a_dtype, const void* w, int w_dtype, const int32_t* order,
                           const int32_t* meta, int n_pairs, int n_experts, int tile_rows, int top, int width, int ff,
                           float* pair_out, cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0 || top <= 0 || ff <= 0 || width <= 0 || !act || !w || !order || !meta || !pair_out)
    SB_FAIL(SB_ERR_ARG, "sb_moe_down: pairs=%d experts=%d top=%d ff=%d width=%d", n_pairs, n_experts, top, ff, width);
  if (!sb_valid_dtype(a_dtype) || a_dtype != w_dtype) SB_FAIL(SB_ERR_ARG, "sb_moe_down: dtype codes %d %d", a_dtype, w_dtype);
  if (tile_rows != sb_moe_tile_rows(a_dtype, n_pairs, n_experts, ff, width))
    SB_FAIL(SB_ERR_ARG, "sb_moe_down: tiles of %d pairs are not what sb_moe_tile_rows gives", tile_rows);
  const int tiles = sb_moe_max_tiles(n_pairs, n_experts, tile_rows);
  if (tile_rows != BM) {
    if (((uintptr_t)act | (uintptr_t)w) & 15) SB_FAIL(SB_ERR_ARG, "sb_moe_down: operands must be 16-byte aligned");
    const int rc = tile_rows == 128
                       ? launch_mma<4, false>(act, w, order, meta, tiles, top, width, ff, 0.0f, 0.0f, pair_out, stream)
                       : launch_mma<2, false>(act, w, order, meta, tiles, top, width, ff, 0.0f, 0.0f, pair_out, stream);
    if (rc) return rc;
    SB_CHECK_LAUNCH("sb_moe_down");
    return SB_OK;
  }
  const dim3 grid(tiles, (width + BN - 1) / BN);
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
