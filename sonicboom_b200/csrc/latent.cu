// Kernels of attention over a cached low-rank latent.
//
// The cache holds, per token, the normed latent c (rank values) and one rotated key part kr
// (rd values) that all heads share.  With per-head matrices Uk [dim, rank] and Uv [vdim, rank]
// the score of head h is  q_h . (Uk_h c) + qr_h . kr = (Uk_h^T q_h) . c + qr_h . kr  and the
// head's output is  Uv_h (sum_j p_j c_j):  attention with ONE key/value head whose key row is
// [c | kr] and whose value row is c, between a product per head before it (q_h -> Uk_h^T q_h) and
// one after it.  So the paged attention kernels run unchanged on a cache entry with one head of
// size rank + rd (the value plane carries c and zeros), and this file supplies the rest:
//
//   sb_latent_prep:  finishes the fused projection row [q heads | latent | key part]: RMS norm
//                    of the latent, rotation of every head's rd part and of the key part, the
//                    cache write, and the rotated query parts into the wide query rows;
//   sb_head_linear:  out[r, h, :] = W[h] in[r, h, :], a small product per head over strided rows.
//
// Rotation: of a rotated vector, elements 2i and 2i + 1 (interleaved pairs) or i and i + rot/2
// (i < rot / 2) turn by the angle float(pos) * inv_freq[i], cosine and sine times `rot_scale`;
// elements from `rot` on pass unchanged.
#include "common.cuh"

namespace {

constexpr int PREP_THREADS = 128;
constexpr int MAX_ROT_PAIRS = 512;

template <typename TW, typename TC, typename TQ>
__global__ void __launch_bounds__(PREP_THREADS)
latent_prep_kernel(const float* proj, int ld, int n_heads, int dim, int rd, int rank, int rot,
                   const float* __restrict__ inv_freq, const int32_t* row_seq, const int32_t* row_pos,
                   const int32_t* page_off, const int32_t* page_ids, int page_size,
                   const TW* __restrict__ cnorm, float eps, TC* cache, TQ* q_wide, int q_group, int has_kv,
                   const float* kv, int kv_ld, int interleaved, float rot_scale) {
  __shared__ float cs[MAX_ROT_PAIRS], sn[MAX_ROT_PAIRS];
  __shared__ float red[PREP_THREADS / 32 + 1];
  sb_pdl_launch();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = row_pos[t];
  const int half = rot >> 1;
  for (int i = tid; i < half; i += PREP_THREADS) {
    const float theta = (float)pos * inv_freq[i];
    cs[i] = cosf(theta) * rot_scale;
    sn[i] = sinf(theta) * rot_scale;
  }
  // element d of a rotated vector v: pairs (2i, 2i + 1), or (i, i + rot/2) when not interleaved
  auto turned = [&](const float* v, int d) {
    if (d >= rot) return v[d];
    if (interleaved) {
      const int i = d >> 1;
      return (d & 1) ? sb_rot_hi(v[d - 1], v[d], cs[i], sn[i]) : sb_rot_lo(v[d], v[d + 1], cs[i], sn[i]);
    }
    return d < half ? sb_rot_lo(v[d], v[d + half], cs[d], sn[d])
                    : sb_rot_hi(v[d - half], v[d], cs[d - half], sn[d - half]);
  };
  int page = -1;
  if (has_kv) {
    const int seq = row_seq[t];
    const int first = page_off[seq], n = page_off[seq + 1] - first;
    const int i = pos / page_size;
    page = (pos >= 0 && i < n) ? page_ids[first + i] : -1;
  }
  __syncthreads();
  sb_pdl_wait();
  const float* src = proj + (size_t)t * ld;
  const int hw = dim + rd, wide = rank + rd;
  // the rotated part of every query head, into the tail of its wide query row
  for (int e = tid; e < n_heads * rd; e += PREP_THREADS) {
    const int h = e / rd, d = e % rd;
    const float* qr = src + (size_t)h * hw + dim;
    const float v = turned(qr, d);
    // wide query rows lie [head group][row][head in group]: one group is [row][head]
    q_wide[(((size_t)(h / q_group) * gridDim.x + t) * q_group + h % q_group) * wide + rank + d] = sb_from_f32<TQ>(v);
  }
  if (!has_kv) return;
  // the latent and the shared key part: after the heads in the same row, or rows of their own
  const float* lat = kv ? kv + (size_t)t * kv_ld : src + (size_t)n_heads * hw;
  float s = 0.0f;
  for (int i = tid; i < rank; i += PREP_THREADS) s = fmaf(lat[i], lat[i], s);
  s = sb_warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int i = 0; i < PREP_THREADS / 32; ++i) total += red[i];
    red[PREP_THREADS / 32] = 1.0f / sqrtf(total / (float)rank + eps);
  }
  __syncthreads();
  if (page < 0) return;               // no page of its own at that position: nothing is written
  const float inv = red[PREP_THREADS / 32];
  TC* krow = cache + (((size_t)page * 2) * page_size + pos % page_size) * wide;
  TC* vrow = cache + (((size_t)page * 2 + 1) * page_size + pos % page_size) * wide;
  for (int i = tid; i < rank; i += PREP_THREADS) {
    const TC c = sb_from_f32<TC>((lat[i] * inv) * sb_to_f32<TW>(cnorm[i]));
    krow[i] = c;
    vrow[i] = c;
  }
  const float* kr = lat + rank;
  for (int d = tid; d < rd; d += PREP_THREADS) {
    krow[rank + d] = sb_from_f32<TC>(turned(kr, d));
    vrow[rank + d] = sb_from_f32<TC>(0.0f);
  }
}

// out[r, h, n] = sum_k in[r, h, k] * W[h, n, k], k ascending in float32.  32 x 64 outputs a block,
// 2 x 4 a thread, K in chunks of 16 through shared memory.
constexpr int HL_BM = 32, HL_BN = 64, HL_BK = 16, HL_THREADS = 256;

template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(HL_THREADS)
head_linear_kernel(const TI* in, size_t in_ld, size_t in_hs, const TW* __restrict__ W, int n_rows,
                   int N, int K, TO* out, size_t out_ld, size_t out_hs) {
  __shared__ float As[HL_BK][HL_BM + 1];
  __shared__ float Ws[HL_BK][HL_BN + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const int h = blockIdx.z, r0 = blockIdx.x * HL_BM, n0 = blockIdx.y * HL_BN;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const TI* a = in + (size_t)h * in_hs;
  const TW* w = W + (size_t)h * N * K;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += HL_BK) {
    for (int e = tid; e < HL_BM * HL_BK; e += HL_THREADS) {
      const int r = e / HL_BK, k = e % HL_BK;
      As[k][r] = (r0 + r < n_rows && k0 + k < K) ? sb_to_f32<TI>(a[(size_t)(r0 + r) * in_ld + k0 + k]) : 0.0f;
    }
    for (int e = tid; e < HL_BN * HL_BK; e += HL_THREADS) {
      const int n = e / HL_BK, k = e % HL_BK;
      Ws[k][n] = (n0 + n < N && k0 + k < K) ? sb_to_f32<TW>(w[(size_t)(n0 + n) * K + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HL_BK; ++k) {
      const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Ws[k][tx + 16 * j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + ty * 2 + i;
    if (r >= n_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n < N) out[(size_t)r * out_ld + (size_t)h * out_hs + n] = sb_from_f32<TO>(acc[i][j]);
    }
  }
}

// The same on tensor cores for bfloat16 weights and outputs at many rows: mma.sync m16n8k16 with
// float32 accumulation, operands read from global memory straight into fragments (a float32
// input is rounded to bfloat16 on the way, as every product's activation is).  A warp owns 32
// rows x 64 outputs of one head; K is a multiple of 16, N even, and every offset even.
constexpr int HM_WARPS = 4, HM_ROWS = 32 * HM_WARPS, HM_COLS = 64;

__device__ __forceinline__ uint32_t pack2(const float* p) {
  const float2 f = *reinterpret_cast<const float2*>(p);
  __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<uint32_t*>(&b);
}
__device__ __forceinline__ uint32_t pack2(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }

template <typename TI>
__global__ void __launch_bounds__(HM_WARPS * 32)
head_linear_mma_kernel(const TI* in, size_t in_ld, size_t in_hs, const __nv_bfloat16* __restrict__ W, int n_rows,
                       int N, int K, __nv_bfloat16* out, size_t out_ld, size_t out_hs) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int h = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int r0 = blockIdx.x * HM_ROWS + warp * 32, n0 = blockIdx.y * HM_COLS;
  const TI* a = in + (size_t)h * in_hs;
  const __nv_bfloat16* w = W + (size_t)h * N * K;
  float acc[2][8][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t af[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const int ra = r0 + mt * 16 + gid, rb = ra + 8;
      const TI* pa = a + (size_t)ra * in_ld + k0 + tig * 2;
      const TI* pb = a + (size_t)rb * in_ld + k0 + tig * 2;
      af[mt][0] = ra < n_rows ? pack2(pa) : 0u;
      af[mt][1] = rb < n_rows ? pack2(pb) : 0u;
      af[mt][2] = ra < n_rows ? pack2(pa + 8) : 0u;
      af[mt][3] = rb < n_rows ? pack2(pb + 8) : 0u;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j * 8 + gid;
      uint32_t b0 = 0u, b1 = 0u;
      if (n < N) {
        const __nv_bfloat16* pw = w + (size_t)n * K + k0 + tig * 2;
        b0 = pack2(pw);
        b1 = pack2(pw + 8);
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(acc[mt][j][0]), "+f"(acc[mt][j][1]), "+f"(acc[mt][j][2]), "+f"(acc[mt][j][3])
                     : "r"(af[mt][0]), "r"(af[mt][1]), "r"(af[mt][2]), "r"(af[mt][3]), "r"(b0), "r"(b1));
    }
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j * 8 + tig * 2;
      if (n >= N) continue;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = r0 + mt * 16 + gid + half * 8;
        if (r < n_rows)
          *reinterpret_cast<__nv_bfloat162*>(out + (size_t)r * out_ld + (size_t)h * out_hs + n) =
              __floats2bfloat162_rn(acc[mt][j][half * 2], acc[mt][j][half * 2 + 1]);
      }
    }
}

// The same for at most HS_ROWS rows (decode): a warp per output column of a head streams that
// column's weights once, the lanes share out K, and the rows' sums meet by shuffles.
constexpr int HS_ROWS = 8, HS_WARPS = 8;

template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(HS_WARPS * 32)
head_linear_skinny_kernel(const TI* in, size_t in_ld, size_t in_hs, const TW* __restrict__ W, int n_rows,
                          int N, int K, TO* out, size_t out_ld, size_t out_hs) {
  sb_pdl_launch();
  const int h = blockIdx.y, lane = threadIdx.x & 31;
  const int n = blockIdx.x * HS_WARPS + (threadIdx.x >> 5);
  if (n >= N) return;
  const TW* w = W + ((size_t)h * N + n) * K;
  const TI* a = in + (size_t)h * in_hs;
  float acc[HS_ROWS] = {};
  sb_pdl_wait();
  for (int k = lane; k < K; k += 32) {
    const float wv = sb_to_f32<TW>(w[k]);
#pragma unroll
    for (int r = 0; r < HS_ROWS; ++r)
      if (r < n_rows) acc[r] = fmaf(wv, sb_to_f32<TI>(a[(size_t)r * in_ld + k]), acc[r]);
  }
#pragma unroll
  for (int r = 0; r < HS_ROWS; ++r) {
    const float v = sb_warp_sum(acc[r]);
    if (lane == 0 && r < n_rows) out[(size_t)r * out_ld + (size_t)h * out_hs + n] = sb_from_f32<TO>(v);
  }
}

}  // namespace

extern "C" int sb_latent_prep(const float* proj, int n_rows, int n_heads, int dim, int rd, int rank,
                              int rot, const float* inv_freq, const int32_t* row_seq,
                              const int32_t* row_pos, const int32_t* page_off, const int32_t* page_ids,
                              int page_size, const void* cnorm, int cnorm_dtype, float eps, void* cache,
                              int cache_dtype, void* q_wide, int q_dtype, int q_group, int has_kv,
                              const float* kv, int kv_ld, int interleaved, float rot_scale, cudaStream_t stream) {
  if (kv && (!has_kv || kv_ld < rank + rd))
    SB_FAIL(SB_ERR_ARG, "sb_latent_prep: latent rows of their own need a cache write and %d values a row", rank + rd);
  if (q_group <= 0 || n_heads % q_group)
    SB_FAIL(SB_ERR_ARG, "sb_latent_prep: groups of %d heads do not divide %d heads", q_group, n_heads);
  if (n_rows <= 0 || n_heads <= 0 || dim < 0 || rd < 0 || rank <= 0 || !proj || !q_wide || !row_pos)
    SB_FAIL(SB_ERR_ARG, "sb_latent_prep: rows=%d heads=%d dim=%d rd=%d rank=%d", n_rows, n_heads, dim, rd, rank);
  if (rot < 0 || rot % 2 || rot > rd || rot / 2 > MAX_ROT_PAIRS)
    SB_FAIL(SB_ERR_ARG, "sb_latent_prep: %d rotated dimensions of %d (even, at most %d)", rot, rd, 2 * MAX_ROT_PAIRS);
  if (rot > 0 && !inv_freq) SB_FAIL(SB_ERR_ARG, "sb_latent_prep: no frequency table");
  if (has_kv && (!cache || !cnorm || !row_seq || !page_off || !page_ids || page_size <= 0))
    SB_FAIL(SB_ERR_ARG, "sb_latent_prep: a cache write needs the cache, its norm weight and the page tables");
  if (!sb_valid_dtype(q_dtype) || (has_kv && (!sb_valid_dtype(cache_dtype) || !sb_valid_dtype(cnorm_dtype))))
    SB_FAIL(SB_ERR_ARG, "sb_latent_prep: dtype codes %d %d %d", q_dtype, cache_dtype, cnorm_dtype);
  const int ld = n_heads * (dim + rd) + (has_kv && !kv ? rank + rd : 0);
  SB_DISPATCH_DTYPE(has_kv ? cnorm_dtype : SB_F32, TW, {
    SB_DISPATCH_DTYPE(has_kv ? cache_dtype : SB_F32, TC, {
      SB_DISPATCH_DTYPE(q_dtype, TQ, {
        sb_launch<SB_K_ELEMENTWISE>(latent_prep_kernel<TW, TC, TQ>, dim3(n_rows), dim3(PREP_THREADS), 0, stream,
                                    proj, ld, n_heads, dim, rd, rank, rot, inv_freq, row_seq, row_pos, page_off,
                                    page_ids, page_size, (const TW*)cnorm, eps, (TC*)cache, (TQ*)q_wide, q_group, has_kv,
                                    kv, kv_ld, interleaved, rot_scale);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_latent_prep");
  return SB_OK;
}

extern "C" int sb_head_linear(const void* in, int in_dtype, size_t in_ld, size_t in_hs, const void* W,
                              int w_dtype, int n_rows, int n_heads, int N, int K, void* out, int out_dtype,
                              size_t out_ld, size_t out_hs, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || N <= 0 || K <= 0 || !in || !W || !out)
    SB_FAIL(SB_ERR_ARG, "sb_head_linear: rows=%d heads=%d N=%d K=%d", n_rows, n_heads, N, K);
  if (n_heads > 65535 || (N + HL_BN - 1) / HL_BN > 65535)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_head_linear: %d heads, %d outputs", n_heads, N);
  if (!sb_valid_dtype(in_dtype) || !sb_valid_dtype(w_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_head_linear: dtype codes %d %d %d", in_dtype, w_dtype, out_dtype);
  const dim3 grid((n_rows + HL_BM - 1) / HL_BM, (N + HL_BN - 1) / HL_BN, n_heads);
  const dim3 skinny((N + HS_WARPS - 1) / HS_WARPS, n_heads);
  const size_t in_size = in_dtype == SB_F32 ? 4 : 2;
  const bool mma = n_rows > HS_ROWS && w_dtype == SB_BF16 && out_dtype == SB_BF16 && K % 16 == 0 && N % 2 == 0 &&
                   in_ld % 2 == 0 && in_hs % 2 == 0 && out_ld % 2 == 0 && out_hs % 2 == 0 &&
                   (uintptr_t)in % (2 * in_size) == 0 && (uintptr_t)W % 4 == 0 && (uintptr_t)out % 4 == 0;
  if (mma) {
    const dim3 grid_mma((n_rows + HM_ROWS - 1) / HM_ROWS, (N + HM_COLS - 1) / HM_COLS, n_heads);
    if (in_dtype == SB_F32)
      sb_launch<SB_K_OTHER>(head_linear_mma_kernel<float>, grid_mma, dim3(HM_WARPS * 32), 0, stream, (const float*)in,
                            in_ld, in_hs, (const __nv_bfloat16*)W, n_rows, N, K, (__nv_bfloat16*)out, out_ld, out_hs);
    else
      sb_launch<SB_K_OTHER>(head_linear_mma_kernel<__nv_bfloat16>, grid_mma, dim3(HM_WARPS * 32), 0, stream,
                            (const __nv_bfloat16*)in, in_ld, in_hs, (const __nv_bfloat16*)W, n_rows, N, K,
                            (__nv_bfloat16*)out, out_ld, out_hs);
    SB_CHECK_LAUNCH("sb_head_linear");
    return SB_OK;
  }
  SB_DISPATCH_DTYPE(in_dtype, TI, {
    SB_DISPATCH_DTYPE(w_dtype, TW, {
      SB_DISPATCH_DTYPE(out_dtype, TO, {
        if (n_rows <= HS_ROWS)
          sb_launch<SB_K_OTHER>(head_linear_skinny_kernel<TI, TW, TO>, skinny, dim3(HS_WARPS * 32), 0, stream,
                                (const TI*)in, in_ld, in_hs, (const TW*)W, n_rows, N, K, (TO*)out, out_ld, out_hs);
        else
          sb_launch<SB_K_OTHER>(head_linear_kernel<TI, TW, TO>, grid, dim3(HL_THREADS), 0, stream, (const TI*)in, in_ld,
                                in_hs, (const TW*)W, n_rows, N, K, (TO*)out, out_ld, out_hs);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_head_linear");
  return SB_OK;
}
