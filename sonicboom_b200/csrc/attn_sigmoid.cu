// Attention whose weights are not normalised over the keys: the weight of a visible key is
// sigmoid(cap(q . k * scale) + bias_h), cap(s) = softcap * tanh(s / softcap) (softcap 0: none), a
// number per query head added to the score, and out = sum_j weight_j v_j.  Visible for the query
// at absolute position i: key j <= i with i - j < window (window 0: every earlier key) or
// j < keep_first, the first tokens of a sequence that a window keeps.
//
// The plain kernel: one block per (row, query head), float32 arithmetic, keys in ascending order
// in chunks at absolute positions, so a sum depends on the positions only, not on the batch or on
// where the pages lie.  It reads the same paged cache as the softmax kernels.
//
// The tensor-core kernel (bfloat16, head sizes 64 and 128, pages of 64 keys): mma.sync m16n8k16
// for q . k and for weights . v, float32 scores, weights and sums.  For one sequence and one
// key/value head the rows are the pairs (new token, query head of the group), 128 to a block, 16
// to a warp; key tiles of one cache page come in ascending order through a double-buffered
// cp.async pipeline: the pages of the kept first keys that lie before the window, then the
// window's.  A weight is rounded to bfloat16 only as the operand of the second product.  Tiles
// lie at absolute positions and a key that a row does not see adds an exact zero, so a row's sum
// does not depend on the rows around it.  With at most 16 rows for a sequence and key/value head
// (decoding) a block's tiles are two pages wide and its 8 warps share every tile's keys.
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

// ------------------------------------------------------------------------------ tensor cores
typedef __nv_bfloat16 bf16;
constexpr int KT = 64;                 // keys per tile = cache page size
constexpr int TC_BM = 128, TC_THREADS = TC_BM / 16 * 32;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
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
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct SigmoidParams {
  const bf16* q;               // [rows, n_q_heads, HD]
  bf16* out;                   // [rows, n_q_heads * HD]
  const int32_t* seq_row0;     // [n_seqs + 1]
  const int32_t* seq_pos0;     // [n_seqs] position of a sequence's first new row
  const int32_t* page_off;     // [n_seqs + 1]
  const int32_t* page_ids;
  const bf16* cache;           // [page][k|v][kv head][KT][HD]
  int n_q_heads, n_kv_heads, window, keep_first;
  float scale, softcap;
  const float* head_bias;      // [n_q_heads] or null
};

template <int HD>
constexpr int tc_smem() { return (TC_BM + 4 * KT) * (HD + 8) * 2; }

template <int HD>
__global__ void __launch_bounds__(TC_THREADS, 2) attn_sigmoid_mma_kernel(const SigmoidParams p) {
  constexpr int LDS = HD + 8;          // shared-memory row stride: an odd number of 16-byte chunks
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t qs = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t kv0 = qs + TC_BM * LDS * 2;                  // K0, V0, K1, V1
  sb_pdl_launch();
  sb_pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blockIdx.x = (block of rows, key/value head), heads fastest and the last rows first
  const int b = blockIdx.z, kvh = blockIdx.x % p.n_kv_heads;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int row0 = p.seq_row0[b], n_new = p.seq_row0[b + 1] - row0, pos0 = p.seq_pos0[b];
  const int R = n_new * G;
  const int r_base = (int)(gridDim.x / p.n_kv_heads - 1 - blockIdx.x / p.n_kv_heads) * TC_BM;
  if (r_base >= R) return;
  const int r_last = min(R, r_base + TC_BM) - 1;
  if (pos0 < 0 || (pos0 + n_new - 1) / KT >= p.page_off[b + 1] - p.page_off[b]) {
    // positions without pages in the sequence's own list: nothing is read, zeros are written
    for (int idx = tid; idx < (r_last - r_base + 1) * HD; idx += TC_THREADS) {
      const int r = r_base + idx / HD;
      p.out[((size_t)(row0 + r / G) * p.n_q_heads + kvh * G + r % G) * HD + idx % HD] = __float2bfloat16(0.0f);
    }
    return;
  }
  const int32_t* pages = p.page_ids + p.page_off[b];
  auto load_tile = [&](int stage, int page) {
    const uint32_t ks = kv0 + stage * 2 * KT * LDS * 2, vs = ks + KT * LDS * 2;
    const bf16* kbase = p.cache + (((size_t)page * 2) * p.n_kv_heads + kvh) * (size_t)(KT * HD);
    const bf16* vbase = kbase + (size_t)p.n_kv_heads * (KT * HD);
    for (int idx = tid; idx < KT * (HD / 8); idx += TC_THREADS) {
      const int row = idx / (HD / 8), ch = idx % (HD / 8);
      const uint32_t off = (uint32_t)(row * LDS + ch * 8) * 2;
      cp_async16(ks + off, kbase + row * HD + ch * 8, true);
      cp_async16(vs + off, vbase + row * HD + ch * 8, true);
    }
  };
  for (int idx = tid; idx < TC_BM * (HD / 8); idx += TC_THREADS) {
    const int row = idx / (HD / 8), ch = idx % (HD / 8);
    const int r = r_base + row;
    const bool valid = r < R;
    const int t = valid ? r / G : 0, g = valid ? r % G : 0;
    cp_async16(qs + (uint32_t)(row * LDS + ch * 8) * 2,
               p.q + ((size_t)(row0 + t) * p.n_q_heads + kvh * G + g) * HD + ch * 8, valid);
  }
  // the block's tiles in ascending order: those of kept first keys before the window, then the window's
  const int p_lo = pos0 + r_base / G, p_hi = pos0 + r_last / G;
  const int tile_lo = (p.window > 0 ? max(0, p_lo - p.window + 1) : 0) / KT, tile_hi = p_hi / KT;
  const int n_kept = p.window > 0 && p.keep_first > 0 ? min((p.keep_first - 1) / KT + 1, tile_lo) : 0;
  const int n_tiles = n_kept + tile_hi - tile_lo + 1;
  auto tile_at = [&](int i) { return i < n_kept ? i : tile_lo + i - n_kept; };
  load_tile(0, pages[tile_at(0)]);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // the query fragments are read from shared memory again for every tile: registers for two blocks an SM
  const uint32_t q_frag = qs + (uint32_t)((warp * 16 + (lane & 15)) * LDS + (lane >> 4) * 8) * 2;
  const int ra = r_base + warp * 16 + (lane >> 2), rb = ra + 8;
  const int pos_a = ra < R ? pos0 + ra / G : -1, pos_b = rb < R ? pos0 + rb / G : -1;
  const float pb_a = p.head_bias && ra < R ? p.head_bias[kvh * G + ra % G] : 0.0f;
  const float pb_b = p.head_bias && rb < R ? p.head_bias[kvh * G + rb % G] : 0.0f;
  const bool active = r_base + warp * 16 < R;              // a warp without rows only helps to copy
  const float two_inv_cap = p.softcap > 0.0f ? 2.0f / p.softcap : 0.0f;
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    const uint32_t ks = kv0 + stage * 2 * KT * LDS * 2, vs = ks + KT * LDS * 2;
    if (it + 1 < n_tiles) {
      load_tile(stage ^ 1, pages[tile_at(it + 1)]);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = tile_at(it) * KT;
    // a warp none of whose rows sees a key of the tile adds only zeros: it skips the tile
    const int w_lo = pos0 + (r_base + warp * 16) / G, w_hi = pos0 + min(R - 1, r_base + warp * 16 + 15) / G;
    const bool any = active && key0 <= w_hi &&
                     (p.window == 0 || key0 + KT - 1 > w_lo - p.window || key0 < p.keep_first);
    if (any) {
      float s[KT / 8][4];
#pragma unroll
      for (int j = 0; j < KT / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[j][i] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t qf[4];
        ldmatrix_x4(q_frag + kk * 32, qf[0], qf[1], qf[2], qf[3]);
#pragma unroll
        for (int j = 0; j < KT / 16; ++j) {
          const int row = j * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int col = kk * 16 + ((lane >> 3) & 1) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(ks + (uint32_t)(row * LDS + col) * 2, b0, b1, b2, b3);
          mma_bf16(s[2 * j], qf, b0, b1);
          mma_bf16(s[2 * j + 1], qf, b2, b3);
        }
      }
      const int t = lane & 3;
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = key0 + j * 8 + 2 * t + (i & 1);
          const int pos = (i < 2) ? pos_a : pos_b;
          const bool seen = key <= pos && (p.window == 0 || pos - key < p.window || key < p.keep_first);
          float v = s[j][i] * p.scale;
          // cap * tanh(v / cap) = cap * (1 - 2 / (exp(2 v / cap) + 1))
          if (p.softcap > 0.0f) v = p.softcap * (1.0f - __fdividef(2.0f, __expf(fminf(v * two_inv_cap, 80.0f)) + 1.0f));
          v += (i < 2) ? pb_a : pb_b;
          s[j][i] = seen ? __fdividef(1.0f, 1.0f + __expf(fminf(-v, 80.0f))) : 0.0f;
        }
      }
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dj = 0; dj < HD / 16; ++dj) {
          const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int col = dj * 16 + (lane >> 4) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vs + (uint32_t)(row * LDS + col) * 2, b0, b1, b2, b3);
          mma_bf16(o[2 * dj], a, b0, b1);
          mma_bf16(o[2 * dj + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  const int t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? rb : ra;
    if (r >= R) continue;
    bf16* dst = p.out + ((size_t)(row0 + r / G) * p.n_q_heads + kvh * G + r % G) * HD;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t4) = pack_bf16(o[j][half * 2], o[j][half * 2 + 1]);
  }
}

// At most 16 rows for a sequence and key/value head (decoding): one block, whose tiles are two
// pages (128 keys) wide; each of the 8 warps takes 16 keys of every tile for all rows, and the
// warps' sums are added in warp order at the end.
constexpr int DEC_ROWS = 16, DEC_KEYS = 2 * KT, DEC_STAGES = 3;     // two tiles in flight beside the one in work
template <int HD>
constexpr int dec_smem() { return (DEC_ROWS + DEC_STAGES * 2 * DEC_KEYS) * (HD + 8) * 2; }

template <int HD>
__global__ void __launch_bounds__(TC_THREADS) attn_sigmoid_mma_decode_kernel(const SigmoidParams p) {
  constexpr int LDS = HD + 8;
  static_assert(TC_THREADS / 32 * 16 == DEC_KEYS, "a warp for every 16 keys of a tile");
  static_assert(TC_THREADS / 32 * DEC_ROWS * HD * 4 <= DEC_STAGES * 2 * DEC_KEYS * LDS * 2, "the warps' sums fit the tiles' space");
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t qs = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t kv0 = qs + DEC_ROWS * LDS * 2;               // K and V of 128 keys for each stage
  sb_pdl_launch();
  sb_pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, kvh = blockIdx.x;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int row0 = p.seq_row0[b], n_new = p.seq_row0[b + 1] - row0, pos0 = p.seq_pos0[b];
  const int R = n_new * G;
  if (R <= 0) return;
  if (pos0 < 0 || (pos0 + n_new - 1) / KT >= p.page_off[b + 1] - p.page_off[b]) {
    for (int idx = tid; idx < R * HD; idx += TC_THREADS)
      p.out[((size_t)(row0 + idx / HD / G) * p.n_q_heads + kvh * G + idx / HD % G) * HD + idx % HD] = __float2bfloat16(0.0f);
    return;
  }
  const int32_t* pages = p.page_ids + p.page_off[b];
  const int p_hi = pos0 + n_new - 1;
  const int tile_lo = (p.window > 0 ? max(0, pos0 - p.window + 1) : 0) / KT, tile_hi = p_hi / KT;
  const int n_kept = p.window > 0 && p.keep_first > 0 ? min((p.keep_first - 1) / KT + 1, tile_lo) : 0;
  const int n_pages = n_kept + tile_hi - tile_lo + 1, n_tiles = (n_pages + 1) / 2;
  auto page_at = [&](int i) { return i < n_kept ? i : tile_lo + i - n_kept; };
  auto load_tile = [&](int stage, int it) {
    const uint32_t ks = kv0 + stage * 2 * DEC_KEYS * LDS * 2, vs = ks + DEC_KEYS * LDS * 2;
    for (int idx = tid; idx < DEC_KEYS * (HD / 8); idx += TC_THREADS) {
      const int row = idx / (HD / 8), ch = idx % (HD / 8);
      const int pi = 2 * it + row / KT;
      const bool ok = pi < n_pages;                            // an odd last page: zeros beside it
      const bf16* kbase = p.cache + (((size_t)(ok ? pages[page_at(pi)] : 0) * 2) * p.n_kv_heads + kvh) * (size_t)(KT * HD);
      const bf16* vbase = kbase + (size_t)p.n_kv_heads * (KT * HD);
      const uint32_t off = (uint32_t)(row * LDS + ch * 8) * 2;
      cp_async16(ks + off, kbase + (row % KT) * HD + ch * 8, ok);
      cp_async16(vs + off, vbase + (row % KT) * HD + ch * 8, ok);
    }
  };
  for (int idx = tid; idx < DEC_ROWS * (HD / 8); idx += TC_THREADS) {
    const int row = idx / (HD / 8), ch = idx % (HD / 8);
    const bool valid = row < R;
    const int t = valid ? row / G : 0, g = valid ? row % G : 0;
    cp_async16(qs + (uint32_t)(row * LDS + ch * 8) * 2,
               p.q + ((size_t)(row0 + t) * p.n_q_heads + kvh * G + g) * HD + ch * 8, valid);
  }
  cp_async_commit();                                           // the query rows: a group of their own
#pragma unroll
  for (int st = 0; st < DEC_STAGES - 1; ++st) {
    if (st < n_tiles) load_tile(st, st);
    cp_async_commit();
  }
  cp_async_wait<DEC_STAGES - 1>();
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const int row = lane & 15, col = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qs + (uint32_t)(row * LDS + col) * 2, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  const int ra = lane >> 2, rb = ra + 8;
  const int pos_a = ra < R ? pos0 + ra / G : -1, pos_b = rb < R ? pos0 + rb / G : -1;
  const float pb_a = p.head_bias && ra < R ? p.head_bias[kvh * G + ra % G] : 0.0f;
  const float pb_b = p.head_bias && rb < R ? p.head_bias[kvh * G + rb % G] : 0.0f;
  const float two_inv_cap = p.softcap > 0.0f ? 2.0f / p.softcap : 0.0f;
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;
  const int krow0 = warp * 16;                                 // this warp's keys of every tile
  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % DEC_STAGES;
    const uint32_t ks = kv0 + stage * 2 * DEC_KEYS * LDS * 2, vs = ks + DEC_KEYS * LDS * 2;
    cp_async_wait<DEC_STAGES - 2>();
    __syncthreads();          // the tile has landed, and every warp is done with the stage that is filled next
    if (it + DEC_STAGES - 1 < n_tiles) load_tile((it + DEC_STAGES - 1) % DEC_STAGES, it + DEC_STAGES - 1);
    cp_async_commit();
    const int pi = 2 * it + krow0 / KT;
    if (pi < n_pages) {
      const int key0 = page_at(pi) * KT + krow0 % KT;
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[j][i] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = krow0 + (lane & 7) + ((lane >> 4) << 3);
        const int col = kk * 16 + ((lane >> 3) & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(ks + (uint32_t)(row * LDS + col) * 2, b0, b1, b2, b3);
        mma_bf16(s[0], qf[kk], b0, b1);
        mma_bf16(s[1], qf[kk], b2, b3);
      }
      const int t = lane & 3;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = key0 + j * 8 + 2 * t + (i & 1);
          const int pos = (i < 2) ? pos_a : pos_b;
          const bool seen = key <= pos && (p.window == 0 || pos - key < p.window || key < p.keep_first);
          float v = s[j][i] * p.scale;
          if (p.softcap > 0.0f) v = p.softcap * (1.0f - __fdividef(2.0f, __expf(fminf(v * two_inv_cap, 80.0f)) + 1.0f));
          v += (i < 2) ? pb_a : pb_b;
          s[j][i] = seen ? __fdividef(1.0f, 1.0f + __expf(fminf(-v, 80.0f))) : 0.0f;
        }
      }
      uint32_t a[4];
      a[0] = pack_bf16(s[0][0], s[0][1]);
      a[1] = pack_bf16(s[0][2], s[0][3]);
      a[2] = pack_bf16(s[1][0], s[1][1]);
      a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int dj = 0; dj < HD / 16; ++dj) {
        const int row = krow0 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int col = dj * 16 + (lane >> 4) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vs + (uint32_t)(row * LDS + col) * 2, b0, b1, b2, b3);
        mma_bf16(o[2 * dj], a, b0, b1);
        mma_bf16(o[2 * dj + 1], a, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // the warps' sums, added in warp order
  float* part = reinterpret_cast<float*>(smem + DEC_ROWS * LDS * 2);
  const int t4 = lane & 3;
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    float* dst = part + ((size_t)warp * DEC_ROWS) * HD + j * 8 + 2 * t4;
    dst[ra * HD] = o[j][0], dst[ra * HD + 1] = o[j][1];
    dst[rb * HD] = o[j][2], dst[rb * HD + 1] = o[j][3];
  }
  __syncthreads();
  for (int idx = tid; idx < R * HD; idx += TC_THREADS) {
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < TC_THREADS / 32; ++w) sum += part[(size_t)w * DEC_ROWS * HD + idx];
    const int r = idx / HD;
    p.out[((size_t)(row0 + r / G) * p.n_q_heads + kvh * G + r % G) * HD + idx % HD] = __float2bfloat16(sum);
  }
}

template <int HD>
int launch_sigmoid_mma(const SigmoidParams& p, int n_seqs, int max_new, cudaStream_t stream) {
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(attn_sigmoid_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tc_smem<HD>());
    if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_attention_sigmoid: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  const int G = p.n_q_heads / p.n_kv_heads;
  if (max_new * G <= DEC_ROWS) {
    static bool dec_opted = false;
    if (!dec_opted) {
      cudaError_t e = cudaFuncSetAttribute(attn_sigmoid_mma_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           dec_smem<HD>());
      if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_attention_sigmoid: shared memory opt-in failed: %s", cudaGetErrorString(e));
      dec_opted = true;
    }
    sb_launch(attn_sigmoid_mma_decode_kernel<HD>, dim3(p.n_kv_heads, 1, n_seqs), dim3(TC_THREADS), (size_t)dec_smem<HD>(),
              stream, p);
    return SB_OK;
  }
  const int row_blocks = (max_new * G + TC_BM - 1) / TC_BM;
  const dim3 grid(row_blocks * p.n_kv_heads, 1, n_seqs);
  sb_launch(attn_sigmoid_mma_kernel<HD>, grid, dim3(TC_THREADS), (size_t)tc_smem<HD>(), stream, p);
  return SB_OK;
}

}  // namespace

extern "C" int sb_attention_sigmoid(const void* q, void* out, int act_dtype, int n_rows, const int32_t* row_seq,
                                    const int32_t* row_pos, int n_seqs, int max_new, const int32_t* seq_row0,
                                    const int32_t* seq_pos0, const int32_t* page_off, const int32_t* page_ids,
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
  // bfloat16 at head sizes 64 and 128 over pages of 64 keys: tensor cores
  if (act_dtype == SB_BF16 && cache_dtype == SB_BF16 && page_size == KT && (hd == 64 || hd == 128) && seq_row0 &&
      seq_pos0 && n_seqs > 0 && max_new > 0 && n_seqs <= 65535) {
    SigmoidParams p;
    p.q = (const bf16*)q, p.out = (bf16*)out, p.seq_row0 = seq_row0, p.seq_pos0 = seq_pos0;
    p.page_off = page_off, p.page_ids = page_ids, p.cache = (const bf16*)cache;
    p.n_q_heads = n_q_heads, p.n_kv_heads = n_kv_heads, p.window = window, p.keep_first = keep_first;
    p.scale = scale, p.softcap = softcap, p.head_bias = head_bias;
    const int rc = hd == 64 ? launch_sigmoid_mma<64>(p, n_seqs, max_new, stream)
                            : launch_sigmoid_mma<128>(p, n_seqs, max_new, stream);
    if (rc) return rc;
    SB_CHECK_LAUNCH("sb_attention_sigmoid");
    return SB_OK;
  }
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
