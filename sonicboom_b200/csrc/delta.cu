// The generalized delta rule: a recurrence over a matrix state with a decay per key channel and a
// removal along the unit key,
//
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      o_t = S_t^T r_t,
//
// per head, u = k / sqrt(sum(k^2) + key_eps); decay and removal act on S_(t-1), then k v^T is added.  Column j of S
// (the `dim` values of one value channel) obeys  s <- w * s - (a * u) (u . s) + k v_j,  o_j = s . r,
// so columns are independent.
//
//   sb_delta_prep: per row, from the mixer's one input product: the decays
//                  w = exp(-decay_scale * sigmoid(W2 tanh(z1) + w0)), the removal rates
//                  a = sigmoid(a_raw + a_bias) times the unit key, and the unit key, into
//                  aux [rows, 3, heads * dim] (w | a * u | u)
//   sb_delta_scan: the recurrence token by token in float32, for prompts, portions and single
//                  tokens alike.  A column is shared by sixteen lanes that keep their channels of it
//                  in registers for the whole step; a block has eight such groups; tokens are
//                  staged sixteen at a time in shared memory, one or two groups ahead of the one
//                  in work (cp.async).  Only u . s, which the update needs, is summed over the
//                  lanes token by token; the lanes' parts of the outputs wait for the group's end.  State: float32 [slot, heads, dim(value), dim(key)].
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LPC = 16;              // lanes that share a column
constexpr int COLS = 8;              // columns of a block
constexpr int THREADS = LPC * COLS;  // 128
constexpr int TB = 16;               // tokens staged together

constexpr int PREP_ROWS = 8;         // rows a block of sb_delta_prep works on
constexpr int PREP_THREADS = 256;    // and its channels, one a thread

// A block takes PREP_ROWS rows and 256 channels: a channel's row of the decay map's second matrix
// is read once (16 bytes at a time where it can be) for all of the block's rows.
template <typename TW>
__global__ void __launch_bounds__(PREP_THREADS)
delta_prep_kernel(const float* proj, int n_rows, int ld, int k_off, int a_off, int z_off, int n_heads, int dim, int rank,
                  const TW* __restrict__ w2, const TW* __restrict__ w0, const TW* __restrict__ a_bias,
                  float decay_scale, float key_eps, float* aux) {
  extern __shared__ float sm[];        // PREP_ROWS x rank tanh values, then 1 / |k| per row and head of the block
  float* th = sm;
  float* inv = sm + PREP_ROWS * rank;
  sb_pdl_launch();
  sb_pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r0 = blockIdx.x * PREP_ROWS, nr = min(PREP_ROWS, n_rows - r0);
  const int hk = n_heads * dim;
  const int c0 = blockIdx.y * PREP_THREADS, c = c0 + tid;
  const int h_first = c0 / dim, nh = min(hk - 1, c0 + PREP_THREADS - 1) / dim - h_first + 1;
  for (int i = tid; i < PREP_ROWS * rank; i += PREP_THREADS) {
    const int r = i / rank, j = i - r * rank;
    th[i] = r < nr ? tanhf(proj[(size_t)(r0 + r) * ld + z_off + j]) : 0.0f;
  }
  for (int i = warp; i < nr * nh; i += PREP_THREADS / 32) {
    const int r = i / nh, h = h_first + i - r * nh;
    const float* krow = proj + (size_t)(r0 + r) * ld + k_off + h * dim;
    float s = 0.0f;
    for (int cc = lane; cc < dim; cc += 32) s = fmaf(krow[cc], krow[cc], s);
    s = sb_warp_sum(s);
    if (lane == 0) inv[i] = 1.0f / sqrtf(s + key_eps);
  }
  __syncthreads();
  if (c >= hk) return;
  float z[PREP_ROWS];
  const float z0 = sb_to_f32<TW>(w0[c]);
#pragma unroll
  for (int r = 0; r < PREP_ROWS; ++r) z[r] = z0;
  const TW* wr = w2 + (size_t)c * rank;
  if (sizeof(TW) == 2 && rank % 8 == 0 && !((uintptr_t)w2 & 15)) {
    for (int j = 0; j < rank; j += 8) {
      const uint4 pack = *reinterpret_cast<const uint4*>(wr + j);
      const TW* wv = reinterpret_cast<const TW*>(&pack);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float wf = sb_to_f32<TW>(wv[jj]);
#pragma unroll
        for (int r = 0; r < PREP_ROWS; ++r) z[r] = fmaf(wf, th[r * rank + j + jj], z[r]);
      }
    }
  } else {
    for (int j = 0; j < rank; ++j) {
      const float wf = sb_to_f32<TW>(wr[j]);
#pragma unroll
      for (int r = 0; r < PREP_ROWS; ++r) z[r] = fmaf(wf, th[r * rank + j], z[r]);
    }
  }
  const float ab = sb_to_f32<TW>(a_bias[c]);
  const int hl = c / dim - h_first;
#pragma unroll
  for (int r = 0; r < PREP_ROWS; ++r) {
    if (r >= nr) break;
    const float* row = proj + (size_t)(r0 + r) * ld;
    float* o = aux + (size_t)(r0 + r) * 3 * hk;
    const float sg = 1.0f / (1.0f + expf(-z[r]));
    const float a = 1.0f / (1.0f + expf(-(row[a_off + c] + ab)));
    const float u = row[k_off + c] * inv[r * nh + hl];
    o[c] = expf(-decay_scale * sg);
    o[hk + c] = a * u;
    o[2 * hk + c] = u;
  }
}

// Copies of VEC floats (16 or 4 bytes) that complete in the background; 0 source bytes: zeros.
template <int VEC>
__device__ __forceinline__ void delta_cp_async(float* dst, const float* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? VEC * 4 : 0;
  if (VEC == 4)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}

// NPL channels per lane: lane `sub` of a column keeps channels sub + 16 i.  Groups of TB tokens
// are staged STAGES - 1 groups ahead with cp.async (in pieces of VEC floats: 4 where every row,
// offset and head size is a multiple of 4 floats, else 1), so the loads of later tokens are in
// flight while the recurrence, a chain from token to token, runs.
template <int NPL, int VEC, int STAGES>
__global__ void __launch_bounds__(THREADS)
delta_scan_kernel(const float* proj, int ld, int r_off, int k_off, int v_off, const float* aux,
                  const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim, float* state, float* out) {
  extern __shared__ __align__(16) float smem[];
  constexpr int PAD = NPL * LPC;                 // channels with padding
  constexpr int ROW = 5 * PAD + COLS;            // r, k, w, a*u, u, then the block's values
  sb_pdl_launch();
  const int b = blockIdx.z, h = blockIdx.y;
  const int tid = threadIdx.x, sub = tid % LPC, cl = tid / LPC;
  const int col0 = blockIdx.x * COLS, col = col0 + cl;
  const int hk = n_heads * dim;
  if (PAD > dim) {                                 // channels past the head's size stay zero for good
    for (int i = tid; i < STAGES * TB * ROW; i += THREADS) smem[i] = 0.0f;
    __syncthreads();
  }
  sb_pdl_wait();
  const int row0 = seq_row0[b], n = seq_row0[b + 1] - row0;
  const int slot = seq_slot[b];
  const int dimv = dim / VEC, per_tok = 5 * dimv + COLS / VEC;
  auto stage = [&](int buf, int t0) {
    const int cnt = min(TB, n - t0);
    float* base = smem + buf * TB * ROW;
    // a thread keeps to its pieces of a token and walks over the group's tokens
    for (int q = tid; q < per_tok; q += THREADS) {
      const float* src;
      size_t stride;
      float* dst;
      bool ok = true;
      if (q < 5 * dimv) {
        const int arr = q / dimv, c = (q - arr * dimv) * VEC;
        const size_t rw = (size_t)(row0 + t0);
        if (arr < 2) src = proj + rw * ld + (arr == 0 ? r_off : k_off) + h * dim + c, stride = ld;
        else src = aux + rw * 3 * hk + (size_t)(arr - 2) * hk + h * dim + c, stride = (size_t)3 * hk;
        dst = base + arr * PAD + c;
      } else {
        const int c = (q - 5 * dimv) * VEC;
        ok = col0 + c < dim;
        src = ok ? proj + (size_t)(row0 + t0) * ld + v_off + h * dim + col0 + c : proj, stride = ok ? ld : 0;
        dst = base + 5 * PAD + c;
      }
      for (int tt = 0; tt < cnt; ++tt) delta_cp_async<VEC>(dst + tt * ROW, src + tt * stride, ok);
    }
  };
  const int n_groups = (n + TB - 1) / TB;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_groups) stage(s, s * TB);
    asm volatile("cp.async.commit_group;\n");
  }
  float* srow = state + (((size_t)slot * n_heads + h) * dim + (col < dim ? col : 0)) * dim;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = sub + LPC * i;
    S[i] = (col < dim && c < dim) ? srow[c] : 0.0f;
  }
  for (int gi = 0; gi < n_groups; ++gi) {
    const int t0 = gi * TB, cnt = min(TB, n - t0);
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
    __syncthreads();            // the group has landed, and every thread is done with the buffer staged next
    if (gi + STAGES - 1 < n_groups) stage((gi + STAGES - 1) % STAGES, (gi + STAGES - 1) * TB);
    asm volatile("cp.async.commit_group;\n");
    const float* grp = smem + (gi % STAGES) * TB * ROW;
    float op[TB];                                  // this lane's part of every token's o . r
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
      op[tt] = 0.0f;
      if (tt < cnt) {
        const float* tok = grp + tt * ROW;
        const float v = tok[5 * PAD + cl];
        float d0 = 0.0f, d1 = 0.0f;                // u . s (old state), even and odd pieces apart
#pragma unroll
        for (int i = 0; i < NPL; i += 2) {
          d0 = fmaf(tok[4 * PAD + sub + LPC * i], S[i], d0);
          d1 = fmaf(tok[4 * PAD + sub + LPC * (i + 1)], S[i + 1], d1);
        }
        float d = d0 + d1;
        d += __shfl_xor_sync(0xffffffffu, d, 8);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
        for (int i = 0; i < NPL; i += 2) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = sub + LPC * (i + e);
            float s = tok[2 * PAD + c] * S[i + e];
            s = fmaf(-tok[3 * PAD + c], d, s);
            s = fmaf(tok[PAD + c], v, s);
            S[i + e] = s;
            if (e == 0) o0 = fmaf(s, tok[c], o0);
            else o1 = fmaf(s, tok[c], o1);
          }
        }
        op[tt] = o0 + o1;
      }
    }
    // the sixteen lanes of a column add their parts of the group's sixteen sums in four rounds of
    // exchanges, halving what a lane keeps each time: the same tree of additions for every token,
    // and lane `sub` ends with the sum of token `sub`
    float a8[8], a4[4], a2[2];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float mine = (sub & 8) ? op[8 + j] : op[j], other = (sub & 8) ? op[j] : op[8 + j];
      a8[j] = mine + __shfl_xor_sync(0xffffffffu, other, 8);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float mine = (sub & 4) ? a8[4 + j] : a8[j], other = (sub & 4) ? a8[j] : a8[4 + j];
      a4[j] = mine + __shfl_xor_sync(0xffffffffu, other, 4);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float mine = (sub & 2) ? a4[2 + j] : a4[j], other = (sub & 2) ? a4[j] : a4[2 + j];
      a2[j] = mine + __shfl_xor_sync(0xffffffffu, other, 2);
    }
    const float mine1 = (sub & 1) ? a2[1] : a2[0], other1 = (sub & 1) ? a2[0] : a2[1];
    const float sum = mine1 + __shfl_xor_sync(0xffffffffu, other1, 1);
    if (sub < cnt && col < dim) out[((size_t)(row0 + t0 + sub) * n_heads + h) * dim + col] = sum;
  }
  asm volatile("cp.async.wait_group 0;\n");
  if (col < dim) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int c = sub + LPC * i;
      if (c < dim) srow[c] = S[i];
    }
  }
}

int delta_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 1;
  }
  return n;
}

template <int NPL, int VEC, int STAGES>
cudaError_t launch_delta_staged(dim3 grid, cudaStream_t stream, const float* proj, int ld, int r_off, int k_off,
                                int v_off, const float* aux, const int32_t* seq_row0, const int32_t* seq_slot,
                                int n_heads, int dim, float* state, float* out) {
  constexpr size_t smem = (size_t)STAGES * TB * (5 * NPL * LPC + COLS) * sizeof(float);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<NPL, VEC, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
  }
  configured = true;
  return sb_launch<SB_K_OTHER>(delta_scan_kernel<NPL, VEC, STAGES>, grid, dim3(THREADS), smem, stream, proj, ld, r_off,
                               k_off, v_off, aux, seq_row0, seq_slot, n_heads, dim, state, out);
}

// Three stages of token groups; two where three would not fit an SM (the largest heads) or would
// cost the grid a second wave of blocks.  The stages change when a token is copied, not a sum.
template <int NPL, int VEC>
cudaError_t launch_delta(dim3 grid, cudaStream_t stream, const float* proj, int ld, int r_off, int k_off, int v_off,
                         const float* aux, const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim,
                         float* state, float* out) {
  constexpr size_t smem3 = (size_t)3 * TB * (5 * NPL * LPC + COLS) * sizeof(float);
  const long per_sm = (long)((227 * 1024) / (smem3 + 1024));
  const long blocks = (long)grid.x * grid.y * grid.z;
  if (NPL < 16 && blocks <= (long)delta_sm_count() * (per_sm < 16 ? per_sm : 16))
    return launch_delta_staged<NPL, VEC, (NPL < 16 ? 3 : 2)>(grid, stream, proj, ld, r_off, k_off, v_off, aux, seq_row0,
                                                             seq_slot, n_heads, dim, state, out);
  return launch_delta_staged<NPL, VEC, 2>(grid, stream, proj, ld, r_off, k_off, v_off, aux, seq_row0, seq_slot, n_heads, dim,
                                          state, out);
}

}  // namespace

extern "C" int sb_delta_prep(const float* proj, int n_rows, int ld, int k_off, int a_off, int z_off, int n_heads,
                             int dim, int rank, const void* w2, const void* w0, const void* a_bias, int w_dtype,
                             float decay_scale, float key_eps, float* aux, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || dim <= 0 || rank <= 0 || !proj || !w2 || !w0 || !a_bias || !aux)
    SB_FAIL(SB_ERR_ARG, "sb_delta_prep: rows=%d heads=%d dim=%d rank=%d", n_rows, n_heads, dim, rank);
  if (!sb_valid_dtype(w_dtype)) SB_FAIL(SB_ERR_ARG, "sb_delta_prep: dtype code %d", w_dtype);
  const int hk = n_heads * dim;
  if (k_off < 0 || a_off < 0 || z_off < 0 || k_off + hk > ld || a_off + hk > ld || z_off + rank > ld)
    SB_FAIL(SB_ERR_ARG, "sb_delta_prep: offsets %d %d %d in rows of %d", k_off, a_off, z_off, ld);
  const size_t smem = (size_t)PREP_ROWS * (rank + PREP_THREADS / dim + 2) * sizeof(float);
  if (smem > 48 * 1024) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_prep: rank %d", rank);
  const dim3 grid((n_rows + PREP_ROWS - 1) / PREP_ROWS, (hk + PREP_THREADS - 1) / PREP_THREADS);
  if (grid.y > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_prep: %d channels", hk);
  SB_DISPATCH_DTYPE(w_dtype, TW, {
    sb_launch<SB_K_ELEMENTWISE>(delta_prep_kernel<TW>, grid, dim3(PREP_THREADS), smem, stream, proj, n_rows, ld, k_off, a_off,
                                z_off, n_heads, dim, rank, (const TW*)w2, (const TW*)w0, (const TW*)a_bias, decay_scale,
                                key_eps, aux);
  });
  SB_CHECK_LAUNCH("sb_delta_prep");
  return SB_OK;
}

extern "C" int sb_delta_scan(const float* proj, int ld, int r_off, int k_off, int v_off, const float* aux, int n_seqs,
                             const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim, float* state,
                             float* out, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || dim <= 0 || !proj || !aux || !state || !out || !seq_row0 || !seq_slot)
    SB_FAIL(SB_ERR_ARG, "sb_delta_scan: seqs=%d heads=%d dim=%d", n_seqs, n_heads, dim);
  if (dim > 16 * LPC) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_scan: head size %d is above %d", dim, 16 * LPC);
  if (n_heads > 65535 || n_seqs > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_scan: %d heads, %d sequences", n_heads, n_seqs);
  const dim3 grid((dim + COLS - 1) / COLS, n_heads, n_seqs);
  const int npl = (dim + LPC - 1) / LPC;
  cudaError_t e;
#define SB_DELTA_ARGS grid, stream, proj, ld, r_off, k_off, v_off, aux, seq_row0, seq_slot, n_heads, dim, state, out
  const bool wide = !((ld | r_off | k_off | v_off | dim) & 3) && !(((uintptr_t)proj | (uintptr_t)aux) & 15);
#define SB_DELTA_PICK(N) (wide ? launch_delta<N, 4>(SB_DELTA_ARGS) : launch_delta<N, 1>(SB_DELTA_ARGS))
  if (npl <= 2) e = SB_DELTA_PICK(2);
  else if (npl <= 4) e = SB_DELTA_PICK(4);
  else if (npl <= 8) e = SB_DELTA_PICK(8);
  else e = SB_DELTA_PICK(16);
#undef SB_DELTA_PICK
#undef SB_DELTA_ARGS
  if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_delta_scan: launch failed: %s", cudaGetErrorString(e));
  return SB_OK;
}
