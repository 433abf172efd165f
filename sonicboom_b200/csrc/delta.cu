// The generalized delta rule: a recurrence over a matrix state with a decay per key channel and a
// removal along the unit key,
//
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      o_t = S_t^T r_t,
//
// per head, u = k / sqrt(sum(k^2) + key_eps), both products reading the old state.  Column j of S
// (the `dim` values of one value channel) obeys  s <- w * s - (a * u) (u . s) + k v_j,  o_j = s . r,
// so columns are independent.
//
//   sb_delta_prep: per row, from the mixer's one input product: the decays
//                  w = exp(-decay_scale * sigmoid(W2 tanh(z1) + w0)), the removal rates
//                  a = sigmoid(a_raw + a_bias) times the unit key, and the unit key, into
//                  aux [rows, 3, heads * dim] (w | a * u | u)
//   sb_delta_scan: the recurrence token by token in float32, for prompts, portions and single
//                  tokens alike.  A column is shared by eight lanes that keep their channels of it
//                  in registers for the whole step; a block has sixteen such groups; tokens are
//                  staged sixteen at a time in shared memory.  State: float32 [slot, heads, dim(value), dim(key)].
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LPC = 8;               // lanes that share a column
constexpr int COLS = 16;             // columns of a block
constexpr int THREADS = LPC * COLS;  // 128
constexpr int TB = 16;               // tokens staged together

template <typename TW>
__global__ void __launch_bounds__(256)
delta_prep_kernel(const float* proj, int ld, int k_off, int a_off, int z_off, int n_heads, int dim, int rank,
                  const TW* __restrict__ w2, const TW* __restrict__ w0, const TW* __restrict__ a_bias,
                  float decay_scale, float key_eps, float* aux) {
  extern __shared__ float sm[];        // rank tanh values, then one 1 / |k| per head
  float* th = sm;
  float* inv = sm + rank;
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t r = blockIdx.x;
  const float* row = proj + r * ld;
  const int hk = n_heads * dim;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) th[j] = tanhf(row[z_off + j]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int h = warp; h < n_heads; h += n_warps) {
    float s = 0.0f;
    for (int c = lane; c < dim; c += 32) {
      const float k = row[k_off + h * dim + c];
      s = fmaf(k, k, s);
    }
    s = sb_warp_sum(s);
    if (lane == 0) inv[h] = 1.0f / sqrtf(s + key_eps);
  }
  __syncthreads();
  float* o = aux + r * 3 * hk;
  for (int c = threadIdx.x; c < hk; c += blockDim.x) {
    float z = sb_to_f32<TW>(w0[c]);
    const TW* wr = w2 + (size_t)c * rank;
    for (int j = 0; j < rank; ++j) z = fmaf(sb_to_f32<TW>(wr[j]), th[j], z);
    const float sg = 1.0f / (1.0f + expf(-z));
    const float a = 1.0f / (1.0f + expf(-(row[a_off + c] + sb_to_f32<TW>(a_bias[c]))));
    const float u = row[k_off + c] * inv[c / dim];
    o[c] = expf(-decay_scale * sg);
    o[hk + c] = a * u;
    o[2 * hk + c] = u;
  }
}

// NPL channels per lane: lane `sub` of a column keeps channels sub + 8 i.
template <int NPL>
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
  for (int i = tid; i < TB * ROW; i += THREADS) smem[i] = 0.0f;     // padding stays zero for good
  sb_pdl_wait();
  const int row0 = seq_row0[b], n = seq_row0[b + 1] - row0;
  const int slot = seq_slot[b];
  float* srow = state + (((size_t)slot * n_heads + h) * dim + (col < dim ? col : 0)) * dim;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = sub + LPC * i;
    S[i] = (col < dim && c < dim) ? srow[c] : 0.0f;
  }
  __syncthreads();
  for (int t0 = 0; t0 < n; t0 += TB) {
    const int cnt = min(TB, n - t0);
    // stage the group's tokens: five vectors of `dim` and the block's values of v
    for (int e = tid; e < cnt * 5 * dim; e += THREADS) {
      const int tt = e / (5 * dim), rest = e - tt * 5 * dim, arr = rest / dim, c = rest - arr * dim;
      const size_t rw = (size_t)(row0 + t0 + tt);
      float v;
      if (arr == 0) v = proj[rw * ld + r_off + h * dim + c];
      else if (arr == 1) v = proj[rw * ld + k_off + h * dim + c];
      else v = aux[rw * 3 * hk + (size_t)(arr - 2) * hk + h * dim + c];
      smem[tt * ROW + arr * PAD + c] = v;
    }
    for (int e = tid; e < cnt * COLS; e += THREADS) {
      const int tt = e / COLS, c = e - tt * COLS;
      smem[tt * ROW + 5 * PAD + c] = col0 + c < dim ? proj[(size_t)(row0 + t0 + tt) * ld + v_off + h * dim + col0 + c] : 0.0f;
    }
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float* tok = smem + tt * ROW;
      const float v = tok[5 * PAD + cl];
      float d = 0.0f;
#pragma unroll
      for (int i = 0; i < NPL; ++i) d = fmaf(tok[4 * PAD + sub + LPC * i], S[i], d);       // u . s (old state)
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      float o = 0.0f;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int c = sub + LPC * i;
        float s = tok[2 * PAD + c] * S[i];
        s = fmaf(-tok[3 * PAD + c], d, s);
        s = fmaf(tok[PAD + c], v, s);
        S[i] = s;
        o = fmaf(s, tok[c], o);
      }
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      if (sub == 0 && col < dim) out[((size_t)(row0 + t0 + tt) * n_heads + h) * dim + col] = o;
    }
    __syncthreads();
  }
  if (col < dim) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int c = sub + LPC * i;
      if (c < dim) srow[c] = S[i];
    }
  }
}

template <int NPL>
cudaError_t launch_delta(dim3 grid, cudaStream_t stream, const float* proj, int ld, int r_off, int k_off, int v_off,
                         const float* aux, const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim,
                         float* state, float* out) {
  constexpr size_t smem = (size_t)TB * (5 * NPL * LPC + COLS) * sizeof(float);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<NPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  configured = true;
  return sb_launch<SB_K_OTHER>(delta_scan_kernel<NPL>, grid, dim3(THREADS), smem, stream, proj, ld, r_off, k_off, v_off, aux,
                               seq_row0, seq_slot, n_heads, dim, state, out);
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
  const size_t smem = (size_t)(rank + n_heads) * sizeof(float);
  if (smem > 48 * 1024) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_prep: rank %d with %d heads", rank, n_heads);
  SB_DISPATCH_DTYPE(w_dtype, TW, {
    sb_launch<SB_K_ELEMENTWISE>(delta_prep_kernel<TW>, dim3(n_rows), dim3(256), smem, stream, proj, ld, k_off, a_off, z_off,
                                n_heads, dim, rank, (const TW*)w2, (const TW*)w0, (const TW*)a_bias, decay_scale,
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
  if (dim > 32 * LPC) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_scan: head size %d is above %d", dim, 32 * LPC);
  if (n_heads > 65535 || n_seqs > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_delta_scan: %d heads, %d sequences", n_heads, n_seqs);
  const dim3 grid((dim + COLS - 1) / COLS, n_heads, n_seqs);
  const int npl = (dim + LPC - 1) / LPC;
  cudaError_t e;
#define SB_DELTA_ARGS grid, stream, proj, ld, r_off, k_off, v_off, aux, seq_row0, seq_slot, n_heads, dim, state, out
  if (npl <= 2) e = launch_delta<2>(SB_DELTA_ARGS);
  else if (npl <= 4) e = launch_delta<4>(SB_DELTA_ARGS);
  else if (npl <= 8) e = launch_delta<8>(SB_DELTA_ARGS);
  else if (npl <= 16) e = launch_delta<16>(SB_DELTA_ARGS);
  else e = launch_delta<32>(SB_DELTA_ARGS);
#undef SB_DELTA_ARGS
  if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_delta_scan: launch failed: %s", cudaGetErrorString(e));
  return SB_OK;
}
