// The linear recurrence with a matrix state and a decay per key channel,
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,
//
// per head, token by token in float32, for prompts, portions and single tokens alike: every token
// is the same arithmetic whatever the step brings, so a result does not depend on how a sequence
// was cut or on what else the step holds.  The decay is one value per (token, head, key channel)
// read from a tensor, one fixed value per head, or one value per (token, head) read from a tensor.
// Several heads may share one q and k (`heads_per_qk` neighbouring heads read the same ones), as
// the heads of a state-space layer share its input and output maps.
//
// A column of S (the `dim` values that belong to one value channel) is shared by 16 lanes that
// keep their runs of it in registers for the whole step (of one column, or of two neighbouring
// ones when the step has blocks enough: what a lane reads of a token then serves both); a block
// has eight such groups of lanes.  Tokens come in groups of 16: a group's q, k, decays and the block's values are staged in
// shared memory with cp.async one or two groups ahead of the one that is computed; per token a
// lane multiplies and adds its runs, and the 16 lanes' partial dot products of the group's 16
// tokens are added in 15 exchanges, after which lane i holds token i's sum (the same tree of
// additions for every token, wherever in a group it falls).  State: float32 [slot, heads, vdim,
// dim] (column by column).
#include "common.cuh"

namespace {

constexpr int LANES = 16;            // lanes that share a column
constexpr int GROUPS = 8;            // groups of 16 lanes in a block (four warps)
constexpr int TB = 16;               // tokens of a group
constexpr int THREADS = LANES * GROUPS;

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Lane `sub` keeps NPL channels of its column in runs of R = min(NPL, 4): run j holds channels
// j * 16 R + sub * R ... + R - 1, so that the 16 lanes' loads of a run are one contiguous stretch.
template <int NPL>
struct Runs {
  static constexpr int R = NPL < 4 ? NPL : 4;
  __device__ static __forceinline__ int channel(int sub, int i) { return (i / R) * (LANES * R) + sub * R + i % R; }
};

// STAGES groups of tokens in shared memory: one in use, the others on their way.
// CPT columns per thread: a lane keeps its runs of CPT neighbouring columns, so that what it reads of
// a token's q, k and decays serves CPT columns.
template <int NPL, int MODE, bool VEC, int STAGES, int CPT>
__global__ void __launch_bounds__(THREADS)
linrec_scan_kernel(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay,
                   const float* __restrict__ head_decay, const float* token_decay, int heads_per_qk,
                   const int32_t* seq_row0, const int32_t* seq_slot,
                   int n_heads, int dim, int vdim, float* state, float* out) {
  extern __shared__ __align__(16) float smem[];
  constexpr bool PER_CHANNEL = MODE == 1;               // a decay per key channel
  constexpr bool PER_TOKEN = MODE == 2;                 // a decay per token and head
  constexpr int PAD = NPL * LANES;                      // channels with padding
  constexpr int NARR = PER_CHANNEL ? 3 : 2;             // q, k (, decay)
  constexpr int R = Runs<NPL>::R;
  constexpr int COLS = GROUPS * CPT;                   // columns of a block
  constexpr int ROW = NARR * PAD + COLS + (PER_TOKEN ? 4 : 0);   // floats of a staged token
  sb_pdl_launch();
  const int b = blockIdx.z, h = blockIdx.y;
  const int tid = threadIdx.x, sub = tid % LANES, cl = tid / LANES;
  const int col0 = blockIdx.x * COLS, col = col0 + cl * CPT;      // this thread's first column
  const int row0 = seq_row0[b], n = seq_row0[b + 1] - row0;
  const int slot = seq_slot[b];
  const float a_head = MODE == 0 ? head_decay[h] : 1.0f;
  const int hq = h / heads_per_qk;                      // the q and k this head reads
  // padding channels and columns stay zero for good: cp.async writes the others only
  if (dim < PAD || vdim - col0 < COLS) {
    for (int i = tid; i < STAGES * TB * ROW; i += THREADS) smem[i] = 0.0f;
    __syncthreads();
  }
  sb_pdl_wait();
  float* srow = state + (((size_t)slot * n_heads + h) * vdim) * dim;
  float S[CPT][NPL];
#pragma unroll
  for (int x = 0; x < CPT; ++x)
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int c = Runs<NPL>::channel(sub, i);
      S[x][i] = (col + x < vdim && c < dim) ? srow[(size_t)(col + x) * dim + c] : 0.0f;
    }
  const size_t per_row = (size_t)n_heads * dim;
  const int n_cols = min(COLS, vdim - col0);

  // What this thread copies of every token, worked out once: piece k of the thread is 16 bytes
  // (VEC) or one value of q, k, the decays or the block's values; `src[k]` points into the
  // sequence's first row, `step[k]` is that tensor's row stride.
  constexpr int V = VEC ? 4 : 1;
  constexpr int PIECES = NARR * PAD / V + COLS / V + (PER_TOKEN ? 1 : 0);     // at most, per token
  constexpr int MINE = (PIECES + THREADS - 1) / THREADS;
  const float* src[MINE];
  int dst[MINE], step[MINE], width[MINE];               // width: values of the piece (0: none)
  {
    const int per_arr = dim / V, n_vals = (n_cols + V - 1) / V;
#pragma unroll
    for (int k = 0; k < MINE; ++k) {
      const int e = tid + k * THREADS;
      const int arr = e / per_arr;
      src[k] = proj, dst[k] = 0, step[k] = 0, width[k] = 0;
      if (arr < NARR) {
        const int c = (e - arr * per_arr) * V;
        src[k] = arr == 0 ? proj + (size_t)row0 * ld + q_off + hq * dim + c
               : arr == 1 ? proj + (size_t)row0 * ld + k_off + hq * dim + c
                          : decay + (size_t)row0 * per_row + (size_t)h * dim + c;
        step[k] = arr == 2 ? (int)per_row : ld;
        dst[k] = arr * PAD + c;
        width[k] = V;
      } else if (e - NARR * per_arr < n_vals) {
        const int c = (e - NARR * per_arr) * V;
        src[k] = proj + (size_t)row0 * ld + v_off + h * vdim + col0 + c;
        step[k] = ld;
        dst[k] = NARR * PAD + c;
        width[k] = min(V, n_cols - c);
      } else if (PER_TOKEN && e - NARR * per_arr == n_vals) {
        src[k] = token_decay + (size_t)row0 * n_heads + h;
        step[k] = n_heads;
        dst[k] = NARR * PAD + COLS;
        width[k] = 1;
      }
    }
  }
  // stages tokens [t0, t0 + cnt) of the sequence into stage `st`
  auto stage = [&](int st, int t0, int cnt) {
    float* dst0 = smem + (size_t)st * TB * ROW;
#pragma unroll
    for (int k = 0; k < MINE; ++k) {
      if (width[k] == 0) continue;
      const float* from = src[k] + (size_t)t0 * step[k];
      float* to = dst0 + dst[k];
      if (width[k] == 4) {
        for (int tt = 0; tt < cnt; ++tt) cp_async16(to + tt * ROW, from + (size_t)tt * step[k]);
      } else {
        for (int tt = 0; tt < cnt; ++tt)
          for (int u = 0; u < width[k]; ++u) cp_async4(to + tt * ROW + u, from + (size_t)tt * step[k] + u);
      }
    }
    cp_commit();
  };

  const int n_groups = (n + TB - 1) / TB;
  for (int g = 0; g < STAGES - 1; ++g) {
    if (g < n_groups) stage(g, g * TB, min(TB, n - g * TB));
    else cp_commit();
  }
  for (int g = 0; g < n_groups; ++g) {
    const int t0 = g * TB, cnt = min(TB, n - t0);
    cp_wait<STAGES - 2>();                              // group g has landed (for this thread's copies)
    __syncthreads();                                    // ... for everybody's, and group g - 1 is no longer read
    {
      const int g2 = g + STAGES - 1;
      if (g2 < n_groups) stage(g2 % STAGES, g2 * TB, min(TB, n - g2 * TB));
      else cp_commit();
    }
    const float* base = smem + (size_t)(g % STAGES) * TB * ROW;
    float acc[CPT][TB];
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
#pragma unroll
      for (int x = 0; x < CPT; ++x) acc[x][tt] = 0.0f;
      if (tt < cnt) {
        const float* tok = base + tt * ROW;
        float v[CPT];
#pragma unroll
        for (int x = 0; x < CPT; ++x) v[x] = tok[NARR * PAD + cl * CPT + x];
        const float a_tok = PER_TOKEN ? tok[NARR * PAD + COLS] : a_head;
#pragma unroll
        for (int j = 0; j < NPL / R; ++j) {
          float qv[R], kv[R], av[R];
          const int c = j * (LANES * R) + sub * R;
          if (R == 4) {
            *reinterpret_cast<float4*>(qv) = *reinterpret_cast<const float4*>(tok + c);
            *reinterpret_cast<float4*>(kv) = *reinterpret_cast<const float4*>(tok + PAD + c);
            if (PER_CHANNEL) *reinterpret_cast<float4*>(av) = *reinterpret_cast<const float4*>(tok + 2 * PAD + c);
          } else {
#pragma unroll
            for (int u = 0; u < R; ++u) {
              qv[u] = tok[c + u];
              kv[u] = tok[PAD + c + u];
              if (PER_CHANNEL) av[u] = tok[2 * PAD + c + u];
            }
          }
#pragma unroll
          for (int x = 0; x < CPT; ++x)
#pragma unroll
            for (int u = 0; u < R; ++u) {
              const float sv = fmaf(PER_CHANNEL ? av[u] : a_tok, S[x][j * R + u], kv[u] * v[x]);
              S[x][j * R + u] = sv;
              acc[x][tt] = fmaf(sv, qv[u], acc[x][tt]);
            }
        }
      }
    }
    // the lanes' partial sums of the group's tokens, added so that lane i ends with token i's sum:
    // at every step a lane keeps the half of its values whose token number has the step's bit as
    // the lane has it, and gets the partner's sums of those tokens
#pragma unroll
    for (int x = 0; x < CPT; ++x) {
#pragma unroll
      for (int w = TB / 2; w > 0; w >>= 1) {
        const bool up = sub & w;
#pragma unroll
        for (int i = 0; i < w; ++i) {
          const float keep = up ? acc[x][i + w] : acc[x][i];
          const float give = up ? acc[x][i] : acc[x][i + w];
          acc[x][i] = keep + __shfl_xor_sync(0xffffffffu, give, w);
        }
      }
      if (sub < cnt && col + x < vdim) out[((size_t)(row0 + t0 + sub) * n_heads + h) * vdim + col + x] = acc[x][0];
    }
  }
#pragma unroll
  for (int x = 0; x < CPT; ++x) {
    if (col + x >= vdim) continue;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int c = Runs<NPL>::channel(sub, i);
      if (c < dim) srow[(size_t)(col + x) * dim + c] = S[x][i];
    }
  }
}

template <int NPL>
constexpr size_t scan_smem(int mode, int stages, int cpt) {
  return (size_t)stages * TB * ((mode == 1 ? 3 : 2) * NPL * LANES + GROUPS * cpt + (mode == 2 ? 4 : 0)) * sizeof(float);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 1;
  }
  return n;
}

// Blocks that fit the GPU at once with this much shared memory each.
long fits(size_t smem) {
  const long per_sm = (long)((227 * 1024) / (smem + 1024));
  return (long)sm_count() * (per_sm < 16 ? per_sm : 16);
}

template <int NPL, int PC, bool VEC, int STAGES, int CPT>
cudaError_t launch_scan(dim3 grid, cudaStream_t stream, const float* proj, int ld, int q_off, int k_off, int v_off,
                        const float* decay, const float* head_decay, const float* token_decay, int heads_per_qk, const int32_t* seq_row0,
                        const int32_t* seq_slot, int n_heads, int dim, int vdim, float* state, float* out) {
  constexpr size_t smem = scan_smem<NPL>(PC, STAGES, CPT);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(linrec_scan_kernel<NPL, PC, VEC, STAGES, CPT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  configured = true;
  return sb_launch<SB_K_OTHER>(linrec_scan_kernel<NPL, PC, VEC, STAGES, CPT>, grid, dim3(THREADS), smem, stream, proj, ld,
                               q_off, k_off, v_off, decay, head_decay, token_decay, heads_per_qk, seq_row0, seq_slot, n_heads, dim, vdim, state, out);
}

// Three stages, unless the grid then needs a second wave of blocks that two stages spare it.
template <int NPL, int PC, bool VEC, int CPT>
cudaError_t launch_scan_staged(int n_seqs, cudaStream_t stream, const float* proj, int ld, int q_off, int k_off,
                               int v_off, const float* decay, const float* head_decay, const float* token_decay, int heads_per_qk, const int32_t* seq_row0,
                               const int32_t* seq_slot, int n_heads, int dim, int vdim, float* state, float* out) {
  const dim3 grid((vdim + GROUPS * CPT - 1) / (GROUPS * CPT), n_heads, n_seqs);
  const long blocks = (long)grid.x * grid.y * grid.z;
  constexpr bool three_fit = scan_smem<NPL>(PC, 3, CPT) <= 226 * 1024;      // a block's limit
  if constexpr (!three_fit)
    return launch_scan<NPL, PC, VEC, 2, CPT>(grid, stream, proj, ld, q_off, k_off, v_off, decay, head_decay, token_decay, heads_per_qk, seq_row0,
                                             seq_slot, n_heads, dim, vdim, state, out);
  else if (blocks > fits(scan_smem<NPL>(PC, 3, CPT)) && blocks <= fits(scan_smem<NPL>(PC, 2, CPT)))
    return launch_scan<NPL, PC, VEC, 2, CPT>(grid, stream, proj, ld, q_off, k_off, v_off, decay, head_decay, token_decay, heads_per_qk, seq_row0,
                                             seq_slot, n_heads, dim, vdim, state, out);
  else
    return launch_scan<NPL, PC, VEC, 3, CPT>(grid, stream, proj, ld, q_off, k_off, v_off, decay, head_decay, token_decay, heads_per_qk, seq_row0,
                                             seq_slot, n_heads, dim, vdim, state, out);
}

int g_force_cpt = 0;

// Columns per thread: two when that still gives half of the SMs a block, else one.  Measured on
// B200, 2,048 tokens of one sequence, key size 128, 256 value channels a head: 8 heads (128 blocks
// of two columns a thread) 238 us against 303 us with one column, 14 heads 324 against 506 us;
// 6 heads of 64 x 64 (24 blocks) 173 against 156 us.
template <int NPL, int PC, bool VEC>
cudaError_t launch_scan_cols(int n_seqs, cudaStream_t stream, const float* proj, int ld, int q_off, int k_off,
                             int v_off, const float* decay, const float* head_decay, const float* token_decay, int heads_per_qk, const int32_t* seq_row0,
                             const int32_t* seq_slot, int n_heads, int dim, int vdim, float* state, float* out) {
  const long blocks2 = (long)((vdim + 2 * GROUPS - 1) / (2 * GROUPS)) * n_heads * n_seqs;
  const bool two = g_force_cpt ? g_force_cpt == 2 : (NPL <= 8 && 2 * blocks2 >= sm_count());
  if (two)
    return launch_scan_staged<NPL, PC, VEC, (NPL <= 8 ? 2 : 1)>(n_seqs, stream, proj, ld, q_off, k_off, v_off, decay,
                                                                 head_decay, token_decay, heads_per_qk, seq_row0, seq_slot, n_heads, dim, vdim, state, out);
  return launch_scan_staged<NPL, PC, VEC, 1>(n_seqs, stream, proj, ld, q_off, k_off, v_off, decay, head_decay, token_decay, heads_per_qk, seq_row0,
                                             seq_slot, n_heads, dim, vdim, state, out);
}

}  // namespace

extern "C" int sb_linrec_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay,
                              const float* head_decay, const float* token_decay, int heads_per_qk, int n_seqs,
                              const int32_t* seq_row0, const int32_t* seq_slot, int n_heads, int dim, int vdim,
                              float* state, float* out, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || dim <= 0 || vdim <= 0 || !proj || !state || !out || !seq_row0 || !seq_slot)
    SB_FAIL(SB_ERR_ARG, "sb_linrec_scan: seqs=%d heads=%d dim=%d vdim=%d", n_seqs, n_heads, dim, vdim);
  if ((decay != nullptr) + (head_decay != nullptr) + (token_decay != nullptr) != 1)
    SB_FAIL(SB_ERR_ARG, "sb_linrec_scan: exactly one of the three kinds of decay is given");
  if (heads_per_qk <= 0 || n_heads % heads_per_qk)
    SB_FAIL(SB_ERR_ARG, "sb_linrec_scan: %d heads do not share q and k in groups of %d", n_heads, heads_per_qk);
  if (dim > 32 * LANES) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_linrec_scan: key size %d is above %d", dim, 32 * LANES);
  if (n_heads > 65535 || n_seqs > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_linrec_scan: %d heads, %d sequences", n_heads, n_seqs);
  const int npl = (dim + LANES - 1) / LANES;
  // 16-byte copies when every staged stretch starts on a 16-byte boundary
  const bool vec = dim % 4 == 0 && vdim % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                   !((uintptr_t)proj & 15) && !((uintptr_t)decay & 15);
  cudaError_t e;
#define SB_LINREC_ARGS n_seqs, stream, proj, ld, q_off, k_off, v_off, decay, head_decay, token_decay, heads_per_qk, seq_row0, seq_slot, n_heads, dim, vdim, state, out
#define SB_LINREC_LAUNCH(N)                                                                   \
  e = decay ? (vec ? launch_scan_cols<N, 1, true>(SB_LINREC_ARGS) : launch_scan_cols<N, 1, false>(SB_LINREC_ARGS)) \
      : token_decay ? (vec ? launch_scan_cols<N, 2, true>(SB_LINREC_ARGS) : launch_scan_cols<N, 2, false>(SB_LINREC_ARGS)) \
            : (vec ? launch_scan_cols<N, 0, true>(SB_LINREC_ARGS) : launch_scan_cols<N, 0, false>(SB_LINREC_ARGS))
  if (npl <= 1) SB_LINREC_LAUNCH(1);
  else if (npl <= 2) SB_LINREC_LAUNCH(2);
  else if (npl <= 4) SB_LINREC_LAUNCH(4);
  else if (npl <= 8) SB_LINREC_LAUNCH(8);
  else if (npl <= 16) SB_LINREC_LAUNCH(16);
  else SB_LINREC_LAUNCH(32);
#undef SB_LINREC_LAUNCH
#undef SB_LINREC_ARGS
  if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_linrec_scan: launch failed: %s", cudaGetErrorString(e));
  return SB_OK;
}

// For measurements and tests: 1 or 2 columns per thread for every call, 0 by the sizes again.
extern "C" void sb_linrec_force_columns(int cpt) { g_force_cpt = cpt == 1 || cpt == 2 ? cpt : 0; }
