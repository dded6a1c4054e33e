// The matrix-memory recurrence (mLSTM) with exponential gates and a running maximum.
//
// Per sequence and head, with q (already scaled), k in R^dim, v in R^vdim and the log gates
// i_t (input) and f_t (forget):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          S in R^{dim x vdim}
//     n_t = the same recurrence with k_t alone                                   n in R^dim
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// S, n and m start at zero.  The gates come from two pre-activations x_i, x_f (a projection plus
// a bias): i = cap tanh(x_i / cap), f = logsigmoid(cap tanh(x_f / cap)).
//
// n is S for a value that is always one, so the state is kept as one matrix of vdim + 1 columns,
// and the columns are independent of each other: a thread owns a column, walks the step's
// tokens in order and never meets another thread.  Every column also keeps a copy of m (row
// `dim` of the state), so that no column ever reads what another one writes.  State per slot:
// float32 [heads, dim + 1, vdim + 1].  The walk is the recurrence itself, token by token in
// float32, for prompts, portions of prompts and single tokens alike, so a position's result
// does not depend on how its sequence was cut into steps.
//
//   sb_mlstm_scan:  numerators S_t^T q_t for all vdim + 1 columns and m_t, per row and head;
//   sb_mlstm_out:   the division, the RMS norm of each head's output, its weight, the output
//                   gate sigmoid(g), in the activation dtype.
//
// Projection row (float32): [q heads*dim | k heads*dim | v heads*vdim | g heads*vdim | x_i heads |
// x_f heads].
#include <math.h>

#include "common.cuh"

namespace {

constexpr int VB = 64;          // columns (threads) per block
constexpr int TC = 16;          // tokens staged in shared memory at a time

__device__ __forceinline__ float log_sigmoid(float z) {
  return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

// DIM > 0: the column lives in DIM registers; DIM == 0: any dim, the column lives in shared memory.
template <int DIM, typename TB>
__global__ void __launch_bounds__(VB)
mlstm_scan_kernel(const float* proj, int ld, const int32_t* seq_row0, const int32_t* seq_slot, int H,
                  int dim_rt, int vdim, const TB* __restrict__ i_bias, const TB* __restrict__ f_bias,
                  float cap, float q_scale, float* state, float* num, float* m_row) {
  extern __shared__ float smem[];
  const int dim = DIM > 0 ? DIM : dim_rt;
  float* q_s = smem;                       // [TC][dim]
  float* k_s = q_s + TC * dim;             // [TC][dim]
  float* v_s = k_s + TC * dim;             // [TC][VB]
  float* ig_s = v_s + TC * VB;             // [TC]
  float* fg_s = ig_s + TC;                 // [TC]
  float* S_s = fg_s + TC;                  // [dim][VB] when DIM == 0
  sb_pdl_launch();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int jj = blockIdx.z * VB + tid, cols = vdim + 1;
  const bool active = jj < cols;
  const int row0 = seq_row0[b], T = seq_row0[b + 1] - row0;
  float* st = state + ((size_t)seq_slot[b] * H + h) * (size_t)(dim + 1) * cols;
  const float bi = sb_to_f32<TB>(i_bias[h]), bf = sb_to_f32<TB>(f_bias[h]);
  sb_pdl_wait();
  float S_r[DIM > 0 ? DIM : 1];
  if (DIM > 0) {
#pragma unroll
    for (int d = 0; d < (DIM > 0 ? DIM : 1); ++d) S_r[d] = active ? st[(size_t)d * cols + jj] : 0.0f;
  } else {
    for (int d = 0; d < dim; ++d) S_s[d * VB + tid] = active ? st[(size_t)d * cols + jj] : 0.0f;
  }
  float m = st[(size_t)dim * cols + (active ? jj : vdim)];
  const int q_off = h * dim, k_off = H * dim + h * dim, v_off = 2 * H * dim + h * vdim;
  const int i_off = 2 * H * dim + 2 * H * vdim + h, f_off = i_off + H;
  for (int t0 = 0; t0 < T; t0 += TC) {
    const int nt = min(TC, T - t0);
    __syncthreads();
    for (int e = tid; e < nt * dim; e += VB) {
      const float* src = proj + (size_t)(row0 + t0 + e / dim) * ld;
      q_s[e] = src[q_off + e % dim] * q_scale;
      k_s[e] = src[k_off + e % dim];
    }
    for (int tt = 0; tt < nt; ++tt)
      v_s[tt * VB + tid] = jj < vdim ? proj[(size_t)(row0 + t0 + tt) * ld + v_off + jj] : (jj == vdim ? 1.0f : 0.0f);
    if (tid < nt) {
      const float* src = proj + (size_t)(row0 + t0 + tid) * ld;
      ig_s[tid] = cap * tanhf((src[i_off] + bi) / cap);
      fg_s[tid] = log_sigmoid(cap * tanhf((src[f_off] + bf) / cap));
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float fm = fg_s[tt] + m, ig = ig_s[tt];
      const float mn = fmaxf(fm, ig);
      const float a = expf(fm - mn), bv = expf(ig - mn) * v_s[tt * VB + tid];
      m = mn;
      const float* kt = k_s + tt * dim;
      const float* qt = q_s + tt * dim;
      float acc = 0.0f;
      if (DIM > 0) {
#pragma unroll
        for (int d = 0; d < (DIM > 0 ? DIM : 1); ++d) {
          const float s = fmaf(S_r[d], a, kt[d] * bv);
          S_r[d] = s;
          acc = fmaf(s, qt[d], acc);
        }
      } else {
        for (int d = 0; d < dim; ++d) {
          const float s = fmaf(S_s[d * VB + tid], a, kt[d] * bv);
          S_s[d * VB + tid] = s;
          acc = fmaf(s, qt[d], acc);
        }
      }
      const size_t row = (size_t)(row0 + t0 + tt);
      if (active) num[(row * H + h) * cols + jj] = acc;
      if (jj == 0) m_row[row * H + h] = mn;
    }
  }
  if (active) {
    if (DIM > 0) {
#pragma unroll
      for (int d = 0; d < (DIM > 0 ? DIM : 1); ++d) st[(size_t)d * cols + jj] = S_r[d];
    } else {
      for (int d = 0; d < dim; ++d) st[(size_t)d * cols + jj] = S_s[d * VB + tid];
    }
    st[(size_t)dim * cols + jj] = m;
  }
}

constexpr int OUT_THREADS = 128;

template <typename TW, typename TO>
__global__ void __launch_bounds__(OUT_THREADS)
mlstm_out_kernel(const float* num, const float* m_row, const float* proj, int ld, int g_off, int H,
                 int vdim, const TW* __restrict__ norm_w, float eps, TO* out) {
  __shared__ float red[OUT_THREADS / 32 + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t row = blockIdx.x;
  const int h = blockIdx.y, tid = threadIdx.x;
  const float* nr = num + (row * H + h) * (size_t)(vdim + 1);
  const float den = fmaxf(fabsf(nr[vdim]), expf(-m_row[row * H + h])) + 1e-6f;
  float s = 0.0f;
  for (int j = tid; j < vdim; j += OUT_THREADS) {
    const float o = nr[j] / den;
    s = fmaf(o, o, s);
  }
  s = sb_warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int i = 0; i < OUT_THREADS / 32; ++i) total += red[i];
    red[OUT_THREADS / 32] = 1.0f / sqrtf(total / (float)vdim + eps);
  }
  __syncthreads();
  const float inv = red[OUT_THREADS / 32];
  const float* g = proj + row * ld + g_off + h * vdim;
  for (int j = tid; j < vdim; j += OUT_THREADS) {
    const float o = (nr[j] / den) * inv * sb_to_f32<TW>(norm_w[h * vdim + j]);
    out[row * (size_t)(H * vdim) + h * vdim + j] = sb_from_f32<TO>(o / (1.0f + expf(-g[j])));
  }
}

template <int DIM, typename TB>
int launch_scan(dim3 grid, size_t smem, cudaStream_t stream, const float* proj, int ld,
                const int32_t* seq_row0, const int32_t* seq_slot, int H, int dim, int vdim, const void* ib,
                const void* fb, float cap, float q_scale, float* state, float* num, float* m_row) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel<DIM, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_mlstm_scan: shared memory opt-in failed: %s", cudaGetErrorString(e));
  }
  sb_launch<SB_K_OTHER>(mlstm_scan_kernel<DIM, TB>, grid, dim3(VB), smem, stream, proj, ld, seq_row0, seq_slot, H, dim,
                        vdim, (const TB*)ib, (const TB*)fb, cap, q_scale, state, num, m_row);
  return SB_OK;
}

}  // namespace

extern "C" int sb_mlstm_scan(const float* proj, int n_seqs, const int32_t* seq_row0,
                             const int32_t* seq_slot, int n_heads, int dim, int vdim, const void* i_bias,
                             const void* f_bias, int bias_dtype, float cap, float q_scale, float* state,
                             float* num, float* m_row, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || dim <= 0 || vdim <= 0 || !proj || !seq_row0 || !seq_slot || !state || !num ||
      !m_row || !i_bias || !f_bias)
    SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: seqs=%d heads=%d dim=%d vdim=%d", n_seqs, n_heads, dim, vdim);
  if (!(cap > 0.0f)) SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: gate cap %g must be positive", cap);
  if (!sb_valid_dtype(bias_dtype)) SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: dtype code %d", bias_dtype);
  if (n_heads > 65535 || n_seqs > 2147483647 / 1) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_mlstm_scan: %d heads", n_heads);
  const int ld = 2 * n_heads * dim + 2 * n_heads * vdim + 2 * n_heads;
  const dim3 grid(n_seqs, n_heads, (vdim + 1 + VB - 1) / VB);
  const bool in_regs = dim == 16 || dim == 32 || dim == 64 || dim == 128;
  const size_t smem = sizeof(float) * ((size_t)2 * TC * dim + TC * VB + 2 * TC + (in_regs ? 0 : (size_t)dim * VB));
  if (smem > 200 * 1024) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_mlstm_scan: key size %d needs %zu bytes of shared memory", dim, smem);
  int rc = SB_OK;
#define SB_SCAN(D) rc = launch_scan<D, TB>(grid, smem, stream, proj, ld, seq_row0, seq_slot, n_heads, dim, vdim, i_bias, f_bias, cap, q_scale, state, num, m_row)
  SB_DISPATCH_DTYPE(bias_dtype, TB, {
    if (dim == 16) SB_SCAN(16);
    else if (dim == 32) SB_SCAN(32);
    else if (dim == 64) SB_SCAN(64);
    else if (dim == 128) SB_SCAN(128);
    else SB_SCAN(0);
  });
#undef SB_SCAN
  if (rc != SB_OK) return rc;
  SB_CHECK_LAUNCH("sb_mlstm_scan");
  return SB_OK;
}

extern "C" int sb_mlstm_out(const float* num, const float* m_row, const float* proj, int n_rows,
                            int n_heads, int dim, int vdim, const void* norm_w, int norm_w_dtype, float eps,
                            void* out, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || dim <= 0 || vdim <= 0 || !num || !m_row || !proj || !norm_w || !out)
    SB_FAIL(SB_ERR_ARG, "sb_mlstm_out: rows=%d heads=%d dim=%d vdim=%d", n_rows, n_heads, dim, vdim);
  if (!sb_valid_dtype(norm_w_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_mlstm_out: dtype codes %d %d", norm_w_dtype, out_dtype);
  if (n_heads > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_mlstm_out: %d heads", n_heads);
  const int ld = 2 * n_heads * dim + 2 * n_heads * vdim + 2 * n_heads;
  const int g_off = 2 * n_heads * dim + n_heads * vdim;
  SB_DISPATCH_DTYPE(norm_w_dtype, TW, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      sb_launch<SB_K_ELEMENTWISE>(mlstm_out_kernel<TW, TO>, dim3(n_rows, n_heads), dim3(OUT_THREADS), 0, stream, num,
                                  m_row, proj, ld, g_off, n_heads, vdim, (const TW*)norm_w, eps, (TO*)out);
    });
  });
  SB_CHECK_LAUNCH("sb_mlstm_out");
  return SB_OK;
}
