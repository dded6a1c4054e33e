// The matrix-memory recurrence (mLSTM) with exponential gates and a running maximum.
//
// Per sequence and head, with q (scaled), k in R^dim, v in R^vdim and the log gates
// i_t (input) and f_t (forget):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          S in R^{dim x vdim}
//     n_t = the same recurrence with k_t alone                                   n in R^dim
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// S, n and m start at zero.  The gates come from two pre-activations x_i, x_f (a projection plus
// a bias): i = cap tanh(x_i / cap), f = logsigmoid(cap tanh(x_f / cap)).
//
// n is S for a value that is always one, so the state is kept as one matrix of vdim + 1 columns,
// and the columns are independent of each other.  A column's dim values are shared out over DS
// lanes of a warp (lane s keeps d = s, s + DS, ... in registers), the lanes' partial sums of
// S_t^T q_t meet by shuffles, and columns never meet: every column also keeps a copy of m, so
// that no column reads what another one writes.  State per slot: float32 [heads, vdim + 1,
// col_stride], a column's dim values side by side and its copy of m after them (col_stride is
// dim + 1 or more; a multiple of 4 lets runs of four values travel in 16-byte accesses).  The walk is the
// recurrence itself, token by token in float32, for prompts, portions of prompts and single
// tokens alike, so a position's result does not depend on how its sequence was cut into steps.
// Tokens are staged in shared memory a chunk at a time; per chunk the gates are worked out by a
// thread per token, the running maximum by one thread in order (an add and a max per token),
// and the two decay factors again by a thread per token.
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

constexpr int SCAN_THREADS = 256;
constexpr int MAX_TC = 32;      // most tokens staged at a time

__device__ __forceinline__ float log_sigmoid(float z) {
  return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// DS lanes share a column, NPT values of it each (DS * NPT >= dim; values past dim stay zero).
// A chunk's q, k, v and gate pre-activations are copied into one of two shared-memory stages
// with cp.async while the chunk before it is walked.
template <int DS, int NPT, typename TB>
__global__ void __launch_bounds__(SCAN_THREADS)
mlstm_scan_kernel(const float* proj, int ld, const int32_t* seq_row0, const int32_t* seq_slot, int H,
                  int dim, int vdim, int col_stride, int tc, const TB* __restrict__ i_bias, const TB* __restrict__ f_bias,
                  float cap, float q_scale, float* state, float* num, float* m_row) {
  constexpr int CPB = SCAN_THREADS / DS;   // columns per block
  // Which of a column's values lane ls keeps as S[i]: with NPT a multiple of 4, runs of four
  // neighbours (16-byte shared-memory loads of k and q), the runs dealt out over the lanes;
  // else every DS-th value.
  constexpr bool VEC = NPT % 4 == 0;
  auto d_of = [](int ls_, int i) { return VEC ? (i / 4) * (DS * 4) + ls_ * 4 + i % 4 : ls_ + DS * i; };
  extern __shared__ __align__(16) float smem[];
  const int dim_p = DS * NPT;
  const int stage = (2 * tc * dim_p + tc * CPB + 2 * tc + 3) & ~3;      // floats of one stage: q, k, v, x_i, x_f (16-byte steps)
  float* ig_s = smem + 2 * stage;          // [tc] log input gate, then its factor exp(i - m)
  float* fg_s = ig_s + tc;                 // [tc] log forget gate, then its factor exp(f + m' - m)
  float* m_s = fg_s + tc;                  // [tc + 1]: m before the chunk, then after each token
  sb_pdl_launch();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int c = tid / DS, ls = tid % DS;
  const int jj = blockIdx.z * CPB + c, cols = vdim + 1;
  const bool active = jj < cols;
  const int row0 = seq_row0[b], T = seq_row0[b + 1] - row0;
  float* st = state + (((size_t)seq_slot[b] * H + h) * cols + (active ? jj : 0)) * (size_t)col_stride;
  const float bi = sb_to_f32<TB>(i_bias[h]), bf = sb_to_f32<TB>(f_bias[h]);
  const int q_off = h * dim, k_off = H * dim + h * dim, v_off = 2 * H * dim + h * vdim;
  const int i_off = 2 * H * dim + 2 * H * vdim + h, f_off = i_off + H;
  // what cp.async never writes: the padding past dim, and the columns past vdim (1 for the
  // normalizer's column, 0 beyond)
  for (int e = tid; e < 2 * stage; e += SCAN_THREADS) {
    const int r = e % stage;
    float v = 0.0f;
    if (r >= 2 * tc * dim_p && r < 2 * tc * dim_p + tc * CPB)
      v = blockIdx.z * CPB + (r - 2 * tc * dim_p) % CPB == vdim ? 1.0f : 0.0f;
    smem[e] = v;
  }
  __syncthreads();
  sb_pdl_wait();

  auto load_chunk = [&](int t0, int buf) {
    const int nt = min(tc, T - t0);
    float* q_s = smem + buf * stage;
    float* k_s = q_s + tc * dim_p;
    float* v_s = k_s + tc * dim_p;
    float* xi_s = v_s + tc * CPB;
    float* xf_s = xi_s + tc;
    for (int e = tid; e < nt * dim; e += SCAN_THREADS) {
      const int tt = e / dim, d = e % dim;
      const float* src = proj + (size_t)(row0 + t0 + tt) * ld;
      cp_async4(q_s + tt * dim_p + d, src + q_off + d);
      cp_async4(k_s + tt * dim_p + d, src + k_off + d);
    }
    const int nv = min(CPB, vdim - (int)blockIdx.z * CPB);      // columns of this block that are values
    for (int e = tid; e < nt * nv; e += SCAN_THREADS) {
      const int tt = e / nv, j = e % nv;
      cp_async4(v_s + tt * CPB + j, proj + (size_t)(row0 + t0 + tt) * ld + v_off + blockIdx.z * CPB + j);
    }
    if (tid < nt) {
      const float* src = proj + (size_t)(row0 + t0 + tid) * ld;
      cp_async4(xi_s + tid, src + i_off);
      cp_async4(xf_s + tid, src + f_off);
    }
    cp_async_commit();
  };

  load_chunk(0, 0);
  float S[NPT];
#pragma unroll
  for (int g = 0; g < (VEC ? NPT / 4 : NPT); ++g) {
    if (VEC) {                       // a run of four in one 16-byte load where it lies inside the column
      const int d = d_of(ls, g * 4);
      if (active && d + 3 < dim && col_stride % 4 == 0) {
        const float4 v = *reinterpret_cast<const float4*>(st + d);
        S[(g * 4) % NPT] = v.x; S[(g * 4 + 1) % NPT] = v.y; S[(g * 4 + 2) % NPT] = v.z; S[(g * 4 + 3) % NPT] = v.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) S[(g * 4 + e) % NPT] = (active && d + e < dim) ? st[d + e] : 0.0f;
      }
    } else {
      const int d = d_of(ls, g);
      S[g % NPT] = (active && d < dim) ? st[d] : 0.0f;
    }
  }
  if (tid == 0) m_s[0] = st[dim];
  float m_last = 0.0f;
  int buf = 0;
  for (int t0 = 0; t0 < T; t0 += tc, buf ^= 1) {
    const int nt = min(tc, T - t0);
    if (t0 + tc < T) {
      load_chunk(t0 + tc, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* q_s = smem + buf * stage;
    const float* k_s = q_s + tc * dim_p;
    const float* v_s = k_s + tc * dim_p;
    const float* xi_s = v_s + tc * CPB;
    const float* xf_s = xi_s + tc;
    if (tid < nt) {
      ig_s[tid] = cap * tanhf((xi_s[tid] + bi) / cap);
      fg_s[tid] = log_sigmoid(cap * tanhf((xf_s[tid] + bf) / cap));
    }
    __syncthreads();
    if (tid == 0) {
      float m = m_s[0];
      for (int tt = 0; tt < nt; ++tt) {
        m = fmaxf(fg_s[tt] + m, ig_s[tt]);
        m_s[tt + 1] = m;
      }
    }
    __syncthreads();
    if (tid < nt) {
      const float mn = m_s[tid + 1];
      const float keep = expf(fg_s[tid] + m_s[tid] - mn), take = expf(ig_s[tid] - mn);
      fg_s[tid] = keep;
      ig_s[tid] = take;
      if (blockIdx.z == 0) m_row[(size_t)(row0 + t0 + tid) * H + h] = mn;
    }
    __syncthreads();
    // DS tokens at a time: every lane keeps its partial sum of each of them, and the DS x DS
    // partial sums are added up across the lanes in log2(DS) exchanges of halves (DS - 1 shuffles
    // for DS tokens), after which lane ls holds the whole sum of token ls of the group.
    for (int g0 = 0; g0 < nt; g0 += DS) {
      float acc[DS];
#pragma unroll
      for (int u = 0; u < DS; ++u) {
        const int tt = g0 + u;
        acc[u] = 0.0f;
        if (tt < nt) {
          const float a = fg_s[tt], bv = ig_s[tt] * v_s[tt * CPB + c];
          const float* kt = k_s + tt * dim_p;
          const float* qt = q_s + tt * dim_p;
          float acc1 = 0.0f;
          if (VEC) {
#pragma unroll
            for (int i4 = 0; i4 < NPT / 4; ++i4) {
              const float4 kv = *reinterpret_cast<const float4*>(kt + i4 * (DS * 4) + ls * 4);
              const float4 qv = *reinterpret_cast<const float4*>(qt + i4 * (DS * 4) + ls * 4);
              const float k4[4] = {kv.x, kv.y, kv.z, kv.w}, q4[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float sv = fmaf(S[i4 * 4 + e], a, k4[e] * bv);
                S[i4 * 4 + e] = sv;
                if (e & 1) acc1 = fmaf(sv, q4[e], acc1);
                else acc[u] = fmaf(sv, q4[e], acc[u]);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
              const float sv = fmaf(S[i], a, kt[ls + DS * i] * bv);
              S[i] = sv;
              if (i & 1) acc1 = fmaf(sv, qt[ls + DS * i], acc1);
              else acc[u] = fmaf(sv, qt[ls + DS * i], acc[u]);
            }
          }
          acc[u] += acc1;
        }
      }
#pragma unroll
      for (int o = DS / 2; o > 0; o >>= 1) {
        const bool up = (ls & o) != 0;
#pragma unroll
        for (int u = 0; u < o; ++u) {
          const float give = up ? acc[u] : acc[u + o];
          const float keep = up ? acc[u + o] : acc[u];
          acc[u] = keep + __shfl_xor_sync(0xffffffffu, give, o);
        }
      }
      if (active && g0 + ls < nt) num[((size_t)(row0 + t0 + g0 + ls) * H + h) * cols + jj] = acc[0] * q_scale;
    }
    m_last = m_s[nt];
    __syncthreads();                       // everyone is done with this stage and with m_s
    if (tid == 0) m_s[0] = m_last;
  }
  if (active) {
#pragma unroll
    for (int g = 0; g < (VEC ? NPT / 4 : NPT); ++g) {
      if (VEC) {
        const int d = d_of(ls, g * 4);
        if (d + 3 < dim && col_stride % 4 == 0) {
          *reinterpret_cast<float4*>(st + d) =
              make_float4(S[(g * 4) % NPT], S[(g * 4 + 1) % NPT], S[(g * 4 + 2) % NPT], S[(g * 4 + 3) % NPT]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (d + e < dim) st[d + e] = S[(g * 4 + e) % NPT];
        }
      } else {
        const int d = d_of(ls, g);
        if (d < dim) st[d] = S[g % NPT];
      }
    }
    if (ls == 0) st[dim] = m_last;
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

template <int DS, int NPT, typename TB>
int launch_scan(int n_seqs, int tc, cudaStream_t stream, const float* proj, int ld, const int32_t* seq_row0,
                const int32_t* seq_slot, int H, int dim, int vdim, int col_stride, const void* ib, const void* fb, float cap,
                float q_scale, float* state, float* num, float* m_row) {
  constexpr int CPB = SCAN_THREADS / DS;
  const size_t smem = sizeof(float) * (2 * ((((size_t)2 * tc * DS * NPT + (size_t)tc * CPB + 2 * tc) + 3) & ~(size_t)3) + 3 * tc + 1);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel<DS, NPT, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) SB_FAIL(SB_ERR_CUDA, "sb_mlstm_scan: shared memory opt-in failed: %s", cudaGetErrorString(e));
  }
  const dim3 grid(n_seqs, H, (vdim + 1 + CPB - 1) / CPB);
  sb_launch<SB_K_OTHER>(mlstm_scan_kernel<DS, NPT, TB>, grid, dim3(SCAN_THREADS), smem, stream, proj, ld, seq_row0,
                        seq_slot, H, dim, vdim, col_stride, tc, (const TB*)ib, (const TB*)fb, cap, q_scale, state, num, m_row);
  return SB_OK;
}

}  // namespace

extern "C" int sb_mlstm_scan(const float* proj, int n_seqs, const int32_t* seq_row0,
                             const int32_t* seq_slot, int n_heads, int dim, int vdim, const void* i_bias,
                             const void* f_bias, int bias_dtype, float cap, float q_scale, int max_new,
                             float* state, int col_stride, float* num, float* m_row, cudaStream_t stream) {
  if (col_stride < dim + 1) SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: a state column of %d values cannot hold %d + 1", col_stride, dim);
  if (n_seqs <= 0 || n_heads <= 0 || dim <= 0 || vdim <= 0 || !proj || !seq_row0 || !seq_slot || !state || !num ||
      !m_row || !i_bias || !f_bias)
    SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: seqs=%d heads=%d dim=%d vdim=%d", n_seqs, n_heads, dim, vdim);
  if (!(cap > 0.0f)) SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: gate cap %g must be positive", cap);
  if (!sb_valid_dtype(bias_dtype)) SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: dtype code %d", bias_dtype);
  if (n_heads > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_mlstm_scan: %d heads", n_heads);
  if (max_new < 1) SB_FAIL(SB_ERR_ARG, "sb_mlstm_scan: max_new = %d", max_new);
  if (dim > 1024) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_mlstm_scan: key size %d is above 1024", dim);
  const int ld = 2 * n_heads * dim + 2 * n_heads * vdim + 2 * n_heads;
  // tokens staged at a time: as many as keep q and k of a chunk within 32 KB
  int tc = MAX_TC;
  while (tc > 4 && (size_t)tc * dim * 8 > 32 * 1024) tc >>= 1;
  while (tc > 1 && tc / 2 >= max_new) tc >>= 1;            // no longer than the step's longest portion
  int rc = SB_OK;
#define SB_SCAN(DS, NPT) rc = launch_scan<DS, NPT, TB>(n_seqs, tc, stream, proj, ld, seq_row0, seq_slot, n_heads, dim, vdim, col_stride, i_bias, f_bias, cap, q_scale, state, num, m_row)
  SB_DISPATCH_DTYPE(bias_dtype, TB, {
    // 16 lanes a column up to 256 values: with 32 lanes the exchanges cost more than the warps gain
    // (a 2,048-token prompt at dim 128: 472 to 931 us against 490 to 627 us, one token 25 to 38 us against 15 to 20 us)
    if (dim <= 16) SB_SCAN(16, 1);
    else if (dim <= 32) SB_SCAN(16, 2);
    else if (dim <= 64) SB_SCAN(16, 4);
    else if (dim <= 128) SB_SCAN(16, 8);
    else if (dim <= 256) SB_SCAN(16, 16);
    else if (dim <= 512) SB_SCAN(32, 16);
    else SB_SCAN(32, 32);
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
