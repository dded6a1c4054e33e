// The linear recurrence with a matrix state and a decay per key channel,
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,
//
// per head, token by token in float32, for prompts, portions and single tokens alike: every token
// is the same arithmetic whatever the step brings, so a result does not depend on how a sequence
// was cut or on what else the step holds.  The decay is either one value per (token, head, key
// channel) read from a tensor, or one fixed value per head.
//
// A column of S (the `dim` values that belong to one value channel) is shared by 16 lanes that
// keep their runs of it in registers for the whole step; a warp holds two columns, a block
// eight.  Per token a lane multiplies and adds its run, and the lanes' partial dot products
// with q are added by four exchanges.  The next token's q, k, decay and v are requested before
// the running token is computed.  State: float32 [slot, heads, vdim, dim] (column by column).
#include "common.cuh"

namespace {

constexpr int LANES = 16;            // lanes that share a column
constexpr int COLS = 8;              // columns of a block (four warps)

template <int NPL>
struct Tok {
  float q[NPL], k[NPL], a[NPL], v;
};

template <int NPL>
__device__ __forceinline__ void load_tok(Tok<NPL>& t, const float* row, int q_off, int k_off, int v_off,
                                         const float* arow, float a_head, int c0, int dim, int col, bool col_ok) {
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = c0 + i;
    const bool ok = c < dim;
    t.q[i] = ok ? row[q_off + c] : 0.0f;
    t.k[i] = ok ? row[k_off + c] : 0.0f;
    t.a[i] = arow ? (ok ? arow[c] : 1.0f) : a_head;
  }
  t.v = col_ok ? row[v_off + col] : 0.0f;
}

template <int NPL>
__global__ void __launch_bounds__(LANES * COLS)
linrec_scan_kernel(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay,
                   const float* __restrict__ head_decay, const int32_t* seq_row0, const int32_t* seq_slot,
                   int n_heads, int dim, int vdim, float* state, float* out) {
  sb_pdl_launch();
  const int b = blockIdx.z, h = blockIdx.y;
  const int sub = threadIdx.x % LANES;
  const int col = blockIdx.x * COLS + threadIdx.x / LANES;
  const bool col_ok = col < vdim;
  const int c0 = sub * NPL;
  const int row0 = seq_row0[b], n = seq_row0[b + 1] - row0;
  const int slot = seq_slot[b];
  const float a_head = head_decay ? head_decay[h] : 1.0f;
  sb_pdl_wait();
  float* srow = state + (((size_t)slot * n_heads + h) * vdim + (col_ok ? col : 0)) * dim;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) S[i] = (col_ok && c0 + i < dim) ? srow[c0 + i] : 0.0f;
  const int qo = q_off + h * dim, ko = k_off + h * dim, vo = v_off + h * vdim;
  const size_t per_row = (size_t)n_heads * dim;
  Tok<NPL> cur, nxt;
  if (n > 0)
    load_tok<NPL>(cur, proj + (size_t)row0 * ld, qo, ko, vo,
                  decay ? decay + (size_t)row0 * per_row + (size_t)h * dim : nullptr, a_head, c0, dim, col, col_ok);
  for (int t = 0; t < n; ++t) {
    if (t + 1 < n) {
      const size_t r = (size_t)row0 + t + 1;
      load_tok<NPL>(nxt, proj + r * ld, qo, ko, vo, decay ? decay + r * per_row + (size_t)h * dim : nullptr,
                    a_head, c0, dim, col, col_ok);
    }
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      S[i] = fmaf(cur.a[i], S[i], cur.k[i] * cur.v);
      acc = fmaf(S[i], cur.q[i], acc);
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (sub == 0 && col_ok) out[((size_t)(row0 + t) * n_heads + h) * vdim + col] = acc;
    cur = nxt;
  }
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < NPL; ++i)
      if (c0 + i < dim) srow[c0 + i] = S[i];
  }
}

}  // namespace

extern "C" int sb_linrec_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay,
                              const float* head_decay, int n_seqs, const int32_t* seq_row0,
                              const int32_t* seq_slot, int n_heads, int dim, int vdim, float* state,
                              float* out, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || dim <= 0 || vdim <= 0 || !proj || !state || !out || !seq_row0 || !seq_slot)
    SB_FAIL(SB_ERR_ARG, "sb_linrec_scan: seqs=%d heads=%d dim=%d vdim=%d", n_seqs, n_heads, dim, vdim);
  if ((decay == nullptr) == (head_decay == nullptr))
    SB_FAIL(SB_ERR_ARG, "sb_linrec_scan: exactly one of the two kinds of decay is given");
  if (dim > 16 * LANES) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_linrec_scan: key size %d is above %d", dim, 16 * LANES);
  if (n_heads > 65535 || n_seqs > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_linrec_scan: %d heads, %d sequences", n_heads, n_seqs);
  const dim3 grid((vdim + COLS - 1) / COLS, n_heads, n_seqs);
  const int npl = (dim + LANES - 1) / LANES;
#define SB_LINREC_LAUNCH(N)                                                                                   \
  sb_launch<SB_K_OTHER>(linrec_scan_kernel<N>, grid, dim3(LANES * COLS), 0, stream, proj, ld, q_off, k_off,  \
                        v_off, decay, head_decay, seq_row0, seq_slot, n_heads, dim, vdim, state, out)
  if (npl <= 1) SB_LINREC_LAUNCH(1);
  else if (npl <= 2) SB_LINREC_LAUNCH(2);
  else if (npl <= 4) SB_LINREC_LAUNCH(4);
  else if (npl <= 8) SB_LINREC_LAUNCH(8);
  else SB_LINREC_LAUNCH(16);
#undef SB_LINREC_LAUNCH
  SB_CHECK_LAUNCH("sb_linrec_scan");
  return SB_OK;
}
