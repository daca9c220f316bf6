// Operand preparation and result finalisation kernels (all HBM-bound, each touches its data once).
#pragma once

#include "flk_common.cuh"

namespace flk {

// ---------------------------------------------------------------------------------------------
// prep_rows: X[n x d] (any of the two legal layouts) -> Xs[n_pad x ld] row-major with
//   Xs[i,k] = X[i,k] / sigma[k]   (zero for i >= n or k >= d)   and   norms[i] = sum_k Xs[i,k]^2.
// This is "mat / sigma" + square_norm of distance_kernel.py:151-154 done in one pass.  TIn may be
// narrower than T (fp32 data prepared for fp64 arithmetic, the reference's `no_single_kernel` upcast).
// A block handles 64 rows; columns are walked in chunks of 64 through a shared tile so that both
// the read (along whichever stride is 1) and the write (row-major) are coalesced.  The norm is
// summed by one thread per row in column order, so it is deterministic.
// ---------------------------------------------------------------------------------------------
constexpr int kPrepRows = 64;
constexpr int kPrepCols = 64;
constexpr int kPrepSubBlocks = 8;  // 64-row groups per CTA of prep_rows_kernel: a gated-off launch over 1e7 rows is
                                   // then 2e4 empty CTAs instead of 1.6e5 (0.3 ms of pure block scheduling)

template <typename T, typename TIn = T>
__global__ void __launch_bounds__(256) prep_rows_kernel(const TIn* __restrict__ X, int64_t n, int d,
                                                        int64_t rs, int64_t cs,
                                                        const T* __restrict__ sigma, T sigma_scalar,
                                                        int sigma_len, T* __restrict__ Xs, int ld,
                                                        int64_t n_pad,
                                                        T* __restrict__ norms, Gate gate) {
  if (!gate_open(gate)) return;
  __shared__ T tile[kPrepRows][kPrepCols + 1];
  __shared__ T sig[kPrepCols];
  const int tid = threadIdx.x;
  for (int sub = 0; sub < kPrepSubBlocks; ++sub) {
  const int64_t row0 = ((int64_t)blockIdx.x * kPrepSubBlocks + sub) * kPrepRows;
  if (row0 >= n_pad) break;  // uniform across the block
  T nrm = 0;
  for (int k0 = 0; k0 < ld; k0 += kPrepCols) {
    const int kw = min(kPrepCols, ld - k0);
    if (tid < kPrepCols) {
      int k = k0 + tid;
      T s = 1;
      if (k < d) s = (sigma != nullptr) ? sigma[sigma_len == 1 ? 0 : k] : sigma_scalar;
      sig[tid] = s;
    }
    // load (coalesced along the unit stride)
    if (cs == 1) {
      for (int idx = tid; idx < kPrepRows * kPrepCols; idx += 256) {
        int r = idx / kPrepCols, k = idx % kPrepCols;
        int64_t gi = row0 + r;
        T val = 0;
        if (gi < n && k0 + k < d) val = (T)X[gi * rs + (int64_t)(k0 + k)];
        tile[r][k] = val;
      }
    } else {
      for (int idx = tid; idx < kPrepRows * kPrepCols; idx += 256) {
        int k = idx / kPrepRows, r = idx % kPrepRows;
        int64_t gi = row0 + r;
        T val = 0;
        if (gi < n && k0 + k < d) val = (T)X[gi * rs + (int64_t)(k0 + k) * cs];
        tile[r][k] = val;
      }
    }
    __syncthreads();
    // scale + store row-major
    for (int idx = tid; idx < kPrepRows * kPrepCols; idx += 256) {
      int r = idx / kPrepCols, k = idx % kPrepCols;
      if (k < kw) {
        T val = tile[r][k] / sig[k];
        tile[r][k] = val;
        int64_t gi = row0 + r;
        if (gi < n_pad) Xs[gi * ld + k0 + k] = val;
      }
    }
    __syncthreads();
    if (tid < kPrepRows) {
      for (int k = 0; k < kw; ++k) {
        T val = tile[tid][k];
        nrm += val * val;
      }
    }
    __syncthreads();
  }
  if (tid < kPrepRows) {
    int64_t gi = row0 + tid;
    if (gi < n_pad && norms != nullptr) norms[gi] = nrm;
  }
  __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// norm_rows: out[i] = sum_k (X[i,k] / sigma)^2 for a scalar sigma (the stand-alone square_norm).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) norm_rows_kernel(const T* __restrict__ X, int64_t n, int d, int64_t rs,
                                                        int64_t cs, T sigma, T* __restrict__ out) {
  __shared__ T tile[kPrepRows][kPrepCols + 1];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * kPrepRows;
  T nrm = 0;
  for (int k0 = 0; k0 < d; k0 += kPrepCols) {
    const int kw = min(kPrepCols, d - k0);
    for (int idx = tid; idx < kPrepRows * kPrepCols; idx += 256) {
      int r, k;
      if (cs == 1) {
        r = idx / kPrepCols;
        k = idx % kPrepCols;
      } else {
        k = idx / kPrepRows;
        r = idx % kPrepRows;
      }
      int64_t gi = row0 + r;
      T val = 0;
      if (gi < n && k < kw) val = X[gi * rs + (int64_t)(k0 + k) * cs];
      tile[r][k] = val;
    }
    __syncthreads();
    if (tid < kPrepRows) {
      for (int k = 0; k < kw; ++k) {
        T val = tile[tid][k] / sigma;
        nrm += val * val;
      }
    }
    __syncthreads();
  }
  if (tid < kPrepRows && row0 + tid < n) out[row0 + tid] = nrm;
}

// ---------------------------------------------------------------------------------------------
// Vector operands are kept in a "column-chunked" layout  vbuf[t_chunks][s_pad][tt]  (tp = t_chunks
// * tt columns, zero padded): the slice a sweep needs for one chunk of tt columns and one tile of
// rows is then one contiguous run, which is what a bulk copy wants.
// prep_vec: v[s x t] (strided) -> vbuf, zero padded.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int64_t chunked_index(int64_t row, int col, int64_t rows_pad, int tt) {
  return ((int64_t)(col / tt) * rows_pad + row) * tt + (col % tt);
}

template <typename T>
__global__ void __launch_bounds__(256) prep_vec_kernel(const T* __restrict__ v, int64_t s, int t,
                                                       int64_t rs, int64_t cs, T* __restrict__ vbuf,
                                                       int64_t s_pad, int tp, int tt) {
  int64_t total = s_pad * tp;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = idx / tp;
    int c = (int)(idx % tp);
    T val = 0;
    if (r < s && c < t) val = v[r * rs + (int64_t)c * cs];
    vbuf[chunked_index(r, c, s_pad, tt)] = val;
  }
}

// ---------------------------------------------------------------------------------------------
// finalize: sums the per-chunk partial results raw[n_chunks][r_pad][tp] (fixed order, so the
// result is deterministic; rows from `main_rows` on have `n_chunks_tail` partials instead, see the
// two-segment grids of the tensor-core kernel), optionally adds add[r x t] (the "+ w" of fmmv.py:759), and writes
//   mode 0: out[r x t] with the caller's strides,
//   mode 1: a padded buffer in the column-chunked layout out[t_chunks][r_pad][tt] whose rows >= r
//           and columns >= t are zero (it becomes the vector operand of the second sweep of fdmmv).
// `timeout_word` (tensor-core sweeps only, else null): when a bounded wait of the sweep gave up, CTAs of that
// launch left their partials unwritten; every live result is then stored as NaN, so that a caller who never
// reads the status word cannot mistake the garbage for a product.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) finalize_kernel(const T* __restrict__ raw, int n_chunks,
                                                       int64_t r_pad, int tp, int64_t r, int t,
                                                       const T* __restrict__ add, int64_t add_rs,
                                                       int64_t add_cs, T* __restrict__ out,
                                                       int64_t out_rs, int64_t out_cs, int padded_out,
                                                       int tt, int64_t main_rows, int n_chunks_tail, Gate gate,
                                                       const int* __restrict__ timeout_word) {
  if (!gate_open(gate)) return;
  const bool poisoned = timeout_word != nullptr && *reinterpret_cast<const volatile int*>(timeout_word) != 0;
  int64_t total = r_pad * tp;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = idx / tp;
    int c = (int)(idx % tp);
    bool live = (i < r && c < t);
    T acc = 0;
    if (live) {
      const int nch = i < main_rows ? n_chunks : n_chunks_tail;
      for (int ch = 0; ch < nch; ++ch) acc += raw[(int64_t)ch * total + idx];
      if (add != nullptr) acc += add[i * add_rs + (int64_t)c * add_cs];
      if (poisoned) acc = (T)NAN;
    }
    if (padded_out) {
      out[chunked_index(i, c, r_pad, tt)] = acc;
    } else if (live) {
      out[i * out_rs + (int64_t)c * out_cs] = acc;
    }
  }
}

inline int grid_for(int64_t total, int block = 256, int max_blocks = 148 * 16) {
  int64_t b = ceil_div(total, block);
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

}  // namespace flk
