// Kernel matrix assembly:  out[i][j] = k(a_i, b_j)  for i < n, j < m, written with the caller's strides.
//
// This is the "fmm" product of the reference (falkon/mmv_ops/fmm.py:298-388): the preconditioner
// needs K(C, C) once per fit (falkon/preconditioner/flk_preconditioner.py:80-92).  The arithmetic
// follows the reference: rows pre-divided by sigma, squared distance by norm expansion in the order
// (|a|^2 - 2 a.b) + |b|^2, clamp at 1e-20, then the kernel function.  T is the arithmetic type and
// TOut the stored type: with `no_single_kernel` (the reference's default, falkon/mmv_ops/fmm.py:619-622)
// fp32 data is evaluated in fp64 and rounded once on store.
//
// The kernel is bound by the n x m store (4 or 8 bytes per entry); a 64 x 64 CTA tile with a 4 x 4
// register micro-tile and 16-feature shared-memory steps keeps the FMA work far below that.
#pragma once

#include "flk_common.cuh"

namespace flk {

template <typename T, typename TOut, int KT>
__global__ void __launch_bounds__(256) kmat_kernel(const T* __restrict__ A, const T* __restrict__ an,
                                                   const T* __restrict__ B, const T* __restrict__ bn, int ld,
                                                   TOut* __restrict__ out, int64_t n, int64_t m, int64_t out_rs,
                                                   int64_t out_cs) {
  constexpr int BT = 64, DK = 16;
  __shared__ T As[BT][DK + 1];
  __shared__ T Bs[BT][DK + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t row0 = (int64_t)blockIdx.y * BT, col0 = (int64_t)blockIdx.x * BT;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;
  for (int k0 = 0; k0 < ld; k0 += DK) {
    // operand rows are padded (rows to a multiple of 512, features to `ld`), so no bounds checks on loads
    for (int idx = tid; idx < BT * DK; idx += 256) {
      const int r = idx / DK, k = idx - r * DK;
      const bool in = (k0 + k) < ld;
      As[r][k] = in ? A[(row0 + r) * ld + k0 + k] : (T)0;
      Bs[r][k] = in ? B[(col0 + r) * ld + k0 + k] : (T)0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < DK; ++k) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[ty + 16 * i][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[tx + 16 * j][k];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row0 + ty + 16 * i;
    if (r >= n) continue;
    const T ani = an[r];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = col0 + tx + 16 * j;
      if (c >= m) continue;
      T d2 = (ani - (T)2 * acc[i][j]) + bn[c];
      d2 = d2 < (T)1e-20 ? (T)1e-20 : d2;
      out[r * out_rs + c * out_cs] = (TOut)kernel_eval<KT>(d2);
    }
  }
}

template <typename T, typename TOut>
int launch_kmat(int kernel, const T* A, const T* an, const T* B, const T* bn, int ld, TOut* out, int64_t n, int64_t m,
                int64_t out_rs, int64_t out_cs, cudaStream_t stream) {
  dim3 grid((unsigned)ceil_div(m, 64), (unsigned)ceil_div(n, 64), 1);
  switch (kernel) {
    case FLK_GAUSSIAN:
      kmat_kernel<T, TOut, FLK_GAUSSIAN><<<grid, 256, 0, stream>>>(A, an, B, bn, ld, out, n, m, out_rs, out_cs);
      break;
    case FLK_LAPLACIAN:
      kmat_kernel<T, TOut, FLK_LAPLACIAN><<<grid, 256, 0, stream>>>(A, an, B, bn, ld, out, n, m, out_rs, out_cs);
      break;
    case FLK_MATERN15:
      kmat_kernel<T, TOut, FLK_MATERN15><<<grid, 256, 0, stream>>>(A, an, B, bn, ld, out, n, m, out_rs, out_cs);
      break;
    case FLK_MATERN25:
      kmat_kernel<T, TOut, FLK_MATERN25><<<grid, 256, 0, stream>>>(A, an, B, bn, ld, out, n, m, out_rs, out_cs);
      break;
    default: return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
  }
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

}  // namespace flk
