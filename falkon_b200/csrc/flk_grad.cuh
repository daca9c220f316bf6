// Pair weights of the backward pass of the kernel products.
//
// For out = K(X1, X2) v with upstream gradient G (n x t), or out = K(X1, X2) with upstream gradient S
// (n x m), every gradient the reference obtains by re-running the block product under autograd
// (falkon/mmv_ops/fmmv.py:405-485, falkon/mmv_ops/fmm.py KernelMmFnFull.backward) is a plain matrix
// product with
//
//     W[i][j] = 2 dk/dD2 (D2_ij) * s_ij,     s_ij = G_i . v_j   (or S_ij),
//
// where D2 is the squared distance of the sigma-scaled rows:  with a = W 1, b = W^T 1,
//     dL/dX1~ = a o X1~ - W X2~,   dL/dX2~ = b o X2~ - W^T X1~,
//     dL/dsigma_k = -(1 / sigma_k) sum_ij W_ij (x~_ik - c~_jk)^2,   dL/dv = K^T G.
// This file computes W in one pass: the distance by norm expansion exactly as the forward product does
// (the reference's autograd differentiates that same expansion, falkon/kernels/distance_kernel.py:88-101),
// the t-long dot G_i . v_j, the derivative of the radial profile, and the store.  Where the forward clamps
// D2 at 1e-20 the derivative is zero, as torch's clamp_min gives.  The products with W are left to the caller.
#pragma once

#include "flk_common.cuh"

namespace flk {

// 2 * d k / d D2 at the (clamped) squared distance d2
template <int KT>
__device__ __forceinline__ float kernel_dweight(float d2) {
  if (KT == FLK_GAUSSIAN) {
    return -expf(-0.5f * d2);
  } else if (KT == FLK_LAPLACIAN) {
    const float s = sqrtf(d2);
    return -expf(-s) / s;
  } else if (KT == FLK_MATERN15) {
    return -3.0f * expf(-sqrtf(d2) * 1.7320508075688772f);
  } else {
    const float s = sqrtf(d2) * 2.23606797749979f;
    return (-5.0f / 3.0f) * (1.0f + s) * expf(-s);
  }
}

template <int KT>
__device__ __forceinline__ double kernel_dweight(double d2) {
  if (KT == FLK_GAUSSIAN) {
    return -exp_nonpositive(-0.5 * d2);
  } else if (KT == FLK_LAPLACIAN) {
    const double s = sqrt(d2);
    return -exp_nonpositive(-s) / s;
  } else if (KT == FLK_MATERN15) {
    return -3.0 * exp_nonpositive(-sqrt(d2) * 1.7320508075688772);
  } else {
    const double s = sqrt(d2) * 2.23606797749979;
    return (-5.0 / 3.0) * (1.0 + s) * exp_nonpositive(-s);
  }
}

// A, B: sigma-scaled operands in the padded workspace layout (rows to a multiple of 512, features to `ld`).
// Upstream gradient: factors G (n x t) and V (m x t) when t > 0, else the dense matrix S (n x m); all three
// are caller tensors with arbitrary strides.
template <typename T, typename TIO, int KT>
__global__ void __launch_bounds__(256)
    kgrad_kernel(const T* __restrict__ A, const T* __restrict__ an, const T* __restrict__ B,
                 const T* __restrict__ bn, int ld, const TIO* __restrict__ G, int64_t g_rs, int64_t g_cs,
                 const TIO* __restrict__ V, int64_t v_rs, int64_t v_cs, int t, const TIO* __restrict__ S,
                 int64_t s_rs, int64_t s_cs, TIO* __restrict__ out, int64_t n, int64_t m, int64_t out_rs,
                 int64_t out_cs) {
  constexpr int BT = 64, DK = 16;
  __shared__ T As[BT][DK + 1];
  __shared__ T Bs[BT][DK + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t row0 = (int64_t)blockIdx.y * BT, col0 = (int64_t)blockIdx.x * BT;
  T acc[4][4], sacc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = sacc[i][j] = 0;

  for (int k0 = 0; k0 < ld; k0 += DK) {
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

  // s_ij = G_i . v_j, same tiling over the t columns (caller tensors: bounds-checked loads)
  for (int k0 = 0; k0 < t; k0 += DK) {
    for (int idx = tid; idx < BT * DK; idx += 256) {
      const int r = idx / DK, k = idx - r * DK;
      const bool kin = (k0 + k) < t;
      As[r][k] = (kin && row0 + r < n) ? (T)G[(row0 + r) * g_rs + (int64_t)(k0 + k) * g_cs] : (T)0;
      Bs[r][k] = (kin && col0 + r < m) ? (T)V[(col0 + r) * v_rs + (int64_t)(k0 + k) * v_cs] : (T)0;
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
        for (int j = 0; j < 4; ++j) sacc[i][j] += a[i] * b[j];
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
      const T d2 = (ani - (T)2 * acc[i][j]) + bn[c];
      const T s = t > 0 ? sacc[i][j] : (T)S[r * s_rs + c * s_cs];
      const T wgt = d2 < (T)1e-20 ? (T)0 : kernel_dweight<KT>(d2) * s;
      out[r * out_rs + c * out_cs] = (TIO)wgt;
    }
  }
}

template <typename T, typename TIO>
int launch_kgrad(int kernel, const T* A, const T* an, const T* B, const T* bn, int ld, const TIO* G, int64_t g_rs,
                 int64_t g_cs, const TIO* V, int64_t v_rs, int64_t v_cs, int t, const TIO* S, int64_t s_rs,
                 int64_t s_cs, TIO* out, int64_t n, int64_t m, int64_t out_rs, int64_t out_cs, cudaStream_t stream) {
  dim3 grid((unsigned)ceil_div(m, 64), (unsigned)ceil_div(n, 64), 1);
#define FLK_KGRAD_CASE(KT)                                                                                       \
  case KT:                                                                                                       \
    kgrad_kernel<T, TIO, KT><<<grid, 256, 0, stream>>>(A, an, B, bn, ld, G, g_rs, g_cs, V, v_rs, v_cs, t, S, s_rs, \
                                                       s_cs, out, n, m, out_rs, out_cs);                         \
    break;
  switch (kernel) {
    FLK_KGRAD_CASE(FLK_GAUSSIAN)
    FLK_KGRAD_CASE(FLK_LAPLACIAN)
    FLK_KGRAD_CASE(FLK_MATERN15)
    FLK_KGRAD_CASE(FLK_MATERN25)
    default: return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
  }
#undef FLK_KGRAD_CASE
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

}  // namespace flk
