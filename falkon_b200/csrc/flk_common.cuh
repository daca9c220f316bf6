// Shared definitions for the kernel-vector-product library (device math, error plumbing).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/falkon_b200.h"

namespace flk {

// ---------------------------------------------------------------------------------------------
// Error reporting: every entry point returns a status code and leaves a message that
// flk_last_error() hands back; nothing throws, aborts or traps.
// ---------------------------------------------------------------------------------------------
inline char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define FLK_CUDA_TRY(expr)                                                                      \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess)                                                                      \
      return ::flk::fail(FLK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                         __FILE__, __LINE__);                                                   \
  } while (0)

#define FLK_TRY(expr)            \
  do {                           \
    int _s = (expr);             \
    if (_s != FLK_OK) return _s; \
  } while (0)

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline int64_t ceil_div(int64_t x, int64_t m) { return (x + m - 1) / m; }

// All padded row counts are multiples of this many rows, so every tile shape used by the
// SIMT kernel (128 x 128 / 128 x 64) and by the tensor-core kernel (512 x 128) divides them.
constexpr int64_t kRowPad = 512;

// Device-side gate.  When the tensor-core path is chosen its SIMT alternative is launched behind
// it; which of the two does the work is decided by a flag the image builder writes in device
// memory, so the choice costs no host round trip.  A gated kernel returns at once unless
// (*flag != 0) == want.  flag == nullptr means "always run".
struct Gate {
  const int* flag;
  int want;
};
__device__ __forceinline__ bool gate_open(const Gate& g) {
  if (g.flag == nullptr) return true;
  return (*reinterpret_cast<const volatile int*>(g.flag) != 0) == (g.want != 0);
}

// ---------------------------------------------------------------------------------------------
// Kernel functions on the clamped squared distance (in length-scale units).
//   Gaussian      exp(-d2/2)                                   (distance_kernel.py:140-159)
//   Laplacian     exp(-sqrt(d2))                               (distance_kernel.py:182-204)
//   Matern 1.5    (1 + sqrt(3 d2)) exp(-sqrt(3 d2))            (distance_kernel.py:246-257)
//   Matern 2.5    (1 + sqrt(5 d2) + 5/3 d2) exp(-sqrt(5 d2))   (distance_kernel.py:258-269)
// fp32 uses the MUFU approximations (ex2.approx, sqrt.approx); fp64 uses full-precision libm.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float kLog2e = 1.4426950408889634f;

template <int KT>
__device__ __forceinline__ float kernel_eval(float d2) {
  if (KT == FLK_GAUSSIAN) {
    return ex2_approx(d2 * (-0.5f * kLog2e));
  } else if (KT == FLK_LAPLACIAN) {
    return ex2_approx(sqrt_approx(d2) * (-kLog2e));
  } else if (KT == FLK_MATERN15) {
    float s = sqrt_approx(d2) * 1.7320508075688772f;
    return (1.0f + s) * ex2_approx(s * (-kLog2e));
  } else {
    float s = sqrt_approx(d2) * 2.23606797749979f;
    return fmaf(d2, 5.0f / 3.0f, 1.0f + s) * ex2_approx(s * (-kLog2e));
  }
}

template <int KT>
__device__ __forceinline__ double kernel_eval(double d2) {
  if (KT == FLK_GAUSSIAN) {
    return exp(-0.5 * d2);
  } else if (KT == FLK_LAPLACIAN) {
    return exp(-sqrt(d2));
  } else if (KT == FLK_MATERN15) {
    double s = sqrt(d2) * 1.7320508075688772;
    return (1.0 + s) * exp(-s);
  } else {
    double s = sqrt(d2) * 2.23606797749979;
    return (d2 * (5.0 / 3.0) + s + 1.0) * exp(-s);
  }
}

// 16-byte asynchronous global->shared copy (Ampere-style cp.async; used by the SIMT kernel).
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
template <int BYTES>
__device__ __forceinline__ void cp_async_small(void* smem, const void* gmem) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(s), "l"(gmem), "n"(BYTES));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

}  // namespace flk
