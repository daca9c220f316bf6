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
// it; which of the two does the work is decided by flags the image builders write in device
// memory, so the choice costs no host round trip.  There are kRangeWords consecutive flag words
// (one for what changes with every call, one per operand whose images may be kept across calls);
// a gated kernel returns at once unless (any word != 0) == want.  flag == nullptr means "always run".
constexpr int kRangeWords = 3;
struct Gate {
  const int* flag;
  int want;
};
__device__ __forceinline__ bool range_raised(const int* words) {
  const volatile int* w = reinterpret_cast<const volatile int*>(words);
  return (w[0] | w[1] | w[2]) != 0;
}
__device__ __forceinline__ bool gate_open(const Gate& g) {
  if (g.flag == nullptr) return true;
  return range_raised(g.flag) == (g.want != 0);
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

// exp(x) for x <= 0 in double precision, about half the FP64-pipe work of the general library routine (the fp64
// kernels at small d spend most of their time here).  x = (64 m + j) ln2 / 64 + r with |r| <= ln2 / 128:
// exp(x) = 2^m * 2^(j/64) * (1 + r + r^2/2 + ... + r^5/120); the integer part comes out of the 1.5 * 2^52
// rounding trick, 2^(j/64) from a 64-entry table, the truncation error of the polynomial is below 4e-17.
// Results below the normal range (x < -708) are flushed to zero.
__device__ const double kExp2Table64[64] = {
    1.0, 1.0108892860517005, 1.0218971486541166, 1.0330248790212284,
    1.0442737824274138, 1.0556451783605572, 1.0671404006768237, 1.0787607977571199,
    1.0905077326652577, 1.102382583307841, 1.1143867425958924, 1.1265216186082418,
    1.1387886347566916, 1.1511892299529827, 1.1637248587775775, 1.1763969916502812,
    1.189207115002721, 1.202156731452703, 1.215247359980469, 1.22848053610687,
    1.241857812073484, 1.255380757024691, 1.2690509571917332, 1.2828700160787783,
    1.2968395546510096, 1.3109612115247644, 1.3252366431597413, 1.339667524053303,
    1.3542555469368927, 1.3690024229745905, 1.383909881963832, 1.3989796725383112,
    1.4142135623730951, 1.42961333839197, 1.4451808069770467, 1.460917794180647,
    1.4768261459394993, 1.4929077282912648, 1.5091644275934228, 1.5255981507445384,
    1.5422108254079407, 1.559004400237837, 1.5759808451078865, 1.593142151342267,
    1.6104903319492543, 1.6280274218573478, 1.645755478153965, 1.6636765803267364,
    1.681792830507429, 1.7001063537185235, 1.718619298122478, 1.7373338352737062,
    1.7562521603732995, 1.7753764925265212, 1.7947090750031072, 1.8142521755003989,
    1.8340080864093424, 1.8539791250833855, 1.8741676341103, 1.8945759815869656,
    1.9152065613971474, 1.9360617934922943, 1.9571441241754002, 1.978456026387951};

__device__ __forceinline__ double exp_nonpositive(double x) {
  const double kMagic = 6755399441055744.0;                 // 1.5 * 2^52
  const double t = fma(x, 92.33248261689366, kMagic);       // x * 64 / ln2, rounded to an integer in the low bits
  const int n = __double2loint(t);
  const double nf = t - kMagic;
  double r = fma(nf, -0.010830424695086549, x);             // ln2 / 64, high part (20 trailing zero bits)
  r = fma(nf, -1.162596423439437e-12, r);                   // low part
  double p = fma(r, 1.0 / 120.0, 1.0 / 24.0);
  p = fma(p, r, 1.0 / 6.0);
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p *= r;                                                   // expm1(r)
  const double tj = __ldg(&kExp2Table64[n & 63]);
  const double y = fma(tj, p, tj);
  const long long bits = __double_as_longlong(y) + ((long long)(n >> 6) << 52);
  return x < -708.0 ? 0.0 : __longlong_as_double(bits);
}

template <int KT>
__device__ __forceinline__ double kernel_eval(double d2) {
  if (KT == FLK_GAUSSIAN) {
    return exp_nonpositive(-0.5 * d2);
  } else if (KT == FLK_LAPLACIAN) {
    return exp_nonpositive(-sqrt(d2));
  } else if (KT == FLK_MATERN15) {
    double s = sqrt(d2) * 1.7320508075688772;
    return (1.0 + s) * exp_nonpositive(-s);
  } else {
    double s = sqrt(d2) * 2.23606797749979;
    return (d2 * (5.0 / 3.0) + s + 1.0) * exp_nonpositive(-s);
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
