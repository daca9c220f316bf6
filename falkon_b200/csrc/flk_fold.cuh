// Folded reduction-side images for the Gaussian single-column sweep (flk_tc.cuh, FOLD = true).
//
//   out_i = sum_j k(a_i, b_j) vec_j = sum_j sign(vec_j) 2^(acc_ij + log2 |vec_j|)
//
// The exponent acc_ij comes out of the tensor-core product of the operand images.  Its reduction-side part,
// -|b_j|^2 / 2 (carried as two or three fp16 pieces), is a per-row constant, so log2 |vec_j| can be added to it
// when the image is built; the sweep's epilogue then needs no vector at all, only the sign.  Rows are written in
// an order that makes the sign constant over every 128-row tile: entries with vec_j >= 0 first (in their original
// order), a gap of null rows (contributing exactly 2^-200 -> 0), then the negative entries right-aligned at the end
// of a fixed number of tiles (ceil(s / 128) + 1, so that the layout does not depend on the data).  The magnitudes
// are stored relative to 2^e, e = exponent of max_j |vec_j|: the terms that matter then have exponents near zero,
// where the fp32 accumulator of the tensor cores resolves 2^-24 or better; the sweep multiplies its sums by 2^e.
//
// Three launches per folded operand: count (non-negative entries per 128-row block, maximum magnitude), scan (one
// CTA; exclusive prefix of the counts, first negative tile, exponent), build (one thread per row: scaled fp16
// split of the row as in prep_images_kernel, norm - log2 |vec| split into fp16 pieces, 16-byte stores into the
// row's place in the swizzled tile image).  The vector changes with every call, so this image is never cached.
#pragma once

#include "flk_tc.cuh"

namespace flk {
namespace tc {

constexpr int kFoldWordsSweep1 = 8;    // status-block word where the fold block of the first sweep starts
constexpr int kFoldWordsSweep2 = 16;   // ... of the second sweep
constexpr float kFoldNullPiece = 200.0f;  // a null row's exponent is -200: 2^-200 flushes to zero in fp32
constexpr double kFoldFlushBelow = -120.0;  // entries this far (in log2) below the largest one are stored as null

inline int fold_tiles(int64_t s) { return (int)ceil_div(std::max<int64_t>(s, 1), (int64_t)kTileRows) + 1; }
inline int64_t fold_image_rows(int64_t s) { return round_up((int64_t)fold_tiles(s) * kTileRows, kRowPad); }
inline int fold_blocks(int64_t s) { return (int)ceil_div(std::max<int64_t>(s, 1), (int64_t)kTileRows); }

constexpr int kFoldCountSub = 8;  // 128-row blocks counted per CTA (fewer, fatter CTAs: the kernel is all overhead)

__global__ void __launch_bounds__(128) fold_count_kernel(const float* __restrict__ vec, int64_t s, int nblk,
                                                         int* __restrict__ blk_pos, int* __restrict__ fold,
                                                         int* __restrict__ status) {
  unsigned max_bits = 0u;
  bool bad = false;
  for (int sub = 0; sub < kFoldCountSub; ++sub) {
    const int b = blockIdx.x * kFoldCountSub + sub;
    if (b >= nblk) break;  // uniform across the block
    const int64_t row = (int64_t)b * kTileRows + threadIdx.x;
    const bool live = row < s;
    const float v = live ? vec[row] : 0.0f;
    const float a = fabsf(v);
    const bool finite = a <= 3.4028234663852886e38f;  // false for inf and NaN
    bad = bad || (live && !finite);
    const int cnt = __syncthreads_count(live && !(v < 0.0f));
    if (threadIdx.x == 0) blk_pos[b] = cnt;
    if (live && finite) max_bits = max(max_bits, __float_as_uint(a));
  }
  if (bad) atomicOr(status + kStatusRange, 1);  // the SIMT kernels reproduce inf / NaN propagation
  max_bits = __reduce_max_sync(0xFFFFFFFFu, max_bits);
  if ((threadIdx.x & 31) == 0 && max_bits != 0u) atomicMax(reinterpret_cast<unsigned*>(fold + kFoldMaxBits), max_bits);
}

// One CTA: blk_pos[nblk] -> exclusive prefix sums in place; fold block filled in.
__global__ void __launch_bounds__(1024) fold_scan_kernel(int* __restrict__ blk_pos, int nblk, int64_t s,
                                                         int n_col_tiles, int* __restrict__ fold) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < nblk; base += 1024) {
    const int i = base + tid;
    const int x = i < nblk ? blk_pos[i] : 0;
    int incl = x;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int y = __shfl_up_sync(0xFFFFFFFFu, incl, off);
      if (lane >= off) incl += y;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int y = __shfl_up_sync(0xFFFFFFFFu, w, off);
        if (lane >= off) w += y;
      }
      warp_sums[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int before = carry_s + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - x;
    if (i < nblk) blk_pos[i] = before;
    __syncthreads();
    if (tid == 0) carry_s += warp_sums[31];
    __syncthreads();
  }
  if (tid == 0) {
    const int64_t positives = carry_s;
    const int64_t negatives = s - positives;
    const int64_t neg_start = (int64_t)n_col_tiles * kTileRows - negatives;
    fold[kFoldNegTile] = (int)(neg_start / kTileRows);
    fold[kFoldPositives] = (int)positives;
    const unsigned bits = (unsigned)fold[kFoldMaxBits];
    int e = (int)(bits >> 23) - 127;  // exponent of the largest magnitude (0 when every entry is zero)
    if (bits == 0u) e = 0;
    if (e < -126) e = -126;
    fold[kFoldExp] = e;
  }
}

// Shared-memory staging of the build kernel: every thread assembles the K-vector of its row ([ch | cl | ch | 1.. |
// -m.. | 0..], kp fp16 values) in a private strip, region by region, and then moves it out with 16-byte stores.
// The strips are kFoldStripHalves apart: 104 fp16 = 52 words, an odd multiple of 4 words, so that the 16-byte
// reads of consecutive rows spread over the banks.
constexpr int kFoldStripHalves = 104;  // >= the largest padded K of the resident kernel (96), multiple of 8

__device__ __forceinline__ void fold_store_strip(__half* __restrict__ img, int64_t dst_row, int kp,
                                                 const __half* strip) {
  const int64_t tile = dst_row / kTileRows;
  const int r = (int)(dst_row - tile * kTileRows);
  __half* base = img + tile * ((int64_t)kTileRows * kp);
  for (int c = 0; c < kp / 8; ++c)
    *reinterpret_cast<uint4*>(base + image_offset(r, c * 8)) = *reinterpret_cast<const uint4*>(strip + c * 8);
}

__global__ void __launch_bounds__(128) fold_build_kernel(const float* __restrict__ X, int64_t s, int64_t rs, int64_t cs,
                                                         int d, const float* __restrict__ sigma, float sigma_scalar,
                                                         int sigma_len, float scale, int kp, int npieces,
                                                         const float* __restrict__ vec,
                                                         const int* __restrict__ blk_pos, int nblk,
                                                         const int* __restrict__ fold, int n_col_tiles,
                                                         __half* __restrict__ img_b, int* __restrict__ status) {
  __shared__ float xin[kTileRows * 33];
  __shared__ __align__(16) __half strips[kTileRows * kFoldStripHalves];
  __shared__ float sig[32];
  __shared__ int warp_pos[4];
  const int tid = threadIdx.x;
  const int64_t positives = fold[kFoldPositives];
  const int64_t neg_start = (int64_t)n_col_tiles * kTileRows - (s - positives);
  __half* strip = strips + tid * kFoldStripHalves;
  const __half one = __float2half_rn(1.0f), zero = __float2half_rn(0.0f);
  {  // a null row to start with: every slot zero (the exponent piece is set below)
    uint4* z = reinterpret_cast<uint4*>(strip);
    for (int c = 0; c < kp / 8; ++c) z[c] = make_uint4(0u, 0u, 0u, 0u);
  }
  if ((int)blockIdx.x >= nblk) {
    // the gap between the non-negative entries and the (right-aligned) negative ones: null rows
    const int64_t g = positives + (int64_t)((int)blockIdx.x - nblk) * kTileRows + tid;
    strip[3 * d + npieces] = __float2half_rn(-kFoldNullPiece);
    if (g < neg_start) fold_store_strip(img_b, g, kp, strip);
    return;
  }
  const int64_t row0 = (int64_t)blockIdx.x * kTileRows;
  if (tid < 32) sig[tid] = (tid < d) ? (sigma != nullptr ? sigma[sigma_len == 1 ? 0 : tid] : sigma_scalar) : 1.0f;
  if (cs == 1 && rs == d) {
    // dense row-major rows: the tile is one contiguous run
    const int64_t base = row0 * d;
    const int64_t limit = s * d;
    for (int idx = tid; idx < kTileRows * d; idx += 128) {
      const int r = idx / d, k = idx - r * d;
      xin[r * 33 + k] = (base + idx < limit) ? X[base + idx] : 0.0f;
    }
  } else if (cs == 1) {
    for (int idx = tid; idx < kTileRows * d; idx += 128) {
      const int r = idx / d, k = idx - r * d;
      const int64_t gi = row0 + r;
      xin[r * 33 + k] = (gi < s) ? X[gi * rs + k] : 0.0f;
    }
  } else {
    for (int idx = tid; idx < kTileRows * d; idx += 128) {
      const int k = idx / kTileRows, r = idx - k * kTileRows;
      const int64_t gi = row0 + r;
      xin[r * 33 + k] = (gi < s) ? X[gi * rs + (int64_t)k * cs] : 0.0f;
    }
  }
  __syncthreads();
  const int r = tid;
  const bool live = (row0 + r) < s;
  const float v = live ? vec[row0 + r] : 0.0f;
  const float a = fabsf(v);
  // the row's data: scaled features split into fp16 hi + lo, squared norm of what the two parts represent.  A row
  // whose vector entry is zero stays a null row and needs none of it.
  bool data = live && a > 0.0f && a <= 3.4028234663852886e38f;
  double nrm = 0.0;
  bool out_of_range = false;
  if (data || live) {
    for (int k = 0; k < d; ++k) {
      const float xs = xin[r * 33 + k] / sig[k];  // x / sigma, rounded as in the reference
      float xt = xs * scale;
      if (!(fabsf(xt) <= 400.0f)) {
        out_of_range = true;
        xt = 0.0f;
      }
      const __half hi = __float2half_rn(xt);
      const float hif = __half2float(hi);
      const __half lo = __float2half_rn(xt - hif);
      const double rep = (double)hif + (double)__half2float(lo);
      nrm += rep * rep;
      strip[k] = hi;           // B: [ch | cl | ch]
      strip[d + k] = lo;
      strip[2 * d + k] = hi;
    }
  }
  double half_norm = 0.5 * nrm;
  if (half_norm > (double)kNormLimit) {
    out_of_range = true;
    half_norm = 0.0;
  }
  if (out_of_range && live) atomicOr(status + kStatusRange, 1);
  const bool nonneg = !(v < 0.0f);
  // position among the block's rows of the same sign
  const unsigned ballot = __ballot_sync(0xFFFFFFFFu, live && nonneg);
  if ((tid & 31) == 0) warp_pos[tid >> 5] = __popc(ballot);
  __syncthreads();
  int pos_before = 0;  // non-negative live rows of this block before this one
  for (int w = 0; w < (tid >> 5); ++w) pos_before += warp_pos[w];
  pos_before += __popc(ballot & ((1u << (tid & 31)) - 1u));
  if (!live) return;
  const int64_t blk_before = blk_pos[blockIdx.x];  // non-negative rows in earlier blocks (all of which are live)
  const int64_t dst = nonneg ? blk_before + pos_before : neg_start + (row0 - blk_before) + (r - pos_before);
  // the exponent piece: |b|^2 / 2 - (log2 |v| - e), split into fp16 pieces (last one rounded up)
  float lg = 0.0f;
  if (data) {
    // log2 |v| - e in fp32: |v| = 2^ex * mant with mant in [1, 2); log2f of the mantissa is accurate to an ulp of a
    // number below 1, the exponents subtract exactly
    int ex;
    const float mant = frexpf(a, &ex);  // a = mant * 2^ex, mant in [0.5, 1)
    lg = (float)(ex - fold[kFoldExp]) + log2f(mant);
    if ((double)lg < kFoldFlushBelow || out_of_range) data = false;
  }
  if (data) {
    double rem = half_norm - (double)lg;
    for (int i = 0; i < npieces; ++i) {
      const float remf = __double2float_ru(rem);
      const float pc = __half2float(i == npieces - 1 ? __float2half_ru(remf) : __float2half_rn(remf));
      strip[3 * d + npieces + i] = __float2half_rn(-pc);
      strip[3 * d + i] = one;
      rem -= (double)pc;
    }
  } else {
    for (int k = 0; k < 3 * d; ++k) strip[k] = zero;
    strip[3 * d + npieces] = __float2half_rn(-kFoldNullPiece);
  }
  fold_store_strip(img_b, dst, kp, strip);
}

// Builds the folded image of X (s live rows) for the vector `vec` (dense, s entries) into img_b
// (fold_image_rows(s) rows); `fold` = this sweep's fold block (zeroed by the caller), `blk_pos` = scratch of
// fold_blocks(s) ints.  Three launches.
inline int build_folded_image(int kernel, const void* X, int64_t s, int64_t rs, int64_t cs, int d,
                              const float* sigma_dev, float sigma_scalar, int sigma_len, const float* vec,
                              int* blk_pos, int* fold, void* img_b, int* status, cudaStream_t stream) {
  const int nblk = fold_blocks(s), tiles = fold_tiles(s);
  const int kp = (int)padded_k(d);
  const float scale = (float)sqrt(scale_sq_for(kernel));
  fold_count_kernel<<<(nblk + kFoldCountSub - 1) / kFoldCountSub, 128, 0, stream>>>(vec, s, nblk, blk_pos, fold, status);
  FLK_CUDA_TRY(cudaGetLastError());
  fold_scan_kernel<<<1, 1024, 0, stream>>>(blk_pos, nblk, s, tiles, fold);
  FLK_CUDA_TRY(cudaGetLastError());
  fold_build_kernel<<<nblk + 2, 128, 0, stream>>>(reinterpret_cast<const float*>(X), s, rs, cs, d, sigma_dev,
                                                   sigma_scalar, sigma_len, scale, kp, norm_pieces(d), vec, blk_pos,
                                                   nblk, fold, tiles, reinterpret_cast<__half*>(img_b), status);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

}  // namespace tc
}  // namespace flk
