// Wide-T SIMT kernel-vector product:  raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t]  for
// up to 32 vector columns per pass.
//
// kmv_simt_kernel contracts at most four vector columns per pass and re-evaluates the kernel block
// for every further group of four, which is the right trade when t is small.  For many columns
// (multi-output regression, one-hot targets: t = 32 in the dense benchmark configuration) this
// kernel evaluates each kernel value ONCE: a CTA forms the BR x BC block of kernel values exactly
// like kmv_simt_kernel (register micro-tiles over cp.async-staged operand chunks, reference
// operation order, clamp, kernel function), parks it in shared memory, and multiplies it with the
// BC x 32 tile of `vec` in a second register-tiled product whose 8 x 2 accumulators per thread
// live in registers for the whole chunk of column tiles.  Per kernel value that is d + 32
// multiply-adds instead of 8 (d + 4).  Every output element is owned by one thread, so there is
// no cross-thread reduction; chunk partials are summed by finalize_kernel in a fixed order.
#pragma once

#include "flk_common.cuh"
#include "flk_simt.cuh"

namespace flk {

constexpr int kWideT = 32;  // vector columns per pass

template <typename T>
constexpr size_t wide_smem_bytes() {
  using C = SimtCfg<T>;
  constexpr int BR = 16 * C::TR, BC = 16 * C::TC, LD = C::DK + C::VEC;
  return sizeof(T) * (size_t)(2 * BR * LD + 2 * BC * LD + 2 * BC * kWideT + 2 * BC + BC * (BR + C::VEC));
}

template <typename T, int KT>
__global__ void __launch_bounds__(256, 1) kmv_wide_kernel(SimtArgs<T> p) {
  using C = SimtCfg<T>;
  using Vec = typename C::Vec;
  constexpr int TR = C::TR, TC = C::TC, DK = C::DK, VEC = C::VEC;
  constexpr int BR = 16 * TR, BC = 16 * TC, LD = DK + VEC, KLD = BR + VEC, TW = kWideT;
  static_assert(TR == 8, "the second product assumes 8 rows per thread");
  if (!gate_open(p.gate)) return;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* As = reinterpret_cast<T*>(smem_raw);  // [2][BR][LD]
  T* Bs = As + 2 * BR * LD;                // [2][BC][LD]
  T* vs = Bs + 2 * BC * LD;                // [2][BC][TW]
  T* bns = vs + 2 * BC * TW;               // [2][BC]
  T* Ks = bns + 2 * BC;                    // [BC][KLD]  kernel values of the current tile, column-major

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int row_tile = blockIdx.x % p.row_tiles;
  const int chunk = blockIdx.x / p.row_tiles;
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int tile_end = min(tile_begin + p.tiles_per_chunk, p.n_col_tiles);
  const int ntiles = tile_end - tile_begin;
  const int nk = (p.ld + DK - 1) / DK;
  const int steps = ntiles * nk;
  const int ld = p.ld;
  const T* Ag = p.A + (int64_t)row_tile * BR * ld;

  T an[TR];
#pragma unroll
  for (int i = 0; i < TR; ++i) an[i] = p.an[(int64_t)row_tile * BR + ty + 16 * i];

  T acc[TR][TC];
  T oacc[TR][2];  // rows ty * 8 + i, vector columns 2 * tx + {0, 1}
#pragma unroll
  for (int i = 0; i < TR; ++i) {
    oacc[i][0] = 0;
    oacc[i][1] = 0;
#pragma unroll
    for (int j = 0; j < TC; ++j) acc[i][j] = 0;
  }

  auto issue = [&](int s) {
    const int tl = s / nk, kc = s - tl * nk;
    const int buf = s & 1;
    const int k0 = kc * DK;
    const int kw = min(DK, ld - k0);
    const int pieces = kw / VEC;  // 16-byte pieces per row
    if (nk > 1 || s == 0) {
      T* dst = As + (nk > 1 ? buf : 0) * BR * LD;
      for (int q = tid; q < BR * pieces; q += 256) {
        int r = q / pieces, pc = q - r * pieces;
        cp_async16(dst + r * LD + pc * VEC, Ag + (int64_t)r * ld + k0 + pc * VEC);
      }
    }
    const int64_t col0 = (int64_t)(tile_begin + tl) * BC;
    T* dstb = Bs + buf * BC * LD;
    const T* Bg = p.B + col0 * ld + k0;
    for (int q = tid; q < BC * pieces; q += 256) {
      int r = q / pieces, pc = q - r * pieces;
      cp_async16(dstb + r * LD + pc * VEC, Bg + (int64_t)r * ld + pc * VEC);
    }
    if (kc == 0) {
      const int vb = tl & 1;
      // BC rows of TW values: one contiguous run in the column-chunked vector layout
      const T* vg = p.vec + ((int64_t)blockIdx.y * p.s_pad + col0) * TW;
      T* vd = vs + vb * BC * TW;
      constexpr int V16 = BC * TW * (int)sizeof(T) / 16;
      for (int q = tid; q < V16; q += 256)
        cp_async16(reinterpret_cast<char*>(vd) + 16 * q, reinterpret_cast<const char*>(vg) + 16 * q);
      if (tid < BC) cp_async_small<(int)sizeof(T)>(bns + vb * BC + tid, p.bn + col0 + tid);
    }
  };

  issue(0);
  cp_async_commit();

  int tl = 0, kc = 0;
  for (int s = 0; s < steps; ++s) {
    if (s + 1 < steps) issue(s + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const T* a_s = As + (nk > 1 ? (s & 1) : 0) * BR * LD;
    const T* b_s = Bs + (s & 1) * BC * LD;
    const int kw = min(DK, ld - kc * DK);
    for (int k = 0; k < kw; k += VEC) {
      Vec b[TC];
#pragma unroll
      for (int j = 0; j < TC; ++j) b[j] = *reinterpret_cast<const Vec*>(b_s + (tx + 16 * j) * LD + k);
#pragma unroll
      for (int i = 0; i < TR; ++i) {
        Vec a = *reinterpret_cast<const Vec*>(a_s + (ty + 16 * i) * LD + k);
#pragma unroll
        for (int j = 0; j < TC; ++j) acc[i][j] = dot_vec(a, b[j], acc[i][j]);
      }
    }

    if (kc == nk - 1) {
      // 1. kernel values of this tile -> shared memory (column-major: Ks[column][row])
      const T* bn_s = bns + (tl & 1) * BC;
#pragma unroll
      for (int j = 0; j < TC; ++j) {
        const T bnj = bn_s[tx + 16 * j];
#pragma unroll
        for (int i = 0; i < TR; ++i) {
          // same operation order as the reference: (|a|^2 - 2 a.b) + |b|^2, then clamp
          T d2 = (an[i] - (T)2 * acc[i][j]) + bnj;
          d2 = d2 < (T)1e-20 ? (T)1e-20 : d2;
          Ks[(tx + 16 * j) * KLD + ty + 16 * i] = kernel_eval<KT>(d2);
          acc[i][j] = 0;
        }
      }
      __syncthreads();
      // 2. out[rows ty*8.., columns 2 tx..] += K[rows, :] vec[:, columns]
      const T* v_s = vs + (tl & 1) * BC * TW;
#pragma unroll 4
      for (int k = 0; k < BC; ++k) {
        T kr[TR];
#pragma unroll
        for (int i = 0; i < TR; i += VEC) {
          const Vec kk = *reinterpret_cast<const Vec*>(Ks + k * KLD + ty * TR + i);
          if constexpr (VEC == 2) {
            kr[i] = kk.x;
            kr[i + 1] = kk.y;
          } else {
            kr[i] = kk.x;
            kr[i + 1] = kk.y;
            kr[i + 2] = kk.z;
            kr[i + 3] = kk.w;
          }
        }
        const T v0 = v_s[k * TW + 2 * tx], v1 = v_s[k * TW + 2 * tx + 1];
#pragma unroll
        for (int i = 0; i < TR; ++i) {
          oacc[i][0] += kr[i] * v0;
          oacc[i][1] += kr[i] * v1;
        }
      }
      kc = 0;
      ++tl;
    } else {
      ++kc;
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TR; ++i) {
    const int64_t row = (int64_t)row_tile * BR + ty * TR + i;
    T* dst = p.raw + ((int64_t)chunk * p.r_pad + row) * p.tp + blockIdx.y * TW + 2 * tx;
    dst[0] = oacc[i][0];
    dst[1] = oacc[i][1];
  }
}

template <typename T, int KT>
int launch_wide(const SimtArgs<T>& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  constexpr size_t smem = wide_smem_bytes<T>();
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_wide_kernel<T, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid((unsigned)(args.row_tiles * n_chunks), (unsigned)t_chunks, 1);
  kmv_wide_kernel<T, KT><<<grid, 256, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <typename T>
int launch_wide_any(int kernel, const SimtArgs<T>& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_wide<T, FLK_GAUSSIAN>(args, n_chunks, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_wide<T, FLK_LAPLACIAN>(args, n_chunks, t_chunks, stream);
    case FLK_MATERN15: return launch_wide<T, FLK_MATERN15>(args, n_chunks, t_chunks, stream);
    case FLK_MATERN25: return launch_wide<T, FLK_MATERN25>(args, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace flk
