// SIMT (FP32 / FP64 FMA-pipe) kernel-vector product:  raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t]
//
// Serves every dtype / feature count / kernel function; the tensor-core kernels (flk_tc.cuh,
// flk_tck.cuh) take over for fp32 with up to 1024 features, flk_wide.cuh / flk_dmma.cuh for many
// vector columns.  The (rows x columns) kernel block lives only
// in registers: a CTA owns a tile of BR rows, keeps it in shared memory, streams tiles of BC
// columns through a cp.async double buffer, forms the BR x BC dot products with an 8 x TC
// register micro-tile per thread, applies  d2 = max(|a|^2 + |b|^2 - 2 a.b, 1e-20)  and the
// kernel function in registers and immediately contracts with the TT columns of `vec`.
// Row sums are combined across the 16 threads that share a row with warp shuffles at the end,
// and written to a per-chunk partial buffer that finalize_kernel sums in a fixed order
// (no atomics: results are bit-reproducible run to run).
#pragma once

#include "flk_common.cuh"

namespace flk {

template <typename T>
struct SimtCfg;
template <>
struct SimtCfg<float> {
  static constexpr int TR = 8, TC = 8, DK = 32, VEC = 4;
  typedef float4 Vec;
};
template <>
struct SimtCfg<double> {
  static constexpr int TR = 8, TC = 4, DK = 16, VEC = 2;
  typedef double2 Vec;
};

__device__ __forceinline__ float dot_vec(const float4& a, const float4& b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  acc = fmaf(a.w, b.w, acc);
  return acc;
}
__device__ __forceinline__ double dot_vec(const double2& a, const double2& b, double acc) {
  acc = fma(a.x, b.x, acc);
  acc = fma(a.y, b.y, acc);
  return acc;
}

template <typename T>
struct SimtArgs {
  const T* A;    // [r_pad x ld] scaled rows (output side)
  const T* an;   // [r_pad] squared norms
  const T* B;    // [s_pad x ld] scaled rows (reduction side)
  const T* bn;   // [s_pad]
  const T* vec;  // [t_chunks][s_pad][TT], zero padded
  T* raw;        // [n_chunks][r_pad][tp]
  int ld;        // padded feature count (multiple of VEC)
  int tp;        // padded number of vector columns (multiple of TT)
  int64_t r_pad;
  int64_t s_pad;
  int row_tiles;        // ceil(r / BR)
  int n_col_tiles;      // ceil(s / BC)
  int tiles_per_chunk;  // column tiles per chunk
  int n_chunks;         // chunks of the reduction side (row_tiles x n_chunks virtual blocks per column group)
  Gate gate;            // run only when the gate is open (see flk_common.cuh)
};

template <typename T, int TT>
constexpr size_t simt_smem_bytes() {
  using C = SimtCfg<T>;
  constexpr int BR = 16 * C::TR, BC = 16 * C::TC, LD = C::DK + C::VEC;
  return sizeof(T) * (size_t)(2 * BR * LD + 2 * BC * LD + 2 * BC * TT + 2 * BC);
}

template <typename T, int KT, int TT>
__global__ void __launch_bounds__(256, (TT == 1 ? 2 : 1)) kmv_simt_kernel(SimtArgs<T> p) {
  using C = SimtCfg<T>;
  using Vec = typename C::Vec;
  constexpr int TR = C::TR, TC = C::TC, DK = C::DK, VEC = C::VEC;
  constexpr int BR = 16 * TR, BC = 16 * TC, LD = DK + VEC;
  if (!gate_open(p.gate)) return;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* As = reinterpret_cast<T*>(smem_raw);  // [2][BR][LD]
  T* Bs = As + 2 * BR * LD;                // [2][BC][LD]
  T* vs = Bs + 2 * BC * LD;                // [2][BC][TT]
  T* bns = vs + 2 * BC * TT;               // [2][BC]

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  // Virtual block index: a launch may cover the (row tile, chunk) pairs with fewer CTAs than pairs.  The gated
  // alternative of a tensor-core call is launched that way -- when its gate is closed (the normal case) a few
  // hundred CTAs return at once instead of tens of thousands.
  for (int vb = blockIdx.x; vb < p.row_tiles * p.n_chunks; vb += gridDim.x) {
  const int row_tile = vb % p.row_tiles;
  const int chunk = vb / p.row_tiles;
  const int t0 = blockIdx.y * TT;
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
  T oacc[TR][TT];
#pragma unroll
  for (int i = 0; i < TR; ++i) {
#pragma unroll
    for (int t = 0; t < TT; ++t) oacc[i][t] = 0;
#pragma unroll
    for (int j = 0; j < TC; ++j) acc[i][j] = 0;
  }

  // 16-byte pieces per row of a chunk: DK / VEC (a power of two) for a full chunk, fewer for the last one of a row.
  // Row and piece of copy q are q / pieces and the remainder; the division by the run-time count of the last chunk
  // is a multiplication by its 16-bit reciprocal (exact for q < 8192), computed once.
  constexpr int kFullPieces = DK / VEC;
  static_assert((kFullPieces & (kFullPieces - 1)) == 0 && BR * kFullPieces < 8192, "piece arithmetic");
  const int last_pieces = (ld - (nk - 1) * DK) / VEC;
  const int last_recip = (65536 + last_pieces - 1) / last_pieces;
  auto issue = [&](int s, int tl, int kc) {  // chunk kc of tile tl is step s
    const int buf = s & 1;
    const int k0 = kc * DK;
    const bool full = kc < nk - 1 || last_pieces == kFullPieces;
    const int pieces = full ? kFullPieces : last_pieces;
    const int recip = full ? 65536 / kFullPieces : last_recip;
    if (nk > 1 || s == 0) {
      T* dst = As + (nk > 1 ? buf : 0) * BR * LD;
      for (int q = tid; q < BR * pieces; q += 256) {
        const int r = (q * recip) >> 16, pc = q - r * pieces;
        cp_async16(dst + r * LD + pc * VEC, Ag + (int64_t)r * ld + k0 + pc * VEC);
      }
    }
    const int64_t col0 = (int64_t)(tile_begin + tl) * BC;
    T* dstb = Bs + buf * BC * LD;
    const T* Bg = p.B + col0 * ld + k0;
    for (int q = tid; q < BC * pieces; q += 256) {
      const int r = (q * recip) >> 16, pc = q - r * pieces;
      cp_async16(dstb + r * LD + pc * VEC, Bg + (int64_t)r * ld + pc * VEC);
    }
    if (kc == 0 && tid < BC) {
      const int vb = tl & 1;
      T* vd = vs + (vb * BC + tid) * TT;
      const T* vg = p.vec + ((int64_t)blockIdx.y * p.s_pad + col0 + tid) * TT;
      constexpr int VB = TT * (int)sizeof(T);
      if (VB == 4) {
        cp_async_small<4>(vd, vg);
      } else if (VB == 8) {
        cp_async_small<8>(vd, vg);
      } else if (VB == 16) {
        cp_async16(vd, vg);
      } else {
        cp_async16(vd, vg);
        cp_async16(reinterpret_cast<char*>(vd) + 16, reinterpret_cast<const char*>(vg) + 16);
      }
      cp_async_small<(int)sizeof(T)>(bns + vb * BC + tid, p.bn + col0 + tid);
    }
  };

  issue(0, 0, 0);
  cp_async_commit();

  int tl = 0, kc = 0;
  for (int s = 0; s < steps; ++s) {
    cp_async_wait<0>();  // chunk s has landed
    __syncthreads();     // ... for every thread, and every thread is done with step s - 1, whose buffers are free now
    // (one barrier per step: the copies of chunk s + 1 go into those buffers and have the whole step to land)
    if (s + 1 < steps) {
      if (kc + 1 == nk)
        issue(s + 1, tl + 1, 0);
      else
        issue(s + 1, tl, kc + 1);
    }
    cp_async_commit();

    const T* a_s = As + (nk > 1 ? (s & 1) : 0) * BR * LD;
    const T* b_s = Bs + (s & 1) * BC * LD;
    const int kw = min(DK, ld - kc * DK);
    auto k_iter = [&](int k) {
      Vec b[TC];
#pragma unroll
      for (int j = 0; j < TC; ++j) b[j] = *reinterpret_cast<const Vec*>(b_s + (tx + 16 * j) * LD + k);
#pragma unroll
      for (int i = 0; i < TR; ++i) {
        Vec a = *reinterpret_cast<const Vec*>(a_s + (ty + 16 * i) * LD + k);
#pragma unroll
        for (int j = 0; j < TC; ++j) acc[i][j] = dot_vec(a, b[j], acc[i][j]);
      }
    };
    for (int k = 0; k < kw; k += VEC) k_iter(k);

    if (kc == nk - 1) {
      const T* v_s = vs + (tl & 1) * BC * TT;
      const T* bn_s = bns + (tl & 1) * BC;
#pragma unroll
      for (int j = 0; j < TC; ++j) {
        const T bnj = bn_s[tx + 16 * j];
        T vv[TT];
#pragma unroll
        for (int t = 0; t < TT; ++t) vv[t] = v_s[(tx + 16 * j) * TT + t];
#pragma unroll
        for (int i = 0; i < TR; ++i) {
          // same operation order as the reference: (|a|^2 - 2 a.b) + |b|^2, then clamp
          T d2 = (an[i] - (T)2 * acc[i][j]) + bnj;
          d2 = d2 < (T)1e-20 ? (T)1e-20 : d2;
          const T kv = kernel_eval<KT>(d2);
#pragma unroll
          for (int t = 0; t < TT; ++t) oacc[i][t] += kv * vv[t];
          acc[i][j] = 0;
        }
      }
      kc = 0;
      ++tl;
    } else {
      ++kc;
    }
  }

  // combine the 16 threads (consecutive lanes) that hold partial sums of the same rows
#pragma unroll
  for (int i = 0; i < TR; ++i) {
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      T x = oacc[i][t];
      x += __shfl_xor_sync(0xffffffffu, x, 8);
      x += __shfl_xor_sync(0xffffffffu, x, 4);
      x += __shfl_xor_sync(0xffffffffu, x, 2);
      x += __shfl_xor_sync(0xffffffffu, x, 1);
      if (tx == 0) {
        int64_t row = (int64_t)row_tile * BR + ty + 16 * i;
        p.raw[((int64_t)chunk * p.r_pad + row) * p.tp + t0 + t] = x;
      }
    }
  }
  __syncthreads();  // the next virtual block reuses the shared buffers
  }
}

// Launch helper: one instantiation per (dtype, kernel function, TT).
template <typename T, int KT, int TT>
int launch_simt(const SimtArgs<T>& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  constexpr size_t smem = simt_smem_bytes<T, TT>();
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_simt_kernel<T, KT, TT>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  } else if (dev >= 16) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_simt_kernel<T, KT, TT>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  // one CTA per (row tile, chunk); the gated alternative gets a small grid that walks them (see the kernel)
  const int64_t blocks = (int64_t)args.row_tiles * n_chunks;
  dim3 grid((unsigned)(args.gate.flag != nullptr && args.gate.want ? std::min<int64_t>(blocks, 148 * 4) : blocks),
            (unsigned)t_chunks, 1);
  kmv_simt_kernel<T, KT, TT><<<grid, 256, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <typename T, int KT>
int launch_simt_tt(const SimtArgs<T>& args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  switch (tt) {
    case 1: return launch_simt<T, KT, 1>(args, n_chunks, t_chunks, stream);
    case 2: return launch_simt<T, KT, 2>(args, n_chunks, t_chunks, stream);
    case 4: return launch_simt<T, KT, 4>(args, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported TT=%d", tt);
}

template <typename T>
int launch_simt_any(int kernel, const SimtArgs<T>& args, int tt, int n_chunks, int t_chunks,
                    cudaStream_t stream) {
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_simt_tt<T, FLK_GAUSSIAN>(args, tt, n_chunks, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_simt_tt<T, FLK_LAPLACIAN>(args, tt, n_chunks, t_chunks, stream);
    case FLK_MATERN15: return launch_simt_tt<T, FLK_MATERN15>(args, tt, n_chunks, t_chunks, stream);
    case FLK_MATERN25: return launch_simt_tt<T, FLK_MATERN25>(args, tt, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace flk
