// fp64 tensor-core (DMMA) kernel-vector product for many vector columns:
//   raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t],  32 vector columns per pass.
//
// Same data flow as kmv_wide_kernel (flk_wide.cuh) -- a CTA forms a 128 x 64 block of kernel values from
// cp.async-staged 16-feature operand chunks, parks it in shared memory and multiplies it with the 64 x 32
// tile of `vec` -- but both products run on the fp64 tensor-core instruction
// mma.sync.m8n8k4.f64 (tcgen05 has no fp64 kind): eight multiply-adds per lane and instruction instead of
// one, which removes the issue and operand-fetch pressure that keeps the DFMA version at 42 % of the pipe.
// On B200 DMMA and DFMA have the same peak (37 TFLOP/s measured for both), so the gain is efficiency, not
// a higher ceiling.
//
// Fragment layouts of m8n8k4 (lane = 4 g + q): A[8 x 4] row-major: lane holds A[g][q]; B[4 x 8] "col":
// lane holds B[q][g]; C[8 x 8]: lane holds C[g][2 q], C[g][2 q + 1].  Shared-memory pitches (20, 68 and 36
// doubles) are chosen so that each half-warp's fragment load touches 16 different banks pairs.
// Arithmetic order per kernel value is the reference's: (|a|^2 - 2 a.b) + |b|^2, clamp at 1e-20, kernel function.
#pragma once

#include "flk_common.cuh"
#include "flk_simt.cuh"

namespace flk {
namespace dmma {

constexpr int BR = 128, BC = 64, DK = 16, LD = 20, TW = 32, KLD = 68, VLD = 36;
// Operand chunks, the vector tile and the column norms go through three-deep rings: the copy of step s + 2 is
// issued after the barrier of step s into the buffer that step s - 1 read, so one barrier per step suffices.
constexpr int NST = 3;
// Warps per CTA.  First product: NW / 2 row groups x 2 column groups of 32; second product: NW row groups.
#ifndef FLK_DMMA_WARPS
#define FLK_DMMA_WARPS 16
#endif
constexpr int NW = FLK_DMMA_WARPS, NT = 32 * NW;
constexpr int MT1 = BR / (NW / 2) / 8;  // 8-row MMA tiles per warp, first product
constexpr int MT2 = BR / NW / 8;        // ... second product

constexpr size_t smem_bytes() {
  return sizeof(double) * (size_t)(NST * BR * LD + NST * BC * LD + NST * BC * VLD + NST * BC + BR * KLD);
}

__device__ __forceinline__ void mma884(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

template <int KT>
__global__ void __launch_bounds__(NT, 1) kmv_dmma_kernel(SimtArgs<double> p) {
  if (!gate_open(p.gate)) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* As = reinterpret_cast<double*>(smem_raw);  // [NST][BR][LD]
  double* Bs = As + NST * BR * LD;                    // [NST][BC][LD]
  double* Vs = Bs + NST * BC * LD;                    // [NST][BC][VLD]
  double* bns = Vs + NST * BC * VLD;                  // [NST][BC]
  double* Ks = bns + NST * BC;                        // [BR][KLD] kernel values of the current tile, row-major

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, q = lane & 3;
  const int wr = warp % (NW / 2), wc = warp / (NW / 2);  // first product: rows wr * 8 MT1.., columns wc * 32..
  const int row_tile = blockIdx.x % p.row_tiles;
  const int chunk = blockIdx.x / p.row_tiles;
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int tile_end = min(tile_begin + p.tiles_per_chunk, p.n_col_tiles);
  const int ntiles = tile_end - tile_begin;
  const int ld = p.ld;
  const int nk = (ld + DK - 1) / DK;
  const int steps = ntiles * nk;
  const double* Ag = p.A + (int64_t)row_tile * BR * ld;

  double an[MT1];
#pragma unroll
  for (int mt = 0; mt < MT1; ++mt) an[mt] = p.an[(int64_t)row_tile * BR + wr * 8 * MT1 + mt * 8 + g];

  double acc[MT1][4][2];
  double oacc[MT2][4][2];  // second product: rows warp * 8 MT2 + mt * 8 + g, vector columns nt * 8 + 2q + {0, 1}
#pragma unroll
  for (int mt = 0; mt < MT1; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = 0.0;
#pragma unroll
  for (int mt = 0; mt < MT2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) oacc[mt][nt][0] = oacc[mt][nt][1] = 0.0;

  // row / piece of this thread's 16-byte pieces in a full chunk: the same for the A rows r0 and r0 + 64 and the B row r0
  static_assert(NT == 512 && BR == 128 && BC == 64 && DK == 16, "the full-chunk copy pattern assumes 512 threads");
  const int piece_src = (tid >> 3) * ld + (tid & 7) * 2;   // offset of the piece in a row-major operand (doubles)
  const int piece_dst = (tid >> 3) * LD + (tid & 7) * 2;   // ... in a shared-memory chunk
  int issue_tl = 0, issue_kc = 0, issue_buf = 0;            // tile, chunk and ring buffer of the next issue() call
  auto issue = [&](int s) {
    const int tl = issue_tl, kc = issue_kc;
    const int buf = issue_buf;
    if (++issue_kc == nk) {
      issue_kc = 0;
      ++issue_tl;
    }
    if (++issue_buf == NST) issue_buf = 0;
    const int k0 = kc * DK;
    const int kw = min(DK, ld - k0);   // even (ld is a multiple of 2)
    const int kw4 = (kw + 3) & ~3;     // the MMA consumes features in groups of four
    const int pieces = kw / 2;         // 16-byte pieces per row
    const int64_t col0 = (int64_t)(tile_begin + tl) * BC;
    double* dstb = Bs + buf * BC * LD;
    const double* Bg = p.B + col0 * ld + k0;
    if (kw == DK) {
      // full chunk (the common case): eight 16-byte pieces per row, so row and piece are a shift and a mask
      // (the general form divides by a run-time number, which costs more than the copies themselves)
      if (nk > 1 || s == 0) {
        double* dst = As + (nk > 1 ? buf : 0) * BR * LD + piece_dst;
        const double* src = Ag + k0 + piece_src;
        cp_async16(dst, src);
        cp_async16(dst + 64 * LD, src + 64 * ld);
      }
      cp_async16(dstb + piece_dst, Bg + piece_src);
    } else {
      if (nk > 1 || s == 0) {
        double* dst = As + (nk > 1 ? buf : 0) * BR * LD;
        for (int x = tid; x < BR * pieces; x += NT) {
          int r = x / pieces, pc = x - r * pieces;
          cp_async16(dst + r * LD + pc * 2, Ag + (int64_t)r * ld + k0 + pc * 2);
        }
        if (kw4 != kw)  // zero the features the last group of four reads beyond kw
          for (int r = tid; r < BR; r += NT) dst[r * LD + kw] = dst[r * LD + kw + 1] = 0.0;
      }
      for (int x = tid; x < BC * pieces; x += NT) {
        int r = x / pieces, pc = x - r * pieces;
        cp_async16(dstb + r * LD + pc * 2, Bg + (int64_t)r * ld + pc * 2);
      }
      if (kw4 != kw)
        for (int r = tid; r < BC; r += NT) dstb[r * LD + kw] = dstb[r * LD + kw + 1] = 0.0;
    }
    if (kc == 0) {
      const int vb = tl % NST;
      const double* vg = p.vec + ((int64_t)blockIdx.y * p.s_pad + col0) * TW;  // BC rows of TW values, contiguous
      double* vd = Vs + vb * BC * VLD;
#pragma unroll
      for (int x = tid; x < BC * (TW / 2); x += NT) {
        const int r = x / (TW / 2), pc = x % (TW / 2);  // compile-time divisor
        cp_async16(vd + r * VLD + pc * 2, vg + r * TW + pc * 2);
      }
      if (tid < BC) cp_async_small<8>(bns + vb * BC + tid, p.bn + col0 + tid);
    }
  };

  issue(0);
  cp_async_commit();
  if (steps > 1) issue(1);
  cp_async_commit();

  int tl = 0, kc = 0;
  for (int s = 0; s < steps; ++s) {
    cp_async_wait<1>();   // chunk s has landed (chunk s + 1 may still be in flight)
    __syncthreads();      // ... for every thread, and every warp is done with step s - 1
    // The copies of chunk s + 2 (into the buffer that step s - 1 read) are issued AFTER the first group of MMAs of
    // this step: their address arithmetic then runs while the MMAs are queued in the fp64 pipe, instead of every
    // warp doing it at the same time right behind the barrier with the pipe empty.

    const double* a_s = As + (nk > 1 ? (s % NST) : 0) * BR * LD + (wr * 8 * MT1 + g) * LD + q;
    const double* b_s = Bs + (s % NST) * BC * LD + (wc * 32 + g) * LD + q;
    const int kw4 = (min(DK, ld - kc * DK) + 3) & ~3;
    auto k_group = [&](int k) {
      double a[MT1], b[4];
#pragma unroll
      for (int mt = 0; mt < MT1; ++mt) a[mt] = a_s[mt * 8 * LD + k];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) b[nt] = b_s[nt * 8 * LD + k];
#pragma unroll
      for (int mt = 0; mt < MT1; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma884(acc[mt][nt], a[mt], b[nt]);
    };
    if (kw4 == DK) {  // full chunk: unrolled, so the fragment loads of the next group overlap the MMAs of this one
      k_group(0);
      if (s + 2 < steps) issue(s + 2);
      cp_async_commit();
#pragma unroll
      for (int k = 4; k < DK; k += 4) k_group(k);
    } else {
      if (s + 2 < steps) issue(s + 2);
      cp_async_commit();
      for (int k = 0; k < kw4; k += 4) k_group(k);
    }

    if (kc == nk - 1) {
      // 1. kernel values of this tile -> shared memory
      const double* bn_s = bns + (tl % NST) * BC;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int c = wc * 32 + nt * 8 + 2 * q;
        const double bn0 = bn_s[c], bn1 = bn_s[c + 1];
#pragma unroll
        for (int mt = 0; mt < MT1; ++mt) {
          double d0 = (an[mt] - 2.0 * acc[mt][nt][0]) + bn0;
          double d1 = (an[mt] - 2.0 * acc[mt][nt][1]) + bn1;
          d0 = d0 < 1e-20 ? 1e-20 : d0;
          d1 = d1 < 1e-20 ? 1e-20 : d1;
          double2 kv;
          kv.x = kernel_eval<KT>(d0);
          kv.y = kernel_eval<KT>(d1);
          *reinterpret_cast<double2*>(Ks + (wr * 8 * MT1 + mt * 8 + g) * KLD + c) = kv;
          acc[mt][nt][0] = acc[mt][nt][1] = 0.0;
        }
      }
      __syncthreads();
      // 2. out[rows warp * 8 MT2.., 32 columns] += K[rows, 0..63] vec[0..63, :]
      const double* k_s = Ks + (warp * 8 * MT2 + g) * KLD + q;
      const double* v_s = Vs + (tl % NST) * BC * VLD + q * VLD + g;
#pragma unroll 4
      for (int k = 0; k < BC; k += 4) {
        double a[MT2], b[4];
#pragma unroll
        for (int mt = 0; mt < MT2; ++mt) a[mt] = k_s[mt * 8 * KLD + k];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) b[nt] = v_s[k * VLD + nt * 8];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int mt = 0; mt < MT2; ++mt) mma884(oacc[mt][nt], a[mt], b[nt]);
      }
      kc = 0;
      ++tl;
    } else {
      ++kc;
    }
  }

#pragma unroll
  for (int mt = 0; mt < MT2; ++mt) {
    const int64_t row = (int64_t)row_tile * BR + warp * 8 * MT2 + mt * 8 + g;
    double* dst = p.raw + ((int64_t)chunk * p.r_pad + row) * p.tp + blockIdx.y * TW + 2 * q;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      double2 o;
      o.x = oacc[mt][nt][0];
      o.y = oacc[mt][nt][1];
      *reinterpret_cast<double2*>(dst + nt * 8) = o;
    }
  }
}

template <int KT>
int launch_inst(const SimtArgs<double>& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  constexpr size_t smem = smem_bytes();
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_dmma_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid((unsigned)(args.row_tiles * n_chunks), (unsigned)t_chunks, 1);
  kmv_dmma_kernel<KT><<<grid, NT, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

inline int launch(int kernel, const SimtArgs<double>& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_inst<FLK_GAUSSIAN>(args, n_chunks, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_inst<FLK_LAPLACIAN>(args, n_chunks, t_chunks, stream);
    case FLK_MATERN15: return launch_inst<FLK_MATERN15>(args, n_chunks, t_chunks, stream);
    case FLK_MATERN25: return launch_inst<FLK_MATERN25>(args, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace dmma
}  // namespace flk
