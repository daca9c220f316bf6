// Tensor-core kernel-vector product for fp32 data with MANY features (30 < d <= kMaxD):
//
//   raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t]
//
// Same formulation as flk_tc.cuh -- split-fp16 operand images whose MMA accumulator is the exponent of the
// kernel function, MUFU / FMA-pipe exponential epilogue, the contraction with `vec` fused -- but the K
// dimension of the exponent GEMM (3 d + 6 fp16 elements) no longer fits shared memory for a resident row
// block, so this kernel is an ordinary K-loop GEMM pipeline: a CTA owns 256 output rows (two 128-row MMA
// blocks), walks the 128-column tiles of its chunk, and for every tile streams the operand images slab by slab
// (32 fp16 = 64 bytes of K per row: 8 KB for each of the two A blocks and for the B tile) through a ring of
// bulk copies; each slab feeds four tcgen05.mma (2 row blocks x 2 K-steps).  The two row blocks have two TMEM
// accumulators each (512 columns in all), so the MMAs of tile j+1 run under the epilogue of tile j.  The
// kernel is bound by the tensor pipe / the L2 traffic of the re-streamed operands (3 x the bytes of a plain
// GEMM of the same shape, because every feature appears three times in the split), not by MUFU.
// Warps 0-15: epilogue (TMEM lane quarter = warp % 4, row block = (warp / 4) % 2, column half of the tile =
// warp / 8; the two halves of a row are added at the end through shared memory); warps 16, 17: MMA issuers, one
// per row block (the barrier round trip between two slabs of one issuer runs under the MMAs of the other; warp 16
// owns the TMEM allocation); warp 18: bulk-copy producer.  Every wait is bounded as in flk_tc.cuh.
#pragma once

#include "flk_tc.cuh"

namespace flk {
namespace tck {

using namespace tc;  // PTX wrappers, image layout, epilogue helpers

constexpr int kRowBlocksL = 2;
constexpr int kRowsPerCtaL = kRowBlocksL * kTileRows;  // 256
constexpr int kMaxDL = 1024;
constexpr int kSlabBytes = kTileRows * kSlabK * 2;      // 8 KB: one 128-row slab of an operand image
constexpr int kStages = 8;
constexpr int kMaxResidentSlabs = 8;                    // both A blocks stay in shared memory up to this many slabs
constexpr int kColSplitL = 2;                           // epilogue warps per (row block, lane quarter): each takes 64 columns of a tile
constexpr int kEpiWarpsL = 4 * kRowBlocksL * kColSplitL;
constexpr int kMmaWarpL = kEpiWarpsL;                   // warps 16, 17: MMA issuer of row block (warp - 16)
constexpr int kProducerWarpL = kEpiWarpsL + kRowBlocksL;
// warp 19 does no work: it completes the warpgroup of the two issuers and the producer, so that this group can
// hand registers to the four epilogue warpgroups (setmaxnreg works on whole warpgroups, see flk_tc.cuh).  20 warps
// = 5 per SM sub-partition = 96 registers per thread at launch; afterwards 16 x 104 + 4 x 64 = 20 x 96.
constexpr int kThreadsL = (kEpiWarpsL + kRowBlocksL + 2) * 32;
constexpr int kRegsEpilogueL = 104;
constexpr int kRegsOthersL = 64;
static_assert(kEpiWarpsL * kRegsEpilogueL + 4 * kRegsOthersL <= (kThreadsL / 32) * 96,
              "register re-partitioning exceeds the pool the CTA is launched with");

inline bool supports_d(int64_t d) { return d > tc::kMaxD && d <= kMaxDL; }
inline int used_k(int64_t d) { return (int)(3 * d + 6); }  // always three norm pieces
inline int k_steps(int64_t d) { return (int)(round_up(used_k(d), kMmaK) / kMmaK); }
inline int64_t padded_k(int64_t d) { return round_up(used_k(d), kSlabK); }
inline int n_slabs(int64_t d) { return (int)(padded_k(d) / kSlabK); }

// ---------------------------------------------------------------------------------------------
// Operand images for any feature count: one block = one 128-row tile, one thread = one row.  The image is
// built slab by slab in shared memory (so that the global writes are coalesced 8 KB runs); the row's
// features are re-read from X for each of the three copies the split needs (they stay in L1 / L2).
// K layout of a row, as in flk_tc.cuh:  A = [xh | xh | xl | -n1 -n2 -n3 | 1 1 1 | 0..],
//                                       B = [ch | cl | ch | 1 1 1 | -m1 -m2 -m3 | 0..].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) prep_images_large_kernel(const float* __restrict__ X, int64_t n, int64_t rs,
                                                                int64_t cs, int d, const float* __restrict__ sigma,
                                                                float sigma_scalar, int sigma_len, float scale,
                                                                int nslab, __half* __restrict__ img_a,
                                                                __half* __restrict__ img_b, int* __restrict__ range_word) {
  __shared__ __align__(16) __half slab[2][kTileRows * kSlabK];  // A and B version of the current slab
  const int r = threadIdx.x;
  const int64_t row = (int64_t)blockIdx.x * kTileRows + r;
  const bool live = row < n;
  const float* xr = X + (live ? row : 0) * rs;
  auto scaled = [&](int f) -> float {
    const float s = sigma != nullptr ? sigma[sigma_len == 1 ? 0 : f] : sigma_scalar;
    return (xr[(int64_t)f * cs] / s) * scale;  // x / sigma rounded as in the reference, then the kernel's scale
  };
  // pass 1: squared norm of the value the two fp16 parts represent, range check
  double nrm = 0.0;
  bool out_of_range = false;
  if (live) {
    for (int f = 0; f < d; ++f) {
      float xt = scaled(f);
      if (!(fabsf(xt) <= 400.0f)) {
        out_of_range = true;
        xt = 0.0f;
      }
      const float hi = __half2float(__float2half_rn(xt));
      const float lo = __half2float(__float2half_rn(xt - hi));
      const double rep = (double)hi + (double)lo;
      nrm += rep * rep;
    }
  }
  double half_norm = 0.5 * nrm;
  if (half_norm > (double)kNormLimit) {
    out_of_range = true;
    half_norm = 0.0;
  }
  if (out_of_range && live) atomicOr(range_word, 1);
  float piece[3];
  {
    double rem = half_norm;
    for (int i = 0; i < 3; ++i) {
      const float remf = __double2float_ru(rem);
      const float pc = __half2float(i == 2 ? __float2half_ru(remf) : __float2half_rn(remf));
      piece[i] = pc;
      rem -= (double)pc;
    }
  }
  const __half one = __float2half_rn(1.0f), zero = __float2half_rn(0.0f);
  // pass 2: slabs
  for (int s = 0; s < nslab; ++s) {
    for (int e = 0; e < kSlabK; ++e) {
      const int k = s * kSlabK + e;  // K index
      __half va = zero, vb = zero;
      if (live) {
        if (k < 3 * d) {
          const int region = k / d, f = k - region * d;
          float xt = scaled(f);
          if (!(fabsf(xt) <= 400.0f)) xt = 0.0f;
          const __half hi = __float2half_rn(xt);
          const __half lo = __float2half_rn(xt - __half2float(hi));
          va = region == 2 ? lo : hi;   // A: hi, hi, lo
          vb = region == 1 ? lo : hi;   // B: hi, lo, hi
        } else if (k < 3 * d + 3) {
          va = __float2half_rn(-piece[k - 3 * d]);
          vb = one;
        } else if (k < 3 * d + 6) {
          va = one;
          vb = __float2half_rn(-piece[k - 3 * d - 3]);
        }
      }
      const int off = r * kSlabK + ((((e >> 3) ^ ((r >> 1) & 3))) << 3) + (e & 7);
      slab[0][off] = va;
      slab[1][off] = vb;
    }
    __syncthreads();
    const int64_t base = ((int64_t)blockIdx.x * nslab + s) * (kTileRows * kSlabK);
    for (int which = 0; which < 2; ++which) {
      __half* dst = which == 0 ? img_a : img_b;
      if (dst == nullptr) continue;
      uint4* out4 = reinterpret_cast<uint4*>(dst + base);
      const uint4* in4 = reinterpret_cast<const uint4*>(slab[which]);
      for (int idx = r; idx < kTileRows * kSlabK / 8; idx += 128) out4[idx] = in4[idx];
    }
    __syncthreads();
  }
}

inline int prep_images_large(int kernel, const void* X, int64_t n, int64_t rs, int64_t cs, int d,
                             const float* sigma_dev, float sigma_scalar, int sigma_len, int64_t rows_pad, void* img_a,
                             void* img_b, int* range_word, cudaStream_t stream) {
  const float scale = (float)sqrt(scale_sq_for(kernel));
  const int blocks = (int)(rows_pad / kTileRows);
  prep_images_large_kernel<<<blocks, 128, 0, stream>>>(reinterpret_cast<const float*>(X), n, rs, cs, d, sigma_dev,
                                                       sigma_scalar, sigma_len, scale, n_slabs(d),
                                                       reinterpret_cast<__half*>(img_a),
                                                       reinterpret_cast<__half*>(img_b), range_word);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Sweep kernel
// ---------------------------------------------------------------------------------------------
struct SweepArgsL {
  const __half* img_a;  // [r_pad / 128][nslab] slabs (output side)
  const __half* img_b;  // [s_pad / 128][nslab] slabs (reduction side)
  const float* vec;     // [t_chunks][s_pad][TT]
  float* raw;           // [n_chunks][r_pad][tp]
  int* status;
  int tp;
  int64_t r_pad;
  int64_t s_pad;
  int row_tiles;        // ceil(r / 256)
  int n_col_tiles;      // ceil(s / 128)
  int tiles_per_chunk;
  int nslab;            // K slabs per operand tile
  int ksteps;           // MMA K-steps carrying data (two per slab, possibly one in the last slab)
};

// ARES: the two A blocks of the CTA (256 rows x nslab slabs, at most 128 KB) are loaded once and stay resident;
// a ring stage then carries the B slab only (8 KB instead of 24 KB), which cuts the L2 traffic three-fold.
// With 32 vector columns per pass the vector tiles are 16 KB each: two of them and a six-stage operand ring.
template <int TT>
struct RingCfg {
  static constexpr int S = TT == kWideTT ? 6 : kStages;
  static constexpr int VS = TT == kWideTT ? 2 : kVecStages;
};

template <int TT, bool ARES>
constexpr size_t tck_smem_bytes() {
  return 1024 + (ARES ? (size_t)kRowBlocksL * kMaxResidentSlabs * kSlabBytes : 0) +
         (size_t)RingCfg<TT>::S * (ARES ? 1 : 3) * kSlabBytes + (size_t)RingCfg<TT>::VS * kColsPerTile * TT * 4 + 512 +
         (size_t)kRowsPerCtaL * TT * 4 /* partial sums of the second column half */;
}

// Kernel function + contraction with 32 vector columns for 32 accumulator columns held in registers: per kernel
// value one exponential, then 16 packed multiply-adds against the 32 vector entries of that column (read as
// eight 16-byte broadcasts from shared memory).
template <int KT, int C0 = 0>
__device__ __forceinline__ void epilogue_wide32(const uint32_t (&r)[32], const float* vsm, uint64_t (&osum)[16]) {
  if constexpr (C0 < 32) {
    float k0, k1;
    eval_pair<KT, poly_pair<KT>(C0 / 2)>(r[C0], r[C0 + 1], k0, k1);
    const float kv[2] = {k0, k1};
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint64_t kk = pack2(kv[c], kv[c]);
      const ulonglong2* v = reinterpret_cast<const ulonglong2*>(vsm + (C0 + c) * kWideTT);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const ulonglong2 vv = v[i];
        osum[2 * i] = fma2(kk, vv.x, osum[2 * i]);
        osum[2 * i + 1] = fma2(kk, vv.y, osum[2 * i + 1]);
      }
    }
    epilogue_wide32<KT, C0 + 2>(r, vsm, osum);
  }
}

__device__ __forceinline__ void report_timeout(int* status, int code) { atomicExch(status + kStatusTimeout, code); }

template <int KT, int TT, bool ARES>
__global__ void __launch_bounds__(kThreadsL, 1) kmv_tck_kernel(const SweepArgsL p) {
  constexpr int S = RingCfg<TT>::S, VS = RingCfg<TT>::VS;
  constexpr int kStageBytes = (ARES ? 1 : 3) * kSlabBytes;  // [A block 0 | A block 1 |] B tile
  constexpr int kAResBytes = ARES ? kRowBlocksL * kMaxResidentSlabs * kSlabBytes : 0;
  extern __shared__ unsigned char tck_smem_raw[];
  const uint32_t raw_addr = smem_u32(tck_smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  // Shared-memory map as 32-bit shared addresses from one base (generic pointers to every ring and barrier would
  // stay live across all warp roles): [A blocks, ARES only] | operand ring | vector ring | barrier block | combine.
  // barrier block: s_full[S] | s_empty[S] | v_full[VS] | v_empty[VS] | t_full[4] | t_empty[4] (index rb * 2 + buf) |
  // a_full | tmem pointer | abort flag
  const uint32_t sm = raw_addr + pad;
  constexpr uint32_t kRingOff = kAResBytes;
  constexpr uint32_t kVecOff = kRingOff + S * kStageBytes;
  constexpr uint32_t kBarsOff = kVecOff + VS * kColsPerTile * TT * 4;
  constexpr uint32_t kSFull = kBarsOff, kSEmpty = kSFull + 8 * S, kVFull = kSEmpty + 8 * S, kVEmpty = kVFull + 8 * VS;
  constexpr uint32_t kTFull = kVEmpty + 8 * VS, kTEmpty = kTFull + 32, kAFull = kTEmpty + 32;
  constexpr uint32_t kTmemPtr = kAFull + 8, kAbort = kTmemPtr + 4, kCombineOff = kBarsOff + 512;
  static_assert(kAbort + 4 <= kCombineOff, "barrier block overflows its 512 bytes");

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int row_tile = blockIdx.x % p.row_tiles;
  const int chunk = blockIdx.x / p.row_tiles;
  const int tchunk = blockIdx.y;
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int tile_end = min(tile_begin + p.tiles_per_chunk, p.n_col_tiles);
  const int ntiles = tile_end - tile_begin;
  const int nslab = p.nslab;

  __shared__ int skip_launch;
  if (tid == 0) {
    const volatile int* st = reinterpret_cast<const volatile int*>(p.status);
    skip_launch = (st[kStatusTimeout] != 0 || range_raised(p.status + kStatusRange)) ? 1 : 0;
  }
  __syncthreads();
  if (skip_launch) return;

  if (tid == 0) {
#pragma unroll 1
    for (int s = 0; s < S; ++s) {
      mbar_init(sm + kSFull + 8 * s, 1);
      mbar_init(sm + kSEmpty + 8 * s, kRowBlocksL);  // one MMA commit per issuer
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(sm + kVFull + 8 * s, 1);
      mbar_init(sm + kVEmpty + 8 * s, kEpiWarpsL);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(sm + kTFull + 8 * i, 1);
      mbar_init(sm + kTEmpty + 8 * i, 4 * kColSplitL);  // the eight warps of that row block
    }
    mbar_init(sm + kAFull, 1);
    st_shared_i32_volatile(sm + kAbort, 0);
    fence_barrier_init();
  }
  if (warp == kMmaWarpL) {
    tmem_alloc(sm + kTmemPtr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = (uint32_t)ld_shared_i32_volatile(sm + kTmemPtr);

  if (warp > kProducerWarpL) {
    reg_release<kRegsOthersL>();  // filler warp of the issuers' and the producer's warpgroup
  } else if (warp == kProducerWarpL) {
    // ------------------------------ bulk-copy producer ------------------------------
    reg_release<kRegsOthersL>();
    const __half* a_base = p.img_a + (int64_t)row_tile * kRowBlocksL * nslab * (kTileRows * kSlabK);
    const float* vec_base = p.vec + (int64_t)tchunk * p.s_pad * TT;
    if (ARES && elect_one()) {
      // the CTA's two A blocks are contiguous in the image: [row block][slab]
      const uint32_t bytes = (uint32_t)(kRowBlocksL * nslab * kSlabBytes);
      mbar_expect_tx(sm + kAFull, bytes);
      for (int i = 0; i < kRowBlocksL * nslab; ++i)
        bulk_copy_g2s(sm + i * kSlabBytes, a_base + (int64_t)i * (kTileRows * kSlabK), kSlabBytes,
                      sm + kAFull);
    }
    __syncwarp();
    uint32_t gs = 0;  // running slab counter
    bool ok = true;
    for (int j = 0; ok && j < ntiles; ++j) {
      const int64_t ct = tile_begin + j;
      const int vstage = j % VS;
      if (!mbar_wait(sm + kVEmpty + 8 * vstage, ((j / VS) & 1) ^ 1)) {
        if (lane == 0) report_timeout(p.status, kErrProducer | 2);
        st_shared_i32_volatile(sm + kAbort, 1);
        break;
      }
      if (elect_one()) {
        const uint32_t vbar = sm + kVFull + 8 * vstage;
        mbar_expect_tx(vbar, kColsPerTile * TT * 4);
        bulk_copy_g2s(sm + kVecOff + vstage * kColsPerTile * TT * 4, vec_base + ct * kColsPerTile * TT,
                      kColsPerTile * TT * 4, vbar);
      }
      __syncwarp();
      const __half* b_base = p.img_b + ct * nslab * (kTileRows * kSlabK);
      for (int s = 0; s < nslab; ++s, ++gs) {
        const int stage = (int)(gs % (uint32_t)S);
        if (ld_shared_i32_volatile(sm + kAbort)) { ok = false; break; }
        if (!mbar_wait(sm + kSEmpty + 8 * stage, ((gs / (uint32_t)S) & 1u) ^ 1u)) {
          if (lane == 0) report_timeout(p.status, kErrProducer | 1);
          st_shared_i32_volatile(sm + kAbort, 1);
          ok = false;
          break;
        }
        if (elect_one()) {
          const uint32_t bar = sm + kSFull + 8 * stage;
          const uint32_t dst = sm + kRingOff + stage * kStageBytes;
          mbar_expect_tx(bar, kStageBytes);
          if (!ARES) {
            bulk_copy_g2s(dst, a_base + (int64_t)s * (kTileRows * kSlabK), kSlabBytes, bar);
            bulk_copy_g2s(dst + kSlabBytes, a_base + ((int64_t)nslab + s) * (kTileRows * kSlabK), kSlabBytes, bar);
          }
          bulk_copy_g2s(dst + (ARES ? 0 : 2) * kSlabBytes, b_base + (int64_t)s * (kTileRows * kSlabK), kSlabBytes, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp >= kMmaWarpL) {
    // ------------------------------ MMA issuers (one per row block) ------------------------------
    reg_release<kRegsOthersL>();
    const int rb = warp - kMmaWarpL;
    uint32_t gs = 0;
    bool ok = true;
    if (ARES && !mbar_wait(sm + kAFull, 0)) {
      if (lane == 0) report_timeout(p.status, kErrMma | 1);
      st_shared_i32_volatile(sm + kAbort, 1);
      ok = false;
    }
    for (int j = 0; ok && j < ntiles; ++j) {
      const int buf = j & 1;
      if (ld_shared_i32_volatile(sm + kAbort)) break;
      // this row block's accumulator of this buffer must have been drained (tile j - 2)
      if (!mbar_wait(sm + kTEmpty + 8 * (rb * 2 + buf), ((j >> 1) & 1) ^ 1)) {
        if (lane == 0) report_timeout(p.status, kErrMma | 3);
        st_shared_i32_volatile(sm + kAbort, 1);
        break;
      }
      const uint32_t d_tmem = tmem_base + (uint32_t)((rb * 2 + buf) * kColsPerTile);
      for (int s = 0; s < nslab; ++s, ++gs) {
        const int stage = (int)(gs % (uint32_t)S);
        if (!mbar_wait(sm + kSFull + 8 * stage, (gs / (uint32_t)S) & 1u)) {
          if (lane == 0) report_timeout(p.status, kErrMma | 2);
          st_shared_i32_volatile(sm + kAbort, 1);
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t sbase = sm + kRingOff + stage * kStageBytes;
          const uint64_t b_desc = make_smem_desc(sbase + (ARES ? 0 : 2) * kSlabBytes);
          const uint64_t a_desc = make_smem_desc(ARES ? sm + (rb * nslab + s) * kSlabBytes
                                                      : sbase + rb * kSlabBytes);
          const int nks = min(2, p.ksteps - 2 * s);  // K-steps of this slab that carry data
          for (int ks = 0; ks < nks; ++ks)
            mma_f16(d_tmem, a_desc + (uint64_t)(ks * 2), b_desc + (uint64_t)(ks * 2), kInstrDesc,
                    (s > 0 || ks > 0) ? 1u : 0u);
          mma_commit(sm + kSEmpty + 8 * stage);
          if (s == nslab - 1) mma_commit(sm + kTFull + 8 * (rb * 2 + buf));
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    reg_claim<kRegsEpilogueL>();
    const int q = warp & 3;
    const int rb = (warp >> 2) & 1;
    const int half = warp >> 3;  // columns half * 64 .. + 63 of every tile
    constexpr int NSUM = TT == kWideTT ? 16 : 2;
    // two-level summation for TT <= 4, as in the resident kernel (here the second level fits in registers);
    // the many-column form keeps one level and relies on the planner's bound on the chunk length
    uint64_t osum[NSUM], otot[TT == kWideTT ? 1 : NSUM];
#pragma unroll
    for (int i = 0; i < NSUM; ++i) osum[i] = 0ull;
#pragma unroll
    for (int i = 0; i < (TT == kWideTT ? 1 : NSUM); ++i) otot[i] = 0ull;
    bool epi_ok = true;
    for (int j0 = 0; j0 < ntiles && epi_ok; j0 += tc::kFlushTiles) {
    if constexpr (TT != kWideTT) {
      if (j0 > 0) {
#pragma unroll
        for (int i = 0; i < NSUM; ++i) {
          otot[i] = tc::add2(otot[i], osum[i]);
          osum[i] = 0ull;
        }
      }
    }
    const int j1 = min(j0 + tc::kFlushTiles, ntiles);
    for (int j = j0; j < j1; ++j) {
      const int vstage = j % VS, buf = j & 1;
      if (ld_shared_i32_volatile(sm + kAbort)) { epi_ok = false; break; }
      if (!mbar_wait(sm + kVFull + 8 * vstage, (j / VS) & 1) ||
          !mbar_wait(sm + kTFull + 8 * (rb * 2 + buf), (j >> 1) & 1)) {
        report_timeout(p.status, kErrEpilogue | 1);
        st_shared_i32_volatile(sm + kAbort, 1);
        epi_ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) +
                             (uint32_t)((rb * 2 + buf) * kColsPerTile + half * 64);
      const float* vsm = reinterpret_cast<const float*>(tck_smem_raw + pad + kVecOff) + (vstage * kColsPerTile + half * 64) * TT;
      if constexpr (TT == kWideTT) {
        // 32 running sums per thread leave room for one 32-column piece at a time
        uint32_t ra[32];
        tmem_ld32(taddr, ra);
        tmem_ld_wait_on(ra);
        epilogue_wide32<KT>(ra, vsm, osum);
        tmem_ld32(taddr + 32, ra);
        tmem_ld_wait_on(ra);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm + kTEmpty + 8 * (rb * 2 + buf));
        epilogue_wide32<KT>(ra, vsm + 32 * TT, osum);
      } else {
        uint32_t ra[32], rc[32];
        tmem_ld32(taddr, ra);
        tmem_ld_wait_on(ra);
        tmem_ld32(taddr + 32, rc, ra);
        tmem_ld_wait_on(rc);
        // this warp's 64 columns are in registers: hand the accumulator back before evaluating them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm + kTEmpty + 8 * (rb * 2 + buf));
        epilogue_32<KT, TT>(ra, vsm, osum);
        epilogue_32<KT, TT>(rc, vsm + 32 * TT, osum);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sm + kVEmpty + 8 * vstage);
    }
    }
    // per-thread sums of this column half
    if constexpr (TT != kWideTT) {
#pragma unroll
      for (int i = 0; i < NSUM; ++i) osum[i] = tc::add2(otot[i], osum[i]);
    }
    float o[TT];
    if constexpr (TT == kWideTT) {
#pragma unroll
      for (int i = 0; i < 16; ++i) unpack2(osum[i], o[2 * i], o[2 * i + 1]);
    } else {
      float a0, a1, b0, b1;
      unpack2(osum[0], a0, a1);
      unpack2(osum[1], b0, b1);
      if constexpr (TT == 1) {
        o[0] = (a0 + a1) + (b0 + b1);
      } else if constexpr (TT == 2) {
        o[0] = a0 + b0;
        o[1] = a1 + b1;
      } else {
        o[0] = a0;
        o[1] = a1;
        o[2] = b0;
        o[3] = b1;
      }
    }
    const int rloc = rb * kTileRows + q * 32 + lane;
    float* combine = reinterpret_cast<float*>(tck_smem_raw + pad + kCombineOff);  // [256 rows][TT]
    if (half == 1) {
#pragma unroll
      for (int t = 0; t < TT; ++t) combine[rloc * TT + t] = o[t];
    }
    // all sixteen epilogue warps meet here (named barrier 1; the issuer and producer warps do not take part)
    asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarpsL * 32) : "memory");
    if (half == 0 && epi_ok && ld_shared_i32_volatile(sm + kAbort) == 0) {
      const int64_t row = (int64_t)row_tile * kRowsPerCtaL + rloc;
      float* dst = p.raw + ((int64_t)chunk * p.r_pad + row) * p.tp + tchunk * TT;
#pragma unroll
      for (int t = 0; t < TT; ++t) dst[t] = o[t] + combine[rloc * TT + t];
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  const bool aborted = (ld_shared_i32_volatile(sm + kAbort) != 0);
  if (aborted && warp == kProducerWarpL && lane == 0) {
    // give this CTA's own bulk copies a bounded chance to land before the shared memory is released
    if (ARES) mbar_wait(sm + kAFull, 0);
#pragma unroll 1
    for (uint32_t bar = sm + kSFull; bar < sm + kSFull + 8 * S; bar += 8)
      if (!mbar_try_wait(bar, 0)) mbar_try_wait(bar, 1);
#pragma unroll 1
    for (uint32_t bar = sm + kVFull; bar < sm + kVFull + 8 * VS; bar += 8)
      if (!mbar_try_wait(bar, 0)) mbar_try_wait(bar, 1);
  }
  __syncthreads();
  if (warp == kMmaWarpL) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int KT, int TT, bool ARES>
int launch_inst(const SweepArgsL& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  constexpr size_t smem = tck_smem_bytes<TT, ARES>();
  static_assert(smem > 116 * 1024 && smem <= 227 * 1024, "one CTA per SM is assumed; shared memory budget");
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_tck_kernel<KT, TT, ARES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid((unsigned)(args.row_tiles * n_chunks), (unsigned)t_chunks, 1);
  kmv_tck_kernel<KT, TT, ARES><<<grid, kThreadsL, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <int KT>
int launch_tt(const SweepArgsL& args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  const bool ares = args.nslab <= kMaxResidentSlabs;
  switch (tt) {
    case 1: return ares ? launch_inst<KT, 1, true>(args, n_chunks, t_chunks, stream)
                        : launch_inst<KT, 1, false>(args, n_chunks, t_chunks, stream);
    case 2: return ares ? launch_inst<KT, 2, true>(args, n_chunks, t_chunks, stream)
                        : launch_inst<KT, 2, false>(args, n_chunks, t_chunks, stream);
    case 4: return ares ? launch_inst<KT, 4, true>(args, n_chunks, t_chunks, stream)
                        : launch_inst<KT, 4, false>(args, n_chunks, t_chunks, stream);
    case kWideTT:  // 16 KB vector tiles and 32 KB of partial sums leave no room for resident A blocks
      return launch_inst<KT, kWideTT, false>(args, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported TT=%d", tt);
}

inline int launch_sweep(int kernel, int d, SweepArgsL args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  args.nslab = n_slabs(d);
  args.ksteps = k_steps(d);
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_tt<FLK_GAUSSIAN>(args, tt, n_chunks, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_tt<FLK_LAPLACIAN>(args, tt, n_chunks, t_chunks, stream);
    case FLK_MATERN15: return launch_tt<FLK_MATERN15>(args, tt, n_chunks, t_chunks, stream);
    case FLK_MATERN25: return launch_tt<FLK_MATERN25>(args, tt, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace tck
}  // namespace flk
