// Tensor-core kernel-vector product for fp32 data with MANY features (30 < d <= kMaxD):
//
//   raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t]
//
// Same formulation as flk_tc.cuh -- split-fp16 operands whose MMA accumulator is the exponent of the kernel
// function, MUFU / FMA-pipe exponential epilogue, the contraction with `vec` fused -- but the K dimension of the
// exponent GEMM no longer fits shared memory for a resident row block of 512 rows, so this kernel is a K-loop GEMM
// pipeline: a CTA owns one or two 128-row MMA blocks, walks the column tiles of its chunk, and for every tile streams
// the reduction-side operand slab by slab (32 fp16 = 64 bytes of K per row, 8 KB per 128 rows) through a ring of
// bulk copies.  Two TMEM accumulators per accumulator group (512 columns in all), so the MMAs of step j+1 run
// under the epilogue of step j.
//
// Compact split.  With x = xh + xl, c = ch + cl in fp16, the exponent needs  xh.ch + xh.cl + xl.ch - |x|^2/2 - |c|^2/2.
// Instead of laying the three products out along K (three copies of the features in each operand), an operand
// image holds every part ONCE:
//     [ hi parts: ds slabs | lo parts: ds slabs | tail slab ],   ds = ceil(d / 32),
//     tail of an output-side image  = [-n1 -n2 -n3 | 1 1 1 | 0 ...],  of a reduction-side image = [1 1 1 | -m1 -m2 -m3 | 0 ...]
// and the issuer pairs the slabs: for every feature slab three MMAs per K-step, (A hi, B hi), (A hi, B lo),
// (A lo, B hi), plus one MMA on the tails.  That is the same number of MMAs (3 ceil(d / 16) + 1 per tile) on two
// thirds of the operand bytes -- and what bounds a K-loop kernel here is operand delivery from L2 (a 128 x 128 x 16 MMA
// takes 64 clocks; measured: about 55 B/clk per SM can be streamed while all SMs do the same).  Three shapes, by the
// number of feature slabs (bytes per clock and SM that the bulk copies must sustain for the tensor pipe to stay busy):
//   kResident2 (d <= 128): both 128-row blocks of the CTA stay in shared memory (2 x (2 ds + 1) slabs); a ring
//       stage is the hi and the lo slab of one feature slab of a 128-column tile: 16 KB per twelve MMAs = 21 B/clk;
//   kResident1 (d <= 192): ONE 128-row block stays resident and the CTA walks PAIRS of column tiles with
//       128 x 256 x 16 MMAs from a single issuer: 32 KB per six such MMAs = 42 B/clk;
//   kStream (more features, and the 32-column epilogue whose vector tiles and partial sums need the shared memory):
//       a stage carries the hi and lo slabs of both row blocks and of the column tile: 48 KB per twelve MMAs = 62 B/clk.
// Warps 0-15: epilogue (TMEM lane quarter = warp % 4, accumulator group = (warp / 4) % 2, 64-column half of the
// group's 128 columns = warp / 8; the partial sums of a row are added at the end through shared memory); warps 16,
// 17: MMA issuers, one per accumulator group (warp 16 alone in kResident1; it owns the TMEM allocation); warp 18:
// bulk-copy producer.  Every wait is bounded as in flk_tc.cuh.
#pragma once

#include "flk_tc.cuh"

namespace flk {
namespace tck {

using namespace tc;  // PTX wrappers, swizzle, epilogue helpers

constexpr int kGroupsL = 2;                             // accumulator groups
constexpr int kMaxDL = 1024;
constexpr int kSlabBytes = kTileRows * kSlabK * 2;      // 8 KB: one 128-row slab of an operand image
constexpr int kMaxStagesL = 12;                         // barrier slots of the operand ring
constexpr int kMinStagesL = 3;
constexpr int kColSplitL = 2;                           // epilogue warps per (group, lane quarter): each takes 64 columns
constexpr int kEpiWarpsL = 4 * kGroupsL * kColSplitL;
constexpr int kMmaWarpL = kEpiWarpsL;                   // warps 16, 17: MMA issuer of group (warp - 16)
constexpr int kProducerWarpL = kEpiWarpsL + kGroupsL;
// warp 19 does no work: it completes the warpgroup of the two issuers and the producer, so that this group can
// hand registers to the four epilogue warpgroups (setmaxnreg works on whole warpgroups, see flk_tc.cuh).  20 warps
// = 5 per SM sub-partition = 96 registers per thread at launch; afterwards 16 x 104 + 4 x 64 = 20 x 96.
constexpr int kThreadsL = (kEpiWarpsL + kGroupsL + 2) * 32;
constexpr int kRegsEpilogueL = 104;
constexpr int kRegsOthersL = 64;
static_assert(kEpiWarpsL * kRegsEpilogueL + 4 * kRegsOthersL <= (kThreadsL / 32) * 96,
              "register re-partitioning exceeds the pool the CTA is launched with");
constexpr int kMaxSmemL = 226 * 1024;  // dynamic shared memory of a CTA: the 227 KB limit less the kernel's static variables

// M = 128, N = 256 form of the instruction descriptor (see tc::kInstrDesc)
constexpr uint32_t kInstrDescN256 = (1u << 4) | ((uint32_t)((2 * kColsPerTile) >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);

enum TileMode { kStream = 0, kResident2 = 1, kResident1 = 2 };
// rows of a CTA and columns of one step of its tile loop
__host__ __device__ constexpr int rows_per_cta(int mode) { return mode == kResident1 ? kTileRows : 2 * kTileRows; }
__host__ __device__ constexpr int cols_per_step(int mode) { return mode == kResident1 ? 2 * kColsPerTile : kColsPerTile; }
constexpr int kRowsPerCtaL = 2 * kTileRows;  // 256, the kStream / kResident2 shapes

inline bool supports_d(int64_t d) { return d > tc::kMaxD && d <= kMaxDL; }
inline int feature_slabs(int64_t d) { return (int)((d + kSlabK - 1) / kSlabK); }   // ds
inline int n_slabs(int64_t d) { return 2 * feature_slabs(d) + 1; }                 // hi | lo | tail
inline int64_t padded_k(int64_t d) { return (int64_t)n_slabs(d) * kSlabK; }        // fp16 elements per image row
inline int last_k_steps(int64_t d) { return (int)((d - (int64_t)(feature_slabs(d) - 1) * kSlabK + kMmaK - 1) / kMmaK); }

// ---- shared-memory plan (host and device agree through these functions) ----
// fixed part: barrier block (512 B) | partial sums of the other column groups | vector ring, rounded to 1 KB
__host__ __device__ constexpr int vec_stages(int tt) { return tt == kWideTT ? 2 : kVecStages; }
__host__ __device__ constexpr uint32_t vec_tile_bytes(int tt, int mode) { return (uint32_t)(cols_per_step(mode) * tt * 4); }
__host__ __device__ constexpr uint32_t combine_bytes(int tt, int mode) {
  // kResident1: three of the four column groups of a row hand their sums over; otherwise one of two
  return (uint32_t)((mode == kResident1 ? 3 * kTileRows : kRowsPerCtaL) * tt * 4);
}
__host__ __device__ constexpr uint32_t fixed_bytes(int tt, int mode) {
  return (512u + combine_bytes(tt, mode) + (uint32_t)vec_stages(tt) * vec_tile_bytes(tt, mode) + 1023u) & ~1023u;
}
// a ring stage: [hi | lo] slabs of the column tile (kResident2), of both tiles of the pair (kResident1: hi, hi, lo,
// lo), or of both row blocks and the column tile (kStream: A0 hi, A0 lo, A1 hi, A1 lo, B hi, B lo)
__host__ __device__ constexpr uint32_t stage_bytes(int mode) {
  return (uint32_t)((mode == kStream ? 6 : (mode == kResident1 ? 4 : 2)) * kSlabBytes);
}
__host__ __device__ constexpr uint32_t resident_bytes(int mode, int nslab) {
  return (uint32_t)((mode == kResident2 ? 2 : (mode == kResident1 ? 1 : 0)) * nslab * kSlabBytes);
}
__host__ __device__ constexpr int ring_stages(int tt, int mode, int nslab) {
  const int room = (kMaxSmemL - 1024 - (int)fixed_bytes(tt, mode) - (int)resident_bytes(mode, nslab)) / (int)stage_bytes(mode);
  return room < kMaxStagesL ? room : kMaxStagesL;
}
inline size_t smem_bytes(int tt, int mode, int nslab) {
  return 1024 + (size_t)fixed_bytes(tt, mode) + resident_bytes(mode, nslab) +
         (size_t)ring_stages(tt, mode, nslab) * stage_bytes(mode);
}
// tile shape for `d` features and `tt` vector columns per pass: the most resident shape whose ring still has four
// stages (three for the streaming shape)
inline int tile_mode(int64_t d, int tt) {
  if (tt == tc::kWideTT) return kStream;
  const int ns = n_slabs(d);
  if (ring_stages(tt, kResident2, ns) >= 4) return kResident2;
  if (ring_stages(tt, kResident1, ns) >= 3) return kResident1;
  return kStream;
}

// ---------------------------------------------------------------------------------------------
// Operand images for any feature count: one block = one 128-row tile, one thread = one row.  The image is
// built slab by slab in shared memory (so that the global writes are coalesced 8 KB runs).  Layout of a row:
// see the head of this file; the two images of an operand differ in the tail slab only.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) prep_images_large_kernel(const float* __restrict__ X, int64_t n, int64_t rs,
                                                                int64_t cs, int d, const float* __restrict__ sigma,
                                                                float sigma_scalar, int sigma_len, float scale,
                                                                int ds, __half* __restrict__ img_a,
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
  const int nslab = 2 * ds + 1;
  // pass 2: slabs
  for (int s = 0; s < nslab; ++s) {
    for (int e = 0; e < kSlabK; ++e) {
      __half va = zero, vb = zero;
      if (live) {
        if (s < 2 * ds) {
          const int f = (s < ds ? s : s - ds) * kSlabK + e;
          if (f < d) {
            float xt = scaled(f);
            if (!(fabsf(xt) <= 400.0f)) xt = 0.0f;
            const __half hi = __float2half_rn(xt);
            va = vb = s < ds ? hi : __float2half_rn(xt - __half2float(hi));
          }
        } else if (e < 3) {
          va = __float2half_rn(-piece[e]);
          vb = one;
        } else if (e < 6) {
          va = one;
          vb = __float2half_rn(-piece[e - 3]);
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
                                                       sigma_scalar, sigma_len, scale, feature_slabs(d),
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
  int row_tiles;        // ceil(r / rows of a CTA)
  int n_col_tiles;      // steps of the tile loop over the whole reduction side: ceil(s / columns per step)
  int tiles_per_chunk;  // in the same unit
  int ds;               // feature slabs; an image row has 2 ds + 1 slabs
  int last_ksteps;      // K-steps of the last feature slab that carry data (1 or 2)
  int ring;             // stages of the operand ring
};

__device__ __forceinline__ void report_timeout(int* status, int code) { atomicExch(status + kStatusTimeout, code); }

template <int KT, int TT, int MODE>
__global__ void __launch_bounds__(kThreadsL, 1) kmv_tck_kernel(const SweepArgsL p) {
  constexpr int VS = vec_stages(TT);
  constexpr uint32_t kStageBytes = stage_bytes(MODE), kVecTileBytes = vec_tile_bytes(TT, MODE);
  constexpr int kRowsCta = rows_per_cta(MODE);
  constexpr int kStepCols = cols_per_step(MODE);
  constexpr int kABlocks = kRowsCta / kTileRows;
  constexpr int kBTiles = kStepCols / kColsPerTile;
  // kResident1: the two accumulator groups are neighbouring column tiles of one A block, so ONE issuer covers both
  // with 256-column MMAs
  constexpr bool kOneMma = MODE == kResident1;
  constexpr int kIssuers = kOneMma ? 1 : kGroupsL;
  // barrier block: s_full[12] | s_empty[12] | v_full[VS] | v_empty[VS] | t_full[4] | t_empty[4] | a_full | tmem
  // pointer | abort flag;  then the partial sums and the vector ring (fixed sizes), the resident A slabs, the ring
  constexpr uint32_t kSFull = 0, kSEmpty = kSFull + 8 * kMaxStagesL, kVFull = kSEmpty + 8 * kMaxStagesL;
  constexpr uint32_t kVEmpty = kVFull + 8 * VS, kTFull = kVEmpty + 8 * VS, kTEmpty = kTFull + 32;
  constexpr uint32_t kAFull = kTEmpty + 32, kTmemPtr = kAFull + 8, kAbort = kTmemPtr + 4;
  constexpr uint32_t kCombineOff = 512, kVecOff = kCombineOff + combine_bytes(TT, MODE);
  static_assert(kAbort + 4 <= kCombineOff, "barrier block overflows its 512 bytes");
  extern __shared__ unsigned char tck_smem_raw[];
  const uint32_t raw_addr = smem_u32(tck_smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  // 32-bit shared addresses from one base (generic pointers to every ring and barrier would stay live across all
  // warp roles)
  const uint32_t sm = raw_addr + pad;
  const int ds = p.ds;
  const int nslab = 2 * ds + 1;
  const uint32_t S = (uint32_t)p.ring;
  const uint32_t sm_a = sm + fixed_bytes(TT, MODE);            // resident A slabs (if any)
  const uint32_t sm_ring = sm_a + resident_bytes(MODE, nslab);  // operand ring

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int row_tile = blockIdx.x % p.row_tiles;
  const int chunk = blockIdx.x / p.row_tiles;
  const int tchunk = blockIdx.y;
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int tile_end = min(tile_begin + p.tiles_per_chunk, p.n_col_tiles);
  const int ntiles = tile_end - tile_begin;

  __shared__ int skip_launch;
  if (tid == 0) {
    const volatile int* st = reinterpret_cast<const volatile int*>(p.status);
    skip_launch = (st[kStatusTimeout] != 0 || range_raised(p.status + kStatusRange)) ? 1 : 0;
  }
  __syncthreads();
  if (skip_launch) return;

  if (tid == 0) {
#pragma unroll 1
    for (uint32_t s = 0; s < S; ++s) {
      mbar_init(sm + kSFull + 8 * s, 1);
      mbar_init(sm + kSEmpty + 8 * s, kIssuers);  // one MMA commit per issuer
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(sm + kVFull + 8 * s, 1);
      mbar_init(sm + kVEmpty + 8 * s, kEpiWarpsL);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(sm + kTFull + 8 * i, 1);
      // the warps that drain that accumulator: the eight of its group, or all sixteen (one accumulator per buffer)
      mbar_init(sm + kTEmpty + 8 * i, (kOneMma ? 2 : 1) * 4 * kColSplitL);
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
    constexpr int64_t kSlabElems = kTileRows * kSlabK;
    const __half* a_base = p.img_a + (int64_t)row_tile * kABlocks * nslab * kSlabElems;
    const float* vec_base = p.vec + (int64_t)tchunk * p.s_pad * TT;
    if (MODE != kStream && elect_one()) {
      // the CTA's A blocks are contiguous in the image: [row block][slab]
      const uint32_t bytes = (uint32_t)(kABlocks * nslab * kSlabBytes);
      mbar_expect_tx(sm + kAFull, bytes);
      for (int i = 0; i < kABlocks * nslab; ++i)
        bulk_copy_g2s(sm_a + i * kSlabBytes, a_base + (int64_t)i * kSlabElems, kSlabBytes, sm + kAFull);
    }
    __syncwarp();
    uint32_t stage = 0, wrap = 0;  // ring position of the running stage counter and its wrap parity
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
        mbar_expect_tx(vbar, kVecTileBytes);
        bulk_copy_g2s(sm + kVecOff + vstage * kVecTileBytes, vec_base + ct * kStepCols * TT, kVecTileBytes, vbar);
      }
      __syncwarp();
      // first B tile of this step; kResident1 takes the following tile too (the image is padded to four tiles)
      const __half* b_base = p.img_b + ct * kBTiles * nslab * kSlabElems;
      for (int st = 0; st <= ds; ++st) {  // ds feature slabs, then the tail
        if (ld_shared_i32_volatile(sm + kAbort)) { ok = false; break; }
        if (!mbar_wait(sm + kSEmpty + 8 * stage, wrap ^ 1u)) {
          if (lane == 0) report_timeout(p.status, kErrProducer | 1);
          st_shared_i32_volatile(sm + kAbort, 1);
          ok = false;
          break;
        }
        if (elect_one()) {
          const uint32_t bar = sm + kSFull + 8 * stage;
          const uint32_t dst = sm_ring + stage * kStageBytes;
          const bool tail = st == ds;
          // slab index of the hi part (or of the tail) and distance to the lo part within an image tile
          const int64_t s_hi = tail ? 2 * ds : st;
          mbar_expect_tx(bar, tail ? kStageBytes / 2 : kStageBytes);
          if (MODE == kStream) {
            // [A0 hi | A0 lo | A1 hi | A1 lo | B hi | B lo]; the tails take the hi positions
#pragma unroll
            for (int rb = 0; rb < 2; ++rb) {
              const __half* a_tile = a_base + (int64_t)rb * nslab * kSlabElems;
              bulk_copy_g2s(dst + rb * 2 * kSlabBytes, a_tile + s_hi * kSlabElems, kSlabBytes, bar);
              if (!tail) bulk_copy_g2s(dst + (rb * 2 + 1) * kSlabBytes, a_tile + (s_hi + ds) * kSlabElems, kSlabBytes, bar);
            }
            bulk_copy_g2s(dst + 4 * kSlabBytes, b_base + s_hi * kSlabElems, kSlabBytes, bar);
            if (!tail) bulk_copy_g2s(dst + 5 * kSlabBytes, b_base + (s_hi + ds) * kSlabElems, kSlabBytes, bar);
          } else {
            // [hi of the step's kBTiles tiles | lo of the same tiles]
#pragma unroll
            for (int t = 0; t < kBTiles; ++t) {
              const __half* b_tile = b_base + (int64_t)t * nslab * kSlabElems;
              bulk_copy_g2s(dst + t * kSlabBytes, b_tile + s_hi * kSlabElems, kSlabBytes, bar);
              if (!tail)
                bulk_copy_g2s(dst + (kBTiles + t) * kSlabBytes, b_tile + (s_hi + ds) * kSlabElems, kSlabBytes, bar);
            }
          }
        }
        __syncwarp();
        if (++stage == S) {
          stage = 0;
          wrap ^= 1u;
        }
      }
    }
  } else if (warp >= kMmaWarpL) {
    // ------------------------------ MMA issuers (one per accumulator group) ------------------------------
    // group = row block of the CTA (kStream, kResident2) or column tile of the pair (kResident1)
    reg_release<kRegsOthersL>();
    const int grp = warp - kMmaWarpL;
    uint32_t stage = 0, wrap = 0;
    bool ok = grp < kIssuers;  // kResident1: warp 16 issues 256-column MMAs for both groups, warp 17 has no work
    if (ok && MODE != kStream && !mbar_wait(sm + kAFull, 0)) {
      if (lane == 0) report_timeout(p.status, kErrMma | 1);
      st_shared_i32_volatile(sm + kAbort, 1);
      ok = false;
    }
    constexpr uint32_t kIdesc = kOneMma ? kInstrDescN256 : kInstrDesc;
    for (int j = 0; ok && j < ntiles; ++j) {
      const int buf = j & 1;
      if (ld_shared_i32_volatile(sm + kAbort)) break;
      // this group's accumulator of this buffer must have been drained (step j - 2)
      const int acc = kOneMma ? buf : grp * 2 + buf;
      if (!mbar_wait(sm + kTEmpty + 8 * acc, ((j >> 1) & 1) ^ 1)) {
        if (lane == 0) report_timeout(p.status, kErrMma | 3);
        st_shared_i32_volatile(sm + kAbort, 1);
        break;
      }
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * (kOneMma ? 2 : 1) * kColsPerTile);
      for (int st = 0; st <= ds; ++st) {
        if (!mbar_wait(sm + kSFull + 8 * stage, wrap)) {
          if (lane == 0) report_timeout(p.status, kErrMma | 2);
          st_shared_i32_volatile(sm + kAbort, 1);
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t sbase = sm_ring + stage * kStageBytes;
          const bool tail = st == ds;
          // hi slab (or tail) of this group's A block and of the step's B columns; the lo slabs follow at fixed distances
          uint32_t a_hi, a_lo, b_hi, b_lo;
          if (MODE == kStream) {
            a_hi = sbase + grp * 2 * kSlabBytes;
            a_lo = a_hi + kSlabBytes;
            b_hi = sbase + 4 * kSlabBytes;
            b_lo = b_hi + kSlabBytes;
          } else {
            const uint32_t a_blk = sm_a + (MODE == kResident2 ? grp * nslab : 0) * kSlabBytes;
            a_hi = a_blk + (tail ? 2 * ds : st) * kSlabBytes;
            a_lo = a_hi + ds * kSlabBytes;
            b_hi = sbase;
            b_lo = sbase + kBTiles * kSlabBytes;
          }
          const uint64_t ah = make_smem_desc(a_hi), bh = make_smem_desc(b_hi);
          if (tail) {
            mma_f16(d_tmem, ah, bh, kIdesc, 1u);
          } else {
            const uint64_t al = make_smem_desc(a_lo), bl = make_smem_desc(b_lo);
            const int nks = st == ds - 1 ? p.last_ksteps : 2;  // K-steps of this slab that carry data
            for (int ks = 0; ks < nks; ++ks) {
              const uint64_t ko = (uint64_t)(ks * 2);  // 32 bytes per K-step inside the 64-byte swizzle row
              mma_f16(d_tmem, ah + ko, bh + ko, kIdesc, (st > 0 || ks > 0) ? 1u : 0u);
              mma_f16(d_tmem, ah + ko, bl + ko, kIdesc, 1u);
              mma_f16(d_tmem, al + ko, bh + ko, kIdesc, 1u);
            }
          }
          mma_commit(sm + kSEmpty + 8 * stage);
          if (tail) mma_commit(sm + kTFull + 8 * acc);
        }
        __syncwarp();
        if (++stage == S) {
          stage = 0;
          wrap ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    reg_claim<kRegsEpilogueL>();
    const int q = warp & 3;
    const int grp = (warp >> 2) & 1;
    const int half = warp >> 3;  // columns half * 64 .. + 63 of the group's 128
    constexpr int NSUM = TT == kWideTT ? 16 : 2;
    // two-level summation for TT <= 4, as in the resident kernel (here the second level fits in registers);
    // the many-column form keeps one level and relies on the planner's bound on the chunk length
    uint64_t osum[NSUM], otot[TT == kWideTT ? 1 : NSUM];
#pragma unroll
    for (int i = 0; i < NSUM; ++i) osum[i] = 0ull;
#pragma unroll
    for (int i = 0; i < (TT == kWideTT ? 1 : NSUM); ++i) otot[i] = 0ull;
    bool epi_ok = true;
    // vector entries of this warp's columns inside a vector tile
    constexpr int kGroupCols = MODE == kResident1 ? kColsPerTile : 0;
    const int vcol = grp * kGroupCols + half * 64;
    // steps summed in one running sum before it is folded away (one level only for the many-column form)
    constexpr int kFlush = TT == kWideTT ? (1 << 30) : tc::kFlushTiles;
    for (int j0 = 0; j0 < ntiles && epi_ok; j0 += kFlush) {
    if constexpr (TT != kWideTT) {
      if (j0 > 0) {
#pragma unroll
        for (int i = 0; i < NSUM; ++i) {
          otot[i] = tc::add2(otot[i], osum[i]);
          osum[i] = 0ull;
        }
      }
    }
    const int j1 = TT == kWideTT ? ntiles : min(j0 + kFlush, ntiles);
    for (int j = j0; j < j1; ++j) {
      const int vstage = j % VS, buf = j & 1;
      if (ld_shared_i32_volatile(sm + kAbort)) { epi_ok = false; break; }
      const int acc = kOneMma ? buf : grp * 2 + buf;
      if (!mbar_wait(sm + kVFull + 8 * vstage, (j / VS) & 1) || !mbar_wait(sm + kTFull + 8 * acc, (j >> 1) & 1)) {
        report_timeout(p.status, kErrEpilogue | 1);
        st_shared_i32_volatile(sm + kAbort, 1);
        epi_ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) +
                             (uint32_t)((kOneMma ? buf * 2 + grp : grp * 2 + buf) * kColsPerTile + half * 64);
      // generic pointer rebuilt from the 32-bit shared address, so that no 64-bit base stays live across the loop
      const float* vsm = reinterpret_cast<const float*>(
          __cvta_shared_to_generic(sm + kVecOff + vstage * kVecTileBytes + (uint32_t)(vcol * TT * 4)));
      if constexpr (TT == kWideTT) {
        // 32 running sums per thread leave room for 16 columns at a time: four pieces through two register blocks,
        // the load of the next piece in flight while this one is evaluated; the accumulator goes back to its issuer
        // once the last piece is in registers
        uint32_t rw0[16], rw1[16];
        tmem_ld16(taddr, rw0);
        tmem_ld_wait_on(rw0);
        tmem_ld16(taddr + 16, rw1);
        epilogue_wide16<KT, 0>(rw0, vsm, osum);
        tmem_ld_wait_on(rw1);
        tmem_ld16(taddr + 32, rw0);
        epilogue_wide16<KT, 8>(rw1, vsm + 16 * TT, osum);
        tmem_ld_wait_on(rw0);
        tmem_ld16(taddr + 48, rw1);
        epilogue_wide16<KT, 0>(rw0, vsm + 32 * TT, osum);
        tmem_ld_wait_on(rw1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm + kTEmpty + 8 * acc);
        epilogue_wide16<KT, 8>(rw1, vsm + 48 * TT, osum);
      } else {
        // 32 columns at a time through one register block (two blocks in flight left no room for the constants of
        // the polynomial exponential); the accumulator goes back once the second piece is in registers -- the other
        // buffer of this group keeps the issuer busy meanwhile
        uint32_t ra[32];
        tmem_ld32(taddr, ra);
        tmem_ld_wait_on(ra);
        epilogue_32<KT, TT>(ra, vsm, osum);
        tmem_ld32(taddr + 32, ra);
        tmem_ld_wait_on(ra);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm + kTEmpty + 8 * acc);
        epilogue_32<KT, TT>(ra, vsm + 32 * TT, osum);
      }
      // the vector tile goes back to the producer, whose bulk copy will overwrite it
      const uint32_t zero = smem_reads_done(osum[0] ^ osum[NSUM - 1]);
      __syncwarp();
      if (lane == 0) mbar_arrive(sm + kVEmpty + 8 * vstage + zero);
    }
    }
    // per-thread sums of this warp's columns
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
    // Column groups of one output row meet in shared memory; the warp holding group 0 adds them in a fixed order.
    // kStream / kResident2: a row (row block grp) has the two halves; kResident1: a row has the four (grp, half).
    constexpr int kParts = MODE == kResident1 ? 4 : 2;
    const int part = MODE == kResident1 ? grp * 2 + half : half;
    const int rloc = (MODE == kResident1 ? 0 : grp * kTileRows) + q * 32 + lane;
    float* combine = reinterpret_cast<float*>(__cvta_shared_to_generic(sm + kCombineOff));  // [kParts - 1][rows of the CTA][TT]
    if (part > 0) {
#pragma unroll
      for (int t = 0; t < TT; ++t) combine[((part - 1) * kRowsCta + rloc) * TT + t] = o[t];
    }
    // all sixteen epilogue warps meet here (named barrier 1; the issuer and producer warps do not take part)
    asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarpsL * 32) : "memory");
    if (part == 0 && epi_ok && ld_shared_i32_volatile(sm + kAbort) == 0) {
      const int64_t row = (int64_t)row_tile * kRowsCta + rloc;
      float* dst = p.raw + ((int64_t)chunk * p.r_pad + row) * p.tp + tchunk * TT;
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        float acc = o[t];
#pragma unroll
        for (int g = 0; g < kParts - 1; ++g) acc += combine[(g * kRowsCta + rloc) * TT + t];
        dst[t] = acc;
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  const bool aborted = (ld_shared_i32_volatile(sm + kAbort) != 0);
  if (aborted && warp == kProducerWarpL && lane == 0) {
    // give this CTA's own bulk copies a bounded chance to land before the shared memory is released
    if (MODE != kStream) mbar_wait(sm + kAFull, 0);
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

template <int KT, int TT, int MODE>
int launch_inst(SweepArgsL args, int n_chunks, int t_chunks, cudaStream_t stream) {
  const int nslab = 2 * args.ds + 1;
  args.ring = ring_stages(TT, MODE, nslab);
  const size_t smem = smem_bytes(TT, MODE, nslab);
  // one CTA per SM is assumed (each takes all 512 TMEM columns): the shared memory must not let a second one in
  if (smem <= 116 * 1024 || smem > (size_t)kMaxSmemL || args.ring < kMinStagesL)
    return fail(FLK_ERR_BAD_ARG, "internal: K-loop kernel shared-memory plan (%zu bytes, %d stages)", smem, args.ring);
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_tck_kernel<KT, TT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kMaxSmemL));
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid((unsigned)(args.row_tiles * n_chunks), (unsigned)t_chunks, 1);
  kmv_tck_kernel<KT, TT, MODE><<<grid, kThreadsL, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <int KT, int TT>
int launch_mode(const SweepArgsL& args, int mode, int n_chunks, int t_chunks, cudaStream_t stream) {
  if constexpr (TT != kWideTT) {
    if (mode == kResident2) return launch_inst<KT, TT, kResident2>(args, n_chunks, t_chunks, stream);
    if (mode == kResident1) return launch_inst<KT, TT, kResident1>(args, n_chunks, t_chunks, stream);
  }
  return launch_inst<KT, TT, kStream>(args, n_chunks, t_chunks, stream);
}

template <int KT>
int launch_tt(const SweepArgsL& args, int tt, int mode, int n_chunks, int t_chunks, cudaStream_t stream) {
  switch (tt) {
    case 1: return launch_mode<KT, 1>(args, mode, n_chunks, t_chunks, stream);
    case 2: return launch_mode<KT, 2>(args, mode, n_chunks, t_chunks, stream);
    case 4: return launch_mode<KT, 4>(args, mode, n_chunks, t_chunks, stream);
    case kWideTT: return launch_mode<KT, kWideTT>(args, mode, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported TT=%d", tt);
}

// `args.row_tiles`, `n_col_tiles` and `tiles_per_chunk` must have been planned for tile_mode(d, tt).
inline int launch_sweep(int kernel, int d, SweepArgsL args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  args.ds = feature_slabs(d);
  args.last_ksteps = last_k_steps(d);
  const int mode = tile_mode(d, tt);
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_tt<FLK_GAUSSIAN>(args, tt, mode, n_chunks, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_tt<FLK_LAPLACIAN>(args, tt, mode, n_chunks, t_chunks, stream);
    case FLK_MATERN15: return launch_tt<FLK_MATERN15>(args, tt, mode, n_chunks, t_chunks, stream);
    case FLK_MATERN25: return launch_tt<FLK_MATERN25>(args, tt, mode, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace tck
}  // namespace flk
