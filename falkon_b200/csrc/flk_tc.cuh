// Tensor-core (tcgen05 / TMEM) kernel-vector product for fp32 data with few features (d <= 30).
//
//   raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t]
//
// Idea: the whole exponent of the kernel function is produced by ONE tf32 MMA.  Each data row is
// pre-scaled by sqrt(alpha)/sigma (alpha depends on the kernel function) and split into a tf32
// "hi" and "lo" part; the squared norm is split into 2 or 3 tf32 parts.  With the K dimension laid
// out as
//      A row (output side)    : [ xh | xh | xl | -n1 -n2 (-n3) | 1 1 (1) | 0.. ]
//      B row (reduction side) : [ 2ch | 2cl | 2ch | 1 1 (1) | -m1 -m2 (-m3) | 0.. ]
// the fp32 accumulator of  A . B^T  is  2 x.c - |x|^2 - |c|^2 = -alpha * D^2  with fp32-level
// accuracy (3xTF32: the dropped xl.cl term is below fp32 rounding).  The epilogue then needs only
// a min/max, one or two MUFU ops and the FMA with `vec` per kernel evaluation, so the FP32 pipe no
// longer carries the d-long dot product and the MUFU unit becomes the bound.
//
// Data movement: operands are stored in HBM as ready-made shared-memory images of 128-row tiles
// (128-byte-swizzled, K-major "core matrix" layout that tcgen05.mma reads), so a tile is one
// contiguous bulk copy (cp.async.bulk, the TMA engine, completion on an mbarrier) with no tensor
// map.  A CTA keeps 256 output rows (two 128-row MMA blocks) resident, streams 128-column B tiles
// through a ring, and ping-pongs two TMEM accumulators per row block so the MMA of tile j+1
// overlaps the epilogue of tile j.  Warp roles: warps 0-7 epilogue (one TMEM lane = one output
// row per thread), warp 8 bulk-copy producer, warp 9 MMA issuer and TMEM owner.
//
// Every wait on an mbarrier is bounded; when one gives up the CTA records a code in the status
// word, stops issuing work, drains its own copies, frees its TMEM and returns.
#pragma once

#include "flk_common.cuh"

namespace flk {
namespace tc {

constexpr int kRowsPerCta = 256;   // two 128-row MMA blocks
constexpr int kColsPerTile = 128;  // MMA N
constexpr int kTileRows = 128;     // rows per operand tile image
constexpr int kSlabK = 32;         // tf32 elements per 128-byte swizzle row
constexpr int kMaxD = 30;
constexpr int kThreads = 320;
constexpr uint64_t kWaitTimeoutNs = 1000000000ull;  // every device-side wait gives up after 1 s

inline bool supports_d(int64_t d) { return d >= 1 && d <= kMaxD; }
// number of tf32 pieces the squared norm is split into (3 when it costs no extra MMA K-step)
inline int norm_pieces(int64_t d) { return (round_up(3 * d + 6, 8) == round_up(3 * d + 4, 8)) ? 3 : 2; }
inline int used_k(int64_t d) { return (int)(3 * d + 2 * norm_pieces(d)); }
inline int k_steps(int64_t d) { return (int)(round_up(used_k(d), 8) / 8); }
inline int64_t padded_k(int64_t d) { return round_up(used_k(d), kSlabK); }
inline int n_slabs(int64_t d) { return (int)(padded_k(d) / kSlabK); }

// alpha such that the accumulator equals -alpha * D^2 (D^2 = squared distance in length-scale units)
inline double alpha_for(int kernel) {
  const double l2e = 1.4426950408889634;
  switch (kernel) {
    case FLK_GAUSSIAN: return 0.5 * l2e;
    case FLK_LAPLACIAN: return l2e * l2e;
    case FLK_MATERN15: return 3.0 * l2e * l2e;
    default: return 5.0 * l2e * l2e;
  }
}

// float offset of element (row r, k index e) inside a 128-row tile image
__host__ __device__ inline int image_offset(int r, int e) {
  return (e >> 5) * (kTileRows * kSlabK) + r * kSlabK + ((((e & 31) >> 2) ^ (r & 7)) << 2) + (e & 3);
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t y;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
  return __uint_as_float(y);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false when the phase did not complete within kWaitTimeoutNs.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 0; it < (1u << 30); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u && global_timer_ns() - t0 > kWaitTimeoutNs) return false;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzle shared-memory matrix descriptor (8-row groups 1024 bytes apart).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address
  desc |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset between 8-row groups
  desc |= (uint64_t)1 << 46;                      // descriptor version (sm_100)
  desc |= (uint64_t)2 << 61;                      // SWIZZLE_128B
  return desc;
}
// tf32 x tf32 -> f32, M = 128, N = 128, both operands K-major
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kColsPerTile >> 3) << 17) |
                                ((uint32_t)(128 >> 4) << 24);

// ---------------------------------------------------------------------------------------------
// Kernel functions on the accumulator (= -alpha D^2)
// ---------------------------------------------------------------------------------------------
template <int KT>
__device__ __forceinline__ float eval_acc(float acc) {
  if (KT == FLK_GAUSSIAN) {
    return ex2_approx(fminf(acc, 0.0f));
  } else {
    const float q = sqrt_approx(fmaxf(-acc, 0.0f));  // q = c * D * log2(e), c = 1, sqrt(3), sqrt(5)
    const float e = ex2_approx(-q);
    if (KT == FLK_LAPLACIAN) return e;
    const float s = q * 0.6931471805599453f;
    if (KT == FLK_MATERN15) return fmaf(q, 0.6931471805599453f, 1.0f) * e;
    return fmaf(s, fmaf(s, 1.0f / 3.0f, 1.0f), 1.0f) * e;
  }
}

// ---------------------------------------------------------------------------------------------
// Operand images
// ---------------------------------------------------------------------------------------------
// One block = one 128-row tile.  Reads X (either legal layout) through a shared tile so the read
// is coalesced, builds the swizzled image(s) in shared memory, and writes them out linearly.
__global__ void __launch_bounds__(128) prep_images_kernel(const float* __restrict__ X, int64_t n, int64_t rs,
                                                          int64_t cs, int d, const float* __restrict__ sigma,
                                                          float sigma_scalar, int sigma_len, float sqrt_alpha,
                                                          int kp, int npieces, float* __restrict__ img_a,
                                                          float* __restrict__ img_b) {
  extern __shared__ __align__(16) float prep_smem[];
  float* xin = prep_smem;                 // [128][33] scaled inputs
  float* img = prep_smem + 128 * 33;      // [128 * kp]
  __shared__ float sig[32];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * kTileRows;
  if (tid < 32) sig[tid] = (tid < d) ? (sigma != nullptr ? sigma[sigma_len == 1 ? 0 : tid] : sigma_scalar) : 1.0f;
  if (cs == 1) {
    for (int idx = tid; idx < kTileRows * d; idx += 128) {
      int r = idx / d, k = idx - r * d;
      int64_t gi = row0 + r;
      xin[r * 33 + k] = (gi < n) ? X[gi * rs + k] : 0.0f;
    }
  } else {
    for (int idx = tid; idx < kTileRows * d; idx += 128) {
      int k = idx / kTileRows, r = idx - k * kTileRows;
      int64_t gi = row0 + r;
      xin[r * 33 + k] = (gi < n) ? X[gi * rs + (int64_t)k * cs] : 0.0f;
    }
  }
  __syncthreads();
  const int r = tid;
  const bool live = (row0 + r) < n;
  double nrm = 0.0;
  for (int k = 0; k < d; ++k) {
    float xs = xin[r * 33 + k] / sig[k];  // x / sigma, rounded as in the reference
    float xt = xs * sqrt_alpha;
    xin[r * 33 + k] = xt;
    nrm += (double)xt * (double)xt;
  }
  float piece[3];
  {
    double rem = nrm;
    for (int i = 0; i < 3; ++i) {
      float p = (i < npieces) ? to_tf32((float)rem) : 0.0f;
      piece[i] = p;
      rem -= (double)p;
    }
  }
  const int tile_elems = kTileRows * kp;
  for (int which = 0; which < 2; ++which) {
    float* dst = which == 0 ? img_a : img_b;
    if (dst == nullptr) continue;  // uniform across the block
    for (int idx = tid; idx < tile_elems; idx += 128) img[idx] = 0.0f;
    __syncthreads();
    if (live) {
      for (int k = 0; k < d; ++k) {
        const float xt = xin[r * 33 + k];
        const float hi = to_tf32(xt);
        const float lo = to_tf32(xt - hi);
        if (which == 0) {
          img[image_offset(r, k)] = hi;
          img[image_offset(r, d + k)] = hi;
          img[image_offset(r, 2 * d + k)] = lo;
        } else {
          img[image_offset(r, k)] = 2.0f * hi;
          img[image_offset(r, d + k)] = 2.0f * lo;
          img[image_offset(r, 2 * d + k)] = 2.0f * hi;
        }
      }
      for (int i = 0; i < npieces; ++i) {
        const int e_norm = 3 * d + (which == 0 ? 0 : npieces) + i;
        const int e_one = 3 * d + (which == 0 ? npieces : 0) + i;
        img[image_offset(r, e_norm)] = -piece[i];
        img[image_offset(r, e_one)] = 1.0f;
      }
    }
    __syncthreads();
    float4* out4 = reinterpret_cast<float4*>(dst + (int64_t)blockIdx.x * tile_elems);
    const float4* in4 = reinterpret_cast<const float4*>(img);
    for (int idx = tid; idx < tile_elems / 4; idx += 128) out4[idx] = in4[idx];
    __syncthreads();
  }
}

inline int prep_images(int kernel, const void* X, int64_t n, int64_t rs, int64_t cs, int d, const float* sigma_dev,
                       float sigma_scalar, int sigma_len, int64_t rows_pad, float* img_a, float* img_b,
                       cudaStream_t stream) {
  const int kp = (int)padded_k(d);
  const size_t smem = sizeof(float) * (size_t)(128 * 33 + kTileRows * kp);
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(prep_images_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(sizeof(float) * (128 * 33 + kTileRows * 96))));
    if (dev < 16) configured[dev] = true;
  }
  const float sqrt_alpha = (float)sqrt(alpha_for(kernel));
  const int blocks = (int)(rows_pad / kTileRows);
  prep_images_kernel<<<blocks, 128, smem, stream>>>(reinterpret_cast<const float*>(X), n, rs, cs, d, sigma_dev,
                                                    sigma_scalar, sigma_len, sqrt_alpha, kp, norm_pieces(d), img_a,
                                                    img_b);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Main sweep kernel
// ---------------------------------------------------------------------------------------------
struct SweepArgs {
  const float* img_a;  // [r_pad / 128] tile images (output side)
  const float* img_b;  // [s_pad / 128] tile images (reduction side)
  const float* vec;    // [t_chunks][s_pad][TT]
  float* raw;          // [n_chunks][r_pad][tp]
  int* status;         // device status word (0 = clean)
  int tp;
  int64_t r_pad;
  int64_t s_pad;
  int row_tiles;        // ceil(r / 256)
  int n_col_tiles;      // ceil(s / 128)
  int tiles_per_chunk;
  int ksteps;           // MMA K-steps (8 tf32 each) actually carrying data
};

template <int NSLAB>
struct TcCfg {
  static constexpr int KP = NSLAB * kSlabK;
  static constexpr int STAGES = NSLAB == 3 ? 2 : (NSLAB == 2 ? 3 : 6);
  static constexpr int TILE_BYTES = kTileRows * KP * 4;   // one operand tile image
  static constexpr int A_BYTES = 2 * TILE_BYTES;          // 256 resident rows
};

template <int NSLAB, int TT>
constexpr size_t tc_smem_bytes() {
  using C = TcCfg<NSLAB>;
  return 1024 /* alignment slack */ + (size_t)C::A_BYTES + (size_t)C::STAGES * C::TILE_BYTES +
         (size_t)C::STAGES * kColsPerTile * TT * 4 + 256 /* barriers + tmem pointer */;
}

// error codes written to the status word: role * 16 + which wait
enum { kErrProducer = 0x10, kErrMma = 0x20, kErrEpilogue = 0x30 };

template <int KT, int NSLAB, int TT>
__global__ void __launch_bounds__(kThreads, 1) kmv_tc_kernel(const SweepArgs p) {
  using C = TcCfg<NSLAB>;
  constexpr int S = C::STAGES;
  extern __shared__ unsigned char tc_smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  const uint32_t raw_addr = smem_u32(tc_smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* smem = tc_smem_raw + pad;
  unsigned char* a_smem = smem;
  unsigned char* b_smem = smem + C::A_BYTES;
  float* vs = reinterpret_cast<float*>(b_smem + S * C::TILE_BYTES);  // [S][128][TT]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(vs) + S * kColsPerTile * TT * 4);
  // barrier map: [0] a_full, [1..S] b_full, [1+S..2S] b_empty, then tmem_full[4], tmem_empty[4]
  uint64_t* bar_a_full = bars;
  uint64_t* bar_b_full = bars + 1;
  uint64_t* bar_b_empty = bars + 1 + S;
  uint64_t* bar_t_full = bars + 1 + 2 * S;
  uint64_t* bar_t_empty = bars + 5 + 2 * S;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 9 + 2 * S);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int row_tile = blockIdx.x % p.row_tiles;
  const int chunk = blockIdx.x / p.row_tiles;
  const int tchunk = blockIdx.y;
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int tile_end = min(tile_begin + p.tiles_per_chunk, p.n_col_tiles);
  const int ntiles = tile_end - tile_begin;

  // a CTA of this launch already gave up: do not start (keeps a failed launch short)
  __shared__ int launch_already_failed;
  if (tid == 0) launch_already_failed = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
  __syncthreads();
  if (launch_already_failed) return;

  if (tid == 0) {
    mbar_init(smem_u32(bar_a_full), 1);
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(bar_b_full + s), 1);
      mbar_init(smem_u32(bar_b_empty + s), 1 + 8);  // MMA commit + one arrive per epilogue warp
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(bar_t_full + i), 1);
      mbar_init(smem_u32(bar_t_empty + i), 4);  // the 4 warps of the row block's warpgroup
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_ptr), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 8) {
    // ------------------------------ bulk-copy producer ------------------------------
    if (lane == 0) {
      const float* a_src = p.img_a + (int64_t)row_tile * 2 * (kTileRows * C::KP);
      mbar_expect_tx(smem_u32(bar_a_full), C::A_BYTES);
      bulk_copy_g2s(smem_u32(a_smem), a_src, C::TILE_BYTES, smem_u32(bar_a_full));
      bulk_copy_g2s(smem_u32(a_smem) + C::TILE_BYTES, a_src + kTileRows * C::KP, C::TILE_BYTES,
                    smem_u32(bar_a_full));
      const float* vec_base = p.vec + (int64_t)tchunk * p.s_pad * TT;
      for (int j = 0; j < ntiles; ++j) {
        const int stage = j % S;
        if (*abort_flag) break;
        if (!mbar_wait(smem_u32(bar_b_empty + stage), ((j / S) & 1) ^ 1)) {
          atomicExch(p.status, kErrProducer | 1);
          *abort_flag = 1;
          break;
        }
        const int64_t ct = tile_begin + j;
        const uint32_t bar = smem_u32(bar_b_full + stage);
        mbar_expect_tx(bar, C::TILE_BYTES + kColsPerTile * TT * 4);
        bulk_copy_g2s(smem_u32(b_smem) + stage * C::TILE_BYTES, p.img_b + ct * (kTileRows * C::KP), C::TILE_BYTES,
                      bar);
        bulk_copy_g2s(smem_u32(vs) + stage * kColsPerTile * TT * 4, vec_base + ct * kColsPerTile * TT,
                      kColsPerTile * TT * 4, bar);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(smem_u32(bar_a_full), 0);
      if (!ok) {
        atomicExch(p.status, kErrMma | 1);
        *abort_flag = 1;
      }
      const uint64_t a_desc0 = make_smem_desc(smem_u32(a_smem));
      for (int j = 0; ok && j < ntiles; ++j) {
        const int stage = j % S, buf = j & 1;
        if (*abort_flag) break;
        if (!mbar_wait(smem_u32(bar_b_full + stage), (j / S) & 1)) {
          atomicExch(p.status, kErrMma | 2);
          *abort_flag = 1;
          break;
        }
        const uint64_t b_desc0 = make_smem_desc(smem_u32(b_smem) + stage * C::TILE_BYTES);
        for (int rb = 0; rb < 2; ++rb) {
          if (!mbar_wait(smem_u32(bar_t_empty + rb * 2 + buf), ((j >> 1) & 1) ^ 1)) {
            atomicExch(p.status, kErrMma | 3);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)((rb * 2 + buf) * kColsPerTile);
          for (int ks = 0; ks < p.ksteps; ++ks) {
            // 32 bytes (8 tf32) per K-step inside a 128-byte swizzle row; 16 KiB per 32-wide slab
            const uint64_t koff = (uint64_t)((ks >> 2) * ((kTileRows * 128) >> 4) + (ks & 3) * 2);
            const uint64_t adesc = a_desc0 + (uint64_t)(rb * (C::TILE_BYTES >> 4)) + koff;
            const uint64_t bdesc = b_desc0 + koff;
            mma_tf32(d_tmem, adesc, bdesc, kInstrDesc, ks > 0 ? 1u : 0u);
          }
          mma_commit(smem_u32(bar_t_full + rb * 2 + buf));
        }
        if (!ok) break;
        mma_commit(smem_u32(bar_b_empty + stage));
      }
    }
  } else {
    // ------------------------------ epilogue (warps 0-7) ------------------------------
    const int rb = warp >> 2;  // row block = warpgroup
    const int q = warp & 3;    // TMEM lane quarter this warp may access
    float oacc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) oacc[t] = 0.0f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int stage = j % S, buf = j & 1;
      if (*abort_flag) { ok = false; break; }
      if (!mbar_wait(smem_u32(bar_b_full + stage), (j / S) & 1) ||
          !mbar_wait(smem_u32(bar_t_full + rb * 2 + buf), (j >> 1) & 1)) {
        atomicExch(p.status, kErrEpilogue | 1);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const float* vsm = vs + stage * kColsPerTile * TT;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((rb * 2 + buf) * kColsPerTile);
#pragma unroll 1
      for (int c0 = 0; c0 < kColsPerTile; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        tmem_ld_wait();
        if constexpr (TT == 1) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 v4 = *reinterpret_cast<const float4*>(vsm + c0 + c);
            oacc[0] = fmaf(eval_acc<KT>(__uint_as_float(r[c + 0])), v4.x, oacc[0]);
            oacc[0] = fmaf(eval_acc<KT>(__uint_as_float(r[c + 1])), v4.y, oacc[0]);
            oacc[0] = fmaf(eval_acc<KT>(__uint_as_float(r[c + 2])), v4.z, oacc[0]);
            oacc[0] = fmaf(eval_acc<KT>(__uint_as_float(r[c + 3])), v4.w, oacc[0]);
          }
        } else if constexpr (TT == 2) {
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float4 v4 = *reinterpret_cast<const float4*>(vsm + (c0 + c) * 2);
            const float k0 = eval_acc<KT>(__uint_as_float(r[c + 0]));
            const float k1 = eval_acc<KT>(__uint_as_float(r[c + 1]));
            oacc[0] = fmaf(k0, v4.x, oacc[0]);
            oacc[1] = fmaf(k0, v4.y, oacc[1]);
            oacc[0] = fmaf(k1, v4.z, oacc[0]);
            oacc[1] = fmaf(k1, v4.w, oacc[1]);
          }
        } else {
          static_assert(TT % 4 == 0, "TT must be 1, 2 or a multiple of 4");
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float kv = eval_acc<KT>(__uint_as_float(r[c]));
#pragma unroll
            for (int t4 = 0; t4 < TT; t4 += 4) {
              const float4 v4 = *reinterpret_cast<const float4*>(vsm + (c0 + c) * TT + t4);
              oacc[t4 + 0] = fmaf(kv, v4.x, oacc[t4 + 0]);
              oacc[t4 + 1] = fmaf(kv, v4.y, oacc[t4 + 1]);
              oacc[t4 + 2] = fmaf(kv, v4.z, oacc[t4 + 2]);
              oacc[t4 + 3] = fmaf(kv, v4.w, oacc[t4 + 3]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(bar_t_empty + rb * 2 + buf));
        mbar_arrive(smem_u32(bar_b_empty + stage));
      }
    }
    if (ok) {
      const int64_t row = (int64_t)row_tile * kRowsPerCta + rb * 128 + q * 32 + lane;
      float* dst = p.raw + ((int64_t)chunk * p.r_pad + row) * p.tp + tchunk * TT;
#pragma unroll
      for (int t = 0; t < TT; ++t) dst[t] = oacc[t];
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 8 && lane == 0) {
    // give this CTA's own bulk copies a bounded chance to land before the shared memory is released
    mbar_wait(smem_u32(bar_a_full), 0);
    for (int s = 0; s < S; ++s) {
      for (int par = 0; par < 2; ++par) {
        if (mbar_try_wait(smem_u32(bar_b_full + s), par)) break;
      }
    }
  }
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int KT, int NSLAB, int TT>
int launch_sweep_inst(const SweepArgs& args, int n_chunks, int t_chunks, cudaStream_t stream) {
  constexpr size_t smem = tc_smem_bytes<NSLAB, TT>();
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_tc_kernel<KT, NSLAB, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid((unsigned)(args.row_tiles * n_chunks), (unsigned)t_chunks, 1);
  kmv_tc_kernel<KT, NSLAB, TT><<<grid, kThreads, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <int KT, int NSLAB>
int launch_sweep_tt(const SweepArgs& args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  switch (tt) {
    case 1: return launch_sweep_inst<KT, NSLAB, 1>(args, n_chunks, t_chunks, stream);
    case 2: return launch_sweep_inst<KT, NSLAB, 2>(args, n_chunks, t_chunks, stream);
    case 4: return launch_sweep_inst<KT, NSLAB, 4>(args, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported TT=%d", tt);
}

template <int KT>
int launch_sweep_kt(int nslab, const SweepArgs& args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  switch (nslab) {
    case 1: return launch_sweep_tt<KT, 1>(args, tt, n_chunks, t_chunks, stream);
    case 2: return launch_sweep_tt<KT, 2>(args, tt, n_chunks, t_chunks, stream);
    case 3: return launch_sweep_tt<KT, 3>(args, tt, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported slab count %d", nslab);
}

inline int launch_sweep(int kernel, int d, SweepArgs args, int tt, int n_chunks, int t_chunks, cudaStream_t stream) {
  args.ksteps = k_steps(d);
  const int nslab = n_slabs(d);
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_sweep_kt<FLK_GAUSSIAN>(nslab, args, tt, n_chunks, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_sweep_kt<FLK_LAPLACIAN>(nslab, args, tt, n_chunks, t_chunks, stream);
    case FLK_MATERN15: return launch_sweep_kt<FLK_MATERN15>(nslab, args, tt, n_chunks, t_chunks, stream);
    case FLK_MATERN25: return launch_sweep_kt<FLK_MATERN25>(nslab, args, tt, n_chunks, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace tc
}  // namespace flk
