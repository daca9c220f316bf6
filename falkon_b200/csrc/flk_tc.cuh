// Tensor-core (tcgen05 / TMEM) kernel-vector product for fp32 data with few features (d <= 30).
//
//   raw[chunk][i][t] = sum_{j in chunk} k(a_i, b_j) vec[j][t]
//
// Idea: the whole exponent of the kernel function is produced by ONE fp16 MMA with fp32
// accumulation.  Each data row is pre-scaled by s / sigma (s depends on the kernel function) and
// split into an fp16 "hi" and an fp16 "lo" part (22 significant bits together); half the squared
// norm is split into 2 or 3 fp16 parts.  With the K dimension laid out as
//      A row (output side)    : [ xh | xh | xl | -n1 -n2 (-n3) | 1 1 (1) | 0.. ]
//      B row (reduction side) : [ ch | cl | ch | 1 1 (1) | -m1 -m2 (-m3) | 0.. ]
// the fp32 accumulator of  A . B^T  is  x.c - |x|^2/2 - |c|^2/2 = -(s^2/2) D^2  with fp32-level
// accuracy (every fp16 x fp16 product is exact in fp32; the dropped xl.cl term is below fp32
// rounding).  The epilogue then needs only a min/max, one or two MUFU ops and the FMA with `vec`
// per kernel evaluation: the FP32 pipe no longer carries the d-long dot product, and the MUFU
// unit (16 lanes per SM) becomes the bound.  Part of the exponentials is therefore evaluated by a
// degree-5 polynomial on the FMA pipe instead (range reduction with the round-to-integer trick),
// which runs beside the MUFU unit.
//
// fp16 has a narrow exponent: a row whose scaled half squared norm exceeds kNormLimit cannot be
// represented.  The image builder raises a flag in device memory when it meets such a row; the
// sweep kernel then does nothing and the caller's SIMT kernels (launched behind it, gated on the
// same flag) produce the result instead.  No host round trip is involved.
//
// Data movement: operands are stored in HBM as ready-made shared-memory images of 128-row tiles
// (64-byte-swizzled, K-major "core matrix" layout that tcgen05.mma reads), so a tile is one
// contiguous bulk copy (cp.async.bulk, the TMA engine, completion on an mbarrier) with no tensor
// map.  A CTA keeps 512 output rows (four 128-row MMA blocks, one 128-column fp32 accumulator each:
// all 512 TMEM columns) resident and streams 128-column B tiles through a ring.  Sixteen epilogue
// warps (four per row block, one TMEM lane = one output row per thread) read the accumulator in
// 32-column pieces, software-pipelined against the evaluation, and hand the accumulator back to
// the MMA issuer once the second half of it is in registers, so the MMA of tile j+1 of a row
// block (and the barrier round trips around it) runs under the evaluation of the second half of
// tile j, and the other three row blocks keep the MUFU and FMA pipes busy meanwhile.
// Warps 16-19 = MMA issuers, one per row block and per SM sub-partition (a queued tcgen05.mma
// delays the other warps of its sub-partition, so the issue load is spread evenly; warp 16 also
// owns the TMEM allocation), warp 20 = bulk-copy producer.
//
// Every wait on an mbarrier is bounded; when one gives up the CTA records a code in the status
// word, stops issuing work, drains its own copies, frees its TMEM and returns.
#pragma once

#include <cuda_fp16.h>

#include "flk_common.cuh"

namespace flk {
namespace tc {

constexpr int kRowBlocks = 4;                       // 128-row MMA blocks per CTA
constexpr int kTileRows = 128;                      // rows per operand tile image (MMA M)
constexpr int kRowsPerCta = kRowBlocks * kTileRows; // 512
constexpr int kColsPerTile = 128;                   // MMA N
constexpr int kSlabK = 32;                          // fp16 elements per 64-byte swizzle row
constexpr int kMmaK = 16;                           // fp16 elements per MMA K-step
constexpr int kMaxD = 30;
constexpr int kEpilogueWarps = 4 * kRowBlocks;
constexpr int kMmaWarp0 = kEpilogueWarps;                // warps 16..19: MMA issuer of row block (warp - 16)
constexpr int kProducerWarp = kMmaWarp0 + kRowBlocks;    // warp 20
// Warps 21-23 do no work: they fill up the producer's warpgroup, because registers are handed back and
// claimed (setmaxnreg) by whole warpgroups of four consecutive warps.
constexpr int kThreads = (kEpilogueWarps + kRowBlocks + 4) * 32;
// Register budget per thread.  A CTA of 24 warps puts six warps on each SM sub-partition (16384 registers
// each), so the kernel starts with 80 registers per thread (6 x 32 x 80 = 15360 per sub-partition).  The MMA
// issuers and the producer need few: both warpgroups hand registers back at once and the four epilogue
// warpgroups (one warp per sub-partition each) claim them.  The pool that setmaxnreg redistributes is what the
// CTA was launched with (24 warps x 80), so the new counts must add up to no more than that, or the claim
// would wait for ever.  With 80 the epilogue spilled a register or two in most instantiations, and a spilled
// register may be one that a tcgen05.ld in flight is still to fill.
// The split (104, 32, 32) compiles every instantiation without spills except the plain (unfolded) Gaussian
// single-column sweep, which needs the milder split (96, 56, 40): both sum to the launch-time pool of
// 24 warps x 80 registers.  The build fails when any tensor-core instantiation reports spills.
template <int KT, int TT, bool FOLD>
struct RegBudget {
  static constexpr bool kMild = KT == FLK_GAUSSIAN && TT == 1 && !FOLD;
  static constexpr int kEpilogue = kMild ? 96 : 104;
  static constexpr int kMma = kMild ? 56 : 32;
  static constexpr int kProducer = kMild ? 40 : 32;
  static_assert(kEpilogueWarps * kEpilogue + 4 * kMma + 4 * kProducer <= (kThreads / 32) * 80,
                "register re-partitioning exceeds the pool the CTA is launched with");
  static_assert(kEpilogue % 8 == 0 && kMma % 8 == 0 && kProducer % 8 == 0, "setmaxnreg takes multiples of 8");
};
constexpr int kVecStages = 4;                       // ring of vector tiles
constexpr uint64_t kWaitTimeoutNs = 1000000000ull;  // every device-side wait gives up after 1 s
constexpr float kNormLimit = 60000.0f;              // largest half squared norm an image may carry
#ifndef FLK_TC_POLY_PAIRS
#define FLK_TC_POLY_PAIRS 4
#endif
// of the 16 column pairs of every 32-column accumulator piece, how many take the FMA-pipe exponential (Gaussian;
// measured on config 2 in 30-step runs under the board's power cap: 2 -> 9.89 ms per fdmmv, 3 -> 9.50, 4 -> 9.37 - 9.47,
// 5 -> 9.59 - 9.64, 6 -> 9.79 - 9.87, 7 -> 10.10)
constexpr int kPolyPairs = FLK_TC_POLY_PAIRS;

// words of the 256-byte status block at the front of the workspace
// kStatusRange: raised by what is built per call (folded images: a vector entry that is not finite, a row out of
// range); kStatusRangeX1 / X2: raised by the image builder of that operand (kept when the caller keeps the images)
enum { kStatusTimeout = 0, kStatusRange = 1, kStatusRangeX1 = 2, kStatusRangeX2 = 3 };
static_assert(kStatusRangeX2 - kStatusRange + 1 == kRangeWords, "the gate reads these words as one group");

inline bool supports_d(int64_t d) { return d >= 1 && d <= kMaxD; }
// number of fp16 pieces half the squared norm is split into (3 when it costs no extra MMA K-step)
inline int norm_pieces(int64_t d) { return (round_up(3 * d + 6, kMmaK) == round_up(3 * d + 4, kMmaK)) ? 3 : 2; }
inline int used_k(int64_t d) { return (int)(3 * d + 2 * norm_pieces(d)); }
inline int k_steps(int64_t d) { return (int)(round_up(used_k(d), kMmaK) / kMmaK); }
inline int64_t padded_k(int64_t d) { return round_up(used_k(d), kSlabK); }
inline int n_slabs(int64_t d) { return (int)(padded_k(d) / kSlabK); }

// s^2 such that the accumulator equals -(s^2 / 2) D^2 (D^2 = squared distance in length-scale
// units): Gaussian -> -(log2(e) / 2) D^2 (ready for ex2); the others -> -D^2.
inline double scale_sq_for(int kernel) { return kernel == FLK_GAUSSIAN ? 1.4426950408889634 : 2.0; }

// fp16-element offset of element (row r, k index e) inside a 128-row tile image
__host__ __device__ inline int image_offset(int r, int e) {
  return (e >> 5) * (kTileRows * kSlabK) + r * kSlabK + ((((e & 31) >> 3) ^ ((r >> 1) & 3)) << 3) + (e & 7);
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// One lane of a converged warp.  Issuing tcgen05.mma / commit / bulk copies under this predicate
// (instead of `lane == 0` inside a divergent branch) lets the compiler keep descriptors and
// addresses in uniform registers; a divergent single-lane issue path costs well over a hundred
// cycles per MMA.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, 0xFFFFFFFF;\n\t"
      "selp.b32 %0, 1, 0, px;\n\t}"
      : "=r"(pred));
  return pred != 0;
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
// A warp that read a shared-memory buffer with ordinary loads hands it back to a bulk-copy producer, which will
// overwrite it through the async proxy.  Two things must hold before the arrive that releases the buffer: the
// loads have returned -- an arrive does not wait for loads in flight, and nothing else does when their consumers
// were scheduled after it; `dep` must depend on the last of them (the running sums they feed), and the returned
// zero is added to the barrier address, so the arrive cannot issue earlier -- and the generic and the async proxy are
// ordered by a proxy fence.  Without this a vector tile was overwritten under the loads of the previous one
// whenever the producer stood waiting for exactly that buffer (wrong sums in a few rows, varying from run to run).
__device__ __forceinline__ uint32_t smem_reads_done(uint64_t dep) {
  uint32_t lo, hi, zero;
  asm volatile("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(dep));
  asm volatile("and.b32 %0, %1, 0;" : "=r"(zero) : "r"(lo ^ hi));
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  return zero;
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
// Low 32 bits of the nanosecond timer (wraps every 4.29 s; differences of two readings stay valid below that).
__device__ __forceinline__ uint32_t timer_lo_ns() {
  uint32_t t;
  asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(t));
  return t;
}
// Bounded wait: false when the phase did not complete within about a second (kWaitTimeoutNs), or after 2^26
// probes, whichever comes first.  A waiting warp backs off with a short nanosleep between probes: a warp that
// spins on a barrier competes for issue slots with the epilogue warps of its SM sub-partition (measured: the
// sub-partition hosting the spinning MMA warp ran its epilogue warps almost 2x slower and set the pace of the
// whole CTA).  Inlined and kept to two registers (start time, probe count): the kernels that use it re-partition
// their registers between warp roles (setmaxnreg), which rules out out-of-line calls.
#ifndef FLK_TC_BACKOFF_NS
#define FLK_TC_BACKOFF_NS 20
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint32_t t0 = timer_lo_ns();
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (FLK_TC_BACKOFF_NS > 0) __nanosleep(FLK_TC_BACKOFF_NS);
    if (mbar_try_wait(bar, parity)) return true;
    if (timer_lo_ns() - t0 > (uint32_t)kWaitTimeoutNs) return false;
  }
  return false;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Register re-partitioning between warp roles; both are executed by all four warps of a warpgroup.
template <int N>
__device__ __forceinline__ void reg_release() {  // lower this warpgroup's register count to N
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_claim() {  // raise it to N (waits until the pool holds enough)
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
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

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// The two wrappers below carry extra operands whose only purpose is to pin the instruction order the
// software pipeline needs (the compiler is otherwise free to move independent arithmetic across
// them): a load is issued BEFORE the evaluation of the piece that is already in registers, and the
// wait for it comes AFTER that evaluation.
//   tmem_ld32(taddr, dst, held): issues the load into `dst`; `held` (the piece about to be
//     evaluated) is tied as read-write, so its evaluation cannot be scheduled above the issue.
//   tmem_ld_wait_on(dst, acc): waits for the load into `dst`; the running sums `acc` are tied as
//     read-write, so every evaluation that feeds them is scheduled above the wait.
#define FLK_R32_OUT(r)                                                                                         \
  "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),  \
      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),   \
      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),  \
      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
#define FLK_R32_INOUT(r)                                                                                       \
  "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),  \
      "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),   \
      "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),  \
      "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
#define FLK_TMEM_LD32_TEXT                                                                   \
  "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                  \
  "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                  \
  "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(FLK_TMEM_LD32_TEXT : FLK_R32_OUT(r) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32], uint32_t (&held)[32]) {
  // operands 0-31 = destination, 32 = address, 33.. = the held piece (tied only)
  asm volatile(FLK_TMEM_LD32_TEXT
               : FLK_R32_OUT(r)
               : "r"(taddr), "r"(held[0]), "r"(held[4]), "r"(held[8]), "r"(held[12]), "r"(held[16]), "r"(held[20]),
                 "r"(held[24]), "r"(held[28])
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[32], uint64_t (&acc)[2]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : FLK_R32_INOUT(r), "+l"(acc[0]), "+l"(acc[1]) : : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : FLK_R32_INOUT(r) : : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[32], float (&acc)[4]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : FLK_R32_INOUT(r), "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
               :
               : "memory");
}
// 16-column variants for the many-column epilogue (its 32 running sums leave room for 16 accumulator columns).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// K-major, 64-byte swizzle shared-memory matrix descriptor (8-row groups 512 bytes apart).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address
  desc |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(512 >> 4) << 32;             // stride byte offset between 8-row groups
  desc |= (uint64_t)1 << 46;                      // descriptor version (sm_100)
  desc |= (uint64_t)4 << 61;                      // SWIZZLE_64B
  return desc;
}
// fp16 x fp16 -> f32, M = 128, N = 128, both operands K-major
constexpr uint32_t kInstrDesc = (1u << 4) | ((uint32_t)(kColsPerTile >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);

// ---------------------------------------------------------------------------------------------
// Packed fp32 pairs (sm_100 add/sub/fma.f32x2: two fp32 operations per issued instruction).  The
// epilogue is bound by instruction issue once part of the exponentials leaves the MUFU unit, so
// everything that can be done on two columns at once is.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ void ld_shared_f4(uint32_t addr, float& a, float& b, float& c, float& d) {
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "r"(addr) : "memory");
}
__device__ __forceinline__ void st_shared_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// ---------------------------------------------------------------------------------------------
// Kernel functions on the accumulator
// ---------------------------------------------------------------------------------------------
// 2^x on the FMA pipe for a pair of arguments: n = round(x) through the 1.5 * 2^23 trick, degree-5
// minimax polynomial of 2^f on f = x - n in [-1/2, 1/2] (relative error 2.4e-7), exponent patched
// in with integer arithmetic.  x is clamped at -126 so the patched exponent never wraps; arguments
// a hair above zero (rounding, coincident points) are fine.
__device__ __forceinline__ void ex2_fma_pair(float x0, float x1, float& y0, float& y1) {
  const uint64_t magic = pack2(12582912.0f, 12582912.0f);
  const uint64_t x = pack2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
  const uint64_t t = add2(x, magic);
  const uint64_t f = sub2(x, sub2(t, magic));
  uint64_t p = pack2(0.001327647129073739f, 0.001327647129073739f);
  p = fma2(p, f, pack2(0.009675540961325169f, 0.009675540961325169f));
  p = fma2(p, f, pack2(0.05550713092088699f, 0.05550713092088699f));
  p = fma2(p, f, pack2(0.24022120237350464f, 0.24022120237350464f));
  p = fma2(p, f, pack2(0.6931469440460205f, 0.6931469440460205f));
  p = fma2(p, f, pack2(1.0000001192092896f, 1.0000001192092896f));
  float p0, p1, t0, t1;
  unpack2(p, p0, p1);
  unpack2(t, t0, t1);
  y0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  y1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Distance-type kernel functions: everything but the final exponential.  acc = -D^2; returns the argument of
// the exponential in base 2 and the polynomial factor in front of it.
template <int KT>
__device__ __forceinline__ void pre_exp(float acc, float& arg2, float& factor) {
  const float dist = sqrt_approx(fmaxf(-acc, 0.0f));
  if (KT == FLK_LAPLACIAN) {
    arg2 = dist * (-kLog2e);
    factor = 1.0f;
  } else if (KT == FLK_MATERN15) {
    const float s = dist * 1.7320508075688772f;
    arg2 = s * (-kLog2e);
    factor = 1.0f + s;
  } else {
    const float s = dist * 2.23606797749979f;
    arg2 = s * (-kLog2e);
    factor = fmaf(s, fmaf(s, 1.0f / 3.0f, 1.0f), 1.0f);
  }
}

// Two adjacent accumulator columns -> two kernel values.  POLY selects the FMA-pipe exponential for this pair
// (the square root of the Laplacian / Matern kernels always runs on the MUFU unit).
// Gaussian: acc = -(log2(e) / 2) D^2.  The image builder rounds the norm up, so acc errs on the negative side;
// what is left above zero for coincident points is accumulation rounding (k <= 1 + ~1e-7), which is not worth
// an extra instruction per evaluation.
template <int KT, bool POLY>
__device__ __forceinline__ void eval_pair(uint32_t b0, uint32_t b1, float& k0, float& k1) {
  if constexpr (KT == FLK_GAUSSIAN) {
    if constexpr (POLY) {
      ex2_fma_pair(__uint_as_float(b0), __uint_as_float(b1), k0, k1);
    } else {
      k0 = ex2_approx(__uint_as_float(b0));
      k1 = ex2_approx(__uint_as_float(b1));
    }
  } else {
    float a0, a1, f0, f1;
    pre_exp<KT>(__uint_as_float(b0), a0, f0);
    pre_exp<KT>(__uint_as_float(b1), a1, f1);
    if constexpr (POLY) {
      ex2_fma_pair(a0, a1, k0, k1);
    } else {
      k0 = ex2_approx(a0);
      k1 = ex2_approx(a1);
    }
    if constexpr (KT != FLK_LAPLACIAN) {
      k0 *= f0;
      k1 *= f1;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Operand images
// ---------------------------------------------------------------------------------------------
// One block = one 128-row tile.  Reads X (either legal layout) through a shared tile so the read
// is coalesced, builds the swizzled image(s) in shared memory, and writes them out linearly.
__global__ void __launch_bounds__(128) prep_images_kernel(const float* __restrict__ X, int64_t n, int64_t rs,
                                                          int64_t cs, int d, const float* __restrict__ sigma,
                                                          float sigma_scalar, int sigma_len, float scale,
                                                          int kp, int npieces, __half* __restrict__ img_a,
                                                          __half* __restrict__ img_b, int* __restrict__ range_word) {
  extern __shared__ __align__(16) unsigned char prep_smem_raw[];
  float* xin = reinterpret_cast<float*>(prep_smem_raw);            // [128][33] scaled inputs
  __half* img = reinterpret_cast<__half*>(xin + kTileRows * 33);   // [128 * kp]
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
  // squared norm of the value the two fp16 parts actually represent (keeps coincident points at
  // an accumulator of -|lo|^2 <= 0 up to rounding)
  double nrm = 0.0;
  bool out_of_range = false;
  for (int k = 0; k < d; ++k) {
    const float xs = xin[r * 33 + k] / sig[k];  // x / sigma, rounded as in the reference
    float xt = xs * scale;
    if (!(fabsf(xt) <= 400.0f)) {  // also catches NaN / inf; 400^2 / 2 > kNormLimit
      out_of_range = true;
      xt = 0.0f;
    }
    xin[r * 33 + k] = xt;
    const float hi = __half2float(__float2half_rn(xt));
    const float lo = __half2float(__float2half_rn(xt - hi));
    const double rep = (double)hi + (double)lo;
    nrm += rep * rep;
  }
  double half_norm = 0.5 * nrm;
  if (half_norm > (double)kNormLimit) {
    out_of_range = true;
    half_norm = 0.0;
  }
  if (out_of_range && live) atomicOr(range_word, 1);
  float piece[3];
  {
    // the last piece is rounded up: the represented norm is never below the true one, so the
    // accumulator errs on the negative side (k <= 1 for coincident points up to accumulation rounding)
    double rem = half_norm;
    for (int i = 0; i < 3; ++i) {
      float pc = 0.0f;
      if (i < npieces) {
        const float remf = __double2float_ru(rem);
        pc = __half2float(i == npieces - 1 ? __float2half_ru(remf) : __float2half_rn(remf));
      }
      piece[i] = pc;
      rem -= (double)pc;
    }
  }
  const int tile_elems = kTileRows * kp;
  const __half one = __float2half_rn(1.0f);
  for (int which = 0; which < 2; ++which) {
    __half* dst = which == 0 ? img_a : img_b;
    if (dst == nullptr) continue;  // uniform across the block
    {
      uint32_t* z = reinterpret_cast<uint32_t*>(img);
      for (int idx = tid; idx < tile_elems / 2; idx += 128) z[idx] = 0u;
    }
    __syncthreads();
    if (live) {
      for (int k = 0; k < d; ++k) {
        const float xt = xin[r * 33 + k];
        const __half hi = __float2half_rn(xt);
        const __half lo = __float2half_rn(xt - __half2float(hi));
        img[image_offset(r, k)] = hi;
        img[image_offset(r, d + k)] = which == 0 ? hi : lo;
        img[image_offset(r, 2 * d + k)] = which == 0 ? lo : hi;
      }
      for (int i = 0; i < npieces; ++i) {
        const int e_norm = 3 * d + (which == 0 ? 0 : npieces) + i;
        const int e_one = 3 * d + (which == 0 ? npieces : 0) + i;
        img[image_offset(r, e_norm)] = __float2half_rn(-piece[i]);
        img[image_offset(r, e_one)] = one;
      }
    }
    __syncthreads();
    uint4* out4 = reinterpret_cast<uint4*>(dst + (int64_t)blockIdx.x * tile_elems);
    const uint4* in4 = reinterpret_cast<const uint4*>(img);
    for (int idx = tid; idx < tile_elems / 8; idx += 128) out4[idx] = in4[idx];
    __syncthreads();
  }
}

inline int prep_images(int kernel, const void* X, int64_t n, int64_t rs, int64_t cs, int d, const float* sigma_dev,
                       float sigma_scalar, int sigma_len, int64_t rows_pad, void* img_a, void* img_b, int* range_word,
                       cudaStream_t stream) {
  const int kp = (int)padded_k(d);
  const size_t smem = sizeof(float) * (size_t)(kTileRows * 33) + sizeof(__half) * (size_t)(kTileRows * kp);
  const float scale = (float)sqrt(scale_sq_for(kernel));
  const int blocks = (int)(rows_pad / kTileRows);
  prep_images_kernel<<<blocks, 128, smem, stream>>>(reinterpret_cast<const float*>(X), n, rs, cs, d, sigma_dev,
                                                    sigma_scalar, sigma_len, scale, kp, norm_pieces(d),
                                                    reinterpret_cast<__half*>(img_a),
                                                    reinterpret_cast<__half*>(img_b), range_word);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Main sweep kernel
// ---------------------------------------------------------------------------------------------
struct SweepArgs {
  const __half* img_a;  // [r_pad / 128] tile images (output side)
  const __half* img_b;  // [n_col_tiles] tile images (reduction side; with the vector folded in when `fold` is set)
  const float* vec;     // [t_chunks][s_pad][TT]  (unused with `fold`)
  float* raw;           // [n_chunks][r_pad][tp]
  int* status;          // device status block (word kStatusTimeout, word kStatusRange)
  const int* fold;      // folded sweeps: [kFoldNegTile] first tile of negative vector entries, [kFoldExp] power of
                        // two the stored vector magnitudes were divided by; null for ordinary sweeps
  int tp;
  int64_t r_pad;
  int64_t s_pad;
  int row_tiles;        // ceil(r / 512)
  int n_col_tiles;      // column tiles of the reduction side
  int tiles_per_chunk;
  // two-segment grid: CTAs [0, main_ctas) cover row tiles [0, main_tiles) with `tiles_per_chunk` column
  // tiles each; the remaining CTAs cover the remaining row tiles with `tiles_per_chunk_tail` each
  int main_tiles;
  int main_ctas;
  int tiles_per_chunk_tail;
  int ksteps;           // MMA K-steps (16 fp16 each) actually carrying data
};

// words of the fold block (inside the 256-byte status block, one block per sweep)
enum { kFoldNegTile = 0, kFoldExp = 1, kFoldPositives = 2, kFoldMaxBits = 3, kFoldWords = 8 };

template <int NSLAB>
struct TcCfg {
  static constexpr int KP = NSLAB * kSlabK;
  static constexpr int TILE_BYTES = kTileRows * KP * 2;       // one operand tile image
  static constexpr int A_BYTES = kRowBlocks * TILE_BYTES;     // 512 resident rows
  static constexpr int STAGES = NSLAB == 3 ? 4 : (NSLAB == 2 ? 6 : 12);
};

constexpr int kWideTT = 32;  // vector columns per pass of the many-column epilogue
constexpr int kFlushTiles = 32;  // column tiles (of 128) summed in one running fp32 sum before it is folded away
constexpr int kMaxWideTilesPerChunk = 512;  // many-column epilogue (single-level sums): longest chunk the planner forms

// Ring depths: with 32 vector columns per pass a vector tile is 16 KB, so two of them and one B stage fewer.
// A folded sweep has no vector ring at all.
template <int NSLAB, int TT, bool FOLD>
struct RingOf {
  static constexpr int S = TT == kWideTT ? (NSLAB == 3 ? 3 : (NSLAB == 2 ? 5 : 10)) : TcCfg<NSLAB>::STAGES;
  static constexpr int VS = FOLD ? 0 : (TT == kWideTT ? 2 : kVecStages);
  static constexpr int V_BYTES = VS * kColsPerTile * TT * 4;
};

template <int NSLAB, int TT, bool FOLD>
constexpr size_t tc_smem_bytes() {
  using C = TcCfg<NSLAB>;
  using R = RingOf<NSLAB, TT, FOLD>;
  return 1024 /* alignment slack */ + (size_t)C::A_BYTES + (size_t)R::S * C::TILE_BYTES + (size_t)R::V_BYTES +
         512 /* barriers + tmem pointer */ +
         (TT == kWideTT ? 0 : kRowsPerCta * 16) /* second-level sums, four floats per epilogue thread */;
}

// error codes written to the status word: role * 16 + which wait
enum { kErrProducer = 0x10, kErrMma = 0x20, kErrEpilogue = 0x30 };

// Which column pairs (0..15 within a 32-column piece) take the FMA-pipe exponential: a per-kernel-function
// count (measured optima on config-2 data; the Laplacian / Matern epilogues carry a MUFU square root and more
// FMA work per value; a folded sweep has no shared-memory vector reads competing with the MUFU instructions for
// the same issue queue, so its balance point lies elsewhere: measured ms per fdmmv at N = 1e7, M = 50,000 times
// the sampled SM clock in GHz, 3 -> 429, 4 -> 407, 5 -> 392, 6 -> 382, 7 -> 403, 8 -> 422), spread evenly over the
// piece so both pipes have work throughout.
template <int KT, bool FOLD = false>
__host__ __device__ constexpr int poly_pairs_of() {
#ifndef FLK_TC_POLY_PAIRS_LM
#define FLK_TC_POLY_PAIRS_LM 8
#endif
#ifndef FLK_TC_POLY_PAIRS_M25
#define FLK_TC_POLY_PAIRS_M25 5
#endif
#ifndef FLK_TC_POLY_PAIRS_FOLD
#define FLK_TC_POLY_PAIRS_FOLD 6
#endif
#ifndef FLK_TC_FOLD_SCALAR_SUM
#define FLK_TC_FOLD_SCALAR_SUM 0
#endif
  return KT == FLK_GAUSSIAN ? (FOLD ? FLK_TC_POLY_PAIRS_FOLD : kPolyPairs)
                            : (KT == FLK_MATERN25 ? FLK_TC_POLY_PAIRS_M25 : FLK_TC_POLY_PAIRS_LM);
}
template <int KT, bool FOLD = false>
__host__ __device__ constexpr bool poly_pair(int pr) {
  constexpr int np = poly_pairs_of<KT, FOLD>();
  return np > 0 && ((pr + 1) * np / 16 != pr * np / 16);
}

// Kernel function + contraction for 32 accumulator columns held in registers.  `vsm` points at the
// vector-tile entries of the first of those columns.  The running sums are two packed pairs:
//   TT = 1: four interleaved partial sums of the single output column (summed at the end);
//   TT = 2: osum[0] and osum[1] are two partial sums of the (t0, t1) pair;
//   TT = 4: osum[0] = (t0, t1), osum[1] = (t2, t3).
template <int KT, int TT, int C0 = 0>
__device__ __forceinline__ void epilogue_32(const uint32_t (&r)[32], const float* vsm, uint64_t (&osum)[2]) {
  static_assert(TT == 1 || TT == 2 || TT == 4, "TT must be 1, 2 or 4");
  if constexpr (C0 < 32) {
    float k0, k1, k2, k3;
    eval_pair<KT, poly_pair<KT>(C0 / 2)>(r[C0], r[C0 + 1], k0, k1);
    eval_pair<KT, poly_pair<KT>(C0 / 2 + 1)>(r[C0 + 2], r[C0 + 3], k2, k3);
    if constexpr (TT == 1) {
      const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(vsm + C0);  // (v0, v1), (v2, v3)
      osum[0] = fma2(pack2(k0, k1), v.x, osum[0]);
      osum[1] = fma2(pack2(k2, k3), v.y, osum[1]);
    } else if constexpr (TT == 2) {
      const ulonglong2 va = *reinterpret_cast<const ulonglong2*>(vsm + C0 * 2);      // columns C0, C0 + 1
      const ulonglong2 vb = *reinterpret_cast<const ulonglong2*>(vsm + C0 * 2 + 4);  // columns C0 + 2, C0 + 3
      osum[0] = fma2(pack2(k0, k0), va.x, osum[0]);
      osum[1] = fma2(pack2(k1, k1), va.y, osum[1]);
      osum[0] = fma2(pack2(k2, k2), vb.x, osum[0]);
      osum[1] = fma2(pack2(k3, k3), vb.y, osum[1]);
    } else {
      const float kv[4] = {k0, k1, k2, k3};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(vsm + (C0 + c) * 4);
        const uint64_t kk = pack2(kv[c], kv[c]);
        osum[0] = fma2(kk, v.x, osum[0]);
        osum[1] = fma2(kk, v.y, osum[1]);
      }
    }
    epilogue_32<KT, TT, C0 + 4>(r, vsm, osum);
  }
}

// Folded sweep (Gaussian, one vector column): log2 |vec_j| already sits in the exponent, so a kernel value times
// |vec_j| is ONE exponential and the contraction is a signed sum -- no vector tile, no shared-memory reads.  All
// 128 columns of a tile carry the same sign (the image builder sorts the reduction side by sign), `sgn2` is that
// sign as a packed pair (+1, +1) or (-1, -1).
template <int KT, int C0 = 0>
__device__ __forceinline__ void epilogue_32_fold(const uint32_t (&r)[32], uint64_t sgn2, uint64_t (&osum)[2]) {
  if constexpr (C0 < 32) {
    float k0, k1, k2, k3;
    eval_pair<KT, poly_pair<KT, true>(C0 / 2)>(r[C0], r[C0 + 1], k0, k1);
    eval_pair<KT, poly_pair<KT, true>(C0 / 2 + 1)>(r[C0 + 2], r[C0 + 3], k2, k3);
    osum[0] = fma2(pack2(k0, k1), sgn2, osum[0]);
    osum[1] = fma2(pack2(k2, k3), sgn2, osum[1]);
    epilogue_32_fold<KT, C0 + 4>(r, sgn2, osum);
  }
}

// The same with scalar adds into four running sums.  The packed f32x2 instructions execute on the heavy FMA pipe
// only (two cycles each); scalar FFMA can also go to the light pipe, at twice the issue slots.  Which form of the
// sum is faster depends on which of the two is scarcer: FLK_TC_FOLD_SCALAR_SUM selects it (measured, see the value).
template <int KT, int C0 = 0>
__device__ __forceinline__ void epilogue_32_fold_scalar(const uint32_t (&r)[32], float sgn, float (&fs)[4]) {
  if constexpr (C0 < 32) {
    float k0, k1, k2, k3;
    eval_pair<KT, poly_pair<KT, true>(C0 / 2)>(r[C0], r[C0 + 1], k0, k1);
    eval_pair<KT, poly_pair<KT, true>(C0 / 2 + 1)>(r[C0 + 2], r[C0 + 3], k2, k3);
    fs[0] = fmaf(k0, sgn, fs[0]);
    fs[1] = fmaf(k1, sgn, fs[1]);
    fs[2] = fmaf(k2, sgn, fs[2]);
    fs[3] = fmaf(k3, sgn, fs[3]);
    epilogue_32_fold_scalar<KT, C0 + 4>(r, sgn, fs);
  }
}

// Many-column epilogue: kernel function + contraction with 32 vector columns for 16 accumulator columns held in
// registers: per kernel value one exponential, then 16 packed multiply-adds against the 32 vector entries of that
// column (eight 16-byte broadcasts from shared memory).  PR0 = index of the first column pair within its 32-column
// piece (selects which pairs take the FMA-pipe exponential).
template <int KT, int PR0, int C0 = 0>
__device__ __forceinline__ void epilogue_wide16(const uint32_t (&r)[16], const float* vsm, uint64_t (&osum)[16]) {
  if constexpr (C0 < 16) {
    float k0, k1;
    // every exponential on the MUFU unit: this epilogue is bound by its multiply-adds, the FMA pipe has no room
    // for the polynomial form (and its constants would cost the registers the second register block needs)
    eval_pair<KT, false>(r[C0], r[C0 + 1], k0, k1);
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
    epilogue_wide16<KT, PR0, C0 + 2>(r, vsm, osum);
  }
}

// Shared-memory map of the sweep kernel, as 32-bit shared addresses computed from one base (generic 64-bit
// pointers to every ring and barrier would be live across all three warp roles and cost a dozen registers).
// barrier block: a_full | b_full[S] | b_empty[S] | v_full[VS] | v_empty[VS] | t_full[4] | t_empty[4] | tmem pointer |
// abort flag; then the second-level sums (one float4 per epilogue thread).
template <int NSLAB, int TT, bool FOLD>
struct SmemMap {
  using C = TcCfg<NSLAB>;
  using R = RingOf<NSLAB, TT, FOLD>;
  static constexpr uint32_t A = 0;
  static constexpr uint32_t B = C::A_BYTES;
  static constexpr uint32_t V = B + R::S * C::TILE_BYTES;
  static constexpr uint32_t BARS = V + R::V_BYTES;
  static constexpr uint32_t A_FULL = BARS;
  static constexpr uint32_t B_FULL = BARS + 8;
  static constexpr uint32_t B_EMPTY = B_FULL + 8 * R::S;
  static constexpr uint32_t V_FULL = B_EMPTY + 8 * R::S;
  static constexpr uint32_t V_EMPTY = V_FULL + 8 * R::VS;
  static constexpr uint32_t T_FULL = V_EMPTY + 8 * R::VS;
  static constexpr uint32_t T_EMPTY = T_FULL + 8 * kRowBlocks;
  static constexpr uint32_t TMEM_PTR = T_EMPTY + 8 * kRowBlocks;
  static constexpr uint32_t ABORT = TMEM_PTR + 4;
  static constexpr uint32_t FOLD_NPOS = ABORT + 4;  // folded sweep: positive tiles of this CTA's chunk
  static constexpr uint32_t SUMS = BARS + 512;
  static_assert(FOLD_NPOS + 4 <= SUMS, "barrier block overflows its 512 bytes");
};

__device__ __forceinline__ int ld_shared_i32_volatile(uint32_t addr) {
  int v;
  asm volatile("ld.volatile.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_i32_volatile(uint32_t addr, int v) {
  asm volatile("st.volatile.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Order in which a folded sweep visits the positive and the negative tiles of its chunk: evenly interleaved.
// Every role of the CTA steps through the same sequence: step j is a positive tile when the running count
// acc += npos passes `total` (npos of total steps are).
__device__ __forceinline__ bool fold_step_is_positive(int& acc, int npos, int total) {
  acc += npos;
  const bool pos = acc >= total;
  if (pos) acc -= total;
  return pos;
}

// Epilogue warp w: TMEM lane quarter q = w % 4 (hardware rule: a warp may only touch lanes
// 32 (w % 4) .. +31; warps with the same w % 4 also share an SM sub-partition, so each row block
// has one warp on every sub-partition), row block rb = w / 4.
template <int KT, int NSLAB, int TT, bool FOLD>
__global__ void __launch_bounds__(kThreads, 1) kmv_tc_kernel(const SweepArgs p) {
  static_assert(!FOLD || (KT == FLK_GAUSSIAN && TT == 1), "only the Gaussian single-column sweep folds its vector");
  using C = TcCfg<NSLAB>;
  using M = SmemMap<NSLAB, TT, FOLD>;
  using RB = RegBudget<KT, TT, FOLD>;
  constexpr int S = RingOf<NSLAB, TT, FOLD>::S;
  constexpr int VS = RingOf<NSLAB, TT, FOLD>::VS;
  extern __shared__ unsigned char tc_smem_raw[];
  // the swizzle atoms want a 512-byte aligned base; 1024 keeps every tile image on a round address
  const uint32_t raw_addr = smem_u32(tc_smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  const uint32_t sm = raw_addr + pad;  // shared address of the map's origin

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  int row_tile, chunk, tiles_per_chunk;
  if ((int)blockIdx.x < p.main_ctas) {
    row_tile = blockIdx.x % p.main_tiles;
    chunk = blockIdx.x / p.main_tiles;
    tiles_per_chunk = p.tiles_per_chunk;
  } else {
    const int b = blockIdx.x - p.main_ctas, tail_tiles = p.row_tiles - p.main_tiles;
    row_tile = p.main_tiles + b % tail_tiles;
    chunk = b / tail_tiles;
    tiles_per_chunk = p.tiles_per_chunk_tail;
  }
  const int tchunk = blockIdx.y;
  // Tiles of this CTA's chunk.  Ordinary sweep: tile_begin .. tile_begin + ntiles.  Folded sweep: the image holds
  // the tiles of non-negative vector entries first and those of negative entries from tile [kFoldNegTile] on; a
  // chunk takes an equal share of BOTH ranges and walks them interleaved (fold_step_is_positive), so that the running sums of
  // a thread stay balanced -- summing one sign after the other let them grow to the size of the whole one-sided
  // sum and cost up to 1e-4 of relative accuracy on strongly cancelling sums over 1e5 and more rows.
  int tile_begin = chunk * tiles_per_chunk;
  int ntiles = min(tile_begin + tiles_per_chunk, p.n_col_tiles) - tile_begin;
  int fold_neg0 = 0, fold_npos = 0;  // first negative tile of this chunk, positive tiles in it (tile_begin = its first positive tile)
  if constexpr (FOLD) {
    const int n_chunks = (p.n_col_tiles + tiles_per_chunk - 1) / tiles_per_chunk;
    const int pos_tiles = min(__ldg(p.fold + kFoldNegTile), p.n_col_tiles), neg_tiles = p.n_col_tiles - pos_tiles;
    const int pos_share = (pos_tiles + n_chunks - 1) / n_chunks, neg_share = (neg_tiles + n_chunks - 1) / n_chunks;
    tile_begin = min(chunk * pos_share, pos_tiles);
    fold_npos = min(tile_begin + pos_share, pos_tiles) - tile_begin;
    fold_neg0 = pos_tiles + min(chunk * neg_share, neg_tiles);
    ntiles = fold_npos + min(fold_neg0 + neg_share, p.n_col_tiles) - fold_neg0;
  }

  // Do not start when a CTA of this launch already gave up (keeps a failed launch short) or when
  // the image builder found rows fp16 cannot carry (the SIMT kernels take over).
  __shared__ int skip_launch;
  if (tid == 0) {
    const volatile int* st = reinterpret_cast<const volatile int*>(p.status);
    skip_launch = (st[kStatusTimeout] != 0 || range_raised(p.status + kStatusRange)) ? 1 : 0;
  }
  __syncthreads();
  if (skip_launch) return;

  if (tid == 0) {
    mbar_init(sm + M::A_FULL, 1);
#pragma unroll 1
    for (int s = 0; s < S; ++s) {
      mbar_init(sm + M::B_FULL + 8 * s, 1);
      mbar_init(sm + M::B_EMPTY + 8 * s, kRowBlocks);  // one MMA commit per row-block issuer
    }
#pragma unroll 1
    for (int s = 0; s < VS; ++s) {
      mbar_init(sm + M::V_FULL + 8 * s, 1);
      mbar_init(sm + M::V_EMPTY + 8 * s, kEpilogueWarps);  // one arrive per epilogue warp
    }
#pragma unroll 1
    for (int i = 0; i < kRowBlocks; ++i) {
      mbar_init(sm + M::T_FULL + 8 * i, 1);
      mbar_init(sm + M::T_EMPTY + 8 * i, 4);  // the four warps of that row block
    }
    st_shared_i32_volatile(sm + M::ABORT, 0);
    st_shared_i32_volatile(sm + M::FOLD_NPOS, fold_npos);
    fence_barrier_init();
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(sm + M::TMEM_PTR, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = (uint32_t)ld_shared_i32_volatile(sm + M::TMEM_PTR);

  if (warp > kProducerWarp) {
    reg_release<RB::kProducer>();  // filler warps of the producer's warpgroup
  } else if (warp == kProducerWarp) {
    // ------------------------------ bulk-copy producer ------------------------------
    // The whole warp walks the loop (converged); one elected lane issues the copies.
    reg_release<RB::kProducer>();
    if (elect_one()) {
      const __half* a_src = p.img_a + (int64_t)row_tile * kRowBlocks * (kTileRows * C::KP);
      mbar_expect_tx(sm + M::A_FULL, C::A_BYTES);
      for (int rb = 0; rb < kRowBlocks; ++rb)
        bulk_copy_g2s(sm + M::A + rb * C::TILE_BYTES, a_src + rb * (kTileRows * C::KP), C::TILE_BYTES, sm + M::A_FULL);
    }
    __syncwarp();
    const __half* b_src = p.img_b + (int64_t)tile_begin * (kTileRows * C::KP);
    const float* v_src = FOLD ? nullptr : p.vec + ((int64_t)tchunk * p.s_pad + (int64_t)tile_begin * kColsPerTile) * TT;
    int walk = 0, next_pos = 0, next_neg = fold_neg0 - tile_begin;  // tile offsets from tile_begin
    for (int j = 0; j < ntiles; ++j) {
      const int stage = j % S;
      if (ld_shared_i32_volatile(sm + M::ABORT)) break;
      int tile = j;  // offset of step j's tile from tile_begin
      if constexpr (FOLD) tile = fold_step_is_positive(walk, fold_npos, ntiles) ? next_pos++ : next_neg++;
      bool ok = mbar_wait(sm + M::B_EMPTY + 8 * stage, ((j / S) & 1) ^ 1);
      if constexpr (!FOLD) ok = ok && mbar_wait(sm + M::V_EMPTY + 8 * (j % VS), ((j / VS) & 1) ^ 1);
      if (!ok) {
        if (lane == 0) atomicExch(p.status + kStatusTimeout, kErrProducer | 1);
        st_shared_i32_volatile(sm + M::ABORT, 1);
        break;
      }
      if (elect_one()) {
        const uint32_t bar = sm + M::B_FULL + 8 * stage;
        mbar_expect_tx(bar, C::TILE_BYTES);
        bulk_copy_g2s(sm + M::B + stage * C::TILE_BYTES, b_src + (int64_t)tile * (kTileRows * C::KP), C::TILE_BYTES, bar);
        if constexpr (!FOLD) {
          const int vstage = j % VS;
          const uint32_t vbar = sm + M::V_FULL + 8 * vstage;
          mbar_expect_tx(vbar, kColsPerTile * TT * 4);
          bulk_copy_g2s(sm + M::V + vstage * kColsPerTile * TT * 4, v_src + (int64_t)j * kColsPerTile * TT,
                        kColsPerTile * TT * 4, vbar);
        }
      }
      __syncwarp();
    }
  } else if (warp >= kMmaWarp0) {
    // ------------------------------ MMA issuers ------------------------------
    // One issuer warp per row block, each on its own SM sub-partition: a queued tcgen05.mma holds
    // up the other warps of its sub-partition, so the issue work is spread evenly over the four.
    // All lanes wait on the barriers together; one elected lane issues the MMAs and commits.
    reg_release<RB::kMma>();
    const int rb = warp - kMmaWarp0;
    bool ok = mbar_wait(sm + M::A_FULL, 0);
    if (!ok) {
      if (lane == 0) atomicExch(p.status + kStatusTimeout, kErrMma | 1);
      st_shared_i32_volatile(sm + M::ABORT, 1);
    }
    const uint64_t a_desc0 = make_smem_desc(sm + M::A + rb * C::TILE_BYTES);
    const uint32_t d_tmem = tmem_base + (uint32_t)(rb * kColsPerTile);
    for (int j = 0; ok && j < ntiles; ++j) {
      const int stage = j % S;
      if (ld_shared_i32_volatile(sm + M::ABORT)) break;
      // B tile j has landed, and this row block's accumulator is free (its warps pulled tile j-1
      // into registers)
      if (!mbar_wait(sm + M::B_FULL + 8 * stage, (j / S) & 1) || !mbar_wait(sm + M::T_EMPTY + 8 * rb, (j & 1) ^ 1)) {
        if (lane == 0) atomicExch(p.status + kStatusTimeout, kErrMma | 2);
        st_shared_i32_volatile(sm + M::ABORT, 1);
        break;
      }
      tc_fence_after();
      if (elect_one()) {
        const uint64_t b_desc0 = make_smem_desc(sm + M::B + stage * C::TILE_BYTES);
        for (int ks = 0; ks < p.ksteps; ++ks) {
          // 32 bytes (16 fp16) per K-step, two K-steps per 64-byte swizzle row, 8 KiB per slab
          const uint64_t koff = (uint64_t)((ks >> 1) * ((kTileRows * 64) >> 4) + (ks & 1) * 2);
          mma_f16(d_tmem, a_desc0 + koff, b_desc0 + koff, kInstrDesc, ks > 0 ? 1u : 0u);
        }
        mma_commit(sm + M::T_FULL + 8 * rb);
        mma_commit(sm + M::B_EMPTY + 8 * stage);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    reg_claim<RB::kEpilogue>();
    const int q = warp & 3;    // TMEM lane quarter this warp may access
    const int rb = warp >> 2;  // row block
    constexpr int NSUM = TT == kWideTT ? 16 : 2;  // packed pairs of running sums (see epilogue_32 / epilogue_wide16)
    // Two-level summation (TT <= 4): `osum` collects kFlushTiles column tiles, then is folded into a float4 of
    // this thread in shared memory.  A chunk may span millions of columns; one running fp32 sum over all of them
    // loses about half a digit more than the reference's blocked GEMV does, enough to unsettle an fp32 conjugate
    // gradient at lambda = 1e-7.  The many-column form keeps one level: the planner bounds its chunk length
    // instead (kMaxWideTilesPerChunk).
    uint64_t osum[NSUM];
#pragma unroll
    for (int i = 0; i < NSUM; ++i) osum[i] = 0ull;
    const uint32_t tot = sm + M::SUMS + (uint32_t)(warp * 32 + lane) * 16u;
    if constexpr (TT != kWideTT) st_shared_f4(tot, 0.f, 0.f, 0.f, 0.f);
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(rb * kColsPerTile);
    int walk = 0;  // folded sweep: the count of fold_step_is_positive; the chunk's positive tiles are read from
                   // shared memory at every step (one register less in the loop that has none to spare)
    bool epi_ok = true;

    // outer loop = blocks of kFlushTiles tiles, with the fold between the blocks and outside the hot inner loop
    // (the many-column epilogue sums in one level: a single pass of the outer loop)
    constexpr int kFlush = TT == kWideTT ? (1 << 30) : kFlushTiles;
    for (int j0 = 0; j0 < ntiles && epi_ok; j0 += kFlush) {
      if constexpr (TT != kWideTT) {
        if (j0 > 0) {
          float t0, t1, t2, t3, a0, a1, b0, b1;
          ld_shared_f4(tot, t0, t1, t2, t3);
          unpack2(osum[0], a0, a1);
          unpack2(osum[1], b0, b1);
          st_shared_f4(tot, t0 + a0, t1 + a1, t2 + b0, t3 + b1);
          osum[0] = osum[1] = 0ull;
        }
      }
      const int j1 = TT == kWideTT ? ntiles : min(j0 + kFlush, ntiles);
      for (int j = j0; j < j1; ++j) {
        if (ld_shared_i32_volatile(sm + M::ABORT)) { epi_ok = false; break; }
        bool ok = true;
        if constexpr (!FOLD) ok = mbar_wait(sm + M::V_FULL + 8 * (j % VS), (j / VS) & 1);
        if (!ok || !mbar_wait(sm + M::T_FULL + 8 * rb, j & 1)) {
          atomicExch(p.status + kStatusTimeout, kErrEpilogue | 1);
          st_shared_i32_volatile(sm + M::ABORT, 1);
          epi_ok = false;
          break;
        }
        tc_fence_after();
        if constexpr (FOLD) {
#if FLK_TC_FOLD_SCALAR_SUM
          const float sgn = fold_step_is_positive(walk, ld_shared_i32_volatile(sm + M::FOLD_NPOS), ntiles) ? 1.0f : -1.0f;
          float fs[4];
          unpack2(osum[0], fs[0], fs[1]);
          unpack2(osum[1], fs[2], fs[3]);
          uint32_t ra[32], rc[32];
          tmem_ld32(taddr, ra);
          tmem_ld_wait_on(ra);
          tmem_ld32(taddr + 32, rc, ra);
          epilogue_32_fold_scalar<KT>(ra, sgn, fs);
          tmem_ld_wait_on(rc, fs);
          tmem_ld32(taddr + 64, ra, rc);
          epilogue_32_fold_scalar<KT>(rc, sgn, fs);
          tmem_ld_wait_on(ra, fs);
          tmem_ld32(taddr + 96, rc, ra);
          tmem_ld_wait_on(rc);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(sm + M::T_EMPTY + 8 * rb);
          epilogue_32_fold_scalar<KT>(ra, sgn, fs);
          epilogue_32_fold_scalar<KT>(rc, sgn, fs);
          osum[0] = pack2(fs[0], fs[1]);
          osum[1] = pack2(fs[2], fs[3]);
#else
          const uint64_t sgn2 = fold_step_is_positive(walk, ld_shared_i32_volatile(sm + M::FOLD_NPOS), ntiles)
                                    ? 0x3F8000003F800000ull
                                    : 0xBF800000BF800000ull;
          uint32_t ra[32], rc[32];
          tmem_ld32(taddr, ra);
          tmem_ld_wait_on(ra);
          tmem_ld32(taddr + 32, rc, ra);
          epilogue_32_fold<KT>(ra, sgn2, osum);
          tmem_ld_wait_on(rc, osum);
          tmem_ld32(taddr + 64, ra, rc);
          epilogue_32_fold<KT>(rc, sgn2, osum);
          tmem_ld_wait_on(ra, osum);
          tmem_ld32(taddr + 96, rc, ra);
          tmem_ld_wait_on(rc);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(sm + M::T_EMPTY + 8 * rb);
          epilogue_32_fold<KT>(ra, sgn2, osum);
          epilogue_32_fold<KT>(rc, sgn2, osum);
#endif
        } else {
          // generic pointer rebuilt from the 32-bit shared address: no 64-bit base stays live across the loop
          const float* vsm = reinterpret_cast<const float*>(
              __cvta_shared_to_generic(sm + M::V + (uint32_t)((j % VS) * kColsPerTile * TT * 4)));
          if constexpr (TT == kWideTT) {
            // eight 16-column pieces; the accumulator goes back to its issuer once the last one is in registers
            // (the K-loop kernel keeps two register blocks in flight here; this kernel has no registers left for
            // the second one without spilling)
            uint32_t rw[16];
#pragma unroll
            for (int pc = 0; pc < 8; ++pc) {
              tmem_ld16(taddr + pc * 16, rw);
              tmem_ld_wait_on(rw);
              if (pc == 7) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sm + M::T_EMPTY + 8 * rb);
              }
              if (pc & 1)
                epilogue_wide16<KT, 8>(rw, vsm + pc * 16 * TT, osum);
              else
                epilogue_wide16<KT, 0>(rw, vsm + pc * 16 * TT, osum);
            }
          } else {
            uint32_t ra[32], rc[32];
            // pieces 0 and 2 travel in `ra`, 1 and 3 in `rc`; the next piece loads while this one is evaluated
            tmem_ld32(taddr, ra);
            tmem_ld_wait_on(ra);
            tmem_ld32(taddr + 32, rc, ra);
            epilogue_32<KT, TT>(ra, vsm, osum);
            tmem_ld_wait_on(rc, osum);
            tmem_ld32(taddr + 64, ra, rc);
            epilogue_32<KT, TT>(rc, vsm + 32 * TT, osum);
            tmem_ld_wait_on(ra, osum);
            tmem_ld32(taddr + 96, rc, ra);
            tmem_ld_wait_on(rc);
            // The second half of the accumulator is in registers: hand the accumulator back now, so the
            // MMA of the next tile (and the barrier round trips either side of it) runs under the
            // evaluation of these two pieces.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sm + M::T_EMPTY + 8 * rb);
            epilogue_32<KT, TT>(ra, vsm + 64 * TT, osum);
            epilogue_32<KT, TT>(rc, vsm + 96 * TT, osum);
          }
          // the vector tile goes back to the producer, whose bulk copy will overwrite it
          const uint32_t zero = smem_reads_done(osum[0] ^ osum[NSUM - 1]);
          __syncwarp();
          if (lane == 0) mbar_arrive(sm + M::V_EMPTY + 8 * (j % VS) + zero);
        }
      }
    }
    if (epi_ok) {
      if constexpr (TT != kWideTT) {
        float t0, t1, t2, t3;
        ld_shared_f4(tot, t0, t1, t2, t3);
        osum[0] = add2(pack2(t0, t1), osum[0]);
        osum[1] = add2(pack2(t2, t3), osum[1]);
      }
      const int64_t row = (int64_t)row_tile * kRowsPerCta + rb * kTileRows + q * 32 + lane;
      float* dst = p.raw + ((int64_t)chunk * p.r_pad + row) * p.tp + tchunk * TT;
      if constexpr (TT == kWideTT) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float lo, hi;
          unpack2(osum[i], lo, hi);
          dst[2 * i] = lo;
          dst[2 * i + 1] = hi;
        }
      } else {
        float a0, a1, b0, b1;
        unpack2(osum[0], a0, a1);
        unpack2(osum[1], b0, b1);
        if constexpr (TT == 1) {
          float sum = (a0 + a1) + (b0 + b1);
          // folded: the vector magnitudes were stored divided by 2^e; the factor goes back on here (exact)
          if constexpr (FOLD) sum *= __int_as_float((__ldg(p.fold + kFoldExp) + 127) << 23);
          dst[0] = sum;
        } else if constexpr (TT == 2) {
          dst[0] = a0 + b0;
          dst[1] = a1 + b1;
        } else {
          dst[0] = a0;
          dst[1] = a1;
          dst[2] = b0;
          dst[3] = b1;
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  const bool aborted = ld_shared_i32_volatile(sm + M::ABORT) != 0;
  if (aborted && warp == kProducerWarp && lane == 0) {
    // give this CTA's own bulk copies a bounded chance to land before the shared memory is released
    // (the B and vector "full" barriers lie next to each other in the map: one rolled loop over all of them)
    mbar_wait(sm + M::A_FULL, 0);
#pragma unroll 1
    for (uint32_t bar = sm + M::B_FULL; bar < sm + M::B_FULL + 8 * S; bar += 8) {
      if (!mbar_try_wait(bar, 0)) mbar_try_wait(bar, 1);
    }
#pragma unroll 1
    for (uint32_t bar = sm + M::V_FULL; bar < sm + M::V_FULL + 8 * VS; bar += 8) {
      if (!mbar_try_wait(bar, 0)) mbar_try_wait(bar, 1);
    }
  }
  __syncthreads();
  if (warp == kMmaWarp0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int KT, int NSLAB, int TT, bool FOLD>
int launch_sweep_inst(const SweepArgs& args, int grid_x, int t_chunks, cudaStream_t stream) {
  constexpr size_t smem = tc_smem_bytes<NSLAB, TT, FOLD>();
  static_assert(smem > 116 * 1024, "one CTA per SM is assumed (each CTA takes all 512 TMEM columns)");
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  static bool configured[16] = {false};
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    FLK_CUDA_TRY(cudaFuncSetAttribute(kmv_tc_kernel<KT, NSLAB, TT, FOLD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid((unsigned)grid_x, (unsigned)t_chunks, 1);
  kmv_tc_kernel<KT, NSLAB, TT, FOLD><<<grid, kThreads, smem, stream>>>(args);
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <int KT, int NSLAB>
int launch_sweep_tt(const SweepArgs& args, int tt, int grid_x, int t_chunks, cudaStream_t stream) {
  if constexpr (KT == FLK_GAUSSIAN) {
    if (args.fold != nullptr) {
      if (tt != 1) return fail(FLK_ERR_BAD_ARG, "internal: a folded sweep has one vector column, not %d", tt);
      return launch_sweep_inst<KT, NSLAB, 1, true>(args, grid_x, t_chunks, stream);
    }
  } else if (args.fold != nullptr) {
    return fail(FLK_ERR_BAD_ARG, "internal: only the Gaussian sweep folds its vector");
  }
  switch (tt) {
    case 1: return launch_sweep_inst<KT, NSLAB, 1, false>(args, grid_x, t_chunks, stream);
    case 2: return launch_sweep_inst<KT, NSLAB, 2, false>(args, grid_x, t_chunks, stream);
    case 4: return launch_sweep_inst<KT, NSLAB, 4, false>(args, grid_x, t_chunks, stream);
    case kWideTT: return launch_sweep_inst<KT, NSLAB, kWideTT, false>(args, grid_x, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported TT=%d", tt);
}

template <int KT>
int launch_sweep_kt(int nslab, const SweepArgs& args, int tt, int grid_x, int t_chunks, cudaStream_t stream) {
  switch (nslab) {
    case 1: return launch_sweep_tt<KT, 1>(args, tt, grid_x, t_chunks, stream);
    case 2: return launch_sweep_tt<KT, 2>(args, tt, grid_x, t_chunks, stream);
    case 3: return launch_sweep_tt<KT, 3>(args, tt, grid_x, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "internal: unsupported slab count %d", nslab);
}

inline int launch_sweep(int kernel, int d, SweepArgs args, int tt, int grid_x, int t_chunks, cudaStream_t stream) {
  args.ksteps = k_steps(d);
  const int nslab = n_slabs(d);
  switch (kernel) {
    case FLK_GAUSSIAN: return launch_sweep_kt<FLK_GAUSSIAN>(nslab, args, tt, grid_x, t_chunks, stream);
    case FLK_LAPLACIAN: return launch_sweep_kt<FLK_LAPLACIAN>(nslab, args, tt, grid_x, t_chunks, stream);
    case FLK_MATERN15: return launch_sweep_kt<FLK_MATERN15>(nslab, args, tt, grid_x, t_chunks, stream);
    case FLK_MATERN25: return launch_sweep_kt<FLK_MATERN25>(nslab, args, tt, grid_x, t_chunks, stream);
  }
  return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
}

}  // namespace tc
}  // namespace flk
