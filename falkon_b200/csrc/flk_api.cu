// extern "C" entry points of libfalkon_b200: argument checks, workspace planning, dispatch.
#include <algorithm>
#include <atomic>
#include <vector>

#include "flk_common.cuh"
#include "flk_dmma.cuh"
#include "flk_fmm.cuh"
#include "flk_fold.cuh"
#include "flk_grad.cuh"
#include "flk_prep.cuh"
#include "flk_simt.cuh"
#include "flk_tc.cuh"
#include "flk_tck.cuh"
#include "flk_wide.cuh"

namespace flk {

static std::atomic<int64_t> g_launches{0};
static inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

constexpr int kNumSMs = 148;  // B200

// Optional per-sweep timing (CUDA events recorded on the caller's stream around the dominant
// kernel of each sweep).  Off by default; bench.py turns it on to measure the kernel live.
struct SweepTimer {
  bool enabled = false;
  int device = -1;
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};  // sweep 1 start/stop, sweep 2 start/stop
  bool valid[2] = {false, false};
};
static SweepTimer g_timer;

static int timer_mark(int slot, cudaStream_t stream) {
  if (!g_timer.enabled) return FLK_OK;
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (g_timer.device != dev || g_timer.ev[0] == nullptr) {
    for (int i = 0; i < 4; ++i) {
      if (g_timer.ev[i] != nullptr) cudaEventDestroy(g_timer.ev[i]);
      FLK_CUDA_TRY(cudaEventCreate(&g_timer.ev[i]));
    }
    g_timer.device = dev;
    g_timer.valid[0] = g_timer.valid[1] = false;
  }
  FLK_CUDA_TRY(cudaEventRecord(g_timer.ev[slot], stream));
  if (slot & 1) g_timer.valid[slot >> 1] = true;
  return FLK_OK;
}

// 16 independent ex2.approx chains per thread, nothing else: the MUFU rate of the device.
__global__ void __launch_bounds__(512) mufu_probe_kernel(int iters, float* sink) {
  float x[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = -1.0f - 0.001f * (float)(threadIdx.x + i);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = ex2_approx(x[i]) - 1.5f;
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) s += x[i];
  if (s == 123.456f) *sink = s;  // keeps the loop alive; never true in practice
}

// Clears the 64-word status block at the start of a call, except the range words of operands whose prepared form
// the caller keeps from the previous call.
__global__ void reset_status_kernel(int* status, int keep_x1, int keep_x2) {
  const int i = threadIdx.x;
  if (i >= 64) return;
  if ((keep_x1 && i == tc::kStatusRangeX1) || (keep_x2 && i == tc::kStatusRangeX2)) return;
  status[i] = 0;
}

struct Mat {
  const void* ptr;
  int64_t rows, cols, rs, cs;
};

static int check_mat(const char* name, const Mat& m, bool nullable) {
  if (m.ptr == nullptr) {
    if (nullable) return FLK_OK;
    return fail(FLK_ERR_BAD_ARG, "%s: null pointer", name);
  }
  if (m.rows < 0 || m.cols < 0) return fail(FLK_ERR_BAD_ARG, "%s: negative size", name);
  if (m.rs != 1 && m.cs != 1 && m.rows > 1 && m.cols > 1)
    return fail(FLK_ERR_LAYOUT, "%s: must be memory contiguous along one dimension (strides %lld, %lld)",
                name, (long long)m.rs, (long long)m.cs);
  if (m.rs < 0 || m.cs < 0) return fail(FLK_ERR_LAYOUT, "%s: negative stride", name);
  if (m.rows > 1 && m.cols > 1) {
    if (m.cs == 1 && m.rs < m.cols) return fail(FLK_ERR_LAYOUT, "%s: row stride smaller than width", name);
    if (m.rs == 1 && m.cs != 1 && m.cs < m.rows)
      return fail(FLK_ERR_LAYOUT, "%s: column stride smaller than height", name);
  }
  return FLK_OK;
}

// ---------------------------------------------------------------------------------------------
// One "sweep" = raw[chunks][r_pad][tp] = sum_j k(A_i, B_j) vec[j][:]  over the whole reduction side.
// ---------------------------------------------------------------------------------------------
struct SweepPlan {
  bool tc;            // tensor-core kernel?
  bool kloop;         // ... its K-loop variant for many features (flk_tck.cuh: 256-row CTAs, operands streamed)
  bool fold;          // ... with the vector folded into the reduction-side image (flk_fold.cuh; one tile more)
  int64_t r, s;       // live rows on the output / reduction side
  int64_t r_pad, s_pad;
  int tt, tp, t_chunks;
  int br, bc;         // CTA tile (rows x columns)
  int row_tiles, n_col_tiles, tiles_per_chunk, n_chunks;
  // Two-segment grids (tensor-core kernel): the first `main_tiles` row tiles use (n_chunks, tiles_per_chunk),
  // the remaining ones -- the rows that would otherwise form a last, partly filled wave of CTAs -- are cut into
  // (n_chunks_tail, tiles_per_chunk_tail) shorter pieces.  Uniform plans have main_tiles == row_tiles.
  int main_tiles, n_chunks_tail, tiles_per_chunk_tail;
  int max_chunks() const { return n_chunks > n_chunks_tail ? n_chunks : n_chunks_tail; }
  int64_t grid_x() const {
    return (int64_t)main_tiles * n_chunks + (int64_t)(row_tiles - main_tiles) * n_chunks_tail;
  }
  int64_t raw_elems() const { return (int64_t)max_chunks() * r_pad * tp; }
};

// Vector columns per pass: 1, 2 or 4 for the epilogues that keep two packed pairs of running sums, or 32
// (`use_wide`; one kernel evaluation serves all of them, but the contraction then costs 32 columns of work
// whatever t is).
static void choose_tt(int64_t t, bool use_wide, int* tt, int* tp) {
  if (t <= 1) *tt = 1;
  else if (t == 2) *tt = 2;
  else if (t <= 4 || !use_wide) *tt = 4;
  else *tt = kWideT;
  *tp = (int)round_up(std::max<int64_t>(t, 1), *tt);
}

// Is one pass over groups of 32 columns cheaper than passes over groups of 4?  Relative costs per kernel value
// and pass, from measurements on B200 (N = 1e5, M = 2e4; d = 48 / 128 / 440: 1.6 / 2.5 / 7.6 ms per pass of 4,
// 8.3 / 8.6 / 11.1 ms per pass of 32): tensor-core paths pay max(epilogue, exponent GEMM ~ 0.08 + 0.0033 d) for 4
// columns and about 1.6 + 0.0014 d for 32 (the 32-column epilogue is bound by its multiply-adds and shared-memory
// reads); the SIMT / DMMA paths pay d + 4 + E against d + 32 + E multiply-adds (E = the exponential: about 4 in
// fp32, 40 in software fp64).
static bool wide_pays_off(bool tc, int dtype, int kernel, int64_t d, int64_t t) {
  if (t <= 4) return false;
  const double passes4 = (double)ceil_div(t, 4), passes32 = (double)ceil_div(t, kWideT);
  if (tc) {
    const double epi4 = kernel == FLK_GAUSSIAN ? 0.33 : 0.6;  // the other kernel functions carry a square root
    const double cost4 = std::max(epi4, 0.08 + 0.0033 * (double)d), cost32 = 1.6 + 0.0014 * (double)d;
    return passes32 * cost32 < passes4 * cost4;
  }
  const double e = dtype == FLK_F64 ? 40.0 : 4.0;
  return passes32 * ((double)d + 32.0 + e) < passes4 * ((double)d + 4.0 + e);
}

// `allow_wide`: the plan may group 32 vector columns per pass.  The SIMT alternative of a tensor-core plan shares
// its vector buffers and therefore must be planned with the same column grouping.
// `kloop_d`: feature count when the K-loop tensor-core kernel runs the sweep (its tile shape depends on it), else 0.
static SweepPlan plan_sweep(bool tc, int dtype, int64_t r, int64_t s, int64_t t, bool allow_wide = false,
                            int64_t kloop_d = 0, bool fold = false) {
  const bool kloop = kloop_d > 0;
  SweepPlan p;
  p.tc = tc;
  p.kloop = tc && kloop;
  p.fold = tc && fold;
  p.r = r;
  p.s = s;
  p.r_pad = round_up(std::max<int64_t>(r, 1), kRowPad);
  p.s_pad = round_up(std::max<int64_t>(s, 1), kRowPad);
  choose_tt(t, allow_wide, &p.tt, &p.tp);
  p.t_chunks = p.tp / p.tt;
  if (tc) {
    const int mode = kloop ? tck::tile_mode(kloop_d, p.tt) : 0;
    p.br = kloop ? tck::rows_per_cta(mode) : tc::kRowsPerCta;
    p.bc = kloop ? tck::cols_per_step(mode) : tc::kColsPerTile;
  } else {
    p.br = 128;
    p.bc = (dtype == FLK_F32) ? 128 : 64;
  }
  p.row_tiles = (int)ceil_div(std::max<int64_t>(r, 1), p.br);
  p.n_col_tiles = p.fold ? tc::fold_tiles(s) : (int)ceil_div(std::max<int64_t>(s, 1), p.bc);
  const int64_t resident = tc ? 1 : (p.tt == 1 ? 2 : 1);  // CTAs per SM (launch bounds of kmv_simt_kernel)
  const int64_t slots = kNumSMs * resident;
  if (!tc) {
    // SIMT kernels (small CTAs): split the reduction side into chunks so that the grid fills whole waves
    // of the SMs: among the chunk counts that give at least two waves (when the problem allows), take
    // the one with the best wave efficiency, preferring fewer chunks (less partial-result traffic).
    const int64_t ctas_rows = (int64_t)p.row_tiles * p.t_chunks;
    const int64_t min_tiles = 4;  // keep the row tile's staging cost amortised
    const int64_t max_chunks = std::max<int64_t>(1, std::min<int64_t>(p.n_col_tiles / min_tiles, 4096));
    int64_t best_chunks = 1;
    double best_score = -1.0;
    for (int64_t want = 1; want <= max_chunks; ++want) {
      const int64_t tpc = ceil_div(p.n_col_tiles, want);
      const int64_t chunks = ceil_div(p.n_col_tiles, tpc);
      const int64_t ctas = ctas_rows * chunks;
      const int64_t waves = ceil_div(ctas, slots);
      double eff = (double)ctas / (double)(waves * slots);
      if (ctas < 2 * slots) eff *= 0.5 * (double)ctas / (double)(2 * slots);  // too few CTAs to balance
      if (eff > best_score + 0.01) {
        best_score = eff;
        best_chunks = chunks;
      }
      if (ctas >= 8 * slots) break;
    }
    p.tiles_per_chunk = (int)ceil_div(p.n_col_tiles, best_chunks);
    p.n_chunks = (int)ceil_div(p.n_col_tiles, p.tiles_per_chunk);
    p.main_tiles = p.row_tiles;
    p.n_chunks_tail = p.n_chunks;
    p.tiles_per_chunk_tail = p.tiles_per_chunk;
    return p;
  }
  // Tensor-core kernel: one 512-row CTA per SM at a time, each costing (column tiles + a fixed start-up of
  // about four tiles: operand load, TMEM allocation, drain).  CTAs of equal length run in waves of 148, so
  // the time of a plan is waves x length; a plan may cut the rows of the last, partly filled wave into
  // shorter pieces (second segment).  All candidates are scored with that model; ties go to fewer chunks.
  const double start_up = p.kloop ? 1.0 : 4.0;  // the K-loop variant has no resident operand to load first
  const int64_t R = p.row_tiles, Ct = p.n_col_tiles, Y = p.t_chunks;
  const int64_t c_cap = std::max<int64_t>(1, std::min<int64_t>(Ct, 512));
  double best = 1e300;
  auto consider = [&](int64_t main_tiles, int64_t cm, int64_t ct) {
    const int64_t tpc_m = ceil_div(Ct, cm), tpc_t = ceil_div(Ct, ct);
    const int64_t ch_m = ceil_div(Ct, tpc_m), ch_t = ceil_div(Ct, tpc_t);
    const int64_t ctas_m = main_tiles * ch_m * Y, ctas_t = (R - main_tiles) * ch_t * Y;
    double cost = (double)ceil_div(ctas_m, slots) * ((double)tpc_m + start_up);
    if (ctas_t > 0) cost += (double)ceil_div(ctas_t, slots) * ((double)tpc_t + start_up);
    cost += 1e-3 * (double)std::max(ch_m, ch_t);
    if (cost < best) {
      best = cost;
      p.main_tiles = (int)main_tiles;
      p.n_chunks = (int)ch_m;
      p.tiles_per_chunk = (int)tpc_m;
      p.n_chunks_tail = (int)(ctas_t > 0 ? ch_t : ch_m);
      p.tiles_per_chunk_tail = (int)(ctas_t > 0 ? tpc_t : tpc_m);
    }
  };
  // the many-column epilogue sums a whole chunk in one running fp32 sum per thread: bound its length
  const int64_t c_min = p.tt == tc::kWideTT ? ceil_div(Ct, (int64_t)tc::kMaxWideTilesPerChunk) : 1;
  for (int64_t c = c_min; c <= std::max(c_cap, c_min); ++c) consider(R, c, c);
  if (Y == 1 && !p.kloop) {
    for (int64_t cm : {1, 2, 4}) {  // divisors of 148, so that the first segment ends on a wave boundary
      if (cm < c_min || cm > c_cap || ceil_div(Ct, ceil_div(Ct, cm)) != cm) continue;
      const int64_t main_tiles = (R * cm / slots) * (slots / cm);
      if (main_tiles <= 0 || main_tiles >= R) continue;
      for (int64_t ct = cm + 1; ct <= std::min<int64_t>(c_cap, 64); ++ct) consider(main_tiles, cm, ct);
    }
  }
  return p;
}

static bool tc_eligible(int dtype, int kernel, int64_t d, int64_t t, int flags) {
  (void)kernel;
  (void)t;
  if (flags & FLK_FLAG_FORCE_SIMT) return false;
  if (dtype != FLK_F32) return false;
  return tc::supports_d(d) || tck::supports_d(d);
}

// Bump allocator over the caller's workspace (256-byte granules).
struct Carver {
  char* base;
  int64_t off = 0;
  explicit Carver(void* b) : base(reinterpret_cast<char*>(b)) {}
  void* take(int64_t bytes) {
    void* p = base ? base + off : nullptr;
    off += round_up(std::max<int64_t>(bytes, 1), 256);
    return p;
  }
};

static inline int64_t esize(int dtype) { return dtype == FLK_F32 ? 4 : 8; }
static inline int ld_for(int dtype, int64_t d) { return (int)round_up(d, dtype == FLK_F32 ? 4 : 2); }

// Operand images in the workspace.
struct Operand {
  // SIMT form
  void* xs = nullptr;     // [rows_pad x ld]
  void* norms = nullptr;  // [rows_pad]
  // tensor-core form
  void* img_a = nullptr;  // tile images for the output side
  void* img_b = nullptr;  // tile images for the reduction side
};

struct Layout {
  bool tc;
  bool fold = false;       // Gaussian, t = 1, resident tensor-core kernel: vector folded into the B images
  int* blk_pos = nullptr;  // fold: scratch of the sign partition (one int per 128 rows of the larger operand)
  int64_t total = 0;
  void* status = nullptr;  // 256 bytes: device status word of the tensor-core kernel
  void* sigma = nullptr;   // d entries of T (per-dimension length-scales)
  Operand x1, x2;
  void* vbuf = nullptr;  // padded copy of the vector operand of the first sweep
  void* ubuf = nullptr;  // fdmmv only: u = K v + w, padded
  void* raw1 = nullptr;
  void* raw2 = nullptr;
  SweepPlan s1, s2;
  // SIMT alternative of the tensor-core path (runs only when the image builder raised the range
  // flag): its own sweep plans and partial-result buffers; operands in x1.xs / x2.xs.
  void* fraw1 = nullptr;
  void* fraw2 = nullptr;
  SweepPlan f1, f2;
  int* range_flag() const { return reinterpret_cast<int*>(status) + tc::kStatusRange; }
  int* fold_block(int sweep_idx) const {
    return reinterpret_cast<int*>(status) + (sweep_idx == 0 ? tc::kFoldWordsSweep1 : tc::kFoldWordsSweep2);
  }
};

// need_x1_as_b / need_x2_as_a: which tensor-core images each operand needs.
static Layout make_layout(void* ws, bool dmmv, bool has_v, int dtype, int kernel, int64_t n, int64_t m,
                          int64_t d, int64_t t, int flags) {
  Layout L;
  L.tc = tc_eligible(dtype, kernel, d, t, flags);
  const int64_t es = esize(dtype);
  Carver c(ws);
  L.status = c.take(256);
  L.sigma = c.take(std::max<int64_t>(d, 1) * es);
  const bool kloop = L.tc && tck::supports_d(d);
  const bool wide_ok = wide_pays_off(L.tc, dtype, kernel, d, t);  // every path has a 32-columns-per-pass kernel
  L.fold = L.tc && !kloop && kernel == FLK_GAUSSIAN && t == 1 && !(flags & FLK_FLAG_NO_FOLD);
  L.s1 = plan_sweep(L.tc, dtype, n, m, t, wide_ok, kloop ? d : 0, L.fold);  // rows = X1, reduction over X2
  L.s2 = plan_sweep(L.tc, dtype, m, n, t, wide_ok, kloop ? d : 0, L.fold);  // rows = X2, reduction over X1 (fdmmv only)
  const int64_t n_pad = L.s1.r_pad, m_pad = L.s1.s_pad;
  const bool first = !dmmv || has_v;  // is the first sweep executed?
  if (L.tc) {
    const int64_t kp = kloop ? tck::padded_k(d) : tc::padded_k(d);
    // a folded reduction-side image has one tile more than the operand has (see flk_fold.cuh)
    const int64_t n_rows_b = L.fold ? tc::fold_image_rows(n) : n_pad, m_rows_b = L.fold ? tc::fold_image_rows(m) : m_pad;
    if (first) L.x1.img_a = c.take(n_pad * kp * 2);
    if (first) L.x2.img_b = c.take(m_rows_b * kp * 2);
    if (dmmv) {
      L.x2.img_a = c.take(m_pad * kp * 2);
      L.x1.img_b = c.take(n_rows_b * kp * 2);
    }
    if (L.fold) L.blk_pos = reinterpret_cast<int*>(c.take(((int64_t)tc::fold_blocks(std::max(n, m)) + 2) * 4));
    L.f1 = plan_sweep(false, dtype, n, m, t, wide_ok);
    L.f2 = plan_sweep(false, dtype, m, n, t, wide_ok);
  }
  {
    const int ld = ld_for(dtype, d);
    L.x1.xs = c.take(n_pad * ld * es);
    L.x1.norms = c.take(n_pad * es);
    L.x2.xs = c.take(m_pad * ld * es);
    L.x2.norms = c.take(m_pad * es);
  }
  const int tp = L.s1.tp;
  if (first) {
    L.vbuf = c.take(m_pad * tp * es);
    L.raw1 = c.take(L.s1.raw_elems() * es);
    if (L.tc) L.fraw1 = c.take(L.f1.raw_elems() * es);
  }
  if (dmmv) {
    L.ubuf = c.take(n_pad * tp * es);
    L.raw2 = c.take(L.s2.raw_elems() * es);
    if (L.tc) L.fraw2 = c.take(L.f2.raw_elems() * es);
  }
  L.total = c.off;
  return L;
}

static int check_common(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t) {
  if (dtype != FLK_F32 && dtype != FLK_F64) return fail(FLK_ERR_BAD_ARG, "unknown dtype %d", dtype);
  if (kernel < FLK_GAUSSIAN || kernel > FLK_MATERN25) return fail(FLK_ERR_BAD_ARG, "unknown kernel id %d", kernel);
  if (n < 0 || m < 0 || d < 0 || t < 0) return fail(FLK_ERR_BAD_ARG, "negative dimension");
  if (d == 0 && (n > 0 || m > 0)) return fail(FLK_ERR_BAD_ARG, "data with zero features (d = 0)");
  if (d > (1 << 20) || t > (1 << 20)) return fail(FLK_ERR_UNSUPPORTED, "d or t too large");
  if (n > (int64_t)1 << 40 || m > (int64_t)1 << 40) return fail(FLK_ERR_UNSUPPORTED, "n or m too large");
  return FLK_OK;
}

static int check_sigma(const double* sigma, int64_t sigma_len, int64_t d) {
  if (sigma == nullptr) return fail(FLK_ERR_BAD_ARG, "sigma: null pointer");
  if (sigma_len != 1 && sigma_len != d)
    return fail(FLK_ERR_BAD_ARG, "sigma must have 1 or d=%lld entries, got %lld", (long long)d, (long long)sigma_len);
  return FLK_OK;
}

static int check_workspace(const void* ws, int64_t have, int64_t need) {
  if (ws == nullptr) return fail(FLK_ERR_WORKSPACE, "workspace: null pointer (%lld bytes needed)", (long long)need);
  if ((reinterpret_cast<uintptr_t>(ws) & 255) != 0) return fail(FLK_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if (have < need)
    return fail(FLK_ERR_WORKSPACE, "workspace too small: %lld bytes given, %lld needed", (long long)have, (long long)need);
  return FLK_OK;
}

// Uploads per-dimension length-scales (cast to T, as the reference casts sigma to the data dtype).
template <typename T>
static int upload_sigma(const double* sigma, int64_t sigma_len, void* dst, T* scalar_out, const T** dev_out,
                        cudaStream_t stream) {
  if (sigma_len == 1) {
    *scalar_out = (T)sigma[0];
    *dev_out = nullptr;
    return FLK_OK;
  }
  std::vector<T> tmp((size_t)sigma_len);
  for (int64_t k = 0; k < sigma_len; ++k) tmp[(size_t)k] = (T)sigma[k];
  // pageable source: the runtime stages the bytes before returning, so `tmp` may go out of scope
  FLK_CUDA_TRY(cudaMemcpyAsync(dst, tmp.data(), sizeof(T) * (size_t)sigma_len, cudaMemcpyHostToDevice, stream));
  *scalar_out = (T)1;
  *dev_out = reinterpret_cast<const T*>(dst);
  return FLK_OK;
}

template <typename T, typename TIn = T>
static int run_prep_rows(const Mat& X, const T* sigma_dev, T sigma_scalar, int sigma_len, void* xs, int ld,
                         int64_t rows_pad, void* norms, Gate gate, cudaStream_t stream) {
  int blocks = (int)ceil_div(rows_pad, (int64_t)kPrepRows * kPrepSubBlocks);
  prep_rows_kernel<T, TIn><<<blocks, 256, 0, stream>>>(reinterpret_cast<const TIn*>(X.ptr), X.rows, (int)X.cols, X.rs,
                                                  X.cs, sigma_dev, sigma_scalar, sigma_len,
                                                  reinterpret_cast<T*>(xs), ld, rows_pad,
                                                  reinterpret_cast<T*>(norms), gate);
  count_launch();
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <typename T>
static int run_prep_vec(const Mat& v, void* vbuf, int64_t s_pad, int tp, int tt, cudaStream_t stream) {
  prep_vec_kernel<T><<<grid_for(s_pad * tp), 256, 0, stream>>>(reinterpret_cast<const T*>(v.ptr), v.rows,
                                                                (int)v.cols, v.rs, v.cs,
                                                                reinterpret_cast<T*>(vbuf), s_pad, tp, tt);
  count_launch();
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <typename T>
static int run_finalize(const SweepPlan& sp, const void* raw, const Mat* add, void* out, int64_t out_rs,
                        int64_t out_cs, int64_t t, bool padded, Gate gate, cudaStream_t stream,
                        const int* timeout_word = nullptr) {
  finalize_kernel<T><<<grid_for(sp.r_pad * sp.tp), 256, 0, stream>>>(
      reinterpret_cast<const T*>(raw), sp.n_chunks, sp.r_pad, sp.tp, sp.r, (int)t,
      add ? reinterpret_cast<const T*>(add->ptr) : nullptr, add ? add->rs : 0, add ? add->cs : 0,
      reinterpret_cast<T*>(out), out_rs, out_cs, padded ? 1 : 0, sp.tt, (int64_t)sp.main_tiles * sp.br,
      sp.n_chunks_tail, gate, timeout_word);
  count_launch();
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

template <typename T>
static int run_sweep_simt(int kernel, const SweepPlan& sp, const Operand& a, const Operand& b, int ld,
                          const void* vec, void* raw, Gate gate, cudaStream_t stream, int sweep_idx) {
  SimtArgs<T> args;
  args.A = reinterpret_cast<const T*>(a.xs);
  args.an = reinterpret_cast<const T*>(a.norms);
  args.B = reinterpret_cast<const T*>(b.xs);
  args.bn = reinterpret_cast<const T*>(b.norms);
  args.vec = reinterpret_cast<const T*>(vec);
  args.raw = reinterpret_cast<T*>(raw);
  args.ld = ld;
  args.tp = sp.tp;
  args.r_pad = sp.r_pad;
  args.s_pad = sp.s_pad;
  args.row_tiles = sp.row_tiles;
  args.n_col_tiles = sp.n_col_tiles;
  args.tiles_per_chunk = sp.tiles_per_chunk;
  args.n_chunks = sp.n_chunks;
  args.gate = gate;
  const bool timed = gate.flag == nullptr;  // the gated alternative is not the timed kernel
  if (timed) FLK_TRY(timer_mark(2 * sweep_idx, stream));
  if (sp.tt == kWideT) {
    if constexpr (sizeof(T) == 8) {
      // fp64, many vector columns: both products on the fp64 tensor-core instruction (flk_dmma.cuh)
      FLK_TRY(dmma::launch(kernel, args, sp.n_chunks, sp.t_chunks, stream));
    } else {
      FLK_TRY((launch_wide_any<T>(kernel, args, sp.n_chunks, sp.t_chunks, stream)));
    }
  } else
    FLK_TRY((launch_simt_any<T>(kernel, args, sp.tt, sp.n_chunks, sp.t_chunks, stream)));
  if (timed) FLK_TRY(timer_mark(2 * sweep_idx + 1, stream));
  count_launch();
  return FLK_OK;
}

static int run_sweep_tc(int kernel, const SweepPlan& sp, const void* img_a, const void* img_b, int64_t d,
                        const void* vec, void* raw, void* status, const int* fold, cudaStream_t stream,
                        int sweep_idx) {
  FLK_TRY(timer_mark(2 * sweep_idx, stream));
  if (sp.kloop) {
    tck::SweepArgsL args;
    args.img_a = reinterpret_cast<const __half*>(img_a);
    args.img_b = reinterpret_cast<const __half*>(img_b);
    args.vec = reinterpret_cast<const float*>(vec);
    args.raw = reinterpret_cast<float*>(raw);
    args.status = reinterpret_cast<int*>(status);
    args.tp = sp.tp;
    args.r_pad = sp.r_pad;
    args.s_pad = sp.s_pad;
    args.row_tiles = sp.row_tiles;
    args.n_col_tiles = sp.n_col_tiles;
    args.tiles_per_chunk = sp.tiles_per_chunk;
    FLK_TRY(tck::launch_sweep(kernel, (int)d, args, sp.tt, sp.n_chunks, sp.t_chunks, stream));
  } else {
    tc::SweepArgs args;
    args.img_a = reinterpret_cast<const __half*>(img_a);
    args.img_b = reinterpret_cast<const __half*>(img_b);
    args.vec = reinterpret_cast<const float*>(vec);
    args.raw = reinterpret_cast<float*>(raw);
    args.status = reinterpret_cast<int*>(status);
    args.fold = sp.fold ? fold : nullptr;
    args.tp = sp.tp;
    args.r_pad = sp.r_pad;
    args.s_pad = sp.s_pad;
    args.row_tiles = sp.row_tiles;
    args.n_col_tiles = sp.n_col_tiles;
    args.tiles_per_chunk = sp.tiles_per_chunk;
    args.main_tiles = sp.main_tiles;
    args.main_ctas = sp.main_tiles * sp.n_chunks;
    args.tiles_per_chunk_tail = sp.tiles_per_chunk_tail;
    FLK_TRY(tc::launch_sweep(kernel, (int)d, args, sp.tt, (int)sp.grid_x(), sp.t_chunks, stream));
  }
  FLK_TRY(timer_mark(2 * sweep_idx + 1, stream));
  count_launch();
  return FLK_OK;
}

// Gates of the two alternatives when the tensor-core path is chosen: the tensor-core results count
// while the range flag is clear, the SIMT ones when it is set.  Without the tensor-core path the
// SIMT kernels run unconditionally.
static inline Gate gate_tc(const Layout& L) { return Gate{L.range_flag(), 0}; }
static inline Gate gate_simt(const Layout& L) { return L.tc ? Gate{L.range_flag(), 1} : Gate{nullptr, 0}; }

// Builds the operand forms both paths need: tensor-core tile images (which also raise the range
// flags) and, gated, the scaled rows + norms of the SIMT kernels.  Operands the caller keeps from the previous
// call on this workspace (FLK_FLAG_KEEP_X1 / _X2) are skipped: their images, SIMT forms and range words are
// still in place.
template <typename T>
static int prepare_operands(const Layout& L, int kernel, const Mat& X1, const Mat& X2, int64_t d, const T* sig_dev,
                            T sig_scalar, int sigma_len, int dtype, bool reset_status, int flags, cudaStream_t stream) {
  const bool keep1 = (flags & FLK_FLAG_KEEP_X1) != 0, keep2 = (flags & FLK_FLAG_KEEP_X2) != 0;
  int* status = reinterpret_cast<int*>(L.status);
  if (L.tc) {
    if (reset_status) {
      reset_status_kernel<<<1, 64, 0, stream>>>(status, keep1 ? 1 : 0, keep2 ? 1 : 0);
      FLK_CUDA_TRY(cudaGetLastError());
    } else if (L.fold) {  // the fold blocks start from zero in every call (the leading status words are kept)
      FLK_CUDA_TRY(cudaMemsetAsync(L.fold_block(0), 0, 2 * tc::kFoldWords * sizeof(int), stream));
    }
    auto prep = L.s1.kloop ? tck::prep_images_large : tc::prep_images;
    // folded sweeps build their reduction-side images per sweep, with the vector (build_folded_image)
    void* x1_b = L.fold ? nullptr : L.x1.img_b;
    void* x2_b = L.fold ? nullptr : L.x2.img_b;
    if (!keep1 && (L.x1.img_a != nullptr || x1_b != nullptr)) {
      FLK_TRY(prep(kernel, X1.ptr, X1.rows, X1.rs, X1.cs, (int)d, (const float*)sig_dev, (float)sig_scalar, sigma_len,
                   L.s1.r_pad, L.x1.img_a, x1_b, status + tc::kStatusRangeX1, stream));
      count_launch();
    }
    if (!keep2 && (L.x2.img_a != nullptr || x2_b != nullptr)) {
      FLK_TRY(prep(kernel, X2.ptr, X2.rows, X2.rs, X2.cs, (int)d, (const float*)sig_dev, (float)sig_scalar, sigma_len,
                   L.s1.s_pad, L.x2.img_a, x2_b, status + tc::kStatusRangeX2, stream));
      count_launch();
    }
  }
  const int ld = ld_for(dtype, d);
  // (the SIMT form of a kept operand is as valid as it was: built if its gate was open then, and the gate of a call
  // that keeps every operand can only differ through the per-call range word, i.e. through the vector -- in which
  // case it is built now)
  const bool simt_only = !L.tc;
  if (!(keep1 && simt_only))
    FLK_TRY(run_prep_rows<T>(X1, sig_dev, sig_scalar, sigma_len, L.x1.xs, ld, L.s1.r_pad, L.x1.norms, gate_simt(L), stream));
  if (!(keep2 && simt_only))
    FLK_TRY(run_prep_rows<T>(X2, sig_dev, sig_scalar, sigma_len, L.x2.xs, ld, L.s1.s_pad, L.x2.norms, gate_simt(L), stream));
  return FLK_OK;
}

// One sweep + its finalisation, on whichever path(s) the layout holds.  `a`/`b` = output-side and
// reduction-side operands, `tcp`/`fp` = the tensor-core (or sole SIMT) plan and the SIMT alternative.
// What a folded sweep needs beside the plan: the reduction-side operand as the caller gave it, and sigma.
struct FoldSigma {
  const float* dev = nullptr;
  float scalar = 1.0f;
  int len = 1;
};

template <typename T>
static int sweep_and_finalize(const Layout& L, int kernel, int dtype, int64_t d, int64_t t, const SweepPlan& tcp,
                              const SweepPlan& fp, const Operand& a, const Operand& b, const void* vec, void* raw,
                              void* fraw, const Mat* add, void* out, int64_t out_rs, int64_t out_cs, bool padded,
                              cudaStream_t stream, int sweep_idx, const Mat& bX = Mat{nullptr, 0, 0, 0, 0},
                              const FoldSigma& fold_sig = FoldSigma{}) {
  const int ld = ld_for(dtype, d);
  if (L.tc) {
    if (L.fold) {
      if constexpr (sizeof(T) == 4) {
        // reduction-side image of this sweep with the vector folded in (vec is dense: one column, tt = 1)
        FLK_TRY(tc::build_folded_image(kernel, bX.ptr, bX.rows, bX.rs, bX.cs, (int)d, fold_sig.dev, fold_sig.scalar,
                                       fold_sig.len, reinterpret_cast<const float*>(vec), L.blk_pos,
                                       L.fold_block(sweep_idx), b.img_b, reinterpret_cast<int*>(L.status), stream));
        count_launch(3);
      }
    }
    FLK_TRY(run_sweep_tc(kernel, tcp, a.img_a, b.img_b, d, vec, raw, L.status, L.fold_block(sweep_idx), stream,
                         sweep_idx));
    FLK_TRY(run_finalize<T>(tcp, raw, add, out, out_rs, out_cs, t, padded, gate_tc(L), stream,
                            reinterpret_cast<const int*>(L.status) + tc::kStatusTimeout));
    FLK_TRY(run_sweep_simt<T>(kernel, fp, a, b, ld, vec, fraw, gate_simt(L), stream, sweep_idx));
    FLK_TRY(run_finalize<T>(fp, fraw, add, out, out_rs, out_cs, t, padded, gate_simt(L), stream));
  } else {
    FLK_TRY(run_sweep_simt<T>(kernel, tcp, a, b, ld, vec, raw, gate_simt(L), stream, sweep_idx));
    FLK_TRY(run_finalize<T>(tcp, raw, add, out, out_rs, out_cs, t, padded, gate_simt(L), stream));
  }
  return FLK_OK;
}

// ---------------------------------------------------------------------------------------------
// fmmv / fdmmv on device pointers
// ---------------------------------------------------------------------------------------------
template <typename T>
static int fmmv_impl(int dtype, int kernel, const Mat& X1, const Mat& X2, const Mat& v, void* out,
                     int64_t out_rs, int64_t out_cs, const double* sigma, int64_t sigma_len, void* ws,
                     int64_t ws_bytes, int flags, cudaStream_t stream, bool reset_status = true) {
  const int64_t n = X1.rows, m = X2.rows, d = X1.cols, t = v.cols;
  Layout L = make_layout(ws, false, true, dtype, kernel, n, m, d, t, flags);
  if ((flags & FLK_FLAG_FORCE_TC) && !L.tc)
    return fail(FLK_ERR_UNSUPPORTED, "tensor-core kernel does not cover dtype=%d d=%lld", dtype, (long long)d);
  FLK_TRY(check_workspace(ws, ws_bytes, L.total));
  if (n == 0 || t == 0) return FLK_OK;
  T sig_scalar;
  const T* sig_dev;
  FLK_TRY(upload_sigma<T>(sigma, sigma_len, L.sigma, &sig_scalar, &sig_dev, stream));
  FLK_TRY(prepare_operands<T>(L, kernel, X1, X2, d, sig_dev, sig_scalar, (int)sigma_len, dtype, reset_status, flags, stream));
  FLK_TRY(run_prep_vec<T>(v, L.vbuf, L.s1.s_pad, L.s1.tp, L.s1.tt, stream));
  FoldSigma fs;
  if constexpr (sizeof(T) == 4) fs = FoldSigma{sig_dev, sig_scalar, (int)sigma_len};
  // FLK_FLAG_ACCUMULATE: out += K v (column chunks of a product whose reduction side is split under a memory budget)
  const Mat prev{out, n, t, out_rs, out_cs};
  FLK_TRY(sweep_and_finalize<T>(L, kernel, dtype, d, t, L.s1, L.f1, L.x1, L.x2, L.vbuf, L.raw1, L.fraw1,
                                (flags & FLK_FLAG_ACCUMULATE) ? &prev : nullptr, out, out_rs, out_cs, false, stream, 0,
                                X2, fs));
  return FLK_OK;
}

// `accumulate`: add the result to what `out` already holds (row chunks of X1 are summed this way by the
// host-buffer entry point); `reset_status`: clear the status block first (false for all chunks but the first,
// so that a timeout code or a raised range flag of an earlier chunk stays visible).
template <typename T>
static int fdmmv_impl(int dtype, int kernel, const Mat& X1, const Mat& X2, const Mat& v, const Mat& w, int64_t t,
                      void* out, int64_t out_rs, int64_t out_cs, const double* sigma, int64_t sigma_len,
                      void* ws, int64_t ws_bytes, int flags, cudaStream_t stream, bool accumulate = false,
                      bool reset_status = true) {
  const int64_t n = X1.rows, m = X2.rows, d = X1.cols;
  const bool has_v = v.ptr != nullptr, has_w = w.ptr != nullptr;
  Layout L = make_layout(ws, true, has_v, dtype, kernel, n, m, d, t, flags);
  if ((flags & FLK_FLAG_FORCE_TC) && !L.tc)
    return fail(FLK_ERR_UNSUPPORTED, "tensor-core kernel does not cover dtype=%d d=%lld", dtype, (long long)d);
  FLK_TRY(check_workspace(ws, ws_bytes, L.total));
  if (m == 0 || t == 0) return FLK_OK;
  T sig_scalar;
  const T* sig_dev;
  FLK_TRY(upload_sigma<T>(sigma, sigma_len, L.sigma, &sig_scalar, &sig_dev, stream));
  FLK_TRY(prepare_operands<T>(L, kernel, X1, X2, d, sig_dev, sig_scalar, (int)sigma_len, dtype, reset_status, flags, stream));
  FoldSigma fs;
  if constexpr (sizeof(T) == 4) fs = FoldSigma{sig_dev, sig_scalar, (int)sigma_len};
  if (has_v) {
    // sweep 1: u = K v (+ w), kept as a padded vector operand
    FLK_TRY(run_prep_vec<T>(v, L.vbuf, L.s1.s_pad, L.s1.tp, L.s1.tt, stream));
    FLK_TRY(sweep_and_finalize<T>(L, kernel, dtype, d, t, L.s1, L.f1, L.x1, L.x2, L.vbuf, L.raw1, L.fraw1,
                                  has_w ? &w : nullptr, L.ubuf, 0, 0, true, stream, 0, X2, fs));
  } else {
    FLK_TRY(run_prep_vec<T>(w, L.ubuf, L.s1.r_pad, L.s1.tp, L.s1.tt, stream));
  }
  // sweep 2: out = K^T u  (rows = X2, reduction over X1)
  const Mat prev{out, m, t, out_rs, out_cs};
  FLK_TRY(sweep_and_finalize<T>(L, kernel, dtype, d, t, L.s2, L.f2, L.x2, L.x1, L.ubuf, L.raw2, L.fraw2,
                                accumulate ? &prev : nullptr, out, out_rs, out_cs, false, stream, 1, X1, fs));
  return FLK_OK;
}


// ---------------------------------------------------------------------------------------------
// fmm: the kernel matrix itself (needed once per fit for the preconditioner)
// ---------------------------------------------------------------------------------------------
struct FmmLayout {
  int64_t total = 0;
  void* sigma = nullptr;
  void *xs1 = nullptr, *n1 = nullptr, *xs2 = nullptr, *n2 = nullptr;
  int ld = 0;
  int64_t n_pad = 0, m_pad = 0;
};

static FmmLayout make_fmm_layout(void* ws, int math_dtype, int64_t n, int64_t m, int64_t d) {
  FmmLayout L;
  const int64_t es = esize(math_dtype);
  Carver c(ws);
  L.sigma = c.take(std::max<int64_t>(d, 1) * es);
  L.ld = ld_for(math_dtype, d);
  L.n_pad = round_up(std::max<int64_t>(n, 1), kRowPad);
  L.m_pad = round_up(std::max<int64_t>(m, 1), kRowPad);
  L.xs1 = c.take(L.n_pad * L.ld * es);
  L.n1 = c.take(L.n_pad * es);
  L.xs2 = c.take(L.m_pad * L.ld * es);
  L.n2 = c.take(L.m_pad * es);
  L.total = c.off;
  return L;
}

// T = arithmetic type, TIO = type of the data and of the stored matrix
template <typename T, typename TIO>
static int fmm_impl(int math_dtype, int kernel, const Mat& X1, const Mat& X2, void* out, int64_t out_rs,
                    int64_t out_cs, const double* sigma, int64_t sigma_len, void* ws, int64_t ws_bytes,
                    cudaStream_t stream) {
  const int64_t n = X1.rows, m = X2.rows, d = X1.cols;
  FmmLayout L = make_fmm_layout(ws, math_dtype, n, m, d);
  FLK_TRY(check_workspace(ws, ws_bytes, L.total));
  if (n == 0 || m == 0) return FLK_OK;
  T sig_scalar;
  const T* sig_dev;
  FLK_TRY(upload_sigma<T>(sigma, sigma_len, L.sigma, &sig_scalar, &sig_dev, stream));
  const Gate always{nullptr, 0};
  FLK_TRY((run_prep_rows<T, TIO>(X1, sig_dev, sig_scalar, (int)sigma_len, L.xs1, L.ld, L.n_pad, L.n1, always, stream)));
  FLK_TRY((run_prep_rows<T, TIO>(X2, sig_dev, sig_scalar, (int)sigma_len, L.xs2, L.ld, L.m_pad, L.n2, always, stream)));
  FLK_TRY((launch_kmat<T, TIO>(kernel, (const T*)L.xs1, (const T*)L.n1, (const T*)L.xs2, (const T*)L.n2, L.ld,
                               reinterpret_cast<TIO*>(out), n, m, out_rs, out_cs, stream)));
  count_launch();
  return FLK_OK;
}

// Backward-pass pair weights (flk_grad.cuh) on the same prepared operands as fmm.
template <typename T, typename TIO>
static int kgrad_impl(int math_dtype, int kernel, const Mat& X1, const Mat& X2, const Mat& G, const Mat& V, int64_t t,
                      void* out, int64_t out_rs, int64_t out_cs, const double* sigma, int64_t sigma_len, void* ws,
                      int64_t ws_bytes, cudaStream_t stream) {
  const int64_t n = X1.rows, m = X2.rows, d = X1.cols;
  FmmLayout L = make_fmm_layout(ws, math_dtype, n, m, d);
  FLK_TRY(check_workspace(ws, ws_bytes, L.total));
  if (n == 0 || m == 0) return FLK_OK;
  T sig_scalar;
  const T* sig_dev;
  FLK_TRY(upload_sigma<T>(sigma, sigma_len, L.sigma, &sig_scalar, &sig_dev, stream));
  const Gate always{nullptr, 0};
  FLK_TRY((run_prep_rows<T, TIO>(X1, sig_dev, sig_scalar, (int)sigma_len, L.xs1, L.ld, L.n_pad, L.n1, always, stream)));
  FLK_TRY((run_prep_rows<T, TIO>(X2, sig_dev, sig_scalar, (int)sigma_len, L.xs2, L.ld, L.m_pad, L.n2, always, stream)));
  const bool factors = t > 0;
  FLK_TRY((launch_kgrad<T, TIO>(kernel, (const T*)L.xs1, (const T*)L.n1, (const T*)L.xs2, (const T*)L.n2, L.ld,
                                factors ? (const TIO*)G.ptr : nullptr, G.rs, G.cs, (const TIO*)V.ptr, V.rs, V.cs,
                                (int)t, factors ? nullptr : (const TIO*)G.ptr, G.rs, G.cs,
                                reinterpret_cast<TIO*>(out), n, m, out_rs, out_cs, stream)));
  count_launch();
  return FLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Host-buffer variants: stage dense copies of the operands in the workspace, run, copy back.
// ---------------------------------------------------------------------------------------------
struct Staged {
  Mat dev;          // the device copy, same orientation as the host matrix
  int64_t bytes;    // bytes reserved in the workspace
};

// A strided host matrix is copied as the dense block spanned by its unit-stride dimension.
static Staged plan_stage(const Mat& h, int64_t es, Carver& c) {
  Staged s;
  s.dev = h;
  s.bytes = 0;
  if (h.ptr == nullptr || h.rows == 0 || h.cols == 0) {
    s.dev.ptr = nullptr;
    return s;
  }
  s.bytes = h.rows * h.cols * es;
  s.dev.ptr = c.take(s.bytes);
  const bool row_major = (h.cs == 1) || (h.rs != 1);
  if (row_major) {
    s.dev.rs = h.cols;
    s.dev.cs = 1;
  } else {
    s.dev.rs = 1;
    s.dev.cs = h.rows;
  }
  return s;
}

static int copy_matrix(const Mat& dst, const Mat& src, int64_t es, cudaMemcpyKind kind, cudaStream_t stream) {
  if (src.ptr == nullptr || dst.ptr == nullptr || src.rows == 0 || src.cols == 0) return FLK_OK;
  const bool row_major = (dst.cs == 1 && src.cs == 1);
  // width = contiguous run, height = number of runs
  int64_t width, height, spitch, dpitch;
  if (row_major) {
    width = src.cols * es;
    height = src.rows;
    spitch = (src.rows > 1 ? src.rs : src.cols) * es;
    dpitch = (dst.rows > 1 ? dst.rs : dst.cols) * es;
  } else {
    if (src.rs != 1 || dst.rs != 1) return fail(FLK_ERR_LAYOUT, "internal: orientation mismatch in staged copy");
    width = src.rows * es;
    height = src.cols;
    spitch = (src.cols > 1 ? src.cs : src.rows) * es;
    dpitch = (dst.cols > 1 ? dst.cs : dst.rows) * es;
  }
  if (spitch < width) spitch = width;
  if (dpitch < width) dpitch = width;
  if (spitch == width && dpitch == width) {  // fully contiguous on both sides: one linear copy
    FLK_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(dst.ptr), src.ptr, (size_t)(width * height), kind, stream));
    return FLK_OK;
  }
  FLK_CUDA_TRY(cudaMemcpy2DAsync(const_cast<void*>(dst.ptr), (size_t)dpitch, src.ptr, (size_t)spitch, (size_t)width,
                                 (size_t)height, kind, stream));
  return FLK_OK;
}

// Reads the tensor-core status word after the stream has drained; non-zero means a bounded wait gave up.
static int check_tc_status(const void* inner_ws) {
  int host = 0;
  FLK_CUDA_TRY(cudaMemcpy(&host, inner_ws, sizeof(int), cudaMemcpyDeviceToHost));
  if (host != 0) return fail(FLK_ERR_TIMEOUT, "tensor-core kernel gave up waiting on a barrier (status 0x%x)", host);
  return FLK_OK;
}

struct HostLayout {
  Staged x1, x2, v, w, out;
  void* inner = nullptr;
  int64_t inner_bytes = 0;
  int64_t total = 0;
  int n_chunks = 1;        // row chunks of X1: the copy of chunk c + 1 runs under the kernels of chunk c
  int64_t chunk_rows = 0;  // rows per chunk (the last one may be shorter)
};

constexpr int kMaxHostChunks = 8;  // the copy of the first chunk is the only one no kernel hides: keep it short
constexpr int64_t kMinChunkRows = 131072;

static HostLayout make_host_layout(void* ws, bool dmmv, int dtype, int kernel, const Mat& X1, const Mat& X2,
                                   const Mat& v, const Mat& w, const Mat& out, int64_t t, int flags) {
  HostLayout H;
  const int64_t es = esize(dtype);
  Carver c(ws);
  H.x1 = plan_stage(X1, es, c);
  H.x2 = plan_stage(X2, es, c);
  H.v = plan_stage(v, es, c);
  H.w = plan_stage(w, es, c);
  H.out = plan_stage(out, es, c);
  const int64_t n = X1.rows;
  H.n_chunks = (int)std::max<int64_t>(1, std::min<int64_t>(kMaxHostChunks, n / kMinChunkRows));
  H.chunk_rows = round_up(ceil_div(std::max<int64_t>(n, 1), H.n_chunks), kRowPad);
  H.n_chunks = (int)ceil_div(std::max<int64_t>(n, 1), H.chunk_rows);
  // The workspace of a product is not monotonic in its row count (the sweep planner picks the number of reduction
  // chunks, hence of partial-result buffers, from how the tiles fill waves of CTAs): size the inner workspace for
  // both chunk lengths that occur, the full one and the shorter last one.
  const int64_t full_rows = std::min(n, H.chunk_rows);
  const int64_t last_rows = n - (int64_t)(H.n_chunks - 1) * H.chunk_rows;
  H.inner_bytes = make_layout(nullptr, dmmv, v.ptr != nullptr, dtype, kernel, full_rows, X2.rows, X1.cols, t, flags).total;
  if (last_rows > 0 && last_rows != full_rows)
    H.inner_bytes = std::max(H.inner_bytes, make_layout(nullptr, dmmv, v.ptr != nullptr, dtype, kernel, last_rows,
                                                        X2.rows, X1.cols, t, flags).total);
  H.inner = c.take(H.inner_bytes);
  H.total = c.off;
  return H;
}

// Rows [r0, r0 + rows) of a matrix (a view: same strides).
static Mat row_block(const Mat& m, int64_t r0, int64_t rows, int64_t es) {
  Mat b = m;
  if (m.ptr != nullptr) b.ptr = reinterpret_cast<const char*>(m.ptr) + r0 * m.rs * es;
  b.rows = rows;
  return b;
}

// One copy stream and a few events per device, created on first use and kept for the life of the
// process: the host-buffer entry points push their host->device copies through it so that they
// overlap the kernels running on the caller's stream.
struct CopyLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t ev[kMaxHostChunks + 2] = {};
  bool ready = false;
};
static CopyLane g_copy_lane[64];

static int copy_lane_for_current_device(CopyLane** out) {
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FLK_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  CopyLane& L = g_copy_lane[dev];
  if (!L.ready) {
    FLK_CUDA_TRY(cudaStreamCreateWithFlags(&L.stream, cudaStreamNonBlocking));
    for (auto& e : L.ev) FLK_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    L.ready = true;
  }
  *out = &L;
  return FLK_OK;
}

// Shared body of the two host-buffer entry points.
static int run_host(bool dmmv, int dtype, int kernel, const Mat& a, const Mat& b, const Mat& vv, const Mat& ww,
                    const Mat& oo, int64_t t, const double* sigma_host, int64_t sigma_len, void* workspace,
                    int64_t workspace_bytes, int flags, cudaStream_t st) {
  flags &= ~(FLK_FLAG_KEEP_X1 | FLK_FLAG_KEEP_X2 | FLK_FLAG_ACCUMULATE);  // staged copies are fresh in every call
  const int64_t n = a.rows, m = b.rows, d = a.cols;
  HostLayout H = make_host_layout(workspace, dmmv, dtype, kernel, a, b, vv, ww, oo, t, flags);
  FLK_TRY(check_workspace(workspace, workspace_bytes, H.total));
  if (t == 0 || (dmmv ? m == 0 : n == 0)) return FLK_OK;
  const int64_t es = esize(dtype);
  CopyLane* lane = nullptr;
  FLK_TRY(copy_lane_for_current_device(&lane));
  // the copies must not overtake earlier work of the caller's stream that may still use the workspace
  FLK_CUDA_TRY(cudaEventRecord(lane->ev[0], st));
  FLK_CUDA_TRY(cudaStreamWaitEvent(lane->stream, lane->ev[0], 0));
  FLK_TRY(copy_matrix(H.x2.dev, b, es, cudaMemcpyHostToDevice, lane->stream));
  FLK_TRY(copy_matrix(H.v.dev, vv, es, cudaMemcpyHostToDevice, lane->stream));
  FLK_CUDA_TRY(cudaEventRecord(lane->ev[1], lane->stream));
  for (int c = 0; c < H.n_chunks; ++c) {
    const int64_t r0 = (int64_t)c * H.chunk_rows, rows = std::min(H.chunk_rows, n - r0);
    FLK_TRY(copy_matrix(row_block(H.x1.dev, r0, rows, es), row_block(a, r0, rows, es), es, cudaMemcpyHostToDevice,
                        lane->stream));
    if (dmmv)
      FLK_TRY(copy_matrix(row_block(H.w.dev, r0, rows, es), row_block(ww, r0, rows, es), es, cudaMemcpyHostToDevice,
                          lane->stream));
    FLK_CUDA_TRY(cudaEventRecord(lane->ev[2 + c], lane->stream));
  }
  FLK_CUDA_TRY(cudaStreamWaitEvent(st, lane->ev[1], 0));
  for (int c = 0; c < H.n_chunks; ++c) {
    const int64_t r0 = (int64_t)c * H.chunk_rows, rows = std::min(H.chunk_rows, n - r0);
    FLK_CUDA_TRY(cudaStreamWaitEvent(st, lane->ev[2 + c], 0));
    const Mat xa = row_block(H.x1.dev, r0, rows, es);
    if (dmmv) {
      const Mat wc = row_block(H.w.dev, r0, rows, es);
      void* o = const_cast<void*>(H.out.dev.ptr);
      if (dtype == FLK_F32)
        FLK_TRY(fdmmv_impl<float>(dtype, kernel, xa, H.x2.dev, H.v.dev, wc, t, o, H.out.dev.rs, H.out.dev.cs,
                                  sigma_host, sigma_len, H.inner, H.inner_bytes, flags, st, c > 0, c == 0));
      else
        FLK_TRY(fdmmv_impl<double>(dtype, kernel, xa, H.x2.dev, H.v.dev, wc, t, o, H.out.dev.rs, H.out.dev.cs,
                                   sigma_host, sigma_len, H.inner, H.inner_bytes, flags, st, c > 0, c == 0));
    } else {
      const Mat oc = row_block(H.out.dev, r0, rows, es);
      void* o = const_cast<void*>(oc.ptr);
      if (dtype == FLK_F32)
        FLK_TRY(fmmv_impl<float>(dtype, kernel, xa, H.x2.dev, H.v.dev, o, oc.rs, oc.cs, sigma_host, sigma_len,
                                 H.inner, H.inner_bytes, flags, st, c == 0));
      else
        FLK_TRY(fmmv_impl<double>(dtype, kernel, xa, H.x2.dev, H.v.dev, o, oc.rs, oc.cs, sigma_host, sigma_len,
                                  H.inner, H.inner_bytes, flags, st, c == 0));
    }
  }
  FLK_TRY(copy_matrix(oo, H.out.dev, es, cudaMemcpyDeviceToHost, st));
  FLK_CUDA_TRY(cudaStreamSynchronize(st));
  if (tc_eligible(dtype, kernel, d, t, flags)) FLK_TRY(check_tc_status(H.inner));
  return FLK_OK;
}

}  // namespace flk

using namespace flk;

extern "C" {

int flk_version(void) { return 100; }

const char* flk_last_error(void) { return last_error_buf(); }

const char* flk_status_name(int status) {
  switch (status) {
    case FLK_OK: return "FLK_OK";
    case FLK_ERR_BAD_ARG: return "FLK_ERR_BAD_ARG";
    case FLK_ERR_LAYOUT: return "FLK_ERR_LAYOUT";
    case FLK_ERR_WORKSPACE: return "FLK_ERR_WORKSPACE";
    case FLK_ERR_CUDA: return "FLK_ERR_CUDA";
    case FLK_ERR_UNSUPPORTED: return "FLK_ERR_UNSUPPORTED";
    case FLK_ERR_DEVICE: return "FLK_ERR_DEVICE";
    case FLK_ERR_TIMEOUT: return "FLK_ERR_TIMEOUT";
  }
  return "FLK_UNKNOWN";
}

int flk_check_device(void) {
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  int major = 0, minor = 0;
  FLK_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  FLK_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
  if (major != 10) return fail(FLK_ERR_DEVICE, "device %d has compute capability %d.%d; sm_100 required", dev, major, minor);
  return FLK_OK;
}

int flk_uses_tensor_cores(int dtype, int kernel, int64_t d, int64_t t, int flags) {
  return tc_eligible(dtype, kernel, d, t, flags) ? 1 : 0;
}

int64_t flk_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int flk_square_norm(int dtype, const void* X, int64_t n, int64_t d, int64_t x_rs, int64_t x_cs,
                    const double* sigma_host, int64_t sigma_len, void* out, void* stream) {
  FLK_TRY(check_common(dtype, FLK_GAUSSIAN, n, 0, d, 0));
  Mat mx{X, n, d, x_rs, x_cs};
  FLK_TRY(check_mat("X", mx, n == 0));
  if (out == nullptr && n > 0) return fail(FLK_ERR_BAD_ARG, "out: null pointer");
  if (sigma_host != nullptr && sigma_len != 1 && sigma_len != d)
    return fail(FLK_ERR_BAD_ARG, "sigma must have 1 or d entries");
  if (sigma_host != nullptr && sigma_len != 1)
    return fail(FLK_ERR_UNSUPPORTED, "flk_square_norm takes a scalar sigma only (no workspace to stage a vector)");
  if (n == 0) return FLK_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int blocks = (int)ceil_div(n, kPrepRows);
  if (dtype == FLK_F32) {
    float s = sigma_host ? (float)sigma_host[0] : 1.0f;
    norm_rows_kernel<float><<<blocks, 256, 0, st>>>((const float*)X, n, (int)d, x_rs, x_cs, s, (float*)out);
  } else {
    double s = sigma_host ? sigma_host[0] : 1.0;
    norm_rows_kernel<double><<<blocks, 256, 0, st>>>((const double*)X, n, (int)d, x_rs, x_cs, s, (double*)out);
  }
  count_launch();
  FLK_CUDA_TRY(cudaGetLastError());
  return FLK_OK;
}

int64_t flk_fmmv_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t, int flags) {
  int s = check_common(dtype, kernel, n, m, d, t);
  if (s != FLK_OK) return s;
  return make_layout(nullptr, false, true, dtype, kernel, n, m, d, t, flags).total;
}

int64_t flk_fdmmv_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t, int flags) {
  int s = check_common(dtype, kernel, n, m, d, t);
  if (s != FLK_OK) return s;
  return make_layout(nullptr, true, true, dtype, kernel, n, m, d, t, flags).total;
}

int flk_fmmv(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs, const void* X2,
             int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d, const void* v, int64_t t, int64_t v_rs,
             int64_t v_cs, void* out, int64_t out_rs, int64_t out_cs, const double* sigma_host,
             int64_t sigma_len, void* workspace, int64_t workspace_bytes, int flags, void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, t));
  Mat a{X1, n, d, x1_rs, x1_cs}, b{X2, m, d, x2_rs, x2_cs}, vv{v, m, t, v_rs, v_cs}, oo{out, n, t, out_rs, out_cs};
  FLK_TRY(check_mat("X1", a, n == 0));
  FLK_TRY(check_mat("X2", b, m == 0));
  FLK_TRY(check_mat("v", vv, m == 0 || t == 0));
  FLK_TRY(check_mat("out", oo, n == 0 || t == 0));
  FLK_TRY(check_sigma(sigma_host, sigma_len, d));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FLK_F32)
    return fmmv_impl<float>(dtype, kernel, a, b, vv, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                            workspace_bytes, flags, st);
  return fmmv_impl<double>(dtype, kernel, a, b, vv, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                           workspace_bytes, flags, st);
}

int flk_fdmmv(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs, const void* X2,
              int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d, const void* v, int64_t v_rs, int64_t v_cs,
              const void* w, int64_t w_rs, int64_t w_cs, int64_t t, void* out, int64_t out_rs, int64_t out_cs,
              const double* sigma_host, int64_t sigma_len, void* workspace, int64_t workspace_bytes, int flags,
              void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, t));
  if (v == nullptr && w == nullptr) return fail(FLK_ERR_BAD_ARG, "One of v and w must be specified to run fdMMV.");
  Mat a{X1, n, d, x1_rs, x1_cs}, b{X2, m, d, x2_rs, x2_cs}, vv{v, m, t, v_rs, v_cs}, ww{w, n, t, w_rs, w_cs},
      oo{out, m, t, out_rs, out_cs};
  FLK_TRY(check_mat("X1", a, n == 0));
  FLK_TRY(check_mat("X2", b, m == 0));
  FLK_TRY(check_mat("v", vv, true));
  FLK_TRY(check_mat("w", ww, true));
  FLK_TRY(check_mat("out", oo, m == 0 || t == 0));
  FLK_TRY(check_sigma(sigma_host, sigma_len, d));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool acc = (flags & FLK_FLAG_ACCUMULATE) != 0;
  if (dtype == FLK_F32)
    return fdmmv_impl<float>(dtype, kernel, a, b, vv, ww, t, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                             workspace_bytes, flags, st, acc);
  return fdmmv_impl<double>(dtype, kernel, a, b, vv, ww, t, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                            workspace_bytes, flags, st, acc);
}


int64_t flk_fmmv_host_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t, int flags) {
  int s = check_common(dtype, kernel, n, m, d, t);
  if (s != FLK_OK) return s;
  int dummy = 0;
  Mat a{&dummy, n, d, d, 1}, b{&dummy, m, d, d, 1}, vv{&dummy, m, t, t, 1}, ww{nullptr, 0, 0, 0, 0},
      oo{&dummy, n, t, t, 1};
  return make_host_layout(nullptr, false, dtype, kernel, a, b, vv, ww, oo, t, flags).total;
}

int64_t flk_fdmmv_host_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t, int flags) {
  int s = check_common(dtype, kernel, n, m, d, t);
  if (s != FLK_OK) return s;
  int dummy = 0;
  Mat a{&dummy, n, d, d, 1}, b{&dummy, m, d, d, 1}, vv{&dummy, m, t, t, 1}, ww{&dummy, n, t, t, 1},
      oo{&dummy, m, t, t, 1};
  return make_host_layout(nullptr, true, dtype, kernel, a, b, vv, ww, oo, t, flags).total;
}

int flk_fmmv_host(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs, const void* X2,
                  int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d, const void* v, int64_t t, int64_t v_rs,
                  int64_t v_cs, void* out, int64_t out_rs, int64_t out_cs, const double* sigma_host,
                  int64_t sigma_len, void* workspace, int64_t workspace_bytes, int flags, void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, t));
  Mat a{X1, n, d, x1_rs, x1_cs}, b{X2, m, d, x2_rs, x2_cs}, vv{v, m, t, v_rs, v_cs}, ww{nullptr, 0, 0, 0, 0},
      oo{out, n, t, out_rs, out_cs};
  FLK_TRY(check_mat("X1", a, n == 0));
  FLK_TRY(check_mat("X2", b, m == 0));
  FLK_TRY(check_mat("v", vv, m == 0 || t == 0));
  FLK_TRY(check_mat("out", oo, n == 0 || t == 0));
  FLK_TRY(check_sigma(sigma_host, sigma_len, d));
  return run_host(false, dtype, kernel, a, b, vv, ww, oo, t, sigma_host, sigma_len, workspace, workspace_bytes, flags,
                  reinterpret_cast<cudaStream_t>(stream));
}

int flk_fdmmv_host(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs, const void* X2,
                   int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d, const void* v, int64_t v_rs, int64_t v_cs,
                   const void* w, int64_t w_rs, int64_t w_cs, int64_t t, void* out, int64_t out_rs, int64_t out_cs,
                   const double* sigma_host, int64_t sigma_len, void* workspace, int64_t workspace_bytes, int flags,
                   void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, t));
  if (v == nullptr && w == nullptr) return fail(FLK_ERR_BAD_ARG, "One of v and w must be specified to run fdMMV.");
  Mat a{X1, n, d, x1_rs, x1_cs}, b{X2, m, d, x2_rs, x2_cs}, vv{v, m, t, v_rs, v_cs}, ww{w, n, t, w_rs, w_cs},
      oo{out, m, t, out_rs, out_cs};
  FLK_TRY(check_mat("X1", a, n == 0));
  FLK_TRY(check_mat("X2", b, m == 0));
  FLK_TRY(check_mat("v", vv, true));
  FLK_TRY(check_mat("w", ww, true));
  FLK_TRY(check_mat("out", oo, m == 0 || t == 0));
  FLK_TRY(check_sigma(sigma_host, sigma_len, d));
  return run_host(true, dtype, kernel, a, b, vv, ww, oo, t, sigma_host, sigma_len, workspace, workspace_bytes, flags,
                  reinterpret_cast<cudaStream_t>(stream));
}

int64_t flk_fmm_workspace_bytes(int dtype, int64_t n, int64_t m, int64_t d, int flags) {
  int s = check_common(dtype, FLK_GAUSSIAN, n, m, d, 0);
  if (s != FLK_OK) return s;
  const int math = (dtype == FLK_F32 && (flags & FLK_FLAG_FP64_MATH)) ? FLK_F64 : dtype;
  return make_fmm_layout(nullptr, math, n, m, d).total;
}

int flk_fmm(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs, const void* X2, int64_t m,
            int64_t x2_rs, int64_t x2_cs, int64_t d, void* out, int64_t out_rs, int64_t out_cs,
            const double* sigma_host, int64_t sigma_len, void* workspace, int64_t workspace_bytes, int flags,
            void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, 0));
  Mat a{X1, n, d, x1_rs, x1_cs}, b{X2, m, d, x2_rs, x2_cs}, oo{out, n, m, out_rs, out_cs};
  FLK_TRY(check_mat("X1", a, n == 0));
  FLK_TRY(check_mat("X2", b, m == 0));
  FLK_TRY(check_mat("out", oo, n == 0 || m == 0));
  FLK_TRY(check_sigma(sigma_host, sigma_len, d));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FLK_F64)
    return fmm_impl<double, double>(FLK_F64, kernel, a, b, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                                    workspace_bytes, st);
  if (flags & FLK_FLAG_FP64_MATH)
    return fmm_impl<double, float>(FLK_F64, kernel, a, b, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                                   workspace_bytes, st);
  return fmm_impl<float, float>(FLK_F32, kernel, a, b, out, out_rs, out_cs, sigma_host, sigma_len, workspace,
                                workspace_bytes, st);
}

int flk_kgrad(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs, const void* X2,
              int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d, const void* G, int64_t g_rs, int64_t g_cs,
              const void* v, int64_t t, int64_t v_rs, int64_t v_cs, void* out, int64_t out_rs, int64_t out_cs,
              const double* sigma_host, int64_t sigma_len, void* workspace, int64_t workspace_bytes, int flags,
              void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, 0));
  if (t < 0 || t > INT32_MAX) return fail(FLK_ERR_BAD_ARG, "t = %lld is out of range", (long long)t);
  if (ceil_div(n, 64) > 65535)
    return fail(FLK_ERR_UNSUPPORTED, "flk_kgrad: n = %lld exceeds 64 * 65535 rows per call; split the rows",
                (long long)n);
  if (t == 0 && v != nullptr)
    return fail(FLK_ERR_BAD_ARG, "v must be NULL when t == 0 (G is then the dense n x m upstream gradient)");
  Mat a{X1, n, d, x1_rs, x1_cs}, b{X2, m, d, x2_rs, x2_cs}, oo{out, n, m, out_rs, out_cs};
  Mat gg{G, n, t > 0 ? t : m, g_rs, g_cs}, vv{v, m, t, v_rs, v_cs};
  FLK_TRY(check_mat("X1", a, n == 0));
  FLK_TRY(check_mat("X2", b, m == 0));
  FLK_TRY(check_mat("G", gg, n == 0 || m == 0));
  FLK_TRY(check_mat("v", vv, t == 0 || m == 0));
  FLK_TRY(check_mat("out", oo, n == 0 || m == 0));
  FLK_TRY(check_sigma(sigma_host, sigma_len, d));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FLK_F64)
    return kgrad_impl<double, double>(FLK_F64, kernel, a, b, gg, vv, t, out, out_rs, out_cs, sigma_host, sigma_len,
                                      workspace, workspace_bytes, st);
  if (flags & FLK_FLAG_FP64_MATH)
    return kgrad_impl<double, float>(FLK_F64, kernel, a, b, gg, vv, t, out, out_rs, out_cs, sigma_host, sigma_len,
                                     workspace, workspace_bytes, st);
  return kgrad_impl<float, float>(FLK_F32, kernel, a, b, gg, vv, t, out, out_rs, out_cs, sigma_host, sigma_len,
                                  workspace, workspace_bytes, st);
}

int flk_set_timing(int enable) {
  g_timer.enabled = enable != 0;
  g_timer.valid[0] = g_timer.valid[1] = false;
  return FLK_OK;
}

int flk_get_sweep_ms(float* sweep1_ms, float* sweep2_ms) {
  if (sweep1_ms == nullptr || sweep2_ms == nullptr) return fail(FLK_ERR_BAD_ARG, "null pointer");
  *sweep1_ms = -1.0f;
  *sweep2_ms = -1.0f;
  if (g_timer.valid[0]) {
    FLK_CUDA_TRY(cudaEventSynchronize(g_timer.ev[1]));
    FLK_CUDA_TRY(cudaEventElapsedTime(sweep1_ms, g_timer.ev[0], g_timer.ev[1]));
  }
  if (g_timer.valid[1]) {
    FLK_CUDA_TRY(cudaEventSynchronize(g_timer.ev[3]));
    FLK_CUDA_TRY(cudaEventElapsedTime(sweep2_ms, g_timer.ev[2], g_timer.ev[3]));
  }
  return FLK_OK;
}

int flk_tc_status(const void* workspace, void* stream, int* status_out) {
  if (workspace == nullptr || status_out == nullptr) return fail(FLK_ERR_BAD_ARG, "null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int host[4] = {0, 0, 0, 0};
  FLK_CUDA_TRY(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, st));
  FLK_CUDA_TRY(cudaStreamSynchronize(st));
  *status_out = host[0];
  return FLK_OK;
}

int flk_range_flag(const void* workspace, void* stream, int* flag_out) {
  if (workspace == nullptr || flag_out == nullptr) return fail(FLK_ERR_BAD_ARG, "null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int host[4] = {0, 0, 0, 0};
  FLK_CUDA_TRY(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, st));
  FLK_CUDA_TRY(cudaStreamSynchronize(st));
  *flag_out = (host[tc::kStatusRange] | host[tc::kStatusRangeX1] | host[tc::kStatusRangeX2]) != 0 ? 1 : 0;
  return FLK_OK;
}

int flk_probe_mufu(int iters, void* sink, int64_t* ops_out, void* stream) {
  if (sink == nullptr || ops_out == nullptr || iters <= 0) return fail(FLK_ERR_BAD_ARG, "bad argument");
  const int blocks = kNumSMs * 4, threads = 512;
  mufu_probe_kernel<<<blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(iters, reinterpret_cast<float*>(sink));
  FLK_CUDA_TRY(cudaGetLastError());
  *ops_out = (int64_t)blocks * threads * 16 * iters;
  return FLK_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// flk_fmmv_static: K(X1, X2) v for callers that have no way to obtain scratch memory.
//
// Who needs this: code that runs where device allocation is off the table -- a plug-in inside a host
// application that handed all device memory to its own pool at start-up (a raw cudaMalloc would fail
// or steal from that pool), or a latency-critical loop that cannot afford the device-wide
// synchronisation cudaMalloc / cudaFree imply and has no allocator handle to pass down.  Such a
// caller cannot supply the workspace flk_fmmv asks for.  Here the workspace is a fixed array that
// is part of the library image itself, so nothing is allocated by anyone at call time.
// ---------------------------------------------------------------------------------------------
namespace flk {

// The scratch array.  It lives in every CUDA context that loads this library, from load until the
// process exits, whether or not the entry point is ever called.
static __device__ __align__(256) unsigned char g_static_scratch[FLK_STATIC_SCRATCH_BYTES];

constexpr int kMaxStaticDevices = 64;
static void* g_static_scratch_addr[kMaxStaticDevices] = {nullptr};
static std::atomic<bool> g_static_scratch_ready[kMaxStaticDevices];

// `g_static_scratch` named in host code is only the host-side handle of the symbol, not a device
// address; the address kernels may use has to be asked for, per device, with that device current.
static int static_scratch_for_current_device(void** out) {
  int dev = 0;
  FLK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxStaticDevices)
    return fail(FLK_ERR_UNSUPPORTED, "flk_fmmv_static supports device ordinals below %d", kMaxStaticDevices);
  if (!g_static_scratch_ready[dev].load(std::memory_order_acquire)) {
    void* ptr = nullptr;
    FLK_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return fail(FLK_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_addr[dev] = ptr;  // same value if two threads race here
    g_static_scratch_ready[dev].store(true, std::memory_order_release);
  }
  *out = g_static_scratch_addr[dev];
  return FLK_OK;
}

}  // namespace flk

extern "C" int flk_fmmv_static(int dtype, int kernel, const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
                               const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d, const void* v,
                               int64_t t, int64_t v_rs, int64_t v_cs, void* out, int64_t out_rs, int64_t out_cs,
                               double sigma, int flags, void* stream) {
  FLK_TRY(check_common(dtype, kernel, n, m, d, t));
  const int64_t need = make_layout(nullptr, false, true, dtype, kernel, n, m, d, t, flags).total;
  if (need > (int64_t)FLK_STATIC_SCRATCH_BYTES)
    return fail(FLK_ERR_WORKSPACE,
                "flk_fmmv_static: this problem needs %lld bytes of scratch but the built-in array holds %lld; "
                "use flk_fmmv with a caller-provided workspace",
                (long long)need, (long long)FLK_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  FLK_TRY(static_scratch_for_current_device(&scratch));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // The array still holds whatever the previous call left.  Everything the kernels read is rewritten
  // by this call's preparation steps except the status word at the front, which must start at zero.
  FLK_CUDA_TRY(cudaMemsetAsync(scratch, 0, 256, st));
  // a scalar length-scale only: staging a per-dimension vector would need a temporary host buffer
  return flk_fmmv(dtype, kernel, X1, n, x1_rs, x1_cs, X2, m, x2_rs, x2_cs, d, v, t, v_rs, v_cs, out, out_rs, out_cs,
                  &sigma, 1, scratch, (int64_t)FLK_STATIC_SCRATCH_BYTES, flags, stream);
}
