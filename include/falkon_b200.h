/*
 * falkon_b200 -- C ABI of the B200 (sm_100a) kernel-vector-product library.
 *
 * This is the drop-in boundary for Falkon's implicit kernel-matrix products.  In the reference
 * these products are Python loops over torch ops plus one native operator (falkon::square_norm);
 * the entry points below are what a binding for this path replaces them with.  Every function
 *   - takes plain pointers, sizes and element strides (no torch types),
 *   - returns FLK_OK (0) or a negative flk_status and never throws, aborts or traps,
 *   - allocates nothing: scratch memory is a caller-provided device workspace whose size comes
 *     from the matching *_workspace_bytes query,
 *   - enqueues its work on the given CUDA stream and returns without synchronising, unless its
 *     description says otherwise (the *_host variants synchronise before returning).
 * A workspace belongs to one call at a time: calls whose GPU work can overlap (different streams, different host
 * threads) need a workspace each.  (The Python layer of this repository keeps ONE workspace per device, so its
 * product calls on a device are meant to come from one thread on one stream.)
 *
 * Matrices are 2-D, described by (pointer, rows, row_stride, col_stride) with strides in
 * elements; one of the two strides must be 1 (C order or Fortran order), as the reference
 * requires (falkon/mmv_ops/utils.py:36-39, falkon/utils/tensor_helpers.py:210-213).
 * X1 is n x d, X2 is m x d, v is m x t, w is n x t.
 *
 * The length-scale `sigma` is a HOST array of doubles of length 1 or d, the form in which the
 * reference keeps it (an fp64 parameter, falkon/kernels/distance_kernel.py:20-38); it is cast to
 * the data type per call exactly as the reference does (distance_kernel.py:148).
 */
#ifndef FALKON_B200_H
#define FALKON_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum flk_status {
  FLK_OK = 0,
  FLK_ERR_BAD_ARG = -1,      /* null pointer, negative size, unknown enum value            */
  FLK_ERR_LAYOUT = -2,       /* neither stride is 1, or a stride is too small / misaligned  */
  FLK_ERR_WORKSPACE = -3,    /* workspace missing, misaligned or smaller than required      */
  FLK_ERR_CUDA = -4,         /* a CUDA runtime call failed; see flk_last_error()            */
  FLK_ERR_UNSUPPORTED = -5,  /* valid request outside what this build implements            */
  FLK_ERR_DEVICE = -6,       /* the current device is not an sm_100 (B200-class) GPU        */
  FLK_ERR_TIMEOUT = -7       /* a bounded device-side wait gave up (tensor-core kernel)     */
} flk_status;

typedef enum flk_dtype { FLK_F32 = 0, FLK_F64 = 1 } flk_dtype;

/* Matern with nu = 0.5 is FLK_LAPLACIAN and nu = inf is FLK_GAUSSIAN, as in
 * falkon/kernels/distance_kernel.py:235-238. */
typedef enum flk_kernel {
  FLK_GAUSSIAN = 0,
  FLK_LAPLACIAN = 1,
  FLK_MATERN15 = 2,
  FLK_MATERN25 = 3
} flk_kernel;

/* Bits of the `flags` argument. */
#define FLK_FLAG_FORCE_SIMT 1 /* never use the tensor-core kernel (diagnostics / comparison) */
#define FLK_FLAG_FORCE_TC 2   /* fail with FLK_ERR_UNSUPPORTED instead of using the SIMT kernel */
#define FLK_FLAG_FP64_MATH 4  /* flk_fmm / flk_kgrad: evaluate fp32 data in fp64, round on store */
#define FLK_FLAG_NO_FOLD 8    /* Gaussian, t = 1, tensor-core path: keep the vector out of the operand images
                                 (the sweep then multiplies by it in its epilogue; diagnostics / comparison) */
#define FLK_FLAG_KEEP_X1 32    /* flk_fmmv / flk_fdmmv (device pointers): the workspace still holds what the previous call
                                 on it prepared from X1 -- that call had the same entry point, sizes, strides, sigma,
                                 kernel and the other flag bits, and X1's contents have not changed since -- so X1 is
                                 not prepared again (its operand images and range check stay resident).  The caller
                                 vouches for all of that; nothing can be verified here.  Ignored by the _host entry
                                 points. */
#define FLK_FLAG_KEEP_X2 64    /* the same for X2 */
#define FLK_FLAG_ACCUMULATE 16 /* flk_fmmv / flk_fdmmv: add the result to what `out` holds instead of overwriting it
                                 (chunks of the reduction side are summed this way under a memory budget) */

/* Library version (major * 10000 + minor * 100 + patch). */
int flk_version(void);

/* Message describing the last failure on the calling thread (empty string if none). */
const char* flk_last_error(void);

/* Name of a status code. */
const char* flk_status_name(int status);

/* FLK_OK when the current CUDA device can run this library (compute capability 10.x). */
int flk_check_device(void);

/* 1 when a tcgen05 tensor-core kernel serves this problem (fp32 data, 1 <= d <= 1024), 0 when the SIMT / fp64
 * kernels do. */
int flk_uses_tensor_cores(int dtype, int kernel, int64_t d, int64_t t, int flags);

/*
 * Row-wise squared norms of X / sigma:  out[i] = sum_k (X[i,k] / sigma)^2 , out has n entries, summed in
 * column order in the data's own precision (as the reference accumulates).
 * Replaces falkon::square_norm as the distance kernels call it
 * (falkon/c_ext/ops/square_norm.cpp:23-26, CUDA falkon/c_ext/ops/cuda/cuda_square_norm.cu:48-61; call
 * sites falkon/kernels/distance_kernel.py:153-154).  X is a DEVICE pointer in either memory order.
 * sigma_host may be NULL (no scaling) or point at ONE length-scale (sigma_len = 1): the reference's
 * routine takes no scaling at all, the scalar is a convenience.  A per-dimension vector (sigma_len = d
 * > 1) is refused with FLK_ERR_UNSUPPORTED: the call has no workspace to stage it in; scale the data
 * first, or use the products, which take the vector.  Needs no workspace.
 */
int flk_square_norm(int dtype, const void* X, int64_t n, int64_t d, int64_t x_rs, int64_t x_cs,
                    const double* sigma_host, int64_t sigma_len, void* out, void* stream);

/* Device workspace needed by flk_fmmv for these sizes, in bytes (negative flk_status on error). */
int64_t flk_fmmv_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t,
                                 int flags);

/*
 * out[n x t] = k(X1, X2) v                                   (all pointers are DEVICE pointers)
 * Replaces fmmv / KernelMmvFnFull.forward / mmv_run_thread
 * (falkon/mmv_ops/fmmv.py:960-973, :887-932, :309-402) for dense inputs.  The n x m kernel block
 * is never written to memory.  Either of n, m may be the large dimension: with n small and m
 * large this is the reduction over data rows that the CG right-hand side needs
 * (falkon/optim/conjgrad.py:296).
 */
int flk_fmmv(int dtype, int kernel,
             const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
             const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs,
             int64_t d,
             const void* v, int64_t t, int64_t v_rs, int64_t v_cs,
             void* out, int64_t out_rs, int64_t out_cs,
             const double* sigma_host, int64_t sigma_len,
             void* workspace, int64_t workspace_bytes, int flags, void* stream);

/* Device workspace needed by flk_fdmmv for these sizes, in bytes (negative flk_status on error). */
int64_t flk_fdmmv_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d, int64_t t,
                                  int flags);

/*
 * out[m x t] = k(X1, X2)^T ( k(X1, X2) v + w )               (all pointers are DEVICE pointers)
 * Replaces fdmmv / dmmv_run_thread (falkon/mmv_ops/fmmv.py:976-1131, :683-767) for dense inputs.
 * w may be NULL (treated as zero, fmmv.py:753); v may be NULL (out = k^T w, the contract of
 * falkon/kernels/kernel.py:350-353); at least one of them must be given.
 */
int flk_fdmmv(int dtype, int kernel,
              const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
              const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs,
              int64_t d,
              const void* v, int64_t v_rs, int64_t v_cs,
              const void* w, int64_t w_rs, int64_t w_cs,
              int64_t t,
              void* out, int64_t out_rs, int64_t out_cs,
              const double* sigma_host, int64_t sigma_len,
              void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * Host-buffer variants: X1, X2, v, w and out are HOST pointers (pinned memory gives asynchronous
 * copies; pageable memory works too).  The inputs are staged into the device workspace, the
 * device entry point above runs, and the result is copied back; the call returns after the
 * stream has been synchronised, so `out` is valid on return.  This is the reference's
 * "data on the CPU, compute on the GPU" case (falkon/mmv_ops/fmmv.py:798-854, :1080-1125)
 * for one GPU.  The workspace must hold flk_*_host_workspace_bytes bytes of DEVICE memory.
 *
 * From 262,144 rows up, X1 (and w) travel in up to four row chunks through a copy stream that
 * the library creates once per device (with a handful of events) and keeps: the copy of chunk
 * c + 1 overlaps the kernels of chunk c on the caller's stream; fdmmv sums the per-chunk results
 * in a fixed order (bit-reproducible, but not bit-identical to the one-piece device call).
 * Not for concurrent calls from several host threads on one device.
 */
int64_t flk_fmmv_host_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d,
                                      int64_t t, int flags);
int flk_fmmv_host(int dtype, int kernel,
                  const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
                  const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs,
                  int64_t d,
                  const void* v, int64_t t, int64_t v_rs, int64_t v_cs,
                  void* out, int64_t out_rs, int64_t out_cs,
                  const double* sigma_host, int64_t sigma_len,
                  void* workspace, int64_t workspace_bytes, int flags, void* stream);

int64_t flk_fdmmv_host_workspace_bytes(int dtype, int kernel, int64_t n, int64_t m, int64_t d,
                                       int64_t t, int flags);
int flk_fdmmv_host(int dtype, int kernel,
                   const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
                   const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs,
                   int64_t d,
                   const void* v, int64_t v_rs, int64_t v_cs,
                   const void* w, int64_t w_rs, int64_t w_cs,
                   int64_t t,
                   void* out, int64_t out_rs, int64_t out_cs,
                   const double* sigma_host, int64_t sigma_len,
                   void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * flk_fmmv_static: out[n x t] = k(X1, X2) v without any workspace argument.  (No counterpart in the
 * reference: it exists for embedders, not for parity.)
 *
 * For callers that cannot allocate device memory and therefore cannot give flk_fmmv its workspace:
 * a plug-in whose host application took all device memory into its own pool at start-up, or a
 * real-time loop that must never run into the device-wide synchronisation of cudaMalloc / cudaFree.
 * The scratch memory is a fixed array of FLK_STATIC_SCRATCH_BYTES compiled into the library; each
 * GPU context that loads the library carries it until the process exits.  The call itself performs no
 * cudaMalloc / cudaFree and calls no allocating routine.  Inputs and output are DEVICE pointers owned
 * by the caller, exactly as for flk_fmmv; the length-scale is one scalar.
 *
 * Limits and rules:
 *  - the problem must fit: flk_fmmv_workspace_bytes(dtype, kernel, n, m, d, t, flags) must not exceed
 *    FLK_STATIC_SCRATCH_BYTES, otherwise FLK_ERR_WORKSPACE is returned with a message and nothing runs
 *    (fp32 Gaussian, d = 28, t = 1: about 200,000 rows of X1 and X2 together);
 *  - the first call on each device looks up the array's device address (the device must be current);
 *    make that first call outside any stream capture;
 *  - all calls share the one array: two calls whose GPU work can overlap (different streams, or
 *    different host threads on one device) race on it and corrupt each other.  Calls issued to one
 *    stream are safe.  The array keeps the previous call's contents; the entry point re-zeroes the
 *    part that has to start at zero.
 */
#define FLK_STATIC_SCRATCH_BYTES (64ll << 20)
int flk_fmmv_static(int dtype, int kernel,
                    const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
                    const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs,
                    int64_t d,
                    const void* v, int64_t t, int64_t v_rs, int64_t v_cs,
                    void* out, int64_t out_rs, int64_t out_cs,
                    double sigma, int flags, void* stream);

/*
 * Kernel matrix  out[n x m] = k(X1, X2)  (the reference's fmm, falkon/mmv_ops/fmm.py:298-388, which
 * the preconditioner calls once per fit on the centres, falkon/preconditioner/flk_preconditioner.py:89).
 * `out` has the data's dtype and either memory order.  With FLK_FLAG_FP64_MATH fp32 data is
 * evaluated in fp64 and rounded once on store -- the reference's `no_single_kernel` default
 * (falkon/mmv_ops/fmm.py:619-622), which keeps the Cholesky factorisations that follow stable.
 */
int64_t flk_fmm_workspace_bytes(int dtype, int64_t n, int64_t m, int64_t d, int flags);
int flk_fmm(int dtype, int kernel,
            const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
            const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d,
            void* out, int64_t out_rs, int64_t out_cs,
            const double* sigma_host, int64_t sigma_len,
            void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * Pair weights of the backward pass (device pointers; workspace as for flk_fmm):
 *     out[i][j] = 2 k'(D2_ij) * s_ij ,   k' = dk / dD2 at the squared distance of the sigma-scaled rows,
 *     s_ij = sum_c G[i][c] v[j][c]  (t > 0: G is n x t, v is m x t -- the backward pass of k(X1, X2) v)
 *     s_ij = G[i][j]                (t == 0, v == NULL: G is n x m -- the backward pass of k(X1, X2)).
 * Every gradient that the reference obtains by re-running its block product under autograd
 * (mmv_diff_run_thread, falkon/mmv_ops/fmmv.py:405-485; KernelMmFnFull.backward in falkon/mmv_ops/fmm.py)
 * is a matrix product with this n x m block: with W = out, a = W 1, b = W^T 1 and X~ = X / sigma,
 *     dL/dX1~ = a o X1~ - W X2~ ,  dL/dX2~ = b o X2~ - W^T X1~ ,
 *     dL/dsigma_k = -(1 / sigma_k) sum_ij W_ij (x~_ik - c~_jk)^2 .
 * Entries whose squared distance the forward pass clamps at 1e-20 get weight zero.  The caller splits
 * rows into blocks of at most 64 * 65535.
 */
int flk_kgrad(int dtype, int kernel,
              const void* X1, int64_t n, int64_t x1_rs, int64_t x1_cs,
              const void* X2, int64_t m, int64_t x2_rs, int64_t x2_cs, int64_t d,
              const void* G, int64_t g_rs, int64_t g_cs,
              const void* v, int64_t t, int64_t v_rs, int64_t v_cs,
              void* out, int64_t out_rs, int64_t out_cs,
              const double* sigma_host, int64_t sigma_len,
              void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * Counters for the calling process: number of kernels this library has launched and the status
 * word of the last tensor-core launch read back by flk_tc_status (0 = clean).
 */
int64_t flk_launch_count(void);

/*
 * Optional timing of the dominant kernels, for benchmarking.  After flk_set_timing(1) every
 * fmmv / fdmmv call records CUDA events on its stream around its first sweep (K v) and, for
 * fdmmv, its second sweep (K^T u).  flk_get_sweep_ms waits for those events and returns the two
 * durations of the most recent call in milliseconds (-1 where no such sweep ran).  One set of
 * events per process: not for concurrent use from several threads.
 */
int flk_set_timing(int enable);
int flk_get_sweep_ms(float* sweep1_ms, float* sweep2_ms);

/*
 * Reads the device-side status word that the tensor-core kernel sets when one of its bounded
 * waits gives up (a barrier that never completed).  Synchronises the stream.  0 = clean; any
 * other value encodes which wait ran out.  `workspace` is the workspace of the call to check.
 */
int flk_tc_status(const void* workspace, void* stream, int* status_out);

/*
 * Reads the device-side range flag of the call that last used `workspace`: 1 when the operand
 * images of the tensor-core path could not carry some row (scaled squared norm beyond fp16 range)
 * and the SIMT kernels produced the result instead, 0 otherwise.  Synchronises the stream.
 */
int flk_range_flag(const void* workspace, void* stream, int* flag_out);

/*
 * Measurement aid (no counterpart in the reference): enqueues a kernel that does nothing but
 * `iters` x 16 independent ex2.approx per thread on every SM, so that a benchmark can time it with
 * CUDA events and obtain the MUFU (special-function unit) rate of the device it runs on -- the
 * denominator of the roofline of the Gaussian sweep.  `*ops_out` receives the number of ex2
 * evaluations the launch performs.  `sink` is a device buffer of at least 4 bytes.
 */
int flk_probe_mufu(int iters, void* sink, int64_t* ops_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FALKON_B200_H */
