/*
 * xcorr.h -- C ABI of the B200 (sm_100a) direct 2-D cross-correlation library.
 *
 * The reference project has no FFI layer; its seam is the C++ launcher API declared in
 * repo/cross-corr/src/kernels.cuh:41-283 (free function templates `run_*<float,float>`
 * taking caller-owned device pointers, a matrix size, a search size, matrix counts,
 * tuning integers and sometimes a stream) and, one level up, the per-mode algorithm
 * classes of one_to_one.hpp / one_to_many.hpp / n_to_mn.hpp / n_to_m.hpp.  Every entry
 * point below names the reference interface it stands in for.
 *
 * Conventions shared by all entry points
 *   - float32, row-major, matrices of one array stacked contiguously
 *     (repo/cross-corr/src/matrix.hpp:410-619, data_array).
 *   - `left` is the reference's "ref", `right` its "target"/"deformed".
 *   - out[(sy + rows-1) * (2*cols-1) + (sx + cols-1)] =
 *         sum over the overlap of left[y+sy][x+sx] * right[y][x]
 *     for sx in [-(cols-1), cols-1], sy in [-(rows-1), rows-1]
 *     (repo/cross-corr/src/validate.hpp:95-132); one (2*rows-1) x (2*cols-1) result per pair.
 *   - Device entry points: pointers are device pointers owned by the caller; nothing is
 *     allocated, freed or retained; the launch is asynchronous on `stream` (a
 *     cudaStream_t passed as void*, NULL = legacy default stream) and does not
 *     synchronise.  Unlike the reference launchers, which throw std::runtime_error
 *     (e.g. naive_shuffle_multirow_both.cu:645-665), errors come back as a status
 *     code; nothing is thrown across this boundary.
 *   - Result order (validate.hpp:230-291):
 *       one_to_many  out[t]                left 0 with right t
 *       n_to_m       out[l * n_right + t]  left l with right t
 *       n_to_mn      GROUPED order: right and out matrix l*m + t belong to left l,
 *                    m = n_right / n_left.  This is the in-memory order the reference's
 *                    GPU algorithms use after load_interleaved_from_csv
 *                    (matrix.hpp:484-503); files hold the order t*n_left + l, and
 *                    xcorr_n_to_mn_reorder_f32 converts between the two.
 */
#ifndef XCORR_H
#define XCORR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define XCORR_API
#else
#define XCORR_API __attribute__((visibility("default")))
#endif

typedef enum xcorr_status {
    XCORR_OK = 0,
    XCORR_ERR_NULL_POINTER = 1,      /* a required pointer is NULL */
    XCORR_ERR_INVALID_SIZE = 2,      /* zero rows/cols/counts, n_right % n_left != 0, overflow of uint32 indexing */
    XCORR_ERR_INVALID_HINT = 3,      /* a tuning value outside the supported range */
    XCORR_ERR_WORKSPACE = 4,         /* workspace missing or smaller than xcorr_workspace_bytes() */
    XCORR_ERR_CUDA = 5,              /* a CUDA runtime call failed; see xcorr_last_error_string() */
    XCORR_ERR_UNSUPPORTED = 6,       /* shape needs more shared memory than one SM has */
    XCORR_ERR_DEVICE = 7,            /* bad device index / no usable device for the sharded runner */
    XCORR_ERR_TIMEOUT = 8,           /* a bounded device-side wait gave up */
    XCORR_ERR_INTERNAL = 9           /* host-side failure inside the library (out of host memory, a thread
                                        could not be started): caught at this boundary, never thrown across it */
} xcorr_status;

typedef enum xcorr_mode {
    XCORR_ONE_TO_ONE = 0,
    XCORR_ONE_TO_MANY = 1,
    XCORR_N_TO_MN = 2,
    XCORR_N_TO_M = 3
} xcorr_mode;

/* Kernel families.  The first three mirror the reference's algorithm families; which
 * registry names map to which family is the host program's business. */
typedef enum xcorr_kernel {
    XCORR_KERNEL_AUTO = 0,          /* per-shape selection */
    XCORR_KERNEL_TILE = 1,          /* register-tiled circular-class kernel (the fast path) */
    XCORR_KERNEL_OVERLAP_WISE = 2,  /* one thread per overlap -- run_cross_corr_naive_original, naive_original.cu:131-161 */
    XCORR_KERNEL_WARP_PER_OVERLAP = 3, /* one warp per overlap -- run_ccn_warp_per_shift, naive_warp_per_shift.cu:308-335.
                                       The automatic choice for a handful of small overlaps (at most 8000 in the
                                       call, rows and columns up to 32: a 16 x 16 or 32 x 32 pair) */
    XCORR_KERNEL_FFT = 4,           /* the cuFFT path (xcorr_fft_f32 with the normalized layout); needs the
                                       workspace xcorr_workspace_bytes() reports for this hint.  Never chosen
                                       automatically: its rounding differs from the direct path's */
    XCORR_KERNEL_WARP_STAGED = 5    /* one warp per overlap, operands staged through shared memory --
                                       run_ccn_warp_per_shift_shared_mem, naive_warp_per_shift_shared_mem.cu:392-496 */
} xcorr_kernel;

/* How the rows of one overlap are shared by several warps of the plain warp-per-overlap kernel
 * (row_distribution.cuh:34-284; the sums are added atomically onto the output, which the library
 * zeroes first). */
typedef enum xcorr_row_split {
    XCORR_SPLIT_NONE = 0,        /* one warp per overlap */
    XCORR_SPLIT_RECTANGLE = 1,   /* every output row gets the worker slots of the centre row; surplus ones return */
    XCORR_SPLIT_TRIANGLE = 2     /* exactly the workers each output row needs */
} xcorr_row_split;

/* How partial sums of a row-split launch are combined (the reference's "work
 * distribution" kernels always use atomicAdd on a caller-zeroed buffer,
 * naive_shuffle.cu:307-413, one_to_one.hpp:277). */
typedef enum xcorr_combine {
    XCORR_COMBINE_AUTO = 0,
    XCORR_COMBINE_STORE = 1,     /* no row split; each output written once */
    XCORR_COMBINE_ATOMIC = 2,    /* the library zeroes `out`, then red.global.add.f32 */
    XCORR_COMBINE_WORKSPACE = 3  /* partial images in the workspace + fixed-order reduction: bit-reproducible */
} xcorr_combine;

/* Tuning hints; all zero (or a NULL pointer) = automatic.  These replace the reference's
 * per-algorithm JSON keys (warps_per_thread_block, shifts_per_thread,
 * left_rows_per_iteration, right_matrices_per_thread, rows_per_thread, ...), which the
 * reference bakes into template instantiations. */
typedef struct xcorr_hints {
    int32_t kernel;            /* xcorr_kernel */
    int32_t combine;           /* xcorr_combine */
    int32_t overlap_rows;      /* TILE: y-overlap classes per thread, 1..4 (cf. shifts_per_thread) */
    int32_t class_lanes;       /* TILE: lanes of a warp spread over y-classes: 1,2,4,8,16,32; the
                                  other 32/class_lanes lanes take different right matrices
                                  (cf. right_matrices_per_thread) */
    int32_t warps_x;           /* TILE: warps of a block along x-class tiles (cf. warps_per_thread_block) */
    int32_t warps_y;           /* TILE: warps of a block along y-class groups */
    int32_t row_slices;        /* TILE: number of slices the right rows are split into (cf. rows_per_thread) */
    int32_t block_threads;     /* OVERLAP_WISE / WARP_PER_OVERLAP / WARP_STAGED: threads per block; for the two
                                  warp families 32 * shifts_per_thread_block (a warp per overlap) */
    int32_t schedule;          /* TILE: how work reaches the blocks.  0 auto;
                                  1 static: one block per block task (and row slice);
                                  2 stream-K: the (block task, right row) units of all tasks are cut evenly
                                    over one resident wave of blocks; a block works on whole tasks (plain
                                    stores) and at most two partial ones, which it adds atomically onto
                                    the zeroed output.  Two parts of a task commute; a task in more than
                                    two parts makes the last bits of a result vary between runs, as with
                                    the reference's atomicAdd "work distribution" kernels.  With
                                    combine = workspace the parts go to partial images instead and the
                                    block that finishes a task's last part sums them in the fixed order of
                                    their rows: bit-reproducible for any number of parts, a few percent
                                    slower;
                                  3 warp queue: the warp tasks (one 16-wide x tile and one y group of one
                                    matrix group, all rows) are cut evenly over one resident wave of
                                    blocks whose warps take them from a shared counter: plain stores,
                                    bit-reproducible, balanced to one warp task per SM */
    int32_t host_chunks;       /* host-buffer entry points only: number of pieces the independent result
                                  matrices are cut into so that the input copy, the kernel and the result
                                  copy of successive pieces overlap.  0 auto (by result size, 1..8);
                                  1 one piece (copy in, run, copy out) */
    int32_t reproducible;      /* TILE: 1 = only plans whose results are bit-identical from run to run (no
                                  sum of more than two atomically added parts); 0 = the fastest plan, which
                                  for small inputs may add many parts atomically, like the reference's
                                  "work distribution" kernels.  The environment variable
                                  XCORR_REPRODUCIBLE=1 sets it for every call of the process */
    int32_t rows_per_warp;     /* WARP_PER_OVERLAP with row_split != 0: most rows of an overlap one warp sums
                                  (cf. rows_per_warp of nai_warp_per_shift_work_distribution_one_to_one) */
    int32_t row_split;         /* WARP_PER_OVERLAP: xcorr_row_split (cf. distribution_type) */
    int32_t staged_rows;       /* WARP_STAGED: right rows per shared-memory slab (cf. shared_mem_rows); 0 auto */
    int32_t staged_cols;       /* WARP_STAGED: columns per slab (cf. shared_mem_row_size); 0 auto */
    int32_t staged_rights;     /* WARP_STAGED: right matrices a block takes together, 1..8
                                  (cf. right_matrices_per_block); 0 auto */
    int32_t staged_column_groups; /* WARP_STAGED: 1 = every column slab is a block of its own and the sums are
                                  added atomically onto the zeroed output (cf. column_group_per_block) */
    int32_t staged_warp_rows;  /* WARP_STAGED: how the slab is copied: 0 = the block's threads stride over its
                                  elements, 1 = one warp per row (cf. strided_load = true / false) */
    int32_t fused_rows;        /* TILE: rows of 17..32 columns with 1 y class per thread can run both passes
                                  fused, the right row held in registers.  0 auto (fused), 1 on, 2 off */
    int32_t reserved[1];
} xcorr_hints;

/* ---- device-pointer entry points ------------------------------------------------------
 * One per input mode.  They stand in for the reference launchers the mode's algorithm
 * classes call:
 *   one_to_one   run_ccn_shuffle_multirow_both            kernels.cuh:191-201 (one_to_one.hpp:755)
 *   one_to_many  run_ccn_shuffle_one_to_many_multirow_both_multimat_right
 *                                                          kernels.cuh:227-240 (one_to_many.hpp:379)
 *   n_to_mn      the same launcher once per left matrix on round-robin streams
 *                                                          (n_to_mn.hpp:553-571)
 *   n_to_m       run_ccn_n_to_m_shuffle_multirow_both_multimat_both
 *                                                          kernels.cuh:242-256 (n_to_m.hpp:495)
 * and, through hints->kernel, for run_cross_corr_naive_original (kernels.cuh:41-51) and
 * run_ccn_warp_per_shift (kernels.cuh:98-106).  The search size is always the full
 * (2*cols-1, 2*rows-1), which is what every reference caller passes.
 * `workspace` may be NULL unless the chosen plan combines through the workspace
 * (see xcorr_workspace_bytes); it must be 16-byte aligned (any cudaMalloc pointer is). */
XCORR_API xcorr_status xcorr_one_to_one_f32(const float* d_left, const float* d_right, float* d_out,
                                            uint32_t rows, uint32_t cols,
                                            const xcorr_hints* hints,
                                            void* d_workspace, size_t workspace_bytes, void* stream);

XCORR_API xcorr_status xcorr_one_to_many_f32(const float* d_left, const float* d_right, float* d_out,
                                             uint32_t rows, uint32_t cols, uint32_t n_right,
                                             const xcorr_hints* hints,
                                             void* d_workspace, size_t workspace_bytes, void* stream);

XCORR_API xcorr_status xcorr_n_to_mn_f32(const float* d_left, const float* d_right, float* d_out,
                                         uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                         const xcorr_hints* hints,
                                         void* d_workspace, size_t workspace_bytes, void* stream);

XCORR_API xcorr_status xcorr_n_to_m_f32(const float* d_left, const float* d_right, float* d_out,
                                        uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                        const xcorr_hints* hints,
                                        void* d_workspace, size_t workspace_bytes, void* stream);

/* One pair without any allocation.  (No counterpart in the reference: its algorithm classes
 * always allocate their device buffers themselves, one_to_one.hpp:112-118.)
 *
 * For callers that must not, or cannot, call cudaMalloc at the point where they need a result:
 * code running inside a real-time or latency-critical loop, a plug-in whose host forbids device
 * allocation after start-up, a process whose memory pool is owned by another runtime.  The single
 * 256x256-sized pair is the case that needs scratch memory at all (its rows are divided over
 * all SMs and the partial results are summed afterwards, see xcorr_workspace_bytes); this entry
 * point runs exactly that path with the partial results in an array that is part of the library
 * image instead of a caller-provided workspace.
 *
 *  - The array holds xcorr_noalloc_scratch_bytes() = 32 MiB and exists on every GPU that loads the
 *    library, from load to process exit, whether this entry point is used or not.
 *  - Size limit: the result must fit the array once, (2*rows-1)*(2*cols-1) <= 8 Mi floats (square
 *    inputs up to 1448 x 1448).  Larger inputs are refused with XCORR_ERR_UNSUPPORTED and a message
 *    that names the limit.
 *  - Within the limit there are two ways the partial results are combined.  Inputs whose row
 *    slices fit the array AND one SM's shared memory (square inputs up to about 448 x 448) are
 *    summed through the array in a fixed order: bit-reproducible.  Larger ones need more, finer
 *    slices than the array holds; they are added onto the zeroed result with atomic adds instead
 *    (cudaMemsetAsync + red.global.add, still nothing allocated): the last bits of such a result
 *    can differ from run to run.  Inputs too wide for any slice (more than about 1700 columns)
 *    take the overlap-wise kernel, which needs no scratch.  xcorr_last_launch_string() says which.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
 *    keeps it; make that first call before any stream capture starts on the device.  The address
 *    belongs to the device's context: after cudaDeviceReset (or any teardown of the primary
 *    context) call xcorr_release_host_cache(), which also forgets the kept addresses.
 *  - All calls share the array, and it keeps what the last call left in it.  Nothing has to be
 *    cleared between calls -- every word the summation reads was written earlier in the same
 *    call -- but two calls that overlap on one GPU (different streams, different threads) race on
 *    it: issue them on one stream or otherwise order them.
 *  - Calls no cudaMalloc / cudaFree and no allocating library routine; asynchronous on `stream`
 *    like the other device entry points; the result equals xcorr_one_to_one_f32 up to the float
 *    rounding of a possibly different number of row slices. */
XCORR_API xcorr_status xcorr_one_to_one_noalloc_f32(const float* d_left, const float* d_right, float* d_out,
                                                    uint32_t rows, uint32_t cols, void* stream);
XCORR_API size_t xcorr_noalloc_scratch_bytes(void);

/* Mode-generic form of the four above (same contract). */
XCORR_API xcorr_status xcorr_run_f32(int32_t mode, const float* d_left, const float* d_right, float* d_out,
                                     uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                     const xcorr_hints* hints,
                                     void* d_workspace, size_t workspace_bytes, void* stream);

/* Bytes of workspace the plan chosen for this shape and these hints needs (0 when it
 * needs none).  Replaces the reference's convention that callers of the atomic variants
 * zero the output themselves (one_to_one.hpp:277, :503). */
XCORR_API size_t xcorr_workspace_bytes(int32_t mode, uint32_t rows, uint32_t cols,
                                       uint32_t n_left, uint32_t n_right, const xcorr_hints* hints);

/* Text form of the launch plan this shape and these hints would get (the same text
 * xcorr_last_launch_string reports after a launch); needs no device -- without one a B200
 * (148 SMs, 227 KB shared memory per block) is assumed.  Returns an xcorr_status. */
XCORR_API int32_t xcorr_describe_plan(int32_t mode, uint32_t rows, uint32_t cols,
                                      uint32_t n_left, uint32_t n_right, const xcorr_hints* hints,
                                      char* buffer, size_t buffer_bytes);

/* Number of result matrices of a mode (validate.hpp:214-291 check_num_result_matrices). */
XCORR_API uint64_t xcorr_num_results(int32_t mode, uint32_t n_left, uint32_t n_right);

/* `cross input` shape rules: one_to_one.hpp:20-22, one_to_many.hpp:15-17,
 * n_to_mn.hpp:23-25, n_to_m.hpp:19-21.  Returns 1 for valid, 0 for invalid. */
XCORR_API int32_t xcorr_validate_input_size(int32_t mode, uint32_t rows, uint32_t cols,
                                            uint32_t n_left, uint32_t n_right);

/* ---- FFT path ---------------------------------------------------------------------------
 * The same four modes through cuFFT: zero padding to 2*rows x 2*cols on the device, one batched
 * real-to-complex transform of all inputs, spectrum products left * conj(right), one batched
 * complex-to-real transform of all pairs, unpacking.  Stands in for the reference's
 * fft_original_alg_* / fft_reduced_transfer_* classes (one_to_one.hpp:888-1170,
 * one_to_many.hpp:502-780, n_to_mn.hpp:720-1000), fft_better_hadamard_alg_n_to_m
 * (n_to_m.hpp:647-800) and their kernels run_hadamard_original / run_hadamard_n_to_m_over_*
 * (kernels.cuh, hadamard.cu) and run_scatter (scatter.cu).  Inputs, pair order and stream
 * semantics as for the direct entry points.  Float rounding differs from the direct path
 * (about 1e-6 of the largest result at the benchmark sizes).
 * layout XCORR_FFT_NORMALIZED: `d_out` gets the direct path's result layout,
 *   (2*rows-1) x (2*cols-1) per pair, scaled (fft_helpers.hpp:213-262 normalize_fft_results,
 *   done on the host there).
 * layout XCORR_FFT_RAW: `d_out` gets 2*rows x 2*cols per pair exactly as the inverse transform
 *   leaves it -- shift (sy, sx) at row sy mod 2*rows, column sx mod 2*cols, times 4*rows*cols:
 *   what the reference's fft classes hold in results() and write without --normalize.
 * The workspace (xcorr_fft_workspace_bytes) is required.  cuFFT plans are created on first use
 * of a (device, size, batch) and cached; xcorr_fft_release_plans() destroys them.  A cached plan
 * owns one cuFFT work area: calls of the same shape on the same device must be ordered on one
 * stream (or otherwise not overlap on the GPU) -- unlike the direct entry points, which may run
 * concurrently on different streams with their own workspaces. */
typedef enum xcorr_fft_layout { XCORR_FFT_NORMALIZED = 0, XCORR_FFT_RAW = 1 } xcorr_fft_layout;

XCORR_API size_t xcorr_fft_workspace_bytes(int32_t mode, uint32_t rows, uint32_t cols,
                                           uint32_t n_left, uint32_t n_right, int32_t layout);
XCORR_API xcorr_status xcorr_fft_f32(int32_t mode, const float* d_left, const float* d_right, float* d_out,
                                     uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                     int32_t layout, void* d_workspace, size_t workspace_bytes, void* stream);
XCORR_API void xcorr_fft_release_plans(void);

/* ---- host-buffer entry points -----------------------------------------------------------
 * The reference's whole computation step for one algorithm object: prepare (cudaMalloc),
 * transfer (H2D), run, finalize (D2H), free -- main.cpp:123-174, one_to_one.hpp:112-135 and
 * the other modes' naive_gpu_* classes.  Host pointers in, host result out; synchronous.
 * Device buffers are cached per device and reused across calls; the caller's current device
 * is the same after the call as before it.  n_to_mn takes and returns GROUPED order like the
 * device entry point.
 * Results of more than a few MB are produced in pieces (blocks of right matrices for
 * one_to_many, of left matrices for n_to_m / n_to_mn; hints->host_chunks) on three streams,
 * so that the result copy of one piece runs under the kernel of the next and the input copy
 * of the one after; this needs page-locked host buffers to take effect (pageable ones work,
 * without overlap).  The reference copies, runs and copies back in sequence
 * (cross_corr.hpp:32-72 "Compute" steps). */
XCORR_API xcorr_status xcorr_run_host_f32(int32_t mode, const float* h_left, const float* h_right, float* h_out,
                                          uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                          const xcorr_hints* hints, int32_t device);

/* ---- double precision ----------------------------------------------------------------------
 * The reference parses `--data_type double` and refuses it (main.cpp:433-434); its <double>
 * kernel instantiations are commented out (e.g. naive_shuffle.cu:545-552).  Same modes,
 * layouts (n_to_mn GROUPED) and definition as the float entry points; no workspace, no
 * hints.  The kernel is register-tiled like the float one (circular classes in both directions,
 * operands staged in shared memory; 8 x classes of one y class per thread, double accumulation).
 * Plans that keep every result in one block write with plain stores in a fixed order:
 * bit-reproducible.  Where rows are cut into slices (few pairs, e.g. one 256 x 256 pair: every
 * SM gets a slice) the library zeroes `d_out` and the slices add atomically: two slices commute,
 * more make the last bits vary from run to run; the environment variable XCORR_REPRODUCIBLE=1
 * keeps to at most two slices (and to the second kernel where that does not fit), at the price
 * of idle SMs on single large pairs.  xcorr_last_launch_string() names the plan.
 * Rows too wide to stage take a second kernel (a warp per 8 x 32 block of a result, operands
 * through L1), which the environment variable XCORR_F64_STRIP=1 selects for every call.
 * A handful of small overlaps (at most 8000, rows and columns up to 32) runs on the
 * warp-per-overlap latency kernel, as in single precision.
 * Asynchronous on `stream`. */
XCORR_API xcorr_status xcorr_run_f64(int32_t mode, const double* d_left, const double* d_right, double* d_out,
                                     uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                     void* stream);

/* Host pointers in, host result out (allocate, copy, run, copy back, free); synchronous. */
XCORR_API xcorr_status xcorr_run_host_f64(int32_t mode, const double* h_left, const double* h_right, double* h_out,
                                          uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                          int32_t device);

/* Several problems in one call.  The reference runs its algorithm objects one after the other,
 * each through prepare / transfer / run / finalize (main.cpp:123-174; benchmark.py starts one
 * process per input): a result copy that has to end before the next problem's input copy
 * starts.  Here the problems of a batch share the three streams of the host-buffer path, so
 * the input copy and the kernels of problem k+1 run under the result copy of problem k and
 * the device -> host link stays busy from the first result to the last.  Every job is what
 * one xcorr_run_host_f32 call takes; results are bit-identical to separate calls.  The
 * call returns when every result is in its h_out; the first job that fails ends the batch
 * with its status (results of earlier jobs are complete). */
typedef struct xcorr_host_job {
    int32_t mode;                 /* xcorr_mode */
    uint32_t rows, cols;
    uint32_t n_left, n_right;
    const float* h_left;
    const float* h_right;
    float* h_out;
    const xcorr_hints* hints;     /* NULL = automatic */
} xcorr_host_job;

XCORR_API xcorr_status xcorr_run_host_batch_f32(const xcorr_host_job* jobs, int32_t n_jobs, int32_t device);

/* Same, with the independent result matrices sharded over `n_devices` GPUs of this
 * process (devices[i] are CUDA device indices; NULL = 0..n_devices-1): right matrices for
 * one_to_many, left matrices for n_to_m and n_to_mn (each with all / its own rights), the
 * other operand replicated; one host thread and stream per GPU, no collective.  one_to_one
 * runs on devices[0].  The reference has no multi-GPU path; this extends the stream
 * fan-out of n_to_mn.hpp:329-348 / n_to_m.hpp:293-312 across devices. */
XCORR_API xcorr_status xcorr_run_host_sharded_f32(int32_t mode, const float* h_left, const float* h_right,
                                                  float* h_out, uint32_t rows, uint32_t cols,
                                                  uint32_t n_left, uint32_t n_right,
                                                  const xcorr_hints* hints,
                                                  const int32_t* devices, int32_t n_devices);

/* The shard of units (right matrices or left matrices, see above) that part `index` of
 * `parts` owns: [*first, *first + *count).  Contiguous, sizes differ by at most one. */
XCORR_API void xcorr_shard_range(uint32_t units, int32_t parts, int32_t index,
                                 uint32_t* first, uint32_t* count);

/* Release the cached device buffers of xcorr_run_host*_f32 (all devices) and forget the device
 * addresses xcorr_one_to_one_noalloc_f32 keeps.  Call it before cudaDeviceReset, or after any
 * teardown of a device's primary context: the library keeps nothing else that a reset makes stale. */
XCORR_API void xcorr_release_host_cache(void);

/* ---- n_to_mn order helpers (host memory) -------------------------------------------------
 * matrix.hpp:614-618 get_interleaved_index and :484-552 load/store interleaved.
 * to_grouped != 0: file order (t*n_left + l) -> grouped order (l*m + t); 0: the inverse.
 * `elems` = floats per matrix.  src and dst must not overlap. */
XCORR_API xcorr_status xcorr_n_to_mn_reorder_f32(const float* src, float* dst, uint32_t n_left,
                                                 uint32_t n_total, size_t elems, int32_t to_grouped);

/* ---- diagnostics ---------------------------------------------------------------------------
 * xcorr_last_launch_string: kernel name, grid, block, dynamic shared memory and plan of
 * the calling thread's last launch -- replaces kernel_args.hpp/.cpp (last_kernel_launch_args
 * string echoed by main.cpp:131-133).  Thread-local; valid until the thread's next call. */
XCORR_API const char* xcorr_last_launch_string(void);
XCORR_API const char* xcorr_last_error_string(void);
XCORR_API const char* xcorr_status_string(int32_t status);

/* Number of kernels (library kernels only, not memsets or copies) launched by the calling
 * thread since the counter was last reset. */
XCORR_API uint64_t xcorr_launch_count(void);
XCORR_API void xcorr_reset_launch_count(void);

/* Health of the current device as this library sees it: synchronises the device, then returns
 * XCORR_ERR_CUDA if an earlier launch failed, XCORR_ERR_TIMEOUT if a bounded device-side wait of
 * the library's kernels gave up since the last call of this function (the blocks concerned
 * dropped their work and returned, so results of launches since then are incomplete; the count
 * is in xcorr_last_error_string() and is cleared by this call, the context stays usable), else
 * XCORR_OK.  Stands in for the CUCH(cudaDeviceSynchronize()); CUCH(cudaGetLastError()) pair of
 * main.cpp:267-270. */
XCORR_API xcorr_status xcorr_check_device(void);

/* Test hook for the one device-side wait of the library (a block of the tile kernel waiting for
 * its bulk copies into shared memory).  poll_limit > 0 replaces the number of polls after which
 * the wait gives up (default about 4 million); surplus_bytes > 0 makes every block announce that
 * many bytes more than its copies deliver, so the wait cannot succeed and runs out: the launch
 * then reports XCORR_ERR_TIMEOUT through xcorr_check_device without any fault, hang or lost
 * context (the block takes the surplus back and lets its real copies land before it returns).
 * (0, 0) restores normal operation.  Process-wide; affects launches made after the call. */
XCORR_API void xcorr_debug_stage_wait(uint32_t poll_limit, uint32_t surplus_bytes);

/* Measured FP32 FFMA throughput of the current device in FLOP/s: a dependency-free
 * register-only FFMA kernel on every SM, timed with CUDA events on `stream`
 * (synchronises).  The denominator for "fraction of FFMA peak". */
XCORR_API xcorr_status xcorr_ffma_peak_probe(double* flops_per_second, double* kernel_ms, void* stream);

/* The same for FP64 FMA: the denominator for the double-precision entry points. */
XCORR_API xcorr_status xcorr_dfma_peak_probe(double* flops_per_second, double* kernel_ms, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XCORR_H */
