// Launcher declarations: the only way the C-ABI layer reaches device code.
#pragma once
#include <cuda_runtime.h>
#include <string>
#include "xcorr_plan.h"

namespace xcorr {

// `device` = the current device (remembers per device that the shared-memory limit was raised).
cudaError_t launch_tile(const TileArgs& a, int device, cudaStream_t stream);
cudaError_t launch_reduce_partials(const float* ws, float* out, unsigned long long total_out,
                                   int H, int W, int Hp, int S, int sm_count, cudaStream_t stream);
cudaError_t launch_overlap_wise(const float* left, const float* right, float* out, int H, int W,
                                PairMap pm, unsigned long long npairs, int block_threads,
                                dim3* grid_out, dim3* block_out, cudaStream_t stream);
// rows_per_warp / split (RowSplit): the overlap's rows shared by several warps adding atomically onto
// a zeroed output; split = kSplitNone writes every overlap once.
cudaError_t launch_warp_per_overlap(const float* left, const float* right, float* out, int H, int W,
                                    PairMap pm, unsigned long long npairs, int block_threads,
                                    int rows_per_warp, int split, int sm_count, dim3* grid_out, dim3* block_out,
                                    cudaStream_t stream);
// Staged warp-per-overlap kernel; a.col_groups = 1 adds atomically onto a zeroed output.
size_t staged_smem_bytes(const StagedArgs& a);
cudaError_t launch_warp_staged(const StagedArgs& a, int device, dim3* grid_out, size_t* smem_out, cudaStream_t stream);
// Number of blocks of the tile kernel whose bounded staging wait gave up on the current device
// since the last call (0 in every healthy run); reads and clears the count, synchronises with
// the device.
cudaError_t tile_stage_timeouts(unsigned* count);
// Double precision (xcorr_f64.cu): one warp per 8 output rows x 32 output columns of a pair.
cudaError_t launch_strip_f64(const double* left, const double* right, double* out, int H, int W, PairMap pm,
                             unsigned long long npairs, int sm_count, dim3* grid_out, dim3* block_out,
                             cudaStream_t stream);
// The warp-per-overlap latency kernel in double (a handful of small overlaps; below 2^31 of them).
cudaError_t launch_warp_per_overlap_f64(const double* left, const double* right, double* out, int H, int W,
                                        PairMap pm, unsigned long long npairs, int block_threads, dim3* grid_out,
                                        cudaStream_t stream);
// Double precision, register-tiled (xcorr_f64_tile.cu).  plan_tile_f64 returns false when no plan fits
// one SM's shared memory; a plan with S > 1 needs the output zeroed before the launch.  `reproducible`
// keeps to plans whose results are bit-identical from run to run (at most two row slices).
bool plan_tile_f64(const PairMap& pm, int H, int W, int sm_count, size_t smem_limit, bool reproducible, TilePlan64* out);
cudaError_t launch_tile_f64(const TileArgs64& a, int device, cudaStream_t stream);
cudaError_t launch_dfma_probe(double* sink, int iters, int blocks, cudaStream_t stream);
cudaError_t launch_ffma_probe(float* sink, int iters, int blocks, cudaStream_t stream);

// Built-in scratch of the entry point that allocates nothing: size, and the array's device
// address on the current device (looked up once per device).
size_t noalloc_scratch_bytes();
cudaError_t noalloc_scratch_address(float** ptr);
// Forget the cached addresses (after the application reset a device or tore its context down).
void noalloc_forget_addresses();

// FFT path (xcorr_fft.cu).  Workspace layout in bytes: padded real inputs, spectra of all
// inputs, spectrum products (absent when they overwrite the right spectra: every mode but
// n_to_m), raw inverse transforms (absent when the caller wants the raw result in `out`).
struct FftLayout {
    size_t padded_off, spectra_off, product_off, raw_off, total;
    int product_in_place;
};
FftLayout fft_workspace_layout(const PairMap& pm, int H, int W, unsigned n_right, int raw_result);
// Enqueues the whole path on `stream`.  0 = ok, 1 = CUDA error, 2 = cuFFT error (*err says which);
// *launches is increased by the number of own kernels launched.
int fft_run(const float* left, const float* right, float* out, int H, int W, const PairMap& pm, unsigned n_right,
            int raw_result, void* workspace, int device, int sm_count, cudaStream_t stream, std::string* err,
            int* launches);
void fft_release_plans();

}  // namespace xcorr
