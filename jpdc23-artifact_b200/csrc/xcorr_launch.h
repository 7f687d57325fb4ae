// Launcher declarations: the only way the C-ABI layer reaches device code.
#pragma once
#include <cuda_runtime.h>
#include <string>
#include "xcorr_plan.h"

namespace xcorr {

cudaError_t launch_tile(const TileArgs& a, cudaStream_t stream);
cudaError_t launch_reduce_partials(const float* ws, float* out, unsigned long long total_out,
                                   int H, int W, int Hp, int S, int sm_count, cudaStream_t stream);
cudaError_t launch_overlap_wise(const float* left, const float* right, float* out, int H, int W,
                                PairMap pm, unsigned long long npairs, int block_threads,
                                dim3* grid_out, dim3* block_out, cudaStream_t stream);
cudaError_t launch_warp_per_overlap(const float* left, const float* right, float* out, int H, int W,
                                    PairMap pm, unsigned long long npairs, int block_threads,
                                    int sm_count, dim3* grid_out, dim3* block_out, cudaStream_t stream);
// Number of bounded staging waits of the tile kernel that gave up on the current device since
// the library was loaded (0 in every healthy run); synchronises with the device.
cudaError_t tile_stage_timeouts(unsigned* count);
// Double precision (xcorr_f64.cu): one warp per 8 output rows x 32 output columns of a pair.
cudaError_t launch_strip_f64(const double* left, const double* right, double* out, int H, int W, PairMap pm,
                             unsigned long long npairs, int sm_count, dim3* grid_out, dim3* block_out,
                             cudaStream_t stream);
cudaError_t launch_dfma_probe(double* sink, int iters, int blocks, cudaStream_t stream);
cudaError_t launch_ffma_probe(float* sink, int iters, int blocks, cudaStream_t stream);

// Built-in scratch of the entry point that allocates nothing: size, and the array's device
// address on the current device (looked up once per device).
size_t noalloc_scratch_bytes();
cudaError_t noalloc_scratch_address(float** ptr);

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
