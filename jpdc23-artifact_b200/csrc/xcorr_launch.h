// Launcher declarations: the only way the C-ABI layer reaches device code.
#pragma once
#include <cuda_runtime.h>
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
cudaError_t launch_ffma_probe(float* sink, int iters, int blocks, cudaStream_t stream);

// Built-in scratch of the entry point that allocates nothing: size, and the array's device
// address on the current device (looked up once per device).
size_t noalloc_scratch_bytes();
cudaError_t noalloc_scratch_address(float** ptr);

}  // namespace xcorr
