// C entry points around the REFERENCE's own best CUDA launchers, for the benchmark's
// "reference kernels recompiled for sm_100" comparison and as a third parity witness.
//
// TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference's .cu files are compiled unmodified
// from where the reference checkout lies (oracle/Makefile, target refcuda); this file only
// declares the launchers through the reference's kernels.cuh and forwards to them.
// Device pointers in, asynchronous launch on the default stream (or `stream` where the
// reference launcher has that parameter); C++ exceptions become return code 2.
#include <cuda_runtime.h>
#include <cstdint>
#include <exception>

#include "kernels.cuh"

using namespace cross;

namespace {
dsize2_t msize(uint32_t rows, uint32_t cols) { return dsize2_t{cols, rows}; }
dsize2_t ssize(uint32_t rows, uint32_t cols) { return dsize2_t{2 * cols - 1, 2 * rows - 1}; }
template<typename F> int guarded(F&& f) {
    try { f(); return 0; } catch (std::exception&) { return 2; }
}
}

extern "C" {

// overlap-wise: run_cross_corr_naive_original (naive_original.cu:131-161)
__attribute__((visibility("default")))
int refcuda_overlap_wise(const float* left, const float* right, float* out, uint32_t rows, uint32_t cols,
                         uint32_t n_left, uint32_t batch) {
    return guarded([&] { run_cross_corr_naive_original<float, float>(left, right, out, msize(rows, cols),
                                                                       ssize(rows, cols), n_left, batch, nullptr); });
}

// grouped-overlap, best one-to-one: run_ccn_shuffle_multirow_both (naive_shuffle_multirow_both.cu:634-677)
__attribute__((visibility("default")))
int refcuda_one_to_one(const float* left, const float* right, float* out, uint32_t rows, uint32_t cols,
                       uint32_t warps, uint32_t shifts_per_thread, uint32_t left_rows) {
    return guarded([&] { run_ccn_shuffle_multirow_both<float, float>(left, right, out, msize(rows, cols),
                                                                       ssize(rows, cols), warps, shifts_per_thread,
                                                                       left_rows); });
}

// multi-matrix-right + grouped-overlap, best one-to-many / n-to-mn (one launch per left matrix)
__attribute__((visibility("default")))
int refcuda_one_to_many(const float* left, const float* right, float* out, uint32_t rows, uint32_t cols,
                        uint32_t n_right, uint32_t warps, uint32_t shifts, uint32_t right_mats, uint32_t left_rows,
                        void* stream) {
    return guarded([&] { run_ccn_shuffle_one_to_many_multirow_both_multimat_right<float, float>(
                             left, right, out, msize(rows, cols), ssize(rows, cols), n_right, warps, shifts,
                             right_mats, left_rows, static_cast<cudaStream_t>(stream)); });
}

}
