// C entry point around the REFERENCE's own best n-to-m CUDA launcher (a library of its own:
// that one source file takes hours to compile at the published template limits), for the
// benchmark's "reference kernels recompiled for sm_100" comparison.
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

// multi-matrix-both + grouped-overlap, best n-to-m
__attribute__((visibility("default")))
int refcuda_n_to_m(const float* left, const float* right, float* out, uint32_t rows, uint32_t cols,
                   uint32_t n_left, uint32_t n_right, uint32_t warps, uint32_t shifts, uint32_t left_mats,
                   uint32_t right_mats, uint32_t left_rows) {
    return guarded([&] { run_ccn_n_to_m_shuffle_multirow_both_multimat_both<float, float>(
                             left, right, out, msize(rows, cols), ssize(rows, cols), n_left, n_right, warps,
                             shifts, left_mats, right_mats, left_rows); });
}

}
