// C entry point around the REFERENCE's plain warp-per-overlap launcher, the reference's published
// winner for a 16 x 16 pair.
//
// TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference's .cu files are compiled unmodified
// from where the reference checkout lies (oracle/Makefile, target refcuda_wps); this file only
// declares the launchers through the reference's kernels.cuh and forwards to them.
// Device pointers in, asynchronous launch on the default stream; C++ exceptions become
// return code 2.
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

// run_ccn_warp_per_shift (naive_warp_per_shift.cu:308-335)
__attribute__((visibility("default")))
int refcuda_warp_per_shift(const float* left, const float* right, float* out, uint32_t rows, uint32_t cols,
                           uint32_t shifts_per_thread_block) {
    return guarded([&] { run_ccn_warp_per_shift<float, float>(left, right, out, msize(rows, cols), ssize(rows, cols),
                                                                shifts_per_thread_block); });
}

}
