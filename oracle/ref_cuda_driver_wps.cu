// C entry point around the REFERENCE's plain warp-per-overlap launcher, the reference's published
// winner for a 16 x 16 pair.
//
// TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference's .cu files are compiled unmodified
// from where the reference checkout lies (oracle/Makefile, target refcuda_wps); this file only
// declares the launchers through the reference's kernels.cuh and forwards to them.
// Device pointers in, asynchronous launch on the default stream; C++ exceptions become
// return code 2.  This library is compiled with --default-stream per-thread, so the launcher's
// stream-less <<<>>> goes to the calling thread's own default stream, which -- unlike the legacy
// one -- may be captured into a CUDA graph: refcuda_warp_per_shift_graph_us times the kernel the
// same way the product's small kernels are timed, free of the host's launch rate.
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


// Microseconds of device time per launch: `launches` calls of the launcher recorded into one
// CUDA graph, the graph replayed `replays` times between two events (after one warm-up replay).
// Negative on failure.
__attribute__((visibility("default")))
double refcuda_warp_per_shift_graph_us(const float* left, const float* right, float* out, uint32_t rows, uint32_t cols,
                                       uint32_t shifts_per_thread_block, uint32_t launches, uint32_t replays) {
    if (launches == 0 || replays == 0) return -1.0;
    cudaStream_t s = cudaStreamPerThread;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    double us = -1.0;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1.0;
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return -1.0;
    int rc = 0;
    for (uint32_t i = 0; i < launches && rc == 0; ++i)
        rc = refcuda_warp_per_shift(left, right, out, rows, cols, shifts_per_thread_block);
    const cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (rc == 0 && ce == cudaSuccess && graph &&
        cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess &&
        cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess &&
        cudaGraphLaunch(exec, s) == cudaSuccess && cudaStreamSynchronize(s) == cudaSuccess) {
        bool ok = cudaEventRecord(e0, s) == cudaSuccess;
        for (uint32_t i = 0; i < replays && ok; ++i) ok = cudaGraphLaunch(exec, s) == cudaSuccess;
        float ms = 0.f;
        if (ok && cudaEventRecord(e1, s) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess &&
            cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess)
            us = (double)ms * 1e3 / ((double)launches * replays);
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    (void)cudaGetLastError();
    return us;
}
}
