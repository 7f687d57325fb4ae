// FFT path of the cross-correlation: pad -> batched real-to-complex FFT (cuFFT) -> spectrum
// product left * conj(right) -> batched complex-to-real FFT (cuFFT) -> unpack.
//
// Stands in for the reference's cuFFT algorithms (one_to_one.hpp:888-1170 fft_original_alg_* /
// fft_reduced_transfer_*, one_to_many.hpp:502-780, n_to_mn.hpp:720-1000, n_to_m.hpp:647-800) and
// their kernels: hadamard.cu (hadamard_original, hadamard_n_to_m_over_right / _over_output) and
// scatter.cu (zero padding on the device).  The transforms themselves are library calls, as in
// the reference; what is written here are the three memory-bound kernels around them and the
// plan cache.  Differences from the reference, by design:
//   * inputs arrive unpadded and are padded on the device (the reference's "reduced transfer"
//     variants; its "original" variants pad on the host while parsing the CSV);
//   * the result can be delivered either RAW (2H x 2W per pair, unnormalised, circular shifts:
//     exactly what the reference's fft classes hold in results()) or NORMALIZED (quadrants
//     swapped, the empty row / column dropped, divided by 4HW: fft_helpers.hpp:213-262
//     normalize_fft_results, done there on the host) -- the second is the same layout as the
//     direct path's result;
//   * one product kernel covers the four modes through the pair map.
// Every kernel here is HBM-bound: a handful of bytes per element, no reuse beyond L2.
#include <cuda_runtime.h>
#include <cufft.h>

#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <vector>

#include "xcorr_launch.h"

namespace xcorr {

namespace {

constexpr int kThreads = 256;

// ---- zero padding: (n, H, W) -> (n, 2H, 2W), data in the top-left corner (scatter.cu).
//      One warp per padded row at a time; a unit is 4 consecutive floats (VEC) or one.
template<bool VEC>
__global__ void __launch_bounds__(kThreads) fft_pad_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                           int H, int W, unsigned long long rows_total) {
    const unsigned per_row = VEC ? (unsigned)(2 * W / 4) : (unsigned)(2 * W);
    const unsigned lane = threadIdx.x & 31;
    const unsigned long long warps = (unsigned long long)gridDim.x * (kThreads / 32);
    // four rows per trip, all loads before the stores: the kernel is bound by memory latency
    // times the loads in flight, not by arithmetic
    constexpr int kRows = 4;
    for (unsigned long long r0 = ((unsigned long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * kRows;
         r0 < rows_total; r0 += warps * kRows) {
        for (unsigned u = lane; u < per_row; u += 32) {
            float4 v4[kRows];
            float v1[kRows];
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                const unsigned long long r = r0 + i;
                const unsigned long long mat = r / (unsigned)(2 * H);
                const int y = (int)(r - mat * (unsigned)(2 * H));
                const float* src = in + (mat * H + y) * W;       // only read when y < H
                v4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                v1[i] = 0.f;
                if (r < rows_total && y < H) {
                    if (VEC) { if ((int)(u * 4) < W) v4[i] = __ldg(reinterpret_cast<const float4*>(src + u * 4)); }
                    else if ((int)u < W) v1[i] = __ldg(src + u);
                }
            }
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                const unsigned long long r = r0 + i;
                if (r >= rows_total) continue;
                float* dst = out + r * (2ull * W);
                if (VEC) reinterpret_cast<float4*>(dst)[u] = v4[i];
                else dst[u] = v1[i];
            }
        }
    }
}

// ---- spectrum product: out[pair] = L[l(pair)] * conj(R[r(pair)])  (hadamard.cu:17-24) ---------
// P complex numbers per matrix (P even: 2H rows of W+1).  One unit = two complex numbers.
// pair = l * m + t; the right spectrum is pair itself (one_to_one, one_to_many, n_to_mn in
// grouped order) or t (n_to_m).  `out` may be the right spectra themselves when every right
// matrix is used once.
__global__ void __launch_bounds__(kThreads) fft_product_kernel(const float4* __restrict__ L, const float4* R,
                                                               float4* out, unsigned half_p, unsigned m,
                                                               int right_is_pair, unsigned long long units) {
    for (unsigned long long u = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; u < units;
         u += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long pair = u / half_p;
        const unsigned i = (unsigned)(u - pair * half_p);
        const unsigned long long l = pair / m;
        const unsigned long long r = right_is_pair ? pair : pair - l * m;
        const float4 a = __ldg(L + l * half_p + i);
        const float4 b = R[r * half_p + i];
        float4 c;
        c.x = a.x * b.x + a.y * b.y;
        c.y = a.y * b.x - a.x * b.y;
        c.z = a.z * b.z + a.w * b.w;
        c.w = a.w * b.z - a.z * b.w;
        out[u] = c;
    }
}

// ---- unpack: raw (pairs, 2H, 2W) -> (pairs, 2H-1, 2W-1), shift (sy, sx) read from row
//      sy mod 2H, column sx mod 2W, scaled by 1 / (4HW)  (fft_helpers.hpp:199-262).
//      One warp per output row at a time (one division per row, none per element): the two
//      halves of a row are two contiguous runs of the raw row.
__global__ void __launch_bounds__(kThreads) fft_unpack_kernel(const float* __restrict__ raw, float* __restrict__ out,
                                                              int H, int W, float scale, unsigned long long rows_total) {
    const unsigned OW = 2 * W - 1, OH = 2 * H - 1;
    const unsigned lane = threadIdx.x & 31;
    const unsigned long long warps = (unsigned long long)gridDim.x * (kThreads / 32);
    constexpr int kRows = 2, kCols = 4;               // 8 loads in flight per lane
    for (unsigned long long r0 = ((unsigned long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * kRows;
         r0 < rows_total; r0 += warps * kRows) {
        const float* src[kRows];
#pragma unroll
        for (int i = 0; i < kRows; ++i) {
            const unsigned long long r = min(r0 + i, rows_total - 1);
            const unsigned long long pair = r / OH;
            const unsigned oy = (unsigned)(r - pair * OH);
            const int sy = (int)oy - (H - 1);
            const unsigned ry = sy < 0 ? sy + 2 * H : sy;
            src[i] = raw + (pair * (2ull * H) + ry) * (2ull * W);
        }
        // ox < W-1: sx = ox-(W-1) < 0 -> column ox + W + 1; ox >= W-1: column ox - (W-1)
        for (unsigned x0 = lane; x0 < OW; x0 += 32 * kCols) {
            float v[kRows][kCols];
#pragma unroll
            for (int i = 0; i < kRows; ++i)
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    const unsigned ox = x0 + 32 * j;
                    const unsigned rx = ox < (unsigned)(W - 1) ? ox + W + 1 : ox - (W - 1);
                    v[i][j] = ox < OW ? __ldg(src[i] + rx) : 0.f;
                }
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                if (r0 + i >= rows_total) continue;
                float* dst = out + (r0 + i) * OW;
#pragma unroll
                for (int j = 0; j < kCols; ++j)
                    if (x0 + 32 * j < OW) dst[x0 + 32 * j] = v[i][j] * scale;
            }
        }
    }
}

unsigned grid_for(unsigned long long units, int sm_count) {
    const unsigned long long want = (units + kThreads - 1) / kThreads;
    const unsigned long long cap = (unsigned long long)sm_count * 16;     // resident waves of 256-thread blocks
    return (unsigned)std::max<unsigned long long>(1, std::min(want, cap));
}

// ---- cuFFT plans, cached per (device, size, batch, direction) ---------------------------------
struct PlanEntry {
    int device, h2, w2, batch, forward;
    cufftHandle handle;
    unsigned long long stamp;
};
std::mutex g_plan_mutex;
std::vector<PlanEntry> g_plans;
unsigned long long g_plan_stamp = 0;
constexpr size_t kMaxPlans = 24;

const char* cufft_name(cufftResult r) {
    switch (r) {
    case CUFFT_SUCCESS: return "CUFFT_SUCCESS";
    case CUFFT_INVALID_PLAN: return "CUFFT_INVALID_PLAN";
    case CUFFT_ALLOC_FAILED: return "CUFFT_ALLOC_FAILED";
    case CUFFT_INVALID_VALUE: return "CUFFT_INVALID_VALUE";
    case CUFFT_INTERNAL_ERROR: return "CUFFT_INTERNAL_ERROR";
    case CUFFT_EXEC_FAILED: return "CUFFT_EXEC_FAILED";
    case CUFFT_SETUP_FAILED: return "CUFFT_SETUP_FAILED";
    case CUFFT_INVALID_SIZE: return "CUFFT_INVALID_SIZE";
    default: return "cuFFT error";
    }
}

// Must be called with g_plan_mutex held.
cufftResult get_plan(int device, int h2, int w2, int batch, int forward, cufftHandle* out) {
    for (PlanEntry& e : g_plans)
        if (e.device == device && e.h2 == h2 && e.w2 == w2 && e.batch == batch && e.forward == forward) {
            e.stamp = ++g_plan_stamp;
            *out = e.handle;
            return CUFFT_SUCCESS;
        }
    if (g_plans.size() >= kMaxPlans) {          // drop the plan used longest ago
        size_t victim = 0;
        for (size_t i = 1; i < g_plans.size(); ++i)
            if (g_plans[i].stamp < g_plans[victim].stamp) victim = i;
        cufftDestroy(g_plans[victim].handle);
        g_plans.erase(g_plans.begin() + (long)victim);
    }
    int n[2] = {h2, w2};
    cufftHandle h;
    // contiguous batches: with NULL embeds the strides and distances are the natural ones
    const cufftResult r = cufftPlanMany(&h, 2, n, nullptr, 1, 0, nullptr, 1, 0, forward ? CUFFT_R2C : CUFFT_C2R, batch);
    if (r != CUFFT_SUCCESS) return r;
    g_plans.push_back(PlanEntry{device, h2, w2, batch, forward, h, ++g_plan_stamp});
    *out = h;
    return CUFFT_SUCCESS;
}

size_t align256(size_t b) { return (b + 255) / 256 * 256; }

}  // namespace

FftLayout fft_workspace_layout(const PairMap& pm, int H, int W, unsigned n_right, int raw_result) {
    FftLayout l{};
    const size_t pairs = (size_t)pm.n_left * pm.m;
    const size_t real_mat = 4ull * H * W;                       // 2H x 2W floats
    const size_t cplx_mat = 2ull * H * (W + 1);                 // 2H x (W + 1) complex numbers
    const bool in_place = pm.n_left == 1 || pm.right_stride != 0;
    l.padded_off = 0;
    l.spectra_off = l.padded_off + align256(((size_t)pm.n_left + n_right) * real_mat * sizeof(float));
    l.product_off = l.spectra_off + align256(((size_t)pm.n_left + n_right) * cplx_mat * 2 * sizeof(float));
    l.raw_off = l.product_off + (in_place ? 0 : align256(pairs * cplx_mat * 2 * sizeof(float)));
    l.total = l.raw_off + (raw_result ? 0 : align256(pairs * real_mat * sizeof(float)));
    l.product_in_place = in_place ? 1 : 0;
    return l;
}

int fft_run(const float* left, const float* right, float* out, int H, int W, const PairMap& pm, unsigned n_right,
            int raw_result, void* workspace, int device, int sm_count, cudaStream_t stream, std::string* err,
            int* launches) {
    const FftLayout lay = fft_workspace_layout(pm, H, W, n_right, raw_result);
    char* ws = static_cast<char*>(workspace);
    float* padded = reinterpret_cast<float*>(ws + lay.padded_off);
    float* spectra = reinterpret_cast<float*>(ws + lay.spectra_off);
    const size_t pairs = (size_t)pm.n_left * pm.m;
    const size_t n_in = (size_t)pm.n_left + n_right;
    const size_t real_mat = 4ull * H * W, cplx_mat = 2ull * H * (W + 1);
    float* right_spectra = spectra + (size_t)pm.n_left * cplx_mat * 2;
    float* product = lay.product_in_place ? right_spectra : reinterpret_cast<float*>(ws + lay.product_off);
    float* raw = raw_result ? out : reinterpret_cast<float*>(ws + lay.raw_off);
    if (n_in > 0x7fffffffull || pairs > 0x7fffffffull) { *err = "too many matrices for one cuFFT batch"; return 2; }

    auto cuda_check = [&](cudaError_t e, const char* what) {
        if (e == cudaSuccess) return false;
        *err = std::string(what) + ": " + cudaGetErrorString(e);
        return true;
    };

    // 1. pad both inputs: left matrices first, right matrices after them
    const bool vec = (W % 4 == 0) && reinterpret_cast<uintptr_t>(left) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(right) % 16 == 0;
    for (int side = 0; side < 2; ++side) {
        const float* src = side == 0 ? left : right;
        const size_t n = side == 0 ? pm.n_left : n_right;
        float* dst = padded + (side == 0 ? 0 : (size_t)pm.n_left * real_mat);
        const unsigned long long rows_total = (unsigned long long)n * 2ull * H;
        const unsigned grid = grid_for(rows_total * 32, sm_count);
        if (vec) fft_pad_kernel<true><<<grid, kThreads, 0, stream>>>(src, dst, H, W, rows_total);
        else     fft_pad_kernel<false><<<grid, kThreads, 0, stream>>>(src, dst, H, W, rows_total);
        if (cuda_check(cudaGetLastError(), "fft_pad_kernel")) return 1;
    }
    *launches += 2;

    {
        // 2. forward transforms of all inputs in one batch; 4. inverse transforms of all pairs
        std::lock_guard<std::mutex> lock(g_plan_mutex);
        cufftHandle fwd, inv;
        cufftResult r = get_plan(device, 2 * H, 2 * W, (int)n_in, 1, &fwd);
        if (r == CUFFT_SUCCESS) r = get_plan(device, 2 * H, 2 * W, (int)pairs, 0, &inv);
        if (r == CUFFT_SUCCESS) r = cufftSetStream(fwd, stream);
        if (r == CUFFT_SUCCESS) r = cufftSetStream(inv, stream);
        if (r == CUFFT_SUCCESS) r = cufftExecR2C(fwd, padded, reinterpret_cast<cufftComplex*>(spectra));
        if (r != CUFFT_SUCCESS) { *err = std::string("cuFFT forward: ") + cufft_name(r); return 2; }

        // 3. spectrum products
        const unsigned half_p = (unsigned)(cplx_mat / 2);
        const unsigned long long units = (unsigned long long)pairs * half_p;
        fft_product_kernel<<<grid_for(units, sm_count), kThreads, 0, stream>>>(
            reinterpret_cast<const float4*>(spectra), reinterpret_cast<const float4*>(right_spectra),
            reinterpret_cast<float4*>(product), half_p, pm.m, lay.product_in_place, units);
        if (cuda_check(cudaGetLastError(), "fft_product_kernel")) return 1;

        r = cufftExecC2R(inv, reinterpret_cast<cufftComplex*>(product), raw);
        if (r != CUFFT_SUCCESS) { *err = std::string("cuFFT inverse: ") + cufft_name(r); return 2; }
    }
    *launches += 1;

    // 5. unpack to the direct path's layout
    if (!raw_result) {
        const unsigned long long rows_total = (unsigned long long)pairs * (2ull * H - 1);
        fft_unpack_kernel<<<grid_for(rows_total * 32, sm_count), kThreads, 0, stream>>>(
            raw, out, H, W, 1.0f / (4.0f * (float)H * (float)W), rows_total);
        if (cuda_check(cudaGetLastError(), "fft_unpack_kernel")) return 1;
        *launches += 1;
    }
    return 0;
}

void fft_release_plans() {
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (PlanEntry& e : g_plans) cufftDestroy(e.handle);
    g_plans.clear();
}

}  // namespace xcorr
