// Double-precision direct cross-correlation, register-tiled: the circular classes of the float
// kernel (xcorr_plan.h) in both directions, operands staged in shared memory.
//
// Stands in for what the reference never finished: every <double> instantiation of its kernels is
// commented out (e.g. naive_shuffle.cu:545-552) and `--data_type double` is refused
// (main.cpp:433-434).
//
// Work split.  Pad to Hp x Wp with zeros (Wp a multiple of 8, Hp a multiple of SL).  A warp owns
// one 8-wide tile of x classes and SL y classes: lane (m, q) holds class cy = cyw + q of right
// matrix m of the block's group (ML = 32 / SL matrices per warp).  A block is WX x WY such warps
// sharing one left matrix, ML right matrices and one slice [r0, r1) of right rows, staged once.
//
// Per right row ry the thread walks the left row in chunks of 8 columns u:
//     acc[j] += L[(ry + cy) mod Hp][u] * R[ry][(u - cx0 - j) mod Wp],   j in [0, 8)
// Column j has wrapped in x while u < cx0 + j: those products belong to output shift cx - Wp, the
// others to shift cx.  Unlike the float kernel, which walks the rows twice with one accumulator
// set, this one keeps both sets (32 doubles) and walks once: every chunk left of the tile's own
// goes to the wrapped set, every chunk right of it to the unwrapped one, the tile's own chunk is
// split along its diagonal -- three straight-line bodies of 64 DFMA.  FP64 issues at a quarter of
// the FP32 rate per scheduler, so the 12 shared loads per chunk hide behind the arithmetic.
// y wrap as in the float kernel: class cy wraps from right row Hp - cy on; its sums go to the
// unwrapped output row when the walk reaches that row, to the wrapped one at the end of the slice.
//
// Rows are divided into S slices when one block per task would leave SMs idle or the staged rows
// would not fit; the slices' sums are then added with red.global.add.f64 onto the zeroed output.
#include <cuda_runtime.h>
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <vector>
#include <cstdint>

#include "xcorr_launch.h"

namespace xcorr {
namespace {

constexpr int kDX = 8;                  // x classes per thread

__device__ __forceinline__ void lds128d(uint32_t addr, double& a, double& b) {
    asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];" : "=d"(a), "=d"(b) : "r"(addr));
}

// One chunk of 8 steps.  w[i] holds R[ry][(8 (c - cb - 1) + i) mod Wp], i in [0, 16), so that step kk and
// column j meet w[8 + kk - j].  MODE 0: every product wrapped in x; 1: none; 2: the tile's own
// chunk, wrapped while kk < j.
template<int MODE>
__device__ __forceinline__ void chunk64(double (&accU)[kDX], double (&accW)[kDX], uint32_t laddr, uint32_t w0, uint32_t w1) {
    double w[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lds128d(w0 + 16 * i, w[2 * i], w[2 * i + 1]);
        lds128d(w1 + 16 * i, w[8 + 2 * i], w[9 + 2 * i]);
    }
#pragma unroll
    for (int k2 = 0; k2 < 4; ++k2) {
        double l0, l1;
        lds128d(laddr + 16 * k2, l0, l1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kk = 2 * k2 + h;
            const double l = h == 0 ? l0 : l1;
#pragma unroll
            for (int j = 0; j < kDX; ++j) {
                const bool wrapped = MODE == 0 || (MODE == 2 && kk < j);
                if (wrapped) accW[j] = fma(l, w[8 + kk - j], accW[j]);
                else         accU[j] = fma(l, w[8 + kk - j], accU[j]);
            }
        }
    }
}

// Write (or add) one class's 8 sums of one accumulator set to its output row.
__device__ __forceinline__ void put_row(double* rowptr, const double (&acc)[kDX], int col0, int lo, int hi, bool add) {
#pragma unroll
    for (int j = 0; j < kDX; ++j) {
        const int col = col0 + j;
        if (col >= lo && col < hi) {
            if (add) atomicAdd(rowptr + col, acc[j]); else rowptr[col] = acc[j];
        }
    }
}

__global__ void __launch_bounds__(512, 1) tile_f64_kernel(const TileArgs64 a) {
    extern __shared__ __align__(16) double smem64[];
    const TilePlan64& p = a.p;
    const int H = p.H, W = p.W, Hp = p.Hp, Wp = p.Wp;
    const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31;
    double* sL = smem64;
    double* sR = smem64 + (size_t)p.nstage * p.LS;

    // block -> (left, right group, y block, x block, slice)
    unsigned task = blockIdx.x / (unsigned)p.S;
    const int slice = (int)(blockIdx.x - task * (unsigned)p.S);
    const int bx = (int)(task % (unsigned)p.CX); task /= (unsigned)p.CX;
    const int by = (int)(task % (unsigned)p.CY); task /= (unsigned)p.CY;
    const int rg = (int)(task % (unsigned)p.RG);
    const int l = (int)(task / (unsigned)p.RG);
    const int r0 = (int)(((long long)slice * H) / p.S), r1 = (int)(((long long)(slice + 1) * H) / p.S);

    const int wx = warp % p.WX, wy = warp / p.WX;
    const int q = lane & (p.SL - 1), m = lane >> p.logSL;
    const int cls_per_block = p.WY * p.SL;
    const int cya = by * cls_per_block;
    int rowbase = r0 + cya;
    if (rowbase >= Hp) rowbase -= Hp;
    const int nstage = min(r1 - r0 + cls_per_block - 1, Hp);
    const int rs = r1 - r0;

    // ---- stage: left rows (rowbase + i) mod Hp, i < nstage, and rows [r0, r1) of the group's ML
    //      right matrices; zeros where the padded matrices are zero.  Two doubles per 16-byte copy
    //      where the rows allow it (even column count, aligned operands).
    {
        const double* gL = a.left + (size_t)l * H * W;
        const int units = p.LS >> 1;
        for (int idx = tid; idx < nstage * units; idx += nthr) {
            const int i = idx / units, x = (idx - i * units) * 2;
            int row = rowbase + i;
            if (row >= Hp) row -= Hp;
            double v0 = 0.0, v1 = 0.0;
            if (row < H && x < W) {
                const double* g = gL + (size_t)row * W + x;
                if (a.vec_ok) { const double2 v = *reinterpret_cast<const double2*>(g); v0 = v.x; v1 = v.y; }
                else { v0 = __ldg(g); if (x + 1 < W) v1 = __ldg(g + 1); }
            }
            *reinterpret_cast<double2*>(sL + (size_t)i * p.LS + x) = make_double2(v0, v1);
        }
        const int runits = Wp >> 1, per_mat = rs * runits;
        for (int idx = tid; idx < p.ML * per_mat; idx += nthr) {
            const int mm = idx / per_mat, rem = idx - mm * per_mat;
            const int rr = rem / runits, x = (rem - rr * runits) * 2;
            const unsigned j = (unsigned)rg * p.ML + mm;
            double v0 = 0.0, v1 = 0.0;
            if (j < a.pm.m && x < W) {
                const double* g = a.right + (((size_t)l * a.pm.right_stride + j) * H + (r0 + rr)) * W + x;
                if (a.vec_ok) { const double2 v = *reinterpret_cast<const double2*>(g); v0 = v.x; v1 = v.y; }
                else { v0 = __ldg(g); if (x + 1 < W) v1 = __ldg(g + 1); }
            }
            *reinterpret_cast<double2*>(sR + (size_t)mm * p.RMS + (size_t)rr * Wp + x) = make_double2(v0, v1);
        }
    }
    __syncthreads();

    const int tile_x = bx * p.WX + wx, grp_y = by * p.WY + wy;
    if (tile_x >= p.NTX || grp_y >= p.NGY) return;
    const unsigned jright = (unsigned)rg * p.ML + m;
    const bool live = jright < a.pm.m;
    const int cx0 = tile_x * kDX, cb = tile_x;
    const int cy = grp_y * p.SL + q;
    const int OW = 2 * W - 1;
    double* dst = a.out + ((size_t)l * a.pm.m + jright) * (size_t)(2 * H - 1) * OW;
    const bool add = p.S > 1;

    const uint32_t sL_addr = (uint32_t)__cvta_generic_to_shared(sL);
    const uint32_t rmat = (uint32_t)__cvta_generic_to_shared(sR + (size_t)m * p.RMS);
    const uint32_t ls_bytes = (uint32_t)p.LS * 8, stage_bytes = (uint32_t)nstage * ls_bytes, row_bytes = (uint32_t)Wp * 8;
    uint32_t lofs;
    {
        int i = cy - cya;                       // staged row of left row (r0 + cy) mod Hp
        if (i >= nstage) i -= nstage;
        lofs = (uint32_t)i * ls_bytes;
    }
    double accU[kDX], accW[kDX];
#pragma unroll
    for (int j = 0; j < kDX; ++j) { accU[j] = 0.0; accW[j] = 0.0; }

    const int wrap_row = Hp - cy;               // from this right row on the class has wrapped in y
    uint32_t rrow = rmat;
#pragma unroll 1
    for (int ry = r0; ry < r1; ++ry, rrow += row_bytes) {
        if (ry == wrap_row && ry > r0) {
            // the unwrapped-in-y sums are complete: output row of shift sy = cy
            if (live && cy < H) {
                double* rowptr = dst + (size_t)(cy + H - 1) * OW;
                put_row(rowptr, accU, cx0 + W - 1, 0, OW, add);                 // shift cx: columns < W are real
                put_row(rowptr, accW, cx0 - Wp + W - 1, 0, OW, add);            // shift cx - Wp
            }
#pragma unroll
            for (int j = 0; j < kDX; ++j) { accU[j] = 0.0; accW[j] = 0.0; }
        }
        const uint32_t lrow = sL_addr + lofs;
        // chunk c reads R columns 8 (c - cb - 1) .. + 15 (mod Wp): two aligned runs of 8
        uint32_t w0 = (uint32_t)(((0 - cb - 1) * kDX + 2 * Wp) % Wp) * 8;     // byte offset of the first run for c = 0
#pragma unroll 1
        for (int c = 0; c < p.NCH; ++c) {
            uint32_t w1 = w0 + kDX * 8;
            if (w1 == row_bytes) w1 = 0;
            if (c < cb)       chunk64<0>(accU, accW, lrow + (uint32_t)c * 64, rrow + w0, rrow + w1);
            else if (c > cb)  chunk64<1>(accU, accW, lrow + (uint32_t)c * 64, rrow + w0, rrow + w1);
            else              chunk64<2>(accU, accW, lrow + (uint32_t)c * 64, rrow + w0, rrow + w1);
            w0 = w1;
        }
        lofs += ls_bytes;
        if (lofs == stage_bytes) lofs = 0;
    }
    // end of the slice: the sums belong to the wrapped output row if the class wrapped inside (or
    // before) the slice, else to the unwrapped one
    if (live) {
        const int sy = r1 > wrap_row ? cy - Hp : cy;
        if (sy > -H && sy < H) {
            double* rowptr = dst + (size_t)(sy + H - 1) * OW;
            put_row(rowptr, accU, cx0 + W - 1, 0, OW, add);
            put_row(rowptr, accW, cx0 - Wp + W - 1, 0, OW, add);
        }
    }
}

}  // namespace

// Plan: lanes over y classes so that the padding of the rows stays small and the group of right
// matrices is not larger than the matrices there are; blocks of up to 16 warps; as many row slices
// as it takes to fit one SM's shared memory and to give every SM a block.
bool plan_tile_f64(const PairMap& pm, int H, int W, int sm_count, size_t smem_limit, bool reproducible, TilePlan64* out) {
    TilePlan64 best{};
    double best_cost = -1.0;
    // XCORR_F64_PLAN="SL,warps,S" pins the lane split, the warp cap (8 or 16) and the row slices of the
    // search (0 = free): the tuning switch the cost model below was checked with.
    int want_sl = 0, want_cap = 0, want_s = 0;
    if (const char* e = std::getenv("XCORR_F64_PLAN")) std::sscanf(e, "%d,%d,%d", &want_sl, &want_cap, &want_s);
    const char* dbg = std::getenv("XCORR_PLAN_DEBUG");
    const bool plan_debug = dbg && dbg[0] == '1';
    // The search takes some tens of microseconds of host time, as long as the kernel of a small input:
    // its results are remembered per (counts, size, device limits, switches).
    struct Key {
        uint32_t n_left, m, right_stride; int H, W, sm_count; size_t smem_limit; int reproducible, sl, cap, s;
        bool operator==(const Key& o) const {
            return n_left == o.n_left && m == o.m && right_stride == o.right_stride && H == o.H && W == o.W &&
                   sm_count == o.sm_count && smem_limit == o.smem_limit && reproducible == o.reproducible &&
                   sl == o.sl && cap == o.cap && s == o.s;
        }
    };
    struct Entry { Key key; TilePlan64 plan; bool ok; };
    static std::mutex cache_mutex;
    static std::vector<Entry> cache;
    const Key key{pm.n_left, pm.m, pm.right_stride, H, W, sm_count, smem_limit, reproducible ? 1 : 0, want_sl, want_cap, want_s};
    if (!plan_debug) {
        std::lock_guard<std::mutex> lock(cache_mutex);
        for (const Entry& e : cache)
            if (e.key == key) { if (e.ok) *out = e.plan; return e.ok; }
    }
    for (int SL = 1; SL <= 32; SL *= 2) {
        if (want_sl > 0 && SL != want_sl) continue;
        TilePlan64 p{};
        p.H = H; p.W = W; p.SL = SL; p.ML = 32 / SL;
        p.logSL = 0; while ((1 << p.logSL) < SL) ++p.logSL;
        p.Wp = (W + kDX - 1) / kDX * kDX;
        p.Hp = (H + SL - 1) / SL * SL;
        p.NTX = p.Wp / kDX; p.NCH = p.NTX; p.NGY = p.Hp / SL;
        p.RG = (int)((pm.m + p.ML - 1) / p.ML);
        for (int cap : {8, 16}) {
            if (want_cap > 0 && cap != want_cap) continue;
            int WX = 1;
            for (int d = std::min(p.NTX, cap); d >= 1; --d) if (p.NTX % d == 0) { WX = d; break; }
            int WY = 1;
            for (int d = std::min(p.NGY, std::max(1, cap / WX)); d >= 1; --d) if (p.NGY % d == 0) { WY = d; break; }
            p.WX = WX; p.WY = WY;
            p.CX = p.NTX / WX; p.CY = p.NGY / WY;
            p.threads = 32 * WX * WY;
            const double tasks = (double)pm.n_left * p.RG * p.CX * p.CY;
            if (tasks > 2.0e9) continue;
            p.LS = p.Wp + 2;
            for (int S = 1; S <= (reproducible ? std::min(H, 2) : H); S = S < 8 ? S + 1 : S + S / 4) {
                if (want_s > 0 && S != want_s) { if (S > want_s) break; continue; }
                p.S = S;                 // (two slices commute: still bit-reproducible; more do not)
                const int RS = (H + S - 1) / S;
                p.nstage = std::min(RS + WY * SL - 1, p.Hp);
                p.RMS = RS * p.Wp + 2;
                p.smem_bytes = ((size_t)p.nstage * p.LS + (size_t)p.ML * p.RMS) * sizeof(double);
                if (p.smem_bytes > smem_limit) continue;
                if (tasks * S > 2.0e9) break;
                // cost in multiply-adds of the busiest SM (padding and dead matrix lanes included): its blocks
                // one after the other at the rate its resident warps sustain (122 registers: two blocks of
                // 8 warps, one of 16), staging bytes and 3 us of latency per round of resident blocks, the memset and the
                // atomic adds of sliced rows as bytes over 7 TB/s, 2 % for a warp that serves one matrix
                // only.  Checked against 37 timed plans of the four benchmark shapes (XCORR_F64_PLAN): the
                // model's choice is the fastest timed plan on three and 2 % behind it on the fourth.
                const double blocks = tasks * S;
                const double busiest = std::ceil(blocks / sm_count);
                const int by_smem = (int)((smem_limit + 1024) / (p.smem_bytes + 1024));
                const int blocks_sm = std::max(1, std::min({by_smem, 65536 / (128 * p.threads), 2048 / p.threads}));
                const double resident = std::min<double>(busiest, blocks_sm) * (p.threads / 32.0);
                const double warps_eff = std::min(1.0, resident / 12.0 + 0.25);
                const double macs_block = (double)p.threads * RS * p.Wp * kDX;
                constexpr double kMacsPerSecond = 125e9;        // DFMA of one SM
                const double out_bytes = (double)pm.n_left * pm.m * (2.0 * H - 1) * (2.0 * W - 1) * sizeof(double);
                // (small blocks stage the same left rows more often and run a few percent behind large ones
                // where all blocks start together: 20 x 20 16 x 64, 3 warps against 15: 42 against 36 us)
                const int warps_blk = p.threads / 32;
                const double block_prior = warps_blk >= 12 ? 1.0 : warps_blk >= 6 ? 0.96 : warps_blk >= 4 ? 0.92 : 0.88;
                double cost = busiest * (macs_block / (warps_eff * block_prior) * (p.ML == 1 ? 1.02 : 1.0) +
                                         2.0 * (double)p.smem_bytes) +
                              std::ceil(busiest / blocks_sm) * 3e-6 * kMacsPerSecond;
                if (S > 1) cost += (S + 1.0) * out_bytes / 7e12 * kMacsPerSecond;
                if (plan_debug)
                    std::fprintf(stderr, "plan64 SL=%d WX=%d WY=%d S=%d grid=%.0f smem=%zu cost=%.3g\n", SL, WX, WY, S, blocks,
                                 p.smem_bytes, cost);
                if (best_cost < 0.0 || cost < best_cost) { best_cost = cost; best = p; best.grid = (unsigned)blocks; }
                if (blocks >= 8.0 * sm_count && S > 1) break;      // finer slices only add staging and atomic adds
            }
        }
    }
    {
        std::lock_guard<std::mutex> lock(cache_mutex);
        if (cache.size() >= 256) cache.clear();
        cache.push_back(Entry{key, best, best_cost >= 0.0});
    }
    if (best_cost < 0.0) return false;
    *out = best;
    return true;
}

cudaError_t launch_tile_f64(const TileArgs64& a, int device, cudaStream_t stream) {
    constexpr int kDevices = 64;
    static std::atomic<size_t> raised[kDevices];
    if (a.p.smem_bytes > 48 * 1024 &&
        !(device >= 0 && device < kDevices && raised[device].load(std::memory_order_relaxed) >= a.p.smem_bytes)) {
        cudaError_t e = cudaFuncSetAttribute(tile_f64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.p.smem_bytes);
        if (e != cudaSuccess) return e;
        if (device >= 0 && device < kDevices) raised[device].store(a.p.smem_bytes, std::memory_order_relaxed);
    }
    tile_f64_kernel<<<a.p.grid, a.p.threads, a.p.smem_bytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace xcorr
