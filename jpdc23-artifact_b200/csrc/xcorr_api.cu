// C ABI of the cross-correlation library: argument checks, per-shape planning, launches,
// the host-buffer and multi-GPU front ends, diagnostics.  See include/xcorr.h for the
// contract of every entry point and the reference interface it stands in for.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "xcorr.h"
#include "xcorr_launch.h"
#include "xcorr_plan.h"

namespace {

using namespace xcorr;

// The last launch of the calling thread.  The hot paths only note what was launched (a copy of
// the plan); the text is made when somebody asks for it -- formatting a plan costs about as much
// host time as enqueuing the kernel of a small input.
struct LaunchNote {
    enum Kind { kText, kTile, kStaged, kWarp } kind = kText;
    TilePlan plan{};
    StagedArgs staged{};
    dim3 grid;
    size_t smem = 0;
    int block = 0, split = 0, rows_per_warp = 0;   // kWarp
};
thread_local LaunchNote t_note;
thread_local std::string t_last_launch = "no kernel launched yet";
void set_launch_text(const std::string& text) { t_note.kind = LaunchNote::kText; t_last_launch = text; }
const std::string& last_launch_text();          // defined after describe_plan
thread_local std::string t_last_error;
thread_local uint64_t t_launch_count = 0;

xcorr_status fail(xcorr_status st, const std::string& msg) {
    t_last_error = msg;
    return st;
}

xcorr_status cuda_fail(cudaError_t e, const char* what) {
    t_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return XCORR_ERR_CUDA;
}

#define XC_CUDA(call)                                           \
    do {                                                        \
        cudaError_t e__ = (call);                               \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call);   \
    } while (0)

// Nothing is thrown across the C boundary: the entry points build strings and vectors and start
// threads, so every body that can do so runs inside this.
template<typename F>
xcorr_status guarded(F&& body) noexcept {
    try {
        return body();
    } catch (const std::bad_alloc&) {
        try { t_last_error = "out of host memory inside the library"; } catch (...) {}
        return XCORR_ERR_INTERNAL;
    } catch (const std::exception& e) {
        try { t_last_error = std::string("host-side failure inside the library: ") + e.what(); } catch (...) {}
        return XCORR_ERR_INTERNAL;
    } catch (...) {
        try { t_last_error = "host-side failure inside the library"; } catch (...) {}
        return XCORR_ERR_INTERNAL;
    }
}

// Restores the caller's current device when an entry point that switches devices returns.
struct DeviceGuard {
    int prev = -1;
    DeviceGuard() { if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); prev = -1; } }
    ~DeviceGuard() { if (prev >= 0) (void)cudaSetDevice(prev); }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

// xcorr_debug_stage_wait: bound and surplus of the tile kernel's staging wait (test hook).
std::atomic<unsigned> g_stage_wait_limit{kStageWaitLimit};
std::atomic<unsigned> g_stage_expect_surplus{0};

struct DeviceInfo {
    int sm_count = 0;
    size_t smem_optin = 0;
    bool valid = false;
};

constexpr int kMaxDevices = 64;
DeviceInfo g_dev_info[kMaxDevices];
std::mutex g_dev_info_mutex;

xcorr_status current_device_info(DeviceInfo* out, int* dev_out = nullptr) {
    int dev = 0;
    XC_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(XCORR_ERR_DEVICE, "device index out of range");
    std::lock_guard<std::mutex> lock(g_dev_info_mutex);
    DeviceInfo& d = g_dev_info[dev];
    if (!d.valid) {
        int v = 0;
        XC_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        d.sm_count = v;
        XC_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        d.smem_optin = (size_t)v;
        d.valid = true;
    }
    *out = d;
    if (dev_out) *dev_out = dev;
    return XCORR_OK;
}

// Planning never needs a device: without one it assumes a B200 (148 SMs, 227 KB).
DeviceInfo assumed_device() {
    DeviceInfo d;
    d.sm_count = 148;
    d.smem_optin = kSmemLimit;
    d.valid = true;
    return d;
}

bool pair_map(int32_t mode, uint32_t n_left, uint32_t n_right, PairMap* pm) {
    switch (mode) {
    case XCORR_ONE_TO_ONE:
        if (n_left != 1 || n_right != 1) return false;
        *pm = PairMap{1, 1, 0};
        return true;
    case XCORR_ONE_TO_MANY:
        if (n_left != 1 || n_right == 0) return false;
        *pm = PairMap{1, n_right, 0};
        return true;
    case XCORR_N_TO_MN:
        if (n_left == 0 || n_right == 0 || n_right % n_left != 0) return false;
        *pm = PairMap{n_left, n_right / n_left, n_right / n_left};
        return true;
    case XCORR_N_TO_M:
        if (n_left == 0 || n_right == 0) return false;
        *pm = PairMap{n_left, n_right, 0};
        return true;
    default:
        return false;
    }
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }
int ilog2(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }
bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

int largest_divisor_at_most(int n, int cap) {
    for (int d = std::min(n, cap); d >= 1; --d)
        if (n % d == 0) return d;
    return 1;
}

// Fill the fields that follow from (TY, SL, WX, WY, S).
void finish_plan(TilePlan& p, const PairMap& pm, size_t smem_limit = kSmemLimit) {
    p.ML = 32 / p.SL;
    p.logSL = ilog2(p.SL);
    p.Wp = round_up(p.W, kTX);
    p.Hp = round_up(p.H, p.SL * p.TY);
    p.NTX = p.Wp / kTX;
    p.NCH = p.Wp / 8;
    p.NGY = p.Hp / (p.SL * p.TY);
    p.CX = (p.NTX + p.WX - 1) / p.WX;
    p.CY = (p.NGY + p.WY - 1) / p.WY;
    p.RSmax = (p.H + p.S - 1) / p.S;
    p.RG = (int)((pm.m + p.ML - 1) / p.ML);
    const int cls_per_block = p.schedule == kSchedWarpQueue ? p.Hp : p.WY * p.SL * p.TY;
    p.nstage = std::min(p.RSmax + cls_per_block - 1, p.Hp);
    p.LS = p.Wp + 4;
    p.RMS = round_up(p.RSmax * p.Wp, 32) + 4;
    p.threads = 32 * p.WX * p.WY;
    // the fused row engine exists for 32 padded columns and 1 class per thread
    // ... and not for stream-K, whose segments of a few rows do not repay fetching its long straight-line
    // code (32 x 32 8 x 8: 16.8 against 14.4 us)
    if (p.Wp != 32 || p.TY != 1 || p.schedule == kSchedStreamK) p.fused = 0;
    // staged left rows and per-warp flush staging (+ the warp queue's counter and the staging barrier)
    const size_t left_bytes = (size_t)p.nstage * p.LS * sizeof(float);
    const size_t rest = (size_t)(p.threads / 32) * kFlushBytesPerWarp + 16;
    const size_t per_group = (size_t)p.ML * p.RMS * sizeof(float);
    // The warp queue stages as many matrix groups together as fit (a round of its tasks); a round may
    // run on into the groups of the next left matrices, each of which needs staged rows of its own.
    p.KG = 1; p.KL = 1;
    if (p.schedule == kSchedWarpQueue) {
        for (int kl = std::min<int>((int)pm.n_left, 4); kl >= 1; --kl) {
            if (smem_limit < (size_t)kl * left_bytes + rest + per_group) continue;
            const int kg = (int)std::min<size_t>(16, (smem_limit - (size_t)kl * left_bytes - rest) / per_group);
            // lefts that kg consecutive groups can touch
            const int need = std::min<int>((int)pm.n_left, (kg + p.RG - 2) / p.RG + 1);
            if (kl > need) continue;                       // fewer slots do, more room for groups
            p.KL = kl;
            p.KG = std::max(1, std::min(kg, pm.n_left == 1 ? p.RG : kg));
            break;
        }
    }
    const size_t fixed = (size_t)p.KL * left_bytes + rest;
    p.smem_bytes = fixed + (size_t)p.KG * per_group;
}

// Workspace of a stream-K plan with fix-up: `pieces` partial images, then one counter per task.
size_t fixup_counters_offset(int pieces, unsigned long long total_out) {
    return ((size_t)pieces * total_out * sizeof(float) + 255) / 256 * 256;
}

// Per-shape plan of the tile kernel: micro-tile height, lane split, block shape and how the
// right rows are divided -- none (one block per task, plain stores), S equal slices per task
// (partials combined by atomics or through the workspace) or stream-K (the (task, row)
// units of all tasks cut evenly over as many blocks as fit on the GPU; a block's share is a
// run of whole tasks plus at most two partial ones, partial ones added atomically).
// Every candidate gets an estimated time; the smallest wins.
xcorr_status plan_tile_search(const PairMap& pm, int H, int W, const xcorr_hints* h, const DeviceInfo& dev,
                              TilePlan* out, size_t max_workspace_bytes) {
    TilePlan best{}, best_queue{}, best_queue_few{};   // best_queue*: the warp queue as a candidate of the automatic choice
    double best_time = -1.0, best_queue_time = -1.0, best_queue_few_time = -1.0;
    const int want_ty = h ? h->overlap_rows : 0;
    const int want_sl = h ? h->class_lanes : 0;
    if (want_ty < 0 || want_ty > kMaxTY) return fail(XCORR_ERR_INVALID_HINT, "overlap_rows must be 0..4");
    if (want_sl != 0 && (!is_pow2(want_sl) || want_sl > 32))
        return fail(XCORR_ERR_INVALID_HINT, "class_lanes must be 0 or a power of two <= 32");
    const int want_wx = h ? h->warps_x : 0, want_wy = h ? h->warps_y : 0;
    if (want_wx < 0 || want_wy < 0 || (want_wx ? want_wx : 1) * (want_wy ? want_wy : 1) > kMaxWarps)
        return fail(XCORR_ERR_INVALID_HINT, "warps_x * warps_y must be 1..16");
    const int want_s = h ? h->row_slices : 0;
    if (want_s < 0 || want_s > H) return fail(XCORR_ERR_INVALID_HINT, "row_slices must be 0..rows");
    const int want_combine = h ? h->combine : 0;
    if (want_combine < 0 || want_combine > 3) return fail(XCORR_ERR_INVALID_HINT, "unknown combine mode");
    const int want_fused = h ? h->fused_rows : 0;
    if (want_fused < 0 || want_fused > 2) return fail(XCORR_ERR_INVALID_HINT, "fused_rows must be 0 (auto), 1 (on) or 2 (off)");
    const int want_sched = h ? h->schedule : 0;
    if (want_sched < 0 || want_sched > 3)
        return fail(XCORR_ERR_INVALID_HINT, "schedule must be 0 (auto), 1 (static), 2 (stream-K) or 3 (warp queue)");
    if (want_sched == kSchedStreamK && (want_s > 1 || want_combine == XCORR_COMBINE_STORE))
        return fail(XCORR_ERR_INVALID_HINT, "schedule=2 (stream-K) excludes row_slices > 1 and combine=store");
    if (want_sched == kSchedWarpQueue &&
        (want_s > 1 || want_combine == XCORR_COMBINE_ATOMIC || want_combine == XCORR_COMBINE_WORKSPACE))
        return fail(XCORR_ERR_INVALID_HINT, "schedule=3 (warp queue) writes with plain stores: no row_slices, no atomic/workspace");
    if (want_combine == XCORR_COMBINE_STORE && want_s > 1)
        return fail(XCORR_ERR_INVALID_HINT, "combine=store needs row_slices=1");

    static const bool env_reproducible = [] {
        const char* e = std::getenv("XCORR_REPRODUCIBLE");
        return e && e[0] == '1';
    }();
    const bool reproducible = env_reproducible || (h && h->reproducible == 1);
    static const bool plan_debug = std::getenv("XCORR_PLAN_DEBUG") != nullptr;   // candidates and estimates to stderr
    const double out_bytes = (double)pm.n_left * pm.m * (2.0 * H - 1) * (2.0 * W - 1) * 4.0;
    // Fitted to ~1500 timed plans over 19 shapes on B200: 1 and 2 y classes per thread run the
    // inner loop about equally fast (the per-row cost below aside), 3 and 4 classes slower
    // (register pressure; 64 x 64 x 512: 404 against 361 us).  Plans of 1 class win wherever their
    // shorter warp tasks and fewer flushes per task matter: anything that does not fill the GPU
    // many times over.
    static const double ty_eff[5] = {0.0, 0.97, 0.98, 0.93, 0.85};
    // issue slots one output flush costs, in FFMA-equivalents (fitted to measured plan timings)
    const double kFlushSlots = 150.0;
    // latency of a lone warp's row, besides its chunks (a 16 x 16 batch in one static block of 16
    // rows: 14 us measured, against 10 us when the rows are spread over 16 blocks)
    const double kRowBase = 550.0;
    // issue slots of the per-row code of a warp (two passes: addresses, ranges, the first window),
    // which weigh on narrow matrices and small tiles: 32 x 32, saturated, 1 class per thread runs
    // 13..30 % slower than 2 classes; at 64 x 64 they are level
    const double kRowSlots = 50.0;

    for (int TY = 1; TY <= kMaxTY; ++TY) {
        if (want_ty && TY != want_ty) continue;
        for (int SL = 1; SL <= 32; SL *= 2) {
            if (want_sl && SL != want_sl) continue;
            TilePlan p{};
            p.H = H; p.W = W; p.TY = TY; p.SL = SL; p.WX = 1; p.WY = 1; p.S = 1; p.schedule = kSchedStatic;
            p.fused = want_fused != 2;
            finish_plan(p, pm);
            // block shapes: x tiles first, y groups after that, up to 16 warps; the warp
            // queue only needs a warp count (WX = warps, WY = 1)
            struct Cand { int WX, WY, S, sched; };
            std::vector<Cand> cands;
            const bool static_ok = want_sched == 0 || want_sched == kSchedStatic;
            const bool streamk_ok = (want_sched == 0 || want_sched == kSchedStreamK) && want_s <= 1 &&
                                    want_combine != XCORR_COMBINE_STORE &&
                                    !(want_sched == 0 && want_combine == XCORR_COMBINE_WORKSPACE);
            // The warp queue (pass tasks of unequal length taken longest first by the warps of one
            // resident wave of blocks; plain stores, bit-reproducible) is a candidate of the automatic
            // choice too: it removes the wave quantisation of a few hundred equal block tasks on 148
            // SMs.  Measured on B200 it wins where every warp gets two or more tasks (64 x 64 x 512:
            // 351 against 371 us; 48 x 48 4 x 128: 131 against 148 us) and loses where a warp gets
            // about one (64 x 64 x 128: 120 against 108 us of stream-K), so those are left out.
            const bool queue_auto = want_sched == 0 && want_s <= 1 && want_combine == XCORR_COMBINE_AUTO &&
                                    !want_wx && !want_wy;
            const bool queue_ok = (want_sched == kSchedWarpQueue || queue_auto) && want_s <= 1 &&
                                  want_combine != XCORR_COMBINE_ATOMIC && want_combine != XCORR_COMBINE_WORKSPACE;
            std::vector<std::pair<int, int>> shapes;
            if (want_wx && want_wy) {
                shapes.emplace_back(want_wx, want_wy);
            } else {
                for (int cap : {4, 8, 16}) {
                    int WX = want_wx ? want_wx : largest_divisor_at_most(p.NTX, cap);
                    int WY = want_wy ? want_wy : largest_divisor_at_most(p.NGY, std::max(1, cap / WX));
                    if (WX * WY <= kMaxWarps) shapes.emplace_back(WX, WY);
                }
            }
            for (const auto& shape : shapes) {
                if (static_ok) {
                    const int s_lo = want_s ? want_s : 1;
                    const int s_hi = want_s ? want_s : std::min(H, 64);
                    for (int S = s_lo; S <= s_hi; ++S) cands.push_back({shape.first, shape.second, S, kSchedStatic});
                    // wide matrices: a staged left row is several KB, so only short runs of rows
                    // fit in shared memory -- finer slices, in steps of about 1.5x up to one row each
                    if (!want_s)
                        for (int S = 96; S / 3 * 2 < H; S = S * 3 / 2)
                            if (std::min(S, H) > 64) cands.push_back({shape.first, shape.second, std::min(S, H), kSchedStatic});
                }
                if (streamk_ok) cands.push_back({shape.first, shape.second, 1, kSchedStreamK});
            }
            if (queue_ok) {
                if (want_wx || want_wy) {
                    const int nw = (want_wx ? want_wx : 1) * (want_wy ? want_wy : 1);
                    cands.push_back({nw, 1, 1, kSchedWarpQueue});
                } else {
                    for (int nw : {8, 12, 16})
                        if (!queue_auto || nw >= 12) cands.push_back({nw, 1, 1, kSchedWarpQueue});
                }
            }

            const double sm_rate = 128.0 * 1.8e9 * 0.8;
            for (const Cand& c : cands) {
                p.WX = c.WX; p.WY = c.WY; p.S = c.S; p.schedule = c.sched;
                p.fused = want_fused != 2;                 // (finish_plan clears it where the fused rows do not apply)
                finish_plan(p, pm, dev.smem_optin);
                if (p.smem_bytes > dev.smem_optin) continue;
                if (c.sched == kSchedStatic && want_combine == XCORR_COMBINE_WORKSPACE &&
                    (double)c.S * out_bytes > (double)max_workspace_bytes) continue;
                const double groups = (double)pm.n_left * p.RG;
                const double tasks = c.sched == kSchedWarpQueue ? groups : groups * p.CX * p.CY;
                if (tasks * c.S > 2147483647.0 || groups * p.NGY * p.NTX > 4.0e9) continue;
                // resident warps per SM (1 KB of shared memory reserved per block): below ~12
                // the FFMA pipe idles on shared-memory latency
                const int by_smem = (int)((dev.smem_optin + 1024) / (p.smem_bytes + 1024));
                const int regs = (p.threads <= kSmallBlockThreads && TY >= 3) ? 168 : 128;
                const int by_regs = 65536 / (regs * p.threads);
                const int blocks_sm = std::max(1, std::min(by_smem, by_regs));
                const int resident = blocks_sm * (p.threads / 32);
                const double occ_eff = std::min(1.0, 0.4 + 0.05 * resident);
                // shared-memory wavefronts per 8-step chunk against its FFMA issue slots
                const double wavefronts = 2.0 * TY * std::max(1, p.SL / 8) + 6.0 * std::max(1, p.ML / 8);
                const double smem_util = 4.0 * wavefronts / (8.0 * TY * kTX);
                // (fused rows load a right row once per row and 8 left values: a few wavefronts per 512 FFMA)
                const double smem_eff = p.fused ? 1.0 : 1.0 / (1.0 + std::max(0.0, smem_util - 0.4));
                // measured on B200 over the plan space of the benchmark shapes: large blocks
                // (12..16 warps sharing one staging) and many right matrices per warp run
                // up to ~15 % faster than small blocks / few matrices per warp
                const int warps_blk = p.threads / 32;
                // (fused rows lose less in four-warp blocks: 28 x 28 1 x 1000 runs 43 us in 441 blocks of four
                // warps, 50 us in 128 blocks of fourteen)
                const double block_prior = warps_blk >= 12 ? 1.0 : warps_blk >= 8 ? 0.93 : warps_blk >= 4 ? (p.fused ? 0.92 : 0.87) : 0.8;
                const double lanes_prior = p.ML >= 8 ? 1.0 : p.ML == 4 ? 0.96 : p.ML == 2 ? 0.92 : 0.9;
                // blocks of more than 384 threads run the 128-register build, which spills for
                // TY = 4 (and a little for TY = 3): measured 28 against 47 TFLOP/s on 64 x 64 x 512
                const double build_eff = p.threads > kSmallBlockThreads ? (TY == 4 ? 0.6 : TY == 3 ? 0.9 : 1.0) : 1.0;
                // (fused 32-column rows: one visit per row, straight-line code)
                const double tile_eff = p.fused ? 0.96 / (1.0 + 20.0 / ((double)p.Wp * TY * kTX))
                                                : ty_eff[TY] / (1.0 + kRowSlots / ((double)p.Wp * TY * kTX));
                const double rate = sm_rate * tile_eff * occ_eff * smem_eff * block_prior * lanes_prior * build_eff;
                // filling the staging buffers: bytes over ~64 B/clk from L2 plus a latency
                // chain, paid once per block (per segment / phase)
                // (rows whose length is no multiple of four floats are staged word by word by the block's
                // own threads, ~120 cycles per word and thread: 17 x 30 1 x 100 in two-warp blocks that stage
                // 70 KB each took 34 us, 14 us in blocks of ten warps)
                const double stage_cycles = W % 4 == 0 ? (double)p.smem_bytes / 64.0 + 2000.0
                                                       : (double)p.smem_bytes / 4.0 / p.threads * 120.0 + 2000.0;
                const double t_stage = stage_cycles / 1.9e9;
                double t;
                int comb;
                int sk_parts = 0;
                unsigned grid;
                bool queue_few_tasks = false;
                if (c.sched == kSchedWarpQueue) {
                    // pass tasks (one pass of one warp tile, all rows) of unequal lengths, cut evenly by
                    // weight over one resident wave of blocks and taken longest first by the warps
                    const double units = groups * p.NGY * (double)queue_units_per_yrow(p.NTX);   // quarter chunks per row
                    const double ptasks = groups * p.NGY * (p.fused ? 1.0 : 2.0) * p.NTX;
                    double G = (double)dev.sm_count * blocks_sm;
                    if (G > ptasks) G = ptasks;
                    grid = (unsigned)G;
                    // multiply-adds of a block's share (as the other schedules count them) and of its
                    // longest task; every round ends with the schedulers waiting for the last of its tasks:
                    // a fraction of a longest task each (fitted to 16 timed plans of the benchmark shapes
                    // and their shards)
                    (void)units;
                    const double macs_block = groups * p.NGY * p.NTX * 32.0 * H * p.Wp * TY * kTX / G;
                    const double longest = 32.0 * H * TY * kTX * (p.fused ? (double)p.Wp : 8.0 * (p.NCH - 1));
                    const double rounds = std::ceil((groups / G + 1.0) / p.KG);
                    // (the tile's own two chunks run as triangles with reloaded windows: dearer on narrow rows)
                    // (fused rows: 1.07 from seven timed shapes of 20..32 columns, 31 us .. 190 us)
                    const double narrow = p.fused ? 1.07 : 1.0 + 0.5 / ((double)p.NTX * p.NTX);
                    // One class per thread has half the independent FFMA of two: with 12 resident warps it ran
                    // 2-3 % behind 16 (64 x 64 1 x 512: 360 against 352 us; 32 x 32 32 x 64 fused: 103 against
                    // 101 us; 16 x 16 100 x 4000: 33 against 29 us) -- where the tasks are of one length or a block
                    // has 30 and more of them (48 x 48 4 x 128, 31 per block: 133 against 131 us).  With fewer
                    // tasks of unequal length 16 warps leave the longest ones nothing to pair with (64 x 64
                    // 1 x 256, 28 per block: 194 us with 12 warps, 201 with 16).
                    const bool level_tasks = p.fused || p.NTX == 1 || ptasks / G >= 30.0;
                    const double rate_q = rate * (TY == 1 && resident < 16 && level_tasks ? 0.97 : 1.0);
                    const double t_rate = std::ceil(G / dev.sm_count) *
                                          ((macs_block * narrow + rounds * 4.0 * 0.4 * longest) / rate_q + rounds * t_stage);
                    const double t_serial = std::ceil(ptasks / G / warps_blk) * H * p.Wp * TY * kTX / 1.8e9;
                    t = std::max(t_rate, t_serial);
                    if (queue_auto && ptasks / G < 1.25 * warps_blk) continue;  // about one task per warp: the tail decides
                    queue_few_tasks = ptasks / G < 24.0;      // fewer than six per scheduler
                    comb = kStore;
                } else if (c.sched == kSchedStreamK) {
                    const double units = tasks * H;
                    double G = (double)dev.sm_count * blocks_sm;
                    if (G > units) G = units;
                    grid = (unsigned)G;
                    const double rows_per_block = units / G;
                    const double macs_per_row = (double)p.threads * p.Wp * TY * kTX;
                    // every block: its rows, plus a fixed cost per segment (staging, flush)
                    const double segments = rows_per_block / H + 1.0;
                    const double sk_flush_share = segments * 2.0 * (std::min<double>(p.SL * TY, rows_per_block) + TY) *
                                                  kFlushSlots / (rows_per_block * p.Wp * TY * kTX);
                    // (the staging of blocks resident together overlaps; their arithmetic shares the SM)
                    const double t_rate = std::ceil(G / dev.sm_count) * (rows_per_block + 0.25 * segments) *
                                          macs_per_row / rate * (1.0 + sk_flush_share) + segments * t_stage;
                    // the lone-warp latency bound of the static branch, per segment
                    const double sk_flushes = 2.0 * (std::min<double>(p.SL * TY, rows_per_block) + TY) * segments;
                    const double sk_row_cycles = kRowBase + (p.NCH + 2) * 40.0 + (double)p.Wp * TY * kTX;
                    const double t_serial = (rows_per_block * sk_row_cycles + sk_flushes * 500.0 +
                                             std::max(4000.0, stage_cycles) * segments) / 1.9e9;
                    // every block boundary splits one task; a split task is added atomically twice
                    // (measured on B200 with the coalesced flush: ~3.4 TB/s of atomic traffic, the
                    // memset of the output ~5 TB/s)
                    const double split_share = std::min(1.0, G / tasks);
                    // more than two parts of a task do not commute: last bits then vary run to run
                    // (a price put on reproducibility: such a plan must win by a clear margin).  Whole-task
                    // plans still pay for zeroing and re-reading an output that is not in L2, which
                    // the timings these constants were fitted to (same buffers replayed) do not show:
                    // 64 x 64 x 512 from a cold cache, 0.373 ms against 0.367 ms of the static plan.
                    const double order_penalty = rows_per_block >= H ? 1.03 : 1.06;
                    // most parts any task is cut into: a task of H rows over ranges of at least rpb rows
                    const double rpb = std::floor(units / G);
                    const int parts = (int)((H - 1) / std::max(1.0, rpb)) + 2;
                    // Only on request (combine = workspace): measured on B200 the sum of the parts by
                    // the last block to finish a task sits at the end of that block's work and costs
                    // more than zeroing the output and adding atomically (64 x 64 x 512: 0.387 against
                    // 0.366 ms; 48 x 48 x 2048: 0.483 against 0.448 ms).  What it buys is results that
                    // are bit-reproducible however many parts a task is cut into.
                    const bool fixup = want_combine == XCORR_COMBINE_WORKSPACE &&
                                       (double)parts * out_bytes + tasks * 4.0 + 64.0 <= (double)max_workspace_bytes;
                    if (fixup) {
                        // parts go to partial images with plain stores and are summed in a fixed order by
                        // the block that finishes the task last: two more writes and two reads of a cut
                        // task's results, mostly from L2, under the other blocks' arithmetic
                        // ... and the sum itself is latency-bound: a warp takes two result rows per
                        // round of ~600 cycles per four parts; a block finishes about G/tasks tasks
                        const double fix_rows = (double)p.ML * p.WY * p.SL * TY * 2.0;
                        const double t_fix = std::min(1.0, tasks / G) * std::max(1.0, G / tasks) *
                                             std::ceil(fix_rows / (2.0 * warps_blk)) * std::ceil(parts / 4.0) * 600.0 / 1.9e9;
                        t = std::max(t_rate, t_serial) + 3e-6 + split_share * 4.0 * out_bytes / 5e12 + t_fix;
                        comb = kFixup;
                        sk_parts = parts;
                    } else {
                        if (reproducible && parts > 2) continue;      // three or more atomic addends per result
                        t = (std::max(t_rate, t_serial) + 5e-6 + out_bytes / 5e12 + split_share * 2.0 * out_bytes / 3.4e12) *
                            order_penalty;
                        comb = kAtomic;
                        sk_parts = 0;
                    }
                } else {
                    const int S = c.S;
                    const double rs = (double)H / S;
                    const double macs_per_block = (double)p.threads * rs * p.Wp * TY * kTX;
                    const double busiest = std::ceil(tasks * S / dev.sm_count);
                    // issue slots of the output flushes (kFlushSlots each: SL * TY wrap
                    // flushes and TY final ones per pass) relative to the FFMA of a warp's slice
                    const double flush_share = 2.0 * (std::min<double>(p.SL * TY, rs) + TY) * kFlushSlots /
                                               (rs * p.Wp * TY * kTX);
                    // (fewer blocks than would be resident: the SM's rate is that of the warps it really holds.
                    // Fused rows only, where the lone-warp bound below no longer hides it: 32 x 32 4 x 64 in 128
                    // four-warp blocks runs the same 22.9 us with 47 KB or 80 KB of shared memory per block)
                    const double held = std::min<double>(blocks_sm, busiest) * (p.threads / 32);
                    // (a lone fused warp per scheduler keeps 3/4 of the rate of four: 32 x 32 4 x 64 against 32 x 64)
                    const double rate_s = p.fused ? rate / occ_eff * std::min(1.0, 0.67 + 0.0208 * held) : rate;
                    const double t_rate = busiest * macs_per_block / rate_s * ((rs + 0.25) / rs + flush_share) +
                                          std::ceil(busiest / blocks_sm) * t_stage;
                    // A lone warp is bound by latency, not by the SM's FFMA rate: per right row its
                    // FFMAs one per clock plus ~150 cycles of row overhead per pass and ~40 per
                    // chunk visit, ~500 cycles per output flush (SL * TY wrap flushes and TY final
                    // ones per pass), ~4000 for the staging.  This decides the plan of tiny inputs
                    // (16 x 16: many small warps tasks with few flushes beat one full warp).
                    const double flushes = 2.0 * (std::min<double>(p.SL * TY, rs) + TY);
                    // (fused rows: one visit per row, no windows -- the row's FFMA plus ~60 cycles; timed on
                    // 32 x 32 1 x 32 in four-warp blocks: 11.3 us in all, ~530 cycles per row)
                    const double row_cycles = p.fused ? 60.0 + (double)p.Wp * TY * kTX
                                                      : kRowBase + (p.NCH + 2) * 40.0 + (double)p.Wp * TY * kTX;
                    const double t_serial = (rs * row_cycles + flushes * 500.0 + std::max(4000.0, stage_cycles)) / 1.9e9;
                    comb = want_combine;
                    if (comb == XCORR_COMBINE_AUTO) {
                        comb = S == 1 ? kStore : S == 2 ? kAtomic : kWorkspace;
                        // partial images beyond a few GB (very fine slices of a large result): atomics
                        if (comb == kWorkspace && (double)S * out_bytes > std::min((double)max_workspace_bytes, 4.0 * (1ull << 30)))
                            comb = kAtomic;
                    }
                    if (reproducible && comb == kAtomic && S > 2) continue;
                    // a memset or a second kernel in front of / behind the main one costs a few us
                    double t_combine = 0.0;
                    if (comb == kAtomic) t_combine = 5e-6 + out_bytes / 3e12 + S * out_bytes / 0.4e12;
                    else if (comb == kWorkspace) t_combine = 9e-6 + (2.0 * S + 1.0) * out_bytes / 3e12;
                    t = std::max(t_rate, t_serial) + t_combine;
                    grid = (unsigned)(tasks * S);
                }
                if (plan_debug)
                    std::fprintf(stderr, "plan TY=%d SL=%d WX=%d WY=%d S=%d sched=%d comb=%d grid=%u t=%.2f us\n", TY, SL, c.WX,
                                 c.WY, c.S, c.sched, comb, grid, t * 1e6);
                const bool auto_queue_cand = queue_auto && c.sched == kSchedWarpQueue;
                // (queue candidates with fewer than six tasks per scheduler only compete against stream-K)
                const bool few = auto_queue_cand && queue_few_tasks;
                TilePlan& slot = few ? best_queue_few : auto_queue_cand ? best_queue : best;
                double& slot_time = few ? best_queue_few_time : auto_queue_cand ? best_queue_time : best_time;
                if (slot_time < 0.0 || t < slot_time * 0.9999) {
                    slot_time = t;
                    slot = p;
                    slot.combine = comb;
                    slot.pieces = sk_parts;
                    slot.grid = grid;
                    slot.tasks = (unsigned)tasks;
                }
            }
        }
    }
    // The automatic choice takes the warp queue only against a static plan that leaves a good part of
    // its last wave of blocks empty (128 equal blocks on 148 SMs): that is the loss the queue removes.
    // Against stream-K, which is balanced by construction, it measured slower on the dominant benchmark
    // shape (48 x 48 16 x 128: 460 against 447 us) although the estimates are level.
    if (best_time >= 0.0 && best.schedule == kSchedStreamK) {
        // ... except where stream-K's ranges are a few rows each (a block re-stages and flushes for every
        // one): the queue is taken if its estimate is 8 % better (48 x 48 2 x 128: 74 against 84 us,
        // 4 x 128: 131 against 148 us), also with between one and two tasks per warp
        if (best_queue_few_time >= 0.0 && (best_queue_time < 0.0 || best_queue_few_time < best_queue_time)) {
            best_queue = best_queue_few; best_queue_time = best_queue_few_time;
        }
        if (best_queue_time >= 0.0 && best_queue_time < 0.92 * best_time) { best = best_queue; best_time = best_queue_time; }
    } else if (best_queue_time >= 0.0) {
        bool take = best_time < 0.0;
        if (!take && best.schedule == kSchedStatic) {
            const double blocks = (double)best.tasks * best.S;
            const double wave_fill = blocks / (std::ceil(blocks / dev.sm_count) * dev.sm_count);
            take = wave_fill < 0.9 && best_queue_time < best_time;
            // ... or, with rows of 32 padded columns and more, where the estimates of the two schedules
            // track their measured ratio within 2 %, a queue estimated 6 % faster (32 x 32 1 x 4000:
            // estimated 195 against 210 us, measured 194 against 210 us)
            if (!take && best.Wp >= 32) take = best_queue_time < 0.94 * best_time;
        }
        if (take) { best = best_queue; best_time = best_queue_time; }
    } else if (best_time < 0.0 && best_queue_few_time >= 0.0) {
        best = best_queue_few; best_time = best_queue_few_time;
    }
    if (best_time < 0.0)
        return fail(XCORR_ERR_UNSUPPORTED, "no tile plan fits in shared memory for this shape / these hints");

    const unsigned long long total_out = (unsigned long long)pm.n_left * pm.m *
                                         (2ull * H - 1) * (2ull * W - 1);
    best.workspace_bytes = best.combine == kWorkspace ? (size_t)best.S * total_out * sizeof(float) :
                           best.combine == kFixup ? fixup_counters_offset(best.pieces, total_out) + (size_t)best.tasks * 4 : 0;
    *out = best;
    return XCORR_OK;
}

// The search above looks at a few thousand candidates (~0.1 ms of host time), which is as
// long as the kernel of a small input: plans are remembered per (shape, counts, hints, device).
struct PlanKey {
    uint32_t n_left, m, right_stride;
    int H, W;
    int hint[7];
    int sm_count;
    size_t smem_optin, max_ws;
    bool operator==(const PlanKey& o) const {
        return n_left == o.n_left && m == o.m && right_stride == o.right_stride && H == o.H && W == o.W &&
               std::memcmp(hint, o.hint, sizeof hint) == 0 && sm_count == o.sm_count &&
               smem_optin == o.smem_optin && max_ws == o.max_ws;
    }
};
constexpr int kPlanCacheSize = 64;
struct PlanCache {
    std::mutex mutex;
    PlanKey key[kPlanCacheSize];
    TilePlan plan[kPlanCacheSize];
    int used = 0, next = 0;
};
PlanCache g_plan_cache;

xcorr_status plan_tile(const PairMap& pm, int H, int W, const xcorr_hints* h, const DeviceInfo& dev,
                       TilePlan* out, size_t max_workspace_bytes = SIZE_MAX) {
    PlanKey k{};
    k.n_left = pm.n_left; k.m = pm.m; k.right_stride = pm.right_stride; k.H = H; k.W = W;
    if (h) {
        k.hint[0] = h->overlap_rows; k.hint[1] = h->class_lanes; k.hint[2] = h->warps_x; k.hint[3] = h->warps_y;
        k.hint[4] = h->row_slices;   k.hint[5] = h->combine;
        k.hint[6] = h->schedule + 16 * (h->reproducible == 1) + 32 * h->fused_rows;
    }
    k.sm_count = dev.sm_count; k.smem_optin = dev.smem_optin; k.max_ws = max_workspace_bytes;
    {
        std::lock_guard<std::mutex> lock(g_plan_cache.mutex);
        for (int i = 0; i < g_plan_cache.used; ++i)
            if (g_plan_cache.key[i] == k) { *out = g_plan_cache.plan[i]; return XCORR_OK; }
    }
    const xcorr_status st = plan_tile_search(pm, H, W, h, dev, out, max_workspace_bytes);
    if (st != XCORR_OK) return st;
    std::lock_guard<std::mutex> lock(g_plan_cache.mutex);
    const int slot = g_plan_cache.used < kPlanCacheSize ? g_plan_cache.used++ : (g_plan_cache.next++ % kPlanCacheSize);
    g_plan_cache.key[slot] = k;
    g_plan_cache.plan[slot] = *out;
    return XCORR_OK;
}

int pick_kernel(const xcorr_hints* h) {
    const int k = h ? h->kernel : XCORR_KERNEL_AUTO;
    return k == XCORR_KERNEL_AUTO ? XCORR_KERNEL_TILE : k;
}

// The automatic choice for a handful of small overlaps (one 16 x 16 pair has 961, one 32 x 32
// pair 3969): one warp per overlap straight from global memory, lanes over columns x rows with
// eight rows of loads in flight -- the latency kernel.  As CUDA-graph replays it takes 2.2 us at
// 16 x 16, 3.1 us at 24 x 24 and 3.7 us at 32 x 32 (the tile kernel: 10.2, 6.2 and 7.2 us), 4.8 us
// for eight 16 x 16 pairs (tile: 7.8 us); past 32 rows or columns an overlap takes several
// dependent trips to L2 and the tile kernel wins (40 x 40: 6.9 against 7.2 us, 48 x 48: 11.6
// against 8.0 us).  Not for callers who asked for specific plans.
constexpr double kTinyOverlaps = 8000.0;
bool tiny_auto(const xcorr_hints* h, const PairMap& pm, uint32_t rows, uint32_t cols) {
    if (h && (h->kernel != XCORR_KERNEL_AUTO || h->combine || h->overlap_rows || h->class_lanes || h->warps_x ||
              h->warps_y || h->row_slices || h->schedule || h->block_threads))
        return false;
    if (rows > 32 || cols > 32) return false;
    return (double)pm.n_left * pm.m * (2.0 * rows - 1) * (2.0 * cols - 1) <= kTinyOverlaps;
}

xcorr_status check_sizes(int32_t mode, uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                         PairMap* pm) {
    if (rows == 0 || cols == 0) return fail(XCORR_ERR_INVALID_SIZE, "rows and cols must be positive");
    if (rows > 16384 || cols > 16384) return fail(XCORR_ERR_INVALID_SIZE, "rows and cols are limited to 16384");
    if (!pair_map(mode, n_left, n_right, pm))
        return fail(XCORR_ERR_INVALID_SIZE, "matrix counts do not fit the mode "
                    "(one_to_one 1x1, one_to_many 1xN, n_to_mn N x k*N, n_to_m NxM)");
    return XCORR_OK;
}

// Arguments of the staged warp-per-overlap kernel from the hints (0 = automatic).  The reference
// requires shared_mem_rows >= shifts_per_thread_block (one_to_one.hpp:573-586); this kernel
// takes any slab height.
xcorr_status staged_args(const PairMap& pm, int H, int W, const xcorr_hints* h, const DeviceInfo& dev, StagedArgs* out) {
    StagedArgs a{};
    a.H = H; a.W = W; a.pm = pm;
    const int bt = h ? h->block_threads : 0;
    if (bt != 0 && (bt < 32 || bt > 1024 || bt % 32 != 0))
        return fail(XCORR_ERR_INVALID_HINT, "block_threads must be a multiple of 32 in 32..1024");
    a.shifts = bt ? bt / 32 : 8;
    const int want_rows = h ? h->staged_rows : 0, want_cols = h ? h->staged_cols : 0, want_r = h ? h->staged_rights : 0;
    if (want_rows < 0 || want_cols < 0 || want_r < 0 || want_r > 8)
        return fail(XCORR_ERR_INVALID_HINT, "staged_rows / staged_cols must be positive, staged_rights 1..8 (0 = automatic)");
    a.scols = std::min(want_cols ? want_cols : 32, W);
    a.srows = std::min(want_rows ? want_rows : std::max(a.shifts, 32), H);
    a.rights = (int)std::min<uint32_t>((uint32_t)(want_r ? want_r : 8), pm.m);
    a.col_groups = h && h->staged_column_groups ? 1 : 0;
    a.warp_rows = h && h->staged_warp_rows ? 1 : 0;
    a.groups_per_left = (pm.m + (uint32_t)a.rights - 1) / (uint32_t)a.rights;
    if (staged_smem_bytes(a) > dev.smem_optin) {
        char msg[200];
        std::snprintf(msg, sizeof msg, "the staged slabs (2 x (%d + %d - 1 + %d * %d) rows x %d columns) need %zu bytes of "
                      "shared memory, the device has %zu", a.srows, a.shifts, a.rights, a.srows, a.scols,
                      staged_smem_bytes(a), dev.smem_optin);
        return fail(XCORR_ERR_UNSUPPORTED, msg);
    }
    if ((unsigned long long)pm.n_left * a.groups_per_left * (2ull * W - 1) > 2147483647ull)
        return fail(XCORR_ERR_UNSUPPORTED, "too many (left, right group, x shift) blocks for one launch of the staged kernel");
    *out = a;
    return XCORR_OK;
}

std::string describe_plan(const TilePlan& p) {
    char buf[512];
    std::snprintf(buf, sizeof buf,
                  "kernel=tile<TY=%d> grid=(%u,1,1) block=(%d,1,1) smem=%zu plan{H=%d W=%d Hp=%d Wp=%d SL=%d ML=%d "
                  "WX=%d WY=%d CX=%d CY=%d RG=%d KG=%d KL=%d fused=%d S=%d schedule=%s tasks=%u nstage=%d combine=%s workspace=%zu}",
                  p.TY, p.grid, p.threads, p.smem_bytes, p.H, p.W, p.Hp, p.Wp, p.SL, p.ML, p.WX, p.WY,
                  p.CX, p.CY, p.RG, p.KG, p.KL, p.fused, p.S,
                  p.schedule == kSchedStatic ? "static" : p.schedule == kSchedStreamK ? "stream-k" : "warp-queue",
                  p.tasks, p.nstage,
                  p.combine == kStore ? "store" : p.combine == kAtomic ? "atomic" : p.combine == kFixup ? "fixup" : "workspace",
                  p.workspace_bytes);
    return buf;
}

const std::string& last_launch_text() {
    if (t_note.kind == LaunchNote::kTile) {
        t_last_launch = describe_plan(t_note.plan);
    } else if (t_note.kind == LaunchNote::kStaged) {
        const StagedArgs& sa = t_note.staged;
        char buf[320];
        std::snprintf(buf, sizeof buf, "kernel=warp_staged grid=(%u,%u,%u) block=(%d,1,1) smem=%zu shifts=%d slab=%dx%d rights=%d "
                      "column_groups=%d loads=%s", t_note.grid.x, t_note.grid.y, t_note.grid.z, sa.shifts * 32, t_note.smem,
                      sa.shifts, sa.srows, sa.scols, sa.rights, sa.col_groups, sa.warp_rows ? "warp-per-row" : "strided");
        t_last_launch = buf;
    } else if (t_note.kind == LaunchNote::kWarp) {
        char buf[200];
        std::snprintf(buf, sizeof buf, "kernel=warp_per_overlap grid=(%u,1,1) block=(%d,1,1) smem=0 split=%s rows_per_warp=%d",
                      t_note.grid.x, t_note.block, t_note.split == XCORR_SPLIT_NONE ? "none" :
                      t_note.split == XCORR_SPLIT_RECTANGLE ? "rectangle" : "triangle", t_note.rows_per_warp);
        t_last_launch = buf;
    }
    t_note.kind = LaunchNote::kText;
    return t_last_launch;
}

xcorr_status run_device(int32_t mode, const float* d_left, const float* d_right, float* d_out,
                        uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                        const xcorr_hints* hints, void* d_ws, size_t ws_bytes, void* stream_v) {
    if (!d_left || !d_right || !d_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
    PairMap pm{};
    xcorr_status st = check_sizes(mode, rows, cols, n_left, n_right, &pm);
    if (st != XCORR_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int H = (int)rows, W = (int)cols;
    const unsigned long long npairs = (unsigned long long)pm.n_left * pm.m;
    const unsigned long long total_out = npairs * (2ull * H - 1) * (2ull * W - 1);
    DeviceInfo dev;
    int device = 0;
    st = current_device_info(&dev, &device);
    if (st != XCORR_OK) return st;

    const bool tiny = tiny_auto(hints, pm, rows, cols);
    const int kernel = tiny ? (int)XCORR_KERNEL_WARP_PER_OVERLAP : pick_kernel(hints);
    // four-warp blocks once the tiny path has more than a wave of eight-warp ones' worth of overlaps
    const int bt = hints && hints->block_threads ? hints->block_threads : tiny && total_out > 2000 ? 128 : 256;
    if (bt < 32 || bt > 1024 || bt % 32 != 0)
        return fail(XCORR_ERR_INVALID_HINT, "block_threads must be a multiple of 32 in 32..1024");
    char buf[320];
    if (kernel == XCORR_KERNEL_OVERLAP_WISE) {
        dim3 g, b;
        XC_CUDA(launch_overlap_wise(d_left, d_right, d_out, H, W, pm, npairs, bt, &g, &b, stream));
        std::snprintf(buf, sizeof buf, "kernel=overlap_wise grid=(%u,%u,%u) block=(%u,%u,1) smem=0", g.x, g.y, g.z, b.x, b.y);
        set_launch_text(buf);
        ++t_launch_count;
        return XCORR_OK;
    }
    if (kernel == XCORR_KERNEL_WARP_PER_OVERLAP) {
        const int split = hints && !tiny ? hints->row_split : 0;
        const int rpw = hints && !tiny ? hints->rows_per_warp : 0;
        if (split < 0 || split > 2) return fail(XCORR_ERR_INVALID_HINT, "row_split must be 0 (none), 1 (rectangle) or 2 (triangle)");
        if (split != XCORR_SPLIT_NONE && rpw <= 0)
            return fail(XCORR_ERR_INVALID_HINT, "row_split needs rows_per_warp > 0");
        dim3 g, b;
        // parts of an overlap are added atomically: the output starts at zero (one_to_one.hpp:503)
        if (split != XCORR_SPLIT_NONE) XC_CUDA(cudaMemsetAsync(d_out, 0, total_out * sizeof(float), stream));
        XC_CUDA(launch_warp_per_overlap(d_left, d_right, d_out, H, W, pm, npairs, bt, rpw, split, dev.sm_count, &g, &b, stream));
        t_note.kind = LaunchNote::kWarp; t_note.grid = g; t_note.block = (int)b.x; t_note.split = split; t_note.rows_per_warp = rpw;
        ++t_launch_count;
        return XCORR_OK;
    }
    if (kernel == XCORR_KERNEL_WARP_STAGED) {
        StagedArgs sa{};
        if ((st = staged_args(pm, H, W, hints, dev, &sa)) != XCORR_OK) return st;
        sa.left = d_left; sa.right = d_right; sa.out = d_out;
        if (sa.col_groups) XC_CUDA(cudaMemsetAsync(d_out, 0, total_out * sizeof(float), stream));
        dim3 g;
        size_t smem = 0;
        XC_CUDA(launch_warp_staged(sa, device, &g, &smem, stream));
        t_note.kind = LaunchNote::kStaged; t_note.staged = sa; t_note.grid = g; t_note.smem = smem;
        ++t_launch_count;
        return XCORR_OK;
    }
    if (kernel == XCORR_KERNEL_FFT)
        return xcorr_fft_f32(mode, d_left, d_right, d_out, rows, cols, n_left, n_right, XCORR_FFT_NORMALIZED,
                             d_ws, ws_bytes, stream_v);
    if (kernel != XCORR_KERNEL_TILE) return fail(XCORR_ERR_INVALID_HINT, "unknown kernel family");

    TilePlan p{};
    st = plan_tile(pm, H, W, hints, dev, &p);
    if (st == XCORR_ERR_UNSUPPORTED && (!hints || hints->kernel == XCORR_KERNEL_AUTO)) {
        // no tile plan fits in shared memory (rows of many thousands of columns): the automatic
        // choice falls back to the overlap-wise kernel, which needs none -- slow, but every size
        // the reference accepts is computed
        dim3 g, b;
        XC_CUDA(launch_overlap_wise(d_left, d_right, d_out, H, W, pm, npairs, 256, &g, &b, stream));
        std::snprintf(buf, sizeof buf, "kernel=overlap_wise grid=(%u,%u,%u) block=(%u,%u,1) smem=0 (no tile plan fits)",
                      g.x, g.y, g.z, b.x, b.y);
        set_launch_text(buf);
        ++t_launch_count;
        return XCORR_OK;
    }
    if (st != XCORR_OK) return st;
    if (p.combine == kWorkspace || p.combine == kFixup) {
        const bool explicit_ws = hints && hints->combine == XCORR_COMBINE_WORKSPACE;
        if (!d_ws || ws_bytes < p.workspace_bytes) {
            if (explicit_ws)
                return fail(XCORR_ERR_WORKSPACE, "combine=workspace needs xcorr_workspace_bytes() bytes of workspace");
            // automatic plan without (enough) workspace: fall back to atomics
            if (hints && hints->reproducible == 1 && p.S > 2)
                return fail(XCORR_ERR_WORKSPACE, "the reproducible plan of this shape sums partial images: "
                            "it needs xcorr_workspace_bytes() bytes of workspace");
            p.combine = kAtomic;
            p.workspace_bytes = 0;
        } else if (reinterpret_cast<uintptr_t>(d_ws) % 16 != 0) {
            return fail(XCORR_ERR_WORKSPACE, "workspace must be 16-byte aligned");
        }
    }
    TileArgs a{};
    a.left = d_left; a.right = d_right; a.out = d_out;
    a.ws = (p.combine == kWorkspace || p.combine == kFixup) ? static_cast<float*>(d_ws) : nullptr;
    a.counters = nullptr;
    if (p.combine == kFixup) {
        a.counters = reinterpret_cast<unsigned*>(static_cast<char*>(d_ws) + fixup_counters_offset(p.pieces, total_out));
        XC_CUDA(cudaMemsetAsync(a.counters, 0, (size_t)p.tasks * sizeof(unsigned), stream));
    }
    a.p = p; a.pm = pm; a.total_out = total_out;
    a.vec_ok = (W % 4 == 0) && reinterpret_cast<uintptr_t>(d_left) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(d_right) % 16 == 0;
    a.stage_wait_limit = g_stage_wait_limit.load(std::memory_order_relaxed);
    a.stage_expect_surplus = g_stage_expect_surplus.load(std::memory_order_relaxed);
    t_note.kind = LaunchNote::kTile; t_note.plan = p;
    if (p.combine == kAtomic) XC_CUDA(cudaMemsetAsync(d_out, 0, total_out * sizeof(float), stream));
    XC_CUDA(launch_tile(a, device, stream));
    ++t_launch_count;
    if (p.combine == kWorkspace) {
        XC_CUDA(launch_reduce_partials(a.ws, d_out, total_out, H, W, p.Hp, p.S, dev.sm_count, stream));
        ++t_launch_count;
    }
    return XCORR_OK;
}

// ---- entry point that allocates nothing --------------------------------------------------
xcorr_status run_one_to_one_noalloc(const float* d_left, const float* d_right, float* d_out,
                                    uint32_t rows, uint32_t cols, void* stream_v) {
    if (!d_left || !d_right || !d_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
    PairMap pm{};
    xcorr_status st = check_sizes(XCORR_ONE_TO_ONE, rows, cols, 1, 1, &pm);
    if (st != XCORR_OK) return st;
    const int H = (int)rows, W = (int)cols;
    const unsigned long long total_out = (2ull * H - 1) * (2ull * W - 1);
    const size_t limit = noalloc_scratch_bytes();
    if (total_out * sizeof(float) > limit) {
        char msg[320];
        std::snprintf(msg, sizeof msg,
                      "a %u x %u pair has a result of %llu bytes; the entry point that allocates nothing takes results "
                      "of at most %zu bytes, the size of its built-in scratch array ((2*rows-1)*(2*cols-1) <= %zu "
                      "floats, e.g. square inputs up to 1448 x 1448)",
                      rows, cols, total_out * 4ull, limit, limit / sizeof(float));
        return fail(XCORR_ERR_UNSUPPORTED, msg);
    }
    DeviceInfo dev;
    int device = 0;
    if ((st = current_device_info(&dev, &device)) != XCORR_OK) return st;
    // the scratch array's device address, looked up once per device with that device current
    float* scratch = nullptr;
    XC_CUDA(noalloc_scratch_address(&scratch));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // First choice: the kernels and plan space of xcorr_one_to_one_f32 with combine = workspace, the
    // number of row slices capped by what the scratch array holds.  Large inputs need more, finer
    // slices than that (a slice must also fit one SM's shared memory): they take the plan that adds
    // the slices atomically onto the zeroed output, which needs no scratch at all.
    xcorr_hints hints{};
    hints.kernel = XCORR_KERNEL_TILE;
    hints.combine = XCORR_COMBINE_WORKSPACE;
    TilePlan p{};
    st = plan_tile(pm, H, W, &hints, dev, &p, limit);
    if (st == XCORR_ERR_UNSUPPORTED) {
        hints.combine = XCORR_COMBINE_AUTO;
        st = plan_tile(pm, H, W, &hints, dev, &p, limit);
        if (st == XCORR_OK && (p.combine == kWorkspace || p.combine == kFixup)) {
            // (the automatic plan only sums through a workspace that fits the cap; kept as a guard)
            if (p.workspace_bytes > limit) { p.combine = kAtomic; p.workspace_bytes = 0; }
        }
    }
    if (st == XCORR_ERR_UNSUPPORTED) {
        // rows too wide for any slice in shared memory: one thread per overlap, no scratch
        dim3 g, b;
        XC_CUDA(launch_overlap_wise(d_left, d_right, d_out, H, W, pm, 1, 256, &g, &b, stream));
        char buf[160];
        std::snprintf(buf, sizeof buf, "kernel=overlap_wise grid=(%u,%u,%u) block=(%u,%u,1) smem=0 (no tile plan fits)",
                      g.x, g.y, g.z, b.x, b.y);
        set_launch_text(buf);
        ++t_launch_count;
        return XCORR_OK;
    }
    if (st != XCORR_OK) return st;
    TileArgs a{};
    a.left = d_left; a.right = d_right; a.out = d_out;
    a.ws = p.combine == kWorkspace ? scratch : nullptr;
    a.p = p; a.pm = pm; a.total_out = total_out;
    a.vec_ok = (W % 4 == 0) && reinterpret_cast<uintptr_t>(d_left) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(d_right) % 16 == 0;
    a.stage_wait_limit = g_stage_wait_limit.load(std::memory_order_relaxed);
    a.stage_expect_surplus = g_stage_expect_surplus.load(std::memory_order_relaxed);
    t_note.kind = LaunchNote::kTile; t_note.plan = p;
    if (p.combine == kAtomic) XC_CUDA(cudaMemsetAsync(d_out, 0, total_out * sizeof(float), stream));
    XC_CUDA(launch_tile(a, device, stream));
    ++t_launch_count;
    if (p.combine == kWorkspace) {
        XC_CUDA(launch_reduce_partials(scratch, d_out, total_out, H, W, p.Hp, p.S, dev.sm_count, stream));
        ++t_launch_count;
    }
    return XCORR_OK;
}

// ---- host-buffer front end -------------------------------------------------------------
// Copy in, run, copy out -- in pieces: the independent result matrices are cut into up to
// kMaxHostChunks blocks; the input copy of a block, its kernel and its result copy run on
// three streams chained by events, so that the result copy (the longest of the three for
// this path: the result is 2-4 times the size of the input) hides the other two.
constexpr int kMaxHostChunks = 8;

struct HostCache {
    std::mutex mutex;
    float* d_left = nullptr;  size_t left_bytes = 0;
    float* d_right = nullptr; size_t right_bytes = 0;
    float* d_out = nullptr;   size_t out_bytes = 0;
    void* d_ws = nullptr;     size_t ws_bytes = 0;
    cudaStream_t stream = nullptr;       // kernels
    cudaStream_t copy_in = nullptr;      // host -> device
    cudaStream_t copy_out = nullptr;     // device -> host
    std::vector<cudaEvent_t> in_done;    // one pair of events per piece in flight
    std::vector<cudaEvent_t> run_done;
};
HostCache g_host_cache[kMaxDevices];

template<typename T>
xcorr_status grow(T** ptr, size_t* have, size_t need) {
    if (need <= *have) return XCORR_OK;
    if (*ptr) XC_CUDA(cudaFree(*ptr));
    *ptr = nullptr; *have = 0;
    XC_CUDA(cudaMalloc(reinterpret_cast<void**>(ptr), need));
    *have = need;
    return XCORR_OK;
}

// Number of pieces for a host-buffer call: one for one pair; otherwise one per 10 MiB of
// result, each piece keeping at least 128 pairs so that its kernel still fills the GPU
// (measured on B200 with the benchmark shapes: 3 pieces for 33 MB of result, 7-8 for 74 MB).
int host_chunk_count(int32_t mode, const PairMap& pm, uint32_t units, size_t obytes, const xcorr_hints* hints) {
    if (mode == XCORR_ONE_TO_ONE || units <= 1) return 1;
    long long k;
    if (hints && hints->host_chunks > 0) {
        k = hints->host_chunks;
    } else {
        const unsigned long long pairs = (unsigned long long)pm.n_left * pm.m;
        k = (long long)(obytes / (10ull << 20));
        k = std::min<long long>(k, (long long)(pairs / 128));
    }
    k = std::min<long long>(k, kMaxHostChunks);
    k = std::min<long long>(k, units);
    return (int)std::max<long long>(k, 1);
}

// One problem of a host-buffer call, with what the batch runner derives for it.
struct HostJob {
    int32_t mode;
    const float* h_left; const float* h_right; float* h_out;
    uint32_t rows, cols, n_left, n_right;
    const xcorr_hints* hints;
    PairMap pm;
    size_t lbytes, rbytes, obytes;      // operand and result sizes
    size_t loff, roff, ooff;            // where they sit in the device arenas (bytes)
    uint32_t units;
    int chunks;
};

size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

// Several problems in one call: all of them share the three streams, so the input copy and
// the kernels of a problem run under the result copy of the one before it -- the device ->
// host link, the slowest stage of this path, never idles between problems.  Every problem
// keeps its own device buffers (one arena per operand) until the call returns.
xcorr_status run_host_batch(HostJob* jobs, int n_jobs, int32_t device) {
    if (n_jobs <= 0) return XCORR_OK;
    size_t lsum = 0, rsum = 0, osum = 0, wsb = 0;
    int pieces = 0;
    xcorr_status st;
    for (int j = 0; j < n_jobs; ++j) {
        HostJob& J = jobs[j];
        if (!J.h_left || !J.h_right || !J.h_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
        if (J.hints && J.hints->host_chunks < 0) return fail(XCORR_ERR_INVALID_HINT, "host_chunks must be 0 (auto) or positive");
        J.pm = PairMap{};
        if ((st = check_sizes(J.mode, J.rows, J.cols, J.n_left, J.n_right, &J.pm)) != XCORR_OK) return st;
        const size_t in_elems = (size_t)J.rows * J.cols;
        const size_t out_elems = (size_t)(2 * J.rows - 1) * (2 * J.cols - 1);
        J.lbytes = in_elems * J.n_left * sizeof(float);
        J.rbytes = in_elems * J.n_right * sizeof(float);
        J.obytes = out_elems * (size_t)J.pm.n_left * J.pm.m * sizeof(float);
        J.loff = lsum; lsum += align256(J.lbytes);
        J.roff = rsum; rsum += align256(J.rbytes);
        J.ooff = osum; osum += align256(J.obytes);
        // the units a piece is made of: right matrices (one_to_many) or left matrices with all
        // (n_to_m) / their own (n_to_mn) right matrices
        J.units = J.mode == XCORR_ONE_TO_MANY ? J.n_right : J.mode == XCORR_ONE_TO_ONE ? 1u : J.n_left;
        J.chunks = host_chunk_count(J.mode, J.pm, J.units, J.obytes, J.hints);
        pieces += J.chunks;
        // workspace: the largest need among all pieces (their kernels run one after the other)
        for (int i = 0; i < J.chunks; ++i) {
            uint32_t first = 0, count = 0;
            xcorr_shard_range(J.units, J.chunks, i, &first, &count);
            if (count == 0) continue;
            const uint32_t nl = J.mode == XCORR_ONE_TO_MANY || J.mode == XCORR_ONE_TO_ONE ? J.n_left : count;
            const uint32_t nr = J.mode == XCORR_ONE_TO_MANY ? count : J.mode == XCORR_N_TO_MN ? count * J.pm.m : J.n_right;
            wsb = std::max(wsb, xcorr_workspace_bytes(J.mode, J.rows, J.cols, nl, nr, J.hints));
        }
    }
    int ndev = 0;
    XC_CUDA(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev || device >= kMaxDevices) return fail(XCORR_ERR_DEVICE, "no such CUDA device");
    DeviceGuard restore_device;                 // the caller's current device comes back on every return path
    XC_CUDA(cudaSetDevice(device));
    HostCache& c = g_host_cache[device];
    std::lock_guard<std::mutex> lock(c.mutex);
    if (!c.stream) XC_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    if (!c.copy_in) XC_CUDA(cudaStreamCreateWithFlags(&c.copy_in, cudaStreamNonBlocking));
    if (!c.copy_out) XC_CUDA(cudaStreamCreateWithFlags(&c.copy_out, cudaStreamNonBlocking));
    while ((int)c.in_done.size() < pieces) {
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        XC_CUDA(cudaEventCreateWithFlags(&e0, cudaEventDisableTiming));
        c.in_done.push_back(e0);
        XC_CUDA(cudaEventCreateWithFlags(&e1, cudaEventDisableTiming));
        c.run_done.push_back(e1);
    }
    if ((st = grow(&c.d_left, &c.left_bytes, lsum)) != XCORR_OK) return st;
    if ((st = grow(&c.d_right, &c.right_bytes, rsum)) != XCORR_OK) return st;
    if ((st = grow(&c.d_out, &c.out_bytes, osum)) != XCORR_OK) return st;
    if ((st = grow(&c.d_ws, &c.ws_bytes, wsb)) != XCORR_OK) return st;

    std::string plans;
    int piece = 0;
    // Everything below queues work on the three cached streams.  Whatever fails, what was queued
    // has to finish before the call returns: the next call may grow (free) the arenas.
    auto enqueue_all = [&]() -> xcorr_status {
    for (int j = 0; j < n_jobs; ++j) {
        const HostJob& J = jobs[j];
        const int32_t mode = J.mode;
        const PairMap& pm = J.pm;
        const size_t in_elems = (size_t)J.rows * J.cols;
        const size_t out_elems = (size_t)(2 * J.rows - 1) * (2 * J.cols - 1);
        float* const job_left = c.d_left + J.loff / sizeof(float);
        float* const job_right = c.d_right + J.roff / sizeof(float);
        float* const job_out = c.d_out + J.ooff / sizeof(float);
        // the operand every piece needs goes first
        if (mode == XCORR_ONE_TO_MANY || mode == XCORR_ONE_TO_ONE)
            XC_CUDA(cudaMemcpyAsync(job_left, J.h_left, J.lbytes, cudaMemcpyHostToDevice, c.copy_in));
        else if (mode == XCORR_N_TO_M)
            XC_CUDA(cudaMemcpyAsync(job_right, J.h_right, J.rbytes, cudaMemcpyHostToDevice, c.copy_in));
        for (int i = 0; i < J.chunks; ++i, ++piece) {
            uint32_t first = 0, count = 0;
            xcorr_shard_range(J.units, J.chunks, i, &first, &count);
            if (count == 0) continue;
            const float* dl = job_left;
            const float* dr = job_right;
            float* dout = job_out;
            float* hout = J.h_out;
            uint32_t nl = J.n_left, nr = J.n_right;
            size_t piece_out = J.obytes;
            if (mode == XCORR_ONE_TO_ONE) {
                XC_CUDA(cudaMemcpyAsync(job_right, J.h_right, J.rbytes, cudaMemcpyHostToDevice, c.copy_in));
            } else if (mode == XCORR_ONE_TO_MANY) {
                const size_t off = (size_t)first * in_elems;
                XC_CUDA(cudaMemcpyAsync(job_right + off, J.h_right + off, (size_t)count * in_elems * sizeof(float),
                                        cudaMemcpyHostToDevice, c.copy_in));
                dr += off; nr = count;
                dout += (size_t)first * out_elems; hout += (size_t)first * out_elems;
                piece_out = (size_t)count * out_elems * sizeof(float);
            } else {
                const size_t loff = (size_t)first * in_elems;
                XC_CUDA(cudaMemcpyAsync(job_left + loff, J.h_left + loff, (size_t)count * in_elems * sizeof(float),
                                        cudaMemcpyHostToDevice, c.copy_in));
                dl += loff; nl = count;
                if (mode == XCORR_N_TO_MN) {
                    const size_t roff = (size_t)first * pm.m * in_elems;
                    XC_CUDA(cudaMemcpyAsync(job_right + roff, J.h_right + roff,
                                            (size_t)count * pm.m * in_elems * sizeof(float),
                                            cudaMemcpyHostToDevice, c.copy_in));
                    dr += roff; nr = count * pm.m;
                }
                dout += (size_t)first * pm.m * out_elems; hout += (size_t)first * pm.m * out_elems;
                piece_out = (size_t)count * pm.m * out_elems * sizeof(float);
            }
            XC_CUDA(cudaEventRecord(c.in_done[piece], c.copy_in));
            XC_CUDA(cudaStreamWaitEvent(c.stream, c.in_done[piece], 0));
            const xcorr_status rst = run_device(mode, dl, dr, dout, J.rows, J.cols, nl, nr, J.hints, c.d_ws, c.ws_bytes, c.stream);
            if (rst != XCORR_OK) return rst;
            if (i == 0) {
                if (!plans.empty()) plans += "; ";
                plans += (J.chunks > 1 ? "host_chunks=" + std::to_string(J.chunks) + " first{" + last_launch_text() + "}" : last_launch_text());
            }
            XC_CUDA(cudaEventRecord(c.run_done[piece], c.stream));
            XC_CUDA(cudaStreamWaitEvent(c.copy_out, c.run_done[piece], 0));
            XC_CUDA(cudaMemcpyAsync(hout, dout, piece_out, cudaMemcpyDeviceToHost, c.copy_out));
        }
    }
    return XCORR_OK;
    };
    st = enqueue_all();
    if (st != XCORR_OK) {
        const std::string why = t_last_error;
        (void)cudaStreamSynchronize(c.copy_in); (void)cudaStreamSynchronize(c.stream); (void)cudaStreamSynchronize(c.copy_out);
        (void)cudaGetLastError();
        t_last_error = why;
        return st;
    }
    XC_CUDA(cudaStreamSynchronize(c.copy_out));
    set_launch_text(n_jobs > 1 ? "host_batch=" + std::to_string(n_jobs) + " [" + plans + "]" : plans);
    return XCORR_OK;
}

xcorr_status run_host(int32_t mode, const float* h_left, const float* h_right, float* h_out,
                      uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                      const xcorr_hints* hints, int32_t device) {
    HostJob job{};
    job.mode = mode; job.h_left = h_left; job.h_right = h_right; job.h_out = h_out;
    job.rows = rows; job.cols = cols; job.n_left = n_left; job.n_right = n_right; job.hints = hints;
    return run_host_batch(&job, 1, device);
}

}  // namespace

// ============================================================================================
extern "C" {

xcorr_status xcorr_run_f32(int32_t mode, const float* d_left, const float* d_right, float* d_out,
                           uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                           const xcorr_hints* hints, void* d_workspace, size_t workspace_bytes, void* stream) {
    return guarded([&]() -> xcorr_status {
        return run_device(mode, d_left, d_right, d_out, rows, cols, n_left, n_right, hints,
                          d_workspace, workspace_bytes, stream);
    });
}

xcorr_status xcorr_one_to_one_f32(const float* d_left, const float* d_right, float* d_out,
                                  uint32_t rows, uint32_t cols, const xcorr_hints* hints,
                                  void* d_workspace, size_t workspace_bytes, void* stream) {
    return guarded([&]() -> xcorr_status {
        return run_device(XCORR_ONE_TO_ONE, d_left, d_right, d_out, rows, cols, 1, 1, hints,
                          d_workspace, workspace_bytes, stream);
    });
}

xcorr_status xcorr_one_to_one_noalloc_f32(const float* d_left, const float* d_right, float* d_out,
                                          uint32_t rows, uint32_t cols, void* stream) {
    return guarded([&]() -> xcorr_status {
        return run_one_to_one_noalloc(d_left, d_right, d_out, rows, cols, stream);
    });
}

size_t xcorr_noalloc_scratch_bytes(void) { return noalloc_scratch_bytes(); }

xcorr_status xcorr_one_to_many_f32(const float* d_left, const float* d_right, float* d_out,
                                   uint32_t rows, uint32_t cols, uint32_t n_right, const xcorr_hints* hints,
                                   void* d_workspace, size_t workspace_bytes, void* stream) {
    return guarded([&]() -> xcorr_status {
        return run_device(XCORR_ONE_TO_MANY, d_left, d_right, d_out, rows, cols, 1, n_right, hints,
                          d_workspace, workspace_bytes, stream);
    });
}

xcorr_status xcorr_n_to_mn_f32(const float* d_left, const float* d_right, float* d_out,
                               uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                               const xcorr_hints* hints, void* d_workspace, size_t workspace_bytes, void* stream) {
    return guarded([&]() -> xcorr_status {
        return run_device(XCORR_N_TO_MN, d_left, d_right, d_out, rows, cols, n_left, n_right, hints,
                          d_workspace, workspace_bytes, stream);
    });
}

xcorr_status xcorr_n_to_m_f32(const float* d_left, const float* d_right, float* d_out,
                              uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                              const xcorr_hints* hints, void* d_workspace, size_t workspace_bytes, void* stream) {
    return guarded([&]() -> xcorr_status {
        return run_device(XCORR_N_TO_M, d_left, d_right, d_out, rows, cols, n_left, n_right, hints,
                          d_workspace, workspace_bytes, stream);
    });
}

size_t xcorr_fft_workspace_bytes(int32_t mode, uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                 int32_t layout) {
    PairMap pm{};
    if (check_sizes(mode, rows, cols, n_left, n_right, &pm) != XCORR_OK) return 0;
    if (layout != XCORR_FFT_NORMALIZED && layout != XCORR_FFT_RAW) return 0;
    return fft_workspace_layout(pm, (int)rows, (int)cols, n_right, layout == XCORR_FFT_RAW).total;
}

xcorr_status xcorr_fft_f32(int32_t mode, const float* d_left, const float* d_right, float* d_out,
                           uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                           int32_t layout, void* d_workspace, size_t workspace_bytes, void* stream) {
    return guarded([&]() -> xcorr_status {
        if (!d_left || !d_right || !d_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
        PairMap pm{};
        xcorr_status st = check_sizes(mode, rows, cols, n_left, n_right, &pm);
        if (st != XCORR_OK) return st;
        if (layout != XCORR_FFT_NORMALIZED && layout != XCORR_FFT_RAW)
            return fail(XCORR_ERR_INVALID_HINT, "layout must be XCORR_FFT_NORMALIZED or XCORR_FFT_RAW");
        const FftLayout lay = fft_workspace_layout(pm, (int)rows, (int)cols, n_right, layout == XCORR_FFT_RAW);
        if (!d_workspace || workspace_bytes < lay.total)
            return fail(XCORR_ERR_WORKSPACE, "the FFT path needs xcorr_fft_workspace_bytes() bytes of workspace");
        if (reinterpret_cast<uintptr_t>(d_workspace) % 256 != 0)
            return fail(XCORR_ERR_WORKSPACE, "the FFT workspace must be 256-byte aligned");
        DeviceInfo dev;
        int device = 0;
        if ((st = current_device_info(&dev, &device)) != XCORR_OK) return st;
        std::string err;
        int launches = 0;
        const int rc = fft_run(d_left, d_right, d_out, (int)rows, (int)cols, pm, n_right, layout == XCORR_FFT_RAW,
                               d_workspace, device, dev.sm_count, static_cast<cudaStream_t>(stream), &err, &launches);
        t_launch_count += (uint64_t)launches;
        if (rc != 0) return fail(XCORR_ERR_CUDA, err);
        char buf[256];
        std::snprintf(buf, sizeof buf, "kernel=fft transform=%ux%u inputs=%llu pairs=%llu product=%s layout=%s workspace=%zu",
                      2 * rows, 2 * cols, (unsigned long long)pm.n_left + n_right, (unsigned long long)pm.n_left * pm.m,
                      lay.product_in_place ? "in-place" : "separate", layout == XCORR_FFT_RAW ? "raw" : "normalized",
                      lay.total);
        set_launch_text(buf);
        return XCORR_OK;
    });
}

void xcorr_fft_release_plans(void) { fft_release_plans(); }

xcorr_status xcorr_check_device(void) {
    return guarded([&]() -> xcorr_status {
        XC_CUDA(cudaDeviceSynchronize());
        XC_CUDA(cudaGetLastError());
        unsigned timeouts = 0;
        XC_CUDA(tile_stage_timeouts(&timeouts));
        if (timeouts != 0)
            return fail(XCORR_ERR_TIMEOUT, std::to_string(timeouts) + " block(s) of tile_kernel gave up a bounded staging wait "
                        "and dropped their work; results of the launches since the last check are incomplete");
        return XCORR_OK;
    });
}

size_t xcorr_workspace_bytes(int32_t mode, uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                             const xcorr_hints* hints) {
    try {
    PairMap pm{};
    if (check_sizes(mode, rows, cols, n_left, n_right, &pm) != XCORR_OK) return 0;
    if (pick_kernel(hints) == XCORR_KERNEL_FFT)
        return fft_workspace_layout(pm, (int)rows, (int)cols, n_right, 0).total;
    if (pick_kernel(hints) != XCORR_KERNEL_TILE || tiny_auto(hints, pm, rows, cols)) return 0;
    DeviceInfo dev;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0 || current_device_info(&dev) != XCORR_OK) {
        (void)cudaGetLastError();
        dev = assumed_device();
    }
    TilePlan p{};
    if (plan_tile(pm, (int)rows, (int)cols, hints, dev, &p) != XCORR_OK) return 0;
    return p.workspace_bytes;
    } catch (...) {
        return 0;
    }
}

int32_t xcorr_describe_plan(int32_t mode, uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                            const xcorr_hints* hints, char* buffer, size_t buffer_bytes) {
    return guarded([&]() -> xcorr_status {
    if (!buffer || buffer_bytes == 0) return fail(XCORR_ERR_NULL_POINTER, "buffer must not be NULL");
    PairMap pm{};
    xcorr_status st = check_sizes(mode, rows, cols, n_left, n_right, &pm);
    if (st != XCORR_OK) return st;
    std::string text;
    const bool tiny = tiny_auto(hints, pm, rows, cols);
    const int kernel = tiny ? (int)XCORR_KERNEL_WARP_PER_OVERLAP : pick_kernel(hints);
    if (kernel == XCORR_KERNEL_OVERLAP_WISE) text = "kernel=overlap_wise";
    else if (kernel == XCORR_KERNEL_WARP_PER_OVERLAP) text = "kernel=warp_per_overlap";
    else if (kernel == XCORR_KERNEL_WARP_STAGED) text = "kernel=warp_staged";
    else if (kernel == XCORR_KERNEL_FFT) text = "kernel=fft";
    else if (kernel == XCORR_KERNEL_TILE) {
        DeviceInfo dev;
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0 || current_device_info(&dev) != XCORR_OK) {
            (void)cudaGetLastError();
            dev = assumed_device();
        }
        TilePlan p{};
        st = plan_tile(pm, (int)rows, (int)cols, hints, dev, &p);
        if (st == XCORR_ERR_UNSUPPORTED && (!hints || hints->kernel == XCORR_KERNEL_AUTO)) {
            text = "kernel=overlap_wise (no tile plan fits)";
            st = XCORR_OK;
        } else {
            if (st != XCORR_OK) return st;
            text = describe_plan(p);
        }
    } else {
        return fail(XCORR_ERR_INVALID_HINT, "unknown kernel family");
    }
    std::snprintf(buffer, buffer_bytes, "%s", text.c_str());
    return XCORR_OK;
    });
}

uint64_t xcorr_num_results(int32_t mode, uint32_t n_left, uint32_t n_right) {
    PairMap pm{};
    if (!pair_map(mode, n_left, n_right, &pm)) return 0;
    return (uint64_t)pm.n_left * pm.m;
}

int32_t xcorr_validate_input_size(int32_t mode, uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right) {
    PairMap pm{};
    return rows > 0 && cols > 0 && pair_map(mode, n_left, n_right, &pm) ? 1 : 0;
}

xcorr_status xcorr_run_host_f32(int32_t mode, const float* h_left, const float* h_right, float* h_out,
                                uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                const xcorr_hints* hints, int32_t device) {
    return guarded([&]() -> xcorr_status {
        return run_host(mode, h_left, h_right, h_out, rows, cols, n_left, n_right, hints, device);
    });
}

xcorr_status xcorr_run_f64(int32_t mode, const double* d_left, const double* d_right, double* d_out,
                           uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right, void* stream) {
    return guarded([&]() -> xcorr_status {
        if (!d_left || !d_right || !d_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
        PairMap pm{};
        xcorr_status st = check_sizes(mode, rows, cols, n_left, n_right, &pm);
        if (st != XCORR_OK) return st;
        DeviceInfo dev;
        int device = 0;
        if ((st = current_device_info(&dev, &device)) != XCORR_OK) return st;
        // The register-tiled kernel wherever a plan fits; XCORR_F64_STRIP=1 keeps the column-strip
        // kernel (a cross-check with another summation order).
        const char* strip_env = std::getenv("XCORR_F64_STRIP");        // read per call: tests switch it
        const bool force_strip = strip_env && strip_env[0] == '1';
        TilePlan64 tp{};
        const char* rep_env = std::getenv("XCORR_REPRODUCIBLE");
        const bool reproducible = rep_env && rep_env[0] == '1';
        // a handful of small overlaps: the warp-per-overlap latency kernel, as in single precision
        const double overlaps = (double)pm.n_left * pm.m * (2.0 * rows - 1) * (2.0 * cols - 1);
        if (!force_strip && !std::getenv("XCORR_F64_PLAN") && rows <= 32 && cols <= 32 && overlaps <= kTinyOverlaps) {
            dim3 g;
            const int bt = overlaps > 2000.0 ? 128 : 256;
            XC_CUDA(launch_warp_per_overlap_f64(d_left, d_right, d_out, (int)rows, (int)cols, pm,
                                                (unsigned long long)pm.n_left * pm.m, bt, &g,
                                                static_cast<cudaStream_t>(stream)));
            char wbuf[128];
            std::snprintf(wbuf, sizeof wbuf, "kernel=warp_per_overlap_f64 grid=(%u,1,1) block=(%d,1,1) smem=0", g.x, bt);
            set_launch_text(wbuf);
            ++t_launch_count;
            return XCORR_OK;
        }
        if (!force_strip && plan_tile_f64(pm, (int)rows, (int)cols, dev.sm_count, dev.smem_optin, reproducible, &tp)) {
            TileArgs64 ta{};
            ta.left = d_left; ta.right = d_right; ta.out = d_out; ta.p = tp; ta.pm = pm;
            ta.vec_ok = cols % 2 == 0 && reinterpret_cast<uintptr_t>(d_left) % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(d_right) % 16 == 0;
            cudaStream_t s64 = static_cast<cudaStream_t>(stream);
            if (tp.S > 1) {
                const size_t out_bytes = (size_t)pm.n_left * pm.m * (2 * (size_t)rows - 1) * (2 * (size_t)cols - 1) * sizeof(double);
                XC_CUDA(cudaMemsetAsync(d_out, 0, out_bytes, s64));
            }
            XC_CUDA(launch_tile_f64(ta, device, s64));
            char tbuf[256];
            std::snprintf(tbuf, sizeof tbuf, "kernel=tile_f64 grid=(%u,1,1) block=(%d,1,1) smem=%zu plan{Hp=%d Wp=%d SL=%d ML=%d "
                          "WX=%d WY=%d CX=%d CY=%d RG=%d S=%d nstage=%d combine=%s}", tp.grid, tp.threads, tp.smem_bytes, tp.Hp,
                          tp.Wp, tp.SL, tp.ML, tp.WX, tp.WY, tp.CX, tp.CY, tp.RG, tp.S, tp.nstage, tp.S > 1 ? "atomic" : "store");
            set_launch_text(tbuf);
            ++t_launch_count;
            return XCORR_OK;
        }
        dim3 g, b;
        XC_CUDA(launch_strip_f64(d_left, d_right, d_out, (int)rows, (int)cols, pm,
                                 (unsigned long long)pm.n_left * pm.m, dev.sm_count, &g, &b,
                                 static_cast<cudaStream_t>(stream)));
        char buf[128];
        std::snprintf(buf, sizeof buf, "kernel=strip_f64 grid=(%u,1,1) block=(%u,1,1) smem=0", g.x, b.x);
        set_launch_text(buf);
        ++t_launch_count;
        return XCORR_OK;
    });
}

xcorr_status xcorr_run_host_f64(int32_t mode, const double* h_left, const double* h_right, double* h_out,
                                uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right, int32_t device) {
    return guarded([&]() -> xcorr_status {
        if (!h_left || !h_right || !h_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
        PairMap pm{};
        xcorr_status st = check_sizes(mode, rows, cols, n_left, n_right, &pm);
        if (st != XCORR_OK) return st;
        int ndev = 0;
        XC_CUDA(cudaGetDeviceCount(&ndev));
        if (device < 0 || device >= ndev) return fail(XCORR_ERR_DEVICE, "no such CUDA device");
        DeviceGuard restore_device;
        XC_CUDA(cudaSetDevice(device));
        const size_t in_elems = (size_t)rows * cols;
        const size_t lbytes = in_elems * n_left * sizeof(double), rbytes = in_elems * n_right * sizeof(double);
        const size_t obytes = (size_t)(2 * rows - 1) * (2 * cols - 1) * pm.n_left * pm.m * sizeof(double);
        double *dl = nullptr, *dr = nullptr, *dout = nullptr;
        cudaStream_t stream = nullptr;
        cudaError_t e = cudaMalloc(&dl, lbytes);
        if (e == cudaSuccess) e = cudaMalloc(&dr, rbytes);
        if (e == cudaSuccess) e = cudaMalloc(&dout, obytes);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dl, h_left, lbytes, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dr, h_right, rbytes, cudaMemcpyHostToDevice, stream);
        st = XCORR_OK;
        if (e == cudaSuccess) st = xcorr_run_f64(mode, dl, dr, dout, rows, cols, n_left, n_right, stream);
        if (e == cudaSuccess && st == XCORR_OK) e = cudaMemcpyAsync(h_out, dout, obytes, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess && stream) e = cudaStreamSynchronize(stream);
        if (stream) cudaStreamDestroy(stream);
        cudaFree(dl); cudaFree(dr); cudaFree(dout);
        if (st != XCORR_OK) return st;
        if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(XCORR_ERR_CUDA, cudaGetErrorString(e)); }
        return XCORR_OK;
    });
}

xcorr_status xcorr_run_host_batch_f32(const xcorr_host_job* jobs, int32_t n_jobs, int32_t device) {
    return guarded([&]() -> xcorr_status {
        if (n_jobs < 0) return fail(XCORR_ERR_INVALID_SIZE, "n_jobs must not be negative");
        if (n_jobs == 0) return XCORR_OK;
        if (!jobs) return fail(XCORR_ERR_NULL_POINTER, "jobs must not be NULL");
        std::vector<HostJob> hj((size_t)n_jobs);
        for (int j = 0; j < n_jobs; ++j) {
            hj[j].mode = jobs[j].mode;
            hj[j].h_left = jobs[j].h_left; hj[j].h_right = jobs[j].h_right; hj[j].h_out = jobs[j].h_out;
            hj[j].rows = jobs[j].rows; hj[j].cols = jobs[j].cols;
            hj[j].n_left = jobs[j].n_left; hj[j].n_right = jobs[j].n_right;
            hj[j].hints = jobs[j].hints;
        }
        return run_host_batch(hj.data(), n_jobs, device);
    });
}

void xcorr_shard_range(uint32_t units, int32_t parts, int32_t index, uint32_t* first, uint32_t* count) {
    if (parts <= 0 || index < 0 || index >= parts) {
        if (first) *first = 0;
        if (count) *count = 0;
        return;
    }
    const uint64_t lo = (uint64_t)units * (uint64_t)index / (uint64_t)parts;
    const uint64_t hi = (uint64_t)units * (uint64_t)(index + 1) / (uint64_t)parts;
    if (first) *first = (uint32_t)lo;
    if (count) *count = (uint32_t)(hi - lo);
}

xcorr_status xcorr_run_host_sharded_f32(int32_t mode, const float* h_left, const float* h_right, float* h_out,
                                        uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                                        const xcorr_hints* hints, const int32_t* devices, int32_t n_devices) {
    return guarded([&]() -> xcorr_status {
        if (!h_left || !h_right || !h_out) return fail(XCORR_ERR_NULL_POINTER, "left, right and out must not be NULL");
        PairMap pm{};
        xcorr_status st = check_sizes(mode, rows, cols, n_left, n_right, &pm);
        if (st != XCORR_OK) return st;
        if (n_devices <= 0 || n_devices > kMaxDevices) return fail(XCORR_ERR_DEVICE, "n_devices must be 1..64");
        std::vector<int32_t> devs(n_devices);
        for (int i = 0; i < n_devices; ++i) devs[i] = devices ? devices[i] : i;
        if (mode == XCORR_ONE_TO_ONE || n_devices == 1)
            return run_host(mode, h_left, h_right, h_out, rows, cols, n_left, n_right, hints, devs[0]);
    
        const size_t in_elems = (size_t)rows * cols;
        const size_t out_elems = (size_t)(2 * rows - 1) * (2 * cols - 1);
        const uint32_t units = mode == XCORR_ONE_TO_MANY ? n_right : n_left;
        std::vector<xcorr_status> status(n_devices, XCORR_OK);
        std::vector<std::string> errors(n_devices);
        std::vector<std::thread> workers;
        for (int i = 0; i < n_devices; ++i) {
            uint32_t first = 0, count = 0;
            xcorr_shard_range(units, n_devices, i, &first, &count);
            if (count == 0) continue;
            workers.emplace_back([&, i, first, count]() {
                const float* l = h_left;
                const float* r = h_right;
                float* o = h_out;
                uint32_t nl = n_left, nr = n_right;
                if (mode == XCORR_ONE_TO_MANY) {           // a block of right matrices
                    r += (size_t)first * in_elems;
                    o += (size_t)first * out_elems;
                    nr = count;
                } else if (mode == XCORR_N_TO_M) {          // a block of left matrices, all rights
                    l += (size_t)first * in_elems;
                    o += (size_t)first * pm.m * out_elems;
                    nl = count;
                } else {                                    // n_to_mn: lefts with their own m rights
                    l += (size_t)first * in_elems;
                    r += (size_t)first * pm.m * in_elems;
                    o += (size_t)first * pm.m * out_elems;
                    nl = count;
                    nr = count * pm.m;
                }
                status[i] = run_host(mode, l, r, o, rows, cols, nl, nr, hints, devs[i]);
                if (status[i] != XCORR_OK) errors[i] = t_last_error;
            });
        }
        for (auto& w : workers) w.join();
        for (int i = 0; i < n_devices; ++i)
            if (status[i] != XCORR_OK) return fail(status[i], "shard " + std::to_string(i) + ": " + errors[i]);
        return XCORR_OK;
    });
}

void xcorr_release_host_cache(void) {
    noalloc_forget_addresses();
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); return; }
    for (int d = 0; d < kMaxDevices; ++d) {
        HostCache& c = g_host_cache[d];
        std::lock_guard<std::mutex> lock(c.mutex);
        if (!c.d_left && !c.d_right && !c.d_out && !c.d_ws && !c.stream) continue;
        if (cudaSetDevice(d) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (c.d_left) cudaFree(c.d_left);
        if (c.d_right) cudaFree(c.d_right);
        if (c.d_out) cudaFree(c.d_out);
        if (c.d_ws) cudaFree(c.d_ws);
        if (c.stream) cudaStreamDestroy(c.stream);
        if (c.copy_in) cudaStreamDestroy(c.copy_in);
        if (c.copy_out) cudaStreamDestroy(c.copy_out);
        for (cudaEvent_t e : c.in_done) cudaEventDestroy(e);
        for (cudaEvent_t e : c.run_done) cudaEventDestroy(e);
        c.in_done.clear();
        c.run_done.clear();
        c.copy_in = c.copy_out = nullptr;
        c.d_left = c.d_right = c.d_out = nullptr;
        c.d_ws = nullptr;
        c.left_bytes = c.right_bytes = c.out_bytes = c.ws_bytes = 0;
        c.stream = nullptr;
    }
    cudaSetDevice(prev);
}

xcorr_status xcorr_n_to_mn_reorder_f32(const float* src, float* dst, uint32_t n_left, uint32_t n_total,
                                       size_t elems, int32_t to_grouped) {
    return guarded([&]() -> xcorr_status {
        if (!src || !dst) return fail(XCORR_ERR_NULL_POINTER, "src and dst must not be NULL");
        if (n_left == 0 || n_total % n_left != 0) return fail(XCORR_ERR_INVALID_SIZE, "n_total must be a multiple of n_left");
        const uint32_t m = n_total / n_left;
        for (uint32_t i = 0; i < n_total; ++i) {
            // file index i = t*n_left + l  <->  grouped index l*m + t
            const uint32_t l = i % n_left, t = i / n_left;
            const uint32_t g = l * m + t;
            if (to_grouped) std::memcpy(dst + (size_t)g * elems, src + (size_t)i * elems, elems * sizeof(float));
            else            std::memcpy(dst + (size_t)i * elems, src + (size_t)g * elems, elems * sizeof(float));
        }
        return XCORR_OK;
    });
}

const char* xcorr_last_launch_string(void) {
    try { return last_launch_text().c_str(); } catch (...) { return "out of host memory"; }
}
const char* xcorr_last_error_string(void) { return t_last_error.c_str(); }

const char* xcorr_status_string(int32_t status) {
    switch (status) {
    case XCORR_OK: return "ok";
    case XCORR_ERR_NULL_POINTER: return "null pointer";
    case XCORR_ERR_INVALID_SIZE: return "invalid size";
    case XCORR_ERR_INVALID_HINT: return "invalid hint";
    case XCORR_ERR_WORKSPACE: return "workspace missing or too small";
    case XCORR_ERR_CUDA: return "CUDA error";
    case XCORR_ERR_UNSUPPORTED: return "unsupported shape";
    case XCORR_ERR_DEVICE: return "bad device";
    case XCORR_ERR_TIMEOUT: return "device-side wait timed out";
    case XCORR_ERR_INTERNAL: return "host-side failure inside the library";
    default: return "unknown status";
    }
}

void xcorr_debug_stage_wait(uint32_t poll_limit, uint32_t surplus_bytes) {
    g_stage_wait_limit.store(poll_limit ? poll_limit : kStageWaitLimit, std::memory_order_relaxed);
    g_stage_expect_surplus.store(surplus_bytes, std::memory_order_relaxed);
}

uint64_t xcorr_launch_count(void) { return t_launch_count; }
void xcorr_reset_launch_count(void) { t_launch_count = 0; }

xcorr_status xcorr_ffma_peak_probe(double* flops_per_second, double* kernel_ms, void* stream_v) {
    return guarded([&]() -> xcorr_status {
        if (!flops_per_second) return fail(XCORR_ERR_NULL_POINTER, "flops_per_second must not be NULL");
        cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
        DeviceInfo dev;
        xcorr_status st = current_device_info(&dev);
        if (st != XCORR_OK) return st;
        float* sink = nullptr;
        XC_CUDA(cudaMalloc(&sink, sizeof(float)));
        cudaEvent_t e0, e1;
        XC_CUDA(cudaEventCreate(&e0));
        XC_CUDA(cudaEventCreate(&e1));
        const int blocks = dev.sm_count * 2, iters = 4096;
        double best_ms = 1e30;
        for (int rep = 0; rep < 4; ++rep) {            // first repetition is the warm-up
            XC_CUDA(cudaEventRecord(e0, stream));
            XC_CUDA(launch_ffma_probe(sink, iters, blocks, stream));
            XC_CUDA(cudaEventRecord(e1, stream));
            XC_CUDA(cudaEventSynchronize(e1));
            float ms = 0.f;
            XC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
            if (rep > 0 && ms < best_ms) best_ms = ms;
            ++t_launch_count;
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        cudaFree(sink);
        const double flop = 2.0 * 16.0 * 8.0 * (double)iters * 1024.0 * (double)blocks;
        *flops_per_second = flop / (best_ms * 1e-3);
        if (kernel_ms) *kernel_ms = best_ms;
        return XCORR_OK;
    });
}

xcorr_status xcorr_dfma_peak_probe(double* flops_per_second, double* kernel_ms, void* stream_v) {
    return guarded([&]() -> xcorr_status {
        if (!flops_per_second) return fail(XCORR_ERR_NULL_POINTER, "flops_per_second must not be NULL");
        cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
        DeviceInfo dev;
        xcorr_status st = current_device_info(&dev);
        if (st != XCORR_OK) return st;
        double* sink = nullptr;
        XC_CUDA(cudaMalloc(&sink, sizeof(double)));
        cudaEvent_t e0, e1;
        XC_CUDA(cudaEventCreate(&e0));
        XC_CUDA(cudaEventCreate(&e1));
        const int blocks = dev.sm_count * 2, iters = 2048;
        double best_ms = 1e30;
        for (int rep = 0; rep < 4; ++rep) {            // first repetition is the warm-up
            XC_CUDA(cudaEventRecord(e0, stream));
            XC_CUDA(launch_dfma_probe(sink, iters, blocks, stream));
            XC_CUDA(cudaEventRecord(e1, stream));
            XC_CUDA(cudaEventSynchronize(e1));
            float ms = 0.f;
            XC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
            if (rep > 0 && ms < best_ms) best_ms = ms;
            ++t_launch_count;
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        cudaFree(sink);
        const double flop = 2.0 * 16.0 * 8.0 * (double)iters * 1024.0 * (double)blocks;
        *flops_per_second = flop / (best_ms * 1e-3);
        if (kernel_ms) *kernel_ms = best_ms;
        return XCORR_OK;
    });
}

}  // extern "C"
