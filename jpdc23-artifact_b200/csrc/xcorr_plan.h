// Launch plan of the register-tiled circular-class kernel, shared by the planner (host),
// the launcher and the kernel itself.
//
// Circular classes.  Pad the matrices with zeros to Hp x Wp.  For a class
// (cy, cx) in [0,Hp) x [0,Wp) accumulate, over every right element (ry, rx),
//     left[(ry + cy) mod Hp][(rx + cx) mod Wp] * right[ry][rx].
// Every product of the true cross-correlation appears in exactly one class, and within a
// class the terms split by whether the row / column index wrapped:
//     no x wrap -> shift sx = cx          x wrap -> shift sx = cx - Wp
//     no y wrap -> shift sy = cy          y wrap -> shift sy = cy - Hp
// so one class feeds (up to) four outputs and costs exactly Hp*Wp multiply-adds whatever
// the shift: no overlap clamping in the inner loop, no idle lanes at the corners, and the
// total is Hp^2*Wp^2 -- the algorithmic W^2*H^2 when no padding is needed.  This replaces
// the reference's zero-filled out-of-range loads (bound_checked_loads.cuh:23-25) and its
// startup / wind-down ladders (naive_shuffle_multirow_both.cu:244-292).
#pragma once
#include <cstddef>
#include <cstdint>

namespace xcorr {

constexpr int kTX = 16;           // x classes per thread (one 16-wide tile)
constexpr int kMaxTY = 4;         // y classes per thread
constexpr int kMaxWarps = 16;     // warps per block
constexpr int kSmallBlockThreads = 384;  // blocks up to this size run the 168-register build of the kernel
constexpr int kSmemLimit = 227 * 1024;
// per-warp staging area of the output flush: 32 rows of kTX + 1 floats and 32 row addresses
constexpr int kFlushBytesPerWarp = 32 * (kTX + 1) * 4 + 32 * 8;

// kFixup (stream-K only): a part of a task is stored to its own partial image; the block that
// finishes a task's last outstanding part sums the parts in their fixed order into the output.
enum Combine : int { kStore = 1, kAtomic = 2, kWorkspace = 3, kFixup = 4 };
enum Schedule : int { kSchedStatic = 1, kSchedStreamK = 2, kSchedWarpQueue = 3 };

// Warp-queue schedule: weight of a pass task in quarter chunks per row = 4 * full chunks +
// kQueueTriangleWeight (the tile's own two chunks, one triangle each, and the per-row code).
constexpr unsigned kQueueTriangleWeight = 6;
#if defined(__CUDACC__)
__host__ __device__
#endif
inline unsigned queue_units_per_yrow(int NTX) {
    // sum over k < NTX of 2 * (4 * (2*NTX - 2 - 2k) + triangle)
    return 2u * (unsigned)NTX * (4u * (unsigned)(NTX - 1) + kQueueTriangleWeight);
}

// How the pairs of a mode are enumerated: left l in [0, n_left) meets rights
// l*right_stride + j, j in [0, m); the result matrix is l*m + j.
//   one_to_one   n_left=1 m=1        one_to_many  n_left=1 m=n_right
//   n_to_m       m=n_right stride=0  n_to_mn      m=n_right/n_left stride=m
struct PairMap {
    uint32_t n_left;
    uint32_t m;
    uint32_t right_stride;
};

struct TilePlan {
    int H, W;          // true size
    int Hp, Wp;        // padded size: Wp multiple of 16, Hp multiple of SL*TY
    int TY;            // y classes per thread (template parameter of the kernel)
    int SL, ML;        // lanes over y classes / lanes over right matrices, SL*ML = 32
    int logSL;
    int NTX;           // x-class tiles = Wp / 16
    int NCH;           // 8-step chunks per row = Wp / 8
    int NGY;           // y-class groups = Hp / (SL*TY)
    int WX, WY;        // warps of a block along x tiles / y groups
    int CX, CY;        // blocks needed along x tiles / y groups
    int S;             // row slices of the right matrices (1 unless the schedule is static)
    int schedule;      // Schedule
    unsigned tasks;    // block tasks = n_left * RG * CX * CY (warp queue: matrix groups = n_left * RG)
    int RSmax;         // rows of the longest slice
    int RG;            // right-matrix groups per left = ceil(m / ML)
    int KG;            // matrix groups staged together (1 unless the schedule is the warp queue)
    int KL;            // left matrices with staged rows of their own (1 unless the schedule is the warp queue)
    int fused;         // 1: rows of 32 padded columns run both passes fused (one class per thread)
    int nstage;        // left rows staged in shared memory (at most; a short segment stages fewer)
    int LS;            // floats between staged left rows (Wp + 4: row*LS/4 odd -> conflict-free float4)
    int RMS;           // floats between the staged right matrices of one block
    int threads;
    int combine;       // Combine
    int pieces;        // kFixup: most parts any task is cut into (partial images in the workspace)
    unsigned grid;
    size_t smem_bytes;
    size_t workspace_bytes;
};

// Kernel arguments (passed by value).
struct TileArgs {
    const float* left;
    const float* right;
    float* out;
    float* ws;         // partial images: S (kWorkspace) or p.pieces (kFixup) * total_out floats, or nullptr
    unsigned* counters;  // kFixup: one zeroed counter per block task (finished parts)
    TilePlan p;
    PairMap pm;
    int vec_ok;        // rows may be fetched with 16-byte loads
    unsigned long long total_out;  // floats in the whole output array
    unsigned stage_wait_limit;     // polls after which a wait on the staging barrier gives up
    unsigned stage_expect_surplus; // test hook: bytes announced on the staging barrier that never arrive
};

// Default bound of the staging wait: ~4 million polls, a second or so; healthy copies land in microseconds.
constexpr unsigned kStageWaitLimit = 1u << 22;

// Plan and arguments of the double-precision tile kernel (xcorr_f64_tile.cu): the float plan's
// fields where they mean the same; 8 x classes and one y class per thread, static blocks, S row slices.
struct TilePlan64 {
    int H, W, Hp, Wp;
    int SL, ML, logSL;
    int NTX, NCH, NGY;
    int WX, WY, CX, CY, RG;
    int S;             // row slices (S > 1: sums added atomically onto the zeroed output)
    int nstage, LS, RMS;
    int threads;
    unsigned grid;
    size_t smem_bytes;
};
struct TileArgs64 {
    const double* left;
    const double* right;
    double* out;
    TilePlan64 p;
    PairMap pm;
    int vec_ok;        // rows may be fetched two doubles at a time
};

// Arguments of the staged warp-per-overlap kernel: a block owns one x shift, `shifts` consecutive
// y shifts (one per warp) and up to `rights` right matrices of one left; operands go through
// shared memory in slabs of `srows` right rows x `scols` columns, two slabs in flight.
struct StagedArgs {
    const float* left;
    const float* right;
    float* out;
    int H, W;
    PairMap pm;
    int shifts;        // warps per block = consecutive y shifts
    int srows, scols;  // slab: right rows x columns
    int rights;        // right matrices per block (1..8)
    int col_groups;    // 1: every column slab is a block of its own (grid z), sums added atomically
    int warp_rows;     // loader: 0 = threads stride over the slab's elements, 1 = a warp per row
    unsigned groups_per_left;   // ceil(m / rights)
};

// Row split of the plain warp-per-overlap kernel: an overlap's rows are divided over several
// warps ("workers") which add their sums atomically.
enum RowSplit : int { kSplitNone = 0, kSplitRectangle = 1, kSplitTriangle = 2 };

}  // namespace xcorr
