// Device code of the direct 2-D cross-correlation library (sm_100a).
//
// Three kernel families:
//   tile_kernel<TY, BOUND, VARIANT>
//                          register-tiled circular-class kernel; the fast path for every
//                          mode.  Stands in for the reference's warp-shuffle families
//                          (naive_shuffle*.cu): grouped-overlap, multi-matrix-right/both
//                          and, with row slices or stream-K, the split-row ("work
//                          distribution") ones.  Operands are staged with bulk copies
//                          (cp.async.bulk + mbarrier) or 16-byte cp.async.
//   overlap_wise_kernel    one thread per overlap (naive_original.cu:37-102).
//   warp_per_overlap_kernel one warp per overlap (naive_warp_per_shift.cu:192-244).
// plus the fixed-order reduction of workspace partials and the FFMA peak probe.
#include <cuda_runtime.h>
#include <atomic>
#include <cstdint>
#include <mutex>

#include "xcorr_plan.h"
#include "xcorr_launch.h"

namespace xcorr {

// ------------------------------------------------------------------------------------------
// tile kernel
// ------------------------------------------------------------------------------------------
//
// Work split.  A warp owns one 16-wide tile of x classes (the same for all its lanes) and
// SL*TY y classes: lane (m, q), q in [0,SL), holds classes cyw + q + SL*t, t in [0,TY), for
// right matrix m of the block's group (ML = 32/SL matrices per warp).  A block is WX x WY
// such warps sharing one left matrix, ML right matrices and one slice [r0, r1) of right
// rows, all staged in shared memory once.
//
// Per right row ry the thread walks the left row's columns u in chunks of 8:
//     acc[t][j] += L[(ry + cy_t) mod Hp][u] * R[ry][(u - cx0 - j) mod Wp],  j in [0,16)
// The R values a chunk needs are a 23-wide window that slides by one per step; each chunk
// fetches it with six 16-byte loads (all lanes of a matrix read the same addresses), the
// left values are two 16-byte loads per y class: 128*TY FFMA against 2*TY + 6 loads, no
// shuffles, no loop-carried window registers.
//
// x wrap: column j has wrapped while u < cx0 + j.  Instead of two accumulator sets the
// slice is walked twice with one set: pass B (wrapped part, output shift cx - Wp) takes the
// chunks u < cx0 in full and the two chunks of the tile's own columns in their lower
// triangle (step < j); pass A (unwrapped part, output shift cx) takes the upper triangle
// (step >= j) and the chunks behind it.  Together exactly Wp multiply-adds per class and
// row; only the tile's own two chunks are loaded twice.
// y wrap: class cy wraps from row ry = Hp - cy on.  The row loop writes a class's sums to
// the unwrapped output row when it reaches that row, and to the wrapped (or still
// unwrapped) one at the end of the slice.

enum Pass : int { kPassWrapped = 0, kPassUnwrapped = 1 };
enum Build : int { kBuildPlain = 0, kBuildFixup = 1, kBuildQueue = 2 };

// 16-byte shared-memory load through a 32-bit shared-window address (one register per
// address instead of the two a generic pointer takes).
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

// Asynchronous 16-byte copy global -> shared (no register round trip, so a thread can have all
// the copies of a staging loop in flight at once); completed by stage_wait().
__device__ __forceinline__ void stage_copy16(uint32_t dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void stage_wait() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// ---- bulk staging (TMA, non-tensor form): whole rows / whole row blocks of a matrix go
// global -> shared as one cp.async.bulk each, completion counted in bytes on an mbarrier.
// Used when rows need no column padding (cols a multiple of 16) and the operands are 16-byte
// aligned; everything else takes the 16-byte cp.async path above.
// Waits on the mbarrier are bounded: after TileArgs::stage_wait_limit polls (twice) the wait
// gives up.  The block then agrees on that (one vote at its next barrier), counts one timeout in
// g_stage_timeouts (read and cleared by the host through tile_stage_timeouts()), drops the rest
// of its work and returns: nothing is computed from a buffer whose copies did not land.
__device__ unsigned g_stage_timeouts = 0;

__device__ __forceinline__ void mbar_init(uint32_t bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const float* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_complete_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.complete_tx.relaxed.cta.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, unsigned limit) {
    for (int attempt = 0; attempt < 2; ++attempt)
        for (unsigned it = 0; it < limit; ++it)
            if (mbar_poll(bar, parity)) return true;
    return false;
}

// Load the N4*4 floats at `addr` into w[FIRST ...].
template<int FIRST, int N4, int LEN>
__device__ __forceinline__ void window_load(float (&w)[LEN], uint32_t addr) {
#pragma unroll
    for (int i = 0; i < N4; ++i) {
        const float4 v = lds128(addr + 16 * i);
        w[FIRST + 4 * i] = v.x; w[FIRST + 4 * i + 1] = v.y; w[FIRST + 4 * i + 2] = v.z; w[FIRST + 4 * i + 3] = v.w;
    }
}

// One chunk of 8 steps: acc[t][j] += L_t[u0 + kk] * w[16 + kk - j], where w[i] holds
// R[(u0 - cx0 - 16 + i) mod Wp].  TRI < 0: every (step, column) pair.  TRI = 0 / 1: first /
// second chunk of the tile's own columns, where only the pairs on the pass's side of the
// diagonal count: step >= j for the unwrapped pass, step < j for the wrapped one.
template<int TY, int TRI, int PASS>
__device__ __forceinline__ void tile_chunk(float (&acc)[TY][kTX], const float (&w)[24],
                                           const uint32_t (&lp)[TY], uint32_t col_bytes) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int t = 0; t < TY; ++t) {
            bool any = TRI < 0;
#pragma unroll
            for (int k = 0; k < 4; ++k)
#pragma unroll
                for (int j = 0; j < kTX; ++j)
                    any = any || (((8 * TRI + 4 * half + k) >= j) == (PASS == kPassUnwrapped));
            if (!any) continue;               // this half contributes nothing on this side
            const float4 lv = lds128(lp[t] + col_bytes + 16 * half);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int kk = 4 * half + k;
                const float l = k == 0 ? lv.x : k == 1 ? lv.y : k == 2 ? lv.z : lv.w;
#pragma unroll
                for (int j = 0; j < kTX; ++j) {
                    const int step = 8 * (TRI < 0 ? 0 : TRI) + kk;
                    const bool take = TRI < 0 || ((step >= j) == (PASS == kPassUnwrapped));
                    if (take) acc[t][j] = fmaf(l, w[16 + kk - j], acc[t][j]);
                }
            }
        }
    }
}

// All chunks of one right row for one pass.  `rrow` is the shared address of the row's
// first element, `lp` the shared addresses of the TY left rows.
template<int TY>
__device__ __forceinline__ void tile_row(float (&acc)[TY][kTX], const uint32_t (&lp)[TY], uint32_t rrow,
                                         int pass, int cb, int c_begin, int c_end, uint32_t roff_bytes,
                                         int Wp) {
    // chunks taken in full: the same code for both passes.  A tile is two chunks wide and the
    // padded row a whole number of tiles, so both passes take an even number of full chunks:
    // two per trip, no remainder.  Two chunks in flight let the loads of the second run under
    // the FFMAs of the first (+5..10 % measured on B200 against one per trip); four per trip
    // overflow the instruction cache for TY >= 3.
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 2) {
        {
            float w[24];
            window_load<0, 6>(w, rrow + roff_bytes + (uint32_t)c * 32);
            tile_chunk<TY, -1, 0>(acc, w, lp, (uint32_t)c * 32);
        }
        {
            float w[24];
            window_load<0, 6>(w, rrow + roff_bytes + (uint32_t)c * 32 + 32);
            tile_chunk<TY, -1, 0>(acc, w, lp, (uint32_t)c * 32 + 32);
        }
    }
    // the two chunks of the tile's own columns: one triangle per pass
    float w[24];
    if (pass == kPassWrapped) {
        // step < j: w[16 + kk - j] with kk - j in [-15, -1] -> R[Wp - 15 .. Wp - 1]
        window_load<0, 4>(w, rrow + (uint32_t)(Wp - 16) * 4);          // w[i] = R[Wp - 16 + i]
        tile_chunk<TY, 0, kPassWrapped>(acc, w, lp, (uint32_t)cb * 32);
        // second chunk: step = 8 + kk, R[Wp + 8 + kk - j]: shift the window view by 8
        float w2[24];
#pragma unroll
        for (int i = 0; i < 8; ++i) w2[i] = w[i + 8];                  // w2[i] = R[Wp - 8 + i]
        tile_chunk<TY, 1, kPassWrapped>(acc, w2, lp, (uint32_t)(cb + 1) * 32);
    } else {
        // step >= j: first chunk w[16 + kk - j], kk - j in [0, 7] -> R[0 .. 7]
        window_load<16, 2>(w, rrow);                                    // w[16 + i] = R[i]
        tile_chunk<TY, 0, kPassUnwrapped>(acc, w, lp, (uint32_t)cb * 32);
        // second chunk: R[8 + kk - j], 8 + kk - j in [0, 15]
        float w2[24];
        window_load<8, 4>(w2, rrow);                                    // w2[8 + i] = R[i]
        tile_chunk<TY, 1, kPassUnwrapped>(acc, w2, lp, (uint32_t)(cb + 1) * 32);
    }
}

// Per-warp staging area of the output flush: 32 rows of 16 sums (+1 padding word per row)
// and the 32 rows' destination addresses (xcorr_plan.h: kFlushBytesPerWarp).
constexpr int kFlushRowWords = kTX + 1;
static_assert(kFlushBytesPerWarp == 32 * kFlushRowWords * 4 + 32 * 8, "flush staging size");

// Write 16 sums per lane to the lanes' own output rows (lane -> one y class of one right
// matrix; `rowptr` = start of that output row, `has` = the lane has a row to write).  Done by
// the whole warp through a shared-memory transpose, 16 lanes per output row, so that a store
// instruction covers two rows of 16 consecutive floats instead of 32 scattered words.
// The code is one straight run -- 17 stores to shared memory, one warp barrier, 32 loads, 16
// global stores -- because what a flush costs is not its instructions but its dependent
// stalls: the other warps of the scheduler are in the FFMA loop and always ready, so every
// time this warp waits for a result it gets its next issue slot only some hundred cycles
// later (measured on B200: a flush written as a loop of dependent load -> store steps took
// ~10,000 cycles and warps spent 30-50 % of their life in it).  Must be called by all 32 lanes.
__device__ __forceinline__ void warp_flush(float* scratch, const float (&vals)[kTX], bool has, float* rowptr,
                                           int cx0, int W, int Wp, int pass, int combine, int lane) {
    unsigned long long* sbase = reinterpret_cast<unsigned long long*>(scratch + 32 * kFlushRowWords);
    float* row = scratch + lane * kFlushRowWords;
#pragma unroll
    for (int j = 0; j < kTX; ++j) row[j] = vals[j];
    sbase[lane] = has ? reinterpret_cast<unsigned long long>(rowptr) : 0ull;
    __syncwarp();
    const int c = lane & 15;
    const int cx = cx0 + c;
    // unwrapped pass: shift sx = cx; wrapped pass: shift sx = cx - Wp
    const int col = pass == kPassUnwrapped ? cx + W - 1 : cx - Wp + W - 1;
    const bool ok = pass == kPassUnwrapped ? cx < W : col >= 0;
    const int half = lane >> 4;
    float v[16];
    float* base[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int r = 2 * i + half;
        base[i] = reinterpret_cast<float*>(sbase[r]);
        v[i] = scratch[r * kFlushRowWords + c];
    }
    if (combine == kAtomic) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (base[i] != nullptr && ok) atomicAdd(base[i] + col, v[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (base[i] != nullptr && ok) base[i][col] = v[i];
    }
    __syncwarp();
}

// Both passes over the slice's rows for one thread, or (ONEPASS, the warp-queue build) the one pass
// `only_pass` as a task of its own.
template<int TY, bool ONEPASS>
__device__ __forceinline__ void tile_passes(const TilePlan& p, float* __restrict__ dst, uint32_t sL_addr,
                                            uint32_t rmat_addr, int r0, int r1, int cy0, int cya, int cx0,
                                            bool lane_live, int combine, float* flush_scratch, int lane,
                                            int cls_per_block, int only_pass) {
    const int H = p.H, W = p.W, Hp = p.Hp, Wp = p.Wp;
    const int OW = 2 * W - 1;
    // staged left rows of this segment: circular (all Hp rows) or a window of rows
    const int nstage = min(r1 - r0 + cls_per_block - 1, Hp);
    const uint32_t stage_bytes = (uint32_t)(nstage * p.LS * 4);
    const int cb = cx0 >> 3;                  // first chunk of the tile's own columns
    // first right row at which one of the warp's classes wraps in y (classes cyw .. cyw + SL*TY - 1)
    const int wrap_lo = Hp - ((cy0 & ~(p.SL - 1)) + p.SL * TY - 1);

#pragma unroll 1
    for (int pass = ONEPASS ? only_pass : 0; pass < (ONEPASS ? only_pass + 1 : 2); ++pass) {
        // wrapped pass: chunks [0, cb) with window R[Wp - cx0 - 16 + 8c ...];
        // unwrapped pass: chunks [cb + 2, NCH) with window R[8(c - cb) - 16 ...]
        const int c_begin = pass == kPassWrapped ? 0 : cb + 2;
        const int c_end = pass == kPassWrapped ? cb : p.NCH;
        const uint32_t roff_bytes = pass == kPassWrapped ? (uint32_t)(Wp - cx0 - 16) * 4
                                                         : (uint32_t)(-(8 * cb + 16) * 4);
        uint32_t lofs[TY];                    // byte offset of class t's staged left row
#pragma unroll
        for (int t = 0; t < TY; ++t) {
            int i = cy0 + p.SL * t - cya;    // staged row for ry = r0
            if (i >= nstage) i -= nstage;
            lofs[t] = (uint32_t)(i * p.LS * 4);
        }
        float acc[TY][kTX];
#pragma unroll
        for (int t = 0; t < TY; ++t)
#pragma unroll
            for (int j = 0; j < kTX; ++j) acc[t][j] = 0.f;

        // The final sums of the slice are written either by kEndTrips = TY extra trips of the row
        // loop (one copy of the flush code in the kernel; what the 168-register builds of
        // TY >= 3 run fastest with) or by a rolled loop behind it (TY <= 2: with the extra trips
        // the compiler moved all 32 accumulators at every trip of the row loop).  Measured on B200.
        constexpr int kEndTrips = TY >= 3 ? TY : 0;
        uint32_t rrow = rmat_addr;
#pragma unroll 1
        for (int ry = r0; ry < r1 + kEndTrips; ++ry, rrow += (uint32_t)Wp * 4) {
            const bool at_end = kEndTrips > 0 && ry >= r1;
            // A class that starts wrapping at this row: its unwrapped-in-y part is complete.
            // The wrap rows of the warp's SL * TY classes are consecutive (one range check for
            // the warp); those of a lane's classes differ, so at most one of them matches.
            if (at_end || ((unsigned)(ry - wrap_lo) < (unsigned)(p.SL * TY) && ry > r0)) {
                int tsel = -1;
                if (at_end) {
                    tsel = ry - r1;
                } else {
#pragma unroll
                    for (int t = 0; t < TY; ++t)
                        if (ry == Hp - (cy0 + p.SL * t)) tsel = t;
                }
                float vals[kTX];
#pragma unroll
                for (int j = 0; j < kTX; ++j) vals[j] = 0.f;
#pragma unroll
                for (int t = 0; t < TY; ++t) {
                    if (t == tsel) {
#pragma unroll
                        for (int j = 0; j < kTX; ++j) { vals[j] = acc[t][j]; acc[t][j] = 0.f; }
                    }
                }
                const int cyt = cy0 + p.SL * (tsel < 0 ? 0 : tsel);
                // at the end of the slice the sums belong to the wrapped output row if the class
                // wrapped inside (or before) the slice, else to the unwrapped one
                const int sy = (at_end && r1 > Hp - cyt) ? cyt - Hp : cyt;
                const bool has = tsel >= 0 && lane_live && sy > -H && sy < H;
                warp_flush(flush_scratch, vals, has, dst + (size_t)(sy + H - 1) * OW, cx0, W, Wp, pass, combine, lane);
                if (at_end) continue;
            }

            uint32_t lp[TY];
#pragma unroll
            for (int t = 0; t < TY; ++t) lp[t] = sL_addr + lofs[t];
            tile_row<TY>(acc, lp, rrow, pass, cb, c_begin, c_end, roff_bytes, Wp);
#pragma unroll
            for (int t = 0; t < TY; ++t) {
                lofs[t] += (uint32_t)p.LS * 4;
                if (lofs[t] == stage_bytes) lofs[t] = 0;
            }
        }

        // TY <= 2: a rolled loop over the classes (the class's sums picked by compares, not by
        // indexing) keeps this at one more copy of the flush code.
#pragma unroll 1
        for (int te = 0; te < (kEndTrips > 0 ? 0 : TY); ++te) {
            float vals[kTX];
#pragma unroll
            for (int j = 0; j < kTX; ++j) vals[j] = 0.f;
#pragma unroll
            for (int t = 0; t < TY; ++t) {
                if (t == te) {
#pragma unroll
                    for (int j = 0; j < kTX; ++j) vals[j] = acc[t][j];
                }
            }
            const int cyt = cy0 + p.SL * te;
            const int sy = r1 > Hp - cyt ? cyt - Hp : cyt;
            const bool has = lane_live && sy > -H && sy < H;
            warp_flush(flush_scratch, vals, has, dst + (size_t)(sy + H - 1) * OW, cx0, W, Wp, pass, combine, lane);
        }
    }
}

// ---- rows of 32 columns (17 .. 32 true columns), both passes fused -------------------------
// With Wp = 32 a whole right row is 32 registers, so a row needs no sliding windows at all: the
// row is loaded once (8 loads) and serves every step of both passes, each left row of a class is
// 8 loads, and the 32 x 16 (step, column) products per class are straight-line code in which
// every product knows at compile time whether its column index wrapped (wrapped: accW, output
// shift cx - 32; not wrapped: accU, shift cx).  Against the chunked walk above this removes the
// second visit of every row, the window reloads and most of the per-row address code: for 32-wide
// matrices those were a fifth of the executed instructions.  TILE = which of the row's two x
// tiles (cx0 = 16 * TILE).
template<int TY, int TILE>
__device__ __forceinline__ void fused32_row(float (&accU)[TY][kTX], float (&accW)[TY][kTX],
                                            const uint32_t (&lp)[TY], uint32_t rrow) {
    float r[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = lds128(rrow + 16 * i);
        r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int t = 0; t < TY; ++t) {
#pragma unroll
        for (int u4 = 0; u4 < 8; ++u4) {
            const float4 lv = lds128(lp[t] + 16 * u4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int u = 4 * u4 + k;
                const float l = k == 0 ? lv.x : k == 1 ? lv.y : k == 2 ? lv.z : lv.w;
#pragma unroll
                for (int j = 0; j < kTX; ++j) {
                    const int idx = (u - 16 * TILE - j) & 31;
                    if (u >= 16 * TILE + j) accU[t][j] = fmaf(l, r[idx], accU[t][j]);
                    else                    accW[t][j] = fmaf(l, r[idx], accW[t][j]);
                }
            }
        }
    }
}

// Write class `tsel` of both accumulator sets (and clear it); a rolled loop over the two passes
// so that the kernel holds the flush code once per call site.
template<int TY>
__device__ __forceinline__ void fused32_flush(float (&accU)[TY][kTX], float (&accW)[TY][kTX], int tsel, bool has,
                                              float* rowptr, int cx0, int W, int combine, float* flush_scratch, int lane) {
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
        float vals[kTX];
#pragma unroll
        for (int j = 0; j < kTX; ++j) vals[j] = 0.f;
#pragma unroll
        for (int t = 0; t < TY; ++t) {
            if (t == tsel) {
#pragma unroll
                for (int j = 0; j < kTX; ++j) {
                    if (pass == kPassUnwrapped) { vals[j] = accU[t][j]; accU[t][j] = 0.f; }
                    else                        { vals[j] = accW[t][j]; accW[t][j] = 0.f; }
                }
            }
        }
        warp_flush(flush_scratch, vals, has, rowptr, cx0, W, 32, pass, combine, lane);
    }
}

// The rows [r0, r1) of one tile, TILE known at compile time: the row loop holds nothing but the
// row itself, one compare for the next flush event and the left-row pointer updates.
template<int TY, int TILE>
__device__ __forceinline__ void fused32_rows(float (&accU)[TY][kTX], float (&accW)[TY][kTX], uint32_t (&lofs)[TY],
                                             uint32_t sL_addr, uint32_t rrow, int r0, int r1, int Hp, int H, int W,
                                             int SL, uint32_t ls_bytes, uint32_t stage_bytes, int cy0, bool lane_live,
                                             float* __restrict__ dst, int combine, float* flush_scratch, int lane) {
    const int OW = 2 * W - 1;
    // the warp's classes start wrapping in y at the consecutive rows wrap_lo .. wrap_lo + SL*TY - 1:
    // when the walk reaches such a row the class's unwrapped-in-y sums are complete and are written
    const int wrap_lo = Hp - ((cy0 & ~(SL - 1)) + SL * TY - 1);
    const int wrap_hi = wrap_lo + SL * TY;
    int next_evt = max(wrap_lo, r0 + 1);
    if (next_evt >= wrap_hi) next_evt = 0x7fffffff;
#pragma unroll 1
    for (int ry = r0; ry < r1; ++ry, rrow += 32 * 4) {
        if (ry == next_evt) {
            int tsel = -1;
#pragma unroll
            for (int t = 0; t < TY; ++t)
                if (ry == Hp - (cy0 + SL * t)) tsel = t;
            const int cyt = cy0 + SL * (tsel < 0 ? 0 : tsel);
            const bool has = tsel >= 0 && lane_live && cyt < H;
            fused32_flush<TY>(accU, accW, tsel, has, dst + (size_t)(cyt + H - 1) * OW, TILE * kTX, W, combine, flush_scratch, lane);
            next_evt = ry + 1 < wrap_hi ? ry + 1 : 0x7fffffff;
        }
        uint32_t lp[TY];
#pragma unroll
        for (int t = 0; t < TY; ++t) lp[t] = sL_addr + lofs[t];
        fused32_row<TY, TILE>(accU, accW, lp, rrow);
#pragma unroll
        for (int t = 0; t < TY; ++t) {
            lofs[t] += ls_bytes;
            if (lofs[t] == stage_bytes) lofs[t] = 0;
        }
    }
}

template<int TY>
__device__ __forceinline__ void tile_fused32(const TilePlan& p, float* __restrict__ dst, uint32_t sL_addr,
                                             uint32_t rmat_addr, int r0, int r1, int cy0, int cya, int tile,
                                             bool lane_live, int combine, float* flush_scratch, int lane,
                                             int cls_per_block) {
    const int H = p.H, W = p.W, Hp = p.Hp;
    const int OW = 2 * W - 1;
    const int nstage = min(r1 - r0 + cls_per_block - 1, Hp);
    const uint32_t ls_bytes = (uint32_t)p.LS * 4;
    const uint32_t stage_bytes = (uint32_t)nstage * ls_bytes;
    const int cx0 = tile * kTX;
    uint32_t lofs[TY];
#pragma unroll
    for (int t = 0; t < TY; ++t) {
        int i = cy0 + p.SL * t - cya;
        if (i >= nstage) i -= nstage;
        lofs[t] = (uint32_t)i * ls_bytes;
    }
    float accU[TY][kTX], accW[TY][kTX];
#pragma unroll
    for (int t = 0; t < TY; ++t)
#pragma unroll
        for (int j = 0; j < kTX; ++j) { accU[t][j] = 0.f; accW[t][j] = 0.f; }

    if (tile == 0)
        fused32_rows<TY, 0>(accU, accW, lofs, sL_addr, rmat_addr, r0, r1, Hp, H, W, p.SL, ls_bytes, stage_bytes, cy0,
                            lane_live, dst, combine, flush_scratch, lane);
    else
        fused32_rows<TY, 1>(accU, accW, lofs, sL_addr, rmat_addr, r0, r1, Hp, H, W, p.SL, ls_bytes, stage_bytes, cy0,
                            lane_live, dst, combine, flush_scratch, lane);
#pragma unroll 1
    for (int te = 0; te < TY; ++te) {
        const int cyt = cy0 + p.SL * te;
        const int sy = r1 > Hp - cyt ? cyt - Hp : cyt;
        const bool has = lane_live && sy > -H && sy < H;
        fused32_flush<TY>(accU, accW, te, has, dst + (size_t)(sy + H - 1) * OW, cx0, W, combine, flush_scratch, lane);
    }
}

// Stream-K with fix-up: sum the parts of one block task, in the order of their rows, into the
// output.  Part k of the task covers right rows [e_k, e_k+1) (the cuts of the blocks' ranges);
// it has written the unwrapped-in-y row of class c iff e_k < Hp - c and the wrapped one iff
// e_k+1 > Hp - c, both x variants each.  One warp per pair of output rows of the task, lanes over
// their columns; the parts are read with L2 loads (other SMs wrote them during this launch),
// up to four parts of up to eight elements in flight per lane: the sum is latency-bound.
struct FixupTask {            // passed by value: a reference to the kernel's parameters would
    const float* ws;          // force a copy of them onto the stack of every thread
    float* out;
    unsigned long long total_out;
    int H, W, Hp, Wp, ML, WX;
    unsigned tasks, m;
    unsigned task_id, first_block;
    int l, rg, by, bx, n_parts, cls_per_block;
};

__device__ __noinline__ void fixup_finalize(const FixupTask f) {
    const int H = f.H, W = f.W, Hp = f.Hp, Wp = f.Wp;
    const int l = f.l, rg = f.rg, by = f.by, bx = f.bx, n_parts = f.n_parts, cls_per_block = f.cls_per_block;
    const unsigned first_block = f.first_block;
    const int OW = 2 * W - 1, OH = 2 * H - 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const unsigned long long total = (unsigned long long)f.tasks * H;
    const unsigned long long task_u = (unsigned long long)f.task_id * H;
    const int cya = by * cls_per_block;
    const int xw = f.WX * kTX;                    // x classes of the block
    constexpr int kRows = 2, kSlots = 4, kParts = 4, kCuts = 9;
    const int rows_total = f.ML * cls_per_block * 2;
    // row cuts of the first parts, once (64-bit divisions); tasks in more parts recompute them
    int cut[kCuts];
#pragma unroll
    for (int k = 0; k < kCuts; ++k)
        cut[k] = k == 0 ? 0 : k >= n_parts ? H : (int)(total * (first_block + k) / gridDim.x - task_u);
    for (int rbase = warp * kRows; rbase < rows_total; rbase += nwarps * kRows) {
        size_t row_off[kRows];
        int k_lo[kRows], k_hi[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int rid = rbase + r;
            k_lo[r] = 0; k_hi[r] = -1; row_off[r] = 0;
            if (rid >= rows_total) continue;
            const int mm = rid / (cls_per_block * 2);
            const int rem = rid - mm * cls_per_block * 2;
            const int c = cya + (rem >> 1);
            const int wrapped = rem & 1;
            const unsigned j = (unsigned)rg * f.ML + mm;
            const int sy = wrapped ? c - Hp : c;
            if (j >= f.m || c >= Hp || sy <= -H || sy >= H) continue;
            int lo = n_parts, hi = -1;            // parts that wrote this row: a run lo .. hi
            if (n_parts < kCuts) {
#pragma unroll
                for (int k = 0; k < kCuts - 1; ++k)
                    if (k < n_parts && (wrapped ? cut[k + 1] > Hp - c : cut[k] < Hp - c)) { lo = min(lo, k); hi = max(hi, k); }
            } else {
                for (int k = 0; k < n_parts; ++k) {
                    const long long e0 = k == 0 ? 0 : (long long)(total * (first_block + k) / gridDim.x - task_u);
                    const long long e1 = k == n_parts - 1 ? H : (long long)(total * (first_block + k + 1) / gridDim.x - task_u);
                    if (wrapped ? e1 > Hp - c : e0 < Hp - c) { lo = min(lo, k); hi = max(hi, k); }
                }
            }
            k_lo[r] = lo; k_hi[r] = hi;
            row_off[r] = ((size_t)l * f.m + j) * (size_t)OH * OW + (size_t)(sy + H - 1) * OW;
        }
        for (int x0 = 0; x0 < 2 * xw; x0 += 32 * kSlots) {
            int col[kSlots];
#pragma unroll
            for (int sl = 0; sl < kSlots; ++sl) {
                const int xi = x0 + sl * 32 + lane;
                const int xv = xi >= xw;
                const int cx = bx * xw + (xv ? xi - xw : xi);
                const int cc = xv ? cx - Wp + W - 1 : cx + W - 1;
                col[sl] = (xi < 2 * xw && cx < Wp && (xv ? cc >= 0 : cx < W)) ? cc : -1;
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                float sum[kSlots];
#pragma unroll
                for (int sl = 0; sl < kSlots; ++sl) sum[sl] = 0.f;
                for (int kb = k_lo[r]; kb <= k_hi[r]; kb += kParts) {
                    float v[kParts][kSlots];
#pragma unroll
                    for (int kk = 0; kk < kParts; ++kk)
#pragma unroll
                        for (int sl = 0; sl < kSlots; ++sl)
                            v[kk][sl] = (kb + kk <= k_hi[r] && col[sl] >= 0)
                                ? __ldcg(f.ws + (size_t)(kb + kk) * f.total_out + row_off[r] + col[sl]) : 0.f;
#pragma unroll
                    for (int kk = 0; kk < kParts; ++kk)
#pragma unroll
                        for (int sl = 0; sl < kSlots; ++sl) sum[sl] += v[kk][sl];
                }
                if (k_hi[r] >= k_lo[r]) {
#pragma unroll
                    for (int sl = 0; sl < kSlots; ++sl)
                        if (col[sl] >= 0) f.out[row_off[r] + col[sl]] = sum[sl];
                }
            }
        }
    }
}

// Warp-queue schedule: the unit of work is one pass of one warp tile -- (matrix group, y group, x
// tile, wrapped / unwrapped pass), all rows.  The two passes of a tile write different outputs, so
// splitting them costs nothing and makes tasks of different lengths: with NTX tiles per row, pass
// k' = (unwrapped, tile k) and (wrapped, tile NTX-1-k) both take NCH - 2 - 2k full chunks per row
// plus the tile's own two chunks in a triangle.  Task ids run group-major, then y group, then k
// (longest first), then the two passes of that length; weights are in quarter chunks per row.
__device__ __forceinline__ unsigned queue_weight(int k, int NCH) { return 4u * (unsigned)(NCH - 2 - 2 * k) + kQueueTriangleWeight; }
// First task whose weight prefix reaches `units`.
__device__ unsigned long long queue_task_at(unsigned long long units, int NTX, int NCH) {
    const unsigned long long wy = (unsigned long long)queue_units_per_yrow(NTX);
    const unsigned long long yrow = units / wy, rem = units - yrow * wy;
    unsigned j = 0;
    unsigned long long pre = 0;
    while (j < 2u * NTX && pre < rem) { pre += queue_weight((int)(j >> 1), NCH); ++j; }
    return yrow * (2ull * NTX) + j;
}

// BOUND = 384: blocks of up to 12 warps, up to 168 registers per thread (nothing of the hot
// loop spills for TY = 4); BOUND = 512: blocks of 13..16 warps at 128 registers.
// FIXUP: the build that can write parts of a cut stream-K task to partial images and sum them
// (combine = kFixup); kept apart because its extra code cost the other plans 1-2 % when it sat
// in the same kernel.
template<int TY, int BOUND, int VARIANT>
__global__ void __launch_bounds__(BOUND, 1) tile_kernel(const TileArgs a) {
    // Three builds of the kernel: plain (static and stream-K plans), with the fix-up of cut stream-K
    // tasks, and the warp queue.  Code of a schedule that sits in the same kernel costs the others a
    // few percent (instruction fetch, registers held across the row loop): measured on B200.
    constexpr bool FIXUP = VARIANT == kBuildFixup;
    constexpr bool QUEUE = VARIANT == kBuildQueue;
    extern __shared__ __align__(16) float smem[];
    // the fused 32-column rows hold two accumulator sets and a whole right row in registers: built for
    // one class per thread (with two, 16-warp blocks spill and 8..12-warp blocks at 168 registers ran
    // 1.5 times slower than the chunked walk: measured on B200, 32 x 32, 32 x 64 pairs)
    constexpr bool kFused = TY == 1 && !FIXUP;
    const TilePlan& p = a.p;
    float* sL = smem;
    float* sR = smem + (size_t)p.KL * p.nstage * p.LS;
    const int H = p.H, W = p.W, Hp = p.Hp, Wp = p.Wp;
    const int tid = threadIdx.x, nthr = blockDim.x;

    // ---- the block's share of the work.
    //      Static: block = (block task, slice): one segment of right rows.
    //      Stream-K: the (block task, right row) units of all tasks are cut into gridDim.x
    //      equal ranges; a range is one or more segments, each a run of rows of one task.
    //      Warp queue: the warp tasks (one x tile and one y group of one matrix group, all
    //      rows) are cut into gridDim.x equal ranges; a range is one or more phases, each the
    //      tasks of one matrix group, which the block's warps take from a shared counter.
    unsigned long long u, uend;
    int slice = 0;
    if (QUEUE) {
        // p.tasks = matrix groups; the weight units of all tasks cut evenly over the blocks
        if (kFused && p.fused) {                  // whole tiles, all of one length
            const unsigned long long total = (unsigned long long)p.tasks * p.NGY * p.NTX;
            u = total * blockIdx.x / gridDim.x;
            uend = total * (blockIdx.x + 1) / gridDim.x;
        } else {
            const unsigned long long total = (unsigned long long)p.tasks * p.NGY * queue_units_per_yrow(p.NTX);
            u = queue_task_at(total * blockIdx.x / gridDim.x, p.NTX, p.NCH);
            uend = queue_task_at(total * (blockIdx.x + 1) / gridDim.x, p.NTX, p.NCH);
        }
    } else if (p.schedule == kSchedStreamK) {
        const unsigned long long total = (unsigned long long)p.tasks * H;
        u = total * blockIdx.x / gridDim.x;
        uend = total * (blockIdx.x + 1) / gridDim.x;
    } else {
        const unsigned task = blockIdx.x / p.S;
        slice = blockIdx.x - task * p.S;
        u = (unsigned long long)task * H + (unsigned)(((long long)slice * H) / p.S);
        uend = (unsigned long long)task * H + (unsigned)(((long long)(slice + 1) * H) / p.S);
    }

    const int warp = tid >> 5, lane = tid & 31;
    const int wx = warp % p.WX, wy = warp / p.WX;
    const int q = lane & (p.SL - 1);
    const int m = lane >> p.logSL;
    const uint32_t sL_addr = (uint32_t)__cvta_generic_to_shared(sL);
    const uint32_t sR_addr = (uint32_t)__cvta_generic_to_shared(sR);
    const uint32_t rmat_addr = (uint32_t)__cvta_generic_to_shared(sR + (size_t)m * p.RMS);
    float* flush_scratch = reinterpret_cast<float*>(
        reinterpret_cast<char*>(sR + (size_t)p.KG * p.ML * p.RMS) + (size_t)warp * kFlushBytesPerWarp);
    int* queue = reinterpret_cast<int*>(reinterpret_cast<char*>(sR + (size_t)p.KG * p.ML * p.RMS) +
                                        (size_t)(nthr >> 5) * kFlushBytesPerWarp);
    // bulk staging: rows without column padding, 16-byte aligned operands
    const bool bulk = a.vec_ok && W == Wp;
    const uint32_t stage_bar = (uint32_t)__cvta_generic_to_shared(queue) + 8;
    uint32_t stage_parity = 0;
    if (bulk) {
        if (tid == 0) mbar_init(stage_bar);
        __syncthreads();
    }

    while (u < uend) {
        bool stage_ok = true;
        int r0, r1, bx, by, rg, l, combine, ngroups = 1, nlefts = 1;      // (both stay 1 outside the queue build)
        unsigned long long q_begin = 0, q_end = 0, q_yrow0 = 0;      // this round's tasks (warp queue)
        unsigned task_id = 0, first_block = 0;
        int n_parts = 1, part = 0;
        if (QUEUE) {
            // one round: up to KG consecutive matrix groups (of up to KL left matrices), staged together
            const unsigned t2 = (kFused && p.fused) ? (unsigned)p.NTX : 2u * (unsigned)p.NTX;   // tasks per y row
            q_yrow0 = u / t2;
            const unsigned g0 = (unsigned)(q_yrow0 / (unsigned)p.NGY);
            l = (int)(g0 / (unsigned)p.RG);
            rg = (int)(g0 - (unsigned)l * p.RG);
            unsigned g_last = (unsigned)(((uend - 1) / t2) / (unsigned)p.NGY);
            g_last = min(g_last, min(g0 + (unsigned)p.KG - 1u, (unsigned)(l + p.KL) * p.RG - 1u));
            ngroups = (int)(g_last - g0) + 1;
            nlefts = (int)(g_last / (unsigned)p.RG) - l + 1;
            q_begin = u;
            q_end = min(uend, (unsigned long long)(g_last + 1) * p.NGY * t2);
            u = q_end;
            r0 = 0; r1 = H; bx = 0; by = 0;
            combine = kStore;
        } else {
            unsigned task = (unsigned)(u / (unsigned)H);
            task_id = task;
            r0 = (int)(u - (unsigned long long)task * H);
            r1 = (int)min((unsigned long long)H, r0 + (uend - u));
            u += (unsigned)(r1 - r0);
            bx = task % p.CX; task /= p.CX;
            by = task % p.CY; task /= p.CY;
            rg = task % p.RG;
            l = task / p.RG;
            // a whole task is written with plain stores, a part of one is added to the zeroed output
            combine = p.schedule == kSchedStreamK ? ((r0 == 0 && r1 == H) ? (int)kStore : (int)kAtomic) : p.combine;
            if (FIXUP && p.schedule == kSchedStreamK && p.combine == kFixup && combine == kAtomic) {
                // which blocks share this task: block b owns units [total*b/G, total*(b+1)/G)
                const unsigned long long total = (unsigned long long)p.tasks * H;
                const unsigned long long t0 = (unsigned long long)task_id * H;
                first_block = (unsigned)(((t0 + 1) * gridDim.x - 1) / total);
                n_parts = (int)(((t0 + H) * gridDim.x - 1) / total) - (int)first_block + 1;
                part = (int)blockIdx.x - (int)first_block;
                combine = kFixup;
            }
        }

        // y classes the staged left rows must serve: the block's groups, or all in queue mode
        const int cls_per_block = QUEUE ? Hp : p.WY * p.SL * TY;
        const int cya = by * cls_per_block;          // first y class of the block
        int rowbase = r0 + cya;
        if (rowbase >= Hp) rowbase -= Hp;

        // Matrices staged behind each other: the block's group, or the round's groups (warp queue).
        // Staged matrix mm belongs to group rg + mm / ML counted from left l; a round may run on into
        // the groups of the following left matrices, each of which has a slot of staged rows of its own.
        const int nmat = ngroups * p.ML;
        const int log_ml = 5 - p.logSL;
        auto right_of = [&](int mm, size_t& rmat) -> bool {
            const unsigned gg = (unsigned)rg + (unsigned)(mm >> log_ml);
            const unsigned lt = QUEUE ? gg / (unsigned)p.RG : 0u;              // one group outside the queue build
            const unsigned j = (gg - lt * (unsigned)p.RG) * (unsigned)p.ML + (unsigned)(mm & (p.ML - 1));
            rmat = (size_t)(l + lt) * a.pm.right_stride + j;
            return j < a.pm.m;
        };
        const int nstage = min(r1 - r0 + cls_per_block - 1, Hp);   // staged rows per left (== p.nstage in a round)
        const int nlrows = QUEUE ? nlefts * nstage : nstage;
        // ---- stage the left rows: staged row i of a slot holds left row (rowbase + i) mod Hp, zeros
        //      where the padded matrix is zero.
        if (bulk) {
            const int rs = r1 - r0;
            const uint32_t row_bytes = (uint32_t)W * 4, mat_bytes = (uint32_t)(rs * W) * 4;
            if (warp == 0) {
                // one lane announces the bytes, all lanes of the warp issue the copies: staged
                // left rows first, then one copy per right matrix (its rows r0..r1-1 are contiguous)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                uint32_t bytes = 0;
                for (int i = lane; i < nlrows + nmat; i += 32) {
                    if (i < nlrows) {
                        int row = rowbase + (QUEUE ? i % nstage : i);
                        if (row >= Hp) row -= Hp;
                        if (row < H) bytes += row_bytes;
                    } else {
                        size_t rmat;
                        if (right_of(i - nlrows, rmat)) bytes += mat_bytes;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
                if (lane == 0) mbar_expect(stage_bar, bytes + a.stage_expect_surplus);
                __syncwarp();
                for (int i = lane; i < nlrows + nmat; i += 32) {
                    if (i < nlrows) {
                        const int ls = QUEUE ? i / nstage : 0;
                        int row = rowbase + (i - ls * nstage);
                        if (row >= Hp) row -= Hp;
                        if (row < H)
                            bulk_copy(sL_addr + (uint32_t)(i * p.LS) * 4, a.left + ((size_t)(l + ls) * H + row) * W, row_bytes, stage_bar);
                    } else {
                        const int mm = i - nlrows;
                        size_t rmat;
                        if (right_of(mm, rmat))
                            bulk_copy(sR_addr + (uint32_t)(mm * p.RMS) * 4, a.right + (rmat * H + r0) * W, mat_bytes, stage_bar);
                    }
                }
            }
            // rows and matrices of the zero padding: plain stores, one warp per row / matrix
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int i = warp; i < nlrows; i += nthr >> 5) {
                int row = rowbase + (QUEUE ? i % nstage : i);
                if (row >= Hp) row -= Hp;
                if (row >= H)
                    for (int x = lane * 4; x < Wp; x += 128) *reinterpret_cast<float4*>(sL + (size_t)i * p.LS + x) = zero4;
            }
            for (int mm = warp; mm < nmat; mm += nthr >> 5) {
                size_t rmat;
                if (!right_of(mm, rmat))
                    for (int x = lane * 4; x < rs * Wp; x += 128) *reinterpret_cast<float4*>(sR + (size_t)mm * p.RMS + x) = zero4;
            }
            stage_ok = mbar_wait_bounded(stage_bar, stage_parity, a.stage_wait_limit);
            if (!stage_ok) {
                // Gave up.  Before the block leaves, its own copies must have landed (the shared
                // memory they target goes to another block afterwards): take back the bytes a test
                // announced in surplus, then wait once more with the default bound.
                if (a.stage_expect_surplus != 0) {
                    __syncthreads();
                    if (tid == 0) mbar_complete_tx(stage_bar, a.stage_expect_surplus);
                }
                (void)mbar_wait_bounded(stage_bar, stage_parity, kStageWaitLimit);
            }
            stage_parity ^= 1u;
        } else {
        {
            const int units = p.LS >> 2;             // float4 per staged row (last one is padding)
            const int total = nlrows * units;
            for (int idx = tid; idx < total; idx += nthr) {
                const int i = idx / units, c4 = idx - i * units;
                const int ls = QUEUE ? i / nstage : 0;
                int row = rowbase + (i - ls * nstage);
                if (row >= Hp) row -= Hp;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                const int x = c4 * 4;
                if (row < H && x < W) {
                    const float* g = a.left + ((size_t)(l + ls) * H + row) * W + x;
                    if (a.vec_ok) {
                        stage_copy16(sL_addr + (uint32_t)(i * p.LS + x) * 4, g);
                        continue;
                    }
                    v.x = __ldg(g);
                    if (x + 1 < W) v.y = __ldg(g + 1);
                    if (x + 2 < W) v.z = __ldg(g + 2);
                    if (x + 3 < W) v.w = __ldg(g + 3);
                }
                *reinterpret_cast<float4*>(sL + (size_t)i * p.LS + x) = v;
            }
        }
        // ---- stage rows [r0, r1) of the staged right matrices, zeros for the padding
        //      columns and for matrices past the end of a left's group.
        {
            const int units = Wp >> 2;
            const int rs = r1 - r0;
            const int per_mat = rs * units;
            const int total = nmat * per_mat;
            for (int idx = tid; idx < total; idx += nthr) {
                const int mm = idx / per_mat;
                const int rem = idx - mm * per_mat;
                const int rr = rem / units, c4 = rem - rr * units;
                size_t rmat;
                const bool live = right_of(mm, rmat);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                const int x = c4 * 4;
                if (live && x < W) {
                    const float* g = a.right + (rmat * H + (r0 + rr)) * W + x;
                    if (a.vec_ok) {
                        stage_copy16(sR_addr + (uint32_t)(mm * p.RMS + rr * Wp + x) * 4, g);
                        continue;
                    }
                    v.x = __ldg(g);
                    if (x + 1 < W) v.y = __ldg(g + 1);
                    if (x + 2 < W) v.z = __ldg(g + 2);
                    if (x + 3 < W) v.w = __ldg(g + 3);
                }
                *reinterpret_cast<float4*>(sR + (size_t)mm * p.RMS + (size_t)rr * Wp + x) = v;
            }
        }
        stage_wait();
        }
        if (QUEUE && tid == 0) *queue = 0;
        if (__syncthreads_or(!stage_ok)) {
            if (tid == 0) atomicAdd(&g_stage_timeouts, 1u);
            break;
        }

        // ---- this warp's task(s): its fixed tile of the block task (both passes), or tasks popped from
        //      the round's queue -- one pass of a tile, longest first; whole tiles where rows run fused
        const bool fused = kFused && p.fused;
        const unsigned tpy = fused ? (unsigned)p.NTX : 2u * (unsigned)p.NTX;       // queue tasks per y row
        unsigned q_ny = 0, q_nv = 0;
        if (QUEUE) {
            q_ny = (unsigned)((q_end - 1) / tpy - q_yrow0) + 1u;
            q_nv = q_ny * tpy;
        }
        bool first = true;
        while (true) {
            int tile_x, grp_y, slot = 0, only_pass = 0, task_l = l, task_rg = rg;
            if (QUEUE) {
                unsigned v = 0;
                if (lane == 0) v = (unsigned)atomicAdd(queue, 1);
                v = __shfl_sync(0xffffffffu, v, 0);
                if (v >= q_nv) break;
                // queue position v -> (length class k, y row, which of the two tasks of that length)
                const unsigned per_k = fused ? q_ny : 2u * q_ny;
                const unsigned k = v / per_k, rem = v - k * per_k;
                const unsigned long long yrow = q_yrow0 + (fused ? rem : rem >> 1);
                const unsigned which = fused ? 0u : rem & 1u;
                const unsigned long long id = yrow * tpy + (fused ? k : 2u * k + which);
                if (id < q_begin || id >= q_end) continue;     // outside this round's range
                const unsigned g = (unsigned)(yrow / (unsigned)p.NGY);
                grp_y = (int)(yrow - (unsigned long long)g * p.NGY);
                slot = (int)(g - (unsigned)(l * p.RG + rg));
                task_l = (int)(g / (unsigned)p.RG);
                task_rg = (int)(g - (unsigned)task_l * p.RG);
                tile_x = (fused || which == 0) ? (int)k : p.NTX - 1 - (int)k;
                if (!fused) only_pass = which == 0 ? (int)kPassUnwrapped : (int)kPassWrapped;
            } else {
                tile_x = bx * p.WX + wx;
                grp_y = by * p.WY + wy;
                if (!first || tile_x >= p.NTX || grp_y >= p.NGY) break;
                first = false;
            }
            const unsigned jright = (unsigned)task_rg * p.ML + m;
            const bool lane_live = jright < a.pm.m;
            const int cy0 = grp_y * p.SL * TY + q;   // class t of this lane: cy0 + SL*t
            const size_t out_mat = (size_t)task_l * a.pm.m + jright;
            const uint32_t sl_task = QUEUE ? sL_addr + (uint32_t)((task_l - l) * p.nstage * p.LS) * 4 : sL_addr;   // the task's left slot
            float* dst = (combine == kWorkspace ? a.ws + (size_t)slice * a.total_out :
                          (FIXUP && combine == kFixup) ? a.ws + (size_t)part * a.total_out : a.out)
                         + out_mat * (size_t)(2 * W - 1) * (2 * H - 1);
            const uint32_t rsl = QUEUE ? rmat_addr + (uint32_t)(slot * p.ML * p.RMS) * 4 : rmat_addr;
            const int comb = (FIXUP && combine == kFixup) ? (int)kStore : combine;
            if constexpr (kFused) {
                if (fused) {
                    tile_fused32<TY>(p, dst, sl_task, rsl, r0, r1, cy0, cya, tile_x, lane_live, comb, flush_scratch,
                                     lane, cls_per_block);
                    continue;
                }
            }
            tile_passes<TY, QUEUE>(p, dst, sl_task, rsl, r0, r1, cy0, cya, tile_x * kTX, lane_live, comb, flush_scratch, lane,
                                   cls_per_block, only_pass);
        }
        if (FIXUP && combine == kFixup) {
            // this part is written: count it; whoever counts the task's last part sums them
            __threadfence();
            __syncthreads();
            if (tid == 0) *queue = atomicAdd(a.counters + task_id, 1u) + 1u == (unsigned)n_parts ? 1 : 0;
            __syncthreads();
            if (*queue) {
                __threadfence();
                FixupTask f;
                f.ws = a.ws; f.out = a.out; f.total_out = a.total_out;
                f.H = H; f.W = W; f.Hp = Hp; f.Wp = Wp; f.ML = p.ML; f.WX = p.WX;
                f.tasks = p.tasks; f.m = a.pm.m; f.task_id = task_id; f.first_block = first_block;
                f.l = l; f.rg = rg; f.by = by; f.bx = bx; f.n_parts = n_parts; f.cls_per_block = cls_per_block;
                fixup_finalize(f);
            }
        }
        __syncthreads();                          // the next segment reuses the staging buffers
    }
}

// Sum the per-slice partial images in slice order.  One block per output row: slice s wrote
// output row `orow` (shift sy = orow - (H-1)) iff it holds right rows before the class's wrap
// row (sy >= 0) or after it (sy < 0); the other slices' words are unwritten and are skipped.
// The row's contributing slices are a contiguous range, found once per block.
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ ws,
                                                              float* __restrict__ out,
                                                              unsigned long long total_out,
                                                              int H, int W, int Hp, int S) {
    const int OW = 2 * W - 1, OH = 2 * H - 1;
    const unsigned long long rows_total = total_out / (unsigned long long)OW;   // matrices * OH
    for (unsigned long long grow = blockIdx.x; grow < rows_total; grow += gridDim.x) {
        const int orow = (int)(grow % (unsigned long long)OH);
        const int sy = orow - (H - 1);
        const int wrap_row = sy >= 0 ? Hp - sy : -sy;
        // Slice s holds the right rows [s*H/S, (s+1)*H/S).  It wrote this output row iff it starts
        // before the wrap row (sy >= 0: s*H < wrap_row*S) or ends after it (sy < 0:
        // (s+1)*H >= (wrap_row+1)*S): the contributing slices are [s_first, s_last).
        int s_first = 0, s_last = S;
        if (sy >= 0) s_last = (int)min((long long)S, ((long long)wrap_row * S + H - 1) / H);
        else s_first = (int)min((long long)S, max(0ll, ((long long)(wrap_row + 1) * S + H - 1) / H - 1));
        const unsigned long long base = grow * (unsigned long long)OW;
        const float* first = ws + (unsigned long long)s_first * total_out + base;
        for (int x = threadIdx.x; x < OW; x += blockDim.x) {
            // eight loads in flight, added in slice order (skipped slots add 0): the sum is the same
            // sequential one whatever the batch size, and latency is paid once per eight slices
            float sum = 0.f;
            const float* p = first + x;
            for (int s = s_first; s < s_last; s += 8, p += 8 * total_out) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = s + i < s_last ? __ldcg(p + (unsigned long long)i * total_out) : 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) sum += v[i];
            }
            out[base + x] = sum;
        }
    }
}

// ------------------------------------------------------------------------------------------
// overlap-wise: one thread per overlap, both operands straight from global memory
// ------------------------------------------------------------------------------------------
__global__ void overlap_wise_kernel(const float* __restrict__ left, const float* __restrict__ right,
                                    float* __restrict__ out, int H, int W, PairMap pm,
                                    unsigned long long npairs) {
    const int OW = 2 * W - 1, OH = 2 * H - 1;
    const int ox = blockIdx.x * blockDim.x + threadIdx.x;
    const int oy = blockIdx.y * blockDim.y + threadIdx.y;
    if (ox >= OW || oy >= OH) return;
    const int sx = ox - (W - 1), sy = oy - (H - 1);
    const int x0 = max(sx, 0), x1 = min(W + sx, W);
    const int y0 = max(sy, 0), y1 = min(H + sy, H);
    for (unsigned long long pair = blockIdx.z; pair < npairs; pair += gridDim.z) {
        const unsigned long long l = pair / pm.m, j = pair % pm.m;
        const float* L = left + l * (size_t)H * W;
        const float* R = right + (l * pm.right_stride + j) * (size_t)H * W;
        float sum = 0.f;
        for (int yl = y0; yl < y1; ++yl) {
            const float* lrow = L + (size_t)yl * W;
            const float* rrow = R + (size_t)(yl - sy) * W - sx;
            for (int xl = x0; xl < x1; ++xl) sum = fmaf(__ldg(rrow + xl), __ldg(lrow + xl), sum);
        }
        out[pair * (size_t)OW * OH + (size_t)oy * OW + ox] = sum;
    }
}

// ------------------------------------------------------------------------------------------
// warp-per-overlap: lanes over columns x rows of the overlap, butterfly sum
// ------------------------------------------------------------------------------------------
// Row split (naive_warp_per_shift.cu:100-189 with row_distribution.cuh): with rows_per_warp > 0
// the rows of an overlap are shared by several warps ("workers"), each taking
// ceil(overlap rows / workers) of them and adding its sum atomically onto the zeroed output.
// An output row oy has n(oy) = H - |oy - (H-1)| overlapping rows and needs
// ceil(n(oy) / rows_per_warp) workers.  kSplitRectangle gives every output row the
// ceil(H / rows_per_warp) worker slots of the centre row and lets the surplus ones return at
// once; kSplitTriangle enumerates exactly the workers needed (prefix sums in closed form).

// Workers needed by the output rows [0, y) of one result matrix, y <= H (upper half: row j has
// j + 1 overlapping rows): sum over j < y of ceil((j + 1) / r).
__device__ __forceinline__ unsigned long long split_workers_upper(unsigned y, unsigned r) {
    const unsigned long long q = y / r, rem = y % r;
    return (unsigned long long)r * q * (q + 1) / 2 + rem * (q + 1);
}
// ... by the output rows [0, y) for any y <= 2H - 1 (the lower half mirrors the upper one).
__device__ __forceinline__ unsigned long long split_workers_before(unsigned y, unsigned H, unsigned r) {
    if (y <= H) return split_workers_upper(y, r);
    // rows H .. y-1 have 2H-1-j overlapping rows = the rows 2H-1-y .. H-2 of the upper half
    return split_workers_upper(H, r) + split_workers_upper(H - 1, r) - split_workers_upper(2 * H - 1 - y, r);
}

// The sum of one overlap (columns [x0, x1), rows [y0, y1) of the left matrix against the right
// one shifted by (sx, sy)) by one warp, returned in every lane.  Lanes as lc columns x 32 / lc
// rows, lc the power of two that covers the overlap's width: narrow overlaps keep every lane
// busy (the reference spreads the overlap's elements over the lanes with a division per
// element, naive_warp_per_shift.cu:69-70).  Eight rows per trip, rows past the end predicated
// off, with all sixteen loads issued before the first multiply-add: for a pair of 16 x 16 the
// whole sum is one round trip to L2.
template<typename T>
__device__ __forceinline__ T warp_overlap_sum(const T* __restrict__ L, const T* __restrict__ R, int W,
                                              int sx, int sy, int x0, int x1, int y0, int y1, int lane) {
    int lc = 32;
    while (lc > 1 && (lc >> 1) >= x1 - x0) lc >>= 1;
    const int lrn = 32 / lc;
    const int c0 = x0 + (lane & (lc - 1));
    const int yfirst = y0 + lane / lc;
    const T* lbase = L + (size_t)yfirst * W;
    const T* rbase = R + (ptrdiff_t)(yfirst - sy) * W - sx;
    const size_t rstep = (size_t)lrn * W;
    T sum = T(0);
    for (int xl = c0; xl < x1; xl += lc) {
        const T* lp = lbase + xl;
        const T* rp = rbase + xl;
        for (int yl = yfirst; yl < y1; yl += 8 * lrn, lp += 8 * rstep, rp += 8 * rstep) {
            T lv[8], rv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool live = yl + i * lrn < y1;
                lv[i] = live ? __ldg(lp + i * rstep) : T(0);
                rv[i] = live ? __ldg(rp + i * rstep) : T(0);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) sum = fma(rv[i], lv[i], sum);
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    return sum;
}

// The unsplit form with 32-bit task arithmetic: what a handful of overlaps runs on, where the
// 64-bit divisions of the general kernel below are a visible part of the few microseconds.
// Also instantiated for double (the same latency kernel for xcorr_run_f64).
template<typename T>
__global__ void __launch_bounds__(1024) warp_per_overlap_direct_kernel(const T* __restrict__ left,
                                                                       const T* __restrict__ right,
                                                                       T* __restrict__ out, int H, int W,
                                                                       PairMap pm, unsigned ntasks) {
    const unsigned OW = 2u * W - 1, OH = 2u * H - 1, OE = OW * OH;
    const int lane = threadIdx.x & 31;
    const unsigned warps_per_grid = gridDim.x * (blockDim.x >> 5);
    for (unsigned task = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); task < ntasks; task += warps_per_grid) {
        const unsigned pair = ntasks == OE ? 0u : task / OE;
        const unsigned oi = task - pair * OE;
        const unsigned oyu = oi / OW;
        const int oy = (int)oyu, ox = (int)(oi - oyu * OW);
        const int sx = ox - (W - 1), sy = oy - (H - 1);
        const int x0 = max(sx, 0), x1 = min(W + sx, W);
        const int y0 = max(sy, 0), y1 = min(H + sy, H);
        const unsigned l = pm.m == 1 ? pair : pair / pm.m, j = pair - l * pm.m;
        const T* L = left + (size_t)l * H * W;
        const T* R = right + ((size_t)l * pm.right_stride + j) * (size_t)H * W;
        const T sum = warp_overlap_sum<T>(L, R, W, sx, sy, x0, x1, y0, y1, lane);
        if (lane == 0) out[(size_t)pair * OE + oi] = sum;
    }
}

__global__ void warp_per_overlap_kernel(const float* __restrict__ left, const float* __restrict__ right,
                                        float* __restrict__ out, int H, int W, PairMap pm,
                                        unsigned long long ntasks, int rows_per_warp, int split) {
    const int OW = 2 * W - 1, OH = 2 * H - 1;
    const unsigned long long OE = (unsigned long long)OW * OH;
    const int lane = threadIdx.x & 31;
    const unsigned long long warps_per_grid = (unsigned long long)gridDim.x * (blockDim.x >> 5);
    // worker slots of one result matrix: one per overlap, or the split's count per output row
    const unsigned slots_rect = split == kSplitRectangle ? (unsigned)((H + rows_per_warp - 1) / rows_per_warp) : 1u;
    const unsigned long long per_matrix =
        split == kSplitTriangle ? split_workers_before((unsigned)OH, (unsigned)H, (unsigned)rows_per_warp) * OW
                                : OE * slots_rect;
    for (unsigned long long task = (unsigned long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
         task < ntasks; task += warps_per_grid) {
        const unsigned long long pair = task / per_matrix;
        const unsigned long long ti = task - pair * per_matrix;
        int oy, ox, worker = 0, workers = 1;
        if (split == kSplitTriangle) {
            // worker rows: (output row, worker) pairs in row order, each OW overlaps wide
            const unsigned long long wrow = ti / OW;
            ox = (int)(ti - wrow * OW);
            int lo = 0, hi = OH - 1;                       // last row whose prefix is <= wrow
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (split_workers_before((unsigned)mid, (unsigned)H, (unsigned)rows_per_warp) <= wrow) lo = mid; else hi = mid - 1;
            }
            oy = lo;
            worker = (int)(wrow - split_workers_before((unsigned)oy, (unsigned)H, (unsigned)rows_per_warp));
        } else {
            const unsigned long long oi = ti / slots_rect;
            worker = (int)(ti - oi * slots_rect);
            oy = (int)(oi / OW); ox = (int)(oi - (unsigned long long)oy * OW);
        }
        const int sx = ox - (W - 1), sy = oy - (H - 1);
        const int x0 = max(sx, 0), x1 = min(W + sx, W);
        int y0 = max(sy, 0), y1 = min(H + sy, H);
        if (split != kSplitNone) {
            workers = (y1 - y0 + rows_per_warp - 1) / rows_per_warp;
            if (worker >= workers) continue;               // a surplus slot of the rectangle
            const int share = (y1 - y0 + workers - 1) / workers;
            y0 += worker * share;
            y1 = min(y1, y0 + share);
        }
        const unsigned long long l = pair / pm.m, j = pair % pm.m;
        const float* L = left + l * (size_t)H * W;
        const float* R = right + (l * pm.right_stride + j) * (size_t)H * W;
        const float sum = warp_overlap_sum<float>(L, R, W, sx, sy, x0, x1, y0, y1, lane);
        if (lane == 0) {
            float* dst = out + pair * OE + (size_t)oy * OW + ox;
            if (split != kSplitNone) atomicAdd(dst, sum); else *dst = sum;
        }
    }
}

// ------------------------------------------------------------------------------------------
// staged warp-per-overlap: the same warp-per-overlap sum, operands through shared memory
// ------------------------------------------------------------------------------------------
// Stands in for ccn_warp_per_shift_shared_mem (naive_warp_per_shift_shared_mem.cu:157-496,
// shared_mem.cuh:25-218).  A block owns one x shift, `shifts` consecutive y shifts (one per
// warp) and up to RMAX right matrices of one left matrix, so all its warps read the same
// columns: a slab of `srows` right rows x `scols` columns of every right matrix, and the
// srows + shifts - 1 left rows those y shifts meet them with, are copied to shared memory
// (4-byte cp.async: the left columns start at an arbitrary x shift) and every left value a
// lane loads is used for all the block's right matrices.  Two slabs are in flight: the copies
// of the next one run under the arithmetic of the current one.  Small inputs fit one slab,
// which makes this the latency kernel of the library: one wave of blocks, one copy, one sum.
__device__ __forceinline__ void stage_copy4(uint32_t dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst), "l"(src) : "memory");
}

template<int RMAX>
__global__ void __launch_bounds__(1024) warp_staged_kernel(const StagedArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int H = a.H, W = a.W, OW = 2 * W - 1, OH = 2 * H - 1;
    const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;
    const int k = a.shifts, srows = a.srows, scols = a.scols;

    // block -> (left matrix, group of right matrices, x shift), y shifts, column slab
    const unsigned bx = blockIdx.x;
    const int ox = (int)(bx % (unsigned)OW);
    const unsigned gl = bx / (unsigned)OW;
    const unsigned rg = gl % a.groups_per_left, l = gl / a.groups_per_left;
    const int nr = (int)min((unsigned)a.rights, a.pm.m - rg * (unsigned)a.rights);   // live right matrices
    const int sx = ox - (W - 1);
    const int oy0 = (int)blockIdx.y * k;
    const int sy_min = oy0 - (H - 1);
    const int sy_max = min(oy0 + k - 1, OH - 1) - (H - 1);
    const int sy_w = sy_min + warp;
    const bool warp_live = oy0 + warp < OH;
    int cx0 = max(0, -sx), cx1 = min(W, W - sx);               // right columns of the overlap
    if (a.col_groups) {
        cx0 += (int)blockIdx.z * scols;
        cx1 = min(cx1, cx0 + scols);
        if (cx0 >= cx1) return;                                 // the same for the whole block
    }
    const int ry0 = max(0, -sy_max), ry1 = min(H, H - sy_min);  // right rows any warp of the block needs
    const int wy0 = max(0, -sy_w), wy1 = min(H, H - sy_w);      // ... this warp needs

    const float* gL = a.left + (size_t)l * H * W;
    const float* gR = a.right + ((size_t)l * a.pm.right_stride + (size_t)rg * a.rights) * H * W;
    const int lrows = srows + k - 1;
    const int stage_floats = (lrows + a.rights * srows) * scols;
    const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);

    const int nslab_y = ry1 > ry0 ? (ry1 - ry0 + srows - 1) / srows : 0;
    const int nslab_x = (cx1 - cx0 + scols - 1) / scols;
    const int nslabs = nslab_y * nslab_x;

    // copies of slab i into stage s
    auto issue = [&](int i, int s) {
        const int ix = i / nslab_y, iy = i - ix * nslab_y;
        const int cs = cx0 + ix * scols, cw = min(scols, cx1 - cs);
        const int rb = ry0 + iy * srows, n = min(srows, ry1 - rb);
        const uint32_t sL = smem_addr + (uint32_t)(s * stage_floats) * 4;
        const uint32_t sR = sL + (uint32_t)(lrows * scols) * 4;
        // left rows rb + sy_min .. rb + n - 1 + sy_max, kept at their offset from rb + sy_min
        const int lr_lo = max(0, rb + sy_min), lr_hi = min(H, rb + n + sy_max);
        const int nl = max(0, lr_hi - lr_lo);
        const int total_rows = nl + nr * n;
        if (a.warp_rows) {
            for (int row = warp; row < total_rows; row += nthr >> 5) {
                const float* src;
                uint32_t dst;
                if (row < nl) {
                    src = gL + (size_t)(lr_lo + row) * W + cs + sx;
                    dst = sL + (uint32_t)((lr_lo + row - (rb + sy_min)) * scols) * 4;
                } else {
                    const int rr = row - nl, mm = rr / n, r = rr - mm * n;
                    src = gR + ((size_t)mm * H + rb + r) * W + cs;
                    dst = sR + (uint32_t)((mm * srows + r) * scols) * 4;
                }
                for (int c = lane; c < cw; c += 32) stage_copy4(dst + c * 4, src + c);
            }
        } else {
            const int total = total_rows * cw;
            for (int idx = tid; idx < total; idx += nthr) {
                const int row = idx / cw, c = idx - row * cw;
                if (row < nl) {
                    stage_copy4(sL + (uint32_t)((lr_lo + row - (rb + sy_min)) * scols + c) * 4,
                                gL + (size_t)(lr_lo + row) * W + cs + sx + c);
                } else {
                    const int rr = row - nl, mm = rr / n, r = rr - mm * n;
                    stage_copy4(sR + (uint32_t)((mm * srows + r) * scols + c) * 4,
                                gR + ((size_t)mm * H + rb + r) * W + cs + c);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float sum[RMAX];
#pragma unroll
    for (int i = 0; i < RMAX; ++i) sum[i] = 0.f;

    if (nslabs > 0) issue(0, 0);
    for (int i = 0; i < nslabs; ++i) {
        if (i + 1 < nslabs) {
            issue(i + 1, (i + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        {
            const int ix = i / nslab_y, iy = i - ix * nslab_y;
            const int cs = cx0 + ix * scols, cw = min(scols, cx1 - cs);
            const int rb = ry0 + iy * srows, n = min(srows, ry1 - rb);
            const float* sL = smem + (size_t)(i & 1) * stage_floats;
            const float* sR = sL + lrows * scols;
            // lanes: LC columns x 32 / LC rows of the slab per step
            int lc = 32;
            while (lc > 1 && (lc >> 1) >= cw) lc >>= 1;
            const int lrn = 32 / lc;
            const int c0 = lane & (lc - 1), r_off = lane / lc;
            const int ra = max(wy0, rb), rbnd = min(wy1, rb + n);
            if (warp_live) {
                for (int r = ra + r_off; r < rbnd; r += lrn) {
                    const float* lrow = sL + (r - rb + warp) * scols;   // left row r + sy_w
                    const float* rrow = sR + (r - rb) * scols;
                    for (int c = c0; c < cw; c += lc) {
                        const float lv = lrow[c];
#pragma unroll
                        for (int m2 = 0; m2 < RMAX; ++m2)
                            if (m2 < nr) sum[m2] = fmaf(lv, rrow[m2 * srows * scols + c], sum[m2]);
                    }
                }
            }
        }
        __syncthreads();                                   // the stage is refilled two slabs on
    }

    if (!warp_live) return;
#pragma unroll
    for (int m2 = 0; m2 < RMAX; ++m2) {
        float v = sum[m2];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
        if (lane == 0 && m2 < nr) {
            float* dst = a.out + (((size_t)l * a.pm.m + (size_t)rg * a.rights + m2) * OH + (oy0 + warp)) * OW + ox;
            if (a.col_groups) atomicAdd(dst, v); else *dst = v;
        }
    }
}

// ------------------------------------------------------------------------------------------
// FFMA peak probe: 16 independent chains per thread, registers only
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) ffma_probe_kernel(float* sink, float b, float c, int iters) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (float)(threadIdx.x + i) * 1e-3f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int rep = 0; rep < 8; ++rep)
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = fmaf(v[i], b, c);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s += v[i];
    if (s == 123.456f) sink[0] = s;   // never true in practice; keeps the chains alive
}

// ------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------
// Kernels that need more than 48 KB of dynamic shared memory have the limit raised once per
// (kernel instance, device); `raised` remembers the largest size granted so far.
constexpr int kAttrDevices = 64;
template<typename K>
static cudaError_t allow_smem(K kernel, std::atomic<size_t>* raised, int device, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    if (device >= 0 && device < kAttrDevices && raised[device].load(std::memory_order_relaxed) >= bytes) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && device >= 0 && device < kAttrDevices) raised[device].store(bytes, std::memory_order_relaxed);
    return e;
}

template<int TY, int BOUND, int VARIANT>
static cudaError_t launch_tile_instance(const TileArgs& a, int device, cudaStream_t stream) {
    static std::atomic<size_t> raised[kAttrDevices];
    cudaError_t e = allow_smem(tile_kernel<TY, BOUND, VARIANT>, raised, device, a.p.smem_bytes);
    if (e != cudaSuccess) return e;
    tile_kernel<TY, BOUND, VARIANT><<<a.p.grid, a.p.threads, a.p.smem_bytes, stream>>>(a);
    return cudaGetLastError();
}

template<int TY, int BOUND>
static cudaError_t launch_tile_variant(const TileArgs& a, int device, cudaStream_t stream) {
    if (a.p.schedule == kSchedWarpQueue) return launch_tile_instance<TY, BOUND, kBuildQueue>(a, device, stream);
    return a.p.combine == kFixup ? launch_tile_instance<TY, BOUND, kBuildFixup>(a, device, stream)
                                 : launch_tile_instance<TY, BOUND, kBuildPlain>(a, device, stream);
}

template<int TY>
static cudaError_t launch_tile_ty(const TileArgs& a, int device, cudaStream_t stream) {
    return a.p.threads <= kSmallBlockThreads ? launch_tile_variant<TY, kSmallBlockThreads>(a, device, stream)
                                             : launch_tile_variant<TY, kMaxWarps * 32>(a, device, stream);
}

cudaError_t launch_tile(const TileArgs& a, int device, cudaStream_t stream) {
    switch (a.p.TY) {
    case 1: return launch_tile_ty<1>(a, device, stream);
    case 2: return launch_tile_ty<2>(a, device, stream);
    case 3: return launch_tile_ty<3>(a, device, stream);
    case 4: return launch_tile_ty<4>(a, device, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_reduce_partials(const float* ws, float* out, unsigned long long total_out,
                                   int H, int W, int Hp, int S, int sm_count, cudaStream_t stream) {
    const unsigned long long rows_total = total_out / (2ull * W - 1);
    unsigned long long blocks = rows_total;
    const unsigned long long cap = (unsigned long long)sm_count * 32;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    const int threads = 2 * W - 1 >= 256 ? 256 : 2 * W - 1 >= 128 ? 128 : 64;
    reduce_partials_kernel<<<(unsigned)blocks, threads, 0, stream>>>(ws, out, total_out, H, W, Hp, S);
    return cudaGetLastError();
}

cudaError_t launch_overlap_wise(const float* left, const float* right, float* out, int H, int W,
                                PairMap pm, unsigned long long npairs, int block_threads,
                                dim3* grid_out, dim3* block_out, cudaStream_t stream) {
    int bx = 32, by = block_threads / 32;
    if (by < 1) by = 1;
    dim3 block(bx, by);
    const int OW = 2 * W - 1, OH = 2 * H - 1;
    dim3 grid((OW + bx - 1) / bx, (OH + by - 1) / by,
              (unsigned)(npairs < 65535ull ? npairs : 65535ull));
    overlap_wise_kernel<<<grid, block, 0, stream>>>(left, right, out, H, W, pm, npairs);
    *grid_out = grid;
    *block_out = block;
    return cudaGetLastError();
}

cudaError_t launch_warp_per_overlap(const float* left, const float* right, float* out, int H, int W,
                                    PairMap pm, unsigned long long npairs, int block_threads,
                                    int rows_per_warp, int split, int sm_count, dim3* grid_out, dim3* block_out,
                                    cudaStream_t stream) {
    const unsigned long long OW = 2ull * W - 1, OH = 2ull * H - 1;
    unsigned long long per_matrix = OW * OH;
    if (split == kSplitRectangle) {
        per_matrix *= (unsigned long long)((H + rows_per_warp - 1) / rows_per_warp);
    } else if (split == kSplitTriangle) {
        // sum over the output rows of ceil(overlapping rows / rows_per_warp)
        unsigned long long workers = 0;
        for (int y = 0; y < 2 * H - 1; ++y) {
            const int n = y < H ? y + 1 : 2 * H - 1 - y;
            workers += (unsigned long long)((n + rows_per_warp - 1) / rows_per_warp);
        }
        per_matrix = workers * OW;
    }
    const unsigned long long ntasks = per_matrix * npairs;
    const int wpb = block_threads / 32 > 0 ? block_threads / 32 : 1;
    unsigned long long blocks = (ntasks + wpb - 1) / wpb;
    const unsigned long long cap = (unsigned long long)sm_count * 64;
    if (blocks > cap) blocks = cap;
    dim3 grid((unsigned)blocks), block(wpb * 32);
    if (split == kSplitNone && ntasks < (1ull << 31) && npairs * pm.right_stride < (1ull << 31))
        warp_per_overlap_direct_kernel<float><<<grid, block, 0, stream>>>(left, right, out, H, W, pm, (unsigned)ntasks);
    else
        warp_per_overlap_kernel<<<grid, block, 0, stream>>>(left, right, out, H, W, pm, ntasks, rows_per_warp, split);
    *grid_out = grid;
    *block_out = block;
    return cudaGetLastError();
}

cudaError_t launch_warp_per_overlap_f64(const double* left, const double* right, double* out, int H, int W,
                                        PairMap pm, unsigned long long npairs, int block_threads, dim3* grid_out,
                                        cudaStream_t stream) {
    const unsigned long long ntasks = (2ull * W - 1) * (2ull * H - 1) * npairs;
    if (ntasks >= (1ull << 31)) return cudaErrorInvalidValue;
    const int wpb = block_threads / 32 > 0 ? block_threads / 32 : 1;
    dim3 grid((unsigned)((ntasks + wpb - 1) / wpb)), block(wpb * 32);
    warp_per_overlap_direct_kernel<double><<<grid, block, 0, stream>>>(left, right, out, H, W, pm, (unsigned)ntasks);
    *grid_out = grid;
    return cudaGetLastError();
}

size_t staged_smem_bytes(const StagedArgs& a) {
    return 2ull * (size_t)(a.srows + a.shifts - 1 + a.rights * a.srows) * a.scols * sizeof(float);
}

template<int RMAX>
static cudaError_t launch_staged_instance(const StagedArgs& a, dim3 grid, size_t smem, int device, cudaStream_t stream) {
    static std::atomic<size_t> raised[kAttrDevices];
    cudaError_t e = allow_smem(warp_staged_kernel<RMAX>, raised, device, smem);
    if (e != cudaSuccess) return e;
    warp_staged_kernel<RMAX><<<grid, a.shifts * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_warp_staged(const StagedArgs& a, int device, dim3* grid_out, size_t* smem_out, cudaStream_t stream) {
    const int OW = 2 * a.W - 1, OH = 2 * a.H - 1;
    dim3 grid((unsigned)((unsigned long long)a.pm.n_left * a.groups_per_left * OW), (unsigned)((OH + a.shifts - 1) / a.shifts),
              a.col_groups ? (unsigned)((a.W + a.scols - 1) / a.scols) : 1u);
    const size_t smem = staged_smem_bytes(a);
    *grid_out = grid;
    *smem_out = smem;
    if (a.rights <= 1) return launch_staged_instance<1>(a, grid, smem, device, stream);
    if (a.rights <= 2) return launch_staged_instance<2>(a, grid, smem, device, stream);
    if (a.rights <= 4) return launch_staged_instance<4>(a, grid, smem, device, stream);
    return launch_staged_instance<8>(a, grid, smem, device, stream);
}

// ------------------------------------------------------------------------------------------
// scratch for callers that cannot allocate
// ------------------------------------------------------------------------------------------
// Partial images of xcorr_one_to_one_noalloc_f32: S * (2*rows-1) * (2*cols-1) floats, written
// by tile_kernel and summed by reduce_partials_kernel.  A file-scope device array: it exists
// on every GPU that loads this library, from load until the process exits, and is shared by
// all calls (calls that overlap on one GPU would race on it).
constexpr size_t kNoAllocScratchFloats = (size_t)8 << 20;            // 32 MiB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

cudaError_t tile_stage_timeouts(unsigned* count) {
    cudaError_t e = cudaMemcpyFromSymbol(count, g_stage_timeouts, sizeof(unsigned));
    if (e != cudaSuccess || *count == 0) return e;
    const unsigned zero = 0;                     // reported once: the next check starts from zero
    return cudaMemcpyToSymbol(g_stage_timeouts, &zero, sizeof(unsigned));
}

size_t noalloc_scratch_bytes() { return kNoAllocScratchFloats * sizeof(float); }

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address
// a kernel could be given: the address is asked for once per device, with that device
// current, and cached.
constexpr int kScratchDevices = 64;
static std::mutex g_scratch_mutex;
static float* g_scratch_address[kScratchDevices] = {};

cudaError_t noalloc_scratch_address(float** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kScratchDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_address[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_address[dev] = static_cast<float*>(p);
    }
    *ptr = g_scratch_address[dev];
    return cudaSuccess;
}

// The addresses belong to the contexts they were asked in: after the application has reset a
// device or destroyed its primary context they are stale and must be looked up again.
void noalloc_forget_addresses() {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    for (float*& p : g_scratch_address) p = nullptr;
}

cudaError_t launch_ffma_probe(float* sink, int iters, int blocks, cudaStream_t stream) {
    ffma_probe_kernel<<<blocks, 1024, 0, stream>>>(sink, 0.999f, 1e-3f, iters);
    return cudaGetLastError();
}

}  // namespace xcorr
