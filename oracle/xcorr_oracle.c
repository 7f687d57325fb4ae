/*
 * xcorr_oracle.c -- CPU restatement of the reference's definition-based full 2-D
 * cross-correlation.  TEST INFRASTRUCTURE ONLY: this file is the checker for the CUDA
 * library and the timed CPU baseline of the benchmark.  Nothing in the shipped library
 * or in the `cross` host program links, loads or calls it.
 *
 * Parity status: PINNED.  The functions below are checked bit-for-bit (float path) and
 * to 1 ulp-free equality (double path) against the reference's own CPU code
 * (repo/cross-corr/src/validate.hpp compiled unmodified into oracle/_ref/libxcorr_ref.so)
 * and against fixtures that library produced (tests/golden/, made by
 * tests/golden/make_golden.py).  The reference ships no golden vectors of its own.
 *
 * Each function names the reference lines it follows (paths inside the reference
 * project: repo/cross-corr/src/...).
 *
 * Conventions (validate.hpp:95-132): `left` is the reference's "ref", `right` its
 * "target".  For a shift (sx, sy), sx in [-(W-1), W-1], sy in [-(H-1), H-1]:
 *     out[sy + H-1][sx + W-1] = sum over the overlap of left[y+sy][x+sx] * right[y][x]
 * Output is (2H-1) x (2W-1), row-major.  All matrices are row-major float32 and
 * stacked contiguously.
 */
#include <stddef.h>
#include <stdint.h>
#include <math.h>
#include <stdlib.h>

#if defined(__GNUC__)
#define ORACLE_API __attribute__((visibility("default")))
#else
#define ORACLE_API
#endif

/* ---- one shift ------------------------------------------------------------------
 * validate.hpp:94-114 (hadamard_and_sum): iterate the part of `left` that overlaps the
 * shifted `right`, rows outer, columns inner, accumulate sequentially in T. */
static float shift_sum_f32(const float* left, const float* right, int rows, int cols,
                           int sx, int sy) {
    int x0 = sx > 0 ? sx : 0;
    int x1 = cols + sx < cols ? cols + sx : cols;
    int y0 = sy > 0 ? sy : 0;
    int y1 = rows + sy < rows ? rows + sy : rows;
    float sum = 0.0f;
    for (int yl = y0; yl < y1; ++yl) {
        for (int xl = x0; xl < x1; ++xl) {
            /* validate.hpp:110 -- product order target * ref, then += */
            sum += right[(size_t)(yl - sy) * cols + (xl - sx)] * left[(size_t)yl * cols + xl];
        }
    }
    return sum;
}

static double shift_sum_f64(const float* left, const float* right, int rows, int cols,
                            int sx, int sy) {
    int x0 = sx > 0 ? sx : 0;
    int x1 = cols + sx < cols ? cols + sx : cols;
    int y0 = sy > 0 ? sy : 0;
    int y1 = rows + sy < rows ? rows + sy : rows;
    double sum = 0.0;
    for (int yl = y0; yl < y1; ++yl) {
        for (int xl = x0; xl < x1; ++xl) {
            sum += (double)right[(size_t)(yl - sy) * cols + (xl - sx)] *
                   (double)left[(size_t)yl * cols + xl];
        }
    }
    return sum;
}

/* ---- one pair -------------------------------------------------------------------
 * validate.hpp:117-132 (naive_cpu_cross_corr): all shifts, y outer, x inner; result
 * index (x + half.x, y + half.y) with half = (search_size - 1) / 2 = (W-1, H-1). */
ORACLE_API void oracle_xcorr_pair_f32(const float* left, const float* right, float* out,
                                      uint32_t rows, uint32_t cols) {
    int H = (int)rows, W = (int)cols;
    int ow = 2 * W - 1;
    for (int sy = -(H - 1); sy <= H - 1; ++sy)
        for (int sx = -(W - 1); sx <= W - 1; ++sx)
            out[(size_t)(sy + H - 1) * ow + (sx + W - 1)] = shift_sum_f32(left, right, H, W, sx, sy);
}

/* Same loops with the accumulator (and the products) in double: the reference template
 * instantiated with T = double on float32-representable inputs. */
ORACLE_API void oracle_xcorr_pair_f64(const float* left, const float* right, double* out,
                                      uint32_t rows, uint32_t cols) {
    int H = (int)rows, W = (int)cols;
    int ow = 2 * W - 1;
    for (int sy = -(H - 1); sy <= H - 1; ++sy)
        for (int sx = -(W - 1); sx <= W - 1; ++sx)
            out[(size_t)(sy + H - 1) * ow + (sx + W - 1)] = shift_sum_f64(left, right, H, W, sx, sy);
}

static size_t in_elems(uint32_t rows, uint32_t cols) { return (size_t)rows * cols; }
static size_t out_elems(uint32_t rows, uint32_t cols) {
    return (size_t)(2 * rows - 1) * (2 * cols - 1);
}

/* ---- modes ----------------------------------------------------------------------
 * Every mode function takes [first, last) over its natural unit of independent work so
 * that a caller may split the units over host threads; first = 0, last = unit count is
 * the reference's single-threaded loop.  `acc64` selects the double instantiation:
 * out is then double*, else float*. */

/* validate.hpp:214-220: one pair. */
ORACLE_API int oracle_one_to_one(const float* left, const float* right, void* out,
                                 uint32_t rows, uint32_t cols, int acc64) {
    if (!left || !right || !out || rows == 0 || cols == 0) return 1;
    if (acc64) oracle_xcorr_pair_f64(left, right, (double*)out, rows, cols);
    else       oracle_xcorr_pair_f32(left, right, (float*)out, rows, cols);
    return 0;
}

/* validate.hpp:230-239: result i = left[0] x right[i].  Units: right matrices. */
ORACLE_API int oracle_one_to_many(const float* left, const float* right, void* out,
                                  uint32_t rows, uint32_t cols, uint32_t n_right,
                                  uint32_t first, uint32_t last, int acc64) {
    if (!left || !right || !out || rows == 0 || cols == 0 || last > n_right) return 1;
    size_t ie = in_elems(rows, cols), oe = out_elems(rows, cols);
    for (uint32_t i = first; i < last; ++i) {
        if (acc64) oracle_xcorr_pair_f64(left, right + i * ie, (double*)out + i * oe, rows, cols);
        else       oracle_xcorr_pair_f32(left, right + i * ie, (float*)out + i * oe, rows, cols);
    }
    return 0;
}

/* validate.hpp:249-270: FILE order.  n_right = m * n_left; right / result matrix
 * t * n_left + r pairs with left r.  Units: right (= result) matrices in file order. */
ORACLE_API int oracle_n_to_mn(const float* left, const float* right, void* out,
                              uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                              uint32_t first, uint32_t last, int acc64) {
    if (!left || !right || !out || rows == 0 || cols == 0 || n_left == 0) return 1;
    if (n_right % n_left != 0) return 2; /* validate.hpp:254-261 throws */
    if (last > n_right) return 1;
    size_t ie = in_elems(rows, cols), oe = out_elems(rows, cols);
    for (uint32_t i = first; i < last; ++i) {
        uint32_t r = i % n_left; /* i = t * n_left + r */
        if (acc64) oracle_xcorr_pair_f64(left + r * ie, right + i * ie, (double*)out + i * oe, rows, cols);
        else       oracle_xcorr_pair_f32(left + r * ie, right + i * ie, (float*)out + i * oe, rows, cols);
    }
    return 0;
}

/* validate.hpp:279-291: result r * n_right + t = left[r] x right[t].  Units: results. */
ORACLE_API int oracle_n_to_m(const float* left, const float* right, void* out,
                             uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right,
                             uint32_t first, uint32_t last, int acc64) {
    if (!left || !right || !out || rows == 0 || cols == 0) return 1;
    if ((uint64_t)last > (uint64_t)n_left * n_right) return 1;
    size_t ie = in_elems(rows, cols), oe = out_elems(rows, cols);
    for (uint32_t i = first; i < last; ++i) {
        uint32_t r = i / n_right, t = i % n_right;
        if (acc64) oracle_xcorr_pair_f64(left + r * ie, right + t * ie, (double*)out + i * oe, rows, cols);
        else       oracle_xcorr_pair_f32(left + r * ie, right + t * ie, (float*)out + i * oe, rows, cols);
    }
    return 0;
}

/* ---- n_to_mn memory order ---------------------------------------------------------
 * matrix.hpp:614-618 (get_interleaved_index): file index i of `count` matrices in
 * groups of `group_size` goes to memory slot (i % group_size) * (count / group_size)
 * + i / group_size.  With group_size = n_left this turns file order t*n+r into the
 * grouped order r*m+t used by the GPU algorithms (matrix.hpp:484-503). */
ORACLE_API uint32_t oracle_interleaved_index(uint32_t i, uint32_t group_size, uint32_t num_groups) {
    return (i % group_size) * num_groups + i / group_size;
}

/* ---- validation statistics ---------------------------------------------------------
 * validate.hpp:134-188 (validate_result): element-wise |a-b| / max(|a|,|b|), forced to 0
 * when both magnitudes are <= 1e-5; max, mean and population standard deviation
 * (boost variance(lazy) = E[x^2] - E[x]^2).  The reference evaluates the element error
 * in the result's value type (float for `run --validate`, double for `cross validate`);
 * `elem_f32` selects that.  stats = {max, mean, stddev, result-at-max, valid-at-max}. */
ORACLE_API int oracle_validate_result(const double* result, const double* valid, size_t n,
                                      int elem_f32, double stats[5]) {
    if (!result || !valid || !stats || n == 0) return 1;
    double mx = 0.0, s1 = 0.0, s2 = 0.0;
    size_t imax = 0;
    int have = 0;
    for (size_t i = 0; i < n; ++i) {
        double d;
        if (elem_f32) {
            float a = (float)result[i], b = (float)valid[i];
            float eps = 1e-5f;
            if (fabsf(a) <= eps && fabsf(b) <= eps) d = 0.0;
            else d = (double)(fabsf(a - b) / fmaxf(fabsf(a), fabsf(b)));
        } else {
            double a = result[i], b = valid[i];
            if (fabs(a) <= 1e-5 && fabs(b) <= 1e-5) d = 0.0;
            else d = fabs(a - b) / fmax(fabs(a), fabs(b));
        }
        if (!have || d > mx) { mx = d; imax = i; have = 1; }
        s1 += d;
        s2 += d * d;
    }
    double mean = s1 / (double)n;
    double var = s2 / (double)n - mean * mean;
    stats[0] = mx;
    stats[1] = mean;
    stats[2] = sqrt(var > 0.0 ? var : 0.0);
    stats[3] = result[imax];
    stats[4] = valid[imax];
    return 0;
}
