// Host-side (CPU) cross-correlation and result statistics of the `cross` program: what the
// registry's cpu_* algorithms run and what `run --validate` / `cross validate` compare with.
// Same definition, loop order and float accumulation as the reference's CPU path
// (repo/cross-corr/src/validate.hpp:94-132) and its error statistics (:134-188).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <iomanip>
#include <limits>
#include <ostream>
#include <sstream>
#include <string>

namespace cross {

// One pair, all shifts: out[(sy+H-1)*(2W-1) + (sx+W-1)] = sum left[y+sy][x+sx]*right[y][x].
template<typename T, typename IN = float>
void cpu_cross_corr_pair(const IN* left, const IN* right, T* out, int H, int W) {
    const int OW = 2 * W - 1;
    for (int sy = -(H - 1); sy <= H - 1; ++sy) {
        const int y0 = std::max(sy, 0), y1 = std::min(H + sy, H);
        for (int sx = -(W - 1); sx <= W - 1; ++sx) {
            const int x0 = std::max(sx, 0), x1 = std::min(W + sx, W);
            T sum = T{};
            for (int yl = y0; yl < y1; ++yl) {
                const IN* lrow = left + static_cast<std::size_t>(yl) * W;
                const IN* rrow = right + static_cast<std::size_t>(yl - sy) * W - sx;
                for (int xl = x0; xl < x1; ++xl) sum += static_cast<T>(rrow[xl]) * static_cast<T>(lrow[xl]);
            }
            out[static_cast<std::size_t>(sy + H - 1) * OW + (sx + W - 1)] = sum;
        }
    }
}

struct validation_results {
    bool empty = true;
    double diff_max = 0, diff_mean = 0, diff_std_dev = 0, value_result = 0, value_valid = 0;

    static std::string csv_header() { return "Max,Mean,Stddev"; }
    std::string csv_data() const {
        std::stringstream ss;
        ss << std::scientific << diff_max << "," << diff_mean << "," << diff_std_dev;
        return ss.str();
    }
};

inline std::ostream& operator<<(std::ostream& out, const validation_results& r) {
    if (r.empty) {
        out << "No validation\n";
    } else {
        out << "Difference from valid values:\n";
        out << "Max: " << r.diff_max << " (" << std::fixed << r.value_result << " instead of " << r.value_valid << ")\n";
        out.unsetf(std::ios_base::fixed);
        out << std::scientific;
        out << "Mean: " << r.diff_mean << "\n";
        out << "Stddev: " << r.diff_std_dev << "\n";
        out.unsetf(std::ios_base::scientific);
    }
    return out;
}

// validate.hpp:134-188: element error |a-b| / max(|a|,|b|), 0 when both are <= 1e-5, in
// the value type T of the compared arrays; max, mean, population standard deviation.
template<typename T>
validation_results validate_result(const T* result, const T* valid, std::size_t n) {
    validation_results r;
    if (n == 0) return r;
    double mx = 0, s1 = 0, s2 = 0;
    std::size_t imax = 0;
    bool have = false;
    for (std::size_t i = 0; i < n; ++i) {
        const T a = result[i], b = valid[i];
        const T eps = static_cast<T>(1e-5);
        double d;
        if (std::abs(a) <= eps && std::abs(b) <= eps) d = 0.0;
        else d = static_cast<double>(std::abs(a - b) / std::max(std::abs(a), std::abs(b)));
        if (!have || d > mx) { mx = d; imax = i; have = true; }
        s1 += d;
        s2 += d * d;
    }
    r.empty = false;
    r.diff_max = mx;
    r.diff_mean = s1 / static_cast<double>(n);
    const double var = s2 / static_cast<double>(n) - r.diff_mean * r.diff_mean;
    r.diff_std_dev = std::sqrt(std::max(var, 0.0));
    r.value_result = static_cast<double>(result[imax]);
    r.value_valid = static_cast<double>(valid[imax]);
    return r;
}

}  // namespace cross
