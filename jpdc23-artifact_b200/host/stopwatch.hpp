// Adaptive timing: repeat a block until the measured span reaches --min_time, as the
// reference's CUDA_ADAPTIVE_MEASURE / CPU_ADAPTIVE_MEASURE do (stopwatch.hpp:125-141,
// :179-200), and report total / iterations in nanoseconds.
#pragma once
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstddef>
#include <stdexcept>

namespace cross {

struct measurement_result {
    double total_ns = 0.0;
    std::size_t iterations = 0;

    // stopwatch.hpp:26-35: integer nanoseconds per iteration, 0 when nothing was measured.
    long long iteration_ns() const {
        if (total_ns == 0.0) return 0;
        if (iterations == 0) throw std::runtime_error("Zero iterations with non-zero total time");
        return static_cast<long long>(total_ns) / static_cast<long long>(iterations);
    }
};

// stopwatch.hpp:57-71: 0 when the span is long enough, else the iteration count scaled by
// 1.5 x the shortfall, growing by at least 1.5x and at most 100x per round.
inline std::size_t next_iteration_count(double min_time_ns, const measurement_result& res) {
    if (res.total_ns >= min_time_ns) return 0;
    const double ratio = min_time_ns / std::max(res.total_ns, 1.0);
    const double next = std::ceil(static_cast<double>(res.iterations) * std::max(std::min(ratio * 1.5, 100.0), 1.5));
    return static_cast<std::size_t>(next);
}

using wall_clock = std::chrono::high_resolution_clock;

inline double elapsed_ns(wall_clock::time_point start) {
    return std::chrono::duration<double, std::nano>(wall_clock::now() - start).count();
}

}  // namespace cross
