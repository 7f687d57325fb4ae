// C entry points around the REFERENCE's own CPU cross-correlation code.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit includes the reference's
// repo/cross-corr/src/validate.hpp (and through it matrix.hpp, types.cuh) from where the
// reference checkout lies -- no reference source is copied into this repository -- and
// exposes the templates instantiated for float and double through a plain C interface so
// that the tests and the benchmark's CPU-baseline leg can call the unmodified reference
// arithmetic.  Built by oracle/Makefile into oracle/_ref/libxcorr_ref.so.
//
// data_array's storage is private and only fillable through its CSV loader, so inputs are
// copied element-wise through begin()/end() (public iterators).
#include <cstdint>
#include <cstring>
#include <exception>
#include <filesystem>
#include <tuple>
#include <functional>

#include <cmath>
#include <cstdlib>
// The reference is built with nvcc (every source is compiled as CUDA), whose headers put
// the float and double overloads of abs() into the global namespace; validate.hpp calls
// abs() unqualified.  Bring the same overloads into scope for a plain g++ build.
using std::abs;

#include "validate.hpp"

using namespace cross;

namespace {

template<typename T>
data_array<T> make_array(const float* src, uint32_t rows, uint32_t cols, uint32_t n) {
    data_array<T> a{dsize2_t{cols, rows}, n};
    T* dst = a.data();
    const std::size_t total = static_cast<std::size_t>(rows) * cols * n;
    for (std::size_t i = 0; i < total; ++i) dst[i] = static_cast<T>(src[i]);
    return a;
}

template<typename T>
void copy_out(const data_array<T>& res, T* out) {
    std::memcpy(out, res.data(), sizeof(T) * res.size());
}

enum mode_t { ONE_TO_ONE = 0, ONE_TO_MANY = 1, N_TO_MN = 2, N_TO_M = 3 };

template<typename T>
int run_mode(int mode, const float* left, const float* right, T* out,
             uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right) {
    try {
        auto ref = make_array<T>(left, rows, cols, n_left);
        auto target = make_array<T>(right, rows, cols, n_right);
        dsize2_t res_size = result_matrix_size(ref.matrix_size(), target.matrix_size());
        switch (mode) {
        case ONE_TO_ONE: {
            data_array<T> res{res_size, 1};
            cpu_cross_corr_one_to_one(ref, target, res);
            copy_out(res, out);
            return 0;
        }
        case ONE_TO_MANY: {
            data_array<T> res{res_size, n_right};
            cpu_cross_corr_one_to_many(ref, target, res);
            copy_out(res, out);
            return 0;
        }
        case N_TO_MN: {
            // The 3-argument form; the value-returning form allocates n results instead
            // of n*m and throws for m > 1.
            data_array<T> res{res_size, n_right};
            cpu_cross_corr_n_to_mn(ref, target, res);
            copy_out(res, out);
            return 0;
        }
        case N_TO_M: {
            data_array<T> res{res_size, n_left * n_right};
            cpu_cross_corr_n_to_m(ref, target, res);
            copy_out(res, out);
            return 0;
        }
        default:
            return 1;
        }
    } catch (std::exception&) {
        return 2;
    }
}

}

extern "C" {

// mode: 0 one_to_one, 1 one_to_many, 2 n_to_mn (file order), 3 n_to_m.
__attribute__((visibility("default")))
int ref_cpu_cross_corr_f32(int mode, const float* left, const float* right, float* out,
                           uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right) {
    return run_mode<float>(mode, left, right, out, rows, cols, n_left, n_right);
}

__attribute__((visibility("default")))
int ref_cpu_cross_corr_f64(int mode, const float* left, const float* right, double* out,
                           uint32_t rows, uint32_t cols, uint32_t n_left, uint32_t n_right) {
    return run_mode<double>(mode, left, right, out, rows, cols, n_left, n_right);
}

// validate_result on double arrays of n values laid out as one 1 x n matrix.
// elem_f32 != 0 evaluates the element error in float, as `cross run --validate` does.
__attribute__((visibility("default")))
int ref_validate_result(const double* result, const double* valid, uint32_t n, int elem_f32,
                        double stats[5]) {
    try {
        validation_results r;
        if (elem_f32) {
            data_array<float> a{dsize2_t{n, 1}, 1}, b{dsize2_t{n, 1}, 1};
            for (uint32_t i = 0; i < n; ++i) {
                a.data()[i] = static_cast<float>(result[i]);
                b.data()[i] = static_cast<float>(valid[i]);
            }
            r = validate_result(a, b);
        } else {
            data_array<double> a{dsize2_t{n, 1}, 1}, b{dsize2_t{n, 1}, 1};
            std::memcpy(a.data(), result, sizeof(double) * n);
            std::memcpy(b.data(), valid, sizeof(double) * n);
            r = validate_result(a, b);
        }
        stats[0] = r.get_diff_max();
        stats[1] = r.get_diff_mean();
        stats[2] = r.get_diff_std_dev();
        stats[3] = r.get_max_valid();
        stats[4] = r.get_max_actual();
        return 0;
    } catch (std::exception&) {
        return 2;
    }
}

}
