// Algorithm registry and the per-run algorithm object of the `cross` program.
//
// The reference registers one C++ class per (algorithm, input mode) under a string name
// (repo/cross-corr/src/main.cpp:361-411); every class reads its tuning values from the JSON
// arguments with defaults, echoes them as extra columns of the timing CSV
// (additional_properties(), e.g. one_to_one.hpp:744-750) and implements
// load / prepare / transfer / run / finalize / free / store / validate
// (cross_corr.hpp:21-189).  Here one data-driven class does that for every name: the table
// below keeps each name, its mode, its JSON keys with the reference's defaults in the
// reference's column order, and says which kernel family of the CUDA library serves it.
// The arithmetic goes through the C ABI of include/xcorr.h; nothing else touches the GPU.
#pragma once
#include <cuda_runtime.h>

#include <chrono>
#include <filesystem>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "cpu_xcorr.hpp"
#include "json_min.hpp"
#include "matrix_array.hpp"
#include "stopwatch.hpp"
#include "xcorr.h"

namespace cross {

enum class benchmark_type { Unknown, None, Compute, CommonSteps, Algorithm };

benchmark_type parse_benchmark_type(const std::string& token);
const char* to_string(benchmark_type t);

// Thrown for bad algorithm arguments: exit code 1 (argument_error.hpp, main.cpp:675-678).
class argument_error : public std::runtime_error {
public:
    argument_error(const std::string& msg, const std::string& arg) : std::runtime_error(msg), arg_(arg) {}
    const std::string& arg() const { return arg_; }
private:
    std::string arg_;
};

enum class family { cpu, overlap_wise, warp_per_overlap, warp_staged, tile, fft };

struct arg_spec {
    enum class kind { integer, boolean, text };
    std::string key;
    kind type;
    long default_int;        // integer / boolean default
    std::string default_text;
    std::string default_from;  // integer whose default is another key's value (shared_mem_rows)
};

struct algorithm_spec {
    std::string name;
    int mode;                 // xcorr_mode
    family fam;
    std::vector<arg_spec> args;
    bool split_rows;          // the reference's "work distribution" variants: rows_per_thread -> row slices
};

const std::vector<algorithm_spec>& algorithm_registry();
const algorithm_spec* find_algorithm(const std::string& name);
matrix_array normalize_fft_results(const matrix_array& raw);
std::vector<std::string> sorted_algorithm_names(bool include_unavailable);

using string_pairs = std::vector<std::pair<std::string, std::string>>;

class algorithm {
public:
    algorithm(const algorithm_spec& spec, const json_object& args, double min_time_ns, benchmark_type bench,
              std::vector<int> devices);
    ~algorithm();
    algorithm(const algorithm&) = delete;
    algorithm& operator=(const algorithm&) = delete;

    // The computation steps of cross_corr.hpp:32-72; in CommonSteps mode each is wall-clock timed.
    void load(const std::filesystem::path& ref_path, const std::filesystem::path& target_path);
    void prepare();
    void transfer();
    void run();
    void finalize();
    void free();
    void store_results(const std::filesystem::path& out_path);

    validation_results validate(const std::optional<std::filesystem::path>& valid_path) const;
    // `cross run --normalize`: FFT algorithms deliver the direct path's result layout instead of
    // the raw inverse transforms (main.cpp:178-186); no effect on the other families.
    void set_normalize(bool on) { normalize_ = on; }
    // `cross run --pipelined` (or XCORR_PIPELINED=1): the transfer / run / finalize steps become one
    // call of the host-buffer entry point, which overlaps the copies of successive pieces of
    // the result with the kernels; prepare and free then have nothing to do on the device.
    // Not used in Algorithm mode (which times kernels alone) nor for raw FFT results.
    void set_pipelined(bool on) { pipelined_ = on; }

    std::vector<std::string> measurement_labels() const;
    std::vector<measurement_result> measurements() const { return measurements_; }
    void reset_measurements();
    string_pairs additional_properties() const { return properties_; }
    benchmark_type bench() const { return bench_; }
    const algorithm_spec& spec() const { return spec_; }

private:
    struct shard {
        int device = 0;
        cudaStream_t stream = nullptr;
        cudaEvent_t start = nullptr, stop = nullptr;
        uint32_t n_left = 0, n_right = 0;          // counts handed to the library
        std::size_t left_offset = 0, right_offset = 0, out_offset = 0;  // in floats, into the host arrays
        std::size_t left_elems = 0, right_elems = 0, out_elems = 0;
        float* d_left = nullptr;
        float* d_right = nullptr;
        float* d_out = nullptr;
        void* d_ws = nullptr;
        std::size_t ws_bytes = 0;
    };

    const algorithm_spec& spec_;
    double min_time_ns_;
    benchmark_type bench_;
    std::vector<int> devices_;
    xcorr_hints hints_{};
    string_pairs properties_;
    matrix_array left_, right_, result_;
    std::vector<shard> shards_;
    std::vector<measurement_result> measurements_;
    long rows_per_thread_ = 0;       // explicit JSON value, 0 = not given
    bool normalize_ = false;
    bool pipelined_ = false;
    bool pipelined() const { return pipelined_ && on_gpu() && !measure_alg() && !raw_fft(); }

    bool raw_fft() const { return spec_.fam == family::fft && !normalize_; }
    validation_results validate_against(const matrix_array& result,
                                        const std::optional<std::filesystem::path>& valid_path) const;

    bool measure_common() const { return bench_ == benchmark_type::CommonSteps; }
    bool measure_alg() const { return bench_ == benchmark_type::Algorithm; }
    bool on_gpu() const { return spec_.fam != family::cpu; }
    uint32_t rights_per_left() const;
    void build_shards();
    void launch_all();
    void run_cpu();
    template<typename F> void timed_step(std::size_t label, bool sync_gpu, F&& step);
    void sync_all_devices();
};

}  // namespace cross
