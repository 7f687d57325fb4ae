// `cross` -- command line front end, option for option the reference's
// (repo/cross-corr/src/main.cpp:465-683, run_args.cpp:87-150):
//
//   cross [-h] list
//   cross run [-d single] [-o out] [-t times] [-v [valid]] [-n] [-a] [-p]
//             [-b None|Compute|CommonSteps|Algorithm] [-l outer_loops] [-m min_time_s]
//             [--args_path json] [--devices N] [--pipelined] <alg> <ref_path> <target_path>
//   cross validate [-n] [-c] [-p] <template_data_path> <validate_data_path...>
//   cross input <alg_type> <rows> <columns> <left_matrices> <right_matrices>
//
// Exit codes: 0 ok; 1 bad options, unknown algorithm or bad algorithm argument (help is
// printed); 2 any other exception; 3 an exception inside a computation step.
// Additions: `--devices N` (or the environment variable XCORR_DEVICES) shards the independent
// result matrices of the many-matrix modes over the first N GPUs; `--pipelined` (or
// XCORR_PIPELINED=1) runs transfer, kernels and copy-back as one overlapped call.
#include <cuda_runtime.h>

#include <cstdlib>
#include <fstream>
#include <functional>
#include <iostream>
#include <map>
#include <optional>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "algorithms.hpp"

using namespace cross;

namespace {

struct option_error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// Option table entry: long name, short name, takes a value?, may the value be omitted?
struct option_def {
    const char* long_name;
    char short_name;
    bool has_value;
    bool value_optional;
};

struct parsed_args {
    std::map<std::string, std::string> values;   // option -> value ("" for switches / omitted values)
    std::vector<std::string> positional;
    bool has(const std::string& k) const { return values.count(k) != 0; }
};

// Options may come before, between or after the positional arguments, as with
// boost::program_options.  An option whose value may be omitted (--validate) takes the next
// token as its value unless that token starts with '-' or names an algorithm.
parsed_args parse_options(const std::vector<std::string>& tokens, const std::vector<option_def>& defs) {
    parsed_args out;
    auto find_long = [&](const std::string& n) -> const option_def* {
        for (const auto& d : defs) if (n == d.long_name) return &d;
        return nullptr;
    };
    auto find_short = [&](char c) -> const option_def* {
        for (const auto& d : defs) if (d.short_name && c == d.short_name) return &d;
        return nullptr;
    };
    for (std::size_t i = 0; i < tokens.size(); ++i) {
        const std::string& tok = tokens[i];
        const option_def* def = nullptr;
        std::optional<std::string> attached;
        if (tok.size() > 2 && tok[0] == '-' && tok[1] == '-') {
            std::string name = tok.substr(2);
            const auto eq = name.find('=');
            if (eq != std::string::npos) { attached = name.substr(eq + 1); name = name.substr(0, eq); }
            def = find_long(name);
            if (!def) throw option_error("unrecognised option '" + tok + "'");
        } else if (tok.size() >= 2 && tok[0] == '-' && !(std::isdigit(static_cast<unsigned char>(tok[1])) || tok[1] == '.')) {
            def = find_short(tok[1]);
            if (!def) throw option_error("unrecognised option '" + tok + "'");
            if (tok.size() > 2) attached = tok.substr(2);
        } else {
            out.positional.push_back(tok);
            continue;
        }
        std::string value;
        if (def->has_value) {
            if (attached) {
                value = *attached;
            } else if (def->value_optional) {
                if (i + 1 < tokens.size() && !tokens[i + 1].empty() && tokens[i + 1][0] != '-' &&
                    find_algorithm(tokens[i + 1]) == nullptr)
                    value = tokens[++i];
            } else {
                if (i + 1 >= tokens.size())
                    throw option_error(std::string("the required argument for option '--") + def->long_name + "' is missing");
                value = tokens[++i];
            }
        } else if (attached) {
            throw option_error(std::string("option '--") + def->long_name + "' does not take any arguments");
        }
        out.values[def->long_name] = value;
    }
    return out;
}

const std::vector<option_def> kRunOptions = {
    {"data_type", 'd', true, false}, {"out", 'o', true, false}, {"times", 't', true, false},
    {"validate", 'v', true, true}, {"normalize", 'n', false, false}, {"append", 'a', false, false},
    {"no_progress", 'p', false, false}, {"benchmark_type", 'b', true, false},
    {"outer_loops", 'l', true, false}, {"min_time", 'm', true, false}, {"args_path", 0, true, false},
    {"devices", 0, true, false}, {"pipelined", 0, false, false}, {"help", 'h', false, false},
};
const std::vector<option_def> kValidateOptions = {
    {"normalize", 'n', false, false}, {"csv", 'c', false, false}, {"print_header", 'p', false, false},
    {"help", 'h', false, false},
};
const std::vector<option_def> kInputOptions = {{"help", 'h', false, false}};

void print_help(std::ostream& out, const std::string& name) {
    out << "Usage: " << name << " [global options] command [command options]\n";
    out << "Commands: \n";
    out << "\t" << name << " [global options] list\n";
    out << "\t" << name << " [global options] run [run options] <alg> <ref_path> <target_path>\n";
    out << "\t" << name << " [global options] validate [validate options] <validate_data_path> <template_data_path>\n";
    out << "\t" << name << " [global options] input [input options] <alg_type> <rows> <columns> <left_matrices> <right_matrices>\n";
    out << "Global options:\n"
           "  -h [ --help ]                         display this help and exit\n"
           "Validate options:\n"
           "  -n [ --normalize ]                    Normalize the data to be validated as they are denormalized fft output\n"
           "  -c [ --csv ]                          CSV output\n"
           "  -p [ --print_header ]                 Print header\n"
           "Run options:\n"
           "  -d [ --data_type ] arg (=single)      Data type to use for computation\n"
           "  -o [ --out ] arg                      Path of the output file to be created\n"
           "  -t [ --times ] arg (=measurements.csv) File to store the measured times in\n"
           "  -v [ --validate ] [=arg(=)]           If validation of the results should be done and optionally path to a\n"
           "                                        file containing the valid results\n"
           "  -n [ --normalize ]                    If algorithm is fft, normalize the results\n"
           "  -a [ --append ]                       Append time measurements without the header if the times file already\n"
           "                                        exists instead of overwriting it\n"
           "  -p [ --no_progress ]                  Do not print human readable progress, instead any messages to stdout\n"
           "                                        will be formated for machine processing\n"
           "  -b [ --benchmark_type ] arg (=None)   Which part should be measured, available parts are Compute,\n"
           "                                        CommonSteps, Algorithm\n"
           "  -l [ --outer_loops ] arg (=1)         How many measurements of the computation loop should be done with the\n"
           "                                        loaded data\n"
           "  -m [ --min_time ] arg (=1)            The minimum time to consider measurement statistically relevant, in\n"
           "                                        seconds\n"
           "  --args_path arg                       Path to the JSON file containing arguments for the algorithm\n"
           "  --devices arg (=1)                    Number of GPUs to shard the many-matrix modes over\n"
           "  --pipelined                           Transfer, run and copy back as one overlapped call (not in Algorithm mode)\n";
}

std::string join_sorted(const std::vector<std::string>& v) {
    std::string s;
    for (const auto& e : v) { if (!s.empty()) s += ", "; s += e; }
    return s;
}

// simple_logger.hpp:16-45
struct logger {
    bool print_progress;
    bool append_result_stats;
    void log(const std::string& msg) const { if (print_progress) std::cout << msg << std::endl; }
    void result_stats(const validation_results& r, std::optional<bool> header_override) const {
        if (print_progress) {
            std::cout << r;
        } else {
            if ((header_override.has_value() && *header_override) || (!header_override.has_value() && !append_result_stats))
                std::cout << validation_results::csv_header() << "\n";
            std::cout << r.csv_data() << "\n";
        }
    }
};

// main.cpp:81-121: "<label>,<label>_iterations,...,<property names>" then one row per loop.
void output_measurements(const std::filesystem::path& path, const std::vector<std::string>& labels,
                         const std::vector<measurement_result>& results, const string_pairs& props, bool append) {
    std::ofstream f;
    if (append) {
        f.open(path, std::ios_base::app);
    } else {
        f.open(path);
        const char* sep = "";
        for (const auto& l : labels) { f << sep << l << "," << l << "_iterations"; sep = ","; }
        if (!props.empty()) {
            if (!labels.empty()) f << ",";
            sep = "";
            for (const auto& p : props) { f << sep << p.first; sep = ","; }
        }
        f << "\n";
    }
    const char* sep = "";
    for (const auto& r : results) { f << sep << r.iteration_ns() << "," << r.iterations; sep = ","; }
    if (!props.empty()) {
        if (!results.empty()) f << ",";
        sep = "";
        for (const auto& p : props) { f << sep << p.second; sep = ","; }
    }
    f << "\n";
}

std::filesystem::path loop_out_path(const std::filesystem::path& out, std::size_t loop) {
    std::filesystem::path p = out;   // run_args.cpp:142-150
    return p.replace_filename(out.stem().string() + "_" + std::to_string(loop) + out.extension().string());
}

int run_computation_steps(algorithm& alg, const logger& log) {
    struct step { const char* message; const char* name; void (algorithm::*fn)(); };
    const step steps[] = {
        {"Allocating", "allocation", &algorithm::prepare},
        {"Transfering data", "data transfer", &algorithm::transfer},
        {"Running test alg", "computation", &algorithm::run},
        {"Copying output data to host", "finalization", &algorithm::finalize},
        {"Free resources", "free", &algorithm::free},
    };
    for (const auto& s : steps) {
        try {
            log.log(s.message);
            (alg.*(s.fn))();
        } catch (std::exception& e) {
            std::cerr << "Exception occured durign " << s.name << " step: " << e.what()
                      << "\nLast kernel launch arguments:\n" << xcorr_last_launch_string() << std::endl;
            return 3;
        }
    }
    return 0;
}

// ---- `run --data_type double` -------------------------------------------------------------------
// The reference parses the option and refuses it (main.cpp:431-438: the <double> dispatch is
// commented out).  Here every direct algorithm name runs its mode in double through the library's
// double-precision kernel (xcorr_run_f64; the name selects the mode, not a kernel family), the
// cpu_* names through the CPU loop in double; same files, steps, timing labels and exit codes as
// the float path.  The FFT names stay single precision.
struct double_run_options {
    const algorithm_spec* spec;
    std::filesystem::path ref_path, target_path, times_path;
    std::optional<std::filesystem::path> out_path;
    std::optional<std::string> validate;       // empty string: recompute on the CPU
    benchmark_type bench;
    std::size_t outer_loops;
    double min_time_ns;
    bool append, progress;
};

void cpu_run_double(int mode, const basic_matrix_array<double>& left, const basic_matrix_array<double>& right,
                    basic_matrix_array<double>& out, bool grouped) {
    const int H = static_cast<int>(left.rows()), W = static_cast<int>(left.cols());
    const uint32_t nl = left.num_matrices(), nr = right.num_matrices();
    switch (mode) {
    case XCORR_ONE_TO_ONE:
        cpu_cross_corr_pair<double, double>(left.matrix(0), right.matrix(0), out.matrix(0), H, W);
        break;
    case XCORR_ONE_TO_MANY:
        for (uint32_t t = 0; t < nr; ++t) cpu_cross_corr_pair<double, double>(left.matrix(0), right.matrix(t), out.matrix(t), H, W);
        break;
    case XCORR_N_TO_MN: {
        const uint32_t m = nr / nl;
        for (uint32_t r = 0; r < nl; ++r)
            for (uint32_t t = 0; t < m; ++t) {
                const uint32_t idx = grouped ? r * m + t : t * nl + r;
                cpu_cross_corr_pair<double, double>(left.matrix(r), right.matrix(idx), out.matrix(idx), H, W);
            }
        break;
    }
    default:
        for (uint32_t r = 0; r < nl; ++r)
            for (uint32_t t = 0; t < nr; ++t)
                cpu_cross_corr_pair<double, double>(left.matrix(r), right.matrix(t), out.matrix(r * nr + t), H, W);
    }
}

int run_double(const double_run_options& o) {
    using darray = basic_matrix_array<double>;
    const algorithm_spec& spec = *o.spec;
    if (spec.fam == family::fft) {
        std::cerr << "Data type double is not available for the FFT algorithms (cuFFT path is single precision)\n";
        return 1;
    }
    const bool gpu = spec.fam != family::cpu;
    const bool compute_bench = o.bench == benchmark_type::Compute, common = o.bench == benchmark_type::CommonSteps;
    const bool alg_bench = o.bench == benchmark_type::Algorithm;
    logger log{o.progress && !compute_bench, o.append};
    if (gpu) {
        int have = 0;
        if (cudaGetDeviceCount(&have) != cudaSuccess || have == 0)
            throw std::runtime_error("no CUDA device is available; only the cpu_* algorithms run without one");
    }
    std::vector<measurement_result> steps(7);
    auto timed = [&](std::size_t label, auto&& fn) {
        auto t0 = wall_clock::now();
        fn();
        if (gpu) cudaDeviceSynchronize();
        steps[label] = measurement_result{elapsed_ns(t0), 1};
    };
    darray left, right, result;
    const bool grouped = spec.mode == XCORR_N_TO_MN && gpu;     // the library's order for n_to_mn
    try {
        log.log("Loading inputs");
        timed(0, [&] {
            left = darray::load_csv(o.ref_path, gpu);
            right = darray::load_csv(o.target_path, gpu, grouped ? left.num_matrices() : 0);
            if (left.rows() != right.rows() || left.cols() != right.cols())
                throw std::runtime_error("Invalid input matrix sizes, expected ref and target to be the same size");
            if (!xcorr_validate_input_size(spec.mode, left.rows(), left.cols(), left.num_matrices(), right.num_matrices()))
                throw std::runtime_error("Invalid input matrix counts for " + spec.name + ": " +
                                         std::to_string(left.num_matrices()) + " left, " +
                                         std::to_string(right.num_matrices()) + " right");
        });
    } catch (std::exception& e) {
        std::cerr << "Exception occured durign data loading step: " << e.what() << std::endl;
        return 3;
    }
    const uint32_t rows = left.rows(), cols = left.cols(), nl = left.num_matrices(), nr = right.num_matrices();
    const uint64_t n_out = xcorr_num_results(spec.mode, nl, nr);
    const std::size_t out_elems = static_cast<std::size_t>(2 * rows - 1) * (2 * cols - 1);
    double *d_left = nullptr, *d_right = nullptr, *d_out = nullptr;
    measurement_result kernel_result;
    auto check = [](cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    };
    auto xcheck = [](int st) {
        if (st != XCORR_OK)
            throw std::runtime_error(std::string("xcorr: ") + xcorr_status_string(st) + ": " + xcorr_last_error_string());
    };
    auto computation = [&]() -> int {
        struct step { const char* message; const char* name; std::size_t label; std::function<void()> fn; };
        const std::vector<step> seq = {
            {"Allocating", "allocation", 1, [&] {
                 result = darray(2 * rows - 1, 2 * cols - 1, static_cast<dsize_t>(n_out), gpu);
                 if (!gpu) return;
                 check(cudaMalloc(&d_left, left.size() * sizeof(double)), "cudaMalloc");
                 check(cudaMalloc(&d_right, right.size() * sizeof(double)), "cudaMalloc");
                 check(cudaMalloc(&d_out, n_out * out_elems * sizeof(double)), "cudaMalloc");
             }},
            {"Transfering data", "data transfer", 2, [&] {
                 if (!gpu) return;
                 check(cudaMemcpy(d_left, left.data(), left.size() * sizeof(double), cudaMemcpyHostToDevice), "cudaMemcpy");
                 check(cudaMemcpy(d_right, right.data(), right.size() * sizeof(double), cudaMemcpyHostToDevice), "cudaMemcpy");
             }},
            {"Running test alg", "computation", 3, [&] {
                 if (!gpu) { cpu_run_double(spec.mode, left, right, result, false); return; }
                 if (!alg_bench) { xcheck(xcorr_run_f64(spec.mode, d_left, d_right, d_out, rows, cols, nl, nr, nullptr)); return; }
                 // CUDA_ADAPTIVE_MEASURE (stopwatch.hpp:125-141): events around a growing number of launches
                 cudaEvent_t e0, e1;
                 check(cudaEventCreate(&e0), "cudaEventCreate");
                 check(cudaEventCreate(&e1), "cudaEventCreate");
                 std::size_t iterations = 1;
                 do {
                     check(cudaEventRecord(e0, nullptr), "cudaEventRecord");
                     for (std::size_t i = 0; i < iterations; ++i)
                         xcheck(xcorr_run_f64(spec.mode, d_left, d_right, d_out, rows, cols, nl, nr, nullptr));
                     check(cudaEventRecord(e1, nullptr), "cudaEventRecord");
                     check(cudaEventSynchronize(e1), "cudaEventSynchronize");
                     float ms = 0.f;
                     check(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
                     kernel_result = measurement_result{static_cast<double>(ms) * 1e6, iterations};
                     iterations = next_iteration_count(o.min_time_ns, kernel_result);
                 } while (iterations != 0);
                 cudaEventDestroy(e0);
                 cudaEventDestroy(e1);
             }},
            {"Copying output data to host", "finalization", 4, [&] {
                 if (!gpu) return;
                 check(cudaMemcpy(result.data(), d_out, n_out * out_elems * sizeof(double), cudaMemcpyDeviceToHost), "cudaMemcpy");
             }},
            {"Free resources", "free", 5, [&] {
                 cudaFree(d_left); cudaFree(d_right); cudaFree(d_out);
                 d_left = d_right = d_out = nullptr;
             }},
        };
        for (const auto& s : seq) {
            try {
                log.log(s.message);
                if (common) timed(s.label, s.fn); else s.fn();
            } catch (std::exception& e) {
                std::cerr << "Exception occured durign " << s.name << " step: " << e.what()
                          << "\nLast kernel launch arguments:\n" << xcorr_last_launch_string() << std::endl;
                return 3;
            }
        }
        return 0;
    };
    for (std::size_t loop = 0; loop < o.outer_loops; ++loop) {
        measurement_result compute_result;
        if (compute_bench) {
            std::size_t iterations = 1;
            do {
                auto t0 = wall_clock::now();
                for (std::size_t i = 0; i < iterations; ++i) {
                    if (int ret = computation()) return ret;
                    if (gpu) cudaDeviceSynchronize();
                }
                compute_result = measurement_result{elapsed_ns(t0), iterations};
                iterations = next_iteration_count(o.min_time_ns, compute_result);
            } while (iterations != 0);
        } else if (int ret = computation()) {
            return ret;
        }
        if (gpu && xcorr_check_device() != XCORR_OK) {
            std::cerr << "Exception somewhere in CUDA code: " << xcorr_last_error_string()
                      << "\nLast kernel launch arguments:\n" << xcorr_last_launch_string() << std::endl;
            return 3;
        }
        if (o.out_path.has_value()) {
            log.log("Storing results");
            const auto path = o.outer_loops > 1 ? loop_out_path(*o.out_path, loop) : *o.out_path;
            timed(6, [&] { result.store_csv(path, grouped ? nr / nl : 0); });
        }
        if (o.bench != benchmark_type::None) {
            std::vector<std::string> labels;
            std::vector<measurement_result> results;
            if (compute_bench) { labels = {"Computation"}; results = {compute_result}; }
            else if (common) { labels = {"Load", "Prepare", "Transfer", "Run", "Finalize", "Free", "Store"}; results = steps; }
            else if (gpu) { labels = {"Kernel"}; results = {kernel_result}; }
            output_measurements(o.times_path, labels, results, {}, o.append || loop > 0);
        }
        if (!o.validate.has_value()) {
            log.log("No validation");
        } else {
            darray valid;
            if (!o.validate->empty()) {
                log.log("Validating results against " + *o.validate);
                valid = darray::load_csv(*o.validate, false, grouped ? nl : 0);
                if (valid.rows() != result.rows() || valid.cols() != result.cols() || valid.num_matrices() != result.num_matrices())
                    throw std::runtime_error("Cannot validate matrices of different sizes");
            } else {
                log.log("Computing valid results and validating");
                valid = darray(result.rows(), result.cols(), result.num_matrices(), false);
                cpu_run_double(spec.mode, left, right, valid, grouped);
            }
            log.result_stats(validate_result<double>(result.data(), valid.data(), result.size()), !o.append && loop == 0);
        }
    }
    return 0;
}

int command_run(const std::vector<std::string>& tokens, const std::string& prog) {
    parsed_args a = parse_options(tokens, kRunOptions);
    if (a.has("help")) { print_help(std::cout, prog); return 0; }
    if (a.positional.size() < 3) throw option_error("the option '--alg', '--ref_path' or '--target_path' is required but missing");
    if (a.positional.size() > 3) throw option_error("too many positional options have been specified on the command line");
    const std::string alg_name = a.positional[0];
    const std::filesystem::path ref_path = a.positional[1], target_path = a.positional[2];

    const std::string data_type = a.has("data_type") ? a.values["data_type"] : "single";
    const benchmark_type bench = a.has("benchmark_type") ? parse_benchmark_type(a.values["benchmark_type"]) : benchmark_type::None;
    const std::filesystem::path times_path = a.has("times") ? a.values["times"] : "measurements.csv";
    std::optional<std::filesystem::path> out_path;
    if (a.has("out") && !a.values["out"].empty()) out_path = a.values["out"];
    const bool append = a.has("append"), progress = !a.has("no_progress");
    std::size_t outer_loops = 1;
    double min_time_s = 1.0;
    int n_devices = 1;
    try {
        if (a.has("outer_loops")) outer_loops = std::stoul(a.values["outer_loops"]);
        if (a.has("min_time")) min_time_s = std::stod(a.values["min_time"]);
        if (const char* env = std::getenv("XCORR_DEVICES")) n_devices = std::stoi(env);
        if (a.has("devices")) n_devices = std::stoi(a.values["devices"]);
    } catch (std::exception&) {
        throw option_error("the argument for a numeric option is invalid");
    }

    const algorithm_spec* spec = find_algorithm(alg_name);
    if (!spec) {   // run_args.cpp:114-117
        std::cerr << "Unknown algorithm \"" << alg_name << "\", expected one of "
                  << join_sorted(sorted_algorithm_names(false)) << std::endl;
        print_help(std::cerr, prog);
        return 1;
    }
    if (bench == benchmark_type::Unknown) {
        std::cerr << "Unknown benchmark type" << std::endl;
        print_help(std::cerr, prog);
        return 1;
    }
    if (data_type != "single" && data_type != "double") {   // main.cpp:431-438
        std::cerr << "Unknown data type " << data_type << "\n";
        print_help(std::cerr, prog);
        return 1;
    }
    if (data_type == "double") {
        double_run_options o{spec, ref_path, target_path, times_path, out_path, std::nullopt, bench, outer_loops,
                             min_time_s * 1e9, append, progress};
        if (a.has("validate")) o.validate = a.values["validate"];
        return run_double(o);
    }
    if (n_devices < 1) throw option_error("--devices must be at least 1");
    std::vector<int> devices;
    for (int i = 0; i < n_devices; ++i) devices.push_back(i);

    const bool compute_bench = bench == benchmark_type::Compute;
    logger log{progress && !compute_bench, append};

    json_object alg_args;
    if (a.has("args_path")) {
        std::ifstream f(a.values["args_path"]);
        if (!f) throw std::runtime_error("Could not open algorithm arguments file " + a.values["args_path"]);
        alg_args = json_object::parse(f);
    }
    algorithm alg(*spec, alg_args, min_time_s * 1e9, bench, devices);
    alg.set_normalize(a.has("normalize"));
    {
        const char* env = std::getenv("XCORR_PIPELINED");
        alg.set_pipelined(a.has("pipelined") || (env && env[0] == '1'));
    }
    if (spec->fam != family::cpu) {
        int have = 0;
        if (cudaGetDeviceCount(&have) != cudaSuccess || have == 0)
            throw std::runtime_error("no CUDA device is available; only the cpu_* algorithms run without one");
        if (n_devices > have)
            throw std::runtime_error("--devices " + std::to_string(n_devices) + " asked for, " + std::to_string(have) + " present");
    }

    try {
        log.log("Loading inputs");
        alg.load(ref_path, target_path);
    } catch (std::exception& e) {
        std::cerr << "Exception occured durign data loading step: " << e.what() << std::endl;
        return 3;
    }

    for (std::size_t loop = 0; loop < outer_loops; ++loop) {
        measurement_result compute_result;
        if (compute_bench) {   // CPU_ADAPTIVE_MEASURE around all steps, main.cpp:260-265
            std::size_t iterations = 1;
            do {
                auto t0 = wall_clock::now();
                for (std::size_t i = 0; i < iterations; ++i) {
                    int ret = run_computation_steps(alg, log);
                    if (ret != 0) return ret;
                    if (spec->fam != family::cpu) cudaDeviceSynchronize();
                }
                compute_result = measurement_result{elapsed_ns(t0), iterations};
                iterations = next_iteration_count(min_time_s * 1e9, compute_result);
            } while (iterations != 0);
        } else {
            int ret = run_computation_steps(alg, log);
            if (ret != 0) return ret;
        }
        if (spec->fam != family::cpu) {
            // CUCH(cudaDeviceSynchronize()); CUCH(cudaGetLastError()) of main.cpp:267-270, plus the
            // library's own device-side waits
            if (xcorr_check_device() != XCORR_OK) {
                std::cerr << "Exception somewhere in CUDA code: " << xcorr_last_error_string()
                          << "\nLast kernel launch arguments:\n" << xcorr_last_launch_string() << std::endl;
                return 3;
            }
        }
        if (bench != benchmark_type::None) {
            if (!compute_bench) log.log("Collect measurements");
            output_measurements(times_path,
                                compute_bench ? std::vector<std::string>{"Computation"} : alg.measurement_labels(),
                                compute_bench ? std::vector<measurement_result>{compute_result} : alg.measurements(),
                                alg.additional_properties(), append || loop > 0);
            if (!compute_bench) {
                log.log("Reset measurement");
                alg.reset_measurements();
            }
        }
        if (out_path.has_value()) {
            log.log("Storing results");
            alg.store_results(outer_loops > 1 ? loop_out_path(*out_path, loop) : *out_path);
        }
        if (!a.has("validate")) {
            log.log("No validation");
        } else if (!a.values["validate"].empty()) {
            log.log("Validating results against " + a.values["validate"]);
            log.result_stats(alg.validate(std::filesystem::path(a.values["validate"])), !append && loop == 0);
        } else {
            log.log("Computing valid results and validating");
            log.result_stats(alg.validate(std::nullopt), !append && loop == 0);
        }
    }
    return 0;
}

// main.cpp:56-79: compare result files with a template file, element errors in double.
int command_validate(const std::vector<std::string>& tokens, const std::string& prog) {
    parsed_args a = parse_options(tokens, kValidateOptions);
    if (a.has("help")) { print_help(std::cout, prog); return 0; }
    if (a.positional.size() < 2)
        throw option_error("the option '--template_data_path' and '--validate_data_path' are required but missing");
    const bool normalize = a.has("normalize");
    const bool csv = a.has("csv"), header = a.has("print_header");
    logger log{!csv, true};
    matrix_array valid = matrix_array::load_csv(a.positional[0], false);
    std::vector<double> valid_d(valid.data(), valid.data() + valid.size());
    for (std::size_t i = 1; i < a.positional.size(); ++i) {
        log.log("Validating " + a.positional[i]);
        matrix_array target = matrix_array::load_csv(a.positional[i], false);
        if (normalize) target = normalize_fft_results(target);          // main.cpp:74-76
        if (target.rows() != valid.rows() || target.cols() != valid.cols() || target.num_matrices() != valid.num_matrices())
            throw std::runtime_error("Cannot validate matrices of different sizes");
        std::vector<double> target_d(target.data(), target.data() + target.size());
        log.result_stats(validate_result<double>(target_d.data(), valid_d.data(), target_d.size()), i == 1 && header);
    }
    return 0;
}

int command_input(const std::vector<std::string>& tokens, const std::string& prog) {
    parsed_args a = parse_options(tokens, kInputOptions);
    if (a.has("help")) { print_help(std::cout, prog); return 0; }
    if (a.positional.size() != 5)
        throw option_error("input needs <alg_type> <rows> <columns> <left_matrices> <right_matrices>");
    static const std::map<std::string, int> modes = {
        {"one_to_one", XCORR_ONE_TO_ONE}, {"one_to_many", XCORR_ONE_TO_MANY},
        {"n_to_mn", XCORR_N_TO_MN}, {"n_to_m", XCORR_N_TO_M}};
    unsigned long v[4];
    try {
        for (int i = 0; i < 4; ++i) {
            if (!a.positional[i + 1].empty() && a.positional[i + 1][0] == '-') throw std::invalid_argument("negative");
            v[i] = std::stoul(a.positional[i + 1]);
        }
    } catch (std::exception&) {
        throw option_error("the argument for a size is invalid");
    }
    auto it = modes.find(a.positional[0]);
    if (it == modes.end()) {   // main.cpp:347-351
        std::cerr << "Unknown algorithm type \"" << a.positional[0] << "\", expected one of n_to_m, n_to_mn, one_to_many, one_to_one" << std::endl;
        print_help(std::cerr, prog);
        return 1;
    }
    const bool ok = xcorr_validate_input_size(it->second, static_cast<uint32_t>(v[0]), static_cast<uint32_t>(v[1]),
                                              static_cast<uint32_t>(v[2]), static_cast<uint32_t>(v[3])) != 0;
    std::cout << (ok ? "Valid\n" : "Invalid\n");
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    const std::string prog = argc > 0 ? argv[0] : "cross";
    try {
        std::vector<std::string> tokens(argv + 1, argv + argc);
        // global options come before the command; the first non-option token is the command
        std::size_t i = 0;
        bool help = false;
        while (i < tokens.size() && !tokens[i].empty() && tokens[i][0] == '-') {
            if (tokens[i] == "-h" || tokens[i] == "--help") help = true;
            else throw option_error("unrecognised option '" + tokens[i] + "'");
            ++i;
        }
        if (help || i >= tokens.size()) {
            print_help(std::cout, prog);
            return 0;
        }
        const std::string cmd = tokens[i];
        std::vector<std::string> rest(tokens.begin() + i + 1, tokens.end());
        if (cmd == "run") {
            int ret = command_run(rest, prog);
            return ret;
        } else if (cmd == "validate") {
            return command_validate(rest, prog);
        } else if (cmd == "list") {
            for (const auto& n : sorted_algorithm_names(false)) std::cout << n << "\n";
            return 0;
        } else if (cmd == "input") {
            return command_input(rest, prog);
        }
        std::cerr << "Unknown command " << cmd << "\n";
        print_help(std::cerr, prog);
        return 1;
    } catch (option_error& e) {
        std::cerr << "Invalid commandline options: " << e.what() << std::endl;
        return 1;
    } catch (argument_error& e) {
        std::cerr << "Invalid algorithm argument value: " << e.what() << std::endl;
        return 1;
    } catch (std::exception& e) {
        std::cerr << "Exception occured: " << e.what() << std::endl;
        return 2;
    }
}
