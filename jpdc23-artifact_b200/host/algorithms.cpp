#include "algorithms.hpp"

#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstring>

namespace cross {

namespace {

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
#define CUCH(call) cuda_check((call), #call)

void xcorr_check(int status) {
    if (status != XCORR_OK)
        throw std::runtime_error(std::string("xcorr: ") + xcorr_status_string(status) + ": " + xcorr_last_error_string());
}

arg_spec I(const char* key, long def) { return arg_spec{key, arg_spec::kind::integer, def, "", ""}; }
arg_spec B(const char* key, bool def) { return arg_spec{key, arg_spec::kind::boolean, def ? 1 : 0, "", ""}; }
arg_spec T(const char* key, const char* def) { return arg_spec{key, arg_spec::kind::text, 0, def, ""}; }
arg_spec IFROM(const char* key, const char* other) { return arg_spec{key, arg_spec::kind::integer, 0, "", other}; }

std::vector<algorithm_spec> build_registry() {
    const int O2O = XCORR_ONE_TO_ONE, O2M = XCORR_ONE_TO_MANY, NMN = XCORR_N_TO_MN, N2M = XCORR_N_TO_M;
    const arg_spec w = I("warps_per_thread_block", 8);
    const arg_spec streams = I("num_cuda_streams", 8);
    auto smem = [](long shifts) {
        return std::vector<arg_spec>{I("shifts_per_thread_block", shifts), I("shared_mem_row_size", 32),
                                     IFROM("shared_mem_rows", "shifts_per_thread_block"), B("strided_load", true),
                                     B("column_group_per_block", false)};
    };
    auto with = [](std::vector<arg_spec> v, std::initializer_list<arg_spec> more) {
        v.insert(v.end(), more.begin(), more.end());
        return v;
    };
    std::vector<algorithm_spec> r = {
        // CPU path (main.cpp:368-371)
        {"cpu_one_to_one", O2O, family::cpu, {}, false},
        {"cpu_one_to_many", O2M, family::cpu, {}, false},
        {"cpu_n_to_mn", NMN, family::cpu, {}, false},
        {"cpu_n_to_m", N2M, family::cpu, {}, false},
        // overlap-wise (main.cpp:372-375)
        {"nai_orig_one_to_one", O2O, family::overlap_wise, {}, false},
        {"nai_orig_one_to_many", O2M, family::overlap_wise, {}, false},
        {"nai_orig_n_to_mn", NMN, family::overlap_wise, {}, false},
        {"nai_orig_n_to_m", N2M, family::overlap_wise, {streams}, false},
        // warp-shuffle families (main.cpp:376-394) -> register-tiled kernel
        {"nai_shuffle_one_to_one", O2O, family::tile, {w}, false},
        {"nai_shuffle_work_distribution_one_to_one", O2O, family::tile,
         {w, I("rows_per_thread", 10), T("distribution_type", "rectangle")}, true},
        {"nai_shuffle_multimat_right_one_to_one", O2O, family::tile, {w}, false},
        {"nai_shuffle_multimat_right_one_to_many", O2M, family::tile, {w, I("right_matrices_per_thread", 2)}, false},
        {"nai_shuffle_multimat_right_work_distribution_one_to_one", O2O, family::tile,
         {w, I("rows_per_thread", 10), T("distribution_type", "rectangle")}, true},
        {"nai_shuffle_multimat_right_work_distribution_one_to_many", O2M, family::tile,
         {w, I("right_matrices_per_thread", 2), I("rows_per_thread", 10), T("distribution_type", "rectangle")}, true},
        {"nai_shuffle_multimat_right_work_distribution_n_to_mn", NMN, family::tile,
         {w, I("right_matrices_per_thread", 2), I("rows_per_thread", 10), T("distribution_type", "rectangle"), streams}, true},
        {"nai_shuffle_multimat_right_work_distribution_n_to_m", N2M, family::tile,
         {w, I("right_matrices_per_thread", 2), I("rows_per_thread", 10), T("distribution_type", "rectangle"), streams}, true},
        {"nai_shuffle_multimat_both_work_distribution_local_mem_n_to_m", N2M, family::tile,
         {w, I("left_matrices_per_thread", 2), I("right_matrices_per_thread", 2), I("rows_per_thread", 10),
          T("distribution_type", "triangle")}, true},
        {"nai_shuffle_multimat_both_work_distribution_n_to_m", N2M, family::tile,
         {w, I("left_matrices_per_thread", 2), I("right_matrices_per_thread", 2), I("rows_per_thread", 10),
          T("distribution_type", "triangle")}, true},
        {"nai_shuffle_multirow_both_multimat_both_n_to_m", N2M, family::tile,
         {w, I("shifts_per_thread_right_matrix", 2), I("left_matrices_per_thread", 2),
          I("right_matrices_per_thread", 2), I("left_rows_per_iteration", 2)}, false},
        {"nai_shuffle_multirow_right_one_to_one", O2O, family::tile, {w, I("right_rows_per_thread", 4)}, false},
        {"nai_shuffle_multirow_both_one_to_one", O2O, family::tile,
         {w, I("shifts_per_thread", 4), I("left_rows_per_iteration", 3)}, false},
        {"nai_shuffle_multirow_both_local_mem_one_to_one", O2O, family::tile,
         {w, I("shifts_per_thread", 4), I("left_rows_per_iteration", 3)}, false},
        {"nai_shuffle_multirow_right_multimat_right_one_to_one", O2O, family::tile,
         {w, I("right_rows_per_thread", 4)}, false},
        {"nai_shuffle_multirow_right_multimat_right_one_to_many", O2M, family::tile,
         {w, I("right_rows_per_thread", 4), I("right_matrices_per_thread", 4)}, false},
        {"nai_shuffle_multirow_right_multimat_right_n_to_mn", NMN, family::tile,
         {w, I("right_rows_per_thread", 4), I("right_matrices_per_thread", 4), streams}, false},
        {"nai_shuffle_multirow_both_multimat_right_one_to_many", O2M, family::tile,
         {w, I("shifts_per_thread_right_matrix", 4), I("right_matrices_per_thread", 4),
          I("left_rows_per_iteration", 4)}, false},
        {"nai_shuffle_multirow_both_multimat_right_n_to_mn", NMN, family::tile,
         {w, I("shifts_per_thread_right_matrix", 4), I("right_matrices_per_thread", 4),
          I("left_rows_per_iteration", 4), streams}, false},
        // warp-per-overlap and block-per-overlap (main.cpp:395-402)
        {"nai_warp_per_shift_one_to_one", O2O, family::warp_per_overlap, {I("shifts_per_thread_block", 8)}, false},
        {"nai_warp_per_shift_simple_indexing_one_to_one", O2O, family::warp_per_overlap,
         {I("shifts_per_thread_block", 8)}, false},
        {"nai_warp_per_shift_work_distribution_one_to_one", O2O, family::warp_per_overlap,
         {I("shifts_per_thread_block", 8), I("rows_per_warp", 3), T("distribution_type", "rectangle")}, false},
        {"nai_warp_per_shift_shared_mem_one_to_one", O2O, family::warp_staged, smem(32), false},
        {"nai_warp_per_shift_shared_mem_one_to_many", O2M, family::warp_staged,
         with(smem(16), {I("right_matrices_per_block", 8)}), false},
        {"nai_warp_per_shift_shared_mem_n_to_mn", NMN, family::warp_staged,
         with(smem(16), {I("right_matrices_per_block", 8), streams}), false},
        {"nai_warp_per_shift_shared_mem_n_to_m", N2M, family::warp_staged,
         with(smem(16), {I("right_matrices_per_block", 8), streams}), false},
        {"nai_block_per_shift_one_to_one", O2O, family::warp_per_overlap, {I("block_size", 128)}, false},
        // FFT engine (main.cpp:403-409); argument keys of one_to_one.hpp:895,1029-1031, n_to_m.hpp:655-656
        {"fft_orig_one_to_one", O2O, family::fft, {I("hadamard_threads_per_block", 256)}, false},
        {"fft_reduced_transfer_one_to_one", O2O, family::fft,
         {I("scatter_threads_per_block", 256), I("scatter_items_per_thread", 10), I("hadamard_threads_per_block", 256)}, false},
        {"fft_orig_one_to_many", O2M, family::fft, {I("hadamard_threads_per_block", 256)}, false},
        {"fft_reduced_transfer_one_to_many", O2M, family::fft,
         {I("scatter_threads_per_block", 256), I("scatter_items_per_thread", 10), I("hadamard_threads_per_block", 256)}, false},
        {"fft_orig_n_to_mn", NMN, family::fft, {I("hadamard_threads_per_block", 256)}, false},
        {"fft_reduced_transfer_n_to_mn", NMN, family::fft,
         {I("scatter_threads_per_block", 256), I("scatter_items_per_thread", 10), I("hadamard_threads_per_block", 256)}, false},
        {"fft_better_n_to_m", N2M, family::fft,
         {I("hadamard_threads_per_block", 256), I("hadamard_items_per_thread", 10)}, false},
    };
    return r;
}

bool is_pow2(long v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

benchmark_type parse_benchmark_type(const std::string& token) {
    std::string t = token;
    std::transform(t.begin(), t.end(), t.begin(), [](unsigned char c) { return std::tolower(c); });
    if (t == "compute") return benchmark_type::Compute;
    if (t == "commonsteps") return benchmark_type::CommonSteps;
    if (t == "algorithm") return benchmark_type::Algorithm;
    if (t == "none") return benchmark_type::None;
    return benchmark_type::Unknown;
}

const char* to_string(benchmark_type t) {
    switch (t) {
    case benchmark_type::None: return "None";
    case benchmark_type::Compute: return "Compute";
    case benchmark_type::CommonSteps: return "CommonSteps";
    case benchmark_type::Algorithm: return "Algorithm";
    default: return "Unknown";
    }
}

const std::vector<algorithm_spec>& algorithm_registry() {
    static const std::vector<algorithm_spec> registry = build_registry();
    return registry;
}

const algorithm_spec* find_algorithm(const std::string& name) {
    for (const auto& s : algorithm_registry())
        if (s.name == name) return &s;
    return nullptr;
}

std::vector<std::string> sorted_algorithm_names(bool) {
    std::vector<std::string> names;
    for (const auto& s : algorithm_registry())
        names.push_back(s.name);
    std::sort(names.begin(), names.end());
    return names;
}

// ------------------------------------------------------------------------------------------
algorithm::algorithm(const algorithm_spec& spec, const json_object& args, double min_time_ns,
                     benchmark_type bench, std::vector<int> devices)
    : spec_(spec), min_time_ns_(min_time_ns), bench_(bench), devices_(std::move(devices)) {
    if (devices_.empty()) devices_.push_back(0);

    // JSON -> values with the reference's defaults, echoed in the reference's column order
    std::map<std::string, long> ints;
    for (const auto& a : spec_.args) {
        switch (a.type) {
        case arg_spec::kind::integer: {
            long def = a.default_from.empty() ? a.default_int : ints.at(a.default_from);
            long v = args.value(a.key, def);
            if (a.key == "shared_mem_rows") {
                // one_to_one.hpp:573-586: 0 means "as many as shifts", fewer than shifts is an error
                const long shifts = ints.at("shifts_per_thread_block");
                if (v == 0) v = shifts;
                if (v < shifts)
                    throw argument_error("Invalid number of shared memory rows " + std::to_string(v) +
                                         ", must be greater than shifts per thread block " + std::to_string(shifts), a.key);
            } else if (v <= 0) {
                throw argument_error("Invalid value " + std::to_string(v) + " of \"" + a.key + "\", must be positive", a.key);
            }
            ints[a.key] = v;
            properties_.emplace_back(a.key, std::to_string(v));
            break;
        }
        case arg_spec::kind::boolean:
            properties_.emplace_back(a.key, args.value(a.key, a.default_int != 0) ? "1" : "0");
            break;
        case arg_spec::kind::text: {
            std::string v = args.value(a.key, a.default_text);
            if (a.key == "distribution_type" && v != "none" && v != "rectangle" && v != "triangle")
                throw argument_error("Unknown distribution type \"" + v + "\"", a.key);
            properties_.emplace_back(a.key, v);
            break;
        }
        }
    }

    // values -> hints of the CUDA library
    switch (spec_.fam) {
    case family::overlap_wise:
        hints_.kernel = XCORR_KERNEL_OVERLAP_WISE;
        break;
    case family::warp_per_overlap: {
        hints_.kernel = XCORR_KERNEL_WARP_PER_OVERLAP;
        long threads = 256;
        if (ints.count("shifts_per_thread_block")) threads = 32 * ints["shifts_per_thread_block"];
        if (ints.count("block_size")) threads = (ints["block_size"] + 31) / 32 * 32;
        hints_.block_threads = static_cast<int32_t>(std::min<long>(std::max<long>(threads, 32), 1024));
        // nai_warp_per_shift_work_distribution_one_to_one: the rows of an overlap shared by several
        // warps (one_to_one.hpp:470-520)
        if (ints.count("rows_per_warp")) {
            std::string dist = "rectangle";
            for (const auto& pr : properties_)
                if (pr.first == "distribution_type") dist = pr.second;
            hints_.rows_per_warp = static_cast<int32_t>(ints["rows_per_warp"]);
            hints_.row_split = dist == "none" ? XCORR_SPLIT_NONE : dist == "triangle" ? XCORR_SPLIT_TRIANGLE : XCORR_SPLIT_RECTANGLE;
        }
        break;
    }
    case family::warp_staged: {
        // The shared-memory warp-per-overlap family (one_to_one.hpp:540-680, one_to_many.hpp:395-499,
        // n_to_mn.hpp:575-716, n_to_m.hpp:520-645): every key shapes the launch.
        hints_.kernel = XCORR_KERNEL_WARP_STAGED;
        const long shifts = std::min<long>(std::max<long>(ints["shifts_per_thread_block"], 1), 32);
        hints_.block_threads = static_cast<int32_t>(32 * shifts);
        hints_.staged_cols = static_cast<int32_t>(ints["shared_mem_row_size"]);
        hints_.staged_rows = static_cast<int32_t>(ints["shared_mem_rows"]);
        hints_.staged_rights = static_cast<int32_t>(ints.count("right_matrices_per_block") ? ints["right_matrices_per_block"] : 1);
        if (hints_.staged_rights > 8)      // WARP_PER_SHIFT_SHARED_MEM_RIGHT_MATRICES_PER_BLOCK_LIMIT (CMakeLists.txt:45)
            throw argument_error("Invalid number of right matrices per block " + std::to_string(hints_.staged_rights) +
                                 ", must be at most 8", "right_matrices_per_block");
        for (const auto& pr : properties_) {
            if (pr.first == "strided_load") hints_.staged_warp_rows = pr.second == "1" ? 0 : 1;
            if (pr.first == "column_group_per_block") hints_.staged_column_groups = pr.second == "1" ? 1 : 0;
        }
        break;
    }
    case family::fft:
        // The reference's launch-shape keys (threads per block, items per thread) are echoed in
        // the timing file and otherwise unused: the library sizes its own grids.
        hints_.kernel = XCORR_KERNEL_FFT;
        break;
    case family::tile: {
        hints_.kernel = XCORR_KERNEL_TILE;
        // Legacy keys steer the plan only when the file names them; defaults stay automatic.
        for (const char* key : {"shifts_per_thread", "shifts_per_thread_right_matrix"})
            if (args.contains(key)) hints_.overlap_rows = static_cast<int32_t>(std::min<long>(ints[key], 4));
        if (args.contains("right_matrices_per_thread")) {
            const long rm = ints["right_matrices_per_thread"];
            if (is_pow2(rm) && rm <= 32) hints_.class_lanes = static_cast<int32_t>(32 / rm);
        }
        if (spec_.split_rows && args.contains("rows_per_thread")) rows_per_thread_ = ints["rows_per_thread"];
        // keys of this implementation
        hints_.overlap_rows = static_cast<int32_t>(args.value("overlap_rows", static_cast<long>(hints_.overlap_rows)));
        hints_.class_lanes = static_cast<int32_t>(args.value("class_lanes", static_cast<long>(hints_.class_lanes)));
        hints_.warps_x = static_cast<int32_t>(args.value("warps_x", 0L));
        hints_.warps_y = static_cast<int32_t>(args.value("warps_y", 0L));
        hints_.row_slices = static_cast<int32_t>(args.value("row_slices", 0L));
        hints_.reproducible = static_cast<int32_t>(args.value("reproducible", 0L));
        const std::string comb = args.value("combine", std::string("auto"));
        if (comb == "auto") hints_.combine = XCORR_COMBINE_AUTO;
        else if (comb == "store") hints_.combine = XCORR_COMBINE_STORE;
        else if (comb == "atomic") hints_.combine = XCORR_COMBINE_ATOMIC;
        else if (comb == "workspace") hints_.combine = XCORR_COMBINE_WORKSPACE;
        else throw argument_error("Unknown combine mode \"" + comb + "\"", "combine");
        break;
    }
    default:
        break;
    }
    measurements_.resize(measurement_labels().size());
}

algorithm::~algorithm() {
    try { free(); } catch (...) {}
}

std::vector<std::string> algorithm::measurement_labels() const {
    if (measure_common()) return {"Load", "Prepare", "Transfer", "Run", "Finalize", "Free", "Store"};
    if (measure_alg() && on_gpu()) return {"Kernel"};
    return {};
}

void algorithm::reset_measurements() {
    std::fill(measurements_.begin(), measurements_.end(), measurement_result{});
}

uint32_t algorithm::rights_per_left() const {
    switch (spec_.mode) {
    case XCORR_N_TO_MN: return right_.num_matrices() / left_.num_matrices();
    default: return right_.num_matrices();
    }
}

void algorithm::sync_all_devices() {
    if (!on_gpu()) return;
    for (const auto& s : shards_) {
        CUCH(cudaSetDevice(s.device));
        CUCH(cudaDeviceSynchronize());
        CUCH(cudaGetLastError());
    }
}

template<typename F>
void algorithm::timed_step(std::size_t label, bool sync_gpu, F&& step) {
    if (!measure_common()) {
        step();
        return;
    }
    auto t0 = wall_clock::now();
    step();
    if (sync_gpu) sync_all_devices();
    measurements_[label] = measurement_result{elapsed_ns(t0), 1};
}

// ---- load ---------------------------------------------------------------------------------
void algorithm::load(const std::filesystem::path& ref_path, const std::filesystem::path& target_path) {
    timed_step(0, false, [&] {
        const bool pinned = on_gpu();
        left_ = matrix_array::load_csv(ref_path, pinned);
        // GPU n_to_mn algorithms hold the right matrices grouped per left matrix
        // (n_to_mn.hpp:165-172); the CPU algorithm keeps file order (n_to_mn.hpp:95-100).
        const dsize_t group = (spec_.mode == XCORR_N_TO_MN && on_gpu()) ? left_.num_matrices() : 0;
        right_ = matrix_array::load_csv(target_path, pinned, group);
        if (left_.rows() != right_.rows() || left_.cols() != right_.cols())   // cross_corr.hpp:121-130
            throw std::runtime_error(
                "Invalid input matrix sizes, expected ref and target to be the same size: ref = [" +
                std::to_string(left_.cols()) + "," + std::to_string(left_.rows()) + "] target = [" +
                std::to_string(right_.cols()) + "," + std::to_string(right_.rows()) + "]");
        if (!xcorr_validate_input_size(spec_.mode, left_.rows(), left_.cols(), left_.num_matrices(),
                                       right_.num_matrices())) {
            if (spec_.mode == XCORR_N_TO_MN)                                  // n_to_mn.hpp:58-67
                throw std::runtime_error("Invalid input data counts, " + std::to_string(right_.num_matrices()) +
                                         " is not divisible by " + std::to_string(left_.num_matrices()));
            throw std::runtime_error("Invalid input matrix counts for " + spec_.name + ": " +
                                     std::to_string(left_.num_matrices()) + " left, " +
                                     std::to_string(right_.num_matrices()) + " right");
        }
        if (rows_per_thread_ > 0) {
            const long slices = (static_cast<long>(left_.rows()) + rows_per_thread_ - 1) / rows_per_thread_;
            hints_.row_slices = static_cast<int32_t>(std::max<long>(1, std::min<long>(slices, left_.rows())));
        }
    });
}

// ---- prepare ------------------------------------------------------------------------------
void algorithm::build_shards() {
    shards_.clear();
    const std::size_t in_elems = left_.matrix_elems();
    const std::size_t out_elems = static_cast<std::size_t>(result_.rows()) * result_.cols();
    const uint32_t nl = left_.num_matrices(), nr = right_.num_matrices(), m = rights_per_left();
    const int parts = (spec_.mode == XCORR_ONE_TO_ONE) ? 1 : static_cast<int>(devices_.size());
    const uint32_t units = spec_.mode == XCORR_ONE_TO_MANY ? nr : nl;
    for (int i = 0; i < parts; ++i) {
        uint32_t first = 0, count = 0;
        xcorr_shard_range(units, parts, i, &first, &count);
        if (parts == 1) { first = 0; count = units; }
        if (count == 0) continue;
        shard s;
        s.device = devices_[i];
        if (spec_.mode == XCORR_ONE_TO_ONE) {
            s.n_left = 1; s.n_right = 1;
        } else if (spec_.mode == XCORR_ONE_TO_MANY) {       // a block of right matrices, left replicated
            s.n_left = 1; s.n_right = count;
            s.right_offset = first * in_elems;
            s.out_offset = first * out_elems;
        } else if (spec_.mode == XCORR_N_TO_M) {            // a block of left matrices, rights replicated
            s.n_left = count; s.n_right = nr;
            s.left_offset = first * in_elems;
            s.out_offset = static_cast<std::size_t>(first) * m * out_elems;
        } else {                                             // n_to_mn: left matrices with their own rights
            s.n_left = count; s.n_right = count * m;
            s.left_offset = first * in_elems;
            s.right_offset = static_cast<std::size_t>(first) * m * in_elems;
            s.out_offset = static_cast<std::size_t>(first) * m * out_elems;
        }
        s.left_elems = s.n_left * in_elems;
        s.right_elems = s.n_right * in_elems;
        s.out_elems = xcorr_num_results(spec_.mode, s.n_left, s.n_right) * out_elems;
        shards_.push_back(s);
    }
}

void algorithm::prepare() {
    timed_step(1, false, [&] {
        const uint64_t n_out = xcorr_num_results(spec_.mode, left_.num_matrices(), right_.num_matrices());
        // FFT algorithms without --normalize hold the inverse transforms as they are: 2H x 2W,
        // circular shifts, unnormalised (one_to_one.hpp:930, fft_alg.hpp:13-20)
        if (raw_fft())
            result_ = matrix_array(2 * left_.rows(), 2 * left_.cols(), static_cast<dsize_t>(n_out), true);
        else
            result_ = matrix_array(2 * left_.rows() - 1, 2 * left_.cols() - 1, static_cast<dsize_t>(n_out), on_gpu());
        if (!on_gpu() || pipelined()) return;
        build_shards();
        for (auto& s : shards_) {
            CUCH(cudaSetDevice(s.device));
            CUCH(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
            CUCH(cudaEventCreateWithFlags(&s.start, cudaEventBlockingSync));
            CUCH(cudaEventCreateWithFlags(&s.stop, cudaEventBlockingSync));
            CUCH(cudaMalloc(&s.d_left, s.left_elems * sizeof(float)));
            CUCH(cudaMalloc(&s.d_right, s.right_elems * sizeof(float)));
            CUCH(cudaMalloc(&s.d_out, s.out_elems * sizeof(float)));
            s.ws_bytes = raw_fft()
                ? xcorr_fft_workspace_bytes(spec_.mode, left_.rows(), left_.cols(), s.n_left, s.n_right, XCORR_FFT_RAW)
                : xcorr_workspace_bytes(spec_.mode, left_.rows(), left_.cols(), s.n_left, s.n_right, &hints_);
            if (s.ws_bytes) CUCH(cudaMalloc(&s.d_ws, s.ws_bytes));
        }
    });
}

void algorithm::transfer() {
    timed_step(2, true, [&] {
        if (!on_gpu() || pipelined()) return;
        for (auto& s : shards_) {
            CUCH(cudaSetDevice(s.device));
            CUCH(cudaMemcpyAsync(s.d_left, left_.data() + s.left_offset, s.left_elems * sizeof(float),
                                 cudaMemcpyHostToDevice, s.stream));
            CUCH(cudaMemcpyAsync(s.d_right, right_.data() + s.right_offset, s.right_elems * sizeof(float),
                                 cudaMemcpyHostToDevice, s.stream));
        }
        for (auto& s : shards_) {
            CUCH(cudaSetDevice(s.device));
            CUCH(cudaStreamSynchronize(s.stream));
        }
    });
}

// ---- run ----------------------------------------------------------------------------------
void algorithm::launch_all() {
    for (auto& s : shards_) {
        CUCH(cudaSetDevice(s.device));
        if (raw_fft())
            xcorr_check(xcorr_fft_f32(spec_.mode, s.d_left, s.d_right, s.d_out, left_.rows(), left_.cols(),
                                      s.n_left, s.n_right, XCORR_FFT_RAW, s.d_ws, s.ws_bytes, s.stream));
        else
            xcorr_check(xcorr_run_f32(spec_.mode, s.d_left, s.d_right, s.d_out, left_.rows(), left_.cols(),
                                      s.n_left, s.n_right, &hints_, s.d_ws, s.ws_bytes, s.stream));
    }
}

void algorithm::run_cpu() {
    const int H = static_cast<int>(left_.rows()), W = static_cast<int>(left_.cols());
    const uint32_t nl = left_.num_matrices(), nr = right_.num_matrices();
    switch (spec_.mode) {
    case XCORR_ONE_TO_ONE:
        cpu_cross_corr_pair(left_.matrix(0), right_.matrix(0), result_.matrix(0), H, W);
        break;
    case XCORR_ONE_TO_MANY:
        for (uint32_t t = 0; t < nr; ++t) cpu_cross_corr_pair(left_.matrix(0), right_.matrix(t), result_.matrix(t), H, W);
        break;
    case XCORR_N_TO_MN:   // file order: right / result t*n + r pairs with left r (validate.hpp:263-268)
        for (uint32_t r = 0; r < nl; ++r)
            for (uint32_t t = 0; t < nr / nl; ++t)
                cpu_cross_corr_pair(left_.matrix(r), right_.matrix(t * nl + r), result_.matrix(t * nl + r), H, W);
        break;
    default:              // n_to_m: result r*m + t (validate.hpp:284-289)
        for (uint32_t r = 0; r < nl; ++r)
            for (uint32_t t = 0; t < nr; ++t)
                cpu_cross_corr_pair(left_.matrix(r), right_.matrix(t), result_.matrix(r * nr + t), H, W);
    }
}

void algorithm::run() {
    auto once = [&] {
        if (pipelined()) {
            std::vector<int32_t> devs(devices_.begin(), devices_.end());
            xcorr_check(xcorr_run_host_sharded_f32(spec_.mode, left_.data(), right_.data(), result_.data(),
                                                   left_.rows(), left_.cols(), left_.num_matrices(),
                                                   right_.num_matrices(), &hints_, devs.data(),
                                                   static_cast<int32_t>(devs.size())));
        } else if (on_gpu()) {
            launch_all();
        } else {
            run_cpu();
        }
    };
    if (measure_common()) {
        // CPU_ADAPTIVE_MEASURE(3, ..., gpu_sync = true, run_impl) -- cross_corr.hpp:50-54
        std::size_t iterations = 1;
        do {
            auto t0 = wall_clock::now();
            for (std::size_t i = 0; i < iterations; ++i) {
                once();
                sync_all_devices();
            }
            measurements_[3] = measurement_result{elapsed_ns(t0), iterations};
            iterations = next_iteration_count(min_time_ns_, measurements_[3]);
        } while (iterations != 0);
        return;
    }
    if (measure_alg() && on_gpu()) {
        // CUDA_ADAPTIVE_MEASURE(0, ...) -- stopwatch.hpp:125-141: events around `iterations`
        // back-to-back launches, repeated with a growing count until the span >= min_time.
        // With several GPUs every shard is timed on its own device; the slowest one counts.
        std::size_t iterations = 1;
        do {
            for (auto& s : shards_) {
                CUCH(cudaSetDevice(s.device));
                CUCH(cudaEventRecord(s.start, s.stream));
            }
            for (std::size_t i = 0; i < iterations; ++i) launch_all();
            for (auto& s : shards_) {
                CUCH(cudaSetDevice(s.device));
                CUCH(cudaEventRecord(s.stop, s.stream));
            }
            double worst_ms = 0.0;
            for (auto& s : shards_) {
                CUCH(cudaSetDevice(s.device));
                CUCH(cudaEventSynchronize(s.stop));
                float ms = 0.f;
                CUCH(cudaEventElapsedTime(&ms, s.start, s.stop));
                worst_ms = std::max(worst_ms, static_cast<double>(ms));
            }
            measurements_[0] = measurement_result{worst_ms * 1e6, iterations};
            iterations = next_iteration_count(min_time_ns_, measurements_[0]);
        } while (iterations != 0);
        return;
    }
    once();
}

void algorithm::finalize() {
    timed_step(4, true, [&] {
        if (!on_gpu() || pipelined()) return;
        for (auto& s : shards_) {
            CUCH(cudaSetDevice(s.device));
            CUCH(cudaMemcpyAsync(result_.data() + s.out_offset, s.d_out, s.out_elems * sizeof(float),
                                 cudaMemcpyDeviceToHost, s.stream));
        }
        for (auto& s : shards_) {
            CUCH(cudaSetDevice(s.device));
            CUCH(cudaStreamSynchronize(s.stream));
        }
    });
}

void algorithm::free() {
    timed_step(5, false, [&] {
        for (auto& s : shards_) {
            cudaSetDevice(s.device);
            if (s.d_ws) cudaFree(s.d_ws);
            if (s.d_out) cudaFree(s.d_out);
            if (s.d_right) cudaFree(s.d_right);
            if (s.d_left) cudaFree(s.d_left);
            if (s.stop) cudaEventDestroy(s.stop);
            if (s.start) cudaEventDestroy(s.start);
            if (s.stream) cudaStreamDestroy(s.stream);
        }
        shards_.clear();
    });
}

void algorithm::store_results(const std::filesystem::path& out_path) {
    timed_step(6, false, [&] {
        // GPU n_to_mn results are grouped per left matrix; the file gets the reference's
        // order back (store_interleaved_to_csv, n_to_mn.hpp:291-295).
        const dsize_t groups = (spec_.mode == XCORR_N_TO_MN && on_gpu()) ? rights_per_left() : 0;
        result_.store_csv(out_path, groups);
    });
}

// ---- validate -----------------------------------------------------------------------------
// fft_helpers.hpp:213-262 normalize_fft_results: swap the quadrants, drop the unused row and
// column at rows/2 and cols/2, divide by the number of elements of the transform.
matrix_array normalize_fft_results(const matrix_array& raw) {
    const dsize_t RH = raw.rows(), RW = raw.cols();
    matrix_array norm(RH - 1, RW - 1, raw.num_matrices(), false);
    const dsize_t ey = RH / 2, ex = RW / 2;
    const float area = static_cast<float>(RH) * static_cast<float>(RW);
    for (dsize_t i = 0; i < raw.num_matrices(); ++i) {
        const float* src = raw.matrix(i);
        float* dst = norm.matrix(i);
        auto copy = [&](dsize_t sx, dsize_t sy, dsize_t w, dsize_t h, dsize_t tx, dsize_t ty) {
            for (dsize_t y = 0; y < h; ++y)
                for (dsize_t x = 0; x < w; ++x)
                    dst[static_cast<std::size_t>(ty + y) * (RW - 1) + tx + x] =
                        src[static_cast<std::size_t>(sy + y) * RW + sx + x] / area;
        };
        copy(0, 0, ex, ey, (RW - 1) / 2, (RH - 1) / 2);                        // top left -> bottom right
        copy(ex + 1, 0, RW - ex - 1, ey, 0, (RH - 1) / 2);                     // top right -> bottom left
        copy(0, ey + 1, ex, RH - ey - 1, (RW - 1) / 2, 0);                     // bottom left -> top right
        copy(ex + 1, ey + 1, RW - ex - 1, RH - ey - 1, 0, 0);                  // bottom right -> top left
    }
    return norm;
}

validation_results algorithm::validate(const std::optional<std::filesystem::path>& valid_path) const {
    if (raw_fft()) {
        // compare in the normalised layout, like `cross validate --normalize` (main.cpp:74-76)
        const matrix_array norm = normalize_fft_results(result_);
        return validate_against(norm, valid_path);
    }
    return validate_against(result_, valid_path);
}

validation_results algorithm::validate_against(const matrix_array& result_,
                                               const std::optional<std::filesystem::path>& valid_path) const {
    const bool grouped = spec_.mode == XCORR_N_TO_MN && on_gpu();
    if (valid_path.has_value()) {
        matrix_array valid = matrix_array::load_csv(*valid_path, false, grouped ? left_.num_matrices() : 0);
        if (valid.rows() != result_.rows() || valid.cols() != result_.cols() ||
            valid.num_matrices() != result_.num_matrices())
            throw std::runtime_error("Cannot validate matrices of different sizes");
        return validate_result<float>(result_.data(), valid.data(), result_.size());
    }
    // recompute on the CPU, in the memory order of the results
    const int H = static_cast<int>(left_.rows()), W = static_cast<int>(left_.cols());
    const uint32_t nl = left_.num_matrices(), nr = right_.num_matrices();
    matrix_array valid(result_.rows(), result_.cols(), result_.num_matrices(), false);
    switch (spec_.mode) {
    case XCORR_ONE_TO_ONE:
        cpu_cross_corr_pair(left_.matrix(0), right_.matrix(0), valid.matrix(0), H, W);
        break;
    case XCORR_ONE_TO_MANY:
        for (uint32_t t = 0; t < nr; ++t) cpu_cross_corr_pair(left_.matrix(0), right_.matrix(t), valid.matrix(t), H, W);
        break;
    case XCORR_N_TO_MN: {
        const uint32_t m = nr / nl;
        for (uint32_t r = 0; r < nl; ++r)
            for (uint32_t t = 0; t < m; ++t) {
                const uint32_t idx = grouped ? r * m + t : t * nl + r;
                cpu_cross_corr_pair(left_.matrix(r), right_.matrix(idx), valid.matrix(idx), H, W);
            }
        break;
    }
    default:
        for (uint32_t r = 0; r < nl; ++r)
            for (uint32_t t = 0; t < nr; ++t)
                cpu_cross_corr_pair(left_.matrix(r), right_.matrix(t), valid.matrix(r * nr + t), H, W);
    }
    return validate_result<float>(result_.data(), valid.data(), result_.size());
}

}  // namespace cross
