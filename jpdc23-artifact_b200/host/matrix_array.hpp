// Stack of equally sized matrices (float, or double for --data_type double) plus the reference's
// text format.
//
// Counterpart of data_array<T, ALLOC> and impl::csv (repo/cross-corr/src/matrix.hpp:93-187,
// :410-619) with the pinned host allocation of allocator.cuh:16-48.
//
// File format (matrix.hpp:94-185): first line "# <rows>,<cols>[,<count>]", then count*rows
// lines of <cols> comma-separated decimals.  The writer prints std::fixed values (six
// decimals), as the reference does.  One deliberate difference: the reference's writer
// strides rows by the row COUNT (matrix.hpp:180), which is wrong for non-square matrices;
// this writer strides by the column count.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iomanip>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace cross {

using dsize_t = std::uint32_t;

// Host buffer: page-locked when a CUDA device is there (fast H2D/D2H), plain otherwise.
template<typename T>
class basic_host_buffer {
public:
    basic_host_buffer() = default;
    explicit basic_host_buffer(std::size_t count, bool pinned) { allocate(count, pinned); }
    basic_host_buffer(const basic_host_buffer&) = delete;
    basic_host_buffer& operator=(const basic_host_buffer&) = delete;
    basic_host_buffer(basic_host_buffer&& o) noexcept { *this = std::move(o); }
    basic_host_buffer& operator=(basic_host_buffer&& o) noexcept {
        if (this != &o) {
            release();
            data_ = o.data_; count_ = o.count_; pinned_ = o.pinned_;
            o.data_ = nullptr; o.count_ = 0; o.pinned_ = false;
        }
        return *this;
    }
    ~basic_host_buffer() { release(); }

    T* data() { return data_; }
    const T* data() const { return data_; }
    std::size_t size() const { return count_; }

private:
    T* data_ = nullptr;
    std::size_t count_ = 0;
    bool pinned_ = false;

    void allocate(std::size_t count, bool pinned) {
        count_ = count;
        if (count == 0) return;
        if (pinned) {
            void* p = nullptr;
            if (cudaHostAlloc(&p, count * sizeof(T), cudaHostAllocDefault) == cudaSuccess) {
                data_ = static_cast<T*>(p);
                pinned_ = true;
                std::memset(data_, 0, count * sizeof(T));
                return;
            }
            (void)cudaGetLastError();  // no device / no pinned memory: fall through to malloc
        }
        data_ = static_cast<T*>(std::calloc(count, sizeof(T)));
        if (!data_) throw std::bad_alloc();
    }

    void release() {
        if (!data_) return;
        if (pinned_) cudaFreeHost(data_); else std::free(data_);
        data_ = nullptr;
    }
};
using host_buffer = basic_host_buffer<float>;

template<typename T>
class basic_matrix_array {
public:
    basic_matrix_array() = default;
    basic_matrix_array(dsize_t rows, dsize_t cols, dsize_t count, bool pinned)
        : rows_(rows), cols_(cols), count_(count),
          data_(static_cast<std::size_t>(rows) * cols * count, pinned) {}

    dsize_t rows() const { return rows_; }
    dsize_t cols() const { return cols_; }
    dsize_t num_matrices() const { return count_; }
    std::size_t matrix_elems() const { return static_cast<std::size_t>(rows_) * cols_; }
    std::size_t size() const { return data_.size(); }
    T* data() { return data_.data(); }
    const T* data() const { return data_.data(); }
    T* matrix(dsize_t i) { return data_.data() + matrix_elems() * i; }
    const T* matrix(dsize_t i) const { return data_.data() + matrix_elems() * i; }

    // matrix.hpp:614-618: file index i of a file holding num_groups groups of group_size
    // matrices goes to slot (i % group_size) * num_groups + i / group_size.
    static dsize_t interleaved_index(dsize_t i, dsize_t group_size, dsize_t num_groups) {
        return (i % group_size) * num_groups + i / group_size;
    }

    // Binary matrix files (extension .bin), next to the text format: the loader the reference
    // sketches and leaves unimplemented (matrix.hpp:49-91; width then height as 32-bit
    // little-endian words).  Layout: the 8 bytes "XCORRMAT", cols, rows, count as uint32
    // little-endian, then count * rows * cols float32 little-endian, matrices in file order.
    // Parsing tens of MB of decimal text dominates the wall time of a run on the benchmark
    // inputs; this format loads at memory speed.
    static bool is_binary_path(const std::filesystem::path& path) { return path.extension() == ".bin"; }

    static basic_matrix_array load_binary(const std::filesystem::path& path, bool pinned, dsize_t group_size) {
        if constexpr (sizeof(T) != sizeof(float)) throw std::runtime_error("binary matrix files hold float32; use text files with --data_type double");
        std::ifstream in(path, std::ios::binary);
        if (!in) throw std::runtime_error("Could not open file " + path.string());
        char magic[8];
        uint32_t hdr[3];
        if (!in.read(magic, 8) || std::string(magic, 8) != "XCORRMAT" || !in.read(reinterpret_cast<char*>(hdr), 12))
            throw std::runtime_error("Invalid input file format");
        if (!little_endian()) for (auto& v : hdr) v = byte_swap(v);
        const dsize_t cols = hdr[0], rows = hdr[1], count = hdr[2];
        if (rows == 0 || cols == 0 || count == 0) throw std::runtime_error("Invalid input file format");
        if (group_size != 0 && count % group_size != 0)
            throw std::runtime_error("Data array cannot be interleaved, as number of matrices is not divisible by group size");
        basic_matrix_array a(rows, cols, count, pinned);
        const dsize_t num_groups = group_size ? count / group_size : 0;
        const std::size_t mat_bytes = a.matrix_elems() * sizeof(float);
        for (dsize_t i = 0; i < count; ++i) {
            T* dst = a.matrix(group_size ? interleaved_index(i, group_size, num_groups) : i);
            if (!in.read(reinterpret_cast<char*>(dst), static_cast<std::streamsize>(mat_bytes)))
                throw std::runtime_error("Invalid input file format: file ends inside matrix " + std::to_string(i));
            if (!little_endian())
                for (std::size_t e = 0; e < a.matrix_elems(); ++e) {
                    uint32_t w;
                    std::memcpy(&w, dst + e, 4);
                    w = byte_swap(w);
                    std::memcpy(dst + e, &w, 4);
                }
        }
        return a;
    }

    void store_binary(const std::filesystem::path& path, dsize_t num_groups) const {
        if constexpr (sizeof(T) != sizeof(float)) throw std::runtime_error("binary matrix files hold float32; use text files with --data_type double");
        std::ofstream out(path, std::ios::binary);
        if (!out) throw std::runtime_error("Could not open file " + path.string() + " for writing");
        if (num_groups != 0 && count_ % num_groups != 0)
            throw std::runtime_error("Data array cannot be interleaved, as number of matrices is not divisible by group size");
        uint32_t hdr[3] = {cols_, rows_, count_};
        if (!little_endian()) for (auto& v : hdr) v = byte_swap(v);
        out.write("XCORRMAT", 8);
        out.write(reinterpret_cast<const char*>(hdr), 12);
        const dsize_t group_size = num_groups ? count_ / num_groups : 0;
        std::vector<uint32_t> swapped;
        for (dsize_t i = 0; i < count_; ++i) {
            const T* src = matrix(num_groups ? interleaved_index(i, group_size, num_groups) : i);
            if (little_endian()) {
                out.write(reinterpret_cast<const char*>(src), static_cast<std::streamsize>(matrix_elems() * sizeof(float)));
            } else {
                swapped.resize(matrix_elems());
                std::memcpy(swapped.data(), src, matrix_elems() * 4);
                for (auto& w : swapped) w = byte_swap(w);
                out.write(reinterpret_cast<const char*>(swapped.data()), static_cast<std::streamsize>(matrix_elems() * 4));
            }
        }
        if (!out) throw std::runtime_error("Could not write file " + path.string());
    }

    // group_size == 0: file order (load_from_csv, matrix.hpp:437-450); otherwise the
    // grouped order of load_interleaved_from_csv (matrix.hpp:471-503).  A path ending in .bin
    // is read as a binary matrix file.
    static basic_matrix_array load_csv(const std::filesystem::path& path, bool pinned, dsize_t group_size = 0) {
        if (is_binary_path(path)) return load_binary(path, pinned, group_size);
        std::ifstream in(path);
        if (!in) throw std::runtime_error("Could not open file " + path.string());
        dsize_t rows = 0, cols = 0, count = 1;
        read_header(in, rows, cols, count);
        if (group_size != 0 && count % group_size != 0)
            throw std::runtime_error("Data array cannot be interleaved, as number of matrices is not divisible by group size");
        basic_matrix_array a(rows, cols, count, pinned);
        const dsize_t num_groups = group_size ? count / group_size : 0;
        std::string line;
        for (dsize_t i = 0; i < count; ++i) {
            T* dst = a.matrix(group_size ? interleaved_index(i, group_size, num_groups) : i);
            for (dsize_t y = 0; y < rows; ++y) {
                if (!std::getline(in, line))
                    throw std::runtime_error("Failed to read line " + std::to_string(y) + " from csv file");
                parse_row(line, y, cols, dst + static_cast<std::size_t>(y) * cols);
            }
        }
        return a;
    }

    // num_groups == 0: memory order (store_to_csv, matrix.hpp:505-511); otherwise undo the
    // grouping of a load with group_size = count / num_groups... the reference passes the
    // number of groups of the ORIGINAL load, i.e. its group_size (matrix.hpp:523-539).
    void store_csv(const std::filesystem::path& path, dsize_t num_groups = 0) const {
        if (is_binary_path(path)) { store_binary(path, num_groups); return; }
        std::ofstream out(path);
        if (!out) throw std::runtime_error("Could not open file " + path.string() + " for writing");
        if (num_groups != 0 && count_ % num_groups != 0)
            throw std::runtime_error("Data array cannot be interleaved, as number of matrices is not divisible by group size");
        out << "# " << rows_ << "," << cols_ << "," << count_ << "\n";
        out << std::fixed;
        const dsize_t group_size = num_groups ? count_ / num_groups : 0;
        for (dsize_t i = 0; i < count_; ++i) {
            const T* src = matrix(num_groups ? interleaved_index(i, group_size, num_groups) : i);
            for (dsize_t y = 0; y < rows_; ++y) {
                const char* sep = "";
                for (dsize_t x = 0; x < cols_; ++x) {
                    out << sep << src[static_cast<std::size_t>(y) * cols_ + x];
                    sep = ",";
                }
                out << "\n";
            }
        }
    }

private:
    dsize_t rows_ = 0, cols_ = 0, count_ = 0;
    basic_host_buffer<T> data_;

    static bool little_endian() {
        const uint32_t one = 1;
        unsigned char b;
        std::memcpy(&b, &one, 1);
        return b == 1;
    }
    static uint32_t byte_swap(uint32_t v) {
        return (v >> 24) | ((v >> 8) & 0xff00u) | ((v << 8) & 0xff0000u) | (v << 24);
    }

    static void read_header(std::istream& in, dsize_t& rows, dsize_t& cols, dsize_t& count) {
        std::string line;
        if (!std::getline(in, line)) throw std::runtime_error("Could not read file header");
        if (line.compare(0, 2, "# ") != 0) throw std::runtime_error("Invalid file header format");
        std::vector<std::string> tok = split(line.substr(2));
        if (tok.empty() || tok[0].empty()) throw std::runtime_error("Missing matrix header");
        rows = static_cast<dsize_t>(std::stoi(tok[0]));
        if (tok.size() < 2) throw std::runtime_error("Missing number of columns");
        cols = static_cast<dsize_t>(std::stoi(tok[1]));
        count = 1;
        if (tok.size() >= 3) count = static_cast<dsize_t>(std::stoi(tok[2]));
        if (tok.size() > 3) throw std::runtime_error("Invalid matrix header format, too many tokens");
    }

    static std::vector<std::string> split(const std::string& text) {
        std::vector<std::string> out;
        if (text.empty()) return out;
        std::size_t start = 0;
        while (true) {
            std::size_t comma = text.find(',', start);
            if (comma == std::string::npos) { out.push_back(text.substr(start)); break; }
            out.push_back(text.substr(start, comma - start));
            start = comma + 1;
        }
        return out;
    }

    // One text row -> `cols` floats; too long / too short rows throw (matrix.hpp:146-153).
    static void parse_row(const std::string& line, dsize_t y, dsize_t cols, T* dst) {
        const char* p = line.c_str();
        dsize_t x = 0;
        while (*p != '\0' && *p != '\r') {
            if (x == cols)
                throw std::runtime_error("Line " + std::to_string(y) + " is too long, expected " + std::to_string(cols) + " values");
            char* end = nullptr;
            if constexpr (sizeof(T) == sizeof(double)) dst[x] = std::strtod(p, &end); else dst[x] = std::strtof(p, &end);
            if (end == p) throw std::invalid_argument("stof");
            ++x;
            p = end;
            while (*p == ' ') ++p;
            if (*p == ',') ++p;
        }
        if (x != cols)
            throw std::runtime_error("Line" + std::to_string(y) + " is too short, expected " + std::to_string(cols) +
                                     ", got " + std::to_string(x) + " values");
    }
};
using matrix_array = basic_matrix_array<float>;

}  // namespace cross
