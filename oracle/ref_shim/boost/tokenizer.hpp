// Minimal stand-in for the one Boost.Tokenizer use in the reference's matrix.hpp:
// boost::tokenizer<boost::escaped_list_separator<char>> over a line of comma-separated
// numbers, iterated with begin()/end().  Quotes and escapes never occur in matrix files,
// so a plain comma split is enough.  Used only to compile the reference's CPU code into
// the test-side reference library; not part of the shipped library.
#pragma once
#include <string>
#include <string_view>
#include <vector>

namespace boost {

template<typename CH>
struct escaped_list_separator {};

template<typename SEP>
class tokenizer {
public:
    using iterator = std::vector<std::string>::const_iterator;

    explicit tokenizer(std::string_view text) { split(text); }
    explicit tokenizer(const std::string& text) { split(std::string_view(text)); }

    iterator begin() const { return tokens_.begin(); }
    iterator end() const { return tokens_.end(); }

private:
    void split(std::string_view text) {
        if (text.empty()) return;
        std::size_t start = 0;
        while (true) {
            std::size_t comma = text.find(',', start);
            if (comma == std::string_view::npos) {
                tokens_.emplace_back(text.substr(start));
                break;
            }
            tokens_.emplace_back(text.substr(start, comma - start));
            start = comma + 1;
        }
    }
    std::vector<std::string> tokens_;
};

}
