// Minimal JSON reader for algorithm-argument files (`cross run --args_path file.json`).
// The reference reads these with nlohmann::json and `args.value(key, default)`
// (e.g. one_to_one.hpp:739-741): a flat object of numbers, booleans and strings; unknown
// keys are ignored, missing keys take the default.  Nested arrays/objects are parsed and
// skipped.  Throws std::runtime_error on malformed input.
#pragma once
#include <cctype>
#include <cstdlib>
#include <istream>
#include <iterator>
#include <map>
#include <stdexcept>
#include <string>

namespace cross {

class json_object {
public:
    enum class kind { number, boolean, string, null, other };
    struct entry {
        kind k = kind::null;
        double number = 0;
        bool boolean = false;
        std::string text;
    };

    static json_object parse(std::istream& in) {
        std::string text((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        json_object obj;
        std::size_t pos = 0;
        obj.skip_ws(text, pos);
        if (pos >= text.size()) return obj;            // empty file = empty object
        if (text[pos] != '{') throw std::runtime_error("JSON arguments must be an object");
        obj.parse_object(text, pos, true);
        return obj;
    }

    bool contains(const std::string& key) const { return values_.count(key) != 0; }

    long value(const std::string& key, long fallback) const {
        auto it = values_.find(key);
        if (it == values_.end()) return fallback;
        if (it->second.k == kind::number) return static_cast<long>(it->second.number);
        if (it->second.k == kind::boolean) return it->second.boolean ? 1 : 0;
        throw std::runtime_error("JSON key \"" + key + "\" is not a number");
    }

    bool value(const std::string& key, bool fallback) const {
        auto it = values_.find(key);
        if (it == values_.end()) return fallback;
        if (it->second.k == kind::boolean) return it->second.boolean;
        if (it->second.k == kind::number) return it->second.number != 0;
        throw std::runtime_error("JSON key \"" + key + "\" is not a boolean");
    }

    std::string value(const std::string& key, const std::string& fallback) const {
        auto it = values_.find(key);
        if (it == values_.end()) return fallback;
        if (it->second.k == kind::string) return it->second.text;
        throw std::runtime_error("JSON key \"" + key + "\" is not a string");
    }

private:
    std::map<std::string, entry> values_;

    static void skip_ws(const std::string& t, std::size_t& p) {
        while (p < t.size() && std::isspace(static_cast<unsigned char>(t[p]))) ++p;
    }

    static std::string parse_string(const std::string& t, std::size_t& p) {
        if (t[p] != '"') throw std::runtime_error("JSON: expected a string");
        ++p;
        std::string out;
        while (p < t.size() && t[p] != '"') {
            if (t[p] == '\\' && p + 1 < t.size()) {
                ++p;
                switch (t[p]) {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'u': p += 4; out += '?'; break;
                default: out += t[p];
                }
            } else {
                out += t[p];
            }
            ++p;
        }
        if (p >= t.size()) throw std::runtime_error("JSON: unterminated string");
        ++p;
        return out;
    }

    entry parse_value(const std::string& t, std::size_t& p) {
        skip_ws(t, p);
        if (p >= t.size()) throw std::runtime_error("JSON: unexpected end");
        entry e;
        const char c = t[p];
        if (c == '"') {
            e.k = kind::string;
            e.text = parse_string(t, p);
        } else if (c == '{') {
            e.k = kind::other;
            parse_object(t, p, false);
        } else if (c == '[') {
            e.k = kind::other;
            ++p;
            skip_ws(t, p);
            if (p < t.size() && t[p] == ']') { ++p; return e; }
            while (true) {
                parse_value(t, p);
                skip_ws(t, p);
                if (p < t.size() && t[p] == ',') { ++p; continue; }
                if (p < t.size() && t[p] == ']') { ++p; break; }
                throw std::runtime_error("JSON: malformed array");
            }
        } else if (t.compare(p, 4, "true") == 0) {
            e.k = kind::boolean; e.boolean = true; p += 4;
        } else if (t.compare(p, 5, "false") == 0) {
            e.k = kind::boolean; e.boolean = false; p += 5;
        } else if (t.compare(p, 4, "null") == 0) {
            e.k = kind::null; p += 4;
        } else {
            char* end = nullptr;
            e.number = std::strtod(t.c_str() + p, &end);
            if (end == t.c_str() + p) throw std::runtime_error("JSON: unexpected character");
            e.k = kind::number;
            p = static_cast<std::size_t>(end - t.c_str());
        }
        return e;
    }

    void parse_object(const std::string& t, std::size_t& p, bool keep) {
        ++p;  // '{'
        skip_ws(t, p);
        if (p < t.size() && t[p] == '}') { ++p; return; }
        while (true) {
            skip_ws(t, p);
            if (p >= t.size()) throw std::runtime_error("JSON: unterminated object");
            std::string key = parse_string(t, p);
            skip_ws(t, p);
            if (p >= t.size() || t[p] != ':') throw std::runtime_error("JSON: expected ':'");
            ++p;
            entry e = parse_value(t, p);
            if (keep) values_[key] = e;
            skip_ws(t, p);
            if (p < t.size() && t[p] == ',') { ++p; continue; }
            if (p < t.size() && t[p] == '}') { ++p; break; }
            throw std::runtime_error("JSON: malformed object");
        }
    }
};

}  // namespace cross
