// Minimal stand-in for the Boost.Accumulators subset used by the reference's
// validate.hpp: accumulator_set<double, stats<tag::max, tag::mean, tag::variance(lazy)>>,
// called once per sample, then max(acc), mean(acc), variance(acc).  Lazy variance in
// Boost is mean(x^2) - mean(x)^2; the same formula is used here.
#pragma once
#include <cstddef>
#include <limits>

namespace boost { namespace accumulators {

// `tag::variance(lazy)` in the reference is a function TYPE built from two class types.
struct lazy {};

namespace tag {
    struct max {};
    struct mean {};
    struct variance {};
}

template<typename... FEATURES>
struct stats {};

template<typename SAMPLE, typename STATS>
class accumulator_set {
public:
    void operator()(SAMPLE v) {
        if (n_ == 0 || v > max_) max_ = v;
        sum_ += v;
        sum_sq_ += v * v;
        ++n_;
    }
    SAMPLE get_max() const { return n_ ? max_ : -std::numeric_limits<SAMPLE>::infinity(); }
    SAMPLE get_mean() const { return sum_ / static_cast<SAMPLE>(n_); }
    SAMPLE get_variance() const {
        SAMPLE m = get_mean();
        return sum_sq_ / static_cast<SAMPLE>(n_) - m * m;
    }
private:
    std::size_t n_ = 0;
    SAMPLE max_ = 0;
    SAMPLE sum_ = 0;
    SAMPLE sum_sq_ = 0;
};

template<typename ACC> auto max(const ACC& a) { return a.get_max(); }
template<typename ACC> auto mean(const ACC& a) { return a.get_mean(); }
template<typename ACC> auto variance(const ACC& a) { return a.get_variance(); }

}}
