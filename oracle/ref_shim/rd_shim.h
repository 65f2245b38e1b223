/* Force-included (-include) when compiling the reference's text_gen.cpp, and
 * nothing else. TEST INFRASTRUCTURE ONLY.
 *
 * The reference sampler draws from a function-static std::mt19937 seeded from
 * std::random_device (src/transformer/text_gen.cpp:195-197), so it cannot be
 * seeded through its API. This header swaps the seed source for one that
 * returns the value of the GRADREF_SEED environment variable (default 0),
 * leaving every line of the reference source untouched. */
#pragma once
#include <cstdlib>
#include <random>

namespace std {
class oracle_random_device {
public:
    using result_type = unsigned int;
    result_type operator()() {
        const char* s = std::getenv("GRADREF_SEED");
        return s ? static_cast<result_type>(std::strtoul(s, nullptr, 10)) : 0u;
    }
    static constexpr result_type min() { return 0; }
    static constexpr result_type max() { return 0xFFFFFFFFu; }
};
}  // namespace std

#define random_device oracle_random_device
