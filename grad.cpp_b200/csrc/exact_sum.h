// Building blocks for reproducing a sequential fp32 sum of non-negative terms
// with a parallel scan. Plain C++ so that host tests can exercise the same code
// the kernels use.
//
// While a running sum s stays inside one binade [2^e, 2^(e+1)) it is an integer
// multiple S of u = 2^(e-23), and fl(s + a) = (S + inc) * u where inc is a/u
// rounded to nearest, ties going to whichever neighbour makes S + inc even.
// Only a tie consults the running sum, and only its parity, so every term acts
// as a map (parity of S) -> increment; such maps compose associatively.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define GRADB_HD __host__ __device__ __forceinline__
#else
#define GRADB_HD inline
#endif

namespace gradb {

constexpr uint32_t kBinadeEnd = 0x01000000u;  // S reaching 2^24 means the sum left the binade

struct IncPair {  // increment when the incoming S is even / odd
    uint32_t e, o;
};

GRADB_HD uint32_t sat(uint32_t v) { return v < kBinadeEnd ? v : kBinadeEnd; }

// a then b. Values saturate at kBinadeEnd: past that point the scan is void
// anyway and only "has left the binade" matters.
GRADB_HD IncPair compose(IncPair a, IncPair b) {
    IncPair r;
    r.e = sat(a.e + ((a.e & 1u) ? b.o : b.e));
    r.o = sat(a.o + (((a.o + 1u) & 1u) ? b.o : b.e));
    return r;
}

// Increments of one term with bit pattern `bits` (a >= 0, finite) when the
// unit is u = 2^ue, i.e. the running sum has biased exponent ue + 150.
// Branch free: a = man * 2^(ex-150), so a/u = man >> shift with shift = ue - (ex - 150);
// a shift above 25 leaves less than a quarter ulp (no effect), a shift of zero or less means
// a >= 2^23 u, which certainly lifts the sum out of the binade.
GRADB_HD IncPair term_inc(uint32_t bits, int ue) {
    const uint32_t exf = (bits >> 23) & 0xffu;
    const uint32_t man = (bits & 0x7fffffu) | (exf ? 0x800000u : 0u);  // subnormals carry no hidden bit
    const int ex = exf ? (int)exf : 1;
    const int shift = ue - (ex - 150);
    const int sh = shift < 1 ? 1 : (shift > 26 ? 26 : shift);
    const uint32_t q = man >> sh;
    const uint32_t rem = man & ((1u << sh) - 1u), half = 1u << (sh - 1);
    const uint32_t up = rem > half ? 1u : 0u, tie = rem == half ? 1u : 0u;
    IncPair r;
    r.e = q + up + (tie & q & 1u);          // S even: S + q has q's parity, a tie rounds to even
    r.o = q + up + (tie & (q + 1u) & 1u);   // S odd
    if (shift <= 0) r.e = r.o = kBinadeEnd;
    return r;
}

GRADB_HD uint32_t step_S(uint32_t S, IncPair t) { return S + ((S & 1u) ? t.o : t.e); }

// The same term when it is not a tie: its increment does not depend on the parity of S, so the increments of a
// run of such terms simply add up (saturating once at the end: each is at most kBinadeEnd). *tie is set when the
// term IS a tie (the returned value is then meaningless and the caller composes the run's maps with term_inc).
GRADB_HD uint32_t term_inc_plain(uint32_t bits, int ue, uint32_t* tie) {
    const uint32_t exf = (bits >> 23) & 0xffu;
    const uint32_t man = (bits & 0x7fffffu) | (exf ? 0x800000u : 0u);
    const int ex = exf ? (int)exf : 1;
    const int shift = ue - (ex - 150);
    const int sh = shift < 1 ? 1 : (shift > 26 ? 26 : shift);
    const uint32_t rem = man & ((1u << sh) - 1u), half = 1u << (sh - 1);
    *tie |= (rem == half && shift > 0) ? 1u : 0u;
    return shift <= 0 ? kBinadeEnd : (man >> sh) + (rem > half ? 1u : 0u);
}

}  // namespace gradb
