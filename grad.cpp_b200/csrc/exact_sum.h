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
GRADB_HD IncPair term_inc(uint32_t bits, int ue) {
    IncPair r;
    r.e = r.o = 0u;
    if ((bits & 0x7fffffffu) == 0u) return r;
    int ex = (int)((bits >> 23) & 0xffu);
    uint32_t man = bits & 0x7fffffu;
    if (ex == 0) ex = 1; else man |= 0x800000u;  // subnormals carry no hidden bit
    const int shift = ue - (ex - 150);           // a / u = man * 2^-shift
    if (shift <= 0) {                            // a >= 2^23 u: certainly leaves the binade
        r.e = r.o = kBinadeEnd;
        return r;
    }
    if (shift > 25) return r;                    // a < u/4: no effect
    const uint32_t q = shift >= 25 ? 0u : (man >> shift);
    const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half) {
        r.e = r.o = q + 1u;
    } else if (rem < half) {
        r.e = r.o = q;
    } else {
        r.e = q + (q & 1u);         // S even: S + q has q's parity
        r.o = q + ((q + 1u) & 1u);  // S odd
    }
    return r;
}

GRADB_HD uint32_t step_S(uint32_t S, IncPair t) { return S + ((S & 1u) ? t.o : t.e); }

}  // namespace gradb
