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
// run of such terms simply add up. In floating point: a / u is exact (u is a power of two; a product that underflows
// is far below one half either way), adding and subtracting 2^23 rounds it to the nearest integer for a / u < 2^22,
// and the distance to that integer tells a tie. Returns the increment as a float (an integer below 2^22: four of them
// add up exactly); *slow is set for a tie, a term of 2^22 units or more, an infinity or a NaN — the caller then
// composes the run's maps with term_inc, which covers every case. inv_u = 1 / u.
GRADB_HD float term_inc_float(float a, float inv_u, uint32_t* slow) {
#if defined(__CUDA_ARCH__)
    const float t = __fmul_rn(a, inv_u);
    const float r = __fadd_rn(__fadd_rn(t, 8388608.0f), -8388608.0f);
    const float d = __fadd_rn(t, -r);
#else
    volatile float tv = a * inv_u;  // (volatile: the host compiler must not fold the rounding away)
    const float t = tv;
    volatile float up = t + 8388608.0f;
    const float r = up - 8388608.0f;
    const float d = t - r;
#endif
    *slow |= (!(t < 4194304.0f) || d == 0.5f || d == -0.5f) ? 1u : 0u;
    return r;
}
GRADB_HD float unit_reciprocal(int ue) {  // 1 / 2^ue for -127 < ue < 127
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)(127 - ue) << 23;
    return v.f;
}

}  // namespace gradb
