// The selection stage of TextGen on the device: repetition penalty, greedy
// argmax, and sample_from_logits (temperature, top-k, softmax, top-p, draw).
// Reference: src/transformer/text_gen.cpp:14-33, 52-60, 135-209 and
// Tensor::softmax, src/transformer/tensor.cpp:421-452.
//
// The goal is the reference's result bit for bit on identical logits and
// draws, which constrains three things:
//  * exp must return libm's expf bits. The host libm (glibc) implements the
//    published table-driven algorithm (32-entry 2^(i/32) table, cubic
//    polynomial, evaluated in double); expf_libm below restates it with
//    non-contracted IEEE double operations.
//  * the sums the reference accumulates sequentially in fp32 (softmax
//    denominator, top-p running sum in sorted order, kept mass, draw scan) are
//    order dependent. seq_scan below reproduces the sequential result exactly
//    with a block-wide scan: inside one binade the running sum is an integer
//    count of ulps, so "round(a/ulp)" increments compose associatively; the
//    scan restarts whenever the sum enters the next binade.
//  * the quirks are kept: ties at the top-k / top-p thresholds survive, the
//    -1e10 sentinel, cutoff index 0 when the running sum never reaches p,
//    the last id when the draw exceeds the total mass.
#include "select_kernels.cuh"

#include "exact_sum.h"

namespace gradb {

namespace {

constexpr int kSelThreads = 512;  // two CTAs (sequences) per SM: one's serial stretches run under the other's parallel ones
constexpr int kSelWarps = kSelThreads / 32;

// 2^(i/32) as IEEE double bits with i<<47 subtracted, so that adding ki<<47
// both selects the binade and restores the entry (the usual trick of the
// published algorithm).
__constant__ uint64_t c_exp2_tab[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};

// expf with the bits of the host C library's, for finite x <= ~88.
// `tab` = c_exp2_tab copied to shared memory: lanes index it with unrelated values, which the constant cache
// would serve one distinct address at a time.
__device__ __forceinline__ float expf_libm(float x, const uint64_t* tab) {
    if (x < -0x1.9fe368p6f) return 0.0f;     // underflows to zero (also -inf, -1e10 - max)
    // The one input in [-104, 0] where glibc 2.39's FMA-contracted build rounds the other way.
    if (__float_as_uint(x) == 0xc27c65d9u) return 0x1.f45326p-92f;
    if (x != x) return x;
    if (x > 0x1.62e42ep6f) return INFINITY;
    const double InvLn2N = 0x1.71547652b82fep+0 * 32.0;
    const double Shift = 0x1.8p52;
    const double C0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double C1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double C2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double xd = (double)x;
    double z = __dmul_rn(InvLn2N, xd);
    double kd = __dadd_rn(z, Shift);
    const uint64_t ki = (uint64_t)__double_as_longlong(kd);
    kd = __dsub_rn(kd, Shift);
    const double r = __dsub_rn(z, kd);
    const uint64_t t = tab[ki & 31] + (ki << 47);
    const double s = __longlong_as_double((long long)t);
    z = __dadd_rn(__dmul_rn(C0, r), C1);
    const double r2 = __dmul_rn(r, r);
    double y = __dadd_rn(__dmul_rn(C2, r), 1.0);
    y = __dadd_rn(__dmul_rn(z, r2), y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---------------------------------------------------------------------------
// Exact sequential fp32 accumulation of non-negative terms, in parallel.
//
// The reference computes s = fl(s + a[i]) for i = 0, 1, 2, ... While s stays in
// one binade [2^e, 2^(e+1)) it is an integer multiple S of u = 2^(e-23), and
// fl(s + a) = (S + inc) * u with inc = a/u rounded to nearest, ties resolved
// towards an even S + inc. Only a tie looks at the running sum, and only at
// its parity, so each term acts on (S mod 2) as a map parity -> increment, and
// maps compose associatively: a prefix scan gives every running sum. The scan
// is valid up to the first term that lifts the sum out of the binade; that
// term is added natively and the scan restarts in the new binade.
//
// Thread t owns terms [t*per, (t+1)*per). `term(i)` yields a[i]. Stops early
// at the first index whose running sum s satisfies `hit(s)`.
struct ScanResult {
    float sum;   // running sum after the last term consumed
    int hit;     // first index whose running sum satisfied the predicate, or n
};

constexpr int kSerialPrefix = 64;   // terms one thread adds natively before the block-wide passes start
constexpr int kMaxPer = 16;          // terms per thread per pass (register resident)
constexpr int kMaxRange = kMaxPer * kSelThreads;

// One block-wide pass over terms [start, pend) with PER terms per thread. Returns nothing;
// the outcome is left in the shared scan state.
struct ScanShared {
    float sum;
    int next, hit, stop, range;
};

template <int PER, typename Term, typename Hit>
__device__ __forceinline__ void scan_pass(Term& term, Hit& hit, ScanShared* st, IncPair* wtot, int start, int pend,
                                          float s0, int n) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int len = pend - start;
    const int beg = min(pend, start + tid * PER), end = min(pend, beg + PER);
    const uint32_t sb = __float_as_uint(s0);
    const int sex = (int)(sb >> 23);
    const int ue = sex - 150;                          // u = 2^(sex-127-23)
    const uint32_t S0 = (sb & 0x7fffffu) | 0x800000u;  // s0 = S0 * u
    IncPair tinc[PER];
    IncPair loc = {0u, 0u};
#pragma unroll
    for (int i = 0; i < PER; i++) {
        tinc[i].e = tinc[i].o = 0u;
        if (beg + i < end) tinc[i] = term_inc(__float_as_uint(term(beg + i)), ue);
        loc = compose(loc, tinc[i]);
    }
    // inclusive scan of the per-thread maps across the warp, then across warps
    IncPair inc = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        IncPair prev;
        prev.e = __shfl_up_sync(0xffffffffu, inc.e, o);
        prev.o = __shfl_up_sync(0xffffffffu, inc.o, o);
        if (lane >= o) inc = compose(prev, inc);
    }
    if (lane == 31) wtot[w] = inc;
    __syncthreads();
    // scan of the 32 warp totals by every warp (lane i holds warp i's total)
    IncPair wt = lane < kSelWarps ? wtot[lane] : IncPair{0u, 0u};  // identity beyond the last warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        IncPair prev;
        prev.e = __shfl_up_sync(0xffffffffu, wt.e, o);
        prev.o = __shfl_up_sync(0xffffffffu, wt.o, o);
        if (lane >= o) wt = compose(prev, wt);
    }
    IncPair ahead;  // everything before this warp
    ahead.e = __shfl_sync(0xffffffffu, wt.e, (w + 31) & 31);
    ahead.o = __shfl_sync(0xffffffffu, wt.o, (w + 31) & 31);
    if (w == 0) ahead.e = ahead.o = 0u;
    {
        IncPair pl;  // everything before this lane inside the warp
        pl.e = __shfl_up_sync(0xffffffffu, inc.e, 1);
        pl.o = __shfl_up_sync(0xffffffffu, inc.o, 1);
        if (lane == 0) pl.e = pl.o = 0u;
        ahead = compose(ahead, pl);
    }
    // Walk this thread's terms from its now-known starting S.
    uint32_t S = step_S(S0, ahead);
    int my_stop = 0x7fffffff;  // where this thread wants the pass to stop
    int my_kind = 0;           // 1: predicate holds after term my_stop; 2: term my_stop leaves the binade
    if (S < kBinadeEnd) {
#pragma unroll
        for (int i = 0; i < PER; i++) {
            if (my_kind == 0 && beg + i < end) {
                const uint32_t Sn = step_S(S, tinc[i]);
                if (Sn >= kBinadeEnd) {
                    my_stop = beg + i;
                    my_kind = 2;
                } else {
                    S = Sn;
                    if (hit(__uint_as_float(((uint32_t)sex << 23) | (S & 0x7fffffu)))) {
                        my_stop = beg + i;
                        my_kind = 1;
                    }
                }
            }
        }
    }
    if (my_kind != 0) atomicMin(&st->stop, my_stop);
    __syncthreads();
    const int stop = st->stop;
    __syncthreads();
    const float sv = __uint_as_float(((uint32_t)sex << 23) | (S & 0x7fffffu));
    if (stop != 0x7fffffff) {
        if (my_kind != 0 && my_stop == stop) {  // exactly one thread owns that term
            st->stop = 0x7fffffff;
            st->next = stop + 1;
            st->range = max(kSelThreads, min(2 * (stop + 1 - start), kMaxRange));
            if (my_kind == 1) {
                st->hit = stop;
                st->sum = sv;
            } else {
                const float s2 = __fadd_rn(sv, term(stop));  // into the next binade, natively
                st->sum = s2;
                if (hit(s2)) st->hit = stop;
            }
        }
    } else if (end == pend && beg < end) {  // the owner of the pass's last term holds the sum so far
        st->sum = sv;
        st->next = pend;
        st->range = min(2 * len, kMaxRange);
    }
    (void)n;
}

// sh: room for kSelWarps IncPair.
//
// Pass structure: a running sum that starts at zero crosses binades quickly at
// first (1, 2, 4, ... terms apart), so one thread adds the first kSerialPrefix
// terms natively. After that every pass covers an adaptive range (about twice
// what the previous binade consumed, at most kMaxRange terms): each thread keeps
// up to kMaxPer consecutive terms in registers, composes their maps, the block
// scans the per-thread maps, and each thread walks its terms from its now-known
// start looking for the predicate or for the term that leaves the binade.
template <typename Term, typename Hit>
__device__ ScanResult seq_scan(int n, Term term, Hit hit, uint32_t* sh) {
    __shared__ ScanShared st;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    IncPair* wtot = reinterpret_cast<IncPair*>(sh);
    if (tid == 0) {
        float s = 0.0f;
        int i = 0, h = n;
        const int stop = min(n, kSerialPrefix);
        while (i + 4 <= stop && h == n) {  // loads of a group are issued together, adds stay in order
            const float a0 = term(i), a1 = term(i + 1), a2 = term(i + 2), a3 = term(i + 3);
            const float s1 = __fadd_rn(s, a0), s2 = __fadd_rn(s1, a1), s3 = __fadd_rn(s2, a2), s4 = __fadd_rn(s3, a3);
            if (hit(s4)) {  // monotone predicate: the first hit is somewhere in this group
                if (hit(s1)) { h = i; s = s1; i += 1; }
                else if (hit(s2)) { h = i + 1; s = s2; i += 2; }
                else if (hit(s3)) { h = i + 2; s = s3; i += 3; }
                else { h = i + 3; s = s4; i += 4; }
            } else {
                s = s4;
                i += 4;
            }
        }
        while (i < stop && h == n) {
            s = __fadd_rn(s, term(i));
            i++;
            if (hit(s)) h = i - 1;
        }
        st.sum = s;
        st.next = i;
        st.hit = h;
        st.stop = 0x7fffffff;
        st.range = kSelThreads;
    }
    __syncthreads();
    // Every pass consumes at least one term, so the bound is never the exit in practice.
    for (int guard = 0; guard < 8192; guard++) {
        const int start = st.next;
        const float s0 = st.sum;
        if (start >= n || st.hit < n) break;
        const int len = min(st.range, n - start);
        const int pend = start + len;
        const int per = (len + kSelThreads - 1) / kSelThreads;  // <= kMaxPer
        const int beg = min(pend, start + tid * per), end = min(pend, beg + per);
        const uint32_t sb = __float_as_uint(s0);
        const int sex = (int)(sb >> 23);

        if (s0 == 0.0f) {
            // Zeros leave the sum at zero: jump to the first non-zero term of the range.
            if (hit(0.0f)) {
                if (tid == 0) st.hit = start;
                __syncthreads();
                break;
            }
            int first = 0x7fffffff;
            for (int i = beg; i < end; i++) {
                if (term(i) != 0.0f) {
                    first = i;
                    break;
                }
            }
            if (first != 0x7fffffff) atomicMin(&st.stop, first);
            __syncthreads();
            if (tid == 0) {
                const int j = st.stop;
                st.stop = 0x7fffffff;
                if (j == 0x7fffffff) {
                    st.next = pend;
                    st.range = min(2 * len, kMaxRange);
                } else {
                    const float v = term(j);
                    st.sum = v;
                    st.next = j + 1;
                    if (hit(v)) st.hit = j;
                }
            }
            __syncthreads();
            continue;
        }
        if (sex < 30 || sex >= 254) {
            // Tiny or huge running sum: add a stretch natively.
            if (tid == 0) {
                float s = s0;
                int i = start;
                const int stop = min(n, start + 64);
                while (i < stop) {
                    s = __fadd_rn(s, term(i));
                    i++;
                    if (hit(s)) {
                        st.hit = i - 1;
                        break;
                    }
                    const int e2 = (int)(__float_as_uint(s) >> 23);
                    if (e2 >= 30 && e2 < 254) break;
                }
                st.sum = s;
                st.next = i;
            }
            __syncthreads();
            continue;
        }

        // terms per thread this pass: the smallest of 1, 2, 4, 8, 16 that covers the range
        if (per <= 1) scan_pass<1>(term, hit, &st, wtot, start, pend, s0, n);
        else if (per <= 2) scan_pass<2>(term, hit, &st, wtot, start, pend, s0, n);
        else if (per <= 4) scan_pass<4>(term, hit, &st, wtot, start, pend, s0, n);
        else if (per <= 8) scan_pass<8>(term, hit, &st, wtot, start, pend, s0, n);
        else scan_pass<16>(term, hit, &st, wtot, start, pend, s0, n);
        __syncthreads();
    }
    ScanResult r;
    r.sum = st.sum;
    r.hit = st.hit;
    __syncthreads();
    return r;
}

// ---------------------------------------------------------------------------------------------
// Fast path of the exact sequential sum: one sweep instead of one pass per binade.
//
// A cheap prefix sum (pairwise fp32) predicts, for every 16-term chunk, an interval that is
// GUARANTEED to contain the sequential fp32 running sum throughout the chunk (sequential
// summation of n non-negative terms is within (n-1) * 2^-24 of the exact sum, under 2^-10 for
// n <= 16384; the interval is widened by 2^-9). A chunk whose interval lies inside one binade is
// "safe": its binade is known in advance and nothing can leave it, so its parity -> increment map
// can be built immediately. Runs of safe chunks that share a binade are composed by a segmented
// scan; the few chunks that straddle a power of two are added natively. One thread then walks
// the resulting short list (tens of items) carrying the exact sum, and finally the one chunk of a
// run whose start misses the predicate and whose end meets it walks its terms from its exact start
// (the sums never decrease and the predicate is monotone). Any surprise (a start outside
// the predicted binade, an unexpected exit) abandons the sweep and the pass-per-binade scan above
// redoes the work, so exactness never rests on the prediction.
constexpr int kFastPer = 16;
constexpr int kFastMax = kFastPer * kSelThreads;

struct SegVal {  // segmented-scan payload: map composed since the segment head, and that head
    IncPair m;
    int head;  // index of the head chunk if one lies inside the scanned window, else -1
};
__device__ __forceinline__ SegVal seg_combine(const SegVal& a, const SegVal& b) {  // a earlier
    if (b.head >= 0) return b;
    SegVal r;
    r.m = compose(a.m, b.m);
    r.head = a.head;
    return r;
}
__device__ __forceinline__ SegVal seg_shfl_up(const SegVal& v, int o) {
    SegVal r;
    r.m.e = __shfl_up_sync(0xffffffffu, v.m.e, o);
    r.m.o = __shfl_up_sync(0xffffffffu, v.m.o, o);
    r.head = __shfl_up_sync(0xffffffffu, v.head, o);
    return r;
}

// Adds v[0..K) to s natively, in order. Returns the position of the first term after which hit(sum) holds (s is then
// the sum after that term), or K (s the sum after all of them). Non-negative terms never lower the sum and the
// predicate is monotone, so only the last sum is tested unless it hits; a group with a negative term or a NaN sum is
// tested term by term.
template <int K, typename Hit>
__device__ __forceinline__ int add_group(float& s, const float (&v)[K], bool has_predicate, Hit& hit) {
    uint32_t signs = 0u;
    float t = s;
#pragma unroll
    for (int k = 0; k < K; k++) {
        signs |= __float_as_uint(v[k]);
        t = __fadd_rn(t, v[k]);
    }
    if (!has_predicate || ((signs >> 31) == 0u && t == t && !hit(t))) {
        s = t;
        return K;
    }
#pragma unroll
    for (int k = 0; k < K; k++) {
        s = __fadd_rn(s, v[k]);
        if (hit(s)) return k;
    }
    return K;
}

// The parity -> increment map of terms [from, end) of a chunk that starts at beg, composed term by term: the rare
// chunk with a tie among its terms. Kept out of line so that its registers do not weigh on the sweep.
__device__ __noinline__ IncPair chunk_map_with_ties(const float* arr, int beg, int from, int end, int ue) {
    IncPair m = {0u, 0u};
    float v[kFastPer];
#pragma unroll
    for (int i = 0; i < kFastPer; i++) v[i] = (beg + i >= from && beg + i < end) ? arr[beg + i] : 0.0f;  // loads first
#pragma unroll
    for (int i = 0; i < kFastPer; i++) m = compose(m, term_inc(__float_as_uint(v[i]), ue));  // (+0 is the identity map)
    return m;
}

// work: 4096 words of shared scratch (the sort's histogram is dead by the time scans run).
// Returns false when the sweep had to be abandoned; the caller then runs seq_scan.
template <typename Hit>
__device__ bool seq_scan_fast(int n, const float* arr, Hit hit, bool has_predicate, uint32_t* work, ScanResult& out) {
    auto term = [arr](int i) { return arr[i]; };
    __shared__ float f_s0;
    __shared__ int f_start, f_hit, f_fail, f_upto;
    __shared__ float f_wd[kSelWarps];
    __shared__ uint32_t f_we[kSelWarps], f_wo[kSelWarps], f_headbits[kSelWarps];
    __shared__ int f_wh[kSelWarps];
    __shared__ int f_items[kSelThreads + 1], f_nitems;  // first chunk of every item (segment or unsafe chunk), in order
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    uint32_t* seg_e = work;
    uint32_t* seg_o = work + kSelThreads;
    int* seg_head = reinterpret_cast<int*>(work + 2 * kSelThreads);
    int* info = reinterpret_cast<int*>(work + 3 * kSelThreads);  // binade of a safe chunk, -1 unsafe; later: start sums

    // ---- leading zeros and a short native prefix (the sum doubles every few terms at first)
    if (tid == 0) {
        f_start = 0x7fffffff;
        f_hit = n;
        f_fail = 0;
    }
    __syncthreads();
    {
        int first = 0x7fffffff;
        for (int i = tid; i < n && first == 0x7fffffff; i += kSelThreads) {
            if (term(i) != 0.0f) first = i;
        }
        if (first != 0x7fffffff) atomicMin(&f_start, first);
    }
    __syncthreads();
    if (tid == 0) {
        int i = f_start;
        float s = 0.0f;
        int h = n;
        if (hit(0.0f)) {
            h = 0;  // the predicate already holds for a zero sum: the very first term triggers it
            i = n;
        } else if (i == 0x7fffffff) {
            i = n;  // all zero
        } else {
            const int stop = min(n, i + kSerialPrefix);
            while (i + 8 <= stop && h == n) {  // loads of a group are issued together
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = term(i + k);
                const int at = add_group<8>(s, v, has_predicate, hit);
                if (at < 8) h = i + at;
                i = h == n ? i + 8 : h + 1;
            }
            while (i < stop && h == n) {
                s = __fadd_rn(s, term(i));
                if (has_predicate && hit(s)) h = i;
                i++;
            }
        }
        f_s0 = s;
        f_start = i;
        f_hit = h;
        f_upto = 0;
    }
    __syncthreads();
    int start = f_start;
    float s0 = f_s0;
    // Windows of at most kFastMax terms, each swept as described above from the exact sum the previous one ended on.
    for (;;) {
    if (f_hit < n || start >= n) {
        out.sum = s0;
        out.hit = f_hit;
        __syncthreads();
        return true;
    }
    // Chunks are 16-aligned in index space so a thread's terms are four 128-bit shared-memory loads
    // (a thread-per-chunk scalar pattern would put the whole warp on two banks).
    const int base0 = start & ~(kFastPer - 1);
    const int wn = min(n, base0 + kFastMax);  // end of this window

    // ---- chunk terms into registers, predicted prefix
    const int beg = base0 + tid * kFastPer, end = min(wn, beg + kFastPer);
    // The prediction only has to be within ~1e-4 of the exact sum: pairwise fp32 sums (error a few
    // 2^-24 per level) are ample, and much cheaper than double precision here.
    float a[kFastPer];
    if ((reinterpret_cast<uintptr_t>(arr) & 15) == 0) {  // uniform
#pragma unroll
        for (int j = 0; j < kFastPer / 4; j++) {
            // may read past n inside the shared-memory allocation; such lanes are masked below
            const float4 v = beg < wn ? *reinterpret_cast<const float4*>(arr + beg + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
            a[4 * j] = v.x;
            a[4 * j + 1] = v.y;
            a[4 * j + 2] = v.z;
            a[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kFastPer; i++) a[i] = beg + i < end ? arr[beg + i] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kFastPer; i++) {
        if (beg + i < start || beg + i >= end) a[i] = 0.0f;  // already consumed by the prefix, or past the end
    }
    const float dsum = (((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]))) +
                       (((a[8] + a[9]) + (a[10] + a[11])) + ((a[12] + a[13]) + (a[14] + a[15])));
    float incl = dsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) f_wd[w] = incl;
    __syncthreads();
    float wpre;
    {   // exclusive scan of the 32 warp sums, by every warp
        float wv = lane < kSelWarps ? f_wd[lane] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, wv, o);
            if (lane >= o) wv += v;
        }
        wpre = __shfl_sync(0xffffffffu, wv, (w + 31) & 31);
        if (w == 0) wpre = 0.f;
    }
    const float P = s0 + (wpre + (incl - dsum));  // predicted sum before this chunk

    // ---- classify: safe <=> the guaranteed interval of the running sum stays in one binade
    const float lo = P * (1.0f - 1.0f / 512.0f), hi = (P + dsum) * (1.0f + 1.0f / 512.0f);
    const int elo = (int)(__float_as_uint(lo) >> 23), ehi = (int)(__float_as_uint(hi) >> 23);
    const bool used = beg < end && beg + kFastPer > start;
    uint32_t sign_seen = 0u;
#pragma unroll
    for (int i = 0; i < kFastPer; i++) sign_seen |= __float_as_uint(a[i]);
    // (a chunk with a negative term is left to the native adds of the walk below: the sums of a safe chunk never decrease)
    const bool safe = used && elo == ehi && elo >= 30 && elo < 254 && (sign_seen >> 31) == 0u;
    SegVal sv;
    sv.m.e = sv.m.o = 0u;
    if (safe) {
        // Without a tie among the chunk's terms (the usual case: a tie needs the bits below the sum's unit to be
        // exactly one half) the increments do not look at the parity and just add up, and each is a / u rounded to
        // the nearest integer: a handful of floating-point operations per term. With a tie, or a term that is not
        // small against the sum, the maps are composed term by term.
        const int ue = elo - 150;
        const float inv_u = unit_reciprocal(ue);
        uint32_t total = 0u, slow = 0u;
#pragma unroll
        for (int q = 0; q < kFastPer / 4; q++) {  // four increments below 2^22 add up exactly in a float
            float four = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) four = __fadd_rn(four, term_inc_float(a[4 * q + i], inv_u, &slow));
            total += (uint32_t)four;
        }
        sv.m.e = sv.m.o = sat(total);
        if (slow != 0u) sv.m = chunk_map_with_ties(arr, beg, max(beg, start), end, ue);  // (fetches the terms again)
    }
    info[tid] = safe ? elo : -1;
    __syncthreads();
    const bool is_head = used && (!safe || tid == 0 || info[tid - 1] != elo);
    sv.head = is_head ? tid : -1;
    const uint32_t hb = __ballot_sync(0xffffffffu, is_head);
    if (lane == 0) f_headbits[w] = hb;

    // ---- segmented inclusive scan of the maps
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const SegVal pv = seg_shfl_up(sv, o);
        if (lane >= o) sv = seg_combine(pv, sv);
    }
    if (lane == 31) {
        f_we[w] = sv.m.e;
        f_wo[w] = sv.m.o;
        f_wh[w] = sv.head;
    }
    __syncthreads();
    {
        SegVal wv;
        wv.m.e = lane < kSelWarps ? f_we[lane] : 0u;
        wv.m.o = lane < kSelWarps ? f_wo[lane] : 0u;
        wv.head = lane < kSelWarps ? f_wh[lane] : -1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const SegVal pv = seg_shfl_up(wv, o);
            if (lane >= o) wv = seg_combine(pv, wv);
        }
        SegVal before;  // everything in earlier warps, cut at the last head
        before.m.e = __shfl_sync(0xffffffffu, wv.m.e, (w + 31) & 31);
        before.m.o = __shfl_sync(0xffffffffu, wv.m.o, (w + 31) & 31);
        before.head = __shfl_sync(0xffffffffu, wv.head, (w + 31) & 31);
        if (w > 0) sv = seg_combine(before, sv);
    }
    seg_e[tid] = sv.m.e;
    seg_o[tid] = sv.m.o;
    seg_head[tid] = sv.head;
    __syncthreads();

    // ---- the items (segments and unsafe chunks) in order: warp 0 turns the head bits into a list, so that the
    // serial walk below does no searching and can request the next item's data ahead of its arithmetic
    const int chunks = (wn - base0 + kFastPer - 1) / kFastPer;
    if (w == 0) {
        uint32_t bits = lane < kSelWarps ? f_headbits[lane] : 0u;
        const int cnt = __popc(bits);
        int pre = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, pre, o);
            if (lane >= o) pre += v;
        }
        const int total = __shfl_sync(0xffffffffu, pre, 31);
        int at = pre - cnt;
        while (bits) {
            f_items[at++] = lane * 32 + __ffs(bits) - 1;
            bits &= bits - 1;
        }
        if (lane == 0) {
            f_items[total] = chunks;
            f_nitems = total;
        }
    }
    __syncthreads();

    // ---- one thread walks the items with the exact sum
    if (tid == 0) {
        float s = s0;
        int h = n, fail = 0, upto = chunks;
        const int nitems = f_nitems;
        int t = f_items[0];
        int e = nitems > 0 ? info[t] : 0;
        for (int k = 0; k < nitems; k++) {
            const int nxt = f_items[k + 1];
            // independent of the running sum: issued before the arithmetic of this item
            const int e_next = nxt < chunks ? info[nxt] : 0;
            const uint32_t me = seg_e[nxt - 1], mo = seg_o[nxt - 1];
            if (e < 0) {  // unsafe chunk: native adds
                const int b0 = base0 + t * kFastPer, e0 = min(wn, b0 + kFastPer);
                float v[kFastPer];
#pragma unroll
                for (int i = 0; i < kFastPer; i++) v[i] = (b0 + i >= start && b0 + i < e0) ? term(b0 + i) : 0.0f;  // loads first
                // (the terms outside [start, e0) are +0 here and leave the sum as it is)
                const int at = add_group<kFastPer>(s, v, has_predicate, hit);
                if (at < kFastPer) h = b0 + at;
            } else {  // run of safe chunks t .. nxt-1 in binade e
                const uint32_t sb = __float_as_uint(s);
                if ((int)(sb >> 23) != e) {
                    fail = 1;
                    break;
                }
                info[t] = (int)sb;  // exact start sum of the segment, for the walkers
                const uint32_t S0 = (sb & 0x7fffffu) | 0x800000u;
                IncPair m;
                m.e = me;
                m.o = mo;
                const uint32_t S1 = step_S(S0, m);
                if (S1 >= kBinadeEnd) {
                    fail = 1;
                    break;
                }
                s = __uint_as_float(((uint32_t)e << 23) | (S1 & 0x7fffffu));
            }
            t = nxt;
            e = e_next;
            if (h < n || (has_predicate && hit(s))) {  // the first hit lies at or before this point
                upto = t;
                break;
            }
        }
        f_s0 = s;
        f_hit = h;
        f_fail = fail;
        f_upto = upto;
    }
    __syncthreads();
    if (f_fail) return false;  // uniform

    // ---- predicate: every safe chunk before `upto` is walked from its exact start
    if (has_predicate && safe && tid < f_upto) {
        const int head = seg_head[tid];
        const uint32_t sb = (uint32_t)info[head];
        const uint32_t S0 = (sb & 0x7fffffu) | 0x800000u;
        IncPair ex;
        ex.e = ex.o = 0u;
        if (head != tid) {
            ex.e = seg_e[tid - 1];
            ex.o = seg_o[tid - 1];
        }
        uint32_t S = step_S(S0, ex);
        IncPair through;  // the head's start to this chunk's end
        through.e = seg_e[tid];
        through.o = seg_o[tid];
        const uint32_t S_end = step_S(S0, through);
        auto as_sum = [elo](uint32_t Sx) { return __uint_as_float(((uint32_t)elo << 23) | (Sx & 0x7fffffu)); };
        // The terms are non-negative, so the sums never decrease, and the predicate stays true once it is: the first
        // hit of a run lies in the one chunk whose start does not satisfy it and whose end does. Only that chunk walks.
        if (!hit(as_sum(S)) && hit(as_sum(S_end))) {
            int mine = 0x7fffffff;
            // tie-free chunk: the increments do not look at the parity of S
            const float inv_u = unit_reciprocal(elo - 150);
            uint32_t slow = 0u, inc[kFastPer];
#pragma unroll
            for (int i = 0; i < kFastPer; i++) inc[i] = (uint32_t)term_inc_float(a[i], inv_u, &slow);
            if (slow == 0u) {
#pragma unroll
                for (int i = 0; i < kFastPer; i++) {
                    if (mine == 0x7fffffff && beg + i >= start && beg + i < end) {
                        S += inc[i];
                        if (hit(as_sum(S))) mine = beg + i;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < kFastPer; i++) {
                    if (mine == 0x7fffffff && beg + i >= start && beg + i < end) {
                        S = step_S(S, term_inc(__float_as_uint(a[i]), elo - 150));
                        if (hit(as_sum(S))) mine = beg + i;
                    }
                }
            }
            if (mine != 0x7fffffff) atomicMin(&f_hit, mine);
        }
    }
    __syncthreads();
    // this window is done: the next one starts where it ended, from its exact sum
    start = wn;
    s0 = f_s0;
    __syncthreads();
    }
}

// Diagnostics build: clock cycles sequence 0's CTA spends per part of the sampled selection (gradb_diag_select_clocks).
#if GRADB_DIAG
__device__ unsigned long long g_sel_clock[16];
#define SEL_CLK(x) const long long x = clock64()
#define SEL_ADD(i, v) do { if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_sel_clock[i], (unsigned long long)(v)); } while (0)
#define SEL_MAX(i, v) do { if (threadIdx.x == 0) atomicMax(&g_sel_clock[i], (unsigned long long)(v)); } while (0)
#else
#define SEL_CLK(x)
#define SEL_ADD(i, v)
#define SEL_MAX(i, v)
#endif

// The exact scan: the one-sweep fast path, or the pass-per-binade scan when it declines. The terms are non-negative
// and `hit` is monotone (true for every sum above one it is true for).
template <typename Hit>
__device__ ScanResult exact_scan(int n, const float* arr, Hit hit, bool has_predicate, uint32_t* sh, uint32_t* work) {
    ScanResult r;
    if (seq_scan_fast(n, arr, hit, has_predicate, work, r)) return r;
    __syncthreads();
    return seq_scan(n, [arr](int i) { return arr[i]; }, hit, sh);
}

// Bitonic sort, descending, of n_pad (power of two) floats held by this CTA (the rarely taken path sorts in global
// memory: a CTA sees its own global writes after a barrier).
__device__ void sort_desc(float* a, int n_pad) {
    for (int k = 2; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pad; i += blockDim.x) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const float x = a[i], y = a[ixj];
                    const bool desc = (i & k) == 0;
                    if (desc ? (x < y) : (x > y)) {
                        a[i] = y;
                        a[ixj] = x;
                    }
                }
            }
            __syncthreads();
        }
    }
}

constexpr int kBuckets = 4096;
constexpr int kBucketMax = 96;  // larger buckets of unequal values fall back to the bitonic sort

// Exclusive prefix sum over hist[0..kBuckets) in place (bucket starts), kBuckets / kSelThreads consecutive buckets
// per thread. All threads call it.
__device__ void bucket_starts(int* hist) {
    __shared__ int wsum[kSelWarps];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    constexpr int kPer = kBuckets / kSelThreads;
    int c[kPer], tot = 0;
#pragma unroll
    for (int i = 0; i < kPer; i++) {
        c[i] = hist[tid * kPer + i];
        tot += c[i];
    }
    int inc = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) wsum[w] = inc;
    __syncthreads();
    int wv = lane < kSelWarps ? wsum[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, wv, o);
        if (lane >= o) wv += v;
    }
    int base = __shfl_sync(0xffffffffu, wv, (w + 31) & 31);
    if (w == 0) base = 0;
    base += inc - tot;
#pragma unroll
    for (int i = 0; i < kPer; i++) {
        hist[tid * kPer + i] = base;
        base += c[i];
    }
    __syncthreads();
}

// Descending bitonic network on N (a power of two) bit patterns held in registers; every index is a compile-time
// constant once unrolled.
template <int N>
__device__ __forceinline__ void sort_regs_desc(uint32_t (&v)[N]) {
#pragma unroll
    for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
            for (int i = 0; i < N; i++) {
                const int l = i ^ j;
                if (l > i) {
                    const uint32_t hi = max(v[i], v[l]), lo = min(v[i], v[l]);
                    const bool desc = (i & k) == 0;
                    v[i] = desc ? hi : lo;
                    v[l] = desc ? lo : hi;
                }
            }
        }
    }
}
// A bucket of 2..N positive floats x[lo..lo+n): fetched side by side, sorted in registers, written back.
template <int N>
__device__ __forceinline__ void sort_bucket_regs(float* x, int lo, int n) {
    uint32_t v[N];
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = i < n ? __float_as_uint(x[lo + i]) : 0u;  // (0 sorts behind every positive value)
    sort_regs_desc<N>(v);
#pragma unroll
    for (int i = 0; i < N; i++) {
        if (i < n) x[lo + i] = __uint_as_float(v[i]);
    }
}

// Exclusive prefix sum over 2 * kBuckets 16-bit counts packed two to a word (sums below 65536), in place.
__device__ void bucket_starts16(uint32_t* hist) {
    __shared__ int wsum16[kSelWarps];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    constexpr int kPer = kBuckets / kSelThreads;  // words per thread
    uint32_t c[kPer];
    int tot = 0;
#pragma unroll
    for (int i = 0; i < kPer; i++) {
        c[i] = hist[tid * kPer + i];
        tot += (int)(c[i] & 0xffffu) + (int)(c[i] >> 16);
    }
    int inc = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) wsum16[w] = inc;
    __syncthreads();
    int wv = lane < kSelWarps ? wsum16[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, wv, o);
        if (lane >= o) wv += v;
    }
    int base = __shfl_sync(0xffffffffu, wv, (w + 31) & 31);
    if (w == 0) base = 0;
    base += inc - tot;
#pragma unroll
    for (int i = 0; i < kPer; i++) {
        const int lo = base, hi = base + (int)(c[i] & 0xffffu);
        base = hi + (int)(c[i] >> 16);
        hist[tid * kPer + i] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    __syncthreads();
}

// Descending sort of n probabilities (non-negative, finite). On entry x[0..n) (shared) and g[0..n) (global) hold the
// same values in index order; on return x holds them sorted, g is untouched. Positive floats order like their bit
// patterns, so a bucket is a range of bit patterns. The buckets follow the values' own distribution: a coarse
// histogram (kCoarse equal ranges of bit patterns) gives every range a power-of-two share of the 2 * kBuckets fine
// buckets in proportion to its count, so a fine bucket holds a few values wherever they crowd (exponentials of
// bell-shaped logits crowd in the middle). Zeros go to the tail unsorted; a histogram + prefix sum (16-bit counts,
// two to a word) places the buckets, the scatter reads the index-order copy in g while it overwrites x, and each
// bucket is finished by insertion. Buckets of many equal values (coarse logits) need no work. Returns false, with x
// unspecified, when the values are not finite or too clustered; the caller then sorts g's copy bitonically.
constexpr int kCoarse = 256;
constexpr int kFineBuckets = 2 * kBuckets;
constexpr int kFineTarget = 7424;  // fine buckets handed out in proportion (each range gets at least one on top)
struct ProbStats {  // of one thread's share of the probabilities: bit patterns of the non-zero ones
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    int nnz = 0, bad = 0;  // bad: a NaN, an infinity or a negative value
    __device__ __forceinline__ void add(float pr) {
        const uint32_t k = __float_as_uint(pr);
        if (k >= 0x7f800000u) bad = 1;
        if (k != 0u) {
            kmin = min(kmin, k);
            kmax = max(kmax, k);
            nnz++;
        }
    }
};
__device__ bool sort_probs_desc(float* x, const float* g, int n, int* hist_words, ProbStats own) {
    __shared__ uint32_t s_kmin, s_kmax;
    __shared__ int s_nnz, s_bad;
    __shared__ int s_coarse[kCoarse];  // counts, then (first fine bucket << 5) | shift inside the range
    uint32_t* hist = reinterpret_cast<uint32_t*>(hist_words);
    const int tid = threadIdx.x;
    if (n >= 65536) return false;  // (16-bit bucket positions; a row in shared memory is shorter anyway)
    if (tid == 0) {
        s_kmin = 0xffffffffu;
        s_kmax = 0u;
        s_nnz = 0;
        s_bad = 0;
    }
    for (int i = tid; i < kBuckets; i += kSelThreads) hist[i] = 0u;
    if (tid < kCoarse) s_coarse[tid] = 0;
    __syncthreads();
    {
        uint32_t kmin = own.kmin, kmax = own.kmax;
        int nnz = own.nnz, bad = own.bad;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
            kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
            nnz += __shfl_xor_sync(0xffffffffu, nnz, o);
            bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        }
        if ((tid & 31) == 0) {
            atomicMin(&s_kmin, kmin);
            atomicMax(&s_kmax, kmax);
            atomicAdd(&s_nnz, nnz);
            if (bad) s_bad = 1;
        }
    }
    __syncthreads();
    if (s_bad) return false;  // uniform; x is still intact
    const int nnz = s_nnz;
    if (nnz == 0) return true;  // all zero: sorted as it stands
    const uint32_t kmax = s_kmax, span = kmax - s_kmin;
    int cshift = 0;
    while ((span >> cshift) >= (uint32_t)kCoarse) cshift++;
    const uint32_t cmask = (1u << cshift) - 1u;
    for (int i = tid; i < n; i += kSelThreads) {
        const uint32_t k = __float_as_uint(x[i]);
        if (k != 0u) atomicAdd(&s_coarse[(kmax - k) >> cshift], 1);
    }
    __syncthreads();
    if (tid < 32) {  // one warp: fine buckets per range (a power of two), their starts
        constexpr int kPerLane = kCoarse / 32;
        int bits[kPerLane], tot = 0;
        const float per_value = (float)kFineTarget / (float)nnz;  // (rounding may add one bucket per range: there is room)
#pragma unroll
        for (int i = 0; i < kPerLane; i++) {
            const int cnt = s_coarse[tid * kPerLane + i];
            const int share = max(1, (int)((float)cnt * per_value));
            bits[i] = min(31 - __clz(share), cshift);  // 2^bits <= share; no finer than single bit patterns
            tot += 1 << bits[i];
        }
        int inc = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (tid >= o) inc += v;
        }
        int start = inc - tot;
#pragma unroll
        for (int i = 0; i < kPerLane; i++) {
            s_coarse[tid * kPerLane + i] = (start << 5) | (cshift - bits[i]);
            start += 1 << bits[i];
        }
    }
    __syncthreads();
    auto bucket_of = [&](uint32_t k) {
        const uint32_t d = kmax - k;
        const int e = s_coarse[d >> cshift];
        return (e >> 5) + (int)((d & cmask) >> (e & 31));
    };
    for (int i = tid; i < n; i += kSelThreads) {
        const uint32_t k = __float_as_uint(x[i]);
        if (k != 0u) {
            const int fb = bucket_of(k);
            atomicAdd(&hist[fb >> 1], 1u << ((fb & 1) * 16));
        }
    }
    __syncthreads();
    bucket_starts16(hist);
    for (int i = tid; i < n; i += kSelThreads) {
        const float v = g[i];
        const uint32_t k = __float_as_uint(v);
        if (k != 0u) {
            const int fb = bucket_of(k);
            const uint32_t old = atomicAdd(&hist[fb >> 1], 1u << ((fb & 1) * 16));
            x[(old >> ((fb & 1) * 16)) & 0xffffu] = v;
        }
    }
    for (int i = nnz + tid; i < n; i += kSelThreads) x[i] = 0.0f;
    __syncthreads();
    // each half word is now the END of its bucket; finish each bucket: a network in registers for up to 16 values, insertion beyond
    const uint16_t* ends = reinterpret_cast<const uint16_t*>(hist);
    for (int bkt = tid; bkt < kFineBuckets; bkt += kSelThreads) {
        const int lo = bkt == 0 ? 0 : ends[bkt - 1], hi = ends[bkt];
        if (hi - lo <= 1) continue;
        if (hi - lo <= 8) {
            sort_bucket_regs<8>(x, lo, hi - lo);
            continue;
        }
        if (hi - lo <= 16) {
            sort_bucket_regs<16>(x, lo, hi - lo);
            continue;
        }
        if (hi - lo > kBucketMax) {
            const float first = x[lo];
            bool same = true;
            for (int i = lo + 1; i < hi && same; i++) same = x[i] == first;
            if (!same) s_bad = 1;
            continue;
        }
        for (int i = lo + 1; i < hi; i++) {
            const float v = x[i];
            int j = i - 1;
            while (j >= lo && x[j] < v) {
                x[j + 1] = x[j];
                j--;
            }
            x[j + 1] = v;
        }
    }
    __syncthreads();
    return s_bad == 0;
}

// Order-preserving map of finite floats to unsigned integers, and back.
__device__ __forceinline__ uint32_t ordered_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_key(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// The k-th largest (1 <= k <= n) of x[0..n), what the reference reads off a full descending sort
// (text_gen.cpp:138-150): the candidates' value range is cut into kBuckets equal parts, the part holding rank k is
// found from a histogram, and the search continues inside that part's actual value range until it is one value.
// NaNs take no part. All threads call it and get the same result.
__device__ float select_kth_desc(const float* x, int n, int k, int* hist) {
    __shared__ uint32_t s_lo, s_hi;
    __shared__ int s_bucket, s_before, s_count, s_few_n;
    constexpr int kKthFew = 256;
    const int tid = threadIdx.x;
    constexpr int kPer = kBuckets / kSelThreads;
    if (tid == 0) {
        s_lo = 0xffffffffu;
        s_hi = 0u;
    }
    __syncthreads();
    {
        uint32_t lo = 0xffffffffu, hi = 0u;
        for (int i = tid; i < n; i += kSelThreads) {
            const float v = x[i];
            if (v == v) {
                const uint32_t key = ordered_key(v);
                lo = min(lo, key);
                hi = max(hi, key);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if ((tid & 31) == 0) {
            atomicMin(&s_lo, lo);
            atomicMax(&s_hi, hi);
        }
    }
    __syncthreads();
    float lo = from_ordered_key(s_lo), hi = from_ordered_key(s_hi);
    int rank = k;
    for (int level = 0; level < 12; level++) {
        const float span = hi - lo;
        if (!(span > 0.0f) || !(span < 3.0e38f)) break;  // one value left (or nothing finite to separate)
        const float scale = (float)(kBuckets - 1) / span;
        auto bucket_of = [&](float v) {
            const int bkt = (int)((hi - v) * scale);  // monotone: larger values land in lower buckets
            return min(max(bkt, 0), kBuckets - 1);
        };
        for (int i = tid; i < kBuckets; i += kSelThreads) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < n; i += kSelThreads) {
            const float v = x[i];
            if (v >= lo && v <= hi) atomicAdd(&hist[bucket_of(v)], 1);
        }
        __syncthreads();
        int counts[kPer];
#pragma unroll
        for (int i = 0; i < kPer; i++) counts[i] = hist[tid * kPer + i];
        __syncthreads();
        bucket_starts(hist);  // hist[b] = candidates in buckets before b
#pragma unroll
        for (int i = 0; i < kPer; i++) {
            const int before = hist[tid * kPer + i];
            if (counts[i] > 0 && before < rank && rank <= before + counts[i]) {
                s_bucket = tid * kPer + i;
                s_before = before;
                s_count = counts[i];
            }
        }
        if (tid == 0) {
            s_lo = 0xffffffffu;
            s_hi = 0u;
            s_few_n = 0;
        }
        __syncthreads();
        const int bkt = s_bucket;
        rank -= s_before;
        if (s_count <= kKthFew) {
            // Few candidates left in the bucket: list them (in any order) and read the rank off by counting, instead
            // of narrowing the range again. hist is free: the list lives in its first words.
            float* few = reinterpret_cast<float*>(hist);
            __syncthreads();
            for (int i = tid; i < n; i += kSelThreads) {
                const float v = x[i];
                if (v >= lo && v <= hi && bucket_of(v) == bkt) few[atomicAdd(&s_few_n, 1)] = v;
            }
            __syncthreads();
            const int c = s_few_n;
            if (tid < c) {
                const float v = few[tid];
                int greater = 0, equal = 0;
                for (int j = 0; j < c; j++) {
                    greater += few[j] > v;
                    equal += few[j] == v;
                }
                if (greater < rank && rank <= greater + equal) s_lo = ordered_key(v);  // (equal values write the same key)
            }
            __syncthreads();
            return from_ordered_key(s_lo);
        }
        {
            uint32_t klo = 0xffffffffu, khi = 0u;
            for (int i = tid; i < n; i += kSelThreads) {
                const float v = x[i];
                if (v >= lo && v <= hi && bucket_of(v) == bkt) {
                    const uint32_t key = ordered_key(v);
                    klo = min(klo, key);
                    khi = max(khi, key);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                klo = min(klo, __shfl_xor_sync(0xffffffffu, klo, o));
                khi = max(khi, __shfl_xor_sync(0xffffffffu, khi, o));
            }
            if ((tid & 31) == 0) {
                atomicMin(&s_lo, klo);
                atomicMax(&s_hi, khi);
            }
        }
        __syncthreads();
        lo = from_ordered_key(s_lo);
        hi = from_ordered_key(s_hi);
        __syncthreads();
    }
    return hi;
}

// The chosen id joins the sequence's history; inside the generate loop it also becomes the next step's input
// unless the sequence stops here (text_gen.cpp:48-63: context full or max_tokens ids emitted).
__device__ __forceinline__ void record_pick(const SelectParams& p, int b, int* hist, int hlen, int pick) {
    if (hlen < p.hist_stride) hist[hlen] = pick;
    p.hist_len[b] = hlen + 1;
    if (p.out_tok) p.out_tok[b] = pick;
    if (p.loop_mode) {
        const int g0 = p.gen[b], g = g0 + 1;
        p.gen[b] = g;
        bool stop = p.pos[b] >= p.capacity || g >= (p.max_new_seq ? p.max_new_seq[b] : p.max_new);
        for (int i = 0; i < p.n_stop; i++) stop = stop || pick == p.stop_ids[i];
        p.cur_tok[b] = stop ? kSkip : pick;
        if (stop) p.done[b] = 1;
        if (p.stream_ids && g0 < p.stream_stride) {
            *reinterpret_cast<volatile int*>(p.stream_ids + (size_t)b * p.stream_stride + g0) = pick + 1;
            __threadfence_system();
        }
    }
}

// The rest of sample_from_logits (text_gen.cpp:156-208) when the top-k filter left n <= kSmallMax candidates: their
// ids (ascending) in idx, their tempered logits in val; srt: room for the next power of two of floats. Softmax over
// the candidates (every other entry is an exact zero), nucleus cutoff on the sorted values, renormalisation, draw --
// the sums formed term by term in index order by one lane, as the reference forms them. x (vocabulary-sized) is
// only used to lay out the probabilities when the caller asked for them. Called by ONE warp (warp barriers only);
// every lane returns the pick.
constexpr int kSmallMax = 256;
__device__ void sort_desc_warp(float* a, int n_pad) {  // bitonic, descending, n_pad a power of two, one warp
    const int lane = threadIdx.x & 31;
    for (int k = 2; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = lane; i < n_pad; i += 32) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const float x = a[i], y = a[ixj];
                    const bool desc = (i & k) == 0;
                    if (desc ? (x < y) : (x > y)) {
                        a[i] = y;
                        a[ixj] = x;
                    }
                }
            }
            __syncwarp();
        }
    }
}
// First j < n whose running sum v[0] + ... + v[j] (added one by one, in order) is >= thresh; n when none is. The
// values are fetched eight at a time ahead of the dependent additions; a +0 past the end leaves the sum as it is.
__device__ __forceinline__ int first_reaching(const float* v, int n, float thresh) {
    float run = 0.0f;
    int found = n;
    for (int j0 = 0; j0 < n && found == n; j0 += 8) {
        float r[8];
#pragma unroll
        for (int t = 0; t < 8; t++) r[t] = j0 + t < n ? v[j0 + t] : 0.0f;
#pragma unroll
        for (int t = 0; t < 8; t++) {
            run = __fadd_rn(run, r[t]);
            if (found == n && j0 + t < n && run >= thresh) found = j0 + t;
        }
    }
    return found;
}
__device__ int select_among_few(const SelectParams& p, int b, int n, const int* idx, float* val, float* srt,
                                const uint64_t* exp_tab, float* x) {
    const int lane = threadIdx.x & 31;
    // max (tensor.cpp:434-440; the filtered entries, -1e10, lie below every candidate)
    float m = -INFINITY;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, val[j]);
    const float mx = warp_max(m);
    for (int j = lane; j < n; j += 32) val[j] = expf_libm(__fsub_rn(val[j], mx), exp_tab);
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0) {
        for (int j = 0; j < n; j++) sum = __fadd_rn(sum, val[j]);
    }
    const float inv_sum = __fdiv_rn(1.0f, __shfl_sync(0xffffffffu, sum, 0));
    for (int j = lane; j < n; j += 32) val[j] = __fmul_rn(val[j], inv_sum);
    __syncwarp();
    if (p.top_p < 1.0f) {  // text_gen.cpp:158-193
        if (n <= 64) {
            // rank of each value among the candidates (equal values ordered by position): its place in the sorted row
            const int j0 = lane, j1 = lane + 32;
            const float v0 = j0 < n ? val[j0] : 0.0f, v1 = j1 < n ? val[j1] : 0.0f;
            int r0 = 0, r1 = 0;
            for (int t = 0; t < n; t++) {
                const float o = val[t];
                r0 += (o > v0) || (o == v0 && t < j0);
                r1 += (o > v1) || (o == v1 && t < j1);
            }
            if (j0 < n) srt[r0] = v0;
            if (j1 < n) srt[r1] = v1;
            __syncwarp();
        } else {
            int n_pad = 128;
            while (n_pad < n) n_pad <<= 1;
            for (int j = lane; j < n_pad; j += 32) srt[j] = j < n ? val[j] : -INFINITY;
            __syncwarp();
            sort_desc_warp(srt, n_pad);
        }
        float cutoff_prob = 0.0f;
        if (lane == 0) {
            // stays 0 when the running sum never reaches p (the zeros after the candidates add nothing)
            const int reached = first_reaching(srt, n, p.top_p);
            cutoff_prob = srt[reached < n ? reached : 0];
        }
        cutoff_prob = __shfl_sync(0xffffffffu, cutoff_prob, 0);
        for (int j = lane; j < n; j += 32) {
            if (val[j] < cutoff_prob) val[j] = 0.0f;
        }
        __syncwarp();
        float kept = 0.0f;
        if (lane == 0) {
            for (int j = 0; j < n; j++) kept = __fadd_rn(kept, val[j]);
        }
        kept = __shfl_sync(0xffffffffu, kept, 0);
        if (kept > 0.0f) {
            for (int j = lane; j < n; j += 32) {
                if (val[j] != 0.0f) val[j] = __fdiv_rn(val[j], kept);  // (zeros stay zero without the division's slow path)
            }
        }
        __syncwarp();
    }
    if (p.probs_out) {
        for (int i = lane; i < p.V; i += 32) x[i] = 0.0f;
        __syncwarp();
        for (int j = lane; j < n; j += 32) x[idx[j]] = val[j];
        __syncwarp();
        for (int i = lane; i < p.V; i += 32) p.probs_out[(size_t)b * p.V + i] = x[i];
    }
    // draw (text_gen.cpp:199-208): first index with u <= running sum, else the last id. Index 0 already satisfies
    // u <= 0 + x[0] when u is not positive, candidate or not.
    int pick = p.V - 1;
    if (lane == 0) {
        const float u = p.uniforms[(size_t)b * p.u_stride + (p.loop_mode ? p.gen[b] : 0)];
        if (u <= 0.0f) {
            pick = 0;
        } else {
            const int reached = first_reaching(val, n, u);
            if (reached < n) pick = idx[reached];
        }
    }
    return __shfl_sync(0xffffffffu, pick, 0);
}

// Sampled selection, one 512-thread CTA per sequence. Shared memory holds ONE vocabulary-sized array (so two
// sequences share an SM): the values in index order, except while the nucleus cutoff is being found, when it holds
// the sorted probabilities and the index-order copy waits in a global scratch row (L2 resident).
// TOPK: compiled with or without the top-k filter and its few-candidates path, so that the registers those need do
// not weigh on the plain nucleus path (the benchmark's) and the other way round.
template <bool TOPK>
__global__ void __launch_bounds__(kSelThreads, 2) select_kernel(const SelectParams p) {
    extern __shared__ __align__(16) float smem[];
    __shared__ uint32_t scan_sh[2 * kSelWarps + 4];
    __shared__ float red_v[kSelWarps];
    __shared__ uint64_t s_exp_tab[32];
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    if (tid < 32) s_exp_tab[tid] = c_exp2_tab[tid];  // published to all threads by the barriers below
    const int V = p.V;
    pdl_trigger();
    pdl_wait();
    if (p.loop_mode && p.done[b]) return;
    SEL_CLK(t0);

    float* x = smem;                                                        // [V] (+ slack the scans may read)
    uint32_t* work = reinterpret_cast<uint32_t*>(smem + p.n_pad);          // 4096 words: histograms, scan scratch
    float* g = p.scratch + (size_t)b * p.scratch_stride;                   // [V] index-order copy, then [n_sort] sort area
    const float* lg = p.logits + (size_t)b * V;
    // the penalty window's ids are fetched alongside the logits (two dependent reads of global memory otherwise wait
    // behind the barrier)
    __shared__ int s_pen_id[kPenaltyWindow];
    int* hist = p.hist + (size_t)b * p.hist_stride;
    const int hlen = p.hist_len[b];
    const int window = min(kPenaltyWindow, hlen);
    if (p.penalty != 1.0f && tid < window) s_pen_id[tid] = hist[hlen - window + tid];
    for (int i = tid; i < V; i += kSelThreads) x[i] = lg[i];
    for (int i = V + tid; i < p.n_pad; i += kSelThreads) x[i] = 0.0f;
    __syncthreads();
    SEL_CLK(t1);
    SEL_ADD(0, 1);
    SEL_ADD(1, t1 - t0);  // logits -> shared memory

    // ---- repetition penalty: last min(50, n) ids, once per occurrence, in order (text_gen.cpp:20-31)
    if (p.penalty != 1.0f) {
        // The reference walks the window in order and penalises an id once per occurrence. Different ids do not
        // interact and the repeated penalties of one id are applied in sequence by one thread (the window position
        // of its first occurrence), so the positions work side by side with the reference's result.
        if (tid < window) {
            const int id = s_pen_id[tid];
            if (GRADB_INDEX_OK(id >= 0 && id < V, p.status, 901)) {
                bool first = true;
                int count = 0;
                for (int k = 0; k < window; k++) {
                    const bool same = s_pen_id[k] == id;
                    first = first && !(same && k < tid);
                    count += same;
                }
                if (first) {
                    float v = x[id];
                    for (int c = 0; c < count; c++) v = v > 0 ? __fdiv_rn(v, p.penalty) : __fmul_rn(v, p.penalty);
                    x[id] = v;
                }
            }
        }
    }
    __syncthreads();

    SEL_CLK(t2);
    SEL_ADD(2, t2 - t1);  // penalty
    const float inv_t = __fdiv_rn(1.0f, p.temperature);  // text_gen.cpp:136
    const bool use_k = TOPK && p.top_k > 0 && p.top_k < V;
    const bool use_p = p.top_p < 1.0f;
    float own_max = -INFINITY;  // of this thread's values; NaNs aside
    bool own_odd = false;       // a NaN among them
    for (int i = tid; i < V; i += kSelThreads) {
        const float v = __fmul_rn(x[i], inv_t);
        x[i] = v;
        own_max = fmaxf(own_max, v);
        if (TOPK) own_odd |= v != v;
    }
    __syncthreads();
    if (TOPK && use_k) {  // text_gen.cpp:138-154: below the k-th largest value -> -1e10, ties kept
        SEL_CLK(t3);
        SEL_ADD(3, t3 - t2);  // temperature
        // Small k (the usual one): a threshold with at least k values at or above it comes from the threads' own maxima
        // -- the j-th largest of each warp's 32, j = ceil(k / warps), and the smallest of those over the warps, so at
        // least j * warps >= k maxima reach it. The few values that reach it are listed; the k-th largest and the
        // survivors in index order are read off the list by counting. Anything unusual (a NaN, too many listed) leaves
        // the row untouched for the search below.
        constexpr int kListK = 256, kListMax = kSelThreads;
        if (p.top_k <= kListK) {
            __shared__ float s_warp_thr[kSelWarps];
            __shared__ float s_kth;
            __shared__ int s_listed;
            const int j = (p.top_k + kSelWarps - 1) / kSelWarps;
            float m = own_max, thr = -INFINITY;
            for (int r = 0; r < j; r++) {
                thr = warp_max(m);
                const uint32_t holders = __ballot_sync(0xffffffffu, m == thr);
                if (lane == __ffs(holders) - 1) m = -INFINITY;  // one holder of the maximum steps aside
            }
            if (lane == 0) s_warp_thr[w] = thr;
            if (tid == 0) s_listed = 0;
            const bool any_odd = __syncthreads_or(own_odd);
            thr = s_warp_thr[0];
            for (int i = 1; i < kSelWarps; i++) thr = fminf(thr, s_warp_thr[i]);
            if (!any_odd && thr > -1e10f) {
                float* l_val = reinterpret_cast<float*>(work);
                int* l_idx = reinterpret_cast<int*>(work + kListMax);
                int* s_idx = reinterpret_cast<int*>(work + 2 * kListMax);
                float* s_val = reinterpret_cast<float*>(work + 2 * kListMax + kSmallMax);
                float* s_srt = reinterpret_cast<float*>(work + 2 * kListMax + 2 * kSmallMax);
                for (int i = tid; i < V; i += kSelThreads) {
                    const float v = x[i];
                    if (v >= thr) {
                        const int at = atomicAdd(&s_listed, 1);
                        if (at < kListMax) {
                            l_val[at] = v;
                            l_idx[at] = i;
                        }
                    }
                }
                __syncthreads();
                const int listed = s_listed;
                if (listed <= kListMax && listed >= p.top_k) {
                    float v = 0.0f;
                    int id = 0;
                    if (tid < listed) {
                        v = l_val[tid];
                        id = l_idx[tid];
                        int greater = 0, equal = 0;
                        for (int t = 0; t < listed; t++) {
                            const float o = l_val[t];
                            greater += o > v;
                            equal += o == v;
                        }
                        if (greater < p.top_k && p.top_k <= greater + equal) s_kth = v;  // (equal values write the same)
                    }
                    __syncthreads();
                    const float kth = s_kth;
                    const bool keep = tid < listed && !(v < kth);
                    const int total = __syncthreads_count(keep);
                    if (total <= kSmallMax && kth > -1e10f) {
                        if (keep) {
                            int at = 0;  // survivors with a smaller id
                            for (int t = 0; t < listed; t++) at += !(l_val[t] < kth) && l_idx[t] < id;
                            s_idx[at] = id;
                            s_val[at] = v;
                        }
                        __syncthreads();
                        SEL_CLK(t5);
                        SEL_ADD(4, t5 - t3);  // threshold, list, k-th value, survivors in index order
                        if (w != 0) return;   // one warp finishes the stage: no block-wide barrier from here on
                        const int pick = select_among_few(p, b, total, s_idx, s_val, s_srt, s_exp_tab, x);
                        SEL_CLK(t6);
                        SEL_ADD(6, t6 - t5);  // the stage on the survivors
                        if (lane == 0) record_pick(p, b, hist, hlen, pick);
                        SEL_CLK(t7);
                        SEL_ADD(7, t7 - t6);  // bookkeeping
                        return;
                    }
                }
            }
            __syncthreads();  // the list area is free again
        }
        const float kth = select_kth_desc(x, V, p.top_k, reinterpret_cast<int*>(work));
        __syncthreads();  // the histogram area is free again
        SEL_CLK(t4);
        SEL_ADD(4, t4 - t3);  // k-th value
        // Few survivors (the usual top-k): everything after the filter only ever sees them. The filtered entries
        // become exp(-1e10 - max) = +0 exactly, and adding +0 never changes a running sum, so the sequential sums
        // of the reference are those of the survivors in index order; one warp does the rest of the stage.
        {
            __shared__ int s_cnt[kSelWarps];
            // each warp compacts a contiguous range, 32 consecutive values per step (ballot + popcount keep the order)
            const int per_warp = ((V + kSelWarps - 1) / kSelWarps + 31) / 32 * 32;
            const int w_lo = min(V, w * per_warp), w_hi = min(V, w_lo + per_warp);
            int cnt = 0;
            bool odd = false;  // a NaN among the values: leave it to the general path
            for (int base = w_lo; base < w_hi; base += 32) {
                const int i = base + lane;
                const float v = i < w_hi ? x[i] : -INFINITY;
                odd |= v != v;
                cnt += __popc(__ballot_sync(0xffffffffu, i < w_hi && !(v < kth)));
            }
            if (lane == 0) s_cnt[w] = cnt;
            const bool any_odd = __syncthreads_or(odd);
            int before = 0, total = 0;
            for (int i = 0; i < kSelWarps; i++) {
                before += i < w ? s_cnt[i] : 0;
                total += s_cnt[i];
            }
            if (!any_odd && total <= kSmallMax && kth > -1e10f) {
                int* s_idx = reinterpret_cast<int*>(work);
                float* s_val = reinterpret_cast<float*>(work + kSmallMax);
                int at = before;
                for (int base = w_lo; base < w_hi; base += 32) {
                    const int i = base + lane;
                    const float v = i < w_hi ? x[i] : -INFINITY;
                    const bool keep = i < w_hi && !(v < kth);
                    const uint32_t mask = __ballot_sync(0xffffffffu, keep);
                    if (keep) {
                        const int pos = at + __popc(mask & ((1u << lane) - 1u));
                        s_idx[pos] = i;
                        s_val[pos] = v;
                    }
                    at += __popc(mask);
                }
                __syncthreads();
                SEL_CLK(t5);
                SEL_ADD(5, t5 - t4);  // count and compact the survivors
                if (w != 0) return;   // one warp finishes the stage: no block-wide barrier from here on
                const int pick = select_among_few(p, b, total, s_idx, s_val, reinterpret_cast<float*>(work + 2 * kSmallMax),
                                                  s_exp_tab, x);
                SEL_CLK(t6);
                SEL_ADD(6, t6 - t5);  // the stage on the survivors
                if (lane == 0) record_pick(p, b, hist, hlen, pick);
                SEL_CLK(t7);
                SEL_ADD(7, t7 - t6);  // bookkeeping
                return;
            }
            __syncthreads();  // (s_cnt is read by all before anyone moves on)
        }
        for (int i = tid; i < V; i += kSelThreads) {
            if (x[i] < kth) {
                x[i] = -1e10f;
                own_max = fmaxf(own_max, -1e10f);  // (only matters when every survivor lies below the sentinel)
            }
        }
        __syncthreads();
    }
    SEL_CLK(g0);
    float mx;
    {
        // (each thread's maximum of its tempered values, with the top-k sentinel where it wrote one)
        float m = warp_max(own_max);
        if (lane == 0) red_v[w] = m;
        __syncthreads();
        m = red_v[0];
        for (int i = 1; i < kSelWarps; i++) m = fmaxf(m, red_v[i]);
        mx = m;
    }
    // softmax (tensor.cpp:434-448): exp(x - max), sequential sum in index order, times 1/sum
    for (int i = tid; i < V; i += kSelThreads) x[i] = expf_libm(__fsub_rn(x[i], mx), s_exp_tab);
    __syncthreads();
    SEL_CLK(g1);
    SEL_ADD(8, g1 - g0);  // maximum and exponentials
    const ScanResult den = exact_scan(V, x, [](float) { return false; }, false, scan_sh, work);
    SEL_CLK(g2);
    SEL_ADD(9, g2 - g1);  // denominator (exact scan)
    const float inv_sum = __fdiv_rn(1.0f, den.sum);
    ProbStats stats;
    for (int i = tid; i < V; i += kSelThreads) {
        const float pr = __fmul_rn(x[i], inv_sum);
        x[i] = pr;
        if (use_p) {
            g[i] = pr;
            stats.add(pr);
        }
    }
    __syncthreads();
    SEL_CLK(g3);
    SEL_ADD(10, g3 - g2);  // probabilities (and their index-order copy)

    if (use_p) {  // text_gen.cpp:158-193
        // The reference sorts (probability, id) pairs; only the sorted VALUES enter its running sum, so the
        // probabilities are sorted directly.
        if (!sort_probs_desc(x, g, V, reinterpret_cast<int*>(work), stats)) {
            __syncthreads();
            float* area = g + V;  // bitonic sort of a padded copy in global memory: slow, and rare
            for (int i = tid; i < p.n_sort; i += kSelThreads) area[i] = i < V ? g[i] : -INFINITY;
            __syncthreads();
            sort_desc(area, p.n_sort);
            for (int i = tid; i < V; i += kSelThreads) x[i] = area[i];
            __syncthreads();
        }
        SEL_CLK(g4);
        SEL_ADD(11, g4 - g3);  // sort
        const float top_p = p.top_p;
        const ScanResult cut = exact_scan(V, x, [top_p](float s) { return s >= top_p; }, true, scan_sh, work);
        const int cutoff = cut.hit < V ? cut.hit : 0;  // never reached: index stays 0
        const float cutoff_prob = x[cutoff];
        __syncthreads();
        SEL_CLK(g5);
        SEL_ADD(12, g5 - g4);  // nucleus cutoff (exact scan with a predicate)
        for (int i = tid; i < V; i += kSelThreads) {
            const float pr = g[i];
            x[i] = pr < cutoff_prob ? 0.0f : pr;
        }
        __syncthreads();
        const ScanResult kept = exact_scan(V, x, [](float) { return false; }, false, scan_sh, work);
        if (kept.sum > 0.0f) {
            const float tk = kept.sum;
            for (int i = tid; i < V; i += kSelThreads) {
                const float v = x[i];
                if (v != 0.0f) x[i] = __fdiv_rn(v, tk);  // (a zero numerator would send the whole warp down the division's slow path)
            }
        }
        __syncthreads();
        SEL_CLK(g6);
        SEL_ADD(13, g6 - g5);  // mask, kept mass (exact scan), renormalisation
    }
    if (p.probs_out) {
        for (int i = tid; i < V; i += kSelThreads) p.probs_out[(size_t)b * V + i] = x[i];
    }
    // draw (text_gen.cpp:199-208): first index with u <= running sum, else the last id
    const float u = p.uniforms[(size_t)b * p.u_stride + (p.loop_mode ? p.gen[b] : 0)];
    const ScanResult dr = exact_scan(V, x, [u](float s) { return u <= s; }, true, scan_sh, work);
    const int pick = dr.hit < V ? dr.hit : V - 1;
    SEL_CLK(g7);
    SEL_ADD(14, g7 - g0);  // the whole stage on the full row, draw included
    SEL_MAX(15, g7 - g0);  // the slowest sequence's

    if (tid == 0) record_pick(p, b, hist, hlen, pick);
}

// Greedy selection without a vocabulary-sized staging buffer: the logits are read once from global memory, the
// (at most 50) penalised entries are kept as a short list of (id, value) overrides in shared memory.
// Any vocabulary size.
constexpr int kGreedyThreads = 512;
constexpr int kGreedyWarps = kGreedyThreads / 32;
constexpr int kPenHash = 128;  // open-addressing table over the <= 50 distinct ids of the window
constexpr int kPenBitWords = 2048;  // bitmap of overridden ids for vocabularies to 65536

__global__ void __launch_bounds__(kGreedyThreads) select_greedy_kernel(const SelectParams p) {
    __shared__ int pen_id[kPenaltyWindow];
    __shared__ float pen_val[kPenaltyWindow];
    __shared__ int pen_n;
    __shared__ int table[kPenHash];  // slot -> index into pen_id, -1 = empty
    __shared__ float red_v[kGreedyWarps];
    __shared__ int red_i[kGreedyWarps];
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int V = p.V;
    pdl_trigger();
    pdl_wait();
    if (p.loop_mode && p.done[b]) return;
    const float* lg = p.logits + (size_t)b * V;
    int* hist = p.hist + (size_t)b * p.hist_stride;
    const int hlen = p.hist_len[b];
    if (tid < kPenHash) table[tid] = -1;
    if (tid == 0) pen_n = 0;
    __syncthreads();
    // ---- repetition penalty: last min(50, n) ids, once per occurrence, in order (text_gen.cpp:20-31)
    if (p.penalty != 1.0f) {
        // The reference walks the window in order and penalises an id once per occurrence. Different ids do not
        // interact and the repeated penalties of one id are applied in sequence by one thread (the window position
        // of its first occurrence), so the positions work side by side with the reference's result; the penalised
        // values become a short list of overrides.
        __shared__ int s_pen_id[kPenaltyWindow];
        const int window = min(kPenaltyWindow, hlen);
        int id = -1;
        if (tid < window) {
            id = hist[hlen - window + tid];
            s_pen_id[tid] = id;
        }
        __syncthreads();
        if (tid < window && GRADB_INDEX_OK(id >= 0 && id < V, p.status, 901)) {
            bool first = true;
            int count = 0;
            for (int k = 0; k < window; k++) {
                const bool same = s_pen_id[k] == id;
                first = first && !(same && k < tid);
                count += same;
            }
            if (first) {
                float v = lg[id];
                for (int c = 0; c < count; c++) v = v > 0 ? __fdiv_rn(v, p.penalty) : __fmul_rn(v, p.penalty);
                const int e = atomicAdd(&pen_n, 1);
                pen_id[e] = id;
                pen_val[e] = v;
            }
        }
        __syncthreads();
        if (tid == 0 && V > kPenBitWords * 32) {  // very large vocabularies look the overrides up in a hash table
            for (int e = 0; e < pen_n; e++) {
                int slot = pen_id[e] & (kPenHash - 1);
                while (table[slot] >= 0) slot = (slot + 1) & (kPenHash - 1);
                table[slot] = e;
            }
        }
    }
    __syncthreads();
    const int n_pen = pen_n;
    // Which ids are overridden: one bit per id (vocabularies to 65536: a single shared-memory word answers for the
    // four ids of a 128-bit load), beyond that the hash table again.
    __shared__ uint32_t pen_bits[kPenBitWords];
    const bool use_bits = n_pen > 0 && V <= kPenBitWords * 32;
    if (use_bits) {
        for (int i = tid; i < (V + 31) / 32; i += kGreedyThreads) pen_bits[i] = 0u;
        __syncthreads();
        if (tid < n_pen) atomicOr(&pen_bits[pen_id[tid] >> 5], 1u << (pen_id[tid] & 31));
        __syncthreads();
    }
    auto overridden = [&](int id) {
        if (n_pen == 0) return false;
        if (use_bits) return ((pen_bits[id >> 5] >> (id & 31)) & 1u) != 0u;
        int slot = id & (kPenHash - 1);
        while (table[slot] >= 0) {
            if (pen_id[table[slot]] == id) return true;
            slot = (slot + 1) & (kPenHash - 1);
        }
        return false;
    };
    // first index of the maximum, strict > (text_gen.cpp:52-60)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto consider = [&](float v, int i) {
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    };
    if ((V & 3) == 0) {
        const float4* lg4 = reinterpret_cast<const float4*>(lg);
        for (int q = tid; q < V / 4; q += kGreedyThreads) {
            const float4 v = __ldcs(lg4 + q);
            const int i = q * 4;
            if (n_pen == 0 || (use_bits && ((pen_bits[i >> 5] >> (i & 31)) & 0xFu) == 0u)) {  // none of the four
                consider(v.x, i);
                consider(v.y, i + 1);
                consider(v.z, i + 2);
                consider(v.w, i + 3);
                continue;
            }
            if (!overridden(i)) consider(v.x, i);
            if (!overridden(i + 1)) consider(v.y, i + 1);
            if (!overridden(i + 2)) consider(v.z, i + 2);
            if (!overridden(i + 3)) consider(v.w, i + 3);
        }
    } else {
        for (int i = tid; i < V; i += kGreedyThreads) {
            if (!overridden(i)) consider(lg[i], i);
        }
    }
    if (tid < n_pen) consider(pen_val[tid], pen_id[tid]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (lane == 0) {
        red_v[w] = bv;
        red_i[w] = bi;
    }
    __syncthreads();
    if (tid == 0) {
        for (int i = 1; i < kGreedyWarps; i++) {
            if (red_v[i] > bv || (red_v[i] == bv && red_i[i] < bi)) {
                bv = red_v[i];
                bi = red_i[i];
            }
        }
        // a NaN in slot 0 is never displaced by the reference's comparison (penalising a NaN leaves a NaN)
        const float x0 = lg[0];
        const int pick = (x0 != x0 || bi == 0x7fffffff) ? 0 : bi;
        record_pick(p, b, hist, hlen, pick);
    }
}

}  // namespace

// Shared memory of the sampled kernel: the vocabulary-sized array, padded to whole 16-term chunks plus one chunk the
// scans may read past the end, and 4096 words of histogram / scan scratch.
size_t select_smem_bytes(int V, int* n_pad_out) {
    const int n_pad = (V + 15) / 16 * 16 + 16;
    if (n_pad_out) *n_pad_out = n_pad;
    return (size_t)n_pad * sizeof(float) + kBuckets * sizeof(int);
}

// Floats of global scratch per sequence: the index-order copy of the probabilities and the area of the fallback sort.
size_t select_scratch_floats(int V) {
    size_t n_sort = 1;
    while (n_sort < (size_t)V) n_sort <<= 1;
    return (size_t)V + n_sort;
}

bool select_sampled_fits(int V) { return select_smem_bytes(V, nullptr) <= 200 * 1024; }

void configure_select(int V) {
    const size_t bytes = select_smem_bytes(V, nullptr);
    if (bytes > 48 * 1024 && bytes <= 200 * 1024) {
        GRADB_CUDA(cudaFuncSetAttribute(select_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        GRADB_CUDA(cudaFuncSetAttribute(select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    // two sequences per SM need the large shared-memory configuration
    GRADB_CUDA(cudaFuncSetAttribute(select_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    (int)cudaSharedmemCarveoutMaxShared));
    GRADB_CUDA(cudaFuncSetAttribute(select_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    (int)cudaSharedmemCarveoutMaxShared));
}

#if GRADB_DIAG
void select_clocks_read(unsigned long long* out16, bool reset) {
    GRADB_CUDA(cudaDeviceSynchronize());
    GRADB_CUDA(cudaMemcpyFromSymbol(out16, g_sel_clock, sizeof(unsigned long long) * 16));
    if (reset) {
        unsigned long long zero[16] = {};
        GRADB_CUDA(cudaMemcpyToSymbol(g_sel_clock, zero, sizeof(zero)));
    }
}
#endif

void launch_select(const SelectParams& p_in, int B, cudaStream_t st) {
    SelectParams p = p_in;
    if (p.greedy) {
        p.n_pad = 0;
        launch_kernel(select_greedy_kernel, dim3(B), dim3(kGreedyThreads), 0, st, p);
        count_launch();
        GRADB_CUDA(cudaGetLastError());
        return;
    }
    const size_t bytes = select_smem_bytes(p.V, &p.n_pad);
    if (bytes > 200 * 1024) {
        throw Error(GRADB_ERR_INVALID,
                    "vocabulary too large for the on-device sampled selection stage (limit 47000 ids; greedy has none)");
    }
    if (!p.scratch) throw Error(GRADB_ERR_INVALID, "sampled selection needs its scratch rows");
    p.scratch_stride = select_scratch_floats(p.V);
    p.n_sort = (int)(p.scratch_stride - (size_t)p.V);
    if (bytes > 48 * 1024 && !g_capturing) {
        GRADB_CUDA(cudaFuncSetAttribute(select_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        GRADB_CUDA(cudaFuncSetAttribute(select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    if (p.top_k > 0 && p.top_k < p.V) launch_kernel(select_kernel<true>, dim3(B), dim3(kSelThreads), bytes, st, p);
    else launch_kernel(select_kernel<false>, dim3(B), dim3(kSelThreads), bytes, st, p);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

}  // namespace gradb
