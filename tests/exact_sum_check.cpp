// Host check of the arithmetic the selection kernel uses to reproduce a
// sequential fp32 sum with a parallel scan (grad.cpp_b200/csrc/exact_sum.h).
// The block of threads is emulated by a loop; the per-term and composition
// code is the very code the kernel compiles.
//
// Usage: exact_sum_check <cases> <seed>; exits non-zero on the first mismatch.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <random>
#include <vector>

#include "../grad.cpp_b200/csrc/exact_sum.h"

using namespace gradb;

static uint32_t fbits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static float bitsf(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

struct Result { float sum; int hit; };

// mode 0: no predicate, 1: s >= thr, 2: thr <= s  (same thing; kept to mirror both call sites)
static bool pred(int mode, float thr, float s) { return mode == 0 ? false : (mode == 1 ? s >= thr : thr <= s); }

static Result sequential(const std::vector<float>& a, int mode, float thr) {
    volatile float s = 0.0f;
    for (size_t i = 0; i < a.size(); i++) {
        s = s + a[i];
        if (pred(mode, thr, s)) return {s, (int)i};
    }
    return {s, (int)a.size()};
}

static Result emulated(const std::vector<float>& a, int mode, float thr, int T) {
    const int n = (int)a.size();
    float s_sum = 0.0f;
    int s_next = 0, s_hit = n;
    for (int guard = 0; guard < 1 << 20; guard++) {
        const int start = s_next;
        if (start >= n || s_hit < n) break;
        const float s0 = s_sum;
        const uint32_t sb = fbits(s0);
        const int sex = (int)(sb >> 23);
        if (s0 == 0.0f) {
            if (pred(mode, thr, 0.0f)) { s_hit = start; break; }
            int j = start;
            while (j < n && a[j] == 0.0f) j++;
            if (j >= n) { s_next = n; continue; }
            s_sum = a[j]; s_next = j + 1;
            if (pred(mode, thr, s_sum)) s_hit = j;
            continue;
        }
        if (sex < 30 || sex >= 254) {
            volatile float s = s0;
            int i = start;
            const int stop = std::min(n, start + 64);
            while (i < stop) {
                s = s + a[i]; i++;
                if (pred(mode, thr, s)) { s_hit = i - 1; break; }
                const int e2 = (int)(fbits(s) >> 23);
                if (e2 >= 30 && e2 < 254) break;
            }
            s_sum = s; s_next = i;
            continue;
        }
        const int ue = sex - 150;
        const uint32_t S0 = (sb & 0x7fffffu) | 0x800000u;
        const int per = (n - start + T - 1) / T;
        std::vector<IncPair> loc(T);
        for (int t = 0; t < T; t++) {
            const int beg = std::min(n, start + t * per), end = std::min(n, beg + per);
            IncPair l = {0u, 0u};
            for (int i = beg; i < end; i++) l = compose(l, term_inc(fbits(a[i]), ue));
            loc[t] = l;
        }
        int stop = n, kind = 0; float stop_sum = 0.f; uint32_t lastS = S0; bool have_last = false;
        IncPair ahead = {0u, 0u};
        for (int t = 0; t < T; t++) {
            const int beg = std::min(n, start + t * per), end = std::min(n, beg + per);
            uint32_t S = step_S(S0, ahead);
            if (S < kBinadeEnd && stop == n) {
                for (int i = beg; i < end; i++) {
                    const uint32_t Sn = step_S(S, term_inc(fbits(a[i]), ue));
                    if (Sn >= kBinadeEnd) { stop = i; kind = 2; break; }
                    S = Sn;
                    const float sv = bitsf(((uint32_t)sex << 23) | (S & 0x7fffffu));
                    if (pred(mode, thr, sv)) { stop = i; kind = 1; break; }
                }
                if (stop < n) {
                    stop_sum = bitsf(((uint32_t)sex << 23) | (S & 0x7fffffu));
                } else if (end == n && beg < end) {
                    lastS = S; have_last = true;
                }
            }
            ahead = compose(ahead, loc[t]);
        }
        if (stop < n) {
            s_next = stop + 1;
            if (kind == 1) { s_hit = stop; s_sum = stop_sum; }
            else {
                volatile float s2 = stop_sum; s2 = s2 + a[stop];
                s_sum = s2;
                if (pred(mode, thr, s_sum)) s_hit = stop;
            }
        } else {
            if (!have_last) { std::fprintf(stderr, "emulation: nobody owns the last term\n"); std::exit(3); }
            s_sum = bitsf(((uint32_t)sex << 23) | (lastS & 0x7fffffu));
            s_next = n;
        }
    }
    return {s_sum, s_hit};
}

// Host emulation of the one-sweep scan (select_kernels.cu::seq_scan_fast): double prefix sum to
// predict each 16-term chunk's binade, maps of safe chunks composed per run, unsafe chunks added
// natively, exact sums carried by one walker, predicate tested per chunk from its exact start.
// Returns false when the sweep declines (the kernel then falls back to the pass-per-binade scan).
static bool emulated_fast(const std::vector<float>& a, int mode, float thr, Result& out, long* unsafe_chunks) {
    const int n = (int)a.size(), PER = 16, PREFIX = 128;
    int i = 0;
    while (i < n && a[i] == 0.0f) i++;
    volatile float s = 0.0f;
    int h = n;
    if (pred(mode, thr, 0.0f)) { out = {0.0f, 0}; return true; }
    if (i == n) { out = {0.0f, n}; return true; }
    {
        const int stop = std::min(n, i + PREFIX);
        while (i < stop && h == n) { s = s + a[i]; if (pred(mode, thr, s)) h = i; i++; }
    }
    if (h < n || i >= n) { out = {s, h}; return true; }
    const int start = i;
    const float s0 = s;
    const int chunks = (n - start + PER - 1) / PER;
    if (chunks > 1024) return false;
    std::vector<int> info(chunks);
    std::vector<IncPair> cmap(chunks);
    std::vector<double> dsum(chunks);
    double P = (double)s0;
    for (int c = 0; c < chunks; c++) {
        const int b = start + c * PER, e = std::min(n, b + PER);
        double d = 0; for (int k = b; k < e; k++) d += (double)a[k];
        const float lo = (float)(P * (1.0 - 1.0 / 512.0)), hi = (float)((P + d) * (1.0 + 1.0 / 512.0));
        const int elo = (int)(fbits(lo) >> 23), ehi = (int)(fbits(hi) >> 23);
        const bool safe = elo == ehi && elo >= 30 && elo < 254;
        info[c] = safe ? elo : -1;
        IncPair m = {0u, 0u};
        if (safe) {  // as the kernel builds it: increments added up when no term is a tie, maps composed otherwise
            uint32_t total = 0u, tie = 0u;
            const float inv_u = unit_reciprocal(elo - 150);
            for (int k0 = b; k0 < e; k0 += 4) {  // four at a time, as the kernel adds them
                float four = 0.0f;
                for (int k = k0; k < std::min(e, k0 + 4); k++) four += term_inc_float(a[k], inv_u, &tie);
                total += (uint32_t)four;
            }
            IncPair composed = {0u, 0u};
            for (int k = b; k < e; k++) composed = compose(composed, term_inc(fbits(a[k]), elo - 150));
            if (tie == 0u) {
                m.e = m.o = sat(total);
                if (composed.e != m.e || composed.o != m.o) {
                    std::fprintf(stderr, "PLAIN MAP MISMATCH chunk %d\n", c);
                    std::exit(1);
                }
            } else {
                m = composed;
            }
        }
        cmap[c] = m;
        P += d;
        if (!safe) (*unsafe_chunks)++;
    }
    float cur = s0;
    int c = 0;
    while (c < chunks && h == n) {
        if (info[c] < 0) {
            const int b = start + c * PER, e = std::min(n, b + PER);
            volatile float v = cur;
            for (int k = b; k < e && h == n; k++) { v = v + a[k]; if (pred(mode, thr, v)) h = k; }
            cur = v;
            c++;
            continue;
        }
        const int e = info[c];
        int c1 = c;
        while (c1 + 1 < chunks && info[c1 + 1] == e) c1++;
        const uint32_t sb = fbits(cur);
        if ((int)(sb >> 23) != e) return false;
        const uint32_t S0 = (sb & 0x7fffffu) | 0x800000u;
        uint32_t S = S0;
        // walk chunk by chunk (the kernel composes with a segmented scan; composition is checked too)
        IncPair run = {0u, 0u};
        for (int cc = c; cc <= c1; cc++) run = compose(run, cmap[cc]);
        const uint32_t S1 = step_S(S0, run);
        if (S1 >= kBinadeEnd) return false;
        const float after = bitsf(((uint32_t)e << 23) | (S1 & 0x7fffffu));
        if (mode != 0 && pred(mode, thr, after)) {
            // find the exact index inside the run
            for (int cc = c; cc <= c1 && h == n; cc++) {
                const int b = start + cc * PER, ee = std::min(n, b + PER);
                for (int k = b; k < ee; k++) {
                    S = step_S(S, term_inc(fbits(a[k]), e - 150));
                    if (pred(mode, thr, bitsf(((uint32_t)e << 23) | (S & 0x7fffffu)))) { h = k; break; }
                }
            }
            if (h == n) return false;  // cannot happen: the run's end satisfied the predicate
        }
        cur = after;
        c = c1 + 1;
    }
    out = {cur, h};
    return true;
}

int main(int argc, char** argv) {
    const int cases = argc > 1 ? std::atoi(argv[1]) : 2000;
    std::mt19937 rng(argc > 2 ? std::atoi(argv[2]) : 1);
    std::uniform_real_distribution<float> U(0.0f, 1.0f);
    std::normal_distribution<float> N(0.0f, 1.0f);
    long checked = 0, fast_ok = 0, fast_declined = 0, unsafe_chunks = 0;
    for (int c = 0; c < cases; c++) {
        const int kind = c % 8;
        const int n = 1 + (int)(rng() % (kind == 7 ? 20000 : 3000));
        std::vector<float> a(n);
        float scale = std::ldexp(1.0f, (int)(rng() % 40) - 30);
        for (int i = 0; i < n; i++) {
            switch (kind) {
                case 0: a[i] = U(rng) * scale; break;                       // plain
                case 1: a[i] = std::exp(N(rng) * 3.0f) * scale; break;      // wide dynamic range
                case 2: a[i] = (rng() % 4 == 0) ? U(rng) * scale : 0.0f; break;  // many zeros
                case 3: a[i] = std::ldexp((float)(1 + rng() % 7), (int)(rng() % 12) - 40); break;  // exact ties likely
                case 4: a[i] = std::ldexp(1.0f, -(int)(rng() % 30)); break; // powers of two: ties everywhere
                case 5: a[i] = U(rng) < 0.01f ? 1.0f : std::ldexp(1.0f, -24) * (float)(rng() % 3); break;  // half-ulp steps
                case 6: a[i] = bitsf((rng() % 0x00800000u) | ((rng() % 3) << 23)); break;  // subnormal/tiny
                default: a[i] = std::exp(N(rng) * 0.7f - 9.0f); break;      // probability-like
            }
        }
        if (kind == 7 || c % 3 == 0) std::sort(a.begin(), a.end(), [](float x, float y) { return x > y; });
        const Result full = sequential(a, 0, 0.f);
        for (int mode = 0; mode < 3; mode++) {
            const float thr = mode == 0 ? 0.f : full.sum * U(rng) * 1.1f;
            const Result want = sequential(a, mode, thr);
            {
                Result fast{};
                if (emulated_fast(a, mode, thr, fast, &unsafe_chunks)) {
                    fast_ok++;
                    const bool sum_ok = mode != 0 || fbits(fast.sum) == fbits(want.sum);
                    if (!sum_ok || fast.hit != want.hit) {
                        std::fprintf(stderr, "FAST MISMATCH case %d kind %d n %d mode %d: sum %a vs %a, hit %d vs %d\n", c,
                                     kind, n, mode, fast.sum, want.sum, fast.hit, want.hit);
                        return 1;
                    }
                } else {
                    fast_declined++;
                }
            }
            for (int T : {1, 7, 64, 1024}) {
                const Result got = emulated(a, mode, thr, T);
                checked++;
                if (fbits(got.sum) != fbits(want.sum) || got.hit != want.hit) {
                    std::fprintf(stderr, "MISMATCH case %d kind %d n %d mode %d T %d: sum %a vs %a, hit %d vs %d\n", c,
                                 kind, n, mode, T, got.sum, want.sum, got.hit, want.hit);
                    return 1;
                }
            }
        }
    }
    std::printf("ok %ld comparisons; one-sweep path: %ld exact, %ld declined, %ld unsafe chunks\n", checked, fast_ok,
                fast_declined, unsafe_chunks);
    return 0;
}
