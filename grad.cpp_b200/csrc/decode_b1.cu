// One decode step of a single sequence (InferenceSession::step, inference.cpp:150-258)
// as ONE persistent cooperative kernel.
//
// At batch 1 every projection is a matrix-vector product that streams its weights
// once; the step is bound by HBM bandwidth and, before that, by latency: some forty
// dependent stages of a few microseconds each. This kernel removes the per-stage
// launch and the cold start of every stage's weight stream:
//
//  * one CTA per SM stays resident for the whole step; there is no grid-wide barrier: every
//    value that crosses CTAs carries its own "ready" mark, and a consumer polls (bounded)
//    exactly the values it needs, so a CTA whose inputs have arrived proceeds at once;
//  * the weights are re-tiled when the model is loaded so that everything one CTA
//    needs for one stage is a single contiguous block; a producer warp walks the
//    step's fixed list of blocks and keeps a four-slot shared-memory ring full with
//    bulk asynchronous copies (TMA, mbarrier completion). The HBM stream therefore
//    runs ahead of the arithmetic, through barriers and reductions;
//  * vectors exchanged between CTAs live in a small global workspace that stays in L2, in two
//    forms. Point-to-point vectors (q, the new K/V row, attention partials) are stored as
//    64-bit {value, epoch} words: one store publishes value and mark together, no fence, and a
//    reader accepts a word only when it carries the epoch of the stage it waits for. Sums over
//    many CTAs (output projection, FFN down) meet in 64-bit fixed-point accumulators whose low
//    bits count the contributions: integer adds commute, so the sum does not depend on arrival
//    order, and a reader accepts an element once its count is complete;
//  * every CTA keeps its own copy of the residual stream in shared memory.
//
// Stages per layer: A norm1+QKV(+RoPE, cache write) | B attention over the cache,
// split along the context | C output projection | D residual+norm2+FFN up (GELU or
// SwiGLU) and, in the same stage, the FFN down product of this CTA's hidden units with
// their rows of the down matrix, added into a fixed-point accumulator that every CTA
// reads in the next stage A; then final norm + tied-embedding logits.
#include <cooperative_groups.h>

#include "decode_b1.cuh"

namespace gradb {

namespace {

constexpr int kCompute = 256;  // compute threads (8 warps)
constexpr int kThreadsB1 = kCompute + 32;  // + producer warp
constexpr int kWarpsB1 = kCompute / 32;
constexpr int kHold = 4;  // vector elements per compute thread: d <= kHold * kCompute
constexpr int kSlots = 4;
constexpr int kSlotBytes = 48 * 1024;
constexpr uint32_t kPollLimit = 1u << 22;   // mbarrier waits (each try suspends for a while)
constexpr uint32_t kSpinLimit = 1u << 20;   // polls of global memory (about a microsecond each)
constexpr int kMaxLayersB1 = 32;  // layer tables are staged in shared memory
// Elements of the fixed-point FFN accumulator sit one per 128-byte line: every CTA adds to every element at
// about the same time, and same-line atomics queue up in one L2 slice.
constexpr int kAccStride = 16;  // in 64-bit words

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, %0;" ::"n"(kCompute) : "memory"); }

// Barrier over the compute threads that also agrees on whether the kernel is giving up: every thread gets the same
// answer, so all of them leave the stage loop together (a plain read of the flag could split them across a barrier).
__device__ __forceinline__ bool cta_dead(volatile int* abort_flag) {
    const uint32_t mine = (uint32_t)*abort_flag;
    uint32_t any;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 p, %1, 0;\n"
        "bar.red.or.pred q, 1, %2, p;\n"
        "selp.u32 %0, 1, 0, q;\n"
        "}\n"
        : "=r"(any)
        : "r"(mine), "n"(kCompute)
        : "memory");
    return any != 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Stage timestamps of CTA 0: compiled in only in the diagnostics build, and there only when a trace was asked for.
struct Tracer {
    unsigned long long* buf;
    int n;
    __device__ __forceinline__ void stamp() {
#if GRADB_DIAG
        if (buf) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            buf[n++] = now;
        }
#endif
    }
};

struct Ring {
    uint64_t* full;
    uint64_t* empty;
    uint8_t* slots;
    int* status;
    volatile int* abort_flag;
    uint32_t n;  // chunks consumed / produced so far
    uint64_t policy;  // producer: L2 evict-first for the weight stream (read once per step; the exchange words and the
                      // K/V rows are what should stay in L2)
};

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, volatile int* abort_flag,
                                          int code) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < kPollLimit; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
    }
    atomicExch(status, code);
    *abort_flag = 1;
    return false;
}

// Producer side: copy `bytes` from global into the next slot.
__device__ __forceinline__ void ring_push(Ring& r, const void* src, uint32_t bytes) {
    const uint32_t s = r.n % kSlots, ph = (r.n / kSlots) & 1;
    if (!mbar_wait(&r.empty[s], ph ^ 1, r.status, r.abort_flag, 211)) return;
    const uint32_t bar = smem_u32(&r.full[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(r.slots + (size_t)s * kSlotBytes)),
        "l"(src), "r"(bytes), "r"(bar), "l"(r.policy)
        : "memory");
    r.n++;
}

// Consumer side: wait for the next chunk, return its address.
__device__ __forceinline__ const uint8_t* ring_acquire(Ring& r) {
    const uint32_t s = r.n % kSlots, ph = (r.n / kSlots) & 1;
    mbar_wait(&r.full[s], ph, r.status, r.abort_flag, 212);
    return r.slots + (size_t)s * kSlotBytes;
}
__device__ __forceinline__ void ring_release(Ring& r) {
    const uint32_t s = r.n % kSlots;
    bar_compute();  // every compute thread has finished reading the slot
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&r.empty[s])) : "memory");
    }
    r.n++;
}

// ---- exchange between CTAs without a barrier
// {value, epoch} words: the 64-bit store is single-copy atomic, so a reader sees the value that belongs to the mark.
__device__ __forceinline__ void ll_store(unsigned long long* p, float v, uint32_t epoch) {
    const unsigned long long w = ((unsigned long long)epoch << 32) | __float_as_uint(v);
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_vol64(const void* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Waits (bounded) until every one of the N words carries `epoch`; on expiry the status word is set.
template <int N>
__device__ __forceinline__ void ll_wait(const unsigned long long* const (&ptr)[N], const bool (&want)[N], uint32_t epoch,
                                        float (&out)[N], int* status, volatile int* abort_flag, int code) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        unsigned long long w[N];
#pragma unroll
        for (int i = 0; i < N; i++) w[i] = want[i] ? ld_vol64(ptr[i]) : ((unsigned long long)epoch << 32);
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; i++) ok = ok && (uint32_t)(w[i] >> 32) == epoch;
        if (ok) {
#pragma unroll
            for (int i = 0; i < N; i++) out[i] = __uint_as_float((uint32_t)w[i]);
            return;
        }
        if (*abort_flag) break;
    }
#pragma unroll
    for (int i = 0; i < N; i++) out[i] = 0.f;
    if (!*abort_flag) {
        atomicExch(status, code);
        *abort_flag = 1;
    }
}

// Fixed-point accumulators: units of 2^-32 above kCountBits of contribution count.
constexpr int kCountBits = 10;  // up to 1023 contributing CTAs
__device__ __forceinline__ void acc_add(long long* p, float y) {
    const long long q = __double2ll_rn((double)y * 4294967296.0);
    const unsigned long long add = ((unsigned long long)q << kCountBits) + 1ull;
    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(p), "l"(add) : "memory");
}
__device__ __forceinline__ float acc_value(unsigned long long w) {
    return (float)((double)((long long)w >> kCountBits) * 2.3283064365386963e-10);
}

// x_s += bias + the KS partial vectors part[ks][d] (marked words), added in slice order once all have arrived.
__device__ bool add_partials(float* x_s, const float* bias, const unsigned long long* part, int KS, uint32_t epoch, int d,
                             int* status, volatile int* abort_flag, int code) {
    float bv[kHold];
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        bv[i] = (bias && k < d) ? __ldg(bias + k) : 0.f;
    }
    if (KS <= 4) {  // every word of this thread in one round of loads
        const unsigned long long* ptr[4 * kHold];
        bool want[4 * kHold];
        float o[4 * kHold];
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            const int k = threadIdx.x + i * kCompute;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                ptr[4 * i + u] = part + (size_t)min(u, KS - 1) * d + min(k, d - 1);
                want[4 * i + u] = k < d && u < KS;
            }
        }
        ll_wait<4 * kHold>(ptr, want, epoch, o, status, abort_flag, code);
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            const int k = threadIdx.x + i * kCompute;
            if (k < d) {
                float acc = x_s[k] + bv[i];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (u < KS) acc += o[4 * i + u];
                }
                x_s[k] = acc;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            const int k = threadIdx.x + i * kCompute;
            if (k < d) {
                float acc = x_s[k] + bv[i];
                for (int s0 = 0; s0 < KS; s0 += 4) {
                    const unsigned long long* ptr[4];
                    bool want[4];
                    float o[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        ptr[u] = part + (size_t)min(s0 + u, KS - 1) * d + k;
                        want[u] = s0 + u < KS;
                    }
                    ll_wait<4>(ptr, want, epoch, o, status, abort_flag, code);
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (s0 + u < KS) acc += o[u];
                    }
                }
                x_s[k] = acc;
            }
        }
    }
    return cta_dead(abort_flag);
}

// x_s += bias + the accumulated vector, once all `expected` contributions of every element have landed.
__device__ bool add_accumulated(float* x_s, const float* bias, const long long* acc, uint32_t expected, int d, int* status,
                                volatile int* abort_flag, int code) {
    float bv[kHold];
    unsigned long long w[kHold];
    bool pend[kHold];
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        pend[i] = k < d;
        bv[i] = (bias && k < d) ? __ldg(bias + k) : 0.f;
        w[i] = 0ull;
    }
    bool gave_up = true;
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        bool all = true;
#pragma unroll
        for (int i = 0; i < kHold; i++) {  // all loads of a round are issued together
            if (pend[i]) w[i] = ld_vol64(acc + (size_t)(threadIdx.x + i * kCompute) * kAccStride);
        }
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            if (pend[i]) pend[i] = (uint32_t)(w[i] & ((1u << kCountBits) - 1u)) != expected;
            all = all && !pend[i];
        }
        if (all || *abort_flag) {
            gave_up = !all;
            break;
        }
    }
    if (gave_up && !*abort_flag) {
        atomicExch(status, code);
        *abort_flag = 1;
    }
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        if (k < d) x_s[k] = (x_s[k] + bv[i]) + acc_value(w[i]);
    }
    return cta_dead(abort_flag);
}

__device__ __forceinline__ float4 ld_tile4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld_tile4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ float ld_tile1(const float* p) { return *p; }
__device__ __forceinline__ float ld_tile1(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// out_s[0..CW) = in_s[0..rows) @ tile, the tile arriving through the ring in chunks of
// whole rows. All compute threads call this together.
// `rows` of the tile's Kt (zero padded) rows carry data. CW is 16, 32 or 64.
template <typename WT>
__device__ void tile_matvec(Ring& ring, const float* in_s, int rows, int Kt, int CW, float* red_s, float* out_s,
                            Tracer& tr) {
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    const int lg = 31 - __clz(CW) - 2;                 // log2 of the column groups (four columns each)
    const int cg = 1 << lg, R = kCompute >> lg;
    const int c4 = t & (cg - 1), r0 = t >> lg;
    const int chunk_rows = (kSlotBytes / (int)sizeof(WT)) >> (lg + 2);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < Kt; base += chunk_rows) {  // same chunking as the producer's
        const int n = min(chunk_rows, rows - base);
        const bool last = base + chunk_rows >= Kt;
        const WT* tile = reinterpret_cast<const WT*>(ring_acquire(ring));
        tr.stamp();
        const WT* tp = tile + ((size_t)r0 << (lg + 2)) + c4 * 4;
        const float* xp = in_s + base + r0;
        const size_t tstep = (size_t)R << (lg + 2);
        int k = r0;
        for (; k + 3 * R < n; k += 4 * R) {  // four rows in flight
            const float4 w0 = ld_tile4(tp), w1 = ld_tile4(tp + tstep), w2 = ld_tile4(tp + 2 * tstep),
                         w3 = ld_tile4(tp + 3 * tstep);
            const float x0 = xp[0], x1 = xp[R], x2 = xp[2 * R], x3 = xp[3 * R];
            acc.x += x0 * w0.x; acc.y += x0 * w0.y; acc.z += x0 * w0.z; acc.w += x0 * w0.w;
            acc.x += x1 * w1.x; acc.y += x1 * w1.y; acc.z += x1 * w1.z; acc.w += x1 * w1.w;
            acc.x += x2 * w2.x; acc.y += x2 * w2.y; acc.z += x2 * w2.z; acc.w += x2 * w2.w;
            acc.x += x3 * w3.x; acc.y += x3 * w3.y; acc.z += x3 * w3.z; acc.w += x3 * w3.w;
            tp += 4 * tstep;
            xp += 4 * R;
        }
        for (; k < n; k += R) {
            const float4 wv = ld_tile4(tp);
            const float xv = xp[0];
            acc.x += xv * wv.x; acc.y += xv * wv.y; acc.z += xv * wv.z; acc.w += xv * wv.w;
            tp += tstep;
            xp += R;
        }
        if (!last) ring_release(ring);
    }
    tr.stamp();
    for (int o = cg; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (lane < cg) *reinterpret_cast<float4*>(&red_s[w * 64 + lane * 4]) = acc;
    // one barrier both hands the last slot back and publishes the per-warp sums
    ring_release(ring);
    if (t < CW) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kWarpsB1; i++) s += red_s[i * 64 + t];
        out_s[t] = s;
    }
    bar_compute();
}

// Sum over the compute threads; every thread gets the total (fixed order).
__device__ __forceinline__ float block_total(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) sh[w] = v;
    bar_compute();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kWarpsB1; i++) s += sh[i];
    bar_compute();
    return s;
}

// Gain and shift of a norm, fetched into registers a stage ahead of their use (an L2 round trip is most of what a
// norm of a few hundred elements would otherwise take).
struct NormVec {
    float g[kHold], b[kHold];
    __device__ __forceinline__ void fetch(const float* gamma, const float* beta, int d, int rms) {
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            const int k = threadIdx.x + i * kCompute;
            g[i] = k < d ? __ldg(gamma + k) : 0.f;
            b[i] = (k < d && !rms) ? __ldg(beta + k) : 0.f;
        }
    }
};

// in_s = norm(x_s) (inference.cpp:30-58).
__device__ void norm_vec(const float* x_s, float* in_s, const NormVec& nv, int d, int rms, float* sh) {
    float xv[kHold];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        xv[i] = k < d ? x_s[k] : 0.f;
        s += rms ? xv[i] * xv[i] : xv[i];
    }
    s = block_total(s, sh);
    float mean = 0.f, r;
    if (rms) {
        r = 1.0f / sqrtf(s / (float)d + 1e-5f);
    } else {
        mean = s / (float)d;
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            const int k = threadIdx.x + i * kCompute;
            const float dl = xv[i] - mean;
            if (k < d) v += dl * dl;
        }
        v = block_total(v, sh);
        r = 1.0f / sqrtf(v / (float)d + 1e-5f);
    }
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        if (k < d) in_s[k] = rms ? nv.g[i] * xv[i] * r : nv.g[i] * (xv[i] - mean) * r + nv.b[i];
    }
    bar_compute();
}

template <typename WT>
__global__ void __launch_bounds__(kThreadsB1, 1) decode_b1_kernel(const B1Params p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kSlots], empty_bar[kSlots];
    __shared__ float red_s[kWarpsB1 * 64];
    __shared__ float out_s[64], out2_s[64], hid_s[64];
    __shared__ float sh[kWarpsB1];
    __shared__ volatile int abort_flag;
    __shared__ B1Layer layers_s[kMaxLayersB1];

    const int g = blockIdx.x, t = threadIdx.x;
    const int token = p.tok[0];
    if (token < 0) return;  // the sequence takes no part in this step (uniform over the grid)
    const int pos = p.pos[0];
    if (!GRADB_INDEX_OK(token < p.V && pos >= 0 && pos < p.T, p.status, 903)) return;  // uniform over the grid
    const bool do_logits = p.logit_tok[0] >= 0;
    const unsigned step = p.sync[0];  // steps this session has run: names the epochs and the accumulator set of this launch
    const int d = p.d, hs = p.hs;

    uint8_t* slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    float* x_s = reinterpret_cast<float*>(slots + (size_t)kSlots * kSlotBytes);
    float* in_s = x_s + d;  // input vector of the current projection: max(d, largest K slice) floats

    {
        // per-layer pointer tables: one coalesced copy now instead of a dependent load per use
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.layers);
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(layers_s);
        const int words = p.L * (int)(sizeof(B1Layer) / 8);
        for (int i = t; i < words; i += kThreadsB1) dst[i] = __ldg(src + i);
    }
    if (t == 0) {
        for (int s = 0; s < kSlots; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty_bar[s])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_flag = 0;
        // This CTA has read its launch state (token, position, step): the words may change once every CTA has.
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync + 1) : "memory");
    }
    __syncthreads();
    Ring ring{full_bar, empty_bar, slots, p.status, &abort_flag, 0, 0};

    if (t >= kCompute) {
        // ---------------------------------------------------------------- producer warp
        if (t == kCompute) {
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(ring.policy));
            const uint32_t wb = (uint32_t)p.wbytes;
            auto push_tile = [&](const void* basep, const B1Mat& m) {
                const uint8_t* src = static_cast<const uint8_t*>(basep) + (size_t)g * m.tile_elems * wb;
                const int chunk_rows = kSlotBytes / (m.CW * (int)wb);
                for (int r = 0; r < m.Kt && !abort_flag; r += chunk_rows) {
                    const int n = min(chunk_rows, m.Kt - r);
                    ring_push(ring, src + (size_t)r * m.CW * wb, (uint32_t)n * m.CW * wb);
                }
            };
            for (int l = 0; l < p.L && !abort_flag; l++) {
                const B1Layer* ly = layers_s + l;
                if (g < p.qkv.tiles) push_tile(ly->qkv, p.qkv);
                if (g < p.o.tiles) push_tile(ly->o, p.o);
                if (g < p.up.tiles) {
                    if (p.modern) push_tile(ly->gate, p.up);
                    push_tile(ly->up, p.up);
                }
                if (g < p.up.tiles) {  // rows [g*CW, g*CW + CW) of the down matrix, whole rows per chunk
                    const int row0 = g * p.up.CW, nrows = min(p.up.CW, p.dff - row0);
                    const int chunk_rows = kSlotBytes / (p.d * (int)wb);
                    const uint8_t* src = static_cast<const uint8_t*>(ly->down) + (size_t)row0 * p.d * wb;
                    for (int r = 0; r < nrows && !abort_flag; r += chunk_rows) {
                        const int n = min(chunk_rows, nrows - r);
                        ring_push(ring, src + (size_t)r * p.d * wb, (uint32_t)n * p.d * wb);
                    }
                }
            }
            if (do_logits) {
                const int r0 = g * p.logit_rows_per_cta, r1 = min(p.V, r0 + p.logit_rows_per_cta);
                for (int r = r0; r < r1 && !abort_flag; r += p.logit_chunk_rows) {
                    const int n = min(p.logit_chunk_rows, r1 - r);
                    ring_push(ring, static_cast<const uint8_t*>(p.emb_w) + (size_t)r * d * wb, (uint32_t)n * d * wb);
                }
            }
        }
        return;
    }

    // -------------------------------------------------------------------- compute warps
    const int lane = t & 31, w = t >> 5;
    Tracer tr{(p.trace && g == 0 && t == 0) ? p.trace : nullptr, 0};
    auto stamp = [&]() { tr.stamp(); };
    stamp();

    // Accumulators come in two sets, used by alternate steps. The set of the NEXT step is cleared here: its last
    // readers finished with the previous launch, and its next adds come with the next one.
    const size_t acc_set = (size_t)p.L * d * kAccStride;  // words per set: one FFN accumulator per layer
    long long* acc_mine = p.acc + (size_t)(step & 1u) * acc_set;
    {
        long long* other = p.acc + (size_t)((step + 1u) & 1u) * acc_set;
        for (int k = g * kCompute + t; k < p.L * d; k += p.G * kCompute) other[(size_t)k * kAccStride] = 0;
    }
    // Epoch of an exchange: unique per (step, layer, kind), never 0 (the workspace starts zeroed).
    const uint32_t epoch0 = step * (uint32_t)(4 * p.L + 1) + 1u;

    // x = E[token] (+ P[pos])  (inference.cpp:159-182)
    for (int k = t; k < d; k += kCompute) {
        float v = __ldg(p.emb32 + (size_t)token * d + k);
        if (p.pos_emb) v += __ldg(p.pos_emb + (size_t)pos * d + k);
        x_s[k] = v;
    }
    bar_compute();

    // context splits of the attention: one per 64 cached positions, so short contexts exchange few partials
    const int S = max(1, min(p.attn_splits, (pos + 64) / 64));
    const float scale = 1.0f / sqrtf((float)hs);

    NormVec nv1, nv2;  // gains/shifts of the next norm1 and norm2, fetched a stage early
    nv1.fetch(layers_s[0].n1g, layers_s[0].n1b, d, p.modern);
    for (int l = 0; l < p.L; l++) {
        const B1Layer* ly = layers_s + l;
        float* kc = p.kcache + (size_t)l * p.layer_cache_stride;
        float* vc = p.vcache + (size_t)l * p.layer_cache_stride;
        long long* acc_f = acc_mine + (size_t)l * d * kAccStride;
        const uint32_t ep_q = epoch0 + 4u * l, ep_kv = ep_q + 1u, ep_att = ep_q + 2u, ep_o = ep_q + 3u;

        // ---- A: (previous FFN output joins the residual) norm1, Q/K/V columns of this CTA
        if (l > 0 && add_accumulated(x_s, (layers_s + l - 1)->b2, acc_f - (size_t)d * kAccStride, (uint32_t)p.up.tiles,
                                     d, p.status, &abort_flag, 221)) {
            break;
        }
        if (g < p.qkv.tiles) {
            const int CW = p.qkv.CW;
            // this thread's output pair: fetch its bias and rotation before the heavy part
            const int n = g * CW + 2 * t;  // column among the 3d outputs
            const bool mine = t < CW / 2 && n < 3 * d;
            const int which = mine ? n / d : 0, n_in = mine ? n - which * d : 0;
            const int h = n_in / hs, c_in = n_in % hs;
            float b0 = 0.f, b1 = 0.f, cs = 1.f, sn = 0.f;
            if (mine) {
                const float* bias = which == 0 ? ly->bq : (which == 1 ? ly->bk : ly->bv);
                b0 = __ldg(bias + n_in);
                b1 = __ldg(bias + n_in + 1);
                if (p.rope_cos && which < 2) {
                    cs = __ldg(p.rope_cos + (size_t)pos * (hs / 2) + c_in / 2);
                    sn = __ldg(p.rope_sin + (size_t)pos * (hs / 2) + c_in / 2);
                }
            }
            stamp();
            norm_vec(x_s, in_s, nv1, d, p.modern, sh);
            stamp();
            tile_matvec<WT>(ring, in_s, d, p.qkv.Kt, p.qkv.CW, red_s, out_s, tr);
            stamp();
            if (mine) {
                float a0 = out_s[2 * t] + b0, a1 = out_s[2 * t + 1] + b1;
                if (p.rope_cos && which < 2) {  // inference.cpp:101-115
                    const float r0 = a0 * cs - a1 * sn, r1 = a0 * sn + a1 * cs;
                    a0 = r0;
                    a1 = r1;
                }
                if (which == 0) {
                    ll_store(p.q_ll + n_in, a0, ep_q);
                    ll_store(p.q_ll + n_in + 1, a1, ep_q);
                } else {
                    // the new row: to this step's readers through the marked copy, to later steps through the cache
                    unsigned long long* row = p.kv_ll + (size_t)(which - 1) * d + n_in;
                    ll_store(row, a0, ep_kv);
                    ll_store(row + 1, a1, ep_kv);
                    float* cache = which == 1 ? kc : vc;
                    *reinterpret_cast<float2*>(cache + ((size_t)h * p.T + pos) * hs + c_in) = make_float2(a0, a1);
                }
            }
        }
        if (cta_dead(&abort_flag)) break;  // also: out_s is free for the next stage
        stamp();

        // ---- B: attention of (head, context split) g over the cached positions (inference.cpp:208-225)
        nv2.fetch(ly->n2g, ly->n2b, d, p.modern);
        if (g < p.H * S) {
            const int head = g / S, split = g % S;
            const int ctx = pos + 1;
            const int cps = (ctx + S - 1) / S;
            const int t0 = split * cps, t1 = min(ctx, t0 + cps);
            const float* K = kc + (size_t)head * p.T * hs;
            const float* V = vc + (size_t)head * p.T * hs;
            float2 qv;
            {
                const unsigned long long* const ptr[2] = {p.q_ll + head * hs + 2 * lane, p.q_ll + head * hs + 2 * lane + 1};
                const bool want[2] = {true, true};
                float o[2];
                ll_wait<2>(ptr, want, ep_q, o, p.status, &abort_flag, 222);
                qv = make_float2(o[0], o[1]);
            }
            stamp();
            float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;
            // eight positions per trip: their K and V rows are requested together; the newest position's rows come
            // from this step's producers
            constexpr int kTrip = 8;
            for (int tt = t0 + w; tt < t1; tt += kTrip * kWarpsB1) {
                float2 kv[kTrip], vv[kTrip];
#pragma unroll
                for (int u = 0; u < kTrip; u++) {
                    const int tu = tt + u * kWarpsB1;
                    if (tu < t1 && tu != pos) {
                        kv[u] = __ldcg(reinterpret_cast<const float2*>(K + (size_t)tu * hs) + lane);
                        vv[u] = __ldcg(reinterpret_cast<const float2*>(V + (size_t)tu * hs) + lane);
                    }
                }
                if (pos >= tt && pos < t1 && (pos - tt) % kWarpsB1 == 0) {  // warp-uniform: this trip holds the newest row
                    const int u_new = (pos - tt) / kWarpsB1;
                    const unsigned long long* kr = p.kv_ll + head * hs + 2 * lane;
                    const unsigned long long* const ptr[4] = {kr, kr + 1, kr + d, kr + d + 1};
                    const bool want[4] = {true, true, true, true};
                    float o[4];
                    ll_wait<4>(ptr, want, ep_kv, o, p.status, &abort_flag, 223);
#pragma unroll
                    for (int u = 0; u < kTrip; u++) {
                        if (u == u_new) {
                            kv[u] = make_float2(o[0], o[1]);
                            vv[u] = make_float2(o[2], o[3]);
                        }
                    }
                }
                // scores of the whole trip first (independent reductions), then one rescale of the running state
                float sc[kTrip];
                float m_trip = -INFINITY;
#pragma unroll
                for (int u = 0; u < kTrip; u++) {
                    const bool in = tt + u * kWarpsB1 < t1;
                    sc[u] = in ? warp_sum(qv.x * kv[u].x + qv.y * kv[u].y) * scale : -INFINITY;
                    m_trip = fmaxf(m_trip, sc[u]);
                }
                const float m_new = fmaxf(m_run, m_trip);
                const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
                l_run *= corr;
                o0 *= corr;
                o1 *= corr;
#pragma unroll
                for (int u = 0; u < kTrip; u++) {
                    if (tt + u * kWarpsB1 < t1) {
                        const float pr = expf(sc[u] - m_new);
                        l_run += pr;
                        o0 += pr * vv[u].x;
                        o1 += pr * vv[u].y;
                    }
                }
                m_run = m_new;
            }
            stamp();
            // combine the warps in order; red_s rows: [w][0..63] = o, then m and l
            red_s[w * 64 + 2 * lane] = o0;
            red_s[w * 64 + 2 * lane + 1] = o1;
            if (lane == 0) {
                out_s[w] = m_run;
                out2_s[w] = l_run;
            }
            bar_compute();
            if (w == 0) {
                float M = -INFINITY;
#pragma unroll
                for (int i = 0; i < kWarpsB1; i++) M = fmaxf(M, out_s[i]);
                float Lsum = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int i = 0; i < kWarpsB1; i++) {
                    const float f = out_s[i] == -INFINITY ? 0.f : expf(out_s[i] - M);
                    Lsum += out2_s[i] * f;
                    a0 += red_s[i * 64 + 2 * lane] * f;
                    a1 += red_s[i * 64 + 2 * lane + 1] * f;
                }
                unsigned long long* part = p.attn_ll + (size_t)g * (hs + 2);
                ll_store(part + 2 * lane, a0, ep_att);
                ll_store(part + 2 * lane + 1, a1, ep_att);
                if (lane == 0) {
                    ll_store(part + hs, M, ep_att);
                    ll_store(part + hs + 1, Lsum, ep_att);
                }
            }
        }
        if (cta_dead(&abort_flag)) break;  // also: red_s / out_s are free for the next stage
        stamp();

        // ---- C: output projection tile; its input rows are combined from the splits
        if (g < p.o.tiles) {
            const int ct = g % p.o.col_tiles, ks = g / p.o.col_tiles;
            const int k0 = ks * p.o.Kt, rows = min(p.o.Kt, d - k0);
            for (int k = t; k < rows; k += kCompute) {
                const int kk = k0 + k, head = kk / hs, dim = kk % hs;
                const unsigned long long* part = p.attn_ll + (size_t)head * S * (hs + 2);
                // splits four at a time: their (max, sum, value) words are requested together, then folded in order
                float M = -INFINITY, Lsum = 0.f, acc = 0.f;
                for (int s0 = 0; s0 < S; s0 += 4) {
                    const unsigned long long* ptr[12];
                    bool want[12];
                    float o[12];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const unsigned long long* ps = part + (size_t)min(s0 + u, S - 1) * (hs + 2);
                        ptr[3 * u] = ps + hs;
                        ptr[3 * u + 1] = ps + hs + 1;
                        ptr[3 * u + 2] = ps + dim;
                        want[3 * u] = want[3 * u + 1] = want[3 * u + 2] = s0 + u < S;
                    }
                    ll_wait<12>(ptr, want, ep_att, o, p.status, &abort_flag, 224);
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const float m = o[3 * u];
                        if (s0 + u < S && m != -INFINITY) {  // an empty split carries no weight
                            const float m_new = fmaxf(M, m);
                            const float c = M == -INFINITY ? 0.f : expf(M - m_new);
                            const float f = expf(m - m_new);
                            Lsum = Lsum * c + o[3 * u + 1] * f;
                            acc = acc * c + o[3 * u + 2] * f;
                            M = m_new;
                        }
                    }
                }
                in_s[k] = acc / Lsum;
            }
            bar_compute();
            stamp();
            tile_matvec<WT>(ring, in_s, rows, p.o.Kt, p.o.CW, red_s, out_s, tr);
            if (t < p.o.CW && ct * p.o.CW + t < d) ll_store(p.o_ll + (size_t)ks * d + ct * p.o.CW + t, out_s[t], ep_o);
        }
        stamp();

        // ---- D: x += attn @ Wo + bo; norm2; FFN up columns of this CTA, then their share of FFN down
        if (add_partials(x_s, ly->bo, p.o_ll, p.o.KS, ep_o, d, p.status, &abort_flag, 225)) break;
        if (l + 1 < p.L) nv1.fetch(layers_s[l + 1].n1g, layers_s[l + 1].n1b, d, p.modern);
        else nv1.fetch(p.fng, p.fnb, d, p.modern);
        if (g < p.up.tiles) {
            stamp();
            norm_vec(x_s, in_s, nv2, d, p.modern, sh);
            stamp();
            const int CW = p.up.CW;
            if (p.modern) {  // silu(gate) * up (inference.cpp:232-239)
                tile_matvec<WT>(ring, in_s, d, p.up.Kt, CW, red_s, out2_s, tr);
                stamp();
                tile_matvec<WT>(ring, in_s, d, p.up.Kt, CW, red_s, out_s, tr);
                stamp();
                if (t < CW) {
                    const float gt = out2_s[t];
                    hid_s[t] = g * CW + t < p.dff ? out_s[t] * (gt / (1.0f + expf(-gt))) : 0.f;
                }
            } else {  // gelu(h @ W1 + b1) (inference.cpp:69-80, 242-244)
                tile_matvec<WT>(ring, in_s, d, p.up.Kt, CW, red_s, out_s, tr);
                if (t < CW) {
                    float hv = 0.f;
                    if (g * CW + t < p.dff) {
                        const float v = out_s[t] + __ldg(ly->b1 + g * CW + t);
                        const float u = 0.79788456f * (v + 0.044715f * v * v * v);
                        hv = 0.5f * v * (1.0f + tanhf(u));
                    }
                    hid_s[t] = hv;
                }
            }
            bar_compute();
            // FFN down (inference.cpp:240-247), this CTA's share: its hidden units times their rows of the down
            // matrix, every thread a few output columns; the partial vector joins the accumulator by integer adds.
            {
                const int row0 = g * CW, nrows = min(CW, p.dff - row0);
                const int chunk_rows = kSlotBytes / (d * (int)sizeof(WT));
                constexpr int kColsPerThread = kHold;
                float y[kColsPerThread] = {};
                for (int r = 0; r < nrows; r += chunk_rows) {
                    const int n = min(chunk_rows, nrows - r);
                    const WT* rows = reinterpret_cast<const WT*>(ring_acquire(ring));
                    stamp();
                    {
                        // columns past d read column 0 and are dropped later, so the loop carries no branch
                        const WT* wp[kColsPerThread];
#pragma unroll
                        for (int c = 0; c < kColsPerThread; c++) wp[c] = rows + (t + c * kCompute < d ? t + c * kCompute : 0);
#pragma unroll 8
                        for (int i = 0; i < n; i++) {
                            const float hv = hid_s[r + i];
#pragma unroll
                            for (int c = 0; c < kColsPerThread; c++) y[c] += hv * ld_tile1(wp[c] + (size_t)i * d);
                        }
                    }
                    ring_release(ring);
                }
                stamp();
#pragma unroll
                for (int c = 0; c < kColsPerThread; c++) {
                    const int col = t + c * kCompute;
                    if (col < d) acc_add(acc_f + (size_t)col * kAccStride, y[c]);
                }
            }
        }
        stamp();
    }

    if (!cta_dead(&abort_flag)) {
        // ---- final norm + tied-embedding logits (inference.cpp:251-254)
        if (do_logits) {
            (void)add_accumulated(x_s, (layers_s + p.L - 1)->b2, acc_mine + (size_t)(p.L - 1) * d * kAccStride,
                                  (uint32_t)p.up.tiles, d, p.status, &abort_flag, 226);
            norm_vec(x_s, in_s, nv1, d, p.modern, sh);
            const int r0 = g * p.logit_rows_per_cta, r1 = min(p.V, r0 + p.logit_rows_per_cta);
            for (int r = r0; r < r1; r += p.logit_chunk_rows) {
                const int n = min(p.logit_chunk_rows, r1 - r);
                const WT* rows = reinterpret_cast<const WT*>(ring_acquire(ring));
                for (int i = w; i < n; i += kWarpsB1) {
                    const WT* er = rows + (size_t)i * d;
                    float acc = 0.f;
                    for (int k = lane * 4; k < d; k += 128) {
                        const float4 e = ld_tile4(er + k);
                        const float4 hv = *reinterpret_cast<const float4*>(&in_s[k]);
                        acc += hv.x * e.x + hv.y * e.y + hv.z * e.z + hv.w * e.w;
                    }
                    acc = warp_sum(acc);
                    if (lane == 0) p.logits[r + i] = acc;
                }
                ring_release(ring);
            }
        }
        stamp();
    }
    if (g == 0 && t == 0) {
        // The launch state moves on only when every CTA has read it (they all have, long ago: the wait is a formality
        // that keeps a late starter from seeing the next step's position).
        const unsigned want = (step + 1u) * (unsigned)p.G;
        bool seen = false;
        for (uint32_t it = 0; it < kSpinLimit && !seen; ++it) {
            unsigned cur;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(cur) : "l"(p.sync + 1) : "memory");
            seen = cur == want;
        }
        if (!seen) atomicExch(p.status, 227);
        if (seen && !abort_flag) {
            p.pos[0] = pos + 1;
            if (p.append_hist) {
                const int n = p.hist_len[0];
                if (n < p.hist_stride) p.hist[n] = token;
                p.hist_len[0] = n + 1;
            }
        }
        p.sync[0] = step + 1u;
    }
}

// dst[tile][kk][c] = W[(ks*Kt + kk)][ct*CW + c] (zero outside), tile = ks*col_tiles + ct.
// Up to three source matrices of n_single columns each are taken side by side (Q | K | V).
template <typename WT>
__global__ void pack_tiles_kernel(const float* s0, const float* s1, const float* s2, int n_single, B1Mat m, WT* dst) {
    const size_t total = (size_t)m.tiles * m.tile_elems;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int tile = (int)(i / m.tile_elems), rem = (int)(i % m.tile_elems);
        const int kk = rem / m.CW, c = rem % m.CW;
        const int ct = tile % m.col_tiles, ks = tile / m.col_tiles;
        const int k = ks * m.Kt + kk, n = ct * m.CW + c;
        float v = 0.f;
        if (k < m.K && n < m.N) {
            const int which = n / n_single, nn = n % n_single;
            const float* src = which == 0 ? s0 : (which == 1 ? s1 : s2);
            v = src[(size_t)k * n_single + nn];
        }
        if constexpr (sizeof(WT) == 4) dst[i] = v;
        else dst[i] = __float2bfloat16_rn(v);
    }
}

// Cheapest (smallest per-CTA tile) way to cut a K x N projection over at most G CTAs.
B1Mat plan_matrix(int K, int N, int G, int max_ks) {
    B1Mat best{};
    long best_cost = -1;
    for (int CW : {16, 32, 64}) {
        const int col_tiles = (N + CW - 1) / CW;
        for (int KS = 1; KS <= max_ks; KS++) {
            if (col_tiles * KS > G) break;
            const int Kt = (((K + KS - 1) / KS) + 3) / 4 * 4;
            if ((long)(KS - 1) * Kt >= K) continue;  // an empty slice
            if (KS > 16) continue;                   // consumers hold at most 16 partials
            const long cost = (long)Kt * CW;
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                best = B1Mat{K, N, CW, KS, Kt, col_tiles, col_tiles * KS, Kt * CW};
            }
        }
    }
    return best;
}

template <typename WT>
void* pack_matrix(const float* s0, const float* s1, const float* s2, int n_single, const B1Mat& m) {
    WT* dst = nullptr;
    const size_t total = (size_t)m.tiles * m.tile_elems;
    GRADB_CUDA(cudaMalloc(&dst, total * sizeof(WT)));
    pack_tiles_kernel<WT><<<512, 256>>>(s0, s1, s2, n_single, m, dst);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
    return dst;
}

size_t b1_smem_bytes(const DeviceModel* m, const B1Plan* plan) {
    const int in_len = std::max(m->desc.d_model, plan->o.Kt);
    return (size_t)kSlots * kSlotBytes + 128 + sizeof(float) * ((size_t)m->desc.d_model + in_len + 8);
}

}  // namespace

B1Plan* b1_make_plan(const DeviceModel* m) {
    auto* plan = new B1Plan();
    const gradb_model_desc& ds = m->desc;
    const int d = ds.d_model, f = ds.d_ff, hs = d / ds.num_heads;
    const bool modern = ds.arch == GRADB_ARCH_MODERN;
    plan->G = m->sm_count;
    plan->wbytes = m->precision == GRADB_BF16 ? 2 : 4;
    if (hs != 64 || d % 8 != 0 || d > kHold * kCompute || ds.num_heads > plan->G || ds.num_layers > kMaxLayersB1) return plan;  // not supported: the generic kernels run instead
    // Q/K/V and FFN-up have non-linear epilogues, so their tiles span the whole reduction.
    plan->qkv = plan_matrix(d, 3 * d, plan->G, 1);
    plan->o = plan_matrix(d, d, plan->G, 16);
    plan->up = plan_matrix(d, f, plan->G, 1);
    if (!plan->qkv.tiles || !plan->o.tiles || !plan->up.tiles) return plan;
    if (plan->up.CW > 64 || kSlotBytes / (d * plan->wbytes) < 1) return plan;
    if (plan->up.tiles >= (1 << kCountBits) || plan->o.KS >= (1 << kCountBits)) return plan;
    plan->logit_rows_per_cta = (ds.vocab_size + plan->G - 1) / plan->G;
    plan->logit_chunk_rows = kSlotBytes / (d * plan->wbytes);
    if (plan->logit_chunk_rows < 1) return plan;
    plan->attn_splits = std::max(1, std::min(16, plan->G / ds.num_heads));
    if (b1_smem_bytes(m, plan) > 227 * 1024) return plan;

    GRADB_CUDA(cudaSetDevice(m->device));
    std::vector<B1Layer> host(ds.num_layers);
    for (int l = 0; l < ds.num_layers; l++) {
        const LayerWeights& w = m->layers[l];
        B1Layer& b = host[l];
        auto pack = [&](const float* s0, const float* s1, const float* s2, int n_single, const B1Mat& mat) {
            void* ptr = plan->wbytes == 2 ? pack_matrix<__nv_bfloat16>(s0, s1, s2, n_single, mat)
                                          : pack_matrix<float>(s0, s1, s2, n_single, mat);
            plan->owned.push_back(ptr);
            return ptr;
        };
        b.qkv = pack(w.wq, w.wk, w.wv, d, plan->qkv);
        b.o = pack(w.wo, nullptr, nullptr, d, plan->o);
        b.gate = modern ? pack(w.gate, nullptr, nullptr, f, plan->up) : nullptr;
        b.up = pack(w.w1, nullptr, nullptr, f, plan->up);
        b.down = plan->wbytes == 2 ? (const void*)w.w216 : (const void*)w.w2;  // read by rows, no repacking
        b.bq = w.bq; b.bk = w.bk; b.bv = w.bv; b.bo = w.bo;
        b.b1 = w.b1; b.b2 = w.b2;
        b.n1g = w.n1g; b.n1b = w.n1b; b.n2g = w.n2g; b.n2b = w.n2b;
    }
    GRADB_CUDA(cudaMalloc(&plan->layers_dev, host.size() * sizeof(B1Layer)));
    GRADB_CUDA(cudaMemcpy(plan->layers_dev, host.data(), host.size() * sizeof(B1Layer), cudaMemcpyHostToDevice));
    GRADB_CUDA(cudaDeviceSynchronize());
    // The kernel needs every CTA resident at once: check that the device agrees.
    const size_t smem = b1_smem_bytes(m, plan);
    int per_sm = 0;
    if (plan->wbytes == 2) {
        GRADB_CUDA(cudaFuncSetAttribute(decode_b1_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
        GRADB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_b1_kernel<__nv_bfloat16>, kThreadsB1,
                                                                 smem));
    } else {
        GRADB_CUDA(cudaFuncSetAttribute(decode_b1_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        GRADB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_b1_kernel<float>, kThreadsB1, smem));
    }
    plan->ok = per_sm >= 1;
    return plan;
}

void b1_free_plan(B1Plan* p) {
    if (!p) return;
    for (void* q : p->owned) cudaFree(q);
    cudaFree(p->layers_dev);
    delete p;
}

namespace {
struct B1Workspace {
    size_t q, kv, attn, o, acc, sync, total;  // byte offsets
};
B1Workspace b1_layout(const DeviceModel* m, const B1Plan* plan) {
    const size_t d = (size_t)m->desc.d_model, hs = d / m->desc.num_heads;
    auto up = [](size_t v) { return (v + 127) & ~size_t(127); };
    B1Workspace w{};
    size_t at = 0;
    w.q = at; at = up(at + d * 8);
    w.kv = at; at = up(at + 2 * d * 8);
    w.attn = at; at = up(at + (size_t)m->desc.num_heads * plan->attn_splits * (hs + 2) * 8);
    w.o = at; at = up(at + (size_t)plan->o.KS * d * 8);
    w.acc = at; at = up(at + 2 * (size_t)m->desc.num_layers * d * kAccStride * 8);
    w.sync = at; at = up(at + 2 * sizeof(unsigned));
    w.total = at;
    return w;
}
}  // namespace

size_t b1_workspace_bytes(const DeviceModel* m, const B1Plan* plan) { return b1_layout(m, plan).total; }

void b1_bind_workspace(B1Params& p, void* workspace, const DeviceModel* m, const B1Plan* plan) {
    const B1Workspace w = b1_layout(m, plan);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    p.q_ll = reinterpret_cast<unsigned long long*>(base + w.q);
    p.kv_ll = reinterpret_cast<unsigned long long*>(base + w.kv);
    p.attn_ll = reinterpret_cast<unsigned long long*>(base + w.attn);
    p.o_ll = reinterpret_cast<unsigned long long*>(base + w.o);
    p.acc = reinterpret_cast<long long*>(base + w.acc);
    p.sync = reinterpret_cast<unsigned*>(base + w.sync);
}

void launch_decode_b1(const B1Params& p, cudaStream_t st) {
    const int in_len = std::max(p.d, p.o.Kt);
    const size_t smem = (size_t)kSlots * kSlotBytes + 128 + sizeof(float) * ((size_t)p.d + in_len + 8);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.G);
    cfg.blockDim = dim3(kThreadsB1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: the grid barrier relies on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (p.wbytes == 2) {
        GRADB_CUDA(cudaLaunchKernelEx(&cfg, decode_b1_kernel<__nv_bfloat16>, p));
    } else {
        GRADB_CUDA(cudaLaunchKernelEx(&cfg, decode_b1_kernel<float>, p));
    }
    count_launch();
}

}  // namespace gradb
