// One decode step of a single sequence (InferenceSession::step, inference.cpp:150-258)
// as ONE persistent cooperative kernel.
//
// At batch 1 every projection is a matrix-vector product that streams its weights
// once; the step is bound by HBM bandwidth and, before that, by latency: some forty
// dependent stages of a few microseconds each. This kernel removes the per-stage
// launch and the cold start of every stage's weight stream:
//
//  * one CTA per SM stays resident for the whole step; stages are separated by a
//    grid-wide barrier (bounded spin on a global counter) instead of kernel launches;
//  * the weights are re-tiled when the model is loaded so that everything one CTA
//    needs for one stage is a single contiguous block; a producer warp walks the
//    step's fixed list of blocks and keeps a four-slot shared-memory ring full with
//    bulk asynchronous copies (TMA, mbarrier completion). The HBM stream therefore
//    runs ahead of the arithmetic, through barriers and reductions;
//  * vectors exchanged between CTAs (q, attention partials, projection partials, the
//    FFN activation) live in a small global workspace that stays in L2 and is read
//    with cache-global loads; split-K partial sums are added by their consumers in a
//    fixed order, so results do not depend on scheduling;
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

constexpr int kCompute = 512;  // compute threads (16 warps)
constexpr int kThreadsB1 = kCompute + 32;  // + producer warp
constexpr int kWarpsB1 = kCompute / 32;
constexpr int kSlots = 4;
constexpr int kSlotBytes = 48 * 1024;
constexpr uint32_t kPollLimit = 1u << 22;
constexpr int kMaxLayersB1 = 32;  // layer tables are staged in shared memory
// Elements of the fixed-point FFN accumulator sit one per 128-byte line: every CTA adds to every element at
// about the same time, and same-line atomics queue up in one L2 slice.
constexpr int kAccStride = 16;  // in 64-bit words

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, %0;" ::"n"(kCompute) : "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct Ring {
    uint64_t* full;
    uint64_t* empty;
    uint8_t* slots;
    int* status;
    volatile int* abort_flag;
    uint32_t n;  // chunks consumed / produced so far
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
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(r.slots + (size_t)s * kSlotBytes)),
                 "l"(src), "r"(bytes), "r"(bar)
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

// Grid-wide barrier over the compute threads of all CTAs. Bounded: on expiry the
// status word is set and the kernel unwinds.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* status, volatile int* abort_flag) {
    bar_compute();
    if (threadIdx.x == 0) {
        // release: everything this CTA wrote (ordered before by the CTA barrier) is visible to
        // whoever later observes the count with an acquire load
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        uint32_t it = 0;
        for (;;) {
            unsigned cur;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(cur) : "l"(counter) : "memory");
            if ((int)(cur - target) >= 0) break;
            if (++it > kPollLimit || *abort_flag) {
                atomicExch(status, 201);
                *abort_flag = 1;
                break;
            }
        }
    }
    bar_compute();
    return *abort_flag == 0;
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
// `rows` of the tile's Kt (zero padded) rows carry data.
template <typename WT>
__device__ void tile_matvec(Ring& ring, const float* in_s, int rows, int Kt, int CW, float* red_s, float* out_s) {
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    const int cg = CW / 4, R = kCompute / cg;
    const int c4 = t % cg, r0 = t / cg;
    const int chunk_rows = kSlotBytes / (CW * (int)sizeof(WT));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < Kt; base += chunk_rows) {  // same chunking as the producer's
        const int n = min(chunk_rows, rows - base);
        const WT* tile = reinterpret_cast<const WT*>(ring_acquire(ring));
#pragma unroll 4
        for (int k = r0; k < n; k += R) {
            const float4 wv = ld_tile4(tile + (size_t)k * CW + c4 * 4);
            const float xv = in_s[base + k];
            acc.x += xv * wv.x;
            acc.y += xv * wv.y;
            acc.z += xv * wv.z;
            acc.w += xv * wv.w;
        }
        ring_release(ring);
    }
    for (int o = cg; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (lane < cg) *reinterpret_cast<float4*>(&red_s[w * 64 + lane * 4]) = acc;
    bar_compute();
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

// in_s = norm(x_s) (inference.cpp:30-58). gamma/beta are fetched before the reductions so their
// latency overlaps them.
__device__ void norm_vec(const float* x_s, float* in_s, const float* gamma, const float* beta, int d, int rms,
                         float* sh) {
    constexpr int kHold = 4;  // elements per thread kept in registers (d <= 2048); beyond that, loaded late
    float gv[kHold], bv[kHold];
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        gv[i] = k < d ? __ldg(gamma + k) : 0.f;
        bv[i] = (k < d && !rms) ? __ldg(beta + k) : 0.f;
    }
    float s = 0.f;
    for (int k = threadIdx.x; k < d; k += kCompute) s += rms ? x_s[k] * x_s[k] : x_s[k];
    s = block_total(s, sh);
    float mean = 0.f, r;
    if (rms) {
        r = 1.0f / sqrtf(s / (float)d + 1e-5f);
    } else {
        mean = s / (float)d;
        float v = 0.f;
        for (int k = threadIdx.x; k < d; k += kCompute) {
            const float dl = x_s[k] - mean;
            v += dl * dl;
        }
        v = block_total(v, sh);
        r = 1.0f / sqrtf(v / (float)d + 1e-5f);
    }
#pragma unroll
    for (int i = 0; i < kHold; i++) {
        const int k = threadIdx.x + i * kCompute;
        if (k < d) in_s[k] = rms ? gv[i] * x_s[k] * r : gv[i] * (x_s[k] - mean) * r + bv[i];
    }
    for (int k = threadIdx.x + kHold * kCompute; k < d; k += kCompute) {
        in_s[k] = rms ? __ldg(gamma + k) * x_s[k] * r : __ldg(gamma + k) * (x_s[k] - mean) * r + __ldg(beta + k);
    }
    bar_compute();
}

// x_s += bias + sum of KS partial vectors (fixed order)
__device__ void add_partials(float* x_s, const float* bias, const float* part, int KS, int d) {
    // All loads of an element are issued before the first add, so they share one trip to L2;
    // the adds keep the slice order.
    constexpr int kMaxKS = 16;
    for (int k = threadIdx.x; k < d; k += kCompute) {
        float pv[kMaxKS];
        const float bv = bias ? __ldg(bias + k) : 0.f;
#pragma unroll
        for (int s = 0; s < kMaxKS; s++) pv[s] = s < KS ? __ldcg(part + (size_t)s * d + k) : 0.f;
        float v = x_s[k] + bv;
#pragma unroll
        for (int s = 0; s < kMaxKS; s++) {
            if (s < KS) v += pv[s];
        }
        x_s[k] = v;
    }
    bar_compute();
}

// x_s += bias + the fixed-point accumulator (units of 2^-32), read past L1: other CTAs' adds land in L2
__device__ void add_fixed(float* x_s, const float* bias, const long long* acc, int d) {
    for (int k = threadIdx.x; k < d; k += kCompute) {
        const float bv = bias ? __ldg(bias + k) : 0.f;
        const long long q = __ldcg(acc + (size_t)k * kAccStride);
        float v = x_s[k] + bv;
        v += (float)((double)q * 2.3283064365386963e-10);
        x_s[k] = v;
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
    const bool do_logits = p.logit_tok[0] >= 0;
    const unsigned base = *p.bar_base;
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
    }
    __syncthreads();
    Ring ring{full_bar, empty_bar, slots, p.status, &abort_flag, 0};

    if (t >= kCompute) {
        // ---------------------------------------------------------------- producer warp
        if (t == kCompute) {
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
    unsigned bar_i = 0;
    int trace_i = 0;
    auto stamp = [&]() {
        if (p.trace && g == 0 && t == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            p.trace[trace_i++] = now;
        }
    };
    auto barrier = [&]() {
        bar_i++;
        stamp();  // stage work done
        const bool okb = grid_barrier(p.bar_counter, base + bar_i * (unsigned)p.G, p.status, &abort_flag);
        stamp();  // barrier passed
        return okb;
    };
    stamp();

    // x = E[token] (+ P[pos])  (inference.cpp:159-182)
    for (int k = t; k < d; k += kCompute) {
        float v = __ldg(p.emb32 + (size_t)token * d + k);
        if (p.pos_emb) v += __ldg(p.pos_emb + (size_t)pos * d + k);
        x_s[k] = v;
    }
    bar_compute();

    const int S = p.attn_splits;
    const float scale = 1.0f / sqrtf((float)hs);
    bool alive = true;

    for (int l = 0; l < p.L && alive; l++) {
        const B1Layer* ly = layers_s + l;
        float* kc = p.kcache + (size_t)l * p.layer_cache_stride;
        float* vc = p.vcache + (size_t)l * p.layer_cache_stride;

        // ---- A: (previous FFN output joins the residual) norm1, Q/K/V columns of this CTA
        if (l > 0) add_fixed(x_s, (layers_s + l - 1)->b2, p.ffn_acc + (size_t)((l - 1) & 1) * d * kAccStride, d);
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
            norm_vec(x_s, in_s, ly->n1g, ly->n1b, d, p.modern, sh);
            tile_matvec<WT>(ring, in_s, d, p.qkv.Kt, p.qkv.CW, red_s, out_s);
            if (mine) {
                {
                    float a0 = out_s[2 * t] + b0, a1 = out_s[2 * t + 1] + b1;
                    if (p.rope_cos && which < 2) {  // inference.cpp:101-115
                        const float r0 = a0 * cs - a1 * sn, r1 = a0 * sn + a1 * cs;
                        a0 = r0;
                        a1 = r1;
                    }
                    if (which == 0) {
                        *reinterpret_cast<float2*>(p.q + n_in) = make_float2(a0, a1);
                    } else {
                        float* cache = which == 1 ? kc : vc;
                        *reinterpret_cast<float2*>(cache + ((size_t)h * p.T + pos) * hs + c_in) = make_float2(a0, a1);
                    }
                }
            }
        }
        if (!(alive = barrier())) break;

        // ---- B: attention of (head, context split) g over the cached positions (inference.cpp:208-225)
        // This layer's FFN accumulator is cleared here: its previous contents (layer l-2) were consumed
        // before the barrier just passed, and the first add comes two barriers from now.
        for (int k = g * kCompute + t; k < d; k += p.G * kCompute) {
            p.ffn_acc[((size_t)(l & 1) * d + k) * kAccStride] = 0;
        }
        if (g < p.H * S) {
            const int head = g / S, split = g % S;
            const int ctx = pos + 1;
            const int cps = (ctx + S - 1) / S;
            const int t0 = split * cps, t1 = min(ctx, t0 + cps);
            const float* K = kc + (size_t)head * p.T * hs;
            const float* V = vc + (size_t)head * p.T * hs;
            const float2 qv = __ldcg(reinterpret_cast<const float2*>(p.q + head * hs) + lane);
            float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;
            // four positions per trip: their K and V rows are requested together
            for (int tt = t0 + w; tt < t1; tt += 4 * kWarpsB1) {
                float2 kv[4], vv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int tu = tt + u * kWarpsB1;
                    if (tu < t1) {
                        kv[u] = __ldcg(reinterpret_cast<const float2*>(K + (size_t)tu * hs) + lane);
                        vv[u] = __ldcg(reinterpret_cast<const float2*>(V + (size_t)tu * hs) + lane);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (tt + u * kWarpsB1 < t1) {
                        const float sc = warp_sum(qv.x * kv[u].x + qv.y * kv[u].y) * scale;
                        const float m_new = fmaxf(m_run, sc);
                        const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
                        const float pr = expf(sc - m_new);
                        l_run = l_run * corr + pr;
                        o0 = o0 * corr + pr * vv[u].x;
                        o1 = o1 * corr + pr * vv[u].y;
                        m_run = m_new;
                    }
                }
            }
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
                float* part = p.attn_part + (size_t)g * (hs + 2);
                *reinterpret_cast<float2*>(part + 2 * lane) = make_float2(a0, a1);
                if (lane == 0) {
                    part[hs] = M;
                    part[hs + 1] = Lsum;
                }
            }
        }
        if (!(alive = barrier())) break;

        // ---- C: output projection tile; its input rows are combined from the splits
        if (g < p.o.tiles) {
            const int ct = g % p.o.col_tiles, ks = g / p.o.col_tiles;
            const int k0 = ks * p.o.Kt, rows = min(p.o.Kt, d - k0);
            for (int k = t; k < rows; k += kCompute) {
                const int kk = k0 + k, head = kk / hs, dim = kk % hs;
                const float* part = p.attn_part + (size_t)head * S * (hs + 2);
                constexpr int kMaxS = 16;  // all loads first: one trip to L2 instead of three
                float ms[kMaxS], ls[kMaxS], os[kMaxS];
#pragma unroll
                for (int s = 0; s < kMaxS; s++) {
                    const bool in = s < S;
                    ms[s] = in ? __ldcg(part + s * (hs + 2) + hs) : -INFINITY;
                    ls[s] = in ? __ldcg(part + s * (hs + 2) + hs + 1) : 0.f;
                    os[s] = in ? __ldcg(part + s * (hs + 2) + dim) : 0.f;
                }
                float M = -INFINITY;
#pragma unroll
                for (int s = 0; s < kMaxS; s++) M = fmaxf(M, ms[s]);
                float Lsum = 0.f, acc = 0.f;
#pragma unroll
                for (int s = 0; s < kMaxS; s++) {
                    const float f = ms[s] == -INFINITY ? 0.f : expf(ms[s] - M);
                    Lsum += ls[s] * f;
                    acc += os[s] * f;
                }
                in_s[k] = acc / Lsum;
            }
            bar_compute();
            tile_matvec<WT>(ring, in_s, rows, p.o.Kt, p.o.CW, red_s, out_s);
            if (t < p.o.CW && ct * p.o.CW + t < d) p.opart[(size_t)ks * d + ct * p.o.CW + t] = out_s[t];
        }
        if (!(alive = barrier())) break;

        // ---- D: x += attn @ Wo + bo; norm2; FFN up columns of this CTA
        add_partials(x_s, ly->bo, p.opart, p.o.KS, d);
        if (g < p.up.tiles) {
            norm_vec(x_s, in_s, ly->n2g, ly->n2b, d, p.modern, sh);
            const int CW = p.up.CW;
            if (p.modern) {  // silu(gate) * up (inference.cpp:232-239)
                tile_matvec<WT>(ring, in_s, d, p.up.Kt, CW, red_s, out2_s);
                tile_matvec<WT>(ring, in_s, d, p.up.Kt, CW, red_s, out_s);
                if (t < CW) {
                    const float gt = out2_s[t];
                    hid_s[t] = g * CW + t < p.dff ? out_s[t] * (gt / (1.0f + expf(-gt))) : 0.f;
                }
            } else {  // gelu(h @ W1 + b1) (inference.cpp:69-80, 242-244)
                tile_matvec<WT>(ring, in_s, d, p.up.Kt, CW, red_s, out_s);
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
                constexpr int kColsPerThread = 4;  // d <= 4 * kCompute
                float y[kColsPerThread] = {0.f, 0.f, 0.f, 0.f};
                for (int r = 0; r < nrows; r += chunk_rows) {
                    const int n = min(chunk_rows, nrows - r);
                    const WT* rows = reinterpret_cast<const WT*>(ring_acquire(ring));
#pragma unroll
                    for (int c = 0; c < kColsPerThread; c++) {
                        const int col = t + c * kCompute;
                        if (col < d) {
                            float a = y[c];
                            for (int i = 0; i < n; i++) a += hid_s[r + i] * ld_tile1(rows + (size_t)i * d + col);
                            y[c] = a;
                        }
                    }
                    ring_release(ring);
                }
                long long* acc = p.ffn_acc + (size_t)(l & 1) * d * kAccStride;
#pragma unroll
                for (int c = 0; c < kColsPerThread; c++) {
                    const int col = t + c * kCompute;
                    if (col < d) {
                        const long long q = __double2ll_rn((double)y[c] * 4294967296.0);
                        asm volatile("red.global.add.u64 [%0], %1;" ::"l"(acc + (size_t)col * kAccStride), "l"(q) : "memory");
                    }
                }
            }
        }
        if (!(alive = barrier())) break;
    }

    if (alive) {
        // ---- final norm + tied-embedding logits (inference.cpp:251-254)
        if (do_logits) {
            add_fixed(x_s, (layers_s + p.L - 1)->b2, p.ffn_acc + (size_t)((p.L - 1) & 1) * d * kAccStride, d);
            norm_vec(x_s, in_s, p.fng, p.fnb, d, p.modern, sh);
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
        if (g == 0 && t == 0) {
            p.pos[0] = pos + 1;
            if (p.append_hist) {
                const int n = p.hist_len[0];
                if (n < p.hist_stride) p.hist[n] = token;
                p.hist_len[0] = n + 1;
            }
            *p.bar_base = base + bar_i * (unsigned)p.G;
        }
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
    if (hs != 64 || d % 8 != 0 || d > 4 * kCompute || ds.num_heads > plan->G || ds.num_layers > kMaxLayersB1) return plan;  // not supported: the generic kernels run instead
    // Q/K/V and FFN-up have non-linear epilogues, so their tiles span the whole reduction.
    plan->qkv = plan_matrix(d, 3 * d, plan->G, 1);
    plan->o = plan_matrix(d, d, plan->G, 16);
    plan->up = plan_matrix(d, f, plan->G, 1);
    if (!plan->qkv.tiles || !plan->o.tiles || !plan->up.tiles) return plan;
    if (plan->up.CW > 64 || kSlotBytes / (d * plan->wbytes) < 1) return plan;
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

size_t b1_workspace_floats(const DeviceModel* m, const B1Plan* plan) {
    const int d = m->desc.d_model, hs = d / m->desc.num_heads;
    return (size_t)d                                                      // q
           + (size_t)m->desc.num_heads * plan->attn_splits * (hs + 2)     // attention partials
           + (size_t)plan->o.KS * d + 4 * (size_t)d * kAccStride + 64;  // + two fixed-point accumulators, one line per element
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
