// Causal prompt attention on the 5th-generation tensor cores (head size 64), for the batched prompt feed and
// scoring of bf16 sessions: the same work as attn_prefill.cu (rows that are consecutive positions of their
// sequences attend to the cache rows at or before them, inference.cpp:208-225), with the two products of every
// (128 queries x 128 keys) tile issued as tcgen05.mma into TMEM instead of warp-level mma.sync.
//
// A work item = one tile of up to 128 consecutive query positions of one (sequence, head). The kernel is
// persistent: one CTA per SM takes items round-robin (head fastest; the host sorts the tiles longest first) and
// treats its (item, key tile) pairs as ONE stream of elements, so that the copies of an item's first tiles, which
// come from HBM, are in flight while the item before it is still being computed; with one CTA per SM and prompts of a
// few hundred positions that latency was otherwise most of a CTA's life. Eight softmax warps, two threads per query
// row (= TMEM lane: a warp reaches the lane quarter given by its index modulo 4), each thread owning half of the row's
// score columns and half of its output dims; the first lanes of two more warps issue everything asynchronous: one the
// Q and K copies and the score MMAs, the other the V copies and the second product's MMAs. Issuing costs its thread
// some tens of cycles per instruction (the instruction queue fills at the rate the tensor core drains it), so it is
// kept off the softmax warps' path; mbarriers tell the issuers when the scores have been read and when P is written.
// The cache stays fp32 and is fed to kind::tf32 MMAs as it lies (TF32 reads fp32 bit patterns):
//
//   S[q, key] (TMEM, 128 cols) = Q[q, :] . K[key, :]      A = Q tile, B = K tile, both dim-contiguous (K-major),
//                                                        brought by TMA tensor copies with the 128-byte swizzle
//   softmax by the row's two threads: causal mask, running max / sum, P = exp(scale (S - max)) -> TMEM (128 cols):
//                                                        the A operand of the second product is read from there,
//                                                        so P never crosses shared memory
//   O_tile[q, dim] (TMEM, 64 cols) = P[q, :] . V[:, dim]   B = V tile as it lies in the cache (keys x dims, brought by
//                                                        the same tensor copies as K): the operand is declared
//                                                        MN-major (dims contiguous, keys the K index), so no
//                                                        transposed copy is made
//   o = o * exp(old max - new max) + O_tile              in registers (32 per thread)
//
// Q has two buffers (the item after next is fetched when an item's last scores are done), K and V two stages each,
// P and O_tile two buffers each in TMEM: the scores of element e+1 are issued as soon as every thread holds element
// e's scores in registers and run under its exponentials; O_tile of element e is collected in element e+1's pass after that element's
// exponentials (so the second product has a whole softmax to finish in), and when that element opens a new item the
// finished item's rows are normalised and written there. A CTA's tiles are copied to shared memory first, so the
// issuing threads never wait for a global load. Tiles further ahead are prefetched towards L2. Cache rows past a
// sequence's context are multiplied by exact zeros of P, so they must be finite: the caches are zeroed when a session
// is created and only ever receive finite rows. All waits are bounded; on expiry the status word is set and the CTA
// falls through to the common exit, which frees TMEM.
#include <cuda.h>

#include <algorithm>

#include "attn_prefill.cuh"

namespace gradb {

namespace {

constexpr int kQT = 128;   // queries per CTA = TMEM lanes
constexpr int kSoftmaxThreads = 256;        // two per query row
constexpr int kThreads = kSoftmaxThreads + 64;  // + two warps whose first lanes issue the copies and the MMAs
constexpr int kKT = 128;   // keys per tile
constexpr int kHS = 64;
constexpr uint32_t kSpin = 1u << 20;
constexpr int kAtomQ = kQT * 128;  // bytes of one swizzle atom of a 128-row operand: 32 floats per row
// shared-memory map (bytes from a 1024-aligned base)
constexpr int kOffQ = 0;                       // 2 buffers of 2 atoms
constexpr int kOffK = kOffQ + 4 * kAtomQ;      // 2 stages of 2 atoms
constexpr int kOffV = kOffK + 4 * kAtomQ;      // 2 stages of 2 atoms: [128 keys][32 dims] each, as stored
constexpr int kSmemBytes = kOffV + 4 * kAtomQ + 1024;
// tensor-memory map (columns): S, P and O_tile (element e uses their buffers e & 1)
constexpr uint32_t kColS = 0, kColP = 128, kColO = 384, kTmemCols = 512;  // P: 2 x 128 columns, O_tile: 2 x 64
#if GRADB_DIAG
constexpr int kMaxListed = 4;    // diagnostics build: small, so that its tests also take the global-memory lookups
#else
constexpr int kMaxListed = 192;  // items of a CTA whose tiles are kept in shared memory
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; also ends (false) when another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* fail) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < kSpin; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*fail) return false;
    }
    if (status) atomicExch(status, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_tile) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major 32-bit operand. The only layout the tensor core takes for it is the 128-byte swizzle in 32-byte units:
// rows are K indices (here keys), 128 bytes = 32 consecutive MN elements (here dims) each, the four 32-byte chunks of
// a row exchanged by (row mod 4) -- what a tensor copy with the "128B, 32B atom" swizzle writes. 4-row groups are
// 512 bytes apart (stride byte offset); the next 32 MN elements start `mn_atom_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_sw128_mn32(const void* smem_tile, uint32_t mn_atom_bytes) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(mn_atom_bytes >> 4) << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
constexpr uint32_t kIdescBMnMajor = 1u << 16;  // B read MN-major (N contiguous) instead of K-major
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// A operand (128 rows x 8 fp32) read from tensor memory: lane = row, one column per element.
__device__ __forceinline__ void umma_tf32_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// 32 consecutive columns of this thread's lane; the caller issues tcgen05.wait::st before handing them on.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    uint32_t r[32];
#pragma unroll
    for (int i = 0; i < 32; i++) r[i] = __float_as_uint(v[i]);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Barrier of the softmax warps that also makes the give-up decision common: every thread contributes what it
// read of the flag before arriving and all of them get the same answer, so none is left alone at a later barrier.
__device__ __forceinline__ bool softmax_barrier_dead(volatile int* fail) {
    const uint32_t mine = (uint32_t)*fail;
    uint32_t any;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 p, %1, 0;\n"
        "bar.red.or.pred q, 1, %2, p;\n"
        "selp.u32 %0, 1, 0, q;\n"
        "}\n"
        : "=r"(any)
        : "r"(mine), "n"(kSoftmaxThreads)
        : "memory");
    return any != 0;
}

// Diagnostics build: CTA 0 adds up the clock cycles one of its warps spends in each part of an element
// (read through gradb_diag_attn_clocks).
#if GRADB_DIAG
__device__ unsigned long long g_attn_clock[16];
#define ATT_CLK(x) const long long x = clock64()
#define ATT_ADD(i, v) do { if (blockIdx.x == 0 && t == 160) atomicAdd(&g_attn_clock[i], (unsigned long long)(v)); } while (0)
#else
#define ATT_CLK(x)
#define ATT_ADD(i, v)
#endif

// One (query tile, head) of the launch: what a CTA works on between two output writes.
struct Item {
    int row0, pos0, nq, h, kv_len, n_kv;
    long long head_row0;  // first cache row of this (sequence, head)
};

__global__ void __launch_bounds__(kThreads, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                      const __grid_constant__ CUtensorMap map_k,
                                                                      const __grid_constant__ CUtensorMap map_v,
                                                                      const PrefillAttnParams p, long long k_row0) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // (two O barriers, by element parity: a thread tells the issuer that P is written before it collects the previous
    // O_tile, so a single barrier could complete two phases while that thread still waits for the first)
    __shared__ __align__(8) uint64_t bar_q[2], bar_k[2], bar_v[2], bar_s, bar_o[2];
    // softmax warps -> issuers: scores read; P written (by element parity, for the same reason as the O barriers:
    // nothing stops the softmax warps from announcing the next P before the issuer has looked at this one)
    __shared__ __align__(8) uint64_t bar_sfree, bar_pready[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int s_fail;
    __shared__ float s_x[2][2][kQT];  // [element parity][half][row]: the two column halves of a row exchange their maxima
    __shared__ float s_l[2][2][kQT];  // [item parity][half][row]: ... and, when an item ends, their sums
    __shared__ int4 s_tiles[kMaxListed];  // this CTA's first items: tile lookups stay off the issuing threads' path
    __shared__ int s_head[kMaxListed];    // ... and their heads (no division there either)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int row = (warp & 3) * 32 + lane;  // query row = TMEM lane
    const int hc = warp >> 2;                // which half of the score columns / output dims this thread owns
    const int n_items = p.n_tiles * p.H;
    const int my_count = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;  // >= 1: grid <= items

    // k-th item of this CTA: items are dealt round-robin, head fastest, so that CTAs working at the same time
    // hold tiles of the same length (the host sorts the tiles longest first)
    auto get_item = [&](int k) {
        int4 tile;
        Item it;
        if (k < kMaxListed) {
            tile = s_tiles[k];
            it.h = s_head[k];
        } else {
            const int idx = (int)blockIdx.x + k * (int)gridDim.x;
            tile = p.tiles[idx / p.H];
            it.h = idx % p.H;
        }
        it.row0 = tile.y;
        it.pos0 = tile.z;
        it.nq = tile.w;
        it.kv_len = tile.z + tile.w;
        it.n_kv = (it.kv_len + kKT - 1) / kKT;
        it.head_row0 = ((long long)tile.x * p.H + it.h) * p.T;
        return it;
    };

    for (int k = t; k < min(my_count, kMaxListed); k += kThreads) {
        const int idx = (int)blockIdx.x + k * (int)gridDim.x;
        s_tiles[k] = p.tiles[idx / p.H];
        s_head[k] = idx % p.H;
    }
    if (t == 0) {
        s_fail = 0;
        mbar_init(&bar_q[0], 1);
        mbar_init(&bar_q[1], 1);
        mbar_init(&bar_k[0], 1);
        mbar_init(&bar_k[1], 1);
        mbar_init(&bar_v[0], 1);
        mbar_init(&bar_v[1], 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o[0], 1);
        mbar_init(&bar_o[1], 1);
        mbar_init(&bar_sfree, kSoftmaxThreads / 32);  // one arrival per softmax warp
        mbar_init(&bar_pready[0], kSoftmaxThreads / 32);
        mbar_init(&bar_pready[1], kSoftmaxThreads / 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_slot + kColS, tmem_p = tmem_slot + kColP, tmem_o = tmem_slot + kColO;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;

    // ---- issuing threads only (first lanes of the two issuer warps). The CTA's work is one stream of (item, key tile) elements; element e uses K stage e & 1 and
    // phase e of the V, S and O barriers; item k uses Q buffer k & 1.
    auto load_q = [&](int k) {
        const Item it = get_item(k);
        uint64_t* bar = &bar_q[k & 1];
        uint8_t* dst = smem + kOffQ + (k & 1) * 2 * kAtomQ;
        mbar_expect_tx(bar, 2 * kAtomQ);
        tma_load_2d(dst, &map_q, it.h * kHS, it.row0, bar);
        tma_load_2d(dst + kAtomQ, &map_q, it.h * kHS + 32, it.row0, bar);
    };
    auto prefetch_q = [&](int k) {  // towards L2
        const Item it = get_item(k);
        asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(&map_q), "r"(it.h * kHS),
                     "r"(it.row0)
                     : "memory");
        asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(&map_q),
                     "r"(it.h * kHS + 32), "r"(it.row0)
                     : "memory");
    };
    auto load_k = [&](const Item& it, int j, int e) {  // keys [j*128, j*128+128) of the item's head, two 32-float halves
        uint64_t* bar = &bar_k[e & 1];
        uint8_t* dst = smem + kOffK + (e & 1) * 2 * kAtomQ;
        mbar_expect_tx(bar, 2 * kAtomQ);
        const int y = (int)(k_row0 + it.head_row0 + (long long)j * kKT);
        tma_load_2d(dst, &map_k, 0, y, bar);
        tma_load_2d(dst + kAtomQ, &map_k, 32, y, bar);
    };
    auto load_v = [&](const Item& it, int j, int e) {  // the same rows of V, as they lie (keys x dims), stage e & 1
        uint64_t* bar = &bar_v[e & 1];
        uint8_t* dst = smem + kOffV + (e & 1) * 2 * kAtomQ;
        mbar_expect_tx(bar, 2 * kAtomQ);
        const int y = (int)(k_row0 + it.head_row0 + (long long)j * kKT);
        tma_load_2d(dst, &map_v, 0, y, bar);
        tma_load_2d(dst + kAtomQ, &map_v, 32, y, bar);
    };
    auto prefetch_kv = [&](const Item& it, int j) {  // towards L2, for the element two ahead of the copies above
        const int rows = min(kKT, it.kv_len - j * kKT);
        const uint32_t bytes = (uint32_t)rows * kHS * 4;
        const size_t at = (size_t)(it.head_row0 + (long long)j * kKT) * kHS;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.vcache + at), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.kcache + at), "r"(bytes) : "memory");
    };
    // S = Q_k K^T for element e (first of its item when j == 0); its operands were requested at least an element ago
    auto issue_scores = [&](int k, int j, int e) {
        if (j == 0 && !mbar_wait(&bar_q[k & 1], (uint32_t)((k >> 1) & 1), p.status, 401, &s_fail)) {
            s_fail = 1;
            return;
        }
        if (!mbar_wait(&bar_k[e & 1], (uint32_t)((e >> 1) & 1), p.status, 402, &s_fail)) {
            s_fail = 1;
            return;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        constexpr uint32_t idesc = umma_idesc_tf32(kQT, kKT);
#pragma unroll
        for (int a = 0; a < 2; a++) {  // 32 dims per atom, 8 per instruction
            const uint64_t qd = umma_desc_sw128(smem + kOffQ + ((k & 1) * 2 + a) * kAtomQ);
            const uint64_t kd = umma_desc_sw128(smem + kOffK + ((e & 1) * 2 + a) * kAtomQ);
#pragma unroll
            for (int kk = 0; kk < 4; kk++) umma_tf32(tmem_s, qd + 2 * kk, kd + 2 * kk, idesc, (a | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&bar_s);
    };
    // the element after (k, j); false past the CTA's last one
    auto step = [&](int& k, int& j, int n_kv) {
        if (++j >= n_kv) {
            j = 0;
            ++k;
        }
        return k < my_count;
    };

    Item it = get_item(0);
    int k = 0, j = 0;
    if (warp == kSoftmaxThreads / 32) {
        // ================= issuer warp A (one lane): copies of Q and K, and the score MMAs =================
        if (lane == 0) {
            load_q(0);
            if (my_count > 1) load_q(1);
            load_k(it, 0, 0);
            {
                int k1 = 0, j1 = 0;
                if (step(k1, j1, it.n_kv)) {
                    const Item it1 = k1 == 0 ? it : get_item(k1);
                    load_k(it1, j1, 1);
                    int k2 = k1, j2 = j1;
                    if (step(k2, j2, it1.n_kv)) prefetch_kv(k2 == k1 ? it1 : get_item(k2), j2);
                }
            }
            issue_scores(0, 0, 0);
            for (int e = 0;; e++) {
                // every softmax thread holds element e's scores: the accumulator and this element's K stage are free
                if (!mbar_wait(&bar_sfree, (uint32_t)(e & 1), p.status, 406, &s_fail)) {
                    s_fail = 1;
                    break;
                }
                int k1 = k, j1 = j;
                const bool more = step(k1, j1, it.n_kv);
                Item it1 = it;
                if (more) {
                    if (k1 != k) it1 = get_item(k1);
                    issue_scores(k1, j1, e + 1);  // runs under element e's exponentials
                    int k2 = k1, j2 = j1;
                    if (step(k2, j2, it1.n_kv)) {
                        const Item it2 = k2 == k1 ? it1 : get_item(k2);
                        load_k(it2, j2, e + 2);
                    }
                }
                // this item's last scores are done, so its Q buffer is free: fetch the item after next into it
                if (j == it.n_kv - 1 && k + 2 < my_count) load_q(k + 2);
                if (!more || s_fail) break;
                it = it1;
                k = k1;
                j = j1;
            }
        }
        __syncwarp();
    } else if (warp == kSoftmaxThreads / 32 + 1) {
        // ================= issuer warp B (one lane): copies of V, prefetches, and the second product's MMAs ==========
        if (lane == 0) {
            load_v(it, 0, 0);
            for (int e = 0;; e++) {
                int k1 = k, j1 = j;
                const bool more = step(k1, j1, it.n_kv);
                const Item it1 = (more && k1 != k) ? get_item(k1) : it;
                // the other V stage was last read by element e-1's product
                if (e > 0 && !mbar_wait(&bar_o[(e - 1) & 1], (uint32_t)(((e - 1) >> 1) & 1), p.status, 408, &s_fail)) {
                    s_fail = 1;
                    break;
                }
                if (more) load_v(it1, j1, e + 1);
                // P of element e is complete in tensor memory
                if (!mbar_wait(&bar_pready[e & 1], (uint32_t)((e >> 1) & 1), p.status, 407, &s_fail) ||
                    !mbar_wait(&bar_v[e & 1], (uint32_t)((e >> 1) & 1), p.status, 403, &s_fail)) {
                    s_fail = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // O_tile = P V. V is the B operand as it lies in the cache: keys are its K index, dims contiguous
                // (MN-major), two 32-dim atoms side by side.
                constexpr uint32_t idesc = umma_idesc_tf32(kQT, kHS) | kIdescBMnMajor;
                const uint64_t vd = umma_desc_sw128_mn32(smem + kOffV + (e & 1) * 2 * kAtomQ, kAtomQ);
#pragma unroll
                for (int ks = 0; ks < kKT / 8; ks++) {  // 8 keys per instruction = 1024 bytes of rows
                    umma_tf32_ta(tmem_o + (uint32_t)((e & 1) * kHS), tmem_p + (uint32_t)((e & 1) * 128 + ks * 8),
                                 vd + (uint64_t)(ks * (1024 >> 4)), idesc, ks != 0 ? 1u : 0u);
                }
                umma_commit(&bar_o[e & 1]);
                // towards L2, off the path of the product above: the K and V tiles three elements ahead, the Q tile
                // three items ahead
                if (more) {
                    int k2 = k1, j2 = j1;
                    if (step(k2, j2, it1.n_kv)) {
                        const Item it2 = k2 == k1 ? it1 : get_item(k2);
                        int k3 = k2, j3 = j2;
                        if (step(k3, j3, it2.n_kv)) prefetch_kv(k3 == k2 ? it2 : get_item(k3), j3);
                    }
                }
                if (j == 0 && k + 3 < my_count) prefetch_q(k + 3);
                if (!more || s_fail) break;
                it = it1;
                k = k1;
                j = j1;
            }
        }
        __syncwarp();
    } else {
        // ================= softmax warps =================
        float o[kHS / 2];
#pragma unroll
        for (int i = 0; i < kHS / 2; i++) o[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's columns only; the halves meet when the item ends
        float corr_prev = 0.f;                 // factor that goes with the O_tile still to be collected
        const float scale2 = p.scale * 1.4426950408889634f;  // exp(x) = ex2(x * log2 e)
        int done_row0 = 0, done_nq = 0, done_h = 0;          // the item whose last O_tile is still to be collected
        bool ok = true;
        // O_tile of the previous element: o = o * (its correction) + O_tile
        auto collect = [&](int e_prev) {
            if (!mbar_wait(&bar_o[e_prev & 1], (uint32_t)((e_prev >> 1) & 1), p.status, 405, &s_fail)) s_fail = 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float ot[32];
            tmem_ld32(tmem_o + (uint32_t)((e_prev & 1) * kHS) + lane_off + hc * 32, ot);
#pragma unroll
            for (int i = 0; i < 32; i++) o[i] = o[i] * corr_prev + ot[i];
        };
        // rows of the finished item: o / (sum of both halves), this thread's 32 dims
        auto write_out = [&](float l_mine, float l_other) {
            if (row >= done_nq) return;
            const float inv = 1.0f / (l_mine + l_other);
            const size_t at = (size_t)(done_row0 + row) * p.d + done_h * kHS + hc * 32;
            if (p.out16) {
                // 64 bytes per thread, rows 1.5 KB apart: two 256-bit stores fill whole 32-byte sectors
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    uint32_t w8[8];
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const __nv_bfloat162 b = __floats2bfloat162_rn(o[16 * i + 2 * q] * inv, o[16 * i + 2 * q + 1] * inv);
                        w8[q] = *reinterpret_cast<const uint32_t*>(&b);
                    }
                    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p.out16 + at + 16 * i),
                                 "r"(w8[0]), "r"(w8[1]), "r"(w8[2]), "r"(w8[3]), "r"(w8[4]), "r"(w8[5]), "r"(w8[6]), "r"(w8[7])
                                 : "memory");
                }
            }
            if (p.out) {
                float4* dst = reinterpret_cast<float4*>(p.out + at);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    dst[i] = make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
                }
            }
        };

        int e = 0;
        for (;; e++) {
            // ---- this thread's 64 score columns of its row, into registers
            ATT_CLK(c0);
            if (!mbar_wait(&bar_s, (uint32_t)(e & 1), p.status, 404, &s_fail)) s_fail = 1;
            ATT_CLK(c1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // Scores stay unscaled: exp(scale * (s - max)) is one multiply-add and one ex2 per entry. A 32-column
            // block that lies wholly above the diagonal for every row of this warp is neither read nor exponentiated.
            const int key0 = j * kKT + hc * 64;
            const int warp_q0 = it.pos0 + (warp & 3) * 32;  // first query position of this warp's rows
            const int qpos = it.pos0 + row;  // this row's position (rows past the tile's end compute, unused)
            float sc[64];
            float m_half = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int kc = key0 + c * 32;
                if (kc <= warp_q0 + 31) {  // warp-uniform
                    float part[32];
                    tmem_ld32(tmem_s + lane_off + hc * 64 + c * 32, part);
                    if (kc + 31 > warp_q0) {  // the diagonal crosses this block
#pragma unroll
                        for (int i = 0; i < 32; i++) part[i] = kc + i <= qpos ? part[i] : -INFINITY;
                    }
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        sc[c * 32 + i] = part[i];
                        m_half = fmaxf(m_half, part[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) sc[c * 32 + i] = -INFINITY;
                }
            }
            // the scores are in registers: tell issuer A (one arrival per warp)
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_sfree);
            s_x[e & 1][hc][row] = m_half;
            if (j == 0) s_l[k & 1][hc][row] = l_run;  // the finished item's sum (nothing yet before the first)
            ATT_CLK(c2);
            const bool dead = softmax_barrier_dead(&s_fail);  // maxima (and sums) exchanged
            ATT_CLK(c3);
            if (dead) {
                ok = false;
                break;
            }
            ATT_CLK(c4);
            // ---- exponentials of this thread's columns -> P (buffer e & 1: the previous element's P may still be read)
            // Every row sees key 0, so the running maximum is finite from the first tile on and a masked entry
            // (-inf) comes out of ex2 as an exact zero.
            const float l_done = l_run;  // (if this element opens an item: the finished item's sum)
            if (j == 0) {
                m_run = -INFINITY;
                l_run = 0.f;
            }
            const float m_new = fmaxf(m_run, fmaxf(m_half, s_x[e & 1][hc ^ 1][row]));
            const float corr = ex2_approx((m_run - m_new) * scale2);  // first tile: ex2(-inf) = 0
            const float off = -m_new * scale2;
            float l_tile = 0.f;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                float pv[32];
                if (key0 + c * 32 <= warp_q0 + 31) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        pv[i] = ex2_approx(fmaf(sc[c * 32 + i], scale2, off));
                        l_tile += pv[i];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) pv[i] = 0.f;
                }
                tmem_st32(tmem_p + (uint32_t)((e & 1) * 128) + lane_off + hc * 64 + c * 32, pv);
            }
            l_run = l_run * corr + l_tile;
            m_run = m_new;
            // P is written: tell issuer B (one arrival per warp)
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_pready[e & 1]);
            ATT_CLK(c5);
            // ---- the previous element's O_tile, by now long complete
            if (e > 0) collect(e - 1);
            corr_prev = corr;
            ATT_CLK(c5b);
            if (j == 0 && e > 0) {  // that was the previous item's last O_tile
                write_out(l_done, s_l[k & 1][hc ^ 1][row]);
#pragma unroll
                for (int i = 0; i < kHS / 2; i++) o[i] = 0.f;
            }
            ATT_CLK(c6);
            ATT_ADD(0, 1);
            ATT_ADD(1, c1 - c0);   // wait for the scores
            ATT_ADD(2, c2 - c1);   // scores -> registers, mask, max
            ATT_ADD(3, c3 - c2);   // barrier (maxima exchanged)
            ATT_ADD(4, c5b - c5);  // previous O_tile (wait + read + rescale)
            ATT_ADD(5, c6 - c5b);  // item change: write-out
            ATT_ADD(6, c5 - c4);   // exponentials -> P, store wait, arrival
            int k1 = k, j1 = j;
            const bool more = step(k1, j1, it.n_kv);
            if (k1 != k) {
                done_row0 = it.row0;
                done_nq = it.nq;
                done_h = it.h;
            }
            if (!more) break;
            if (k1 != k) it = get_item(k1);
            k = k1;
            j = j1;
        }
        if (ok) {
            collect(e);
            if (s_fail) ok = false;
        }
        s_l[(k + 1) & 1][hc][row] = l_run;
        asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
        if (ok) write_out(l_run, s_l[(k + 1) & 1][hc ^ 1][row]);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

#if GRADB_DIAG
void attn_clocks_read(unsigned long long* out16, bool reset) {
    GRADB_CUDA(cudaDeviceSynchronize());
    GRADB_CUDA(cudaMemcpyFromSymbol(out16, g_attn_clock, sizeof(unsigned long long) * 16));
    if (reset) {
        unsigned long long zero[16] = {};
        GRADB_CUDA(cudaMemcpyToSymbol(g_attn_clock, zero, sizeof(zero)));
    }
}
#endif

void prefill_attention_tc_configure() {
    GRADB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
}

// tiles: up to 128 positions each. map_q: fp32 map over the query rows (boxes of 32 columns x 128 rows); map_k: fp32
// map over the whole K cache as rows of 64 floats; k_row0: first row of this layer in it.
void launch_prefill_attention_tc(const PrefillAttnParams& p, const CUtensorMap& map_q, const CUtensorMap& map_k,
                                 const CUtensorMap& map_v, long long k_row0, int sm_count, cudaStream_t st) {
    if (p.n_tiles <= 0) return;
    const int items = p.n_tiles * p.H;
    launch_kernel(attn_prefill_tc_kernel, dim3(std::min(items, sm_count)), dim3(kThreads), (size_t)kSmemBytes, st, map_q,
                  map_k, map_v, p, k_row0);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

}  // namespace gradb
