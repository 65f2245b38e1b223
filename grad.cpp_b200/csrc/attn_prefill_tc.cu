// Causal prompt attention on the 5th-generation tensor cores (head size 64), for the batched prompt feed and
// scoring of bf16 sessions: the same work as attn_prefill.cu (rows that are consecutive positions of their
// sequences attend to the cache rows at or before them, inference.cpp:208-225), with the two products of every
// (128 queries x 128 keys) tile issued as tcgen05.mma into TMEM instead of warp-level mma.sync.
//
// One CTA = one tile of up to 128 consecutive query positions of one (sequence, head); 256 threads, two per query row
// (= TMEM lane: a warp reaches the lane quarter given by its index modulo 4), each owning half of the row's score
// columns and half of its output dims. The cache stays fp32 and is fed to kind::tf32 MMAs as it lies (TF32 reads fp32 bit patterns):
//
//   S[q, key] (TMEM, 128 cols) = Q[q, :] . K[key, :]      A = Q tile, B = K tile, both dim-contiguous (K-major),
//                                                        brought by TMA tensor copies with the 128-byte swizzle
//   softmax by the row's two threads: scale, causal mask, running max / sum, P = exp(S - max) -> TMEM (128 cols):
//                                                        the A operand of the second product is read from there,
//                                                        so P never crosses shared memory
//   O_tile[q, dim] (TMEM, 64 cols) = P[q, :] . V[:, dim]   B must be key-contiguous: the V tile (a contiguous block
//                                                        of the head-major cache, one bulk copy) is transposed
//                                                        through shared memory by the threads while S is computed
//   o = o * exp(old max - new max) + O_tile              in registers (32 per thread)
//
// The K tile has two stages, so the scores of tile j+1 are issued as soon as every thread holds tile j's scores in
// registers and run under tile j's exponentials; O_tile of tile j is collected at the start of tile j+1's pass, after
// that tile's scores have been read. The next V tile is requested as soon as the transpose is done. All waits are
// bounded; on expiry the status word is set and the CTA falls through to the common exit, which frees TMEM.
#include <cuda.h>

#include "attn_prefill.cuh"

namespace gradb {

namespace {

constexpr int kQT = 128;   // queries per CTA = TMEM lanes
constexpr int kThreads = 256;
constexpr int kKT = 128;   // keys per tile
constexpr int kHS = 64;
constexpr uint32_t kSpin = 1u << 20;
constexpr int kAtomQ = kQT * 128;  // bytes of one swizzle atom of a 128-row operand: 32 floats per row
constexpr int kAtomV = kHS * 128;  // bytes of one atom of the transposed V operand: 64 rows (dims) x 32 keys
// shared-memory map (bytes from a 1024-aligned base)
constexpr int kOffQ = 0;                       // 2 atoms
constexpr int kOffK = kOffQ + 2 * kAtomQ;      // 2 stages of 2 atoms
constexpr int kOffVraw = kOffK + 4 * kAtomQ;   // [128 keys][64] as stored
constexpr int kOffVt = kOffVraw + kKT * kHS * 4;  // 4 atoms (32 keys each)
constexpr int kSmemBytes = kOffVt + 4 * kAtomV + 1024;
// tensor-memory map (columns): S, P, O_tile
constexpr uint32_t kColS = 0, kColP = 128, kColO = 256, kTmemCols = 512;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
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

// Byte offset of the 16-byte chunk `c16` (0..7) of row `r` inside a swizzle atom (128-byte rows, 8-row groups).
__device__ __forceinline__ uint32_t sw128(int r, int c16) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c16 ^ (r & 7)) << 4));
}

__global__ void __launch_bounds__(kThreads, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                      const __grid_constant__ CUtensorMap map_k,
                                                                      const PrefillAttnParams p, long long k_row0) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_q, bar_k[2], bar_v, bar_s, bar_o;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int s_fail;
    __shared__ float s_x[2][kQT];  // the two column halves of a row exchange their maxima (and, at the end, sums)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int row = (warp & 3) * 32 + lane;  // query row = TMEM lane
    const int hc = warp >> 2;                // which half of the score columns / output dims this thread owns
    const int4 tile = p.tiles[blockIdx.x];
    const int seq = tile.x, row0 = tile.y, pos0 = tile.z, nq = tile.w, h = blockIdx.y;
    const int kv_len = pos0 + nq;
    const int n_kv = (kv_len + kKT - 1) / kKT;
    const long long head_row0 = ((long long)seq * p.H + h) * p.T;  // first cache row of this (sequence, head)

    if (t == 0) {
        s_fail = 0;
        mbar_init(&bar_q, 1);
        mbar_init(&bar_k[0], 1);
        mbar_init(&bar_k[1], 1);
        mbar_init(&bar_v, 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o, 1);
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

    // thread 0 only: the K tile of keys [j*128, j*128+128) of this head into stage j & 1, two 32-float halves
    auto load_k = [&](int j) {
        uint64_t* bar = &bar_k[j & 1];
        uint8_t* dst = smem + kOffK + (j & 1) * 2 * kAtomQ;
        mbar_expect_tx(bar, 2 * kAtomQ);
        const int y = (int)(k_row0 + head_row0 + (long long)j * kKT);
        tma_load_2d(dst, &map_k, 0, y, bar);
        tma_load_2d(dst + kAtomQ, &map_k, 32, y, bar);
    };
    auto load_v = [&](int j) {  // thread 0 only: the rows of the V tile that exist, as one contiguous block
        const int rows = min(kKT, kv_len - j * kKT);
        const uint32_t bytes = (uint32_t)rows * kHS * 4;
        mbar_expect_tx(&bar_v, bytes);
        const float* src = p.vcache + (size_t)(head_row0 + (long long)j * kKT) * kHS;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(smem + kOffVraw)),
                     "l"(src), "r"(bytes), "r"(smem_u32(&bar_v))
                     : "memory");
    };
    // thread 0 only: S = Q K_j^T once stage j & 1 holds tile j (it was requested at least a tile ago)
    auto issue_scores = [&](int j) {
        if (!mbar_wait(&bar_k[j & 1], (uint32_t)((j >> 1) & 1), p.status, 402, &s_fail)) {
            s_fail = 1;
            return;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        constexpr uint32_t idesc = umma_idesc_tf32(kQT, kKT);
#pragma unroll
        for (int a = 0; a < 2; a++) {  // 32 dims per atom, 8 per instruction
            const uint64_t qd = umma_desc_sw128(smem + kOffQ + a * kAtomQ);
            const uint64_t kd = umma_desc_sw128(smem + kOffK + ((j & 1) * 2 + a) * kAtomQ);
#pragma unroll
            for (int kk = 0; kk < 4; kk++) umma_tf32(tmem_s, qd + 2 * kk, kd + 2 * kk, idesc, (a | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&bar_s);
    };
    if (t == 0) {
        mbar_expect_tx(&bar_q, 2 * kAtomQ);
        tma_load_2d(smem + kOffQ, &map_q, h * kHS, row0, &bar_q);
        tma_load_2d(smem + kOffQ + kAtomQ, &map_q, h * kHS + 32, row0, &bar_q);
        load_k(0);
        if (n_kv > 1) load_k(1);
        load_v(0);
        if (mbar_wait(&bar_q, 0, p.status, 401, &s_fail)) issue_scores(0);
        else s_fail = 1;
    }

    float o[kHS / 2];
#pragma unroll
    for (int i = 0; i < kHS / 2; i++) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's columns only; the halves meet at the end
    float corr_prev = 0.f;                 // factor that goes with the O_tile still to be collected
    const float scale2 = p.scale * 1.4426950408889634f;  // exp(x) = ex2(x * log2 e)
    const int qpos = pos0 + row;  // the position this row's query sits at (rows past the tile's end compute, unused)
    bool ok = true;
    // O_tile of the previous tile: o = o * (its correction) + O_tile
    auto collect = [&](int j_prev) {
        if (!mbar_wait(&bar_o, (uint32_t)(j_prev & 1), p.status, 405, &s_fail)) s_fail = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float ot[32];
        tmem_ld32(tmem_o + lane_off + hc * 32, ot);
#pragma unroll
        for (int i = 0; i < 32; i++) o[i] = o[i] * corr_prev + ot[i];
    };

    for (int j = 0; j < n_kv; j++) {
        const uint32_t ph = (uint32_t)(j & 1);
        // ---- this thread's 64 score columns of its row, into registers
        if (!mbar_wait(&bar_s, ph, p.status, 404, &s_fail)) s_fail = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // Scores stay unscaled: exp(scale * (s - max)) is one multiply-add and one ex2 per entry. A 32-column block
        // that lies wholly above the diagonal for every row of this warp is neither read nor exponentiated.
        const int key0 = j * kKT + hc * 64;
        const int warp_q0 = pos0 + (warp & 3) * 32;  // first query position of this warp's rows
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
        s_x[hc][row] = m_half;
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();  // maxima exchanged; the score accumulator and this tile's K stage are free
        if (s_fail) {
            ok = false;
            break;
        }
        if (t == 0) {  // the next tile's scores run under this tile's exponentials
            if (j + 2 < n_kv) load_k(j + 2);
            if (j + 1 < n_kv) issue_scores(j + 1);
        }
        if (j > 0) collect(j - 1);  // after this the P and transposed-V buffers are free as well

        // ---- V tile -> key-contiguous operand. Lane = dim (reads are consecutive words), one key per step.
        if (!mbar_wait(&bar_v, ph, p.status, 403, &s_fail)) s_fail = 1;
        {
            const int rows = min(kKT, kv_len - j * kKT);
            const float* vraw = reinterpret_cast<const float*>(smem + kOffVraw);
            // four keys at a time: each lane gathers its dim's four values and stores them as one 16-byte chunk
#pragma unroll
            for (int g = warp; g < kKT / 4; g += kThreads / 32) {
                float a[4], b[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int key = g * 4 + i;
                    const bool live = key < rows;  // rows past the context are zero: a masked 0 times stale bits must stay 0
                    a[i] = live ? vraw[key * kHS + lane] : 0.f;
                    b[i] = live ? vraw[key * kHS + 32 + lane] : 0.f;
                }
                uint8_t* atom = smem + kOffVt + (g >> 3) * kAtomV;
                *reinterpret_cast<float4*>(atom + sw128(lane, g & 7)) = make_float4(a[0], a[1], a[2], a[3]);
                *reinterpret_cast<float4*>(atom + sw128(lane + 32, g & 7)) = make_float4(b[0], b[1], b[2], b[3]);
            }
        }
        // ---- exponentials of this thread's columns -> P
        // Every row sees key 0, so the running maximum is finite from the first tile on and a masked entry
        // (-inf) comes out of ex2 as an exact zero.
        const float m_new = fmaxf(m_run, fmaxf(m_half, s_x[hc ^ 1][row]));
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
            tmem_st32(tmem_p + lane_off + hc * 64 + c * 32, pv);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        l_run = l_run * corr + l_tile;
        m_run = m_new;
        corr_prev = corr;
        // the transposed V was written by ordinary stores: order them before the tensor core's reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();  // also: the raw V tile is free
        if (s_fail) {
            ok = false;
            break;
        }
        // ---- O_tile = P V (collected at the start of the next pass, or after the loop)
        if (t == 0) {
            if (j + 1 < n_kv) load_v(j + 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            constexpr uint32_t idesc = umma_idesc_tf32(kQT, kHS);
#pragma unroll
            for (int a = 0; a < 4; a++) {  // 32 keys per atom, 8 per instruction
                const uint64_t vd = umma_desc_sw128(smem + kOffVt + a * kAtomV);
#pragma unroll
                for (int kk = 0; kk < 4; kk++)
                    umma_tf32_ta(tmem_o, tmem_p + (uint32_t)(a * 32 + kk * 8), vd + 2 * kk, idesc, (a | kk) != 0 ? 1u : 0u);
            }
            umma_commit(&bar_o);
        }
    }
    if (ok) {
        collect(n_kv - 1);
        if (s_fail) ok = false;
    }

    s_x[hc][row] = l_run;
    __syncthreads();
    if (ok && row < nq) {
        const float inv = 1.0f / (l_run + s_x[hc ^ 1][row]);
        const size_t at = (size_t)(row0 + row) * p.d + h * kHS + hc * 32;
        if (p.out16) {
            uint4* dst = reinterpret_cast<uint4*>(p.out16 + at);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                __nv_bfloat162 b[4];
#pragma unroll
                for (int k = 0; k < 4; k++) b[k] = __floats2bfloat162_rn(o[8 * i + 2 * k] * inv, o[8 * i + 2 * k + 1] * inv);
                dst[i] = *reinterpret_cast<const uint4*>(b);
            }
        }
        if (p.out) {
            float4* dst = reinterpret_cast<float4*>(p.out + at);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                dst[i] = make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

void prefill_attention_tc_configure() {
    GRADB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
}

// tiles: up to 128 positions each. map_q: fp32 map over the query rows (boxes of 32 columns x 128 rows); map_k: fp32
// map over the whole K cache as rows of 64 floats; k_row0: first row of this layer in it.
void launch_prefill_attention_tc(const PrefillAttnParams& p, const CUtensorMap& map_q, const CUtensorMap& map_k,
                                 long long k_row0, cudaStream_t st) {
    if (p.n_tiles <= 0) return;
    launch_kernel(attn_prefill_tc_kernel, dim3(p.n_tiles, p.H), dim3(kThreads), (size_t)kSmemBytes, st, map_q, map_k, p,
                  k_row0);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

}  // namespace gradb
