// Batched-decode / prompt-feed projections on the 5th-generation tensor cores.
//
// For a batch of sequences the projections of one step are real GEMMs:
//     Y[b, n] = sum_k X[b, k] * W[k, n]        (inference.cpp:14-28, 94-96, 254 for one row)
// They are computed "swapped": the weight tile supplies the 128 MMA rows (one
// TMEM lane per output feature n) and the tokens supply the MMA columns, so any
// batch from 16 to 256 fills the instruction and the epilogue writes rows of
// consecutive features, which is the memory order of every consumer.
//
//   D[n, b] (fp32, TMEM) = A[n, k] (bf16 weights, K-major, TMA) * B[b, k]^T (bf16 activations, K-major, TMA)
//
// One CTA = one 128-feature tile (two tiles for SwiGLU: gate and up) x one token
// tile x one K split. Warp 0 lane 0 feeds a 4-stage shared-memory ring with TMA,
// warp 1 lane 0 issues tcgen05.mma and releases stages with tcgen05.commit, and all
// sixteen warps (four per TMEM lane quarter) run the epilogue from TMEM (bias, RoPE +
// cache write, GELU / SwiGLU, residual add, logits) once the accumulator barrier fires.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in
// the session's status word and falls through to the common exit, which frees
// TMEM. TMA loads here are plain per-CTA loads of this GPU's own memory.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>

#include "gemm_tc.cuh"

namespace gradb {

namespace {

// Ring depth: four stages (fewer only if a stage is very large). Deeper rings were measured slower here:
// they push every variant to one CTA per SM and lengthen the prologue of kernels that run for a few microseconds.
// The widest token tile only occurs with many CTAs per SM's worth of rows (prompt feed, scoring); its ring is
// sized for two CTAs per SM so that one CTA's epilogue runs under the other's main loop.
constexpr int stages_for(int nw, int tn, int kind = 0) {
    const int stage = (nw * 128 * 128 + tn * 128) * (kind == 1 ? 2 : 1);  // 128-byte rows; hi and lo halves in fp32 mode
    const int n = ((tn >= 128 ? 100 : 200) * 1024) / stage;
    return n > 4 ? 4 : (n < 2 ? 2 : n);
}
constexpr int kBlockK = 64;  // bf16 elements = one 128-byte swizzle row
// Warps per TMEM lane quarter in the one-tile-per-CTA kernel's epilogue: the epilogue is a latency chain, so the
// short decode tiles spread their token columns over four warps per quarter (16 warps), the widest tile over two.
constexpr int epi_warps_for(int tn) { return tn <= 64 ? 4 : 2; }  // eight per quarter measured slower
constexpr int kTileM = 128;  // features per MMA
constexpr uint32_t kSpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait. Returns false (and records `code`) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
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
    }
    atomicExch(status, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_tile) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)0 << 16;                   // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
    d |= (uint64_t)1 << 46;                   // descriptor version
    d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16: bf16 x bf16 -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// kind::tf32: fp32 bit patterns in shared memory, the low 13 mantissa bits ignored; K = 8 per instruction.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// TF32-rounded value and TF32-rounded remainder: hi + lo carries 21 or more mantissa bits of x.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hi));
    lo = __uint_as_float(l);
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}
template <int CW>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[CW]) {
    if constexpr (CW == 32) tmem_ld32(taddr, v);
    else if constexpr (CW == 16) tmem_ld16(taddr, v);
    else tmem_ld8(taddr, v);
}

// Epilogue of one output tile, run by the four warps that own the TMEM lane quarters: thread t
// (0..127, t / 32 = the warp's lane quarter) owns feature tile_n * 128 + t; lane_addr is the
// accumulator's TMEM address with the quarter's lane offset applied. nz = number of K splits.
template <int EPI, int NW, int TN, int CW = 32, int KIND = 0>
__device__ __forceinline__ void tc_epilogue(const TcGemmParams& p, uint32_t lane_addr, int t, int tile_n, int tile_b,
                                            int kz, int nz, const int* s_tok, const int* s_pos, const long long* s_off,
                                            int c_begin = 0, int c_end = TN) {
    const int n = tile_n * kTileM + t;  // feature index inside one matrix (for NW=2: same n in gate and up)
    const bool n_ok = n < p.N;
    int which = 0, n_in = n;
    float bias = 0.f;
    if (EPI == TC_QKV) {
        which = n / p.d;
        n_in = n - which * p.d;
        if (n_ok) bias = p.bias[which][n_in];
    } else if (EPI == TC_RESID || EPI == TC_GELU) {
        if (n_ok && p.bias[0] && kz == 0) bias = p.bias[0][n];
    }
    const int h = n_in / p.hs, c_in = n_in % p.hs, half = p.hs / 2;
    const bool rope = EPI == TC_QKV && p.rope_cos != nullptr && which < 2;
    // Per-thread base pointers; the per-token part of every address is staged in shared memory (s_off:
    // element offset of the token's cache row for head 0) or is a multiple of the row pitch.
    const float* cos_t = p.rope_cos + c_in / 2;
    const float* sin_t = p.rope_sin + c_in / 2;
    float* kv_t = (which == 1 ? p.kcache : p.vcache) + (size_t)h * p.T * p.hs + c_in;
    float* out_t = p.out_f32 + (EPI == TC_QKV ? n_in : n);
    __nv_bfloat16* out16_t = p.out_bf16 + n;
    for (int c0 = c_begin; c0 < c_end; c0 += CW) {
        float v[CW], v2[CW];
        tmem_ld<CW>(lane_addr + c0, v);
        if (NW == 2) tmem_ld<CW>(lane_addr + TN + c0, v2);
        // kGroup tokens at a time, in three passes so that independent work is adjacent: every load the
        // group needs (all in flight together), then the arithmetic of all its tokens (one warp per
        // scheduler runs this code, so latency is only hidden by instruction-level parallelism), then the stores.
        constexpr int kGroup = TN >= 128 ? 16 : 8;
#pragma unroll
        for (int j0 = 0; j0 < CW; j0 += kGroup) {
            float aux0[kGroup], aux1[kGroup], res[kGroup];
            int posn[kGroup];
            bool live[kGroup];
#pragma unroll
            for (int jj = 0; jj < kGroup; jj++) {
                const int c = c0 + j0 + jj;
                live[jj] = s_tok[c] >= 0;  // warp-uniform; rows past the batch were staged as skipped
                posn[jj] = s_pos[c];
                aux0[jj] = aux1[jj] = 0.f;
                if (rope) {
                    aux0[jj] = __ldg(cos_t + posn[jj] * half);
                    aux1[jj] = __ldg(sin_t + posn[jj] * half);
                }
                if (EPI == TC_RESID && nz == 1 && live[jj] && n_ok) {
                    aux0[jj] = out_t[(size_t)(tile_b * TN + c) * p.ld_out];
                }
            }
#pragma unroll
            for (int jj = 0; jj < kGroup; jj++) {
                const int j = j0 + jj;
                float val = v[j] + bias;
                if (EPI == TC_QKV) {
                    if (rope) {
                        // pairs (2j, 2j+1) inside a head sit in neighbouring lanes (inference.cpp:101-115)
                        const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                        val = (c_in & 1) ? (other * aux1[jj] + val * aux0[jj]) : (val * aux0[jj] - other * aux1[jj]);
                    }
                } else if (EPI == TC_RESID) {
                    if (nz == 1) val += aux0[jj];
                } else if (EPI == TC_GELU) {
                    const float u = 0.79788456f * (val + 0.044715f * val * val * val);
                    val = 0.5f * val * (1.0f + tanhf(u));
                } else if (EPI == TC_SWIGLU) {
                    const float gte = v[j];
                    val = v2[j] * (gte / (1.0f + __expf(-gte)));
                } else {
                    val = v[j];
                }
                res[jj] = val;
            }
#pragma unroll
            for (int jj = 0; jj < kGroup; jj++) {
                if (!(live[jj] && n_ok)) continue;
                const int c = c0 + j0 + jj;
                const int b = tile_b * TN + c;
                if (EPI == TC_QKV) {
                    if (which == 0) out_t[(size_t)b * p.ld_out] = res[jj];
                    else kv_t[s_off[c]] = res[jj];
                } else if (EPI == TC_RESID) {
                    float* y = out_t + (size_t)b * p.ld_out;
                    if (nz == 1) *y = res[jj];
                    else atomicAdd(y, res[jj]);
                } else if (EPI == TC_GELU || EPI == TC_SWIGLU) {
                    if (KIND == 1) {
                        float hi, lo;
                        split_tf32(res[jj], hi, lo);
                        float* y = p.out_split + (size_t)b * p.ld_out + n;
                        y[0] = hi;
                        y[p.out_lo_elems] = lo;
                    } else {
                        out16_t[(size_t)b * p.ld_out] = __float2bfloat16_rn(res[jj]);
                    }
                } else {  // TC_LOGITS
                    out_t[(size_t)b * p.ld_out] = res[jj];
                }
            }
        }
    }
}

// Shared memory: [stage][A tiles (NW x 16 KB) | B tile (TN x 128 B)], 1024-byte aligned.
// KIND 1 (fp32 mode): each operand tile comes as a TF32 hi tile and a lo tile (two TMA boxes), K blocks are 32
// elements (still one 128-byte swizzle row) and every product is three MMAs: lo*hi + hi*lo + hi*hi.
template <int EPI, int NW, int TN, int KIND = 0>
__global__ void __launch_bounds__(128 * epi_warps_for(TN)) gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_b,
                                                           const TcGemmParams p) {
    constexpr int kStages = stages_for(NW, TN, KIND);
    constexpr int kParts = KIND == 1 ? 2 : 1;
    constexpr int kBlockK = KIND == 1 ? 32 : 64;  // elements per 128-byte row (shadows the bf16 constant)
    constexpr int kATile = kTileM * 128, kBTile = TN * 128;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], accum_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_tok[TN], s_pos[TN];
    __shared__ long long s_off[TN];

    constexpr int kABytes = NW * kParts * kATile;
    constexpr int kBBytes = kParts * kBTile;
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr int kTmemCols = NW * TN < 32 ? 32 : NW * TN;
    static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two");

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, tile_b = blockIdx.y, kz = blockIdx.z;
    const int k_iters_total = p.K / kBlockK;
    const int k_per = (k_iters_total + gridDim.z - 1) / gridDim.z;
    const int k_beg = kz * k_per, k_end = min(k_iters_total, k_beg + k_per);
    const int n_iters = max(0, k_end - k_beg);

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    bool ok = true;

    // The weight tiles do not depend on earlier kernels: start their stream before waiting for the
    // predecessor (programmatic dependent launch); activations, positions and ids come after.
    const int pre = min(n_iters, kStages);
    if (threadIdx.x == 0) {
        for (int it = 0; it < pre; it++) {
            uint8_t* st = smem + (size_t)it * kStageBytes;
            mbar_expect_tx(&full_bar[it], kStageBytes);
            const int kx = (k_beg + it) * kBlockK;
#pragma unroll
            for (int w = 0; w < NW; w++) {
#pragma unroll
                for (int part = 0; part < kParts; part++) {
                    tma_load_2d(st + (w * kParts + part) * kATile, &map_a, kx,
                                (tile_n * NW + w) * kTileM + part * p.a_lo_rows, &full_bar[it]);
                }
            }
        }
    }
    pdl_wait();
    // Activations first: their tiles are what the first MMA waits for; the ids and positions staged
    // below are only read by the epilogue.
    if (threadIdx.x == 0) {
        for (int it = 0; it < pre; it++) {
#pragma unroll
            for (int part = 0; part < kParts; part++) {
                tma_load_2d(smem + (size_t)it * kStageBytes + kABytes + part * kBTile, &map_b, (k_beg + it) * kBlockK,
                            tile_b * TN + part * p.b_lo_rows, &full_bar[it]);
            }
        }
    }
    for (int c = threadIdx.x; c < TN; c += blockDim.x) {
        const int b = blockIdx.y * TN + c;
        const int tk = b < p.B ? p.tok[b] : kSkip;
        const int ps = tk >= 0 ? p.pos[b] : 0;
        const int sq = (tk >= 0 && p.row_seq) ? p.row_seq[b] : b;
        s_tok[c] = tk;
        s_pos[c] = ps;
        s_off[c] = (((long long)sq * p.H) * p.T + ps) * p.hs;
    }
    __syncthreads();

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (the first `pre` stages were requested above)
        for (int it = pre; it < n_iters && ok; it++) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            ok = mbar_wait(&empty_bar[s], ph ^ 1, p.status, 101);
            if (!ok) break;
            uint8_t* st = smem + (size_t)s * kStageBytes;
            mbar_expect_tx(&full_bar[s], kStageBytes);
            const int kx = (k_beg + it) * kBlockK;
#pragma unroll
            for (int w = 0; w < NW; w++) {
#pragma unroll
                for (int part = 0; part < kParts; part++) {
                    tma_load_2d(st + (w * kParts + part) * kATile, &map_a, kx,
                                (tile_n * NW + w) * kTileM + part * p.a_lo_rows, &full_bar[s]);
                }
            }
#pragma unroll
            for (int part = 0; part < kParts; part++) {
                tma_load_2d(st + kABytes + part * kBTile, &map_b, kx, tile_b * TN + part * p.b_lo_rows, &full_bar[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc = KIND == 1 ? umma_idesc_tf32(kTileM, TN) : umma_idesc_bf16(kTileM, TN);
        for (int it = 0; it < n_iters && ok; it++) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            ok = mbar_wait(&full_bar[s], ph, p.status, 102);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint8_t* st = smem + (size_t)s * kStageBytes;
            const uint64_t bdesc = umma_desc_sw128(st + kABytes);
#pragma unroll
            for (int w = 0; w < NW; w++) {
                const uint64_t adesc = umma_desc_sw128(st + w * kParts * kATile);
                if constexpr (KIND == 0) {
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        // 16 bf16 = 32 bytes further along K inside the swizzle row: +2 in the address field
                        umma_bf16(tmem_base + w * TN, adesc + 2 * k, bdesc + 2 * k, idesc, (it | k) != 0 ? 1u : 0u);
                    }
                } else {
                    const uint64_t adesc_lo = umma_desc_sw128(st + (w * kParts + 1) * kATile);
                    const uint64_t bdesc_lo = umma_desc_sw128(st + kABytes + kBTile);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        // 8 tf32 = 32 bytes along K; small cross terms first, then the main product
                        umma_tf32(tmem_base + w * TN, adesc_lo + 2 * k, bdesc + 2 * k, idesc, (it | k) != 0 ? 1u : 0u);
                        umma_tf32(tmem_base + w * TN, adesc + 2 * k, bdesc_lo + 2 * k, idesc, 1u);
                        umma_tf32(tmem_base + w * TN, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
                    }
                }
            }
            umma_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
        }
        umma_commit(&accum_bar);  // accumulator complete
    }
    __syncwarp();

    // ---- epilogue: thread t owns TMEM lane t = feature n0 + t
    if (n_iters > 0) ok = mbar_wait(&accum_bar, 0, p.status, 103);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && n_iters > 0) {
        // TMEM lane quarter = warp modulo 4; the quarter's warps split the token columns between them
        // (one warp per scheduler would leave every latency of this code exposed)
        constexpr int kEW = epi_warps_for(TN);
        constexpr int kCols = TN / kEW;  // token columns per warp
        const int q = warp & 3, part = warp >> 2;
        tc_epilogue<EPI, NW, TN, (kCols >= 32 ? 32 : kCols), KIND>(p, tmem_base + ((uint32_t)(q * 32) << 16), q * 32 + lane,
                                                             tile_n, tile_b, kz, (int)gridDim.z, s_tok, s_pos, s_off,
                                                             part * kCols, (part + 1) * kCols);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The same GEMM for many rows (prompt feed, scoring): persistent, one CTA per SM, warp-specialised.
// With thousands of 128x128 output tiles the one-tile-per-CTA kernel above spends most of each CTA's
// life in its prologue, in the TMA round trips of a short ring and in an epilogue that nothing
// overlaps (tensor pipe 11-26 % busy). Here
//   warp 0 (one lane)  streams A and B tiles through a deep ring, running ahead across tile boundaries,
//   warp 1 (one lane)  issues the MMAs into one of TWO accumulators in TMEM,
//   warps 2-17         drain the other accumulator (the shared epilogue; four warps per TMEM lane quarter,
//                      a quarter of the token columns each), so the epilogue of tile i runs under the main
//                      loop of tile i+1. The epilogue is arithmetic- and latency-bound, hence sixteen warps.
// Tiles are dealt round-robin, feature tile fastest, so CTAs working at the same time share a token tile in L2.
// Token tile: 128, or 256 for the single-weight-tile projections when there are enough rows (one MMA then covers
// 128 x 256 outputs, which needs a quarter fewer operand bytes per multiply-add from L2 and from shared memory; the
// operands, not the arithmetic, set the main loop's pace). The epilogue always works on 128 tokens at a time.
constexpr int kWideTN = 128;
constexpr int kWideHalf = 128;  // tokens per epilogue round = rows of the staged tile
// CG 2: two CTAs of a cluster (the two SMs of a TPC) work as one MMA unit (cta_group::2): the pair computes 256
// features x 256 tokens per tile, each CTA holding its own 128 weight rows and HALF of the token tile, so a CTA
// loads 32 KB per K block for the 128 x 256 outputs it keeps instead of 48 KB, and the ring has room for four stages.
constexpr int wide_stages(int nw, int tn, int cg = 1) { return cg == 2 || (nw == 1 && tn == 128) ? 4 : 3; }
constexpr int kWideStageTileBytes = kWideHalf * kTileM * 4;    // + one fp32 output tile staged for the row-wise epilogue
constexpr size_t wide_smem_bytes(int nw, int tn, int cg = 1) {
    return (size_t)wide_stages(nw, tn, cg) * (nw * kTileM * kBlockK * 2 + tn / cg * kBlockK * 2) + kWideStageTileBytes +
           1024;
}
// Four epilogue warps per TMEM lane quarter: with eight warps in all the epilogue, not the MMA stream, set a tile's
// time (scoring 65536 ids: 23.3 -> 20.6 ms with sixteen; 256-token tiles on top of that measured no gain).
constexpr int kWideEpiWarps = 16;
constexpr int kWideThreads = 64 + 32 * kWideEpiWarps;

// Epilogue pass A of the persistent kernel: accumulator (TMEM, one lane per feature) -> fp32 tile in shared
// memory laid out [token][feature], with the per-feature work done on the way (bias, GELU, SwiGLU).
// Thread t = feature, columns [c_begin, c_end). Consecutive lanes write consecutive words: no bank conflicts.
template <int EPI, int NW, int TN>
__device__ __forceinline__ void wide_epilogue_stage(const TcGemmParams& p, uint32_t lane_addr, int t, int tile_n,
                                                    float* stg, int c_begin, int c_end) {
    const int n = tile_n * kTileM + t;
    const bool n_ok = n < p.N;
    float bias = 0.f;
    if (EPI == TC_QKV) {
        const int which = n / p.d;
        if (n_ok) bias = p.bias[which][n - which * p.d];
    } else if (EPI == TC_RESID || EPI == TC_GELU) {
        if (n_ok && p.bias[0]) bias = p.bias[0][n];
    }
    // columns per TMEM load: the SwiGLU pair holds two loads at once, and the 256-token variants carry more state
    constexpr int CW = (NW == 2 || (TN == 256 && EPI != TC_QKV)) ? 16 : 32;
    for (int c0 = c_begin; c0 < c_end; c0 += CW) {
        float v[CW], v2[CW];
        tmem_ld<CW>(lane_addr + c0, v);
        if (NW == 2) tmem_ld<CW>(lane_addr + TN + c0, v2);
#pragma unroll
        for (int j = 0; j < CW; j++) {
            float val = v[j] + bias;
            if (EPI == TC_GELU) {
                const float u = 0.79788456f * (val + 0.044715f * val * val * val);
                val = 0.5f * val * (1.0f + tanhf(u));
            } else if (EPI == TC_SWIGLU) {
                const float gte = v[j];
                val = v2[j] * (gte / (1.0f + __expf(-gte)));
            }
            stg[(c0 + j) * kTileM + t] = val;
        }
    }
}

// Epilogue pass B: the staged tile, one token row per warp at a time, four consecutive features per lane:
// everything that depends on the token (RoPE angle, cache row, residual row) is fetched once per row and the
// stores are 128-bit and row-contiguous. A warp owns rows we, we + 16, ... of the 128 (eight of them), and the
// pass comes in two parts: wide_rows_fetch issues the eight rows' global loads that do not depend on the
// accumulator (RoPE angles, residual rows) and is called before the staged tile is waited for, so their latency
// runs under the accumulator wait and pass A; wide_rows_finish does the rest. A row past the batch (id < 0)
// reads row 0 of the tile and position 0, and is not stored.
constexpr int kWideRowsPerWarp = kWideHalf / kWideEpiWarps;
constexpr int kWideRowBatch = 4;  // rows whose fetched values are held at a time (registers: 96 per thread)

template <int EPI>
struct WideRowCtx {
    int f, n_in, c_in, which;
    bool f_in, rope;
    float* kv_t;
    __device__ __forceinline__ WideRowCtx(const TcGemmParams& p, int lane, int tile_n) {
        f = tile_n * kTileM + 4 * lane;  // first of this lane's four features
        f_in = f < p.N;                  // N is a multiple of 4 on this path
        which = 0;
        n_in = f;
        if (EPI == TC_QKV) {
            which = f / p.d;  // a 128-feature tile lies inside one of Q, K, V (d is a multiple of 128 on this path)
            n_in = f - which * p.d;
        }
        const int h = n_in / p.hs;
        c_in = n_in % p.hs;
        rope = EPI == TC_QKV && p.rope_cos != nullptr && which < 2;
        kv_t = (which == 1 ? p.kcache : p.vcache) + (size_t)h * p.T * p.hs + c_in;
    }
};

template <int EPI>
__device__ __forceinline__ void wide_rows_fetch(const TcGemmParams& p, const WideRowCtx<EPI>& cx, int we, int i0,
                                                int row_base, const int* s_tok, const int* s_pos,
                                                float4 (&pre)[kWideRowBatch]) {
    if (!cx.f_in) return;
    if (EPI == TC_QKV && cx.rope) {
        // pairs (2j, 2j+1) of a head rotate by the angle of index j (inference.cpp:101-115)
        const int half = p.hs / 2;
#pragma unroll
        for (int i = 0; i < kWideRowBatch; i++) {
            const int c = we + (i0 + i) * kWideEpiWarps;
            const int pos = s_tok[c] >= 0 ? s_pos[c] : 0;
            const float2 cs = __ldg(reinterpret_cast<const float2*>(p.rope_cos + (size_t)pos * half + cx.c_in / 2));
            const float2 sn = __ldg(reinterpret_cast<const float2*>(p.rope_sin + (size_t)pos * half + cx.c_in / 2));
            pre[i] = make_float4(cs.x, cs.y, sn.x, sn.y);
        }
    } else if (EPI == TC_RESID) {
#pragma unroll
        for (int i = 0; i < kWideRowBatch; i++) {
            const int c = we + (i0 + i) * kWideEpiWarps;
            const size_t row = (size_t)(row_base + (s_tok[c] >= 0 ? c : 0)) * p.ld_out;
            pre[i] = *reinterpret_cast<const float4*>(p.out_f32 + row + cx.f);
        }
    }
}

template <int EPI>
__device__ __forceinline__ void wide_rows_lse(const TcGemmParams& p, const WideRowCtx<EPI>& cx, const float* stg, int we,
                                              int lane, int tile_n, int row_base, const int* s_tok, const int* s_pos) {
    // This tile's share of each row's log-sum-exp, and the target's logit if it lives here. The row maxima come
    // from one warp-wide instruction each; four rows' sums are reduced together, exchanging half of the rows at each
    // of the first two butterfly steps (6 shuffles instead of 20): afterwards the eight lanes with (lane >> 3) == i
    // hold row i's sum.
    constexpr int R = kWideRowBatch;
    static_assert(R == 4, "the butterfly below is written for four rows");
    if (tile_n * kTileM >= p.N) return;  // the odd CTA of the last pair when the tile count is odd: nothing to leave
#pragma unroll 1
    for (int i0 = 0; i0 < kWideRowsPerWarp; i0 += R) {
        float4 x[R];
        float m[R], sum[R];
#pragma unroll
        for (int i = 0; i < R; i++) {
            x[i] = *reinterpret_cast<const float4*>(stg + (we + (i0 + i) * kWideEpiWarps) * kTileM + 4 * lane);
            if (!cx.f_in) x[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            const float m4 = fmaxf(fmaxf(x[i].x, x[i].y), fmaxf(x[i].z, x[i].w));
            asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(m[i]) : "f"(m4));
            sum[i] = (expf(x[i].x - m[i]) + expf(x[i].y - m[i])) + (expf(x[i].z - m[i]) + expf(x[i].w - m[i]));
        }
        float w2[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const bool up = lane & 16;
            const float got = __shfl_xor_sync(0xffffffffu, up ? sum[i] : sum[i + 2], 16);
            w2[i] = (up ? sum[i + 2] : sum[i]) + got;
        }
        float tot;
        {
            const bool up = lane & 8;
            const float got = __shfl_xor_sync(0xffffffffu, up ? w2[0] : w2[1], 8);
            tot = (up ? w2[1] : w2[0]) + got;
        }
        tot += __shfl_xor_sync(0xffffffffu, tot, 4);
        tot += __shfl_xor_sync(0xffffffffu, tot, 2);
        tot += __shfl_xor_sync(0xffffffffu, tot, 1);
        const int mine = lane >> 3;  // the row of this batch whose sum this lane holds
        float m_mine = m[0];
#pragma unroll
        for (int i = 1; i < R; i++) m_mine = mine == i ? m[i] : m_mine;
        {
            const int c = we + (i0 + mine) * kWideEpiWarps;
            if ((lane & 7) == 0 && s_tok[c] >= 0) {
                *reinterpret_cast<float2*>(p.out_f32 + (size_t)(row_base + c) * p.ld_out + 2 * tile_n) = make_float2(m_mine, tot);
            }
        }
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int c = we + (i0 + i) * kWideEpiWarps;
            if (s_tok[c] < 0) continue;
            const int tg = s_pos[c] - cx.f;  // `pos` carries the target id on this path
            if (tg >= 0 && tg < 4) p.lse_tgt[row_base + c] = tg == 0 ? x[i].x : (tg == 1 ? x[i].y : (tg == 2 ? x[i].z : x[i].w));
        }
    }
}

template <int EPI>
__device__ __forceinline__ void wide_rows_finish(const TcGemmParams& p, const WideRowCtx<EPI>& cx, const float* stg, int we,
                                                 int lane, int i0, int row_base, const int* s_tok, const long long* s_off,
                                                 const float4 (&pre)[kWideRowBatch]) {
    if (!cx.f_in) return;
#pragma unroll
    for (int i = 0; i < kWideRowBatch; i++) {
        const int c = we + (i0 + i) * kWideEpiWarps;
        if (s_tok[c] < 0) continue;  // warp-uniform
        float4 x = *reinterpret_cast<const float4*>(stg + c * kTileM + 4 * lane);
        const size_t row = (size_t)(row_base + c) * p.ld_out;
        if (EPI == TC_QKV) {
            if (cx.rope) {
                const float a0 = x.x, b0 = x.y, a1 = x.z, b1 = x.w;  // pre = (cos j, cos j+1, sin j, sin j+1)
                x.x = a0 * pre[i].x - b0 * pre[i].z;
                x.y = a0 * pre[i].z + b0 * pre[i].x;
                x.z = a1 * pre[i].y - b1 * pre[i].w;
                x.w = a1 * pre[i].w + b1 * pre[i].y;
            }
            if (cx.which == 0) *reinterpret_cast<float4*>(p.out_f32 + row + cx.n_in) = x;
            else *reinterpret_cast<float4*>(cx.kv_t + s_off[c]) = x;
        } else if (EPI == TC_RESID) {
            *reinterpret_cast<float4*>(p.out_f32 + row + cx.f) =
                make_float4(x.x + pre[i].x, x.y + pre[i].y, x.z + pre[i].z, x.w + pre[i].w);
        } else if (EPI == TC_GELU || EPI == TC_SWIGLU) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(p.out_bf16 + row + cx.f) = pk;
        } else {  // TC_LOGITS
            *reinterpret_cast<float4*>(p.out_f32 + row + cx.f) = x;
        }
    }
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Diagnostics build: CTA 0's three roles add up the clock cycles they spend in each part of a tile
// (read through gradb_diag_wide_clocks).
#if GRADB_DIAG
// GRADB_DIAG_WIDE_SKIP leaves parts of the kernel out so that the others can be timed alone (results are then
// meaningless): 1 no accumulator -> staged tile pass, 2 no row pass, 4 no MMAs, 8 no copies and no waiting for them.
__device__ int g_wide_skip;
#define WIDE_SKIP() (g_wide_skip)
__device__ unsigned long long g_wide_clock[8 * 16];  // [epilogue kind][counter]
#define WIDE_CLK(x) const long long x = clock64()
#define WIDE_ADD(i, v) do { if (blockIdx.x == 0) atomicAdd(&g_wide_clock[EPI * 16 + (i)], (unsigned long long)(v)); } while (0)
#else
#define WIDE_CLK(x)
#define WIDE_ADD(i, v)
#define WIDE_SKIP() 0
#endif

// ---- CTA-pair forms. The even CTA of the pair leads: it issues the MMAs, and the "stage full" and "accumulator
// drained" barriers that it waits on are its own, signalled by both CTAs (a shared-memory address with bit 24
// cleared names the same offset in the pair's even CTA).
constexpr uint32_t kPairLeaderMask = 0xFEFFFFFFu;
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Plain (not multicast) tensor copy into this CTA's shared memory whose bytes are counted on the leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar) & kPairLeaderMask)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far are complete.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPairLeaderMask) : "memory");
}

template <int EPI, int NW, int TN, int CG = 1>
__global__ void __launch_bounds__(kWideThreads, 1) gemm_bf16_tc_wide_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_b,
                                                                const TcGemmParams p, int tiles_n, int total_tiles) {
    static_assert(CG == 1 || (NW == 1 && TN == 256), "CTA pairs: one weight tile per CTA, 256 tokens per pair");
    constexpr int kStages = wide_stages(NW, TN, CG);
    constexpr int kABytes = NW * kTileM * kBlockK * 2;
    constexpr int kBBytes = TN / CG * kBlockK * 2;  // a CTA of a pair holds half of the token tile
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr int kAccCols = NW * TN;          // one accumulator
    constexpr int kTmemCols = 2 * kAccCols;    // two of them: 256 or 512 columns
    static_assert(kTmemCols <= 512, "two accumulators must fit TMEM");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_tok[2][TN], s_pos[2][TN];
    __shared__ long long s_off[2][TN];
    __shared__ volatile int s_fail;  // set when a bounded wait of an epilogue thread expires

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* stg = reinterpret_cast<float*>(smem + (size_t)kStages * kStageBytes);  // [TN][128] fp32 output tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_iters = p.K / kBlockK;
    // Work units: tiles for a lone CTA; for a pair, units of two neighbouring feature tiles (tiles_n counts units),
    // of which this CTA keeps the one with its rank.
    const int rank = CG == 2 ? (int)cluster_cta_rank() : 0;
    const int worker = (int)blockIdx.x / CG, n_workers = (int)gridDim.x / CG;

    pdl_trigger();
    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], CG * kWideEpiWarps);  // one arrival per epilogue warp (of both CTAs of a pair)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        if (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                         "r"((uint32_t)kTmemCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                         "r"((uint32_t)kTmemCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (CG == 2) cluster_sync_all();  // the peer's barriers exist before anything is signalled across
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer
            bool ok = true;
            int it = 0;
            WIDE_CLK(p_begin);
            if (WIDE_SKIP() & 8) ok = false;
            for (int tile = worker; tile < total_tiles && ok; tile += n_workers) {
                const int tile_n = (tile % tiles_n) * CG + rank, tile_b = tile / tiles_n;
                for (int k = 0; k < k_iters; k++, it++) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    WIDE_CLK(w0);
                    ok = mbar_wait(&empty_bar[s], ph ^ 1, p.status, 111);
                    WIDE_CLK(w1);
                    WIDE_ADD(4, w1 - w0);
                    if (!ok) break;
                    uint8_t* st = smem + (size_t)s * kStageBytes;
                    if (CG == 2) {
                        // both CTAs' bytes are counted on the leader's barrier; each copies its weight rows and its
                        // half of the token tile into its own shared memory
                        if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);
                        tma_load_2d_pair(st, &map_a, k * kBlockK, tile_n * kTileM, &full_bar[s]);
                        tma_load_2d_pair(st + kABytes, &map_b, k * kBlockK, tile_b * TN + rank * kWideHalf, &full_bar[s]);
                        continue;
                    }
                    mbar_expect_tx(&full_bar[s], kStageBytes);
#pragma unroll
                    for (int w = 0; w < NW; w++) {
                        tma_load_2d(st + w * (kTileM * kBlockK * 2), &map_a, k * kBlockK, (tile_n * NW + w) * kTileM,
                                    &full_bar[s]);
                    }
                    // the activation map's box is 128 rows: one or two of them, contiguous in the stage
#pragma unroll
                    for (int hb = 0; hb < TN / kWideHalf; hb++) {
                        tma_load_2d(st + kABytes + hb * (kWideHalf * kBlockK * 2), &map_b, k * kBlockK,
                                    tile_b * TN + hb * kWideHalf, &full_bar[s]);
                    }
                }
            }
            WIDE_CLK(p_end);
            WIDE_ADD(5, p_end - p_begin);
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (of a pair: the leader's; the instruction runs on both SMs)
            constexpr uint32_t idesc = umma_idesc_bf16(kTileM * CG, TN);
            bool ok = true;
            int it = 0, lt = 0;
            WIDE_CLK(m_begin);
            for (int tile = worker; tile < total_tiles && ok; tile += n_workers, lt++) {
                const int buf = lt & 1;
                WIDE_CLK(a0);
                ok = mbar_wait(&acc_empty[buf], ((lt >> 1) & 1) ^ 1, p.status, 112);  // drained two tiles ago
                WIDE_CLK(a1);
                WIDE_ADD(0, 1);
                WIDE_ADD(1, a1 - a0);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(buf * kAccCols);
                for (int k = 0; k < k_iters; k++, it++) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    WIDE_CLK(f0);
                    const int skip = WIDE_SKIP();  // 0 in the product build
                    if (!(skip & 8)) ok = mbar_wait(&full_bar[s], ph, p.status, 113);
                    WIDE_CLK(f1);
                    WIDE_ADD(2, f1 - f0);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint8_t* st = smem + (size_t)s * kStageBytes;
                    const uint64_t bdesc = umma_desc_sw128(st + kABytes);
#pragma unroll
                    for (int w = 0; w < NW; w++) {
                        const uint64_t adesc = umma_desc_sw128(st + w * (kTileM * kBlockK * 2));
#pragma unroll
                        for (int kk = 0; kk < kBlockK / 16; kk++) {
                            if (skip & 4) continue;
                            if (CG == 2) umma_bf16_pair(acc, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k | kk) != 0 ? 1u : 0u);
                            else umma_bf16(acc + w * TN, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k | kk) != 0 ? 1u : 0u);
                        }
                    }
                    if (skip & 8) continue;
                    if (CG == 2) umma_commit_pair(&empty_bar[s]);
                    else umma_commit(&empty_bar[s]);
                }
                if (ok) {
                    if (CG == 2) umma_commit_pair(&acc_full[buf]);
                    else umma_commit(&acc_full[buf]);
                }
            }
            WIDE_CLK(m_end);
            WIDE_ADD(3, m_end - m_begin);
        }
        __syncwarp();
    } else {
        // ---- epilogue warps: TMEM lane quarter = warp index modulo 4, kWideEpiWarps / 4 warps per quarter, each
        // taking an equal share of the tile's token columns
        const int q = warp & 3;
        const int t = q * 32 + lane;
        const int hf = (warp - 2) >> 2;
        const int e = (warp - 2) * 32 + lane;  // the first 128 stage one token of the tile each
        int lt = 0;
        for (int tile = worker; tile < total_tiles; tile += n_workers, lt++) {
            const int tile_n = (tile % tiles_n) * CG + rank, tile_b = tile / tiles_n;
            const int buf = lt & 1;
            if (e < TN) {
                const int b = tile_b * TN + e;
                const int tk = b < p.B ? p.tok[b] : kSkip;
                const int ps = tk >= 0 ? p.pos[b] : 0;
                const int sq = (tk >= 0 && p.row_seq) ? p.row_seq[b] : b;
                s_tok[buf][e] = tk;
                s_pos[buf][e] = ps;
                s_off[buf][e] = (((long long)sq * p.H) * p.T + ps) * p.hs;
            }
            // publishes the staged ids to the epilogue warps (and, with the barrier at the end of the previous
            // tile, orders their reuse)
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kWideEpiWarps) : "memory");
            const WideRowCtx<EPI> cx(p, lane, tile_n);
            float4 pre[kWideRowBatch], pre2[kWideRowBatch];
            wide_rows_fetch<EPI>(p, cx, warp - 2, 0, tile_b * TN, s_tok[buf], s_pos[buf], pre);
            WIDE_CLK(e0);
            if (!mbar_wait(&acc_full[buf], (lt >> 1) & 1, p.status, 114)) s_fail = 1;
            WIDE_CLK(e1);
            // The epilogue warps only: makes the give-up decision common, so that no warp is left waiting
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kWideEpiWarps) : "memory");
            if (s_fail) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#if GRADB_DIAG
            long long t_a = 0, t_b = 0, t_bar = 0;
#endif
#pragma unroll 1
            for (int hb = 0; hb < TN / kWideHalf; hb++) {  // 128 tokens at a time through the staged tile
                WIDE_CLK(h0);
                const int skip = WIDE_SKIP();  // 0 in the product build
                const int row_base = tile_b * TN + hb * kWideHalf;
                const int* const tok_h = s_tok[buf] + hb * kWideHalf;
                const int* const pos_h = s_pos[buf] + hb * kWideHalf;
                if (hb > 0) wide_rows_fetch<EPI>(p, cx, warp - 2, 0, row_base, tok_h, pos_h, pre);
                if (!(skip & 1)) {
                    wide_epilogue_stage<EPI, NW, TN>(
                        p, tmem_base + (uint32_t)(buf * kAccCols + hb * kWideHalf) + ((uint32_t)(q * 32) << 16), t, tile_n,
                        stg, hf * (kWideHalf / (kWideEpiWarps / 4)), (hf + 1) * (kWideHalf / (kWideEpiWarps / 4)));
                }
                if (hb == TN / kWideHalf - 1) {
                    // the accumulator is drained: hand it back before the row pass
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2) mbar_arrive_leader(&acc_empty[buf]);
                        else mbar_arrive(&acc_empty[buf]);
                    }
                }
                WIDE_CLK(h1);
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kWideEpiWarps) : "memory");  // staged tile complete
                WIDE_CLK(h2);
                if (skip & 2) {
                    // (diagnostics: row pass left out)
                } else if (EPI == TC_LSE) {
                    wide_rows_lse<EPI>(p, cx, stg, warp - 2, lane, tile_n, row_base, tok_h, pos_h);
                } else {
                    // the second batch's loads are in flight while the first is written
                    static_assert(kWideRowsPerWarp == 2 * kWideRowBatch, "two batches per warp");
                    wide_rows_fetch<EPI>(p, cx, warp - 2, kWideRowBatch, row_base, tok_h, pos_h, pre2);
                    wide_rows_finish<EPI>(p, cx, stg, warp - 2, lane, 0, row_base, tok_h, s_off[buf] + hb * kWideHalf, pre);
                    wide_rows_finish<EPI>(p, cx, stg, warp - 2, lane, kWideRowBatch, row_base, tok_h,
                                          s_off[buf] + hb * kWideHalf, pre2);
                }
                WIDE_CLK(h3);
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kWideEpiWarps) : "memory");  // staged tile free again
                WIDE_CLK(h4);
#if GRADB_DIAG
                t_a += h1 - h0;
                t_b += h3 - h2;
                t_bar += (h2 - h1) + (h4 - h3);
#endif
            }
#if GRADB_DIAG
            if (warp == 2 && lane == 0) {
                WIDE_ADD(6, e1 - e0);
                WIDE_ADD(7, t_a);
                WIDE_ADD(8, t_bar);
                WIDE_ADD(9, t_b);
            }
#endif
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (CG == 2) cluster_sync_all();  // neither CTA frees tensor memory or leaves while the other may still signal it
    if (warp == 1) {
        __syncwarp();
        if (CG == 2) {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                         : "memory");
        } else {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                         : "memory");
        }
    }
}

// fp32 rows -> normalised bf16 rows (LayerNorm or RMSNorm), the tensor-core GEMMs' B operand.
// One 256-thread CTA per row (a warp-per-row variant with fewer CTAs measured slower).
// SPLIT: the fp32-mode operand instead, every value as a TF32 hi/lo pair (out32[i] and out32[lo_elems + i]).
template <bool SPLIT>
__global__ void __launch_bounds__(256) norm_rows_kernel(const float* __restrict__ X, const float* __restrict__ gamma,
                                                        const float* __restrict__ beta, const int* __restrict__ tok,
                                                        __nv_bfloat16* __restrict__ out, float* __restrict__ out32,
                                                        size_t lo_elems, int d, int rms, float eps) {
    __shared__ float sh[8];
    auto put = [&](size_t i, float v) {
        if (SPLIT) {
            float hi, lo;
            split_tf32(v, hi, lo);
            out32[i] = hi;
            out32[lo_elems + i] = lo;
        } else {
            out[i] = __float2bfloat16_rn(v);
        }
    };
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    if (tok[b] < 0) return;
    const float* xr = X + (size_t)b * d;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    auto block_sum = [&](float v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) sh[w] = v;
        __syncthreads();
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) s += sh[i];
        __syncthreads();
        return s;
    };
    float s = 0.f;
    for (int k = threadIdx.x; k < d; k += 256) {
        const float v = xr[k];
        s += rms ? v * v : v;
    }
    s = block_sum(s);
    if (rms) {
        const float r = 1.0f / sqrtf(s / (float)d + eps);
        for (int k = threadIdx.x; k < d; k += 256) put((size_t)b * d + k, gamma[k] * xr[k] * r);
    } else {
        const float mean = s / (float)d;
        float v2 = 0.f;
        for (int k = threadIdx.x; k < d; k += 256) {
            const float dl = xr[k] - mean;
            v2 += dl * dl;
        }
        v2 = block_sum(v2);
        const float inv_std = 1.0f / sqrtf(v2 / (float)d + eps);
        for (int k = threadIdx.x; k < d; k += 256) {
            put((size_t)b * d + k, gamma[k] * (xr[k] - mean) * inv_std + beta[k]);
        }
    }
}

// The same for thousands of rows (prompt feed, scoring): one warp per row, the row held in registers (read once,
// 128-bit loads, 64-bit bf16 stores), rows dealt to warps grid-stride. The row sum is formed in a different order than
// in the one-CTA-per-row kernel, so the two may differ in the last bit of a bf16 output.
constexpr int kNormWarpRows = 2048;   // rows from which this kernel is used
constexpr int kNormWarpChunks = 16;   // 128-element chunks a row may have (d <= 2048)
// SPLIT: the fp32-mode operand, every value as a TF32 hi/lo pair (out32[i] and out32[lo_elems + i]).
template <int MAXC, bool SPLIT>  // 128-element chunks held per lane: 8 (rows to 1024 elements, more warps resident) or 16
__global__ void __launch_bounds__(256) norm_rows_warp_kernel(const float* __restrict__ X, const float* __restrict__ gamma,
                                                             const float* __restrict__ beta, const int* __restrict__ tok,
                                                             __nv_bfloat16* __restrict__ out, float* __restrict__ out32,
                                                             size_t lo_elems, int d, int rms, float eps, int rows) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int chunks = d / 128;
    const float inv_d = 1.0f / (float)d;
    for (int b = blockIdx.x * 8 + (threadIdx.x >> 5); b < rows; b += gridDim.x * 8) {
        if (tok[b] < 0) continue;
        const float4* xr = reinterpret_cast<const float4*>(X + (size_t)b * d);
        float4 x[MAXC];
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < MAXC; c++) {
            if (c < chunks) {
                x[c] = xr[c * 32 + lane];
                s += rms ? (x[c].x * x[c].x + x[c].y * x[c].y) + (x[c].z * x[c].z + x[c].w * x[c].w)
                         : (x[c].x + x[c].y) + (x[c].z + x[c].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        float mean = 0.f, scale;
        if (rms) {
            scale = 1.0f / sqrtf(s * inv_d + eps);
        } else {
            mean = s * inv_d;
            float v2 = 0.f;
#pragma unroll
            for (int c = 0; c < MAXC; c++) {
                if (c < chunks) {
                    const float a = x[c].x - mean, e = x[c].y - mean, f = x[c].z - mean, g = x[c].w - mean;
                    v2 += (a * a + e * e) + (f * f + g * g);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v2 += __shfl_xor_sync(0xffffffffu, v2, o);
            scale = 1.0f / sqrtf(v2 * inv_d + eps);
        }
        uint2* orow = SPLIT ? nullptr : reinterpret_cast<uint2*>(out + (size_t)b * d);
#pragma unroll
        for (int c = 0; c < MAXC; c++) {
            if (c < chunks) {
                const float4 g = reinterpret_cast<const float4*>(gamma)[c * 32 + lane];
                float4 y;
                if (rms) {
                    y = make_float4(g.x * x[c].x * scale, g.y * x[c].y * scale, g.z * x[c].z * scale, g.w * x[c].w * scale);
                } else {
                    const float4 bt = reinterpret_cast<const float4*>(beta)[c * 32 + lane];
                    y = make_float4(g.x * (x[c].x - mean) * scale + bt.x, g.y * (x[c].y - mean) * scale + bt.y,
                                    g.z * (x[c].z - mean) * scale + bt.z, g.w * (x[c].w - mean) * scale + bt.w);
                }
                if (SPLIT) {
                    float4 h, l;
                    split_tf32(y.x, h.x, l.x);
                    split_tf32(y.y, h.y, l.y);
                    split_tf32(y.z, h.z, l.z);
                    split_tf32(y.w, h.w, l.w);
                    const size_t at = (size_t)b * d + (size_t)(c * 32 + lane) * 4;
                    *reinterpret_cast<float4*>(out32 + at) = h;
                    *reinterpret_cast<float4*>(out32 + lo_elems + at) = l;
                } else {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                    orow[c * 32 + lane] = pk;
                }
            }
        }
    }
}

// W (K, N) fp32 row-major -> W^T (N_pad, K) bf16 row-major, with a row mapping for the
// interleaved gate/up layout.
__global__ void transpose_bf16_kernel(const float* __restrict__ W, __nv_bfloat16* __restrict__ out, int K, int N,
                                      int row_offset, int interleave_tiles) {
    __shared__ float tile[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        tile[i][threadIdx.x] = (k < K && n < N) ? W[(size_t)k * N + n] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < K) {
            // interleave: feature n of this matrix lands in 128-row tile pairs [gate tile | up tile]
            const size_t row = interleave_tiles ? (size_t)(n / 128) * 256 + row_offset + (n % 128) : (size_t)row_offset + n;
            out[row * K + k] = __float2bfloat16_rn(tile[threadIdx.x][i]);
        }
    }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            ptr = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }();
    return fn;
}

constexpr size_t tc_smem_bytes(int nw, int tn, int kind) {
    return (size_t)stages_for(nw, tn, kind) * (nw * 128 * 128 + tn * 128) * (kind == 1 ? 2 : 1) + 1024;
}

template <int EPI, int NW, int TN, int KIND>
void launch_t(const CUtensorMap& a, const CUtensorMap& b, const TcGemmParams& p, dim3 grid, cudaStream_t st) {
    constexpr size_t bytes = tc_smem_bytes(NW, TN, KIND);
    auto kernel = gemm_bf16_tc_kernel<EPI, NW, TN, KIND>;
    if (!g_capturing) {
        GRADB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    launch_kernel(kernel, grid, dim3(128 * epi_warps_for(TN)), bytes, st, a, b, p);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

template <int EPI, int NW>
void launch_tn(const CUtensorMap& a, const CUtensorMap& b, const TcGemmParams& p, int tn, dim3 grid, cudaStream_t st,
               int kind) {
    if (kind == 1) {
        switch (tn) {
            case 32: launch_t<EPI, NW, 32, 1>(a, b, p, grid, st); break;
            case 64: launch_t<EPI, NW, 64, 1>(a, b, p, grid, st); break;
            case 128: launch_t<EPI, NW, 128, 1>(a, b, p, grid, st); break;
            default: throw Error(GRADB_ERR_INVALID, "unsupported token tile");
        }
        return;
    }
    switch (tn) {
        case 32: launch_t<EPI, NW, 32, 0>(a, b, p, grid, st); break;
        case 64: launch_t<EPI, NW, 64, 0>(a, b, p, grid, st); break;
        case 128: launch_t<EPI, NW, 128, 0>(a, b, p, grid, st); break;
        default: throw Error(GRADB_ERR_INVALID, "unsupported token tile");
    }
}

}  // namespace

void make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    auto fn = encode_fn();
    if (!fn) throw Error(GRADB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw Error(GRADB_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
}

void make_tensor_map_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                         bool atom32) {
    auto fn = encode_fn();
    if (!fn) throw Error(GRADB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 4};
    const cuuint32_t box[2] = {32, box_rows};  // 32 floats = one 128-byte swizzle row
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw Error(GRADB_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
}

// Largest token tile that still yields enough CTAs to occupy most of the SMs: these GEMMs
// are short, so CTA count (latency hiding across SMs) matters more than MMA width.
namespace {
template <int EPI, int NW, int TN>
void configure_one() {
    GRADB_CUDA(cudaFuncSetAttribute(gemm_bf16_tc_kernel<EPI, NW, TN, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)tc_smem_bytes(NW, TN, 0)));
    GRADB_CUDA(cudaFuncSetAttribute(gemm_bf16_tc_kernel<EPI, NW, TN, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)tc_smem_bytes(NW, TN, 1)));
}
template <int EPI, int NW>
void configure_tiles() {
    configure_one<EPI, NW, 32>();
    configure_one<EPI, NW, 64>();
    configure_one<EPI, NW, 128>();
}
}  // namespace

// Opt every GEMM variant into its dynamic shared memory up front (per device), so that no
// attribute call is needed later, in particular not while a stream is being captured.
void tc_configure_all() {
    configure_tiles<TC_QKV, 1>();
    configure_tiles<TC_RESID, 1>();
    configure_tiles<TC_GELU, 1>();
    configure_tiles<TC_SWIGLU, 2>();
    configure_tiles<TC_LOGITS, 1>();
}

int tc_token_tile(int n_seq, int n_tiles, int want_ctas) {
#if GRADB_DIAG
    if (const char* force = std::getenv("GRADB_TC_TILE")) {  // diagnostics build: 32, 64 or 128
        const int tn = std::atoi(force);
        if (tn == 32 || tn == 64 || tn == 128) return tn;
    }
#endif
    for (int tn : {128, 64, 32}) {
        if (tn > 32 && tn >= 2 * n_seq) continue;  // do not pad a small batch to a wide tile
        if (n_tiles * ((n_seq + tn - 1) / tn) >= want_ctas || tn == 32) return tn;
    }
    return 32;
}

namespace {
template <int EPI, int NW, int TN>
void launch_wide(const CUtensorMap& a, const CUtensorMap& b, const TcGemmParams& p, int tiles_n, int sm_count,
                 cudaStream_t st) {
    constexpr size_t bytes = wide_smem_bytes(NW, TN);
    auto kernel = gemm_bf16_tc_wide_kernel<EPI, NW, TN>;
    if (!g_capturing) {
        GRADB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    const int total = tiles_n * ((p.B + TN - 1) / TN);
    launch_kernel(kernel, dim3(std::min(total, sm_count)), dim3(kWideThreads), bytes, st, a, b, p, tiles_n, total);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

// CTA pairs: a cluster of two per work unit (two neighbouring feature tiles x 256 tokens).
template <int EPI>
void launch_wide_pair(const CUtensorMap& a, const CUtensorMap& b, const TcGemmParams& p, int tiles_n, int sm_count,
                      cudaStream_t st) {
    constexpr size_t bytes = wide_smem_bytes(1, 256, 2);
    auto kernel = gemm_bf16_tc_wide_kernel<EPI, 1, 256, 2>;
    if (!g_capturing) {
        GRADB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    const int units_n = (tiles_n + 1) / 2;
    const int total = units_n * ((p.B + 255) / 256);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (sm_count / 2));
    cfg.blockDim = dim3(kWideThreads);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // Clusters that can be resident together (not every pair of SMs forms one): a persistent grid must not be larger,
    // or the clusters left over would run their statically dealt units in a second round.
    static int resident = 0;
    if (!resident) {
        int n = 0;
        GRADB_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        resident = std::max(1, std::min(n, sm_count / 2));
    }
    cfg.gridDim = dim3(2 * std::min(total, resident));
    cfg.numAttrs = g_pdl ? 2 : 1;
    GRADB_CUDA(cudaLaunchKernelEx(&cfg, kernel, a, b, p, units_n, total));
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

// 256-token tiles once they still leave every SM four tiles or more, as CTA pairs unless GRADB_WIDE_PAIRS=0
// (GRADB_WIDE_TN=128 keeps the narrow tile).
template <int EPI>
void launch_wide_single(const CUtensorMap& a, const CUtensorMap& b, const TcGemmParams& p, int tiles_n, int sm_count,
                        cudaStream_t st) {
    static const bool narrow = [] {
        const char* e = std::getenv("GRADB_WIDE_TN");
        return e && std::atoi(e) == 128;
    }();
    static const bool pairs = [] {
        const char* e = std::getenv("GRADB_WIDE_PAIRS");
        return !(e && e[0] == '0');
    }();
    if (!narrow && tiles_n * ((p.B + 255) / 256) >= 4 * sm_count) {
        if (pairs) launch_wide_pair<EPI>(a, b, p, tiles_n, sm_count, st);
        else launch_wide<EPI, 1, 256>(a, b, p, tiles_n, sm_count, st);
    } else {
        launch_wide<EPI, 1, 128>(a, b, p, tiles_n, sm_count, st);
    }
}
}  // namespace

bool tc_many_rows(const TcGemmParams& p, int token_tile) {
    if (token_tile != kWideTN) return false;
    int dev = 0, sm_count = 0;
    GRADB_CUDA(cudaGetDevice(&dev));
    GRADB_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    const char* off = std::getenv("GRADB_NO_WIDE_GEMM");
    if (off && off[0] == '1') return false;
    const int n_tiles = (p.N + kTileM - 1) / kTileM, tiles_b = (p.B + kWideTN - 1) / kWideTN;
    return p.N % 4 == 0 && n_tiles * tiles_b >= 2 * sm_count;
}

#if GRADB_DIAG
void wide_clocks_read(unsigned long long* out128, bool reset) {
    GRADB_CUDA(cudaDeviceSynchronize());
    if (const char* e = std::getenv("GRADB_DIAG_WIDE_SKIP")) {
        const int v = std::atoi(e);
        GRADB_CUDA(cudaMemcpyToSymbol(g_wide_skip, &v, sizeof(int)));
    }
    GRADB_CUDA(cudaMemcpyFromSymbol(out128, g_wide_clock, sizeof(unsigned long long) * 128));
    if (reset) {
        unsigned long long zero[128] = {};
        GRADB_CUDA(cudaMemcpyToSymbol(g_wide_clock, zero, sizeof(zero)));
    }
}
#endif

void launch_tc_gemm(int epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const TcGemmParams& p, int token_tile,
                    int k_splits, cudaStream_t st, int kind) {
    const int n_tiles = (p.N + kTileM - 1) / kTileM;
    if (token_tile == kWideTN && k_splits == 1 && kind == 0) {
        // Many tiles per SM: the persistent kernel (the one-tile-per-CTA kernel is for the short decode GEMMs).
        static int sm_count = 0;
        if (!sm_count) {
            int dev = 0;
            GRADB_CUDA(cudaGetDevice(&dev));
            GRADB_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
        }
        const char* off = std::getenv("GRADB_NO_WIDE_GEMM");
        const bool wide_off = off && off[0] == '1';
        const int tiles_b = (p.B + kWideTN - 1) / kWideTN;
        // the row-wise epilogue works on four features per lane and on tiles that lie inside one of Q, K, V
        const bool shape_ok = p.N % 4 == 0 && (p.ld_out % 4 == 0 || epi == TC_LSE) &&
                              (epi != TC_QKV || (p.d % kTileM == 0 && p.hs % 4 == 0));
        if (!wide_off && shape_ok && n_tiles * tiles_b >= 2 * sm_count) {
            switch (epi) {
                case TC_QKV: launch_wide_single<TC_QKV>(map_a, map_b, p, n_tiles, sm_count, st); return;
                case TC_RESID: launch_wide_single<TC_RESID>(map_a, map_b, p, n_tiles, sm_count, st); return;
                case TC_GELU: launch_wide_single<TC_GELU>(map_a, map_b, p, n_tiles, sm_count, st); return;
                case TC_SWIGLU: launch_wide<TC_SWIGLU, 2, 128>(map_a, map_b, p, n_tiles, sm_count, st); return;
                case TC_LOGITS: launch_wide_single<TC_LOGITS>(map_a, map_b, p, n_tiles, sm_count, st); return;
                case TC_LSE: launch_wide_single<TC_LSE>(map_a, map_b, p, n_tiles, sm_count, st); return;
                default: break;
            }
        }
    }
    const dim3 grid(n_tiles, (p.B + token_tile - 1) / token_tile, k_splits);
    switch (epi) {
        case TC_QKV: launch_tn<TC_QKV, 1>(map_a, map_b, p, token_tile, grid, st, kind); break;
        case TC_RESID: launch_tn<TC_RESID, 1>(map_a, map_b, p, token_tile, grid, st, kind); break;
        case TC_GELU: launch_tn<TC_GELU, 1>(map_a, map_b, p, token_tile, grid, st, kind); break;
        case TC_SWIGLU: launch_tn<TC_SWIGLU, 2>(map_a, map_b, p, token_tile, grid, st, kind); break;
        case TC_LOGITS: launch_tn<TC_LOGITS, 1>(map_a, map_b, p, token_tile, grid, st, kind); break;
        default: throw Error(GRADB_ERR_INVALID, "this epilogue has no one-tile-per-CTA kernel");
    }
}

namespace {
// The warp-per-row kernel from kNormWarpRows rows on, the one-CTA-per-row kernel below that (and for row lengths
// that are not a multiple of 128 or exceed 2048).
template <bool SPLIT>
void launch_norm_any(const float* X, const float* gamma, const float* beta, const int* tok, __nv_bfloat16* out16,
                     float* out32, size_t lo_elems, int d, int rms, float eps, int B, cudaStream_t st) {
    if (B >= kNormWarpRows && d % 128 == 0 && d <= 128 * kNormWarpChunks) {
        const dim3 grid(std::min((B + 7) / 8, 148 * 8));
        if (d <= 1024) {
            launch_kernel(norm_rows_warp_kernel<8, SPLIT>, grid, dim3(256), 0, st, X, gamma, beta, tok, out16, out32, lo_elems,
                          d, rms, eps, B);
        } else {
            launch_kernel(norm_rows_warp_kernel<16, SPLIT>, grid, dim3(256), 0, st, X, gamma, beta, tok, out16, out32, lo_elems,
                          d, rms, eps, B);
        }
    } else {
        launch_kernel(norm_rows_kernel<SPLIT>, dim3(B), dim3(256), 0, st, X, gamma, beta, tok, out16, out32, lo_elems, d, rms,
                      eps);
    }
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}
}  // namespace

void launch_norm_bf16(const float* X, const float* gamma, const float* beta, const int* tok, __nv_bfloat16* out, int d,
                      int rms, float eps, int B, cudaStream_t st) {
    launch_norm_any<false>(X, gamma, beta, tok, out, nullptr, 0, d, rms, eps, B, st);
}

void launch_norm_split(const float* X, const float* gamma, const float* beta, const int* tok, float* out, size_t lo_elems,
                       int d, int rms, float eps, int B, cudaStream_t st) {
    launch_norm_any<true>(X, gamma, beta, tok, nullptr, out, lo_elems, d, rms, eps, B, st);
}

namespace {
__global__ void split_tf32_kernel(const float* __restrict__ in, float* __restrict__ out, size_t lo_elems, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float hi, lo;
    split_tf32(in[i], hi, lo);
    out[i] = hi;
    out[lo_elems + i] = lo;
}

// W (K, N) fp32 row-major -> W^T (rows, K) fp32 as a TF32 hi/lo pair, same row mapping as transpose_bf16_kernel.
__global__ void transpose_split_kernel(const float* __restrict__ W, float* __restrict__ out, size_t lo_elems, int K, int N,
                                       int row_offset, int interleave_tiles) {
    __shared__ float tile[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        tile[i][threadIdx.x] = (k < K && n < N) ? W[(size_t)k * N + n] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < K) {
            const size_t row = interleave_tiles ? (size_t)(n / 128) * 256 + row_offset + (n % 128) : (size_t)row_offset + n;
            float hi, lo;
            split_tf32(tile[threadIdx.x][i], hi, lo);
            out[row * K + k] = hi;
            out[lo_elems + row * K + k] = lo;
        }
    }
}
}  // namespace

void launch_split_tf32(const float* in, float* out, size_t lo_elems, size_t n, cudaStream_t st) {
    if (!n) return;
    launch_kernel(split_tf32_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, in, out, lo_elems, n);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

void launch_transpose_split(const float* W, float* out, size_t lo_elems, int K, int N, int row_offset, bool interleave,
                            cudaStream_t st) {
    const dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
    transpose_split_kernel<<<grid, block, 0, st>>>(W, out, lo_elems, K, N, row_offset, interleave ? 1 : 0);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

void launch_transpose_bf16(const float* W, __nv_bfloat16* out, int K, int N, int row_offset, bool interleave,
                           cudaStream_t st) {
    const dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
    transpose_bf16_kernel<<<grid, block, 0, st>>>(W, out, K, N, row_offset, interleave ? 1 : 0);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

}  // namespace gradb
