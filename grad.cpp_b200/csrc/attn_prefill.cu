// Causal attention for the batched prompt feed and for scoring, head size 64: many consecutive
// positions of one sequence are queries at once, so a tile of 64 queries shares every K/V tile it
// reads instead of each position streaming the whole prefix on its own (which is what the decode
// kernel does and what made long prompts cost O(len^2) cache reads).
//
// Same arithmetic as the reference's cached attention (src/transformer/inference.cpp:208-225 with
// softmax_row :60-67): s[t] = q . K[t] / sqrt(64) over t <= position, softmax, out = sum s[t] V[t],
// evaluated flash-style (running maximum and sum, rescaled accumulator). Products run on the tensor
// cores in TF32 with fp32 accumulation (mma.sync m16n8k8). The plain variant (one MMA per product) is within
// the error budget of the bf16-weight mode; the X3 variant, used by fp32 sessions, splits every operand into a
// TF32-rounded value and its TF32-rounded remainder and issues three MMAs per product (lo*hi + hi*lo + hi*hi),
// which carries fp32-grade accuracy through both products.
//
// One CTA = one (query tile, head): 4 warps x 16 queries. K and V tiles of 64 positions are
// contiguous in the head-major cache and are staged in shared memory by cp.async, double buffered,
// rows padded to 68 floats so that both fragment read patterns are free of bank conflicts.
#include "attn_prefill.cuh"

namespace gradb {
namespace {

constexpr int kQ = 64;        // queries per CTA
constexpr int kK = 64;        // positions per K/V tile
constexpr int kLd = 68;       // padded row length in shared memory (floats)
constexpr int kTileFloats = kK * kLd;
constexpr int kStageFloats = 2 * kTileFloats;  // K tile + V tile
constexpr int kStages = 2;

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16-byte asynchronous copy; bytes = 0 writes zeros (rows past the last needed position).
__device__ __forceinline__ void cp_async16(float* dst, const float* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Stage one K tile and one V tile (positions [k0, k0 + 64) of one head) into shared memory.
__device__ __forceinline__ void load_tiles(float* stage, const float* kbase, const float* vbase, int k0, int kmax) {
    for (int c = threadIdx.x; c < kK * 16; c += 128) {
        const int row = c >> 4, col = (c & 15) << 2;
        const int key = k0 + row;
        const int bytes = key < kmax ? 16 : 0;
        const size_t off = (size_t)(key < kmax ? key : 0) * 64 + col;
        cp_async16(stage + row * kLd + col, kbase + off, bytes);
        cp_async16(stage + kTileFloats + row * kLd + col, vbase + off, bytes);
    }
}

__device__ __forceinline__ void split2(float x, uint32_t& hi, uint32_t& lo) {
    hi = to_tf32(x);
    lo = to_tf32(x - __uint_as_float(hi));
}

template <bool X3>
__global__ void __launch_bounds__(128) attn_prefill64_kernel(const PrefillAttnParams p) {
    extern __shared__ __align__(16) float smem[];
    pdl_wait();
    const int4 tile = p.tiles[blockIdx.x];  // sequence, first row, first position, queries
    const int seq = tile.x, row0 = tile.y, pos0 = tile.z, nq = tile.w;
    const int h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const float* kbase = p.kcache + ((size_t)seq * p.H + h) * p.T * 64;
    const float* vbase = p.vcache + ((size_t)seq * p.H + h) * p.T * 64;
    const int kmax = pos0 + nq;  // positions 0 .. kmax-1 are visible to the last query of the tile
    const int n_tiles = (kmax + kK - 1) / kK;

    load_tiles(smem, kbase, vbase, 0, kmax);
    cp_async_commit();

    // This warp's 16 queries as A fragments (rows g and g+8 of the warp's block), scaled, in TF32.
    const int q_lo = warp * 16 + g, q_hi = q_lo + 8;
    uint32_t qa[8][4], ql[X3 ? 8 : 1][4];
    {
        const float* qr_lo = p.q + (size_t)(row0 + q_lo) * p.d + h * 64;
        const float* qr_hi = p.q + (size_t)(row0 + q_hi) * p.d + h * 64;
        const bool ok_lo = q_lo < nq, ok_hi = q_hi < nq;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const float q0 = ok_lo ? qr_lo[ks * 8 + t] * p.scale : 0.f, q1 = ok_hi ? qr_hi[ks * 8 + t] * p.scale : 0.f;
            const float q2 = ok_lo ? qr_lo[ks * 8 + t + 4] * p.scale : 0.f, q3 = ok_hi ? qr_hi[ks * 8 + t + 4] * p.scale : 0.f;
            if constexpr (X3) {
                split2(q0, qa[ks][0], ql[ks][0]);
                split2(q1, qa[ks][1], ql[ks][1]);
                split2(q2, qa[ks][2], ql[ks][2]);
                split2(q3, qa[ks][3], ql[ks][3]);
            } else {
                qa[ks][0] = to_tf32(q0);
                qa[ks][1] = to_tf32(q1);
                qa[ks][2] = to_tf32(q2);
                qa[ks][3] = to_tf32(q3);
            }
        }
    }
    const int qpos_lo = pos0 + q_lo, qpos_hi = pos0 + q_hi;
    const int warp_last = pos0 + warp * 16 + 15;  // newest position any query of this warp sees

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int kt = 0; kt < n_tiles; kt++) {
        float* stage = smem + (kt & 1) * kStageFloats;
        if (kt + 1 < n_tiles) {
            load_tiles(smem + ((kt + 1) & 1) * kStageFloats, kbase, vbase, (kt + 1) * kK, kmax);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int k0 = kt * kK;
        if (k0 <= warp_last) {
            const float* Ks = stage;
            const float* Vs = stage + kTileFloats;
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
                    const float* kr = Ks + (nt * 8 + g) * kLd + ks * 8 + t;
                    if constexpr (X3) {
                        uint32_t h0, l0, h1, l1;
                        split2(kr[0], h0, l0);
                        split2(kr[4], h1, l1);
                        mma_tf32(s[nt], ql[ks], h0, h1);
                        mma_tf32(s[nt], qa[ks], l0, l1);
                        mma_tf32(s[nt], qa[ks], h0, h1);
                    } else {
                        mma_tf32(s[nt], qa[ks], __float_as_uint(kr[0]), __float_as_uint(kr[4]));
                    }
                }
            }
            // causal mask: position k0 + nt*8 + 2t (+1) against the query's own position
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const int key = k0 + nt * 8 + 2 * t;
                if (key > qpos_lo) s[nt][0] = -INFINITY;
                if (key + 1 > qpos_lo) s[nt][1] = -INFINITY;
                if (key > qpos_hi) s[nt][2] = -INFINITY;
                if (key + 1 > qpos_hi) s[nt][3] = -INFINITY;
                mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            // position 0 is visible to every query, so after the first tile the maxima are finite
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float c_lo = m_lo == -INFINITY ? 0.f : expf(m_lo - mn_lo);
            const float c_hi = m_hi == -INFINITY ? 0.f : expf(m_hi - mn_hi);
            m_lo = mn_lo;
            m_hi = mn_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                s[nt][0] = expf(s[nt][0] - mn_lo);
                s[nt][1] = expf(s[nt][1] - mn_lo);
                s[nt][2] = expf(s[nt][2] - mn_hi);
                s[nt][3] = expf(s[nt][3] - mn_hi);
                sum_lo += s[nt][0] + s[nt][1];
                sum_hi += s[nt][2] + s[nt][3];
            }
            l_lo = l_lo * c_lo + sum_lo;  // per-lane partial sums; the quad is added up at the end
            l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                o[nt][0] *= c_lo;
                o[nt][1] *= c_lo;
                o[nt][2] *= c_hi;
                o[nt][3] *= c_hi;
            }
            // out += P V. The score fragment of key group ks holds columns (2t, 2t+1) of rows (g, g+8); read as
            // an A fragment its k index t stands for key 2t and t+4 for key 2t+1, so V rows are fetched to match.
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                uint32_t pa[4], pl[4];
                if constexpr (X3) {
                    split2(s[ks][0], pa[0], pl[0]);
                    split2(s[ks][2], pa[1], pl[1]);
                    split2(s[ks][1], pa[2], pl[2]);
                    split2(s[ks][3], pa[3], pl[3]);
                } else {
                    pa[0] = to_tf32(s[ks][0]);
                    pa[1] = to_tf32(s[ks][2]);
                    pa[2] = to_tf32(s[ks][1]);
                    pa[3] = to_tf32(s[ks][3]);
                }
                const float* v0 = Vs + (ks * 8 + 2 * t) * kLd + g;
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
                    if constexpr (X3) {
                        uint32_t h0, l0, h1, l1;
                        split2(v0[nt * 8], h0, l0);
                        split2(v0[kLd + nt * 8], h1, l1);
                        mma_tf32(o[nt], pl, h0, h1);
                        mma_tf32(o[nt], pa, l0, l1);
                        mma_tf32(o[nt], pa, h0, h1);
                    } else {
                        mma_tf32(o[nt], pa, __float_as_uint(v0[nt * 8]), __float_as_uint(v0[kLd + nt * 8]));
                    }
                }
            }
        }
        __syncthreads();  // the stage is refilled two iterations from now
    }

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        const int col = h * 64 + nt * 8 + 2 * t;
        if (q_lo < nq) {
            const size_t at = (size_t)(row0 + q_lo) * p.d + col;
            const float a = o[nt][0] * inv_lo, b = o[nt][1] * inv_lo;
            if (p.out) *reinterpret_cast<float2*>(p.out + at) = make_float2(a, b);
            if (p.out16) *reinterpret_cast<__nv_bfloat162*>(p.out16 + at) = __floats2bfloat162_rn(a, b);
        }
        if (q_hi < nq) {
            const size_t at = (size_t)(row0 + q_hi) * p.d + col;
            const float a = o[nt][2] * inv_hi, b = o[nt][3] * inv_hi;
            if (p.out) *reinterpret_cast<float2*>(p.out + at) = make_float2(a, b);
            if (p.out16) *reinterpret_cast<__nv_bfloat162*>(p.out16 + at) = __floats2bfloat162_rn(a, b);
        }
    }
}

}  // namespace

size_t prefill_attention_smem_bytes() { return (size_t)kStages * kStageFloats * sizeof(float); }

void prefill_attention_configure() {
    GRADB_CUDA(cudaFuncSetAttribute(attn_prefill64_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)prefill_attention_smem_bytes()));
    GRADB_CUDA(cudaFuncSetAttribute(attn_prefill64_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)prefill_attention_smem_bytes()));
}

void launch_prefill_attention(const PrefillAttnParams& p, cudaStream_t st, bool fp32_grade) {
    if (p.n_tiles <= 0) return;
    if (fp32_grade) {
        launch_kernel(attn_prefill64_kernel<true>, dim3(p.n_tiles, p.H), dim3(128), prefill_attention_smem_bytes(), st, p);
    } else {
        launch_kernel(attn_prefill64_kernel<false>, dim3(p.n_tiles, p.H), dim3(128), prefill_attention_smem_bytes(), st, p);
    }
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

}  // namespace gradb
