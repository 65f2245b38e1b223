// Kernels of one decode step (InferenceSession::step, src/transformer/inference.cpp:150-258)
// for a batch of independent sequences.
//
// All of them are bandwidth-bound streaming kernels:
//   embed        x = E[token] (+ P[pos])                                  inference.cpp:159-182
//   fused_gemv   y = epilogue(norm(x) @ W + b), W (in,out) row-major      inference.cpp:14-58, 193-199, 228-247
//                  - thread-block clusters split the reduction dimension; partial sums meet in
//                    distributed shared memory in a fixed order (deterministic results)
//   attn_decode  softmax(q K^T / sqrt(hs)) V over the cached positions     inference.cpp:208-225
//                  - split along the context with a ticket-elected combiner
//   logits       final norm + h @ E^T                                     inference.cpp:251-254
#include <cooperative_groups.h>

#include <mutex>

#include "step_kernels.cuh"

namespace cg = cooperative_groups;

namespace gradb {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTileN = 128;  // columns per CTA: 32 lanes x 4

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sums v[m] over the block; every thread gets the totals. Partial sums are
// combined in warp order, so the result does not depend on scheduling.
template <int MB>
__device__ __forceinline__ void block_sum(float (&v)[MB], float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int m = 0; m < MB; m++) {
        v[m] = warp_sum(v[m]);
        if (lane == 0) sh[w * MB + m] = v[m];
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MB; m++) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kWarps; i++) s += sh[i * MB + m];
        v[m] = s;
    }
    __syncthreads();
}

__device__ __forceinline__ float4 load_w4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load_w4(const __nv_bfloat16* p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}

// ------------------------------------------------------------------ embed

__global__ void embed_kernel(const float* __restrict__ E, const float* __restrict__ P, const int* __restrict__ tok,
                             const int* __restrict__ pos, float* __restrict__ x, int d) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int t = tok[b];
    if (t < 0) return;
    const float4* e = reinterpret_cast<const float4*>(E + (size_t)t * d);
    const float4* p = P ? reinterpret_cast<const float4*>(P + (size_t)pos[b] * d) : nullptr;
    float4* o = reinterpret_cast<float4*>(x + (size_t)b * d);
    for (int j = threadIdx.x; j < d / 4; j += blockDim.x) {
        float4 v = __ldg(e + j);
        // The reference multiplies by the embedding scale 1.0 first (token_embedding.h:12): a no-op in fp32.
        if (p) {
            const float4 q = __ldg(p + j);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        }
        o[j] = v;
    }
}

// End of a step: positions move on; optionally the fed ids join the history the
// repetition penalty reads.
__global__ void advance_kernel(const int* __restrict__ tok, int* __restrict__ pos, int* __restrict__ hist,
                               int* __restrict__ hist_len, int hist_stride, int B) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B || tok[b] < 0) return;
    pos[b] += 1;
    if (hist) {
        const int n = hist_len[b];
        if (n < hist_stride) hist[(size_t)b * hist_stride + n] = tok[b];
        hist_len[b] = n + 1;
    }
}

// Prompt feed with one row per prompt token: copy each sequence's last row into the per-sequence
// residual buffer (the logits are only needed there).
__global__ void gather_last_rows_kernel(const float* __restrict__ rows, const int* __restrict__ row_last,
                                        const int* __restrict__ row_seq, float* __restrict__ x_seq, int d) {
    const int r = blockIdx.x;
    if (row_last[r] < 0) return;
    const float4* src = reinterpret_cast<const float4*>(rows + (size_t)r * d);
    float4* dst = reinterpret_cast<float4*>(x_seq + (size_t)row_seq[r] * d);
    for (int j = threadIdx.x; j < d / 4; j += blockDim.x) dst[j] = src[j];
}

// Prompt feed bookkeeping, rows: the fed ids join their sequence's history.
__global__ void feed_history_kernel(const int* __restrict__ row_tok, const int* __restrict__ row_pos,
                                    const int* __restrict__ row_seq, const int* __restrict__ pos,
                                    const int* __restrict__ hist_len, int* __restrict__ hist, int hist_stride, int R) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int s = row_seq[r];
    const int idx = hist_len[s] + (row_pos[r] - pos[s]);
    if (idx >= 0 && idx < hist_stride) hist[(size_t)s * hist_stride + idx] = row_tok[r];
}
// Prompt feed bookkeeping, sequences: positions and history lengths move on by the ids fed.
__global__ void feed_advance_kernel(const int* __restrict__ seq_count, int* __restrict__ pos, int* __restrict__ hist_len,
                                    int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    pos[b] += seq_count[b];
    hist_len[b] += seq_count[b];
}

// ------------------------------------------------------------- fused gemv

// Shared-memory layout (floats): xs[MB][Kc] | xfull[K] (norm prologue only) | red[kWarps][NW][MB][128]
//                                | part[NW][MB][128] | sh[kWarps*MB]
template <int MB, typename WT, int PRO, int EPI, int NW>
__global__ void __launch_bounds__(kThreads) fused_gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) float smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int KS = (int)cluster.dim_blocks().y;
    const int kr = (int)cluster.block_index().y;
    const int Kc = p.K / KS, k0 = kr * Kc;

    float* xs = smem;
    float* xfull = xs + MB * Kc;
    float* red = xfull + (PRO != PRO_NONE ? p.K : 0);
    float* part = red + kWarps * NW * MB * kTileN;
    float* sh = part + NW * MB * kTileN;

    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int row0 = blockIdx.z * MB;
    const int tile = blockIdx.x;
    int which = 0, n0 = tile * kTileN;
    if (EPI == EPI_QKV) {
        const int tiles_per = (p.N + kTileN - 1) / kTileN;
        which = tile / tiles_per;
        n0 = (tile % tiles_per) * kTileN;
    }

    // ---- prologue: stage (normalised) input rows in shared memory
    bool live[MB];
#pragma unroll
    for (int m = 0; m < MB; m++) live[m] = (row0 + m < p.B) && (p.tok[row0 + m] >= 0);

    if (PRO == PRO_NONE) {
#pragma unroll
        for (int m = 0; m < MB; m++) {
            const float* xr = p.X + (size_t)(row0 + m) * p.ldx + k0;
            for (int k = threadIdx.x; k < Kc; k += kThreads) xs[m * Kc + k] = live[m] ? xr[k] : 0.f;
        }
    } else {
        for (int m = 0; m < MB; m++) {
            if (!live[m]) {  // uniform across the block
                for (int k = threadIdx.x; k < Kc; k += kThreads) xs[m * Kc + k] = 0.f;
                continue;
            }
            const float* xr = p.X + (size_t)(row0 + m) * p.ldx;
            float s[1] = {0.f};
            for (int k = threadIdx.x; k < p.K; k += kThreads) {
                const float v = xr[k];
                xfull[k] = v;
                s[0] += (PRO == PRO_RMSNORM) ? v * v : v;
            }
            block_sum<1>(s, sh);
            if (PRO == PRO_RMSNORM) {
                // inference.cpp:33-41
                const float r = 1.0f / sqrtf(s[0] / (float)p.K + p.eps);
                for (int k = threadIdx.x; k < Kc; k += kThreads) xs[m * Kc + k] = p.gamma[k0 + k] * xfull[k0 + k] * r;
            } else {
                // inference.cpp:44-57: mean, then the variance of the centred values
                const float mean = s[0] / (float)p.K;
                float v2[1] = {0.f};
                for (int k = threadIdx.x; k < p.K; k += kThreads) {
                    const float dlt = xfull[k] - mean;
                    v2[0] += dlt * dlt;
                }
                block_sum<1>(v2, sh);
                const float inv_std = 1.0f / sqrtf(v2[0] / (float)p.K + p.eps);
                for (int k = threadIdx.x; k < Kc; k += kThreads) {
                    xs[m * Kc + k] = p.gamma[k0 + k] * (xfull[k0 + k] - mean) * inv_std + p.beta[k0 + k];
                }
            }
            __syncthreads();
        }
    }
    __syncthreads();

    // ---- main loop: each warp streams rows k0 + 4*(w + 8i) .. +3 of its 128-column tile
    float acc[NW][MB][4];
#pragma unroll
    for (int a = 0; a < NW; a++)
#pragma unroll
        for (int m = 0; m < MB; m++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[a][m][c] = 0.f;

    const int col = n0 + lane * 4;
    if (col < p.N) {
        const WT* Wp[NW];
#pragma unroll
        for (int a = 0; a < NW; a++) {
            const WT* base = static_cast<const WT*>(p.W[EPI == EPI_QKV ? which : a]);
            Wp[a] = base + (size_t)k0 * p.N + col;
        }
        const int groups = Kc / 4;
#pragma unroll 2
        for (int g = w; g < groups; g += kWarps) {
            const int k = 4 * g;
            float4 wv[NW][4];
#pragma unroll
            for (int a = 0; a < NW; a++)
#pragma unroll
                for (int r = 0; r < 4; r++) wv[a][r] = load_w4(Wp[a] + (size_t)(k + r) * p.N);
#pragma unroll
            for (int m = 0; m < MB; m++) {
                const float4 xv = *reinterpret_cast<const float4*>(&xs[m * Kc + k]);
#pragma unroll
                for (int a = 0; a < NW; a++) {
                    acc[a][m][0] += xv.x * wv[a][0].x + xv.y * wv[a][1].x + xv.z * wv[a][2].x + xv.w * wv[a][3].x;
                    acc[a][m][1] += xv.x * wv[a][0].y + xv.y * wv[a][1].y + xv.z * wv[a][2].y + xv.w * wv[a][3].y;
                    acc[a][m][2] += xv.x * wv[a][0].z + xv.y * wv[a][1].z + xv.z * wv[a][2].z + xv.w * wv[a][3].z;
                    acc[a][m][3] += xv.x * wv[a][0].w + xv.y * wv[a][1].w + xv.z * wv[a][2].w + xv.w * wv[a][3].w;
                }
            }
        }
    }

    // ---- reduce over the block's warps, then over the cluster's K slices
#pragma unroll
    for (int a = 0; a < NW; a++)
#pragma unroll
        for (int m = 0; m < MB; m++) {
            *reinterpret_cast<float4*>(&red[((w * NW + a) * MB + m) * kTileN + lane * 4]) =
                make_float4(acc[a][m][0], acc[a][m][1], acc[a][m][2], acc[a][m][3]);
        }
    __syncthreads();
    for (int i = threadIdx.x; i < NW * MB * kTileN; i += kThreads) {
        float s = 0.f;
#pragma unroll
        for (int ww = 0; ww < kWarps; ww++) s += red[ww * NW * MB * kTileN + i];
        part[i] = s;
    }
    cluster.sync();

    // Each CTA of the cluster finishes a 128/KS-column slice of the tile.
    const int cslice = kTileN / KS;
    const int pairs = cslice / 2;
    for (int i = threadIdx.x; i < MB * pairs; i += kThreads) {
        const int m = i / pairs, c = kr * cslice + (i % pairs) * 2;
        const int b = row0 + m, n = n0 + c;
        float v[NW][2];
#pragma unroll
        for (int a = 0; a < NW; a++) v[a][0] = v[a][1] = 0.f;
        for (int r = 0; r < KS; r++) {
            const float* rp = cluster.map_shared_rank(part, r);
#pragma unroll
            for (int a = 0; a < NW; a++) {
                const float2 t = *reinterpret_cast<const float2*>(&rp[(a * MB + m) * kTileN + c]);
                v[a][0] += t.x;
                v[a][1] += t.y;
            }
        }
        if (n >= p.N || !live[m]) continue;
        if (EPI == EPI_RESID) {
            // x += h @ W + b (inference.cpp:22-28)
            float* y = p.Y + (size_t)b * p.ldy + n;
            const float b0 = p.bias[0] ? p.bias[0][n] : 0.f, b1 = p.bias[0] ? p.bias[0][n + 1] : 0.f;
            y[0] += v[0][0] + b0;
            y[1] += v[0][1] + b1;
        } else if (EPI == EPI_GELU) {
            // inference.cpp:69-80
            float* y = p.Y + (size_t)b * p.ldy + n;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float t = v[0][e] + p.bias[0][n + e];
                const float u = 0.79788456f * (t + 0.044715f * t * t * t);
                y[e] = 0.5f * t * (1.0f + tanhf(u));
            }
        } else if (EPI == EPI_SWIGLU) {
            // silu(gate) * up (inference.cpp:82-91, 234-239)
            float* y = p.Y + (size_t)b * p.ldy + n;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float g = v[0][e];
                const float sg = g / (1.0f + expf(-g));
                y[e] = v[1][e] * sg;
            }
        } else {  // EPI_QKV
            float a0 = v[0][0] + p.bias[which][n], a1 = v[0][1] + p.bias[which][n + 1];
            const int position = p.pos[b];
            const int h = n / p.hs, c_in = n % p.hs;
            if (p.rope_cos && which < 2) {
                // inference.cpp:101-115: pairs (2j, 2j+1) inside each head
                const float cs = p.rope_cos[(size_t)position * (p.hs / 2) + c_in / 2];
                const float sn = p.rope_sin[(size_t)position * (p.hs / 2) + c_in / 2];
                const float r0 = a0 * cs - a1 * sn, r1 = a0 * sn + a1 * cs;
                a0 = r0;
                a1 = r1;
            }
            if (which == 0) {
                *reinterpret_cast<float2*>(p.Y + (size_t)b * p.ldy + n) = make_float2(a0, a1);
            } else {
                float* cache = which == 1 ? p.kcache : p.vcache;
                const size_t off = (((size_t)b * p.H + h) * p.T + position) * p.hs + c_in;
                *reinterpret_cast<float2*>(cache + off) = make_float2(a0, a1);
            }
        }
    }
    cluster.sync();
}

// ----------------------------------------------------------------- logits

// One warp per vocabulary row: lanes stride the row in float4, then a shuffle
// reduction. E is (vocab, d) row-major, used transposed (inference.cpp:254).
template <int MB, typename WT>
__global__ void __launch_bounds__(kThreads) logits_kernel(const LogitsParams p) {
    extern __shared__ __align__(16) float smem[];
    float* hs_ = smem;                 // [MB][d] normalised rows
    float* sh = hs_ + MB * p.d;        // reduction scratch
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int row0 = blockIdx.y * MB;
    bool live[MB];
    bool any = false;
#pragma unroll
    for (int m = 0; m < MB; m++) {
        live[m] = (row0 + m < p.B) && (p.tok[row0 + m] >= 0);
        any = any || live[m];
    }
    if (!any) return;

    for (int m = 0; m < MB; m++) {
        if (!live[m]) {
            for (int k = threadIdx.x; k < p.d; k += kThreads) hs_[m * p.d + k] = 0.f;
            continue;
        }
        const float* xr = p.X + (size_t)(row0 + m) * p.d;
        float s[1] = {0.f};
        for (int k = threadIdx.x; k < p.d; k += kThreads) {
            const float v = xr[k];
            s[0] += p.rms ? v * v : v;
        }
        block_sum<1>(s, sh);
        if (p.rms) {
            const float r = 1.0f / sqrtf(s[0] / (float)p.d + p.eps);
            for (int k = threadIdx.x; k < p.d; k += kThreads) hs_[m * p.d + k] = p.gamma[k] * xr[k] * r;
        } else {
            const float mean = s[0] / (float)p.d;
            float v2[1] = {0.f};
            for (int k = threadIdx.x; k < p.d; k += kThreads) {
                const float dlt = xr[k] - mean;
                v2[0] += dlt * dlt;
            }
            block_sum<1>(v2, sh);
            const float inv_std = 1.0f / sqrtf(v2[0] / (float)p.d + p.eps);
            for (int k = threadIdx.x; k < p.d; k += kThreads) {
                hs_[m * p.d + k] = p.gamma[k] * (xr[k] - mean) * inv_std + p.beta[k];
            }
        }
    }
    __syncthreads();

    const WT* E = static_cast<const WT*>(p.E);
    const int rows_per_block = kWarps * p.rows_per_warp;
    const int vbeg = blockIdx.x * rows_per_block + w * p.rows_per_warp;
    for (int v = vbeg; v < vbeg + p.rows_per_warp && v < p.V; v++) {
        const WT* er = E + (size_t)v * p.d;
        float acc[MB];
#pragma unroll
        for (int m = 0; m < MB; m++) acc[m] = 0.f;
        for (int k = lane * 4; k < p.d; k += 128) {
            const float4 e = load_w4(er + k);
#pragma unroll
            for (int m = 0; m < MB; m++) {
                const float4 hv = *reinterpret_cast<const float4*>(&hs_[m * p.d + k]);
                acc[m] += hv.x * e.x + hv.y * e.y + hv.z * e.z + hv.w * e.w;
            }
        }
#pragma unroll
        for (int m = 0; m < MB; m++) {
            const float t = warp_sum(acc[m]);
            if (lane == 0 && live[m]) p.logits[(size_t)(row0 + m) * p.V + v] = t;
        }
    }
}

// -------------------------------------------------------------- attention

// Head size 64. grid (splits, heads, batch); 4 warps per CTA take 32-position
// tiles of the CTA's context range round-robin, each with a running softmax.
// Eight lanes share a K row (two float4 each); for P@V each lane owns two
// output columns.
constexpr int kAttnWarps = 4;

__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode64_kernel(const AttnParams p) {
    constexpr int HS = 64;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    if (p.tok[b] < 0) return;
    const int S = gridDim.x;
    const int ctx = p.pos[b] + 1;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int ntiles = (ctx + 31) / 32;
    const int tps = (ntiles + S - 1) / S;
    const int tile_beg = split * tps, tile_end = min(ntiles, tile_beg + tps);

    const size_t head_base = (((size_t)b * p.H + h) * p.T) * HS;
    const float* K = p.kcache + head_base;
    const float* V = p.vcache + head_base;
    const int sub = lane & 7, rin = lane >> 3;

    const float4 q0 = *reinterpret_cast<const float4*>(p.q + (size_t)b * p.d + h * HS + sub * 8);
    const float4 q1 = *reinterpret_cast<const float4*>(p.q + (size_t)b * p.d + h * HS + sub * 8 + 4);

    float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;
    for (int t = tile_beg + w; t < tile_end; t += kAttnWarps) {
        const int r0 = t * 32;
        const int nrows = min(32, ctx - r0);
        float sc[8];
#pragma unroll
        for (int pp = 0; pp < 8; pp++) {
            const int r = pp * 4 + rin;
            float dsum = 0.f;
            if (r < nrows) {
                const float4* kr = reinterpret_cast<const float4*>(K + (size_t)(r0 + r) * HS + sub * 8);
                const float4 k0 = __ldcs(kr), k1 = __ldcs(kr + 1);
                dsum = q0.x * k0.x + q0.y * k0.y + q0.z * k0.z + q0.w * k0.w + q1.x * k1.x + q1.y * k1.y +
                       q1.z * k1.z + q1.w * k1.w;
            }
            dsum += __shfl_xor_sync(0xffffffffu, dsum, 1);
            dsum += __shfl_xor_sync(0xffffffffu, dsum, 2);
            dsum += __shfl_xor_sync(0xffffffffu, dsum, 4);
            sc[pp] = dsum;
        }
        float mine = 0.f;
#pragma unroll
        for (int pp = 0; pp < 8; pp++) {
            const float v = __shfl_sync(0xffffffffu, sc[pp], (lane & 3) * 8);
            if ((lane >> 2) == pp) mine = v;
        }
        mine = lane < nrows ? mine * p.scale : -INFINITY;
        const float m_new = fmaxf(m_run, warp_max(mine));
        const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
        const float pr = lane < nrows ? expf(mine - m_new) : 0.f;
        l_run = l_run * corr + warp_sum(pr);
        o0 *= corr;
        o1 *= corr;
        m_run = m_new;
        const float2* vr = reinterpret_cast<const float2*>(V + (size_t)r0 * HS) + lane;
#pragma unroll 8
        for (int r = 0; r < nrows; r++) {
            const float pv = __shfl_sync(0xffffffffu, pr, r);
            const float2 vv = __ldcs(vr + (size_t)r * (HS / 2));
            o0 += pv * vv.x;
            o1 += pv * vv.y;
        }
    }

    // combine the CTA's warps (fixed order)
    __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps], sm_o[kAttnWarps][HS];
    __shared__ int sm_last;
    if (lane == 0) {
        sm_m[w] = m_run;
        sm_l[w] = l_run;
    }
    sm_o[w][2 * lane] = o0;
    sm_o[w][2 * lane + 1] = o1;
    __syncthreads();
    if (w != 0) {
        if (S == 1) return;
    }
    float M = -INFINITY, Lsum = 0.f, a0 = 0.f, a1 = 0.f;
    if (w == 0) {
#pragma unroll
        for (int i = 0; i < kAttnWarps; i++) M = fmaxf(M, sm_m[i]);
#pragma unroll
        for (int i = 0; i < kAttnWarps; i++) {
            const float f = sm_m[i] == -INFINITY ? 0.f : expf(sm_m[i] - M);
            Lsum += sm_l[i] * f;
            a0 += sm_o[i][2 * lane] * f;
            a1 += sm_o[i][2 * lane + 1] * f;
        }
        if (S == 1) {
            const float inv = 1.0f / Lsum;
            *reinterpret_cast<float2*>(p.out + (size_t)b * p.d + h * HS + 2 * lane) = make_float2(a0 * inv, a1 * inv);
            if (p.out16) {
                *reinterpret_cast<__nv_bfloat162*>(p.out16 + (size_t)b * p.d + h * HS + 2 * lane) =
                    __floats2bfloat162_rn(a0 * inv, a1 * inv);
            }
            return;
        }
        float* part = p.partial + ((size_t)(b * p.H + h) * S + split) * (HS + 2);
        part[2 * lane] = a0;
        part[2 * lane + 1] = a1;
        if (lane == 0) {
            part[HS] = M;
            part[HS + 1] = Lsum;
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) {
            const int ticket = atomicAdd(p.counters + b * p.H + h, 1);
            sm_last = (ticket == S - 1);
        }
    }
    __syncthreads();
    if (w != 0 || !sm_last) return;
    // Last split to arrive combines all of them, in split order.
    __threadfence();
    const float* base = p.partial + (size_t)(b * p.H + h) * S * (HS + 2);
    float Mt = -INFINITY;
    for (int s = 0; s < S; s++) Mt = fmaxf(Mt, __ldcg(base + s * (HS + 2) + HS));
    float Lt = 0.f, c0 = 0.f, c1 = 0.f;
    for (int s = 0; s < S; s++) {
        const float ms = __ldcg(base + s * (HS + 2) + HS);
        const float f = ms == -INFINITY ? 0.f : expf(ms - Mt);
        Lt += __ldcg(base + s * (HS + 2) + HS + 1) * f;
        c0 += __ldcg(base + s * (HS + 2) + 2 * lane) * f;
        c1 += __ldcg(base + s * (HS + 2) + 2 * lane + 1) * f;
    }
    const float inv = 1.0f / Lt;
    *reinterpret_cast<float2*>(p.out + (size_t)b * p.d + h * HS + 2 * lane) = make_float2(c0 * inv, c1 * inv);
    if (p.out16) {
        *reinterpret_cast<__nv_bfloat162*>(p.out16 + (size_t)b * p.d + h * HS + 2 * lane) =
            __floats2bfloat162_rn(c0 * inv, c1 * inv);
    }
    if (lane == 0) p.counters[b * p.H + h] = 0;
}

// ---- pipelined variant -----------------------------------------------------------------
// Head size 64, persistent: one CTA per SM, seven independent warps. The (sequence, head,
// context split) units are dealt round-robin to the grid's warps; each warp turns its units
// into one flat sequence of 32-position tiles and keeps one tile ahead of the arithmetic in a
// private two-stage shared-memory ring filled by bulk asynchronous copies (one copy for the
// tile's K rows, one for its V rows: both are contiguous in the head-major cache). So the HBM
// stream of a warp continues across unit boundaries instead of restarting per (sequence, head).
// Scores: lane r owns row r of the tile and walks its 64 columns rotated by r, which keeps the
// 128-bit shared-memory reads conflict free and needs no shuffles. P@V: lane owns two columns.
constexpr int kPipeWarps = kAttnPipeWarps;  // independent warps per CTA: as many 2-stage rings as shared memory holds
constexpr int kPipeStages = 2;  // per warp: one tile being consumed, one in flight
constexpr int kPipeTileRows = 32;
constexpr int kPipeStageFloats = 2 * kPipeTileRows * 64;  // K tile then V tile
constexpr uint32_t kPipeSpin = 1u << 22;

struct AttnCursor {  // position in a warp's flat sequence of tiles
    int unit;        // current unit index (advances by the number of warps in the grid)
    int tile, tile_end;
    int b, h, split, ctx;
    int seq;  // cache sequence of row b
};

__device__ __forceinline__ bool attn_unit_setup(const AttnParams& p, int S, int total_units, AttnCursor& c) {
    // Fills the cursor for c.unit; returns false when the unit is beyond the end.
    if (c.unit >= total_units) return false;
    const int hs_units = p.H * S;
    c.b = c.unit / hs_units;
    c.h = (c.unit / S) % p.H;
    c.split = c.unit % S;
    c.seq = c.b;
    if (p.tok[c.b] < 0) {  // sequence sits this step out: no tiles, nothing to finalise
        c.ctx = 0;
        c.tile = c.tile_end = 0;
        return true;
    }
    c.ctx = p.pos[c.b] + 1;
    if (p.row_seq) c.seq = p.row_seq[c.b];
    const int ntiles = (c.ctx + kPipeTileRows - 1) / kPipeTileRows;
    const int tps = (ntiles + S - 1) / S;
    c.tile = c.split * tps;
    c.tile_end = min(ntiles, c.tile + tps);
    if (c.tile_end < c.tile) c.tile_end = c.tile;
    return true;
}

// x as a TF32-rounded value and its TF32-rounded remainder (the fp32 sessions' tensor-core operand format)
__device__ __forceinline__ void split_tf32_pair(float x, float& hi, float& lo) {
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hi));
    lo = __uint_as_float(l);
}
__device__ __forceinline__ void store_split2(float* out, size_t lo_elems, size_t at, float a, float b) {
    float ah, al, bh, bl;
    split_tf32_pair(a, ah, al);
    split_tf32_pair(b, bh, bl);
    *reinterpret_cast<float2*>(out + at) = make_float2(ah, bh);
    *reinterpret_cast<float2*>(out + lo_elems + at) = make_float2(al, bl);
}

__global__ void __launch_bounds__(kPipeWarps * 32, 1) attn_decode64_pipe_kernel(const AttnParams p, int S,
                                                                              int total_units) {
    constexpr int HS = 64;
    extern __shared__ __align__(128) float pipe_smem[];
    __shared__ __align__(8) uint64_t full_bar[kPipeWarps][kPipeStages];
    __shared__ float q_s[kPipeWarps][HS];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int warps_total = gridDim.x * kPipeWarps;
    const int gw = blockIdx.x * kPipeWarps + w;
    float* ring = pipe_smem + (size_t)w * kPipeStages * kPipeStageFloats;

    if (lane == 0) {
        for (int s = 0; s < kPipeStages; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&full_bar[w][s])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_trigger();
    pdl_wait();  // q, positions and the newest K/V rows come from the kernels before this one

    // issue the copies of the tile the fetch cursor points at, then advance it
    AttnCursor fc{};
    fc.unit = gw;
    bool f_ok = attn_unit_setup(p, S, total_units, fc);
    int issued = 0;
    // The cache is read once per step and is far larger than L2: mark its lines first to go, so that the weights the
    // projections re-read every step are what stays.
    uint64_t stream_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(stream_policy));
    auto fetch_next = [&]() {
        while (f_ok && fc.tile >= fc.tile_end) {  // skip units without tiles
            fc.unit += warps_total;
            f_ok = attn_unit_setup(p, S, total_units, fc);
        }
        if (!f_ok) return;
        const int stage = issued % kPipeStages;
        const int r0 = fc.tile * kPipeTileRows;
        const int nrows = min(kPipeTileRows, fc.ctx - r0);
#if GRADB_DIAG
        const bool leave_out = issued == p.diag_skip_tile;  // the hook that lets a wait run out
#else
        constexpr bool leave_out = false;
#endif
        if (lane == 0 && !leave_out) {
            const size_t off = (((size_t)fc.seq * p.H + fc.h) * p.T + r0) * HS;
            const uint32_t bytes = (uint32_t)nrows * HS * 4;
            const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&full_bar[w][stage]);
            const uint32_t dstk = (uint32_t)__cvta_generic_to_shared(ring + (size_t)stage * kPipeStageFloats);
            const uint32_t dstv = dstk + kPipeTileRows * HS * 4;
            // the stage was last read with ordinary loads: order them before the asynchronous writes
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dstk),
                "l"(p.kcache + off), "r"(bytes), "r"(bar), "l"(stream_policy)
                : "memory");
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dstv),
                "l"(p.vcache + off), "r"(bytes), "r"(bar), "l"(stream_policy)
                : "memory");
        }
        issued++;
        fc.tile++;
    };
    for (int i = 0; i < kPipeStages; i++) fetch_next();  // fill the ring

    int consumed = 0;
    AttnCursor cc{};
    cc.unit = gw;
    bool c_ok = attn_unit_setup(p, S, total_units, cc);
    // q of a unit is fetched one unit early so that its latency hides behind the previous unit's tiles
    float qa = 0.f, qb = 0.f;
    if (c_ok && cc.ctx > 0) {
        qa = p.q[(size_t)cc.b * p.d + cc.h * HS + lane];
        qb = p.q[(size_t)cc.b * p.d + cc.h * HS + lane + 32];
    }
    for (; c_ok;) {
        AttnCursor nx = cc;
        nx.unit = cc.unit + warps_total;
        const bool n_ok = attn_unit_setup(p, S, total_units, nx);
        float nqa = 0.f, nqb = 0.f;
        if (n_ok && nx.ctx > 0) {
            nqa = p.q[(size_t)nx.b * p.d + nx.h * HS + lane];
            nqb = p.q[(size_t)nx.b * p.d + nx.h * HS + lane + 32];
        }
        const AttnCursor cur = cc;
        const float cqa = qa, cqb = qb;
        cc = nx;
        c_ok = n_ok;
        qa = nqa;
        qb = nqb;
        if (cur.ctx == 0) continue;  // inactive sequence
        __syncwarp();
        q_s[w][lane] = cqa;
        q_s[w][lane + 32] = cqb;
        __syncwarp();
        float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;
        for (int t = cur.tile; t < cur.tile_end; t++) {
            const int stage = consumed % kPipeStages;
            const uint32_t parity = (consumed / kPipeStages) & 1;
            {
                const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&full_bar[w][stage]);
                uint32_t ok = 0;
#if GRADB_DIAG
                const uint32_t spin = p.diag_spin_limit ? p.diag_spin_limit : kPipeSpin;
#else
                constexpr uint32_t spin = kPipeSpin;
#endif
                for (uint32_t it = 0; it < spin && !ok; ++it) {
                    asm volatile(
                        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                        : "=r"(ok)
                        : "r"(bar), "r"(parity)
                        : "memory");
                }
                if (!ok) {
                    // Bounded: give up on this launch; the host sees the status word. Warps share nothing (own ring,
                    // own barriers, no CTA-wide barrier anywhere in this kernel), so this warp may simply leave - after
                    // the copies it still has in flight into its ring have landed (again bounded).
                    if (lane == 0 && p.status) atomicExch(p.status, 301);
                    for (int c = consumed + 1; c < issued; c++) {
                        const uint32_t ob = (uint32_t)__cvta_generic_to_shared(&full_bar[w][c % kPipeStages]);
                        const uint32_t op = (c / kPipeStages) & 1;
                        uint32_t landed = 0;
                        for (uint32_t it = 0; it < kPipeSpin && !landed; ++it) {
                            asm volatile(
                                "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                                : "=r"(landed)
                                : "r"(ob), "r"(op)
                                : "memory");
                        }
                    }
                    return;
                }
            }
            const float* Kt = ring + (size_t)stage * kPipeStageFloats;
            const float* Vt = Kt + kPipeTileRows * HS;
            const int r0 = t * kPipeTileRows;
            const int nrows = min(kPipeTileRows, cur.ctx - r0);
            // scores: lane r <-> row r, columns visited rotated by r (16-byte chunks)
            float dot = 0.f;
            if (lane < nrows) {
                const float4* kr = reinterpret_cast<const float4*>(Kt + lane * HS);
                const float4* qr = reinterpret_cast<const float4*>(q_s[w]);
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int c = (j + lane) & 15;
                    const float4 kv = kr[c], qv = qr[c];
                    d0 += qv.x * kv.x;
                    d1 += qv.y * kv.y;
                    d2 += qv.z * kv.z;
                    d3 += qv.w * kv.w;
                }
                dot = (d0 + d1) + (d2 + d3);
            }
            const float mine = lane < nrows ? dot * p.scale : -INFINITY;
            const float m_new = fmaxf(m_run, warp_max(mine));
            const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
            const float pr = lane < nrows ? expf(mine - m_new) : 0.f;
            l_run = l_run * corr + warp_sum(pr);
            o0 *= corr;
            o1 *= corr;
            m_run = m_new;
            const float2* vr = reinterpret_cast<const float2*>(Vt) + lane;
            float e0 = 0.f, e1 = 0.f;  // second accumulator pair: two independent chains
            if (nrows == kPipeTileRows) {
#pragma unroll
                for (int r = 0; r < kPipeTileRows; r += 2) {
                    const float pa = __shfl_sync(0xffffffffu, pr, r), pb = __shfl_sync(0xffffffffu, pr, r + 1);
                    const float2 va = vr[r * (HS / 2)], vb = vr[(r + 1) * (HS / 2)];
                    o0 += pa * va.x;
                    o1 += pa * va.y;
                    e0 += pb * vb.x;
                    e1 += pb * vb.y;
                }
            } else {
                for (int r = 0; r < nrows; r++) {
                    const float pv = __shfl_sync(0xffffffffu, pr, r);
                    const float2 vv = vr[r * (HS / 2)];
                    o0 += pv * vv.x;
                    o1 += pv * vv.y;
                }
            }
            o0 += e0;
            o1 += e1;
            consumed++;
            __syncwarp();   // the whole warp is done with this stage ...
            fetch_next();   // ... so the next tile of the sequence may land in it
        }
        // finalise the unit
        if (S == 1) {
            const float inv = 1.0f / l_run;
            *reinterpret_cast<float2*>(p.out + (size_t)cur.b * p.d + cur.h * HS + 2 * lane) = make_float2(o0 * inv, o1 * inv);
            if (p.out16) {
                *reinterpret_cast<__nv_bfloat162*>(p.out16 + (size_t)cur.b * p.d + cur.h * HS + 2 * lane) =
                    __floats2bfloat162_rn(o0 * inv, o1 * inv);
            }
            if (p.out_split) {
                store_split2(p.out_split, p.out_lo_elems, (size_t)cur.b * p.d + cur.h * HS + 2 * lane, o0 * inv, o1 * inv);
            }
            continue;
        }
        const int bh = cur.b * p.H + cur.h;
        float* part = p.partial + ((size_t)bh * S + cur.split) * (HS + 2);
        part[2 * lane] = o0;
        part[2 * lane + 1] = o1;
        if (lane == 0) {
            part[HS] = m_run;
            part[HS + 1] = l_run;
        }
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(p.counters + bh, 1) == S - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) continue;
        // the last split to arrive combines all of them, in split order
        __threadfence();
        const float* base = p.partial + (size_t)bh * S * (HS + 2);
        float Mt = -INFINITY;
        for (int s2 = 0; s2 < S; s2++) Mt = fmaxf(Mt, __ldcg(base + s2 * (HS + 2) + HS));
        float Lt = 0.f, c0 = 0.f, c1 = 0.f;
        for (int s2 = 0; s2 < S; s2++) {
            const float ms = __ldcg(base + s2 * (HS + 2) + HS);
            const float f = ms == -INFINITY ? 0.f : expf(ms - Mt);
            Lt += __ldcg(base + s2 * (HS + 2) + HS + 1) * f;
            c0 += __ldcg(base + s2 * (HS + 2) + 2 * lane) * f;
            c1 += __ldcg(base + s2 * (HS + 2) + 2 * lane + 1) * f;
        }
        const float inv = 1.0f / Lt;
        *reinterpret_cast<float2*>(p.out + (size_t)cur.b * p.d + cur.h * HS + 2 * lane) = make_float2(c0 * inv, c1 * inv);
        if (p.out16) {
            *reinterpret_cast<__nv_bfloat162*>(p.out16 + (size_t)cur.b * p.d + cur.h * HS + 2 * lane) =
                __floats2bfloat162_rn(c0 * inv, c1 * inv);
        }
        if (p.out_split) {
            store_split2(p.out_split, p.out_lo_elems, (size_t)cur.b * p.d + cur.h * HS + 2 * lane, c0 * inv, c1 * inv);
        }
        if (lane == 0) p.counters[bh] = 0;
    }
}

// Any head size: one CTA per (head, sequence), scores kept in shared memory.
// Mirrors the reference loop structure directly (inference.cpp:208-225).
__global__ void __launch_bounds__(128) attn_decode_generic_kernel(const AttnParams p) {
    extern __shared__ float scores[];
    __shared__ float sh[4];
    const int h = blockIdx.y, b = blockIdx.z;
    if (p.tok[b] < 0) return;
    const int ctx = p.pos[b] + 1, hs = p.hs;
    const size_t head_base = (((size_t)b * p.H + h) * p.T) * hs;
    const float* K = p.kcache + head_base;
    const float* V = p.vcache + head_base;
    const float* q = p.q + (size_t)b * p.d + h * hs;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;

    float mx = -INFINITY;
    for (int t = threadIdx.x; t < ctx; t += blockDim.x) {
        float dsum = 0.f;
        for (int j = 0; j < hs; j++) dsum += q[j] * K[(size_t)t * hs + j];
        dsum *= p.scale;
        scores[t] = dsum;
        mx = fmaxf(mx, dsum);
    }
    mx = warp_max(mx);
    if (lane == 0) sh[w] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
    __syncthreads();
    float sum = 0.f;
    for (int t = threadIdx.x; t < ctx; t += blockDim.x) {
        const float e = expf(scores[t] - mx);
        scores[t] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) sh[w] = sum;
    __syncthreads();
    const float inv = 1.0f / (((sh[0] + sh[1]) + sh[2]) + sh[3]);
    for (int c = threadIdx.x; c < hs; c += blockDim.x) {
        float o = 0.f;
        for (int t = 0; t < ctx; t++) o += scores[t] * inv * V[(size_t)t * hs + c];
        p.out[(size_t)b * p.d + h * hs + c] = o;
        if (p.out16) p.out16[(size_t)b * p.d + h * hs + c] = __float2bfloat16_rn(o);
    }
}

// Opt-in to more than 48 KB of dynamic shared memory. Skipped while a stream is
// being captured: every kernel has by then run once eagerly with the same size.
template <typename K>
void set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024 && !g_capturing) {
        GRADB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
}

template <int MB, typename WT, int PRO, int EPI, int NW>
void launch_gemv_t(const GemvParams& p, int n_tiles, int KS, cudaStream_t st) {
    const size_t floats = (size_t)MB * (p.K / KS) + (PRO != PRO_NONE ? p.K : 0) +
                          (size_t)(kWarps + 1) * NW * MB * kTileN + kWarps * MB;
    const size_t bytes = floats * sizeof(float);
    auto kernel = fused_gemv_kernel<MB, WT, PRO, EPI, NW>;
    set_smem(kernel, bytes);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(n_tiles, KS, (p.B + MB - 1) / MB);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = KS;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    GRADB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    count_launch();
}

template <int MB, typename WT>
void launch_gemv_mb(const GemvParams& p, int pro, int epi, int n_tiles, int KS, cudaStream_t st) {
    if (epi == EPI_QKV) {
        if (pro == PRO_RMSNORM) launch_gemv_t<MB, WT, PRO_RMSNORM, EPI_QKV, 1>(p, n_tiles, KS, st);
        else launch_gemv_t<MB, WT, PRO_LAYERNORM, EPI_QKV, 1>(p, n_tiles, KS, st);
    } else if (epi == EPI_RESID) {
        launch_gemv_t<MB, WT, PRO_NONE, EPI_RESID, 1>(p, n_tiles, KS, st);
    } else if (epi == EPI_GELU) {
        launch_gemv_t<MB, WT, PRO_LAYERNORM, EPI_GELU, 1>(p, n_tiles, KS, st);
    } else {
        launch_gemv_t<MB, WT, PRO_RMSNORM, EPI_SWIGLU, 2>(p, n_tiles, KS, st);
    }
}

int pick_mb(int B) { return B >= 8 ? 8 : (B >= 4 ? 4 : (B >= 2 ? 2 : 1)); }

}  // namespace

void launch_gather_last_rows(const float* rows, const int* row_last, const int* row_seq, float* x_seq, int d, int R,
                             cudaStream_t st) {
    gather_last_rows_kernel<<<R, 128, 0, st>>>(rows, row_last, row_seq, x_seq, d);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

void launch_feed_bookkeeping(const int* row_tok, const int* row_pos, const int* row_seq, const int* seq_count, int* pos,
                             int* hist_len, int* hist, int hist_stride, int R, int B, cudaStream_t st) {
    feed_history_kernel<<<(R + 255) / 256, 256, 0, st>>>(row_tok, row_pos, row_seq, pos, hist_len, hist, hist_stride, R);
    feed_advance_kernel<<<(B + 255) / 256, 256, 0, st>>>(seq_count, pos, hist_len, B);
    count_launch(2);
    GRADB_CUDA(cudaGetLastError());
}

void launch_embed(const float* E, const float* P, const int* tok, const int* pos, float* x, int d, int B,
                  cudaStream_t st) {
    launch_kernel(embed_kernel, dim3(B), dim3(128), 0, st, E, P, tok, pos, x, d);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

void launch_advance(const int* tok, int* pos, int* hist, int* hist_len, int hist_stride, int B, cudaStream_t st) {
    launch_kernel(advance_kernel, dim3((B + 127) / 128), dim3(128), 0, st, tok, pos, hist, hist_len, hist_stride, B);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

void launch_gemv(const GemvParams& p, int pro, int epi, bool bf16, int sm_count, cudaStream_t st) {
    const int tiles_per = (p.N + kTileN - 1) / kTileN;
    const int n_tiles = epi == EPI_QKV ? 3 * tiles_per : tiles_per;
    const int MB = pick_mb(p.B);
    const int row_groups = (p.B + MB - 1) / MB;
    // Split the reduction dimension across a cluster until the grid covers the SMs.
    int KS = 1;
    while (KS < 8 && n_tiles * row_groups * KS < sm_count && p.K % (8 * KS) == 0 && p.K / (2 * KS) >= 32) KS *= 2;
#define GRADB_MB_CASE(M)                                                                     \
    case M:                                                                                  \
        if (bf16) launch_gemv_mb<M, __nv_bfloat16>(p, pro, epi, n_tiles, KS, st);            \
        else launch_gemv_mb<M, float>(p, pro, epi, n_tiles, KS, st);                         \
        break;
    switch (MB) {
        GRADB_MB_CASE(1)
        GRADB_MB_CASE(2)
        GRADB_MB_CASE(4)
        GRADB_MB_CASE(8)
    }
#undef GRADB_MB_CASE
}

void launch_logits(const LogitsParams& p_in, bool bf16, cudaStream_t st) {
    LogitsParams p = p_in;
    const int MB = pick_mb(p.B);
    p.rows_per_warp = 4;
    const int rows_per_block = kWarps * p.rows_per_warp;
    const dim3 grid((p.V + rows_per_block - 1) / rows_per_block, (p.B + MB - 1) / MB);
    const size_t bytes = ((size_t)MB * p.d + kWarps * MB) * sizeof(float);
#define GRADB_MB_CASE(M)                                                              \
    case M:                                                                           \
        if (bf16) {                                                                   \
            set_smem(logits_kernel<M, __nv_bfloat16>, bytes);                         \
            logits_kernel<M, __nv_bfloat16><<<grid, kThreads, bytes, st>>>(p);        \
        } else {                                                                      \
            set_smem(logits_kernel<M, float>, bytes);                                 \
            logits_kernel<M, float><<<grid, kThreads, bytes, st>>>(p);                \
        }                                                                             \
        break;
    switch (MB) {
        GRADB_MB_CASE(1)
        GRADB_MB_CASE(2)
        GRADB_MB_CASE(4)
        GRADB_MB_CASE(8)
    }
#undef GRADB_MB_CASE
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// Attention without any allocation: the split partials and arrival tickets live in a fixed
// device array that every GPU loading this library carries until the process exits.
constexpr int kStaticAttnUnits = 4096;  // (sequence, head, split) slots
constexpr int kStaticAttnFloats = kStaticAttnUnits * (64 + 2);
static __device__ __align__(256) float g_static_attn_scratch[kStaticAttnFloats + kStaticAttnUnits];

int static_attention_capacity() { return kStaticAttnUnits; }

// In host code the array's name is only a handle: the device address has to be asked for,
// once per device, with that device current.
static float* static_attn_scratch_address() {
    static std::mutex mu;
    static float* cached[64] = {};
    int dev = 0;
    GRADB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) throw Error(GRADB_ERR_INVALID, "device index out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        float* ptr = nullptr;
        GRADB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_attn_scratch));
        cached[dev] = ptr;
    }
    return cached[dev];
}

void launch_attention_static(const AttnParams& p_in, int B, int splits, cudaStream_t st) {
    if (p_in.hs != 64) throw Error(GRADB_ERR_INVALID, "the allocation-free attention entry point supports head_dim 64");
    const long units = (long)B * p_in.H * splits;
    if (units > kStaticAttnUnits) {
        throw Error(GRADB_ERR_INVALID, "n_seq * heads * splits = " + std::to_string(units) +
                                           " exceeds the fixed scratch of " + std::to_string(kStaticAttnUnits) +
                                           " slots of the allocation-free attention entry point");
    }
    float* scratch = static_attn_scratch_address();
    AttnParams p = p_in;
    p.partial = scratch;
    p.counters = reinterpret_cast<int*>(scratch + kStaticAttnFloats);
    // The array keeps whatever the previous call left; the tickets must start at zero.
    GRADB_CUDA(cudaMemsetAsync(p.counters, 0, (size_t)B * p.H * sizeof(int), st));
    attn_decode64_kernel<<<dim3(splits, p.H, B), kAttnWarps * 32, 0, st>>>(p);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

namespace {
__global__ void count_nonfinite_kernel(const float* __restrict__ x, size_t n, unsigned long long* out) {
    unsigned long long bad = 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        bad += (v != v || fabsf(v) == INFINITY) ? 1ull : 0ull;
    }
    if (bad) atomicAdd(out, bad);
}
}  // namespace

// NaN / Inf scan of a device buffer (diagnostics build's output check). Synchronises the stream.
long long count_nonfinite(const float* x, size_t n, cudaStream_t st) {
    unsigned long long* d = nullptr;
    unsigned long long h = 0;
    GRADB_CUDA(cudaMalloc(&d, sizeof(h)));
    GRADB_CUDA(cudaMemsetAsync(d, 0, sizeof(h), st));
    count_nonfinite_kernel<<<256, 256, 0, st>>>(x, n, d);
    count_launch();
    GRADB_CUDA(cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, st));
    GRADB_CUDA(cudaStreamSynchronize(st));
    cudaFree(d);
    return (long long)h;
}

// Opt the pipelined attention kernel into its shared memory up front (per device).
void attention_configure() {
    const size_t bytes = (size_t)kPipeWarps * kPipeStages * kPipeStageFloats * sizeof(float);
    GRADB_CUDA(cudaFuncSetAttribute(attn_decode64_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
}

void launch_attention(const AttnParams& p, int B, int splits, cudaStream_t st) {
    if (p.hs == 64) {
        // persistent, pipelined kernel: one CTA per SM (its rings take most of the shared memory)
        static int sm_count = 0;
        if (!sm_count) {
            int dev = 0;
            GRADB_CUDA(cudaGetDevice(&dev));
            GRADB_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
        }
        const int total_units = B * p.H * splits;
        const int grid = std::max(1, std::min(sm_count, (total_units + kPipeWarps - 1) / kPipeWarps));
        const size_t bytes = (size_t)kPipeWarps * kPipeStages * kPipeStageFloats * sizeof(float);
        set_smem(attn_decode64_pipe_kernel, bytes);
        launch_kernel(attn_decode64_pipe_kernel, dim3(grid), dim3(kPipeWarps * 32), bytes, st, p, splits, total_units);
    } else {
        const size_t bytes = (size_t)p.T * sizeof(float);
        set_smem(attn_decode_generic_kernel, bytes);
        attn_decode_generic_kernel<<<dim3(1, p.H, B), 128, bytes, st>>>(p);
    }
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// Teacher-forced scoring: one CTA per row, one pass over the row's logits. Every thread keeps a
// running (max, sum of exp(x - max)) over its slice; the pairs are merged by shuffles.
namespace {
constexpr int kLogpThreads = 256;

__device__ __forceinline__ void lse_push(float& m, float& s, float x) {
    if (x > m) {
        s = s * expf(m - x) + 1.0f;
        m = x;
    } else {
        s += expf(x - m);
    }
}
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
    const float M = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * expf(m - M)) + (m2 == -INFINITY ? 0.f : s2 * expf(m2 - M));
    m = M;
}

__global__ void __launch_bounds__(kLogpThreads) row_logp_kernel(const float* __restrict__ logits, size_t ld, int V,
                                                                 const int* __restrict__ tgt,
                                                                 const int* __restrict__ dst, int dst_mul, int dst_add,
                                                                 float* __restrict__ out) {
    pdl_wait();
    const int r = blockIdx.x;
    const float* x = logits + (size_t)r * ld;
    float m = -INFINITY, s = 0.f;
    if ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = V >> 2;
        for (int i = threadIdx.x; i < n4; i += kLogpThreads) {
            const float4 v = __ldg(x4 + i);
            lse_push(m, s, v.x);
            lse_push(m, s, v.y);
            lse_push(m, s, v.z);
            lse_push(m, s, v.w);
        }
        for (int i = (n4 << 2) + threadIdx.x; i < V; i += kLogpThreads) lse_push(m, s, x[i]);
    } else {
        for (int i = threadIdx.x; i < V; i += kLogpThreads) lse_push(m, s, x[i]);
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        lse_merge(m, s, m2, s2);
    }
    __shared__ float sm[kLogpThreads / 32], ss[kLogpThreads / 32];
    if ((threadIdx.x & 31) == 0) {
        sm[threadIdx.x >> 5] = m;
        ss[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        m = sm[0];
        s = ss[0];
        for (int w = 1; w < kLogpThreads / 32; w++) lse_merge(m, s, sm[w], ss[w]);
        const int t = tgt[r];
        float lp = 0.f;
        if (t >= 0 && t < V) lp = (x[t] - m) - logf(s);
        out[dst ? dst[r] : r * dst_mul + dst_add] = lp;
    }
}
}  // namespace

void launch_row_logp(const float* logits, size_t ld, int V, const int* tgt, const int* dst, int dst_mul, int dst_add,
                     float* out, int rows, cudaStream_t st) {
    if (rows <= 0) return;
    launch_kernel(row_logp_kernel, dim3(rows), dim3(kLogpThreads), 0, st, logits, ld, V, tgt, dst, dst_mul, dst_add,
                  out);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

namespace {
__global__ void __launch_bounds__(256) lse_combine_kernel(const float* __restrict__ part, int tiles,
                                                          const float* __restrict__ tgt_logit,
                                                          const int* __restrict__ tgt, int V,
                                                          const int* __restrict__ dst, float* __restrict__ out, int rows) {
    pdl_wait();
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const float2* pr = reinterpret_cast<const float2*>(part) + (size_t)r * tiles;
    float m = -INFINITY, s = 0.f;
    for (int t = lane; t < tiles; t += 32) {
        const float2 v = pr[t];
        lse_merge(m, s, v.x, v.y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        lse_merge(m, s, m2, s2);
    }
    if (lane == 0) {
        const int t = tgt[r];
        out[dst[r]] = (t >= 0 && t < V) ? (tgt_logit[r] - m) - logf(s) : 0.f;
    }
}
}  // namespace

void launch_lse_combine(const float* part, int tiles, const float* tgt_logit, const int* tgt, int V, const int* dst,
                        float* out, int rows, cudaStream_t st) {
    if (rows <= 0) return;
    launch_kernel(lse_combine_kernel, dim3((rows + 7) / 8), dim3(256), 0, st, part, tiles, tgt_logit, tgt, V, dst, out, rows);
    count_launch();
    GRADB_CUDA(cudaGetLastError());
}

}  // namespace gradb
