// Query-tiled causal attention over the KV cache for rows that are consecutive positions of their
// sequences (batched prompt feed, scoring). Head size 64 (attn_prefill.cu).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace gradb {

struct PrefillAttnParams {
    const float* q;                // [rows][d], this layer's queries (RoPE applied)
    const float *kcache, *vcache;  // one layer: [sequences][H][T][64]
    float* out;                    // optional [rows][d]
    __nv_bfloat16* out16;          // optional [rows][d]
    // One entry per tile of up to 64 consecutive positions of one sequence:
    // x = cache sequence, y = first row, z = position of the first row, w = rows in the tile.
    const int4* tiles;
    int n_tiles;
    int H, T, d;
    float scale;
};

void prefill_attention_configure();
// fp32_grade: three TF32 MMAs per product on hi/lo operand pairs (fp32 sessions) instead of one.
void launch_prefill_attention(const PrefillAttnParams& p, cudaStream_t st, bool fp32_grade = false);

}  // namespace gradb
