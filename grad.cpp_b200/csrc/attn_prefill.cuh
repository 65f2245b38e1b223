// Query-tiled causal attention over the KV cache for rows that are consecutive positions of their
// sequences (batched prompt feed, scoring). Head size 64 (attn_prefill.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace gradb {

struct PrefillAttnParams {
    const float* q;                // [rows][d], this layer's queries (RoPE applied)
    const float *kcache, *vcache;  // one layer: [sequences][H][T][64]
    float* out;                    // optional [rows][d]
    __nv_bfloat16* out16;          // optional [rows][d]
    // One entry per tile of up to 64 (tensor-core kernel: 128) consecutive positions of one sequence:
    // x = cache sequence, y = first row, z = position of the first row, w = rows in the tile.
    const int4* tiles;
    int n_tiles;
    int H, T, d;
    float scale;
    int* status = nullptr;  // session status word: set by the tensor-core kernel if a bounded wait expires
};

void prefill_attention_configure();
// The same attention on tcgen05 (attn_prefill_tc.cu), for sessions whose attention may run at TF32 precision: tiles
// of up to 128 positions; map_q = fp32 tensor map over the query rows (boxes of 32 columns x 128 rows), map_k = fp32
// tensor map over the whole K cache as rows of 64 floats, k_row0 = first row of this layer in it.
void prefill_attention_tc_configure();
#if GRADB_DIAG
void attn_clocks_read(unsigned long long* out16, bool reset);  // diagnostics build: per-phase clocks of the kernel below
#endif
void launch_prefill_attention_tc(const PrefillAttnParams& p, const CUtensorMap& map_q, const CUtensorMap& map_k,
                                 const CUtensorMap& map_v, long long k_row0, int sm_count, cudaStream_t st);
// fp32_grade: three TF32 MMAs per product on hi/lo operand pairs (fp32 sessions) instead of one.
void launch_prefill_attention(const PrefillAttnParams& p, cudaStream_t st, bool fp32_grade = false);

}  // namespace gradb
