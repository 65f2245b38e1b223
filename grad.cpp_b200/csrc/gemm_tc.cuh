// Tensor-core projections for batched decode and the prompt feed (gemm_tc.cu).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace gradb {

enum { TC_QKV = 0, TC_RESID = 1, TC_GELU = 2, TC_SWIGLU = 3, TC_LOGITS = 4 };

struct TcGemmParams {
    int K, N, B;  // reduction length, output features (of one matrix), rows (sequences)
    int d, H, hs, T;
    int ld_out;
    const float* bias[3];
    const int *tok, *pos;
    const int* row_seq;  // optional: cache sequence of each row (prompt feed: one row per prompt token); null = row index
    const float *rope_cos, *rope_sin;
    float* out_f32;           // q / residual stream / logits
    __nv_bfloat16* out_bf16;  // FFN activation
    float *kcache, *vcache;
    int* status;  // set non-zero by a kernel whose bounded wait expired
};

// 2-D bf16 tensor map over a row-major (rows, cols) matrix: boxes of 64 columns x box_rows, 128-byte swizzle.
void make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
int tc_token_tile(int n_seq, int n_tiles, int want_ctas);
void tc_configure_all();
void launch_tc_gemm(int epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const TcGemmParams& p, int token_tile,
                    int k_splits, cudaStream_t st);
void launch_norm_bf16(const float* X, const float* gamma, const float* beta, const int* tok, __nv_bfloat16* out, int d,
                      int rms, float eps, int B, cudaStream_t st);
void launch_transpose_bf16(const float* W, __nv_bfloat16* out, int K, int N, int row_offset, bool interleave,
                           cudaStream_t st);

}  // namespace gradb
