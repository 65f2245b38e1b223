// Tensor-core projections for batched decode and the prompt feed (gemm_tc.cu).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace gradb {

// TC_LSE (many-row kernel only): logits are not written; every 128-feature tile leaves, per token, its maximum and
// sum of exp(x - max), plus the logit of the token's target id if the tile holds it (scoring).
enum { TC_QKV = 0, TC_RESID = 1, TC_GELU = 2, TC_SWIGLU = 3, TC_LOGITS = 4, TC_LSE = 5 };

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
    // fp32 mode (3xTF32): every operand is stored as two fp32 matrices, the TF32-rounded value and the
    // TF32-rounded remainder, stacked in one allocation; *_lo_rows is the row distance between the two
    // halves inside the operand's tensor map. The FFN activation is written the same way.
    int a_lo_rows = 0, b_lo_rows = 0;
    float* out_split = nullptr;  // FFN activation: [2][rows][ld_out]
    size_t out_lo_elems = 0;
    // TC_LSE: per (row, feature tile) pairs (max, sum of exp) in out_f32 [rows][ld_out = 2 * tiles]; `pos` carries the
    // rows' target ids; lse_tgt[row] receives the target's logit.
    float* lse_tgt = nullptr;
};

// 2-D bf16 tensor map over a row-major (rows, cols) matrix: boxes of 64 columns x box_rows, 128-byte swizzle.
void make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
int tc_token_tile(int n_seq, int n_tiles, int want_ctas);
void tc_configure_all();
// kind 0: bf16 operands; kind 1: fp32 operands as TF32 hi/lo pairs, three MMAs per product (fp32-grade result).
#if GRADB_DIAG
void wide_clocks_read(unsigned long long* out128, bool reset);  // diagnostics build: per-role clocks of the many-row GEMM
#endif
void launch_tc_gemm(int epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const TcGemmParams& p, int token_tile,
                    int k_splits, cudaStream_t st, int kind = 0);
// True when launch_tc_gemm would run the many-row persistent kernel for this shape (needed by TC_LSE callers).
bool tc_many_rows(const TcGemmParams& p, int token_tile);
// 2-D fp32 tensor map over a row-major (rows, cols) matrix: boxes of 32 columns x box_rows, 128-byte swizzle
// (atom32: in 32-byte units, the form a 32-bit MN-major MMA operand needs; otherwise in 16-byte units).
void make_tensor_map_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                         bool atom32 = false);
// Normalised rows as TF32 hi/lo pairs: out[0][row][d] and out[1][row][d], the halves lo_elems apart.
void launch_norm_split(const float* X, const float* gamma, const float* beta, const int* tok, float* out, size_t lo_elems,
                       int d, int rms, float eps, int B, cudaStream_t st);
// in[n] -> out[n] (TF32-rounded) and out[lo_elems + n] (TF32-rounded remainder)
void launch_split_tf32(const float* in, float* out, size_t lo_elems, size_t n, cudaStream_t st);
// W (K, N) fp32 -> W^T as hi/lo pair [2][rows_total][K], same row mapping as launch_transpose_bf16.
void launch_transpose_split(const float* W, float* out, size_t lo_elems, int K, int N, int row_offset, bool interleave,
                            cudaStream_t st);
void launch_norm_bf16(const float* X, const float* gamma, const float* beta, const int* tok, __nv_bfloat16* out, int d,
                      int rms, float eps, int B, cudaStream_t st);
void launch_transpose_bf16(const float* W, __nv_bfloat16* out, int K, int N, int row_offset, bool interleave,
                           cudaStream_t st);

}  // namespace gradb
