// Launchers of the decode-step kernels (step_kernels.cu).
#pragma once
#include "common.cuh"

namespace gradb {

enum { PRO_NONE = 0, PRO_LAYERNORM = 1, PRO_RMSNORM = 2 };
enum { EPI_QKV = 0, EPI_RESID = 1, EPI_GELU = 2, EPI_SWIGLU = 3 };

struct GemvParams {
    const float* X;  // [B][ldx] input rows
    int ldx;
    int B, K, N;           // N = columns of ONE matrix
    const void* W[3];      // QKV: Wq, Wk, Wv. SwiGLU: gate, up. Others: W[0]
    const float* bias[3];  // may be null (bias-free projections)
    const float *gamma, *beta;
    float eps;
    const int *tok, *pos;  // per-sequence current token (<0: skip) and position
    float* Y;              // q / residual stream / FFN activation
    int ldy;
    // EPI_QKV only
    float *kcache, *vcache;  // this layer's caches: [B][H][T][hs]
    const float *rope_cos, *rope_sin;  // [max_len][hs/2] or null (GPT-2)
    int H, hs, T;
};

struct LogitsParams {
    const float* X;  // [B][d] residual stream
    const void* E;   // (V, d) embedding table, fp32 or bf16
    const float *gamma, *beta;
    float eps;
    int rms;
    const int* tok;
    float* logits;  // [B][V]
    int B, d, V;
    int rows_per_warp;
};

struct AttnParams {
    const float* q;  // [B][d]
    const float *kcache, *vcache;
    const int *tok, *pos;
    const int* row_seq;  // optional: cache sequence of each row (prompt feed); null = row index
    float* out;       // [B][d]
    __nv_bfloat16* out16;  // optional bf16 copy of out (operand of the tensor-core projection)
    // optional TF32 hi/lo copy of out (fp32 sessions' tensor-core operand), halves out_lo_elems apart; written by
    // the pipelined head-size-64 kernel only
    float* out_split = nullptr;
    size_t out_lo_elems = 0;
    float* partial;   // [B][H][S][hs+2] split results: o[hs], max, sum
    int* counters;    // [B][H] arrival tickets, zero between launches
    int* status;      // optional: set non-zero if a bounded wait expires
    int H, hs, T, d;
    float scale;
    // Diagnostics build only: spin limit of the pipelined kernel's tile wait (0 = the normal one) and the index of
    // the tile, counted per warp from 0, whose copy is left out so that the wait for it expires (-1 = none).
    uint32_t diag_spin_limit = 0;
    int diag_skip_tile = -1;
};

long long count_nonfinite(const float* x, size_t n, cudaStream_t st);
void launch_gather_last_rows(const float* rows, const int* row_last, const int* row_seq, float* x_seq, int d, int R,
                             cudaStream_t st);
void launch_feed_bookkeeping(const int* row_tok, const int* row_pos, const int* row_seq, const int* seq_count, int* pos,
                             int* hist_len, int* hist, int hist_stride, int R, int B, cudaStream_t st);
void launch_embed(const float* E, const float* P, const int* tok, const int* pos, float* x, int d, int B,
                  cudaStream_t st);
// Log-probability of each row's target id under log_softmax of the row's logits
// (src/transformer/variable.cpp:465-497 and :547-552): (x[t] - max) - log(sum exp(x - max)),
// 0 for a target outside [0, V). Row r is written to out[dst ? dst[r] : r * dst_mul + dst_add].
void launch_row_logp(const float* logits, size_t ld, int V, const int* tgt, const int* dst, int dst_mul, int dst_add,
                     float* out, int rows, cudaStream_t st);
// Scoring from per-tile log-sum-exp pairs: part[r][t] = (max, sum of exp(x - max)) over feature tile t of row r,
// tgt_logit[r] = the logit of the row's target. out[dst[r]] = (tgt_logit - M) - log(sum_t s_t exp(m_t - M)), or 0
// for a target outside [0, V).
void launch_lse_combine(const float* part, int tiles, const float* tgt_logit, const int* tgt, int V, const int* dst,
                        float* out, int rows, cudaStream_t st);
void launch_advance(const int* tok, int* pos, int* hist, int* hist_len, int hist_stride, int B, cudaStream_t st);
void launch_gemv(const GemvParams& p, int pro, int epi, bool bf16, int sm_count, cudaStream_t st);
void launch_logits(const LogitsParams& p, bool bf16, cudaStream_t st);
// Independent warps per CTA of the persistent cached-attention kernel (one CTA per SM); callers size their context
// splits by it.
constexpr int kAttnPipeWarps = 7;
void launch_attention(const AttnParams& p, int B, int splits, cudaStream_t st);
void attention_configure();
// Same kernel with its scratch in a fixed device array (no allocation); see step_kernels.cu.
void launch_attention_static(const AttnParams& p, int B, int splits, cudaStream_t st);
int static_attention_capacity();

}  // namespace gradb
