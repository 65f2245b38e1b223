// Launcher of the selection-stage kernel (select_kernels.cu).
#pragma once
#include "common.cuh"

namespace gradb {

struct SelectParams {
    const float* logits;  // [B][V]
    int V;
    int n_pad;  // filled by the launcher
    int greedy;
    float temperature, penalty;
    int top_k;
    float top_p;
    const float* uniforms;  // draw of sequence b: uniforms[b*u_stride + (loop_mode ? gen[b] : 0)]
    int u_stride;
    int* hist;  // [B][hist_stride] ids fed and chosen so far
    int hist_stride;
    int* hist_len;  // [B]
    int* out_tok;   // [B] chosen id (optional)
    float* probs_out;  // [B][V] final distribution (optional, sampled mode)
    // generate loop state
    int loop_mode;
    int* gen;      // [B] ids emitted so far
    int* cur_tok;  // [B] input of the next step, or kSkip once a sequence is finished
    int* done;     // [B]
    const int* pos;
    int capacity, max_new;
};

size_t select_smem_bytes(int V, int* n_pad_out);
void configure_select(int V);
void launch_select(const SelectParams& p, int B, cudaStream_t st);

}  // namespace gradb
