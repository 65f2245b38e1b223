// Launcher of the selection-stage kernel (select_kernels.cu).
#pragma once
#include "common.cuh"

namespace gradb {

struct SelectParams {
    const float* logits;  // [B][V]
    int V;
    int n_pad;  // filled by the launcher: floats of the shared-memory array
    int n_sort;             // filled by the launcher: power of two >= V (area of the fallback sort)
    float* scratch;         // [B][select_scratch_floats(V)] global scratch rows (sampled mode)
    size_t scratch_stride;  // filled by the launcher
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
    const int* max_new_seq;  // optional [B]: per-sequence limit on emitted ids instead of max_new
    int n_stop;              // ids that end a sequence when chosen (the id is still emitted); the reference has none
    int stop_ids[8];
    // optional, generate loop only: mapped host memory [B][stream_stride]; the id chosen as a sequence's g-th new id
    // is published at [b][g] as id + 1 (0 = not yet), so the host can hand it on while the loop runs ahead
    int* stream_ids;
    int stream_stride;
    int* status;  // session status word (index checks of the diagnostics build)
};

size_t select_smem_bytes(int V, int* n_pad_out);
size_t select_scratch_floats(int V);
// Sampled selection keeps one sequence's values and their sorted copy in one CTA's shared memory.
bool select_sampled_fits(int V);
void configure_select(int V);
#if GRADB_DIAG
void select_clocks_read(unsigned long long* out16, bool reset);  // diagnostics build: per-part clocks of the sampled kernel
#endif
void launch_select(const SelectParams& p, int B, cudaStream_t st);

}  // namespace gradb
