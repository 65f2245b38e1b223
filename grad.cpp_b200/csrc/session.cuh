// Decode session: KV caches, scratch and the per-token launch sequence for a
// batch of independent sequences (InferenceSession, inference.h:16-57, widened
// to many sequences; TextGen's loops, text_gen.cpp:37-120).
#pragma once
#include "common.cuh"
#include "decode_b1.cuh"
#include "gemm_tc.cuh"
#include "select_kernels.cuh"
#include "step_kernels.cuh"

namespace gradb {

enum KernelClass { KC_EMBED = 0, KC_QKV, KC_ATTN, KC_OPROJ, KC_FFN_UP, KC_FFN_DOWN, KC_LOGITS, KC_ADVANCE, KC_SELECT,
                   KC_STEP_B1, KC_SCORE, kKernelClasses };

struct Session {
    const DeviceModel* m = nullptr;
    int B = 0;  // max_batch
    int T = 0;  // capacity (max_len)
    int V = 0, d = 0, H = 0, hs = 0, dff = 0, L = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int attn_splits = 1;
    int hist_stride = 0;

    // device buffers
    float *x = nullptr, *q = nullptr, *attn = nullptr, *ffn = nullptr, *logits = nullptr;
    float *kcache = nullptr, *vcache = nullptr;  // [L][B][H][T][hs]
    float* attn_partial = nullptr;
    int* attn_counters = nullptr;
    int *tok = nullptr, *pos = nullptr, *hist = nullptr, *hist_len = nullptr;
    int *gen = nullptr, *done = nullptr, *out_tok = nullptr;
    int* tok_matrix = nullptr;  // prompt feed: [steps][2][B] (token rows, logits-mask rows)
    size_t tok_matrix_cap = 0;
    int* pin_tokmat = nullptr;  // its pinned host staging
    size_t pin_tokmat_cap = 0;
    float* uniforms = nullptr;
    size_t uniforms_cap = 0;
    float* probs = nullptr;  // [B][V], allocated on first use
    float* select_scratch = nullptr;  // sampled selection: [B][select_scratch_floats(V)], allocated on first use

    // tensor-core path: bf16 activations (GEMM B operands), their TMA descriptors, device status word
    bool use_tc = false;
    bool use_pdl = true;  // programmatic dependent launch between the kernels of a tensor-core step
    __nv_bfloat16 *h16 = nullptr, *attn16 = nullptr, *ffn16 = nullptr;
    CUtensorMap map_h16[3], map_attn16[3], map_ffn16[3];  // token tiles of 32, 64, 128 rows
    // fp32 mode on the tensor cores: the same operands as TF32 hi/lo pairs [2][rows][width]; the maps of h16 /
    // attn16 / ffn16 above then describe these buffers.
    bool use_tc32 = false;
    float *hS = nullptr, *attnS = nullptr, *ffnS = nullptr;
    int split_rows = 0;  // rows of one half
    int* status = nullptr;
    bool use_tc_attn = false;  // prompt attention on tcgen05 (bf16 sessions, head size 64)
    CUtensorMap map_kcache;    // fp32 map over the whole K cache as rows of 64 floats
    CUtensorMap map_vcache;    // the same over the V cache, swizzled in 32-byte units (MN-major operand of the P V product)

    // batched prompt feed (one row per prompt token, all positions of a chunk at once)
    struct Feed {
        int cap = 0;  // rows per chunk
        float *x = nullptr, *q = nullptr, *attn = nullptr;
        __nv_bfloat16 *h16 = nullptr, *attn16 = nullptr, *ffn16 = nullptr;
        float *hS = nullptr, *attnS = nullptr, *ffnS = nullptr;  // fp32 sessions: TF32 hi/lo pairs [2][cap][width]
        int *row_tok = nullptr, *row_pos = nullptr, *row_seq = nullptr, *row_last = nullptr, *seq_count = nullptr,
            *last_tok = nullptr;
        CUtensorMap map_h16[3], map_attn16[3], map_ffn16[3];
        CUtensorMap map_q;  // fp32 map over the query rows (tensor-core prompt attention)
        int* pin = nullptr;  // pinned host staging of a pass: row tables, counts, scoring targets, tiles
        // teacher-forced scoring: all-row logits of a chunk, per-row target and destination
        int4* tiles = nullptr;  // query tiles of the current chunk (prompt attention)
        std::vector<int4> h_tiles;
        float* score_logits = nullptr;
        float *lse_part = nullptr, *lse_tgt = nullptr;  // fused scoring: per-tile (max, sum) pairs, target logits
        int *row_tgt = nullptr, *row_dst = nullptr;
    } feed;
    float* score_out = nullptr;  // [B * T] target log-probabilities of the windows being scored
    int* score_tgt = nullptr;    // [T][B] targets, position by position (step-by-step scoring)

    // single-sequence persistent kernel: workspace and grid-barrier words
    bool use_b1 = false;
    uint8_t* b1_ws = nullptr;  // marked exchange words, fixed-point accumulators, step counters (decode_b1.cuh)
    size_t b1_ws_bytes = 0;
    unsigned long long* b1_trace = nullptr;  // stage timestamps when GRADB_B1_TRACE=1

    // diagnostics build: spin limit and left-out tile of the attention kernel's wait (see AttnParams)
    uint32_t diag_spin_limit = 0;
    int diag_skip_tile = -1;

    // host mirrors / staging (pinned)
    std::vector<int> h_pos;
    int* h_stage = nullptr;  // pinned, >= 4*B ints
    float last_ms = 0.f;
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
    std::vector<cudaEvent_t> step_events;

    // streaming generation: host-mapped ring of chosen ids and host-written draws
    int* stream_ring = nullptr;   // pinned, mapped: [B][stream_cap]
    float* stream_u = nullptr;    // pinned, mapped: [B][stream_cap]
    size_t stream_cap = 0;

    // serving (slots admitted and decoded independently): per-slot id lists as the host knows them, per-slot
    // limits and draws on the device
    std::vector<std::vector<int>> h_ids;  // ids fed to or chosen for each slot, in order
    std::vector<char> h_live;             // admitted and not yet finished
    std::vector<int> h_gen;               // new ids emitted since admission
    int* max_new_seq = nullptr;           // device [B]
    float* serve_u = nullptr;             // device [B][T + 2] draws, indexed by the slot's emitted-id count
    cudaGraphExec_t serve_graph = nullptr;
    gradb_sampling serve_params{};
    int serve_rows = -1, serve_n_stop = -1, serve_stop[8] = {};

    // decode-step graph (select + step), rebuilt when its parameters change
    cudaGraphExec_t graph = nullptr;
    gradb_sampling graph_params{};
    int graph_nseq = -1, graph_max_new = -1, graph_u_stride = -1;
    bool use_graph = true;

    // Optional per-kernel-class device timing (events around every launch; graphs off).
    bool profiling = false;
    struct Span { int cls; cudaEvent_t a, b; };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> event_pool;
    double class_ms[kKernelClasses] = {};
    uint64_t class_launches[kKernelClasses] = {};
};

Session* create_session(const DeviceModel* m, int max_batch, int max_len, void* stream);
void destroy_session(Session* s);
void reset_session(Session* s);
void session_step(Session* s, const int32_t* tokens, int n_seq, float* logits_host);
void session_prefill(Session* s, const int32_t* tokens, const int32_t* offsets, int n_seq, float* logits_host);
void session_select(Session* s, const gradb_sampling& sp, const float* logits_host, const float* uniforms,
                    int n_seq, int32_t* tokens_out, float* probs_host);
void session_set_history(Session* s, int seq, const int32_t* ids, int n);
void session_generate(Session* s, const int32_t* prompts, const int32_t* offsets, int n_seq,
                      const gradb_sampling& sp, int max_new, const float* uniforms, int32_t* out_ids,
                      int out_stride, int32_t* out_len, float* step_ms, float* prefill_ms);
// generate with every chosen id handed to `on_token` as soon as it exists (TextGen::generate_stream,
// text_gen.cpp:93-120); draws are requested one per sampled id, right before it is needed.
void session_generate_stream(Session* s, const int32_t* prompts, const int32_t* offsets, int n_seq,
                             const gradb_sampling& sp, int max_new, gradb_draw_fn draw, gradb_token_fn on_token,
                             void* user, int32_t* emitted);
// Serving: slots are admitted, decoded and released independently of one another.
void session_admit(Session* s, int n_admit, const int32_t* seqs, const int32_t* prompts, const int32_t* offsets,
                   const int32_t* max_new, const float* const* uniforms, int reuse_prefix, int32_t* reused_out);
void session_decode(Session* s, const gradb_sampling& sp, int n_steps, const int32_t* stop_ids, int n_stop,
                    int32_t* out_ids, int out_stride, int32_t* out_count, int32_t* finished);
void session_release(Session* s, int seq);
int session_slot_ids(const Session* s, int seq, int32_t* ids_out, int capacity);
// Teacher-forced scoring of n_windows windows of seq_len ids (any n_windows; scored max_batch at a
// time from position 0): row_logp_host[w * seq_len + t] = log-probability of targets[w][t] after
// inputs[w][0..t]. Returns the device time in ms.
float session_score(Session* s, const int32_t* inputs, const int32_t* targets, int n_windows, int seq_len,
                    float* row_logp_host);
void session_set_profiling(Session* s, bool on);
void session_cache_row(Session* s, int seq, int layer, int which, int pos, float* row_host);

}  // namespace gradb
