/* gradb - C ABI of the B200 decode engine for grad.cpp models.
 *
 * grad.cpp has no FFI seam of its own: its boundary for this path is the C++
 * class API of its static library (InferenceSession, TextGen, GPTModel::load /
 * save) plus the GPTM checkpoint file. Each entry point below names the
 * reference interface it stands in for (paths relative to the reference
 * project root). include/gradb/engine.hpp rebuilds those C++ classes on top of
 * this ABI, translating status codes back into the reference's exceptions.
 *
 * Conventions
 *  - Every function returns a gradb_status; 0 is success. The message for the
 *    last failure on the calling thread is available from gradb_last_error().
 *  - Pointers named *_host are host memory. Nothing in these signatures is a
 *    device pointer except where the name says *_dev.
 *  - One session = one CUDA stream = one host thread at a time (the reference
 *    makes the same promise: a session owns mutable scratch).
 *  - There is no CPU fallback. Without a CUDA device every call that would
 *    compute returns GRADB_ERR_NO_DEVICE.
 */
#ifndef GRADB_H
#define GRADB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gradb_model gradb_model;
typedef struct gradb_session gradb_session;

typedef enum gradb_status {
    GRADB_OK = 0,
    /* std::runtime_error("InferenceSession: context exceeds max_len"), src/transformer/inference.cpp:151-153 */
    GRADB_ERR_CONTEXT_FULL = 1,
    /* std::out_of_range("InferenceSession: token id out of vocab range"), src/transformer/inference.cpp:154-156 */
    GRADB_ERR_BAD_TOKEN = 2,
    /* std::runtime_error("Failed to load model from <path>: ..."), src/transformer/gpt_model.cpp:521-524 */
    GRADB_ERR_CHECKPOINT = 3,
    GRADB_ERR_CUDA = 4,        /* a CUDA runtime call failed */
    GRADB_ERR_DEVICE_WAIT = 5, /* a bounded device-side wait gave up (status word set by a kernel) */
    GRADB_ERR_INVALID = 6,     /* bad argument or unsupported shape */
    GRADB_ERR_NO_DEVICE = 7,   /* no usable CUDA device */
    GRADB_ERR_IO = 8           /* file could not be opened / written */
} gradb_status;

typedef enum gradb_precision {
    GRADB_FP32 = 0, /* fp32 weights, fp32 KV cache, fp32 arithmetic: the parity mode */
    GRADB_BF16 = 1  /* bf16 weights (fp32 accumulate), fp32 KV cache */
} gradb_precision;

typedef enum gradb_arch { GRADB_ARCH_GPT2 = 0, GRADB_ARCH_MODERN = 1 } gradb_arch;

/* Hyperparameters as the checkpoint header stores them (gpt_model.cpp:305-310),
 * plus the derived FFN width (feedforward.h:24-28) and the optional tokenizer
 * fingerprint trailer (gpt_model.cpp:357-363). */
typedef struct gradb_model_desc {
    int32_t vocab_size;
    int32_t d_model;
    int32_t num_layers;
    int32_t num_heads;
    int32_t max_len;
    int32_t arch; /* gradb_arch */
    int32_t d_ff;
    float dropout_rate;
    int32_t format_version;  /* 1 or 2 as read; written files are always 2 */
    int32_t has_fingerprint; /* 0/1 */
    uint32_t fingerprint_kind;
    uint64_t fingerprint_hash;
} gradb_model_desc;

/* Selection parameters: the arguments of TextGen::generate_greedy /
 * generate_sample (include/grad/transformer/text_gen.h:23-37). */
typedef struct gradb_sampling {
    int32_t greedy;           /* 1: first-maximum argmax (text_gen.cpp:52-60); 0: sample_from_logits */
    float temperature;        /* default 1.0 */
    float repetition_penalty; /* default 1.2; applied over the last 50 ids (text_gen.cpp:14-33) */
    int32_t top_k;            /* 0 = off */
    float top_p;              /* 1.0 = off */
} gradb_sampling;

const char* gradb_last_error(void);
const char* gradb_version(void);
gradb_status gradb_device_count(int* count_out);

/* ---- checkpoint file (no GPU needed) --------------------------------- */

/* Reads and fully validates a GPTM file the way GPTModel::load does
 * (gpt_model.cpp:383-525): header ranges, every tensor's shape, truncation,
 * trailer sections. On failure the message is the reference's text. */
gradb_status gradb_checkpoint_inspect(const char* path, gradb_model_desc* desc_out);

/* Number of tensors a model of this shape stores, and the shape of each in
 * file order (gpt_model.cpp:316-353). */
gradb_status gradb_tensor_count(const gradb_model_desc* desc, int* count_out);
gradb_status gradb_tensor_shape(const gradb_model_desc* desc, int index, int* rows_out, int* cols_out);

/* Writes a version-2 GPTM file from host tensors in file order: the
 * counterpart of GPTModel::save (gpt_model.cpp:292-381), byte for byte. */
gradb_status gradb_checkpoint_write(const char* path, const gradb_model_desc* desc,
                                    const float* const* tensors_host, int n_tensors);

/* ---- model ------------------------------------------------------------ */

/* GPTModel::load (gpt_model.cpp:383) + upload: reads the file, places the
 * weights in HBM in the layouts the kernels want. */
gradb_status gradb_model_load(const char* path, int device, int precision, gradb_model** model_out);

/* Builds a device model from weights already in host memory, in file order:
 * what InferenceSession's constructor does when handed a live GPTModel
 * (inference.cpp:121-148 reads the model's tensors through its accessors). */
gradb_status gradb_model_from_host(const gradb_model_desc* desc, const float* const* tensors_host,
                                   int n_tensors, int device, int precision, gradb_model** model_out);

/* GPTModel::save (gpt_model.cpp:292): writes the fp32 master weights back out. */
gradb_status gradb_model_save(const gradb_model* model, const char* path);
gradb_status gradb_model_describe(const gradb_model* model, gradb_model_desc* desc_out);
void gradb_model_free(gradb_model* model);

/* ---- session ------------------------------------------------------------ */

/* InferenceSession::InferenceSession (inference.cpp:121-148) for max_batch
 * independent sequences: allocates their K/V caches (max_len 0 = the model's)
 * and scratch. stream: a cudaStream_t owned by the caller, or NULL to let the
 * session create one. */
gradb_status gradb_session_create(const gradb_model* model, int max_batch, int max_len, void* stream,
                                  gradb_session** session_out);
void gradb_session_free(gradb_session* session);
/* A fresh context for every sequence (what constructing a new
 * InferenceSession per generate call achieves, text_gen.cpp:42). */
gradb_status gradb_session_reset(gradb_session* session);

/* InferenceSession::position / capacity / vocabSize (inference.h:27-29). */
gradb_status gradb_session_position(const gradb_session* session, int seq, int* position_out);
int gradb_session_capacity(const gradb_session* session);
int gradb_session_vocab(const gradb_session* session);
int gradb_session_max_batch(const gradb_session* session);

/* InferenceSession::step (inference.cpp:150-258) for sequences 0..n_seq-1 at
 * once: appends tokens_host[i] to sequence i and computes its next-token
 * logits. tokens_host[i] < 0 leaves sequence i untouched. logits_host, if not
 * NULL, receives n_seq * vocab floats (a device-to-host copy and a stream
 * synchronise: meant for parity checks, not for the token loop).
 * Errors are detected on the host before any launch, as the reference does
 * before touching state. */
gradb_status gradb_step(gradb_session* session, const int32_t* tokens_host, int n_seq, float* logits_host);

/* Batched prompt feed: the reference feeds a prompt through step() one token
 * at a time (text_gen.cpp:44-46); this processes all prompt tokens of all
 * sequences together and leaves each sequence's cache, position and
 * last-position logits exactly as that loop would. offsets_host has n_seq+1
 * entries into tokens_host. logits_host (optional): n_seq * vocab. */
gradb_status gradb_prefill(gradb_session* session, const int32_t* tokens_host, const int32_t* offsets_host,
                           int n_seq, float* logits_host);

/* The selection stage of TextGen on the logits currently held on the device
 * (text_gen.cpp:14-33 penalty, :52-60 argmax, :135-209 sample_from_logits).
 * uniforms_host: one draw in [0,1) per sequence (ignored when greedy).
 * The chosen ids are appended to each sequence's id history (which the
 * penalty window reads) and returned in tokens_host. */
gradb_status gradb_select(gradb_session* session, const gradb_sampling* params, const float* uniforms_host,
                          int n_seq, int32_t* tokens_host);

/* Replaces sequence i's id history (used by the penalty window) - needed only
 * when tokens were fed with gradb_step rather than gradb_prefill/gradb_generate. */
gradb_status gradb_session_set_history(gradb_session* session, int seq, const int32_t* ids_host, int n);

/* Runs the selection stage on caller-supplied logits instead of the session's
 * (n_seq * vocab floats, host). For checking the sampler on identical logits. */
gradb_status gradb_select_from_logits(gradb_session* session, const gradb_sampling* params,
                                      const float* logits_host, const float* uniforms_host, int n_seq,
                                      int32_t* tokens_host, float* probs_host /* optional, n_seq*vocab */);

/* TextGen::generate_greedy / generate_sample (text_gen.cpp:37-91) for n_seq
 * prompts at once, ids in and ids out, the whole loop enqueued on the device
 * without a host round trip per token.
 *   prompts_host/offsets_host : concatenated prompt ids, n_seq+1 offsets
 *   max_new                   : max_tokens
 *   uniforms_host             : [n_seq][max_new] draws (NULL when greedy)
 *   out_ids_host              : [n_seq][out_stride] prompt followed by the new ids
 *   out_len_host              : [n_seq] total ids written per sequence
 *   step_ms_host (optional)   : [max_new] device time of each decode step
 *   prefill_ms_host (optional): device time of the prompt feed
 * A sequence stops after max_new ids or when its context is full; the id
 * chosen at the boundary is still emitted (text_gen.cpp:62). Resets the session first. */
gradb_status gradb_generate(gradb_session* session, const int32_t* prompts_host, const int32_t* offsets_host,
                            int n_seq, const gradb_sampling* params, int max_new,
                            const float* uniforms_host, int32_t* out_ids_host, int out_stride,
                            int32_t* out_len_host, float* step_ms_host, float* prefill_ms_host);

/* TextGen::generate_stream (text_gen.cpp:93-120): generate as gradb_generate does, handing every
 * chosen id to the caller as soon as the device has chosen it, while the forward step for that id
 * is already running. Per new id i of sequence b, in order: (sampled mode) draw(user, b) is asked
 * for the uniform in [0,1) of that id - after on_token returned for id i-1, the reference's order of
 * events (text_gen.cpp:107-116) - then the selection and the next forward step are queued, and
 * on_token(user, b, i, id) is called when the id arrives in host memory. A non-zero return from
 * on_token ends that sequence (no further ids are chosen for it, no further draws requested).
 * emitted_host (optional): [n_seq] ids handed to on_token per sequence. Resets the session first;
 * the stop rule is gradb_generate's. Callbacks run on the calling thread and must not call into
 * this session. */
typedef float (*gradb_draw_fn)(void* user, int seq);
typedef int (*gradb_token_fn)(void* user, int seq, int index, int32_t token);
gradb_status gradb_generate_stream(gradb_session* session, const int32_t* prompts_host, const int32_t* offsets_host,
                                   int n_seq, const gradb_sampling* params, int max_new, gradb_draw_fn draw,
                                   gradb_token_fn on_token, void* user, int32_t* emitted_host);

/* ---- serving: sequences that come and go ----------------------------------------------------
 * The reference builds a fresh InferenceSession and re-feeds the whole prompt on every call
 * (text_gen.cpp:42-46, 74-78, 100-104). A session here is max_batch slots that are filled,
 * decoded and vacated independently, so a batch keeps running while single sequences finish and
 * new prompts arrive. Results per slot equal an independent generate call on that prompt. */

/* Starts n_admit prompts in the slots seqs_host[i] (each slot's previous sequence ends), feeding all
 * of them in one batched prompt feed without touching the other slots. offsets_host: n_admit+1
 * entries into prompts_host; prompts must not be empty. max_new_host[i]: ids to emit at most
 * (max_tokens). uniforms_host[i]: max_new_host[i] draws for sampled decoding, or NULL (the array
 * itself may be NULL when every sequence is decoded greedily).
 * reuse_prefix != 0: positions of the slot's previous sequence that the new prompt repeats id for
 * id keep their K/V rows and only the rest of the prompt is fed (a follow-up turn of the same
 * conversation costs only its new ids). reused_host (optional): positions kept per prompt. */
gradb_status gradb_session_admit(gradb_session* session, int n_admit, const int32_t* seqs_host,
                                 const int32_t* prompts_host, const int32_t* offsets_host,
                                 const int32_t* max_new_host, const float* const* uniforms_host, int reuse_prefix,
                                 int32_t* reused_host);

/* Runs n_steps decode iterations (choose an id, feed it) for every live slot, queued on the device
 * without a host round trip. A slot finishes when it has emitted its max_new ids, when its context
 * is full (the id chosen at the boundary is still emitted, text_gen.cpp:61-63), or when it chooses
 * one of stop_ids_host (n_stop <= 8; the stop id is emitted; the reference has no such stop).
 * Finished and vacant slots take no part. out_ids_host: [max_batch][out_stride] ids chosen during
 * this call, out_count_host: [max_batch] how many, finished_host: [max_batch] 1 once a slot is done. */
gradb_status gradb_session_decode(gradb_session* session, const gradb_sampling* params, int n_steps,
                                  const int32_t* stop_ids_host, int n_stop, int32_t* out_ids_host, int out_stride,
                                  int32_t* out_count_host, int32_t* finished_host);

/* Ends the slot's sequence. Its cached positions stay available to a later gradb_session_admit
 * with reuse_prefix. */
gradb_status gradb_session_release(gradb_session* session, int seq);

/* The ids of the slot's sequence so far (prompt followed by emitted ids); returns the count in
 * count_out and copies at most capacity of them. */
gradb_status gradb_session_slot_ids(const gradb_session* session, int seq, int32_t* ids_host, int capacity,
                                    int* count_out);

/* Teacher-forced scoring, the device half of `grad eval` (src/cli/eval.cpp:77-133): n_windows
 * windows of seq_len ids each are fed from position 0 (max_batch windows at a time; the session
 * is reset first and left holding the last group) and every position's logits are reduced on the
 * device to the log-probability of that position's target,
 *   row_logp_host[w*seq_len + t] = log_softmax(logits after inputs[w][0..t])[targets[w][t]]
 * (src/transformer/variable.cpp:465-497), 0 where the target is outside [0, vocab)
 * (variable.cpp:547-552). Logits never leave the GPU. inputs must be valid ids (BAD_TOKEN),
 * seq_len <= capacity (CONTEXT_FULL). ms_out (optional): device time. */
gradb_status gradb_score(gradb_session* session, const int32_t* inputs_host, const int32_t* targets_host,
                         int n_windows, int seq_len, float* row_logp_host, float* ms_out);

/* training::mean_loss (src/training/trainer.cpp:319-340) over windows held in memory: windows are
 * taken batch_windows at a time (the reference's eval uses 8, eval.cpp:77); a batch's loss is the
 * fp32 running total of -logp over its rows, in row order, divided by the row count
 * (Variable::nll_loss, variable.cpp:544-553); the result is the window-weighted mean of the batch
 * losses accumulated in double, or -1 with no windows. batch_loss_host (optional):
 * ceil(n_windows / batch_windows) floats. */
gradb_status gradb_mean_loss(gradb_session* session, const int32_t* inputs_host, const int32_t* targets_host,
                             int n_windows, int seq_len, int batch_windows, double* mean_loss_out,
                             float* batch_loss_host, float* ms_out);

/* Device time of the most recent launches, for benchmarks: milliseconds between
 * the start and end events the session records around gradb_step / gradb_prefill /
 * gradb_generate's decode loop. */
gradb_status gradb_session_last_ms(const gradb_session* session, float* ms_out);

/* Row `pos` of layer `layer`'s K (which=0) or V (which=1) cache of sequence
 * `seq`, d_model floats in the reference's head-concatenated order
 * (inference.cpp:195-206). For parity checks of the cache contents. */
gradb_status gradb_session_cache_row(gradb_session* session, int seq, int layer, int which, int pos,
                                     float* row_host);

/* ---- single kernels ------------------------------------------------------ */

/* The cached-attention stage of one decode step on its own (inference.cpp:208-225 with
 * softmax_row :60-67), for n_seq sequences: out[s, h*64..] = softmax(q_h . K_h[0..pos] / sqrt(64)) V_h.
 * All pointers are DEVICE memory: q_dev and out_dev are [n_seq][heads*64]; the caches are
 * [n_seq][heads][max_len][64] (one layer); pos_dev[s] is the index of the newest cached
 * position of sequence s. The context is cut into `splits` ranges whose partial results are
 * combined by the last CTA to finish; the scratch for those partials is allocated and freed
 * inside the call, which therefore synchronises the stream. head_dim must be 64. */
gradb_status gradb_attention_decode(const float* q_dev, const float* kcache_dev, const float* vcache_dev,
                                    const int32_t* pos_dev, int n_seq, int heads, int head_dim, int max_len,
                                    int splits, float* out_dev, void* stream);

/* The same cached-attention kernel for callers that must not allocate. It has no counterpart
 * in the reference. Two kinds of caller need it: hosts that give a plugin a fixed device-memory
 * budget up front (a serving process that reserves all of its device memory at start), and
 * latency-critical loops that cannot afford the allocator: cudaMalloc may block for an unbounded
 * time and cudaFree synchronises the whole device, stalling every other stream of the process.
 * The split partials and arrival
 * tickets live in a fixed array of gradb_attention_static_capacity() = 4096 (sequence, head, split)
 * slots, about 1.1 MB, that every GPU loading this library holds until the process exits; a call
 * with n_seq * heads * splits above that is rejected with GRADB_ERR_INVALID and a message naming
 * the limit. The call issues no cudaMalloc, cudaFree or other allocating routine, does not
 * synchronise, and returns as soon as the work is queued on `stream`.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current); make that first call before starting any stream capture.
 *   - All calls share the array. It keeps the previous call's contents; the tickets are cleared
 *     on `stream` at the start of every call. Two calls that overlap on the GPU (different
 *     streams, or different host threads on one device) race on it: serialise them.
 * Arguments and results are those of gradb_attention_decode. */
gradb_status gradb_attention_decode_static(const float* q_dev, const float* kcache_dev, const float* vcache_dev,
                                           const int32_t* pos_dev, int n_seq, int heads, int head_dim, int max_len,
                                           int splits, float* out_dev, void* stream);
int gradb_attention_static_capacity(void);

/* Built-in device-side tracing (the reference has none for this path; its `grad bench`
 * times whole generations, src/cli/bench.cpp:269-286). While profiling is on, every kernel
 * launch is bracketed by CUDA events on the session's stream (graphs are bypassed) and the
 * elapsed time is accumulated per kernel class. Turning it on or off clears the totals. */
gradb_status gradb_session_set_profiling(gradb_session* session, int on);
int gradb_kernel_class_count(void);
const char* gradb_kernel_class_name(int kernel_class);
/* ms_out / launches_out: gradb_kernel_class_count() entries each. */
gradb_status gradb_session_profile(const gradb_session* session, double* ms_out, uint64_t* launches_out);

/* Kernels launched by this library since it was loaded (every launch through
 * its own launcher is counted). */
uint64_t gradb_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* GRADB_H */
