/* CPU restatement of grad.cpp's KV-cached token loop, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY. This is the parity checker for the CUDA path and
 * the fallback CPU baseline; it is never linked into, loaded by, or called
 * from the product library. Only tests, the smoke check and the benchmark's
 * cpu-baseline leg may use it.
 *
 * Parity status: PINNED. The reference ships no golden vectors for this path,
 * so the restatement is pinned against outputs of the reference itself,
 * compiled unmodified (oracle/_ref), on seeded inputs; the generating script
 * and the resulting fixtures live under tests/golden/.
 *
 * Every function names the reference lines it follows (paths are relative to
 * the reference project root).
 *
 * Build with -DGRO_REAL=double for a double-precision witness of the same
 * algorithm (used to tell oracle rounding from kernel error); the exported
 * names then carry the prefix gro64_ instead of gro_. */
#ifndef GRAD_DECODE_ORACLE_H
#define GRAD_DECODE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GRO_REAL
#define GRO_REAL float
#define GRO(name) gro_##name
#else
#define GRO(name) gro64_##name
#endif

typedef struct gro_model gro_model;
typedef struct gro_session gro_session;

/* Checkpoint ("GPTM") reader. Returns NULL and fills err (if given) with the
 * reference's message text on failure. src/transformer/gpt_model.cpp:383-525 */
gro_model* GRO(model_load)(const char* path, char* err, size_t err_cap);
void GRO(model_free)(gro_model* m);
/* dims[0..8] = vocab, d_model, layers, heads, max_len, arch, d_ff,
 *              has_fingerprint, fingerprint_kind */
void GRO(model_dims)(const gro_model* m, int* dims);
uint64_t GRO(model_fingerprint_hash)(const gro_model* m);

/* src/transformer/inference.cpp:121-148 */
gro_session* GRO(session_new)(const gro_model* m);
void GRO(session_free)(gro_session* s);
void GRO(session_reset)(gro_session* s);
int GRO(session_position)(const gro_session* s);
/* One decode step. 0 ok, 1 context full, 2 token out of range.
 * src/transformer/inference.cpp:150-258 */
int GRO(session_step)(gro_session* s, int token, float* logits_out);
/* Row `pos` of layer `layer`'s K (which=0) or V (which=1) cache, d_model floats. */
void GRO(session_cache_row)(const gro_session* s, int layer, int which, int pos, float* out);

#ifndef GRO_SAMPLER_DECLARED
#define GRO_SAMPLER_DECLARED
/* The selection stage works on float logits only and is shared by both builds.
 * src/transformer/text_gen.cpp:14-33 */
void gro_apply_penalty(float* logits, int vocab, const int* tokens, int n_tokens, float penalty);
/* src/transformer/text_gen.cpp:52-60 */
int gro_argmax(const float* logits, int vocab);
/* src/transformer/text_gen.cpp:135-209 with the uniform draw u supplied by
 * the caller. probs_out (optional) receives the final distribution. */
int gro_sample(const float* logits, int vocab, float temperature, int top_k, float top_p, float u,
               float* probs_out);
#endif

/* generate_greedy / generate_sample control flow, ids in and ids out.
 * Returns the total count (prompt + generated). draws: one per generated
 * token (sampled mode). src/transformer/text_gen.cpp:37-91 */
int GRO(generate)(const gro_model* m, const int* prompt, int n_prompt, int max_tokens, int greedy,
                  float temperature, float repetition_penalty, int top_k, float top_p,
                  const float* draws, int* out, int cap);

/* Teacher-forced scoring the way `grad eval` computes it. Each window of seq_len ids is fed
 * through a fresh session; row (window, position) is scored with log_softmax of that
 * position's logits at targets[row] (max-subtract, exp, sum, log: src/transformer/variable.cpp:465-497;
 * an id outside [0, vocab) contributes nothing: variable.cpp:547-552). A batch is batch_windows
 * consecutive windows; its loss is the sequential fp32 sum of -logp over its rows divided by the
 * row count (variable.cpp:544-553), and the result is the window-weighted mean of the batch losses
 * in double (src/training/trainer.cpp:319-340). The reference runs its full-sequence forward
 * and a SIMD exp here; this restatement uses the step path (which the reference's own parity test
 * ties to that forward) and libm, so agreement is to rounding, not bitwise.
 * batch_loss_out, row_logp_out: optional. Returns 0, or the session_step code. */
int GRO(mean_loss)(const gro_model* m, const int* inputs, const int* targets, int n_windows, int seq_len,
                   int batch_windows, double* mean_out, float* batch_loss_out, float* row_logp_out);

#ifdef __cplusplus
}
#endif
#endif
