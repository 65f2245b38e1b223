// C-callable wrapper around the UNMODIFIED grad.cpp decode path, for ctypes.
// TEST INFRASTRUCTURE ONLY: this file and the library built from it are the
// parity checker and the timed CPU baseline; nothing on the product path may
// link or load them.
//
// It links the reference's own GPTModel::load (src/transformer/gpt_model.cpp:383),
// InferenceSession::step (src/transformer/inference.cpp:150) and TextGen
// (src/transformer/text_gen.cpp:37-209) compiled from the reference sources
// where they lie; no reference source is copied here.
//
// Two access tricks, neither of which edits a reference file:
//  * TextGen::sample_from_logits is private (text_gen.h:18). The header is
//    included with `private` spelled `public` so the sampler can be fed chosen
//    logits directly.
//  * The sampler's RNG is a function-static mt19937 seeded once per process
//    from random_device, which the build replaces by the GRADREF_SEED
//    environment value (rd_shim.h). This wrapper keeps a mirror generator in
//    lockstep so it can report the uniform draw each call consumed. Every
//    sampler call in the process must go through this wrapper for the mirror
//    to stay aligned.

#include <algorithm>
#include <array>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <optional>
#include <random>
#include <span>
#include <sstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

#include "grad/data/dataloader.h"
#include "grad/data/token_file.h"
#include "grad/transformer/gpt_model.h"
#include "grad/transformer/inference.h"
#include "grad/tokenizer/tokenizer.h"
#define private public
#include "grad/transformer/text_gen.h"
#undef private

namespace {

// Emits ids as decimal text so TextGen's string result can be turned back
// into ids at any vocabulary size (without a tokenizer TextGen truncates each
// id to a char, text_gen.cpp:127-132).
class IdTokenizer final : public grad::Tokenizer {
public:
    explicit IdTokenizer(int vocab) : vocab_(vocab) {}
    grad::TokenizerKind kind() const override { return grad::TokenizerKind::BpeV1; }
    std::vector<int> encode(std::string_view) const override { return {}; }
    std::string decode(std::span<const int> ids) const override {
        std::string s;
        for (int id : ids) {
            s += std::to_string(id);
            s += ' ';
        }
        return s;
    }
    int vocab_size() const override { return vocab_; }
    std::optional<int> eos_id() const override { return std::nullopt; }
    std::optional<int> special_id(std::string_view) const override { return std::nullopt; }
    std::uint64_t fingerprint() const override { return 0; }
    void save(const std::string&) const override {}

private:
    int vocab_;
};

thread_local std::string g_error;

unsigned env_seed() {
    const char* s = std::getenv("GRADREF_SEED");
    return s ? static_cast<unsigned>(std::strtoul(s, nullptr, 10)) : 0u;
}

// Mirror of the reference's process-static generator (text_gen.cpp:195-196).
std::mt19937& mirror() {
    static std::mt19937 gen(env_seed());
    return gen;
}

float mirror_draw() {
    std::uniform_real_distribution<float> dis(0.0f, 1.0f);
    return dis(mirror());
}

int parse_ids(const std::string& text, int* out, int cap) {
    std::istringstream in(text);
    int n = 0, id = 0;
    while (in >> id) {
        if (n < cap) out[n] = id;
        n++;
    }
    return n;
}

struct RefModel {
    grad::GPTModel model;
    explicit RefModel(grad::GPTModel&& m) : model(std::move(m)) {}
};

}  // namespace

extern "C" {

const char* gradref_last_error() { return g_error.c_str(); }

void* gradref_model_load(const char* path) {
    try {
        return new RefModel(grad::GPTModel::load(path));
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}

// Random-init (Xavier) model straight from the reference constructor.
void* gradref_model_new(int vocab, int d_model, int layers, int heads, int max_len, int modern) {
    try {
        return new RefModel(grad::GPTModel(vocab, d_model, layers, heads, max_len, 0.0f,
                                           modern ? grad::GPTArch::Modern : grad::GPTArch::GPT2));
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}

int gradref_model_save(void* m, const char* path, int with_fingerprint, unsigned kind,
                       unsigned long long hash) {
    auto* rm = static_cast<RefModel*>(m);
    if (with_fingerprint) {
        rm->model.setTokenizerFingerprint(
            grad::TokenizerFingerprint{static_cast<grad::TokenizerKind>(kind), hash});
    }
    return rm->model.save(path, true) ? 0 : 1;
}

void gradref_model_free(void* m) { delete static_cast<RefModel*>(m); }

// dims[0..6] = vocab, d_model, layers, heads, max_len, arch, d_ff
void gradref_model_dims(void* m, int* dims) {
    const grad::GPTModel& g = static_cast<RefModel*>(m)->model;
    dims[0] = g.getVocabSize();
    dims[1] = g.getDModel();
    dims[2] = g.getNumLayers();
    dims[3] = g.getNumHeads();
    dims[4] = g.getMaxLen();
    dims[5] = static_cast<int>(g.getArch());
    dims[6] = static_cast<int>(g.getBlock(0).getFFN().getLayer1Weights()->getData().getCols());
}

void* gradref_session_new(void* m) {
    return new grad::InferenceSession(static_cast<RefModel*>(m)->model);
}
void gradref_session_free(void* s) { delete static_cast<grad::InferenceSession*>(s); }
int gradref_session_position(void* s) { return static_cast<grad::InferenceSession*>(s)->position(); }

// 0 ok; 1 = runtime_error (context overflow); 2 = out_of_range (bad token).
int gradref_session_step(void* s, int token, float* logits_out) {
    auto* sess = static_cast<grad::InferenceSession*>(s);
    try {
        const float* l = sess->step(token);
        if (logits_out) std::memcpy(logits_out, l, sizeof(float) * sess->vocabSize());
        return 0;
    } catch (const std::out_of_range& e) {
        g_error = e.what();
        return 2;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

// Returns the total number of ids in the result (prompt + generated).
int gradref_generate_greedy(void* m, const int* prompt, int n_prompt, int max_tokens,
                            float repetition_penalty, int* out, int cap) {
    const grad::GPTModel& g = static_cast<RefModel*>(m)->model;
    IdTokenizer tok(g.getVocabSize());
    grad::TextGen gen(g, &tok);
    std::vector<int> p(prompt, prompt + n_prompt);
    return parse_ids(gen.generate_greedy(p, max_tokens, repetition_penalty), out, cap);
}

// Sampled rollout; draws_out (optional, cap entries) receives the uniform
// draw consumed for each generated token, in order.
int gradref_generate_sample(void* m, const int* prompt, int n_prompt, float temperature,
                            int max_tokens, float repetition_penalty, int top_k, float top_p,
                            int* out, int cap, float* draws_out) {
    const grad::GPTModel& g = static_cast<RefModel*>(m)->model;
    IdTokenizer tok(g.getVocabSize());
    grad::TextGen gen(g, &tok);
    std::vector<int> p(prompt, prompt + n_prompt);
    const int total = parse_ids(
        gen.generate_sample(p, temperature, max_tokens, repetition_penalty, top_k, top_p), out, cap);
    const int generated = total - n_prompt;
    for (int i = 0; i < generated; i++) {
        const float u = mirror_draw();
        if (draws_out) draws_out[i] = u;
    }
    return total;
}

// generate_stream: returns the count it reports; ids of the streamed pieces
// are written to out in callback order.
int gradref_generate_stream(void* m, const int* prompt, int n_prompt, float temperature,
                            int max_tokens, float repetition_penalty, int top_k, float top_p,
                            int* out, int cap, float* draws_out) {
    const grad::GPTModel& g = static_cast<RefModel*>(m)->model;
    IdTokenizer tok(g.getVocabSize());
    grad::TextGen gen(g, &tok);
    std::vector<int> p(prompt, prompt + n_prompt);
    int n = 0;
    const int count = gen.generate_stream(
        p,
        [&](const std::string& piece) {
            int id = -1;
            parse_ids(piece, &id, 1);
            if (n < cap) out[n] = id;
            n++;
        },
        temperature, max_tokens, repetition_penalty, top_k, top_p);
    for (int i = 0; i < count; i++) {
        const float u = mirror_draw();
        if (draws_out) draws_out[i] = u;
    }
    return count;
}

// One call of the reference sampler on caller-supplied logits. *draw_out is
// the uniform value that call consumed.
int gradref_sample_from_logits(void* m, const float* logits, int vocab, float temperature,
                               int top_k, float top_p, float* draw_out) {
    const grad::GPTModel& g = static_cast<RefModel*>(m)->model;
    grad::TextGen gen(g, nullptr);
    grad::Tensor t(1, static_cast<size_t>(vocab));
    std::memcpy(t.raw(), logits, sizeof(float) * static_cast<size_t>(vocab));
    const int token = gen.sample_from_logits(t, temperature, top_k, top_p);
    const float u = mirror_draw();
    if (draw_out) *draw_out = u;
    return token;
}

}  // extern "C"

// Teacher-forced scoring through the reference's own full-sequence forward and loss operators
// (GPTModel::forward, Variable::log_softmax, Variable::cross_entropy), batched and averaged the
// way `grad eval` does it (src/training/trainer.cpp:319-340 mean_loss with the batches
// src/data/dataloader.cpp:31-66 assembles). inputs/targets: n_windows x seq_len ids.
// batch_loss_out (optional): one fp32 loss per batch; row_logp_out (optional): the log-probability
// of each row's target, n_windows x seq_len. Returns 0, or 1 with gradref_last_error() set.
extern "C" int gradref_mean_loss(void* m, const int* inputs, const int* targets, int n_windows,
                                 int seq_len, int batch_windows, double* mean_out,
                                 float* batch_loss_out, float* row_logp_out) {
    try {
        grad::GPTModel& g = static_cast<RefModel*>(m)->model;
        grad::NoGradGuard no_grad;
        const size_t S = static_cast<size_t>(seq_len);
        const size_t V = static_cast<size_t>(g.getVocabSize());
        double weighted = 0.0;
        size_t rows = 0;
        int batch_index = 0;
        for (int w0 = 0; w0 < n_windows; w0 += batch_windows, batch_index++) {
            const size_t nb = static_cast<size_t>(std::min(batch_windows, n_windows - w0));
            grad::Tensor in(nb, S, 1), tg(nb, S, 1);
            for (size_t b = 0; b < nb; b++) {
                for (size_t s = 0; s < S; s++) {
                    const size_t at = (static_cast<size_t>(w0) + b) * S + s;
                    in.setValue(b, s, 0, static_cast<float>(inputs[at]));
                    tg.setValue(b, s, 0, static_cast<float>(targets[at]));
                }
            }
            auto in_v = grad::Variable::create(in, false);
            auto tg_v = grad::Variable::create(tg, false);
            auto logits = g.forward(in_v, false);
            auto loss = logits->cross_entropy(tg_v);
            const float batch_loss = loss->getData().getValue(0, 0);
            if (batch_loss_out) batch_loss_out[batch_index] = batch_loss;
            if (row_logp_out) {
                auto logp = logits->log_softmax();
                const float* lp = logp->getData().raw();
                for (size_t r = 0; r < nb * S; r++) {
                    const int t = targets[static_cast<size_t>(w0) * S + r];
                    row_logp_out[static_cast<size_t>(w0) * S + r] =
                        (t >= 0 && static_cast<size_t>(t) < V) ? lp[r * V + static_cast<size_t>(t)] : 0.0f;
                }
            }
            weighted += static_cast<double>(batch_loss) * static_cast<double>(nb);
            rows += nb;
        }
        *mean_out = rows > 0 ? weighted / static_cast<double>(rows) : -1.0;
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

// Token files and batch assembly exactly as `grad eval` uses them: tokenfile::write
// (src/data/token_file.cpp:33-70), MappedTokenDataset (:83-176) and DataLoader (src/data/dataloader.cpp).
extern "C" int gradref_tokenfile_write(const char* path, const int* ids, unsigned long long count, int vocab) {
    try {
        grad::tokenfile::write(path, ids, static_cast<size_t>(count), vocab);
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

// Opens a token file as the reference does and reports {windows, vocab, token count}; on failure
// returns 1 and leaves the reference's message in gradref_last_error().
extern "C" int gradref_dataset_open(const char* path, int seq_length, int stride, unsigned long long* info) {
    try {
        grad::MappedTokenDataset ds(path, seq_length, stride);
        info[0] = ds.size();
        info[1] = static_cast<unsigned long long>(ds.vocabSize());
        info[2] = ds.tokenCount();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

// The windows a DataLoader hands out, batch after batch, for the first max_batches batches
// (all when <= 0). inputs/targets: up to cap_windows x seq_length ids. Returns the window count,
// or -1 with gradref_last_error() set.
extern "C" long long gradref_loader_windows(const char* path, int seq_length, int stride, int batch_size,
                                            int shuffle, unsigned seed, int max_batches, int* inputs,
                                            int* targets, long long cap_windows) {
    try {
        auto ds = std::make_shared<grad::MappedTokenDataset>(path, seq_length, stride);
        grad::DataLoader loader(ds, batch_size, shuffle != 0, seed);
        long long n = 0;
        for (int batches = 0; loader.has_next(); batches++) {
            if (max_batches > 0 && batches >= max_batches) break;
            grad::Batch batch = loader.next_batch();
            const size_t nb = batch.input.getBatchSize();
            for (size_t b = 0; b < nb; b++, n++) {
                if (n >= cap_windows) continue;
                for (int s = 0; s < seq_length; s++) {
                    inputs[n * seq_length + s] = static_cast<int>(batch.input.getValue(b, s, 0));
                    targets[n * seq_length + s] = static_cast<int>(batch.target.getValue(b, s, 0));
                }
            }
        }
        return n;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}
