// C++20 drop-in classes over the C ABI (include/gradb.h).
//
// These mirror the reference's public classes for the token loop so that a caller
// of grad::InferenceSession / grad::TextGen / grad::GPTModel::load can switch by
// changing a namespace:
//   grad::GPTModel::load / save        include/grad/transformer/gpt_model.h:83-86
//   grad::InferenceSession             include/grad/transformer/inference.h:16-29
//   grad::TextGen                      include/grad/transformer/text_gen.h:12-38
//   grad::training::mean_loss          src/training/trainer.cpp:319-340 (what `grad eval` reports), as a
//                                      template over the loader, so grad.cpp's own DataLoader feeds it
// Status codes come back as the reference's exception types and messages
// (src/transformer/inference.cpp:151-156, src/transformer/gpt_model.cpp:385-387, 521-524).
//
// Header-only; link against libgradb.so.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <exception>
#include <functional>
#include <memory>
#include <random>
#include <span>
#include <stdexcept>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

#include "../gradb.h"

namespace gradb {

enum class GPTArch { GPT2 = 0, Modern = 1 };

namespace detail {
[[noreturn]] inline void raise(gradb_status st) {
    const std::string msg = gradb_last_error();
    switch (st) {
        case GRADB_ERR_BAD_TOKEN: throw std::out_of_range(msg);
        default: throw std::runtime_error(msg);
    }
}
inline void check(gradb_status st) {
    if (st != GRADB_OK) raise(st);
}
}  // namespace detail

// Owns the device copy of one checkpoint.
class GPTModel {
public:
    // Throws std::runtime_error("Failed to load model from <path>: ...") like the reference.
    [[nodiscard]] static GPTModel load(const std::string& filepath, int device = 0,
                                       gradb_precision precision = GRADB_FP32) {
        gradb_model* m = nullptr;
        detail::check(gradb_model_load(filepath.c_str(), device, precision, &m));
        return GPTModel(m);
    }
    [[nodiscard]] bool save(const std::string& filepath) const { return gradb_model_save(model_, filepath.c_str()) == GRADB_OK; }

    int getVocabSize() const { return desc_.vocab_size; }
    int getDModel() const { return desc_.d_model; }
    int getNumLayers() const { return desc_.num_layers; }
    int getNumHeads() const { return desc_.num_heads; }
    int getMaxLen() const { return desc_.max_len; }
    GPTArch getArch() const { return static_cast<GPTArch>(desc_.arch); }
    const gradb_model_desc& desc() const { return desc_; }
    const gradb_model* handle() const { return model_; }

    GPTModel(const GPTModel&) = delete;
    GPTModel& operator=(const GPTModel&) = delete;
    GPTModel(GPTModel&& o) noexcept : model_(std::exchange(o.model_, nullptr)), desc_(o.desc_) {}
    GPTModel& operator=(GPTModel&& o) noexcept {
        if (this != &o) {
            gradb_model_free(model_);
            model_ = std::exchange(o.model_, nullptr);
            desc_ = o.desc_;
        }
        return *this;
    }
    ~GPTModel() { gradb_model_free(model_); }

private:
    explicit GPTModel(gradb_model* m) : model_(m) { detail::check(gradb_model_describe(m, &desc_)); }
    gradb_model* model_ = nullptr;
    gradb_model_desc desc_{};
};

// One sequence decoded a token at a time against its KV cache.
class InferenceSession {
public:
    explicit InferenceSession(const GPTModel& model) : logits_(static_cast<size_t>(model.getVocabSize())) {
        detail::check(gradb_session_create(model.handle(), 1, 0, nullptr, &session_));
    }
    ~InferenceSession() { gradb_session_free(session_); }
    InferenceSession(const InferenceSession&) = delete;
    InferenceSession& operator=(const InferenceSession&) = delete;

    // Appends token_id and returns vocab_size logits, valid until the next step().
    // Throws std::runtime_error when the context is full, std::out_of_range for a bad id.
    [[nodiscard]] const float* step(int token_id) {
        const int32_t t = token_id;
        // The ABI treats negative ids as "skip"; the reference rejects them.
        if (token_id < 0) throw std::out_of_range("InferenceSession: token id out of vocab range");
        detail::check(gradb_step(session_, &t, 1, logits_.data()));
        return logits_.data();
    }
    int position() const {
        int p = 0;
        detail::check(gradb_session_position(session_, 0, &p));
        return p;
    }
    int capacity() const { return gradb_session_capacity(session_); }
    int vocabSize() const { return gradb_session_vocab(session_); }

private:
    gradb_session* session_ = nullptr;
    std::vector<float> logits_;
};

// The part of the reference's Tokenizer interface that generation uses
// (include/grad/tokenizer/tokenizer.h:27).
class TokenDecoder {
public:
    virtual ~TokenDecoder() = default;
    [[nodiscard]] virtual std::string decode(std::span<const int> ids) const = 0;
};

class TextGen {
public:
    // Without a decoder each id is emitted as the byte it equals (text_gen.cpp:127-132).
    explicit TextGen(const GPTModel& model, const TokenDecoder* decoder = nullptr) : decoder_(decoder) {
        detail::check(gradb_session_create(model.handle(), 1, 0, nullptr, &session_));
    }
    ~TextGen() { gradb_session_free(session_); }
    TextGen(const TextGen&) = delete;
    TextGen& operator=(const TextGen&) = delete;

    std::string generate_greedy(const std::vector<int>& prompt_tokens, int max_tokens = 50,
                                float repetition_penalty = 1.2f) {
        return to_string(greedy_ids(prompt_tokens, max_tokens, repetition_penalty));
    }
    std::string generate_sample(const std::vector<int>& prompt_tokens, float temperature = 1.0f, int max_tokens = 50,
                                float repetition_penalty = 1.2f, int top_k = 0, float top_p = 1.0f) {
        return to_string(sample_ids(prompt_tokens, temperature, max_tokens, repetition_penalty, top_k, top_p));
    }
    // Calls on_text with each new token's text as soon as the device has chosen it (the forward step for that id is
    // already running); returns how many were generated. One draw is taken from the generator per id, after on_text
    // returned for the previous one, as in the reference (text_gen.cpp:107-116). An exception thrown by on_text ends
    // the generation and is rethrown here.
    int generate_stream(const std::vector<int>& prompt_tokens, const std::function<void(const std::string&)>& on_text,
                        float temperature = 1.0f, int max_tokens = 50, float repetition_penalty = 1.2f, int top_k = 0,
                        float top_p = 1.0f) {
        if (prompt_tokens.empty()) return 0;
        struct Ctx {
            TextGen* self;
            const std::function<void(const std::string&)>* on_text;
            std::uniform_real_distribution<float> dis{0.0f, 1.0f};
            std::exception_ptr error;
        } ctx{this, &on_text, {}, nullptr};
        const gradb_sampling sp{0, temperature, repetition_penalty, top_k, top_p};
        const std::vector<int32_t> p32 = checked_ids(prompt_tokens);
        const int32_t offsets[2] = {0, static_cast<int32_t>(p32.size())};
        int32_t emitted = 0;
        const gradb_status st = gradb_generate_stream(
            session_, p32.data(), offsets, 1, &sp, max_tokens,
            [](void* user, int) { return static_cast<Ctx*>(user)->dis(generator()); },
            [](void* user, int, int, int32_t token) {
                Ctx* c = static_cast<Ctx*>(user);
                try {
                    (*c->on_text)(c->self->to_string({static_cast<int>(token)}));
                    return 0;
                } catch (...) {  // must not unwind through the C frames
                    c->error = std::current_exception();
                    return 1;
                }
            },
            &ctx, &emitted);
        if (ctx.error) std::rethrow_exception(ctx.error);
        detail::check(st);
        return emitted;
    }

    // Id-level variants (prompt followed by the new ids).
    std::vector<int> greedy_ids(const std::vector<int>& prompt, int max_tokens, float repetition_penalty) {
        const gradb_sampling sp{1, 1.0f, repetition_penalty, 0, 1.0f};
        return run(prompt, sp, max_tokens, nullptr);
    }
    std::vector<int> sample_ids(const std::vector<int>& prompt, float temperature, int max_tokens,
                                float repetition_penalty, int top_k, float top_p) {
        // Same draw as the reference: one uniform_real_distribution<float>(0,1) sample of a process-wide
        // mt19937 per generated token (text_gen.cpp:195-199).
        // Exactly as many draws as ids will be emitted (the loop ends early when the context fills,
        // text_gen.cpp:61-63), so the generator is left where the reference would leave it.
        const int room = gradb_session_capacity(session_) - static_cast<int>(prompt.size()) + 1;
        const int emit = prompt.empty() ? 0 : std::max(0, std::min(max_tokens, room));
        std::vector<float> u(static_cast<size_t>(std::max(max_tokens, 1)), 0.0f);
        std::uniform_real_distribution<float> dis(0.0f, 1.0f);
        for (int i = 0; i < emit; i++) u[static_cast<size_t>(i)] = dis(generator());
        const gradb_sampling sp{0, temperature, repetition_penalty, top_k, top_p};
        return run(prompt, sp, max_tokens, u.data());
    }

    // The reference seeds its generator from std::random_device; tests may pin it.
    static void seed(unsigned value) { generator().seed(value); }

private:
    static std::mt19937& generator() {
        static std::random_device rd;
        static std::mt19937 gen(rd());
        return gen;
    }
    std::vector<int> run(const std::vector<int>& prompt, const gradb_sampling& sp, int max_tokens, const float* u) {
        if (prompt.empty()) return {};
        const int32_t offsets[2] = {0, static_cast<int32_t>(prompt.size())};
        const int stride = static_cast<int>(prompt.size()) + std::max(max_tokens, 0) + 1;
        std::vector<int32_t> out(static_cast<size_t>(stride));
        int32_t len = 0;
        const std::vector<int32_t> p32 = checked_ids(prompt);
        detail::check(gradb_generate(session_, p32.data(), offsets, 1, &sp, max_tokens, u, out.data(), stride, &len,
                                     nullptr, nullptr));
        return std::vector<int>(out.begin(), out.begin() + len);
    }
    // The ABI treats negative ids as "skip"; the reference rejects them.
    static std::vector<int32_t> checked_ids(const std::vector<int>& ids) {
        std::vector<int32_t> out(ids.begin(), ids.end());
        for (int32_t t : out) {
            if (t < 0) throw std::out_of_range("InferenceSession: token id out of vocab range");
        }
        return out;
    }
    std::string to_string(const std::vector<int>& ids) const {
        if (decoder_ != nullptr) return decoder_->decode(ids);
        std::string s;
        s.reserve(ids.size());
        for (int id : ids) s += static_cast<char>(id);
        return s;
    }
    gradb_session* session_ = nullptr;
    const TokenDecoder* decoder_;
};

namespace training {

// How mean_loss reads one batch of a loader: appends the batch's input and target ids (row-major, rows x seq) and
// reports its shape. The default suits batches that hold integer id vectors (`input`, `target`, `batch_size`,
// `seq_length`); a grad.cpp build specialises it for grad::Batch, whose ids sit in float tensors
// (include/grad/data/dataloader.h:9-15).
template <typename BatchT>
struct BatchIds {
    static void append(const BatchT& batch, std::vector<int32_t>& in, std::vector<int32_t>& tg, size_t& rows,
                       size_t& seq) {
        in.insert(in.end(), batch.input.begin(), batch.input.end());
        tg.insert(tg.end(), batch.target.begin(), batch.target.end());
        rows = batch.batch_size;
        seq = batch.seq_length;
    }
};

// grad::training::mean_loss (src/training/trainer.cpp:319-340) over any loader with the reference DataLoader's
// has_next() / next_batch() / batch_size(): the loader's next max_batches batches (all that remain when
// max_batches <= 0), each scored with cross entropy averaged over its rows, the batch losses averaged with the
// batches' window counts as weights, accumulated in double in batch order; -1 with no batches.
// Batches are read and scored a bounded number at a time (about resident_windows windows on the device and in
// host memory), so a validation file of any length streams through.
template <typename Loader>
double mean_loss(const GPTModel& model, Loader& loader, int max_batches, int resident_windows = 64) {
    const size_t batch_size = static_cast<size_t>(std::max(1, loader.batch_size()));
    const size_t per_pass = std::max<size_t>(1, static_cast<size_t>(std::max(1, resident_windows)) / batch_size);
    gradb_session* session = nullptr;
    struct Closer {
        gradb_session*& s;
        ~Closer() { gradb_session_free(s); }
    } closer{session};
    std::vector<int32_t> in, tg;
    std::vector<float> losses;
    std::vector<size_t> rows_of;
    double weighted_loss = 0.0;
    size_t rows_total = 0, seq = 0;
    int batches = 0;
    bool more = true;
    while (more) {
        in.clear();
        tg.clear();
        rows_of.clear();
        size_t n = 0;
        while (rows_of.size() < per_pass) {
            if (!loader.has_next() || (max_batches > 0 && batches >= max_batches)) {
                more = false;
                break;
            }
            auto batch = loader.next_batch();
            size_t rows = 0;
            BatchIds<decltype(batch)>::append(batch, in, tg, rows, seq);
            rows_of.push_back(rows);
            n += rows;
            batches++;
        }
        if (n == 0) break;
        if (session == nullptr) {
            const int resident = static_cast<int>(std::max(batch_size, std::min(per_pass * batch_size, n)));
            detail::check(gradb_session_create(model.handle(), resident, 0, nullptr, &session));
        }
        // Only a loader's last batch can be ragged, so cutting the concatenation every batch_size windows
        // reproduces its batches.
        losses.assign(rows_of.size(), 0.0f);
        double unused = 0.0;
        detail::check(gradb_mean_loss(session, in.data(), tg.data(), static_cast<int>(n), static_cast<int>(seq),
                                      static_cast<int>(batch_size), &unused, losses.data(), nullptr));
        for (size_t i = 0; i < rows_of.size(); i++) {
            weighted_loss += static_cast<double>(losses[i]) * static_cast<double>(rows_of[i]);
            rows_total += rows_of[i];
        }
    }
    return rows_total > 0 ? weighted_loss / static_cast<double>(rows_total) : -1.0;
}

}  // namespace training

}  // namespace gradb
