// C++20 drop-in classes over the C ABI (include/gradb.h).
//
// These mirror the reference's public classes for the token loop so that a caller
// of grad::InferenceSession / grad::TextGen / grad::GPTModel::load can switch by
// changing a namespace:
//   grad::GPTModel::load / save        include/grad/transformer/gpt_model.h:83-86
//   grad::InferenceSession             include/grad/transformer/inference.h:16-29
//   grad::TextGen                      include/grad/transformer/text_gen.h:12-38
//   grad::training::mean_loss          src/training/trainer.cpp:319-340 (what `grad eval` reports)
// Status codes come back as the reference's exception types and messages
// (src/transformer/inference.cpp:151-156, src/transformer/gpt_model.cpp:385-387, 521-524).
//
// Header-only; link against libgradb.so.
#pragma once

#include <algorithm>
#include <functional>
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
    // Calls on_text with each new token's text; returns how many were generated.
    int generate_stream(const std::vector<int>& prompt_tokens, const std::function<void(const std::string&)>& on_text,
                        float temperature = 1.0f, int max_tokens = 50, float repetition_penalty = 1.2f, int top_k = 0,
                        float top_p = 1.0f) {
        const std::vector<int> ids =
            sample_ids(prompt_tokens, temperature, max_tokens, repetition_penalty, top_k, top_p);
        int n = 0;
        for (size_t i = prompt_tokens.size(); i < ids.size(); i++, n++) on_text(to_string({ids[i]}));
        return n;
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
        std::vector<float> u(static_cast<size_t>(std::max(max_tokens, 0)));
        std::uniform_real_distribution<float> dis(0.0f, 1.0f);
        for (float& v : u) v = dis(generator());
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
        std::vector<int32_t> p32(prompt.begin(), prompt.end());
        for (int32_t t : p32) {
            if (t < 0) throw std::out_of_range("InferenceSession: token id out of vocab range");
        }
        detail::check(gradb_generate(session_, p32.data(), offsets, 1, &sp, max_tokens, u, out.data(), stride, &len,
                                     nullptr, nullptr));
        return std::vector<int>(out.begin(), out.begin() + len);
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

// Scoring windows over an id stream held in memory: window i covers ids [i*stride, i*stride + seq_length],
// its targets are its inputs shifted by one, and there are (count - seq_length - 1) / stride + 1 of them,
// as the reference's token-file dataset cuts them (src/data/token_file.cpp:149-176). `grad eval` uses
// stride = seq_length (src/cli/eval.cpp:78-79).
class TokenWindows {
public:
    TokenWindows(std::span<const int> stream, int seq_length, int stride)
        : stream_(stream), seq_(seq_length), stride_(stride) {
        if (stride < 1) throw std::invalid_argument("stride must be >= 1");
        if (seq_length < 1) throw std::invalid_argument("seq_length must be >= 1");
        if (stream.size() < static_cast<size_t>(seq_length) + 1) {
            throw std::runtime_error("Not enough tokens for even one sequence");
        }
    }
    [[nodiscard]] size_t size() const {
        return (stream_.size() - static_cast<size_t>(seq_) - 1) / static_cast<size_t>(stride_) + 1;
    }
    [[nodiscard]] int seq_length() const { return seq_; }
    [[nodiscard]] const int* window(size_t index) const { return stream_.data() + index * static_cast<size_t>(stride_); }

private:
    std::span<const int> stream_;
    int seq_, stride_;
};

namespace training {

// Mean loss over the first max_batches batches of batch_size windows (all of them when max_batches <= 0),
// in window order: what grad::training::mean_loss returns for an unshuffled loader
// (src/training/trainer.cpp:319-340; batches as src/data/dataloader.cpp:31-66 assembles them, the
// last one ragged). -1 when there is nothing to score. Windows are scored resident_windows at a time.
inline double mean_loss(const GPTModel& model, const TokenWindows& windows, int max_batches = 0, int batch_size = 8,
                        int resident_windows = 64) {
    size_t n = windows.size();
    if (max_batches > 0) n = std::min(n, static_cast<size_t>(max_batches) * static_cast<size_t>(batch_size));
    if (n == 0) return -1.0;
    const size_t S = static_cast<size_t>(windows.seq_length());
    if (windows.seq_length() > model.getMaxLen()) {
        throw std::runtime_error("seq length exceeds the model's context (" + std::to_string(model.getMaxLen()) + ")");
    }
    std::vector<int32_t> in(n * S), tg(n * S);
    for (size_t w = 0; w < n; w++) {
        const int* ids = windows.window(w);
        for (size_t t = 0; t < S; t++) {
            in[w * S + t] = ids[t];
            tg[w * S + t] = ids[t + 1];
        }
    }
    gradb_session* session = nullptr;
    const int resident = static_cast<int>(std::min<size_t>(n, static_cast<size_t>(std::max(1, resident_windows))));
    detail::check(gradb_session_create(model.handle(), resident, 0, nullptr, &session));
    double mean = -1.0;
    const gradb_status st = gradb_mean_loss(session, in.data(), tg.data(), static_cast<int>(n), windows.seq_length(),
                                            batch_size, &mean, nullptr, nullptr);
    gradb_session_free(session);
    detail::check(st);
    return mean;
}

}  // namespace training

}  // namespace gradb
