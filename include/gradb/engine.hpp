// C++20 drop-in classes over the C ABI (include/gradb.h).
//
// These mirror the reference's public classes for the token loop so that a caller
// of grad::InferenceSession / grad::TextGen / grad::GPTModel::load can switch by
// changing a namespace:
//   grad::GPTModel::load / save        include/grad/transformer/gpt_model.h:83-86
//   grad::InferenceSession             include/grad/transformer/inference.h:16-29
//   grad::TextGen                      include/grad/transformer/text_gen.h:12-38
//   grad::training::mean_loss          src/training/trainer.cpp:319-340 (what `grad eval` reports)
//   grad::tokenfile, MappedTokenDataset include/grad/data/token_file.h:10-70
//   grad::DataLoader                   include/grad/data/dataloader.h:23-46
// Status codes come back as the reference's exception types and messages
// (src/transformer/inference.cpp:151-156, src/transformer/gpt_model.cpp:385-387, 521-524).
//
// Header-only; link against libgradb.so.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <fstream>
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

// ---- the data path of `grad eval`: token files, windows, batch order ----------------------------
//
// Pre-tokenized corpus files: "TOK1", uint32 vocab size, uint64 id count, then the ids as uint16
// (include/grad/data/token_file.h:10-36, src/data/token_file.cpp:14-70).
namespace tokenfile {

inline void write(const std::string& path, const int* data, size_t count, int vocab_size) {
    if (vocab_size <= 0 || vocab_size > 65536) {
        throw std::invalid_argument("token file requires 0 < vocab_size <= 65536 (uint16 storage)");
    }
    std::ofstream file(path, std::ios::binary);
    if (!file.is_open()) throw std::runtime_error("Cannot open for writing: " + path);
    const uint32_t vocab = static_cast<uint32_t>(vocab_size);
    const uint64_t count64 = count;
    file.write("TOK1", 4);
    file.write(reinterpret_cast<const char*>(&vocab), sizeof(vocab));
    file.write(reinterpret_cast<const char*>(&count64), sizeof(count64));
    std::vector<uint16_t> ids(count);
    for (size_t i = 0; i < count; i++) {
        if (data[i] < 0 || data[i] >= vocab_size) {
            throw std::runtime_error("token id out of range for vocab while writing " + path);
        }
        ids[i] = static_cast<uint16_t>(data[i]);
    }
    file.write(reinterpret_cast<const char*>(ids.data()), static_cast<std::streamsize>(count * sizeof(uint16_t)));
    if (!file.good()) throw std::runtime_error("Write failed: " + path);
}
inline void write(const std::string& path, const std::vector<int>& tokens, int vocab_size) {
    write(path, tokens.data(), tokens.size(), vocab_size);
}
[[nodiscard]] inline bool exists(const std::string& path) { return std::ifstream(path, std::ios::binary).good(); }

}  // namespace tokenfile

// Windows of seq_length ids every `stride` ids over a token file; the target is the input shifted
// by one (include/grad/data/token_file.h:45-70, src/data/token_file.cpp:83-176). The file is read
// into memory once (the reference maps it); ids are checked against the header's vocab as each
// window is read, with the reference's messages.
class MappedTokenDataset {
public:
    MappedTokenDataset(const std::string& path, int seq_length, int stride = 1) {
        if (stride < 1) throw std::invalid_argument("stride must be >= 1");
        if (seq_length < 1) throw std::invalid_argument("seq_length must be >= 1");
        seq_length_ = static_cast<size_t>(seq_length);
        stride_ = static_cast<size_t>(stride);
        std::ifstream file(path, std::ios::binary | std::ios::ate);
        if (!file.is_open()) throw std::runtime_error("Cannot open token file: " + path);
        const std::streamoff size = file.tellg();
        constexpr size_t kHeaderBytes = 4 + sizeof(uint32_t) + sizeof(uint64_t);
        if (size < 0 || static_cast<size_t>(size) < kHeaderBytes) {
            throw std::runtime_error("Token file truncated or unreadable: " + path);
        }
        file.seekg(0);
        char header[kHeaderBytes];
        file.read(header, kHeaderBytes);
        if (!file.good()) throw std::runtime_error("Token file truncated or unreadable: " + path);
        if (std::memcmp(header, "TOK1", 4) != 0) throw std::runtime_error("Not a token file (bad magic): " + path);
        uint32_t vocab;
        uint64_t count;
        std::memcpy(&vocab, header + 4, sizeof(vocab));
        std::memcpy(&count, header + 4 + sizeof(vocab), sizeof(count));
        if (vocab == 0 || vocab > 65536) {
            throw std::runtime_error("Token file vocab " + std::to_string(vocab) + " outside (0, 65536]: " + path);
        }
        if (count > (static_cast<size_t>(size) - kHeaderBytes) / sizeof(uint16_t)) {
            throw std::runtime_error("Token file shorter than its header claims: " + path);
        }
        vocab_size_ = static_cast<int>(vocab);
        if (count < seq_length_ + 1) throw std::runtime_error("Not enough tokens for even one sequence: " + path);
        tokens_.resize(static_cast<size_t>(count));
        file.read(reinterpret_cast<char*>(tokens_.data()), static_cast<std::streamsize>(count * sizeof(uint16_t)));
        if (!file.good()) throw std::runtime_error("Token file truncated or unreadable: " + path);
    }

    [[nodiscard]] size_t size() const { return (tokens_.size() - seq_length_ - 1) / stride_ + 1; }

    [[nodiscard]] std::pair<std::vector<int>, std::vector<int>> get_item(size_t index) const {
        if (index >= size()) throw std::out_of_range("MappedTokenDataset index out of range");
        const size_t start = index * stride_;
        const uint16_t* window = tokens_.data() + start;
        for (size_t i = 0; i <= seq_length_; i++) {
            if (window[i] >= vocab_size_) {
                throw std::runtime_error("token id " + std::to_string(window[i]) + " at offset " +
                                         std::to_string(start + i) + " is outside the file's vocab of " +
                                         std::to_string(vocab_size_));
            }
        }
        std::vector<int> input(seq_length_), target(seq_length_);
        for (size_t i = 0; i < seq_length_; i++) {
            input[i] = window[i];
            target[i] = window[i + 1];
        }
        return {input, target};
    }

    [[nodiscard]] int vocabSize() const { return vocab_size_; }
    [[nodiscard]] size_t tokenCount() const { return tokens_.size(); }
    [[nodiscard]] int seqLength() const { return static_cast<int>(seq_length_); }

private:
    std::vector<uint16_t> tokens_;
    int vocab_size_ = 0;
    size_t seq_length_ = 0, stride_ = 0;
};

// A batch of windows: batch_size x seq_length ids each way (the reference's Batch holds the same
// ids as float tensors, include/grad/data/dataloader.h:9-15).
struct Batch {
    size_t batch_size = 0, seq_length = 0;
    std::vector<int32_t> input, target;
};

// Batch order of include/grad/data/dataloader.h:23-46 / src/data/dataloader.cpp:19-72: sequential
// batches in window order with a ragged last batch, or (shuffle) every row's window drawn uniformly
// from a std::mt19937 seeded with `seed`; the generator carries over a reset().
class DataLoader {
public:
    DataLoader(std::shared_ptr<MappedTokenDataset> dataset, int batch_size, bool shuffle = true, unsigned int seed = 42)
        : dataset_(std::move(dataset)), shuffle_(shuffle), rng_(seed) {
        if (batch_size < 1) throw std::invalid_argument("batch_size must be >= 1");
        batch_size_ = static_cast<size_t>(batch_size);
    }
    [[nodiscard]] bool has_next() const { return current_index_ < dataset_->size(); }
    [[nodiscard]] Batch next_batch() {
        if (!has_next()) throw std::runtime_error("No more batches available. Call reset() to start new epoch.");
        const size_t n = std::min(batch_size_, dataset_->size() - current_index_);
        Batch batch;
        batch.batch_size = n;
        batch.seq_length = static_cast<size_t>(dataset_->seqLength());
        std::vector<size_t> indices(n);
        if (shuffle_) {
            std::uniform_int_distribution<size_t> pick(0, dataset_->size() - 1);
            for (size_t b = 0; b < n; b++) indices[b] = pick(rng_);
        } else {
            for (size_t b = 0; b < n; b++) indices[b] = current_index_ + b;
        }
        for (size_t b = 0; b < n; b++) {
            auto [input, target] = dataset_->get_item(indices[b]);
            batch.input.insert(batch.input.end(), input.begin(), input.end());
            batch.target.insert(batch.target.end(), target.begin(), target.end());
        }
        current_index_ += n;
        return batch;
    }
    void reset() { current_index_ = 0; }
    [[nodiscard]] size_t num_batches() const { return (dataset_->size() + batch_size_ - 1) / batch_size_; }
    [[nodiscard]] size_t dataset_size() const { return dataset_->size(); }
    [[nodiscard]] const std::shared_ptr<MappedTokenDataset>& dataset() const { return dataset_; }
    [[nodiscard]] int batch_size() const { return static_cast<int>(batch_size_); }

private:
    std::shared_ptr<MappedTokenDataset> dataset_;
    size_t batch_size_ = 1;
    bool shuffle_;
    size_t current_index_ = 0;
    std::mt19937 rng_;
};

namespace training {

// grad::training::mean_loss (src/training/trainer.cpp:319-340): the loader's next max_batches
// batches (all that remain when max_batches <= 0), each scored with cross entropy averaged over its
// rows, the batch losses averaged with the batches' window counts as weights; -1 with no batches.
// All windows are scored in one device pass, resident_windows at a time; the per-batch averaging
// is done afterwards in the reference's order.
inline double mean_loss(const GPTModel& model, DataLoader& loader, int max_batches, int resident_windows = 64) {
    std::vector<int32_t> in, tg;
    size_t n = 0, seq = 0;
    for (int batches = 0; loader.has_next(); batches++) {
        if (max_batches > 0 && batches >= max_batches) break;
        Batch batch = loader.next_batch();
        in.insert(in.end(), batch.input.begin(), batch.input.end());
        tg.insert(tg.end(), batch.target.begin(), batch.target.end());
        n += batch.batch_size;
        seq = batch.seq_length;
    }
    if (n == 0) return -1.0;
    gradb_session* session = nullptr;
    const int resident = static_cast<int>(std::min<size_t>(n, static_cast<size_t>(std::max(1, resident_windows))));
    detail::check(gradb_session_create(model.handle(), resident, 0, nullptr, &session));
    double mean = -1.0;
    // Only the loader's last batch can be ragged, so cutting the concatenation every batch_size windows
    // reproduces its batches.
    const gradb_status st = gradb_mean_loss(session, in.data(), tg.data(), static_cast<int>(n), static_cast<int>(seq),
                                            loader.batch_size(), &mean, nullptr, nullptr);
    gradb_session_free(session);
    detail::check(st);
    return mean;
}

}  // namespace training

}  // namespace gradb
