// Test support: token files, windows and batch order of `grad eval`'s data path, restated so that the CPU and GPU
// tests can feed gradb::training::mean_loss without the reference tree (which is not present where the GPU tests
// run). Checked against files, windows and picks produced by the reference's own classes
// (tests/golden/ref_tokens.bin, tokenfile_golden.npz). Not part of the product: a grad.cpp build passes its own
// grad::DataLoader to gradb::training::mean_loss.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace gradb {

// // Pre-tokenized corpus files: "TOK1", uint32 vocab size, uint64 id count, then the ids as uint16
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

}  // namespace gradb
