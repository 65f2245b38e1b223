// `--device b200` for grad.cpp's command-line tools: the pieces a grad.cpp checkout adds beside src/cli/ to run
// its token loop (generate, chat, bench's generation section) and its scoring loop (eval) on the B200 engine.
// Compiles against the grad.cpp tree (include/, src/cli/) and include/gradb/engine.hpp; links libgradb.so.
//
//   add_device_option / apply_device   stand in for src/cli/common.cpp:129-147 (which knows cpu|metal)
//   Generator                          stands in for grad::TextGen at its four call sites
//                                      (src/cli/generate.cpp:86-100, chat.cpp:41-61, bench.cpp:271-277)
//   run_generate / run_chat / run_eval / run_bench
//                                      the commands of src/cli/{generate,chat,eval,bench}.cpp with the device switch
#pragma once

#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "cli/args.h"
#include "commands.h"
#include "common.h"
#include "grad/data/dataloader.h"
#include "grad/tokenizer/tokenizer.h"
#include "grad/transformer/gpt_model.h"
#include "grad/transformer/text_gen.h"

#include "gradb/engine.hpp"

// grad::Batch keeps its ids as floats in (batch, seq, 1) tensors (include/grad/data/dataloader.h:9-15).
template <>
struct gradb::training::BatchIds<grad::Batch> {
    static void append(const grad::Batch& batch, std::vector<int32_t>& in, std::vector<int32_t>& tg, size_t& rows,
                       size_t& seq) {
        rows = batch.input.getBatchSize();
        seq = batch.input.getRows();
        for (size_t b = 0; b < rows; b++) {
            for (size_t s = 0; s < seq; s++) {
                in.push_back(static_cast<int32_t>(batch.input.getValue(b, s, 0)));
                tg.push_back(static_cast<int32_t>(batch.target.getValue(b, s, 0)));
            }
        }
    }
};

namespace grad::cli::b200 {

// What --device selected. `b200` runs fp32 (the parity mode), `b200-bf16` bf16 weights; `:N` picks the GPU.
struct DeviceChoice {
    bool b200 = false;
    int index = 0;
    gradb_precision precision = GRADB_FP32;
};

// nullopt when the flag does not name the B200 engine; throws UsageError for a malformed b200 value.
[[nodiscard]] std::optional<DeviceChoice> parse_device(const std::string& flag);

// Declares --device cpu|metal|b200[-bf16][:N] on cmd.
void add_device_option(Command& cmd, std::optional<std::string>& flag);
// B200: checks that a device is there and returns the choice; anything else goes to grad::cli::apply_device.
[[nodiscard]] DeviceChoice apply_device(const std::optional<std::string>& flag);

// grad::Tokenizer::decode as the engine's decoder interface.
class TokenizerDecoder final : public gradb::TokenDecoder {
public:
    explicit TokenizerDecoder(const Tokenizer* tokenizer) : tokenizer_(tokenizer) {}
    [[nodiscard]] std::string decode(std::span<const int> ids) const override { return tokenizer_->decode(ids); }

private:
    const Tokenizer* tokenizer_;
};

// TextGen's three calls (include/grad/transformer/text_gen.h:23-37) on the engine --device chose. The B200 engine
// reads the checkpoint file itself; the CPU engine uses the loaded host model, as before.
class Generator {
public:
    Generator(const DeviceChoice& device, const std::string& checkpoint_path, const GPTModel& host_model,
              const Tokenizer* tokenizer);
    std::string generate_greedy(const std::vector<int>& prompt, int max_tokens, float repetition_penalty);
    std::string generate_sample(const std::vector<int>& prompt, float temperature, int max_tokens,
                                float repetition_penalty, int top_k, float top_p);
    int generate_stream(const std::vector<int>& prompt, const std::function<void(const std::string&)>& on_text,
                        float temperature, int max_tokens, float repetition_penalty, int top_k, float top_p);

private:
    std::unique_ptr<TextGen> cpu_;
    std::unique_ptr<gradb::GPTModel> device_model_;
    std::unique_ptr<TokenizerDecoder> decoder_;
    std::unique_ptr<gradb::TextGen> b200_;
};

int run_generate(const Invocation& invocation);
int run_chat(const Invocation& invocation);
int run_eval(const Invocation& invocation);
int run_bench(const Invocation& invocation);

}  // namespace grad::cli::b200
