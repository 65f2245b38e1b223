#include "b200_backend.h"

#include <cstdlib>
#include <iostream>

namespace grad::cli::b200 {

std::optional<DeviceChoice> parse_device(const std::string& flag) {
    if (flag.rfind("b200", 0) != 0) return std::nullopt;
    DeviceChoice choice;
    choice.b200 = true;
    std::string rest = flag.substr(4);
    if (rest.rfind("-bf16", 0) == 0) {
        choice.precision = GRADB_BF16;
        rest = rest.substr(5);
    }
    if (!rest.empty()) {
        char* end = nullptr;
        const long n = rest[0] == ':' ? std::strtol(rest.c_str() + 1, &end, 10) : -1;
        if (rest[0] != ':' || rest.size() < 2 || *end != '\0' || n < 0 || n > 1023) {
            throw UsageError("--device: expected b200, b200-bf16, b200:N or b200-bf16:N, got '" + flag + "'");
        }
        choice.index = static_cast<int>(n);
    }
    return choice;
}

void add_device_option(Command& cmd, std::optional<std::string>& flag) {
    cmd.option("--device", flag,
               "cpu, metal, or b200 (the token loop and scoring on an NVIDIA B200; b200-bf16 keeps the weights in "
               "bf16; b200:N picks a GPU) (default: GRAD_DEVICE, else cpu)")
        .metavar("cpu|metal|b200");
}

DeviceChoice apply_device(const std::optional<std::string>& flag) {
    std::optional<std::string> named = flag;
    if (!named) {
        if (const char* env = std::getenv("GRAD_DEVICE")) {
            if (std::string(env).rfind("b200", 0) == 0) named = std::string(env);
        }
    }
    if (named) {
        if (const std::optional<DeviceChoice> choice = parse_device(*named)) {
            int count = 0;
            if (gradb_device_count(&count) != GRADB_OK || choice->index >= count) {
                throw std::runtime_error("--device " + *named + ": " +
                                         (count == 0 ? std::string(gradb_last_error())
                                                     : "this machine has " + std::to_string(count) + " CUDA device(s)"));
            }
            std::cout << "Device: b200:" << choice->index
                      << (choice->precision == GRADB_BF16 ? " (bf16 weights, fp32 accumulate)" : " (fp32)") << std::endl;
            return *choice;
        }
    }
    grad::cli::apply_device(flag);
    return {};
}

Generator::Generator(const DeviceChoice& device, const std::string& checkpoint_path, const GPTModel& host_model,
                     const Tokenizer* tokenizer) {
    if (!device.b200) {
        cpu_ = std::make_unique<TextGen>(host_model, tokenizer);
        return;
    }
    device_model_ =
        std::make_unique<gradb::GPTModel>(gradb::GPTModel::load(checkpoint_path, device.index, device.precision));
    if (tokenizer != nullptr) decoder_ = std::make_unique<TokenizerDecoder>(tokenizer);
    b200_ = std::make_unique<gradb::TextGen>(*device_model_, decoder_.get());
}

std::string Generator::generate_greedy(const std::vector<int>& prompt, int max_tokens, float repetition_penalty) {
    return b200_ ? b200_->generate_greedy(prompt, max_tokens, repetition_penalty)
                 : cpu_->generate_greedy(prompt, max_tokens, repetition_penalty);
}

std::string Generator::generate_sample(const std::vector<int>& prompt, float temperature, int max_tokens,
                                       float repetition_penalty, int top_k, float top_p) {
    return b200_ ? b200_->generate_sample(prompt, temperature, max_tokens, repetition_penalty, top_k, top_p)
                 : cpu_->generate_sample(prompt, temperature, max_tokens, repetition_penalty, top_k, top_p);
}

int Generator::generate_stream(const std::vector<int>& prompt, const std::function<void(const std::string&)>& on_text,
                               float temperature, int max_tokens, float repetition_penalty, int top_k, float top_p) {
    return b200_ ? b200_->generate_stream(prompt, on_text, temperature, max_tokens, repetition_penalty, top_k, top_p)
                 : cpu_->generate_stream(prompt, on_text, temperature, max_tokens, repetition_penalty, top_k, top_p);
}

}  // namespace grad::cli::b200
