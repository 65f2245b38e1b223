// generate / chat / eval / bench with `--device b200`: the same arguments, output and control flow as
// src/cli/generate.cpp, chat.cpp, eval.cpp and bench.cpp (generation section), with the model work routed through
// Generator / gradb::training::mean_loss when the B200 engine is selected and through the reference's own classes
// otherwise, so one binary compares the two on the same inputs.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <filesystem>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <numbers>
#include <span>
#include <sstream>

#include "b200_backend.h"
#include "grad/data/dataset.h"
#include "grad/data/token_file.h"
#include "grad/training/trainer.h"
#include "grad/utils/metrics.h"
#include "grad/utils/training_utils.h"

namespace grad::cli::b200 {

namespace {

struct InferenceArgs {
    std::string checkpoint = "shakespeare_final.bin";
    std::string corpus = kDefaultCorpus;
    std::optional<int> vocab;
    std::optional<std::string> tokenizer_flag, device_flag;
    SamplingOptions sampling;
};

void declare_inference_args(Command& cmd, InferenceArgs& a, const char* ckpt_help, const std::string& greedy_help) {
    cmd.optional("ckpt", a.checkpoint, ckpt_help);
    cmd.optional("corpus", a.corpus, "the corpus the checkpoint was trained on, for its tokenizer");
    cmd.optional("vocab", a.vocab, "vocab size; must match the checkpoint's").at_least(1).default_text("the checkpoint's");
    add_sampling_options(cmd, a.sampling, greedy_help);
    add_tokenizer_option(cmd, a.tokenizer_flag, kInferenceTokenizerHelp);
    b200::add_device_option(cmd, a.device_flag);
}

// An empty prompt means "pick one" (src/cli/generate.cpp:41-48): the first speaker tag for the default corpus,
// else the opening of a held-out window (the val token file when prepared, else the last 5 % of the text).
Prompt choose_prompt(const std::string& prompt, const std::string& corpus, int vocab_size, const Tokenizer& tokenizer) {
    if (!prompt.empty()) return prompt_from_text(tokenizer, prompt);
    if (is_default_corpus(corpus)) return prompt_from_text(tokenizer, "ROMEO:\n");
    constexpr int kWindow = 6;
    const std::string val_bin = token_bin_path(corpus, vocab_size, "val", tokenizer.kind());
    if (tokenfile::exists(val_bin)) {
        return sample_prompts(corpus, tokenizer, MappedTokenDataset(val_bin, kWindow, kWindow)).at(0);
    }
    const std::vector<int> ids = tokenizer.encode(read_text_file(corpus));
    const auto held_out = std::span<const int>(ids).subspan(ids.size() * 95 / 100);
    return sample_prompts(corpus, tokenizer,
                          TextDataset(std::vector<int>(held_out.begin(), held_out.end()), kWindow, kWindow))
        .at(0);
}

std::string sampling_label(const SamplingOptions& o) {
    std::ostringstream out;
    out << "temp=" << o.temperature;
    if (o.top_k > 0) out << ", top-k=" << o.top_k;
    if (o.top_p < 1.0f) out << ", top-p=" << o.top_p;
    return out.str();
}

double median_of(std::vector<double> v) {
    std::sort(v.begin(), v.end());
    const size_t mid = v.size() / 2;
    return v.size() % 2 ? v[mid] : (v[mid - 1] + v[mid]) / 2.0;
}

}  // namespace

int run_generate(const Invocation& invocation) {
    InferenceArgs a;
    a.sampling.max_tokens = 150;
    std::string prompt;
    Command cmd(invocation.usage_name(), std::string(invocation.summary));
    cmd.describe("Prints a greedy continuation of the prompt, then a sampled one.");
    cmd.optional("ckpt", a.checkpoint, "checkpoint to sample from");
    cmd.optional("prompt", prompt, "text to continue; empty (\"\") picks one from the corpus's held-out split");
    cmd.optional("corpus", a.corpus, "the corpus the checkpoint was trained on, for its tokenizer");
    cmd.optional("vocab", a.vocab, "vocab size; must match the checkpoint's").at_least(1).default_text("the checkpoint's");
    add_sampling_options(cmd, a.sampling, "print only the greedy continuation");
    add_tokenizer_option(cmd, a.tokenizer_flag, kInferenceTokenizerHelp);
    b200::add_device_option(cmd, a.device_flag);
    if (cmd.parse(invocation.args) == ParseResult::HelpShown) return 0;

    std::cout << "\ngrad.cpp Generation\n" << std::endl;
    const DeviceChoice device = b200::apply_device(a.device_flag);
    const auto [model, tokenizer] =
        load_for_inference(a.checkpoint, a.corpus, a.vocab, parse_tokenizer_flag(a.tokenizer_flag));
    const Prompt chosen = choose_prompt(prompt, a.corpus, model.getVocabSize(), *tokenizer);
    Generator generator(device, a.checkpoint, model, tokenizer.get());

    std::cout << "\n--- Greedy Decoding ---\n" << std::endl;
    std::cout << "Prompt: \"" << chosen.text << "\"" << std::endl;
    std::cout << generator.generate_greedy(chosen.tokens, a.sampling.max_tokens, a.sampling.repetition_penalty)
              << std::endl;
    if (a.sampling.greedy) return 0;

    std::cout << "\n--- Sampling (" << sampling_label(a.sampling) << ") ---\n" << std::endl;
    std::cout << "Prompt: \"" << chosen.text << "\"" << std::endl;
    std::cout << generator.generate_sample(chosen.tokens, a.sampling.temperature, a.sampling.max_tokens,
                                           a.sampling.repetition_penalty, a.sampling.top_k, a.sampling.top_p)
              << std::endl;
    return 0;
}

int run_chat(const Invocation& invocation) {
    InferenceArgs a;
    a.sampling.max_tokens = 200;
    Command cmd(invocation.usage_name(), std::string(invocation.summary));
    cmd.describe("Each line you type is continued by the model, streamed as it is sampled. "
                 "An empty line, 'exit', or 'quit' ends the session.");
    declare_inference_args(cmd, a, "checkpoint to chat with", "always take the most likely token (top-k 1)");
    if (cmd.parse(invocation.args) == ParseResult::HelpShown) return 0;

    std::cout << "\ngrad.cpp Chat\n" << std::endl;
    const DeviceChoice device = b200::apply_device(a.device_flag);
    const auto [model, tokenizer] =
        load_for_inference(a.checkpoint, a.corpus, a.vocab, parse_tokenizer_flag(a.tokenizer_flag));
    Generator generator(device, a.checkpoint, model, tokenizer.get());
    // Streaming goes through the sampling path; restricted to the single most likely token it is greedy decoding
    // (src/cli/chat.cpp:42-44).
    const int top_k = a.sampling.greedy ? 1 : a.sampling.top_k;

    std::cout << "\nThis is a base language model: it continues text in the"
              << " style of its training corpus.\nEmpty line or 'exit' quits.\n"
              << std::endl;
    std::string line;
    while (true) {
        std::cout << "> " << std::flush;
        if (!std::getline(std::cin, line)) break;
        if (line.empty() || line == "exit" || line == "quit") break;
        const std::vector<int> prompt = tokenizer->encode(line + "\n");
        std::cout << line << std::flush;
        generator.generate_stream(
            prompt, [](const std::string& piece) { std::cout << piece << std::flush; }, a.sampling.temperature,
            a.sampling.max_tokens, a.sampling.repetition_penalty, top_k, a.sampling.top_p);
        std::cout << "\n" << std::endl;
    }
    return 0;
}

int run_eval(const Invocation& invocation) {
    std::string checkpoint, corpus;
    std::optional<int> vocab;
    int seq = 256, max_batches = 0;
    std::optional<std::string> tokenizer_flag, device_flag;
    Command cmd(invocation.usage_name(), std::string(invocation.summary));
    cmd.describe("Scores the val split and an equal-sized uniform sample of training windows in non-overlapping "
                 "windows with a fixed seed, so every checkpoint sees the same windows. Needs the corpus's prepared "
                 "token files (see prepare).");
    cmd.positional("ckpt", checkpoint, "checkpoint to score");
    cmd.positional("corpus", corpus, "the corpus the checkpoint was trained on");
    cmd.optional("vocab", vocab, "vocab size; must match the checkpoint's").at_least(1).default_text("the checkpoint's");
    cmd.optional("seq", seq, "window length in tokens").at_least(1);
    cmd.optional("max_batches", max_batches, "batches of 8 windows per split; 0 scores the whole val split")
        .at_least(0)
        .named("--batches");
    add_tokenizer_option(cmd, tokenizer_flag, kInferenceTokenizerHelp);
    b200::add_device_option(cmd, device_flag);
    if (cmd.parse(invocation.args) == ParseResult::HelpShown) return 0;
    const std::optional<TokenizerKind> requested = parse_tokenizer_flag(tokenizer_flag);
    const DeviceChoice device = b200::apply_device(device_flag);

    std::cout << "\ngrad.cpp Evaluation\n" << std::endl;
    GPTModel model = load_checkpoint(checkpoint, vocab);
    const int vocab_size = model.getVocabSize();
    const TokenizerKind kind = choose_tokenizer(corpus, vocab_size, requested, &model);
    const std::string train_bin = token_bin_path(corpus, vocab_size, "train", kind);
    const std::string val_bin = token_bin_path(corpus, vocab_size, "val", kind);
    if (!tokenfile::exists(train_bin) || !tokenfile::exists(val_bin)) {
        throw std::runtime_error("eval needs pre-tokenized files; run: ./build/grad prepare " + corpus + " " +
                                 std::to_string(vocab_size) + " --tokenizer " + tokenizer_kind_flag(kind));
    }
    if (std::ifstream(tokenizer_path(corpus, vocab_size, kind)).good()) {
        const std::unique_ptr<Tokenizer> tokenizer = load_existing_tokenizer(corpus, vocab_size, kind);
        check_tokenizer_matches(model, *tokenizer, checkpoint);
    } else {
        std::cerr << "Warning: no tokenizer file beside " << val_bin
                  << "; cannot check the token files against the checkpoint" << std::endl;
    }
    if (seq > model.getMaxLen()) {
        throw std::runtime_error("seq length exceeds the model's context (" + std::to_string(model.getMaxLen()) + ")");
    }
    constexpr int kBatchSize = 8;         // src/cli/eval.cpp:77
    constexpr unsigned kSeed = 20260921;  // src/cli/eval.cpp:85
    auto val = std::make_shared<MappedTokenDataset>(val_bin, seq, seq);
    auto train = std::make_shared<MappedTokenDataset>(train_bin, seq, seq);
    if (val->vocabSize() != model.getVocabSize()) {
        throw std::runtime_error("token files and checkpoint disagree on vocab size");
    }
    DataLoader val_loader(val, kBatchSize, /*shuffle=*/max_batches > 0, kSeed);
    const int val_batches = max_batches > 0 ? std::min<int>(max_batches, static_cast<int>(val_loader.num_batches()))
                                            : static_cast<int>(val_loader.num_batches());
    DataLoader train_loader(train, kBatchSize, /*shuffle=*/true, kSeed + 1);

    std::error_code size_error;
    const auto corpus_bytes = std::filesystem::file_size(corpus, size_error);
    const double bytes_per_token =
        size_error ? 0.0 : static_cast<double>(corpus_bytes) / static_cast<double>(train->tokenCount() + val->tokenCount());
    if (bytes_per_token > 0.0) {
        std::cout << "Corpus: " << std::fixed << std::setprecision(3) << bytes_per_token << " bytes/token"
                  << std::defaultfloat << std::endl;
    } else {
        std::cerr << "Warning: " << corpus << " not found; bits per byte needs its size and is not reported" << std::endl;
    }

    // The one line that differs: where the windows are scored.
    std::unique_ptr<gradb::GPTModel> device_model;
    if (device.b200) {
        device_model = std::make_unique<gradb::GPTModel>(gradb::GPTModel::load(checkpoint, device.index, device.precision));
    }
    const auto score = [&](DataLoader& loader) {
        const auto start = std::chrono::steady_clock::now();
        const double loss = device.b200 ? gradb::training::mean_loss(*device_model, loader, val_batches)
                                        : training::mean_loss(model, loader, val_batches);
        return std::make_pair(loss, std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count());
    };
    const auto report = [bytes_per_token](const char* split, double loss, long tokens, double seconds) {
        std::cout << std::left << std::setw(8) << split << std::right << std::fixed << " loss " << std::setprecision(4)
                  << loss << "  perplexity " << std::setprecision(3) << std::exp(loss);
        if (bytes_per_token > 0.0) {
            std::cout << "  bits/byte " << std::setprecision(4) << loss / std::numbers::ln2 / bytes_per_token;
        }
        std::cout << "  (" << tokens << " tokens, " << std::setprecision(0) << seconds << "s)" << std::defaultfloat
                  << std::endl;
    };
    utils::print_section("Scoring");
    const long tokens =
        static_cast<long>(std::min<size_t>(static_cast<size_t>(val_batches) * kBatchSize, val->size())) * seq;
    const auto [val_loss, val_s] = score(val_loader);
    report("val", val_loss, tokens, val_s);
    const auto [train_loss, train_s] = score(train_loader);
    report("train", train_loss, static_cast<long>(val_batches) * kBatchSize * seq, train_s);
    return 0;
}

// The generation section of `grad bench` (src/cli/bench.cpp:269-286) on the selected device: the 22M "small"
// configuration, random-init, prompt "ROMEO:\n", 64 sampled ids per trial at temperature 0.8 (repetition penalty
// 1.2, no top-k / top-p), tokenization and model construction outside the timed region, the median of --trials.
// --json writes a record with the reference's schema (src/cli/bench.cpp:132-168); the training figures, which this
// engine does not produce, are left as empty arrays.
int run_bench(const Invocation& invocation) {
    int trials = 5;
    std::string json_path, corpus = kDefaultCorpus;
    std::optional<std::string> device_flag;
    Command cmd(invocation.usage_name(), std::string(invocation.summary));
    cmd.describe("Times 64-token sampled generation of the 22M 'small' model, reporting the median of --trials "
                 "windows. Run it on an otherwise idle machine.");
    cmd.option("--trials", trials, "timed windows; the median is reported").at_least(1);
    cmd.option("--json", json_path, "also write the results as JSON").metavar("PATH");
    cmd.option("--corpus", corpus, "text the v1 tokenizer is built from").metavar("PATH");
    b200::add_device_option(cmd, device_flag);
    if (cmd.parse(invocation.args) == ParseResult::HelpShown) return 0;
    const DeviceChoice device = b200::apply_device(device_flag);

    std::cout << "\ngrad.cpp Benchmark\n" << std::endl;
    constexpr int kVocab = 5000, kDModel = 512, kLayers = 6, kHeads = 8, kMaxLen = 1024, kGenTokens = 64;
    const std::string text = read_text_file(corpus);
    const std::unique_ptr<Tokenizer> tokenizer = load_or_train_tokenizer(corpus, kVocab, TokenizerKind::BpeV1, text);
    GPTModel model(kVocab, kDModel, kLayers, kHeads, kMaxLen, 0.1f);
    size_t parameter_count = 0;
    for (const auto& param : model.getAllParameters()) parameter_count += param->getData().numel();
    std::string checkpoint;
    if (device.b200) {  // the engine reads checkpoint files: hand it this model through one
        checkpoint = (std::filesystem::temp_directory_path() / ("grad_bench_" + std::to_string(::getpid()) + ".bin")).string();
        if (!model.save(checkpoint)) throw std::runtime_error("could not write " + checkpoint);
    }
    Generator generator(device, checkpoint, model, tokenizer.get());
    if (!checkpoint.empty()) std::filesystem::remove(checkpoint);

    utils::print_section("Generation throughput");
    const std::vector<int> prompt = tokenizer->encode("ROMEO:\n");
    std::vector<double> tokens_per_s;
    for (int trial = 0; trial < trials; ++trial) {
        const auto start = std::chrono::steady_clock::now();
        generator.generate_sample(prompt, 0.8f, kGenTokens, 1.2f, 0, 1.0f);
        const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
        tokens_per_s.push_back(kGenTokens / seconds);
        std::cout << "  trial " << (trial + 1) << ": " << std::fixed << std::setprecision(1) << tokens_per_s.back()
                  << " tok/s" << std::endl;
    }
    std::cout << "  median: " << std::fixed << std::setprecision(1) << median_of(tokens_per_s) << " tok/s" << std::endl;
    const size_t peak_memory_mb = utils::get_peak_memory_mb();
    std::cout << "\nPeak RSS: " << peak_memory_mb << " MB" << std::endl;

    if (!json_path.empty()) {
        std::ofstream out(json_path);
        if (!out) throw std::runtime_error("Cannot write benchmark JSON: " + json_path);
        out << "{\n  \"schema_version\": 1,\n  \"engine\": \"grad.cpp\",\n  \"device\": \""
            << (device.b200 ? (device.precision == GRADB_BF16 ? "b200-bf16" : "b200") : "cpu") << "\",\n"
            << "  \"engine_backend\": \"" << (device.b200 ? gradb_version() : "reference") << "\",\n"
            << "  \"parameters\": " << parameter_count << ",\n"
            << "  \"config\": {\"vocab\": " << kVocab << ", \"d_model\": " << kDModel << ", \"layers\": " << kLayers
            << ", \"heads\": " << kHeads << ", \"sequence\": 96, \"batch\": 8},\n"
            << "  \"protocol\": {\"warmup_steps\": 0, \"steps_per_trial\": 0, \"trials\": " << trials << "},\n"
            << "  \"training_steps_per_second\": [],\n  \"training_tokens_per_second\": [],\n"
            << "  \"generation_tokens_per_second\": [";
        for (size_t i = 0; i < tokens_per_s.size(); ++i) {
            out << (i ? ", " : "") << std::fixed << std::setprecision(6) << tokens_per_s[i];
        }
        out << "],\n  \"median_generation_tokens_per_second\": " << median_of(tokens_per_s) << ",\n"
            << "  \"peak_rss_mb\": " << peak_memory_mb << "\n}\n";
        if (!out.good()) throw std::runtime_error("Failed while writing benchmark JSON: " + json_path);
        std::cout << "Benchmark JSON: " << json_path << std::endl;
    }
    return 0;
}

}  // namespace grad::cli::b200
