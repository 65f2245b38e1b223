// grad-b200: the grad command line with `--device b200` on generate, chat, eval and bench. `prepare` is the
// reference's own command (it makes the tokenizer and token files the others read); the rest of grad's commands
// (train, watch, presets) are untouched by the engine and stay in the reference binary.
// Exit codes as in src/main.cpp:94-103: 2 for a malformed command line, 1 for a failure while running.
#include <cstdio>
#include <exception>
#include <iostream>
#include <span>
#include <string_view>
#include <vector>

#include "b200_backend.h"

namespace {

struct Entry {
    std::string_view name;
    int (*run)(const grad::cli::Invocation&);
    std::string_view summary;
};

constexpr Entry kCommands[] = {
    {"prepare", grad::cli::run_prepare, "Pre-tokenize a corpus into memory-mapped .bin token files"},
    {"generate", grad::cli::b200::run_generate, "Sample greedy and sampled continuations from a checkpoint"},
    {"chat", grad::cli::b200::run_chat, "Interactive REPL: type a prompt, watch the model continue it"},
    {"eval", grad::cli::b200::run_eval, "Loss and perplexity on held-out and training windows"},
    {"bench", grad::cli::b200::run_bench, "Generation throughput, median of repeated trials"},
};

void usage(std::ostream& out, std::string_view program) {
    out << "Usage: " << program << " <command> [arguments] [options]\n\nCommands:\n";
    for (const Entry& e : kCommands) out << "  " << e.name << std::string(11 - e.name.size(), ' ') << e.summary << '\n';
    out << "\nRun '" << program << " <command> --help' for a command's arguments and options.\n";
}

int dispatch(int argc, char* argv[]) {
    const std::vector<std::string_view> args(argv, argv + argc);
    const std::string_view program = args.empty() ? "grad-b200" : args[0];
    if (args.size() < 2) {
        usage(std::cerr, program);
        return 2;
    }
    if (args[1] == "-h" || args[1] == "--help" || args[1] == "help") {
        usage(std::cout, program);
        return 0;
    }
    for (const Entry& e : kCommands) {
        if (e.name != args[1]) continue;
        const grad::cli::Invocation invocation{
            .program = program, .command = e.name, .summary = e.summary, .args = std::span(args).subspan(2)};
        try {
            return e.run(invocation);
        } catch (const grad::cli::UsageError& err) {
            std::cerr << "Error: " << err.what() << "\nRun '" << invocation.usage_name() << " --help' for usage."
                      << std::endl;
            return 2;
        } catch (const std::exception& err) {
            std::cerr << "\nError: " << err.what() << std::endl;
            return 1;
        }
    }
    std::cerr << "Error: unknown command '" << args[1] << "'\n\n";
    usage(std::cerr, program);
    return 2;
}

}  // namespace

int main(int argc, char* argv[]) {
    try {
        return dispatch(argc, argv);
    } catch (const std::exception& e) {
        std::fputs("Error: ", stderr);
        std::fputs(e.what(), stderr);
        std::fputs("\n", stderr);
    } catch (...) {
        std::fputs("Error: unknown exception\n", stderr);
    }
    return 1;
}
