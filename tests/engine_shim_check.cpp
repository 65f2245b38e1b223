// Exercises the C++ drop-in classes (include/gradb/engine.hpp) the way the reference's
// own parity test drives its classes (tests/integration/sanity_tests.cpp:293-333):
// load a checkpoint, step a fixed sequence, check errors and a greedy rollout.
// Usage: engine_shim_check <checkpoint> [<token file>] ; prints ids and a few logits for the Python side to compare.
#include <cstdio>
#include <string>
#include <vector>

#include "../include/gradb/engine.hpp"
#include "support/token_data.hpp"

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    try {
        (void)gradb::GPTModel::load(std::string(argv[1]) + ".missing");
        std::printf("FAIL missing file did not throw\n");
        return 1;
    } catch (const std::runtime_error& e) {
        std::printf("missing: %s\n", e.what());
    }
    gradb::GPTModel model = gradb::GPTModel::load(argv[1]);
    std::printf("dims %d %d %d %d %d %d\n", model.getVocabSize(), model.getDModel(), model.getNumLayers(),
                model.getNumHeads(), model.getMaxLen(), static_cast<int>(model.getArch()));
    gradb::InferenceSession session(model);
    const int seq[] = {3, 11, 7, 0, 19, 5};
    for (int t : seq) {
        const float* lg = session.step(t);
        std::printf("logits %d %.9g %.9g %.9g\n", session.position(), lg[0], lg[1], lg[model.getVocabSize() - 1]);
    }
    try {
        (void)session.step(model.getVocabSize());
        std::printf("FAIL bad id did not throw\n");
        return 1;
    } catch (const std::out_of_range& e) {
        std::printf("bad id: %s\n", e.what());
    }
    try {
        while (true) (void)session.step(1);
    } catch (const std::runtime_error& e) {
        std::printf("full at %d of %d: %s\n", session.position(), session.capacity(), e.what());
    }
    gradb::TextGen gen(model);
    const std::vector<int> prompt = {3, 11, 7, 0};
    std::printf("greedy");
    for (int id : gen.greedy_ids(prompt, 8, 1.2f)) std::printf(" %d", id);
    std::printf("\n");
    gradb::TextGen::seed(7);
    std::printf("sample");
    for (int id : gen.sample_ids(prompt, 0.8f, 8, 1.1f, 5, 0.9f)) std::printf(" %d", id);
    std::printf("\n");
    int streamed = 0;
    const int n = gen.generate_stream(prompt, [&](const std::string& s) { streamed += (int)s.size(); }, 0.9f, 5);
    std::printf("stream %d %d\n", n, streamed);
    // streaming is real: an exception thrown from the third callback ends the generation there
    int calls = 0;
    try {
        gen.generate_stream(prompt, [&](const std::string&) { if (++calls == 3) throw std::logic_error("enough"); }, 0.9f, 9);
        std::printf("FAIL callback exception was swallowed\n");
        return 1;
    } catch (const std::logic_error& e) {
        std::printf("stream stopped after %d: %s\n", calls, e.what());
    }
    // the generator is left where the reference leaves it: one draw per emitted id (here the context fills first)
    {
        std::vector<int> longp(static_cast<size_t>(model.getMaxLen() - 2), 1);
        gradb::TextGen::seed(11);
        (void)gen.sample_ids(longp, 0.8f, 10, 1.1f, 0, 1.0f);   // emits 3 ids
        const std::vector<int> after = gen.sample_ids(prompt, 0.8f, 4, 1.1f, 0, 1.0f);
        gradb::TextGen::seed(11);
        (void)gen.sample_ids(longp, 0.8f, 3, 1.1f, 0, 1.0f);    // the same three draws, asked for exactly
        const std::vector<int> again = gen.sample_ids(prompt, 0.8f, 4, 1.1f, 0, 1.0f);
        std::printf("draws %s\n", after == again ? "aligned" : "misaligned");
    }
    std::printf("empty '%s'\n", gen.generate_greedy({}, 5).c_str());
    // `grad eval` (src/cli/eval.cpp:77-133): token file -> windows of 5 ids, stride 5 -> batches of 3
    if (argc >= 3) {
        const std::string tokens = argv[2];
        auto val = std::make_shared<gradb::MappedTokenDataset>(tokens, 5, 5);
        std::printf("dataset %zu %d %zu\n", val->size(), val->vocabSize(), val->tokenCount());
        gradb::DataLoader all(val, 3, /*shuffle=*/false, 20260921u);
        std::printf("batches %zu\n", all.num_batches());
        std::printf("mean_loss_all %.9g\n", gradb::training::mean_loss(model, all, 0));
        gradb::DataLoader capped(val, 3, /*shuffle=*/true, 20260921u);
        gradb::Batch first = capped.next_batch();
        std::printf("shuffled");
        for (int32_t id : first.input) std::printf(" %d", id);
        std::printf("\n");
        capped.reset();
        gradb::DataLoader capped2(val, 3, /*shuffle=*/true, 20260921u);
        std::printf("mean_loss_capped %.9g\n", gradb::training::mean_loss(model, capped2, 2));
        // a copy written by this side must be byte-identical to the reference's file
        std::vector<int> ids;
        for (size_t i = 0; i < val->size(); i++) {
            auto [in, tg] = val->get_item(i);
            ids.insert(ids.end(), in.begin(), in.end());
        }
        gradb::tokenfile::write(tokens + ".copy", ids, val->vocabSize());
        try {
            gradb::MappedTokenDataset bad(std::string(argv[1]), 5, 5);
            std::printf("FAIL checkpoint accepted as token file\n");
            return 1;
        } catch (const std::runtime_error& e) {
            std::printf("bad magic: %s\n", e.what());
        }
        try {
            gradb::MappedTokenDataset huge(tokens, 100000, 5);
            std::printf("FAIL oversized window accepted\n");
            return 1;
        } catch (const std::runtime_error& e) {
            std::printf("too short: %s\n", e.what());
        }
    }
    return 0;
}
