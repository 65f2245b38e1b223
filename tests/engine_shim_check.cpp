// Exercises the C++ drop-in classes (include/gradb/engine.hpp) the way the reference's
// own parity test drives its classes (tests/integration/sanity_tests.cpp:293-333):
// load a checkpoint, step a fixed sequence, check errors and a greedy rollout.
// Usage: engine_shim_check <checkpoint> ; prints ids and a few logits for the Python side to compare.
#include <cstdio>
#include <string>
#include <vector>

#include "../include/gradb/engine.hpp"

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
    std::printf("empty '%s'\n", gen.generate_greedy({}, 5).c_str());
    // `grad eval`: windows of 5 ids with stride 5 over a 23-id stream -> 4 windows, batches of 3 (last one ragged)
    std::vector<int> stream;
    for (int i = 0; i < 23; i++) stream.push_back((i * 7 + 3) % model.getVocabSize());
    const gradb::TokenWindows windows(stream, 5, 5);
    std::printf("windows %zu\n", windows.size());
    std::printf("mean_loss %.9g\n", gradb::training::mean_loss(model, windows, 0, 3));
    std::printf("mean_loss_first %.9g\n", gradb::training::mean_loss(model, windows, 1, 3));
    return 0;
}
