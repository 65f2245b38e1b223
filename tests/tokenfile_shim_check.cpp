// The test-support data classes (tests/support/token_data.hpp: token files, windows, batch order) driven the way
// `grad eval` drives the reference's (src/cli/eval.cpp:77-92). No device work.
// Usage: tokenfile_shim_check <token file> <scratch path>
#include <cstdio>
#include <string>

#include "../include/gradb/engine.hpp"
#include "support/token_data.hpp"

static void dump(const char* tag, gradb::DataLoader& loader, int max_batches) {
    for (int b = 0; loader.has_next(); b++) {
        if (max_batches > 0 && b >= max_batches) break;
        gradb::Batch batch = loader.next_batch();
        for (size_t w = 0; w < batch.batch_size; w++) {
            std::printf("%s", tag);
            for (size_t t = 0; t < batch.seq_length; t++) std::printf(" %d", batch.input[w * batch.seq_length + t]);
            std::printf(" |");
            for (size_t t = 0; t < batch.seq_length; t++) std::printf(" %d", batch.target[w * batch.seq_length + t]);
            std::printf("\n");
        }
    }
}

template <class F>
static void expect_throw(const char* tag, F&& f) {
    try {
        f();
        std::printf("%s\tOK\n", tag);
    } catch (const std::exception& e) {
        std::printf("%s\t%s\n", tag, e.what());
    }
}

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const std::string path = argv[1], scratch = argv[2];
    for (auto [seq, stride] : {std::pair{5, 5}, {12, 12}, {7, 1}, {16, 16}}) {
        gradb::MappedTokenDataset ds(path, seq, stride);
        std::printf("open_%d_%d %zu %d %zu\n", seq, stride, ds.size(), ds.vocabSize(), ds.tokenCount());
    }
    constexpr unsigned kSeed = 20260921;
    {
        auto ds = std::make_shared<gradb::MappedTokenDataset>(path, 5, 5);
        gradb::DataLoader seq(ds, 3, false, kSeed), capped(ds, 3, true, kSeed);
        std::printf("batches %zu\n", seq.num_batches());
        dump("seq", seq, 0);
        dump("capped", capped, 2);
    }
    {
        auto ds = std::make_shared<gradb::MappedTokenDataset>(path, 12, 12);
        gradb::DataLoader train(ds, 8, true, kSeed + 1), ragged(ds, 8, false, kSeed);
        dump("train", train, 2);
        dump("ragged", ragged, 0);
    }
    // write a copy from the ids read back
    {
        gradb::MappedTokenDataset ds(path, 1, 1);
        std::vector<int> ids;
        for (size_t i = 0; i < ds.size(); i++) ids.push_back(ds.get_item(i).first[0]);
        ids.push_back(ds.get_item(ds.size() - 1).second[0]);
        gradb::tokenfile::write(scratch, ids, ds.vocabSize());
        std::printf("exists %d %d\n", gradb::tokenfile::exists(scratch), gradb::tokenfile::exists(scratch + ".nope"));
    }
    expect_throw("stride", [&] { gradb::MappedTokenDataset ds(path, 5, 0); });
    expect_throw("batch", [&] {
        gradb::DataLoader l(std::make_shared<gradb::MappedTokenDataset>(path, 5, 5), 0);
    });
    expect_throw("vocab", [&] { gradb::tokenfile::write(scratch + ".v", std::vector<int>{1}, 70000); });
    expect_throw("range", [&] { gradb::tokenfile::write(scratch + ".r", std::vector<int>{1, 9}, 9); });
    for (int i = 3; i < argc; i++) {
        const std::string damaged = argv[i];
        expect_throw(("damaged" + std::to_string(i - 3)).c_str(), [&] { gradb::MappedTokenDataset ds(damaged, 5, 5); });
    }
    return 0;
}
