// GPTM checkpoint reader/writer (host only).
//
// Format, limits and error texts follow the reference's GPTModel::save / load
// (src/transformer/gpt_model.cpp:187-227 helpers, :292-381 save, :383-525 load).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/gradb.h"

namespace gradb {

struct TensorShape {
    int rows;
    int cols;
};

// d_ff as the reference derives it (include/grad/transformer/feedforward.h:24-28).
int resolve_d_ff(int d_model, bool modern);

// Shapes of every tensor in file order (gpt_model.cpp:316-353).
std::vector<TensorShape> tensor_shapes(const gradb_model_desc& desc);

// Index helpers into the file-order tensor list.
struct TensorIndex {
    int emb = 0, pos = -1;
    int layer0 = 0, per_layer = 0;
    // offsets inside a layer
    int wq = 0, wk = 1, wv = 2, wo = 3, bq = 4, bk = 5, bv = 6, bo = 7;
    int gate = -1, w1 = -1, b1 = -1, w2 = -1, b2 = -1;
    int n1g = 0, n1b = 0, n2g = 0, n2b = 0;
    int final_g = 0, final_b = 0;
    int count = 0;
};
TensorIndex tensor_index(const gradb_model_desc& desc);

struct Checkpoint {
    gradb_model_desc desc{};
    std::vector<std::vector<float>> tensors;  // file order; empty when only inspected
};

// Throws std::runtime_error with the reference's message text
// ("Failed to load model from <path>: <what>", or "Could not open checkpoint
// for reading: <path>"). With keep_data=false the tensor payloads are read
// and checked for truncation but not retained.
Checkpoint read_checkpoint(const std::string& path, bool keep_data);

// Writes a version-2 file. Returns false (message in err) on I/O failure.
bool write_checkpoint(const std::string& path, const gradb_model_desc& desc,
                      const float* const* tensors, int n_tensors, std::string& err);

}  // namespace gradb
