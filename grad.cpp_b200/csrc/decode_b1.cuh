// Single-sequence decode step as ONE persistent cooperative kernel (decode_b1.cu).
#pragma once
#include "common.cuh"

namespace gradb {

// How one (K x N) projection is cut into per-CTA tiles: N into column tiles of CW
// columns, K into KS slices of Kt rows. Tile (ct, ks) belongs to CTA ks*col_tiles+ct
// and is stored contiguously ([Kt][CW], zero padded) so it can be fetched with one
// bulk copy.
struct B1Mat {
    int K, N, CW, KS, Kt, col_tiles, tiles;
    int tile_elems;  // Kt * CW
};

struct B1Layer {
    const void *qkv, *o, *gate, *up;  // packed tiles (fp32 or bf16)
    const void* down;               // FFN down matrix in checkpoint layout [d_ff][d] (fp32 or bf16): read by rows
    const float *bq, *bk, *bv, *bo, *b1, *b2, *n1g, *n1b, *n2g, *n2b;
};

struct B1Plan {
    bool ok = false;
    int G = 0;  // CTAs = SMs
    int wbytes = 4;
    B1Mat qkv{}, o{}, up{}, down{};
    int logit_rows_per_cta = 0, logit_chunk_rows = 0;
    int attn_splits = 1;
    B1Layer* layers_dev = nullptr;  // [L]
    std::vector<void*> owned;       // packed buffers
};

struct B1Params {
    int G, d, dff, H, hs, V, L, T, modern, wbytes;
    B1Mat qkv, o, up, down;
    int logit_rows_per_cta, logit_chunk_rows, attn_splits;
    const B1Layer* layers;
    const float* emb32;  // (V, d) fp32: token lookup
    const void* emb_w;   // (V, d) in the weight precision: logits
    const float *pos_emb, *fng, *fnb, *rope_cos, *rope_sin;
    float *kcache, *vcache;  // [L][1][H][T][hs] of sequence 0
    size_t layer_cache_stride;
    // exchange buffers (global, L2 resident), all starting zeroed
    unsigned long long* q_ll;     // [d] {value, epoch}: the query of the current layer
    unsigned long long* kv_ll;    // [2][d] the new K row and V row of the current layer
    unsigned long long* attn_ll;  // [H * splits][hs + 2] attention partials: values, running max, running sum
    unsigned long long* o_ll;     // [KS][d] output-projection partial vectors, one per K slice
    float* logits;
    // Sum over CTAs of the FFN output, in 2^-32 fixed point above a contribution count (integer adds commute, so the result does not
    // depend on arrival order): [2 sets used by alternate steps][L][d], one 128-byte
    // line per element
    long long* acc;
    const int *tok, *logit_tok;
    int *pos, *hist, *hist_len;
    int hist_stride, append_hist;
    unsigned* sync;  // [0] steps run so far, [1] CTAs that have read their launch state (G per step)
    int* status;
    unsigned long long* trace;  // optional: %globaltimer stamps of CTA 0 at every stage boundary
};

B1Plan* b1_make_plan(const DeviceModel* m);
void b1_free_plan(B1Plan* p);
size_t b1_workspace_bytes(const DeviceModel* m, const B1Plan* plan);
// Points the exchange buffers of `p` into a zeroed workspace of b1_workspace_bytes.
void b1_bind_workspace(B1Params& p, void* workspace, const DeviceModel* m, const B1Plan* plan);
void launch_decode_b1(const B1Params& p, cudaStream_t st);

}  // namespace gradb
