#include "checkpoint.h"

#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace gradb {

namespace {
constexpr uint32_t kMagic = 0x4750544Du;  // bytes "MTPG" on disk, reads as "GPTM" (gpt_model.cpp:187)
constexpr uint32_t kMaxTrailer = 1u << 20;

struct File {
    std::FILE* f = nullptr;
    ~File() {
        if (f) std::fclose(f);
    }
};

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error(what); }

template <typename T>
T scalar(std::FILE* f, const char* what) {
    T v{};
    if (std::fread(&v, sizeof(T), 1, f) != 1) fail(std::string("file ends while reading ") + what);
    return v;
}

void check_range(const char* name, int v, int lo, int hi) {
    if (v < lo || v > hi) {
        fail(std::string("header field ") + name + " = " + std::to_string(v) + " is outside [" +
             std::to_string(lo) + ", " + std::to_string(hi) + "]");
    }
}

void put_le(std::string& out, uint64_t v, int bytes) {
    for (int i = 0; i < bytes; i++) out.push_back(static_cast<char>((v >> (8 * i)) & 0xFFu));
}
uint64_t get_le(const unsigned char* p, int bytes) {
    uint64_t v = 0;
    for (int i = 0; i < bytes; i++) v |= static_cast<uint64_t>(p[i]) << (8 * i);
    return v;
}
}  // namespace

int resolve_d_ff(int d_model, bool modern) {
    return modern ? ((8 * d_model / 3) + 63) / 64 * 64 : 4 * d_model;
}

TensorIndex tensor_index(const gradb_model_desc& desc) {
    const bool modern = desc.arch == GRADB_ARCH_MODERN;
    TensorIndex ix;
    int n = 0;
    ix.emb = n++;
    if (!modern) ix.pos = n++;
    ix.layer0 = n;
    int o = 8;
    if (modern) {
        ix.gate = o++;
        ix.w1 = o++;
        ix.w2 = o++;
    } else {
        ix.w1 = o++;
        ix.b1 = o++;
        ix.w2 = o++;
        ix.b2 = o++;
    }
    ix.n1g = o++;
    ix.n1b = o++;
    ix.n2g = o++;
    ix.n2b = o++;
    ix.per_layer = o;
    n += desc.num_layers * ix.per_layer;
    ix.final_g = n++;
    ix.final_b = n++;
    ix.count = n;
    return ix;
}

std::vector<TensorShape> tensor_shapes(const gradb_model_desc& desc) {
    const bool modern = desc.arch == GRADB_ARCH_MODERN;
    const int d = desc.d_model, f = desc.d_ff;
    std::vector<TensorShape> s;
    s.push_back({desc.vocab_size, d});
    if (!modern) s.push_back({desc.max_len, d});
    for (int l = 0; l < desc.num_layers; l++) {
        for (int i = 0; i < 4; i++) s.push_back({d, d});
        for (int i = 0; i < 4; i++) s.push_back({1, d});
        if (modern) {
            s.push_back({d, f});
            s.push_back({d, f});
            s.push_back({f, d});
        } else {
            s.push_back({d, f});
            s.push_back({1, f});
            s.push_back({f, d});
            s.push_back({1, d});
        }
        for (int i = 0; i < 4; i++) s.push_back({1, d});
    }
    s.push_back({1, d});
    s.push_back({1, d});
    return s;
}

static const char* tensor_name(const gradb_model_desc& desc, const TensorIndex& ix, int i, std::string& buf) {
    if (i == ix.emb) return "token embedding";
    if (i == ix.pos) return "position embedding";
    if (i == ix.final_g) return "final norm gamma";
    if (i == ix.final_b) return "final norm beta";
    const int l = (i - ix.layer0) / ix.per_layer, o = (i - ix.layer0) % ix.per_layer;
    static const char* const attn[] = {"W_q", "W_k", "W_v", "W_o", "b_q", "b_k", "b_v", "b_o"};
    const bool modern = desc.arch == GRADB_ARCH_MODERN;
    const char* what = "";
    if (o < 8) {
        what = attn[o];
    } else if (o == ix.gate) {
        what = "FFN gate";
    } else if (o == ix.w1) {
        what = modern ? "FFN up" : "FFN W1";
    } else if (o == ix.b1) {
        what = "FFN b1";
    } else if (o == ix.w2) {
        what = modern ? "FFN down" : "FFN W2";
    } else if (o == ix.b2) {
        what = "FFN b2";
    } else if (o == ix.n1g) {
        what = "norm1 gamma";
    } else if (o == ix.n1b) {
        what = "norm1 beta";
    } else if (o == ix.n2g) {
        what = "norm2 gamma";
    } else {
        what = "norm2 beta";
    }
    buf = "layer " + std::to_string(l) + " " + what;
    return buf.c_str();
}

Checkpoint read_checkpoint(const std::string& path, bool keep_data) {
    File file;
    file.f = std::fopen(path.c_str(), "rb");
    if (!file.f) throw std::runtime_error("Could not open checkpoint for reading: " + path);
    std::FILE* f = file.f;
    try {
        Checkpoint ck;
        gradb_model_desc& d = ck.desc;
        if (scalar<uint32_t>(f, "magic number") != kMagic) fail("not a grad.cpp checkpoint (wrong magic number)");
        const uint32_t version = scalar<uint32_t>(f, "format version");
        if (version != 1 && version != 2) fail("unsupported format version " + std::to_string(version));
        uint32_t arch = 0;  // version 1 predates the tag: GPT-2 layout
        if (version == 2) {
            arch = scalar<uint32_t>(f, "architecture tag");
            if (arch > 1) fail("unknown architecture tag " + std::to_string(arch));
        }
        d.format_version = static_cast<int32_t>(version);
        d.arch = static_cast<int32_t>(arch);
        d.vocab_size = scalar<int32_t>(f, "vocab_size");
        d.d_model = scalar<int32_t>(f, "d_model");
        d.num_layers = scalar<int32_t>(f, "num_layers");
        d.num_heads = scalar<int32_t>(f, "num_heads");
        d.max_len = scalar<int32_t>(f, "max_len");
        d.dropout_rate = scalar<float>(f, "dropout_rate");
        check_range("vocab_size", d.vocab_size, 1, 1 << 24);
        check_range("d_model", d.d_model, 1, 1 << 16);
        check_range("num_layers", d.num_layers, 1, 1 << 12);
        check_range("num_heads", d.num_heads, 1, d.d_model);
        check_range("max_len", d.max_len, 1, 1 << 20);
        if (d.d_model % d.num_heads != 0) {
            fail("d_model " + std::to_string(d.d_model) + " is not divisible by num_heads " +
                 std::to_string(d.num_heads));
        }
        if (!(d.dropout_rate >= 0.0f && d.dropout_rate < 1.0f)) {
            fail("dropout_rate " + std::to_string(d.dropout_rate) + " is outside [0, 1)");
        }
        d.d_ff = resolve_d_ff(d.d_model, arch == 1);

        const TensorIndex ix = tensor_index(d);
        const std::vector<TensorShape> shapes = tensor_shapes(d);
        if (keep_data) ck.tensors.resize(shapes.size());
        std::vector<float> sink;
        std::string namebuf;
        for (size_t i = 0; i < shapes.size(); i++) {
            const char* what = tensor_name(d, ix, static_cast<int>(i), namebuf);
            const int rows = scalar<int32_t>(f, what);
            const int cols = scalar<int32_t>(f, what);
            if (rows <= 0 || cols <= 0 || rows != shapes[i].rows || cols != shapes[i].cols) {
                fail(std::string(what) + " is " + std::to_string(rows) + "x" + std::to_string(cols) +
                     ", model expects " + std::to_string(shapes[i].rows) + "x" + std::to_string(shapes[i].cols));
            }
            const size_t n = static_cast<size_t>(rows) * static_cast<size_t>(cols);
            std::vector<float>& dst = keep_data ? ck.tensors[i] : sink;
            dst.resize(n);
            if (std::fread(dst.data(), sizeof(float), n, f) != n) fail(std::string("file ends inside ") + what);
        }

        // Tagged trailer sections until a clean end of file (gpt_model.cpp:489-515).
        for (;;) {
            const int c = std::fgetc(f);
            if (c == EOF) break;
            std::ungetc(c, f);
            unsigned char h[8];
            if (std::fread(h, 1, 8, f) != 8) fail("file ends while reading trailer section header");
            const uint32_t len = static_cast<uint32_t>(get_le(h + 4, 4));
            if (len > kMaxTrailer) {
                fail("trailer section has an implausible length (" + std::to_string(len) + " bytes)");
            }
            if (std::memcmp(h, "TKFP", 4) != 0) {
                std::vector<unsigned char> skip(len);
                if (len && std::fread(skip.data(), 1, len, f) != len) fail("file ends inside trailer section");
                continue;
            }
            if (len != 12) fail("tokenizer trailer has length " + std::to_string(len) + ", expected 12");
            unsigned char p[12];
            if (std::fread(p, 1, 12, f) != 12) fail("file ends while reading tokenizer trailer");
            const uint32_t kind = static_cast<uint32_t>(get_le(p, 4));
            if (kind != 1 && kind != 2) fail("unknown tokenizer kind " + std::to_string(kind));
            d.has_fingerprint = 1;
            d.fingerprint_kind = kind;
            d.fingerprint_hash = get_le(p + 4, 8);
        }
        return ck;
    } catch (const std::exception& e) {
        throw std::runtime_error("Failed to load model from " + path + ": " + e.what());
    }
}

bool write_checkpoint(const std::string& path, const gradb_model_desc& desc, const float* const* tensors,
                      int n_tensors, std::string& err) {
    const std::vector<TensorShape> shapes = tensor_shapes(desc);
    if (static_cast<size_t>(n_tensors) != shapes.size()) {
        err = "expected " + std::to_string(shapes.size()) + " tensors, got " + std::to_string(n_tensors);
        return false;
    }
    File file;
    file.f = std::fopen(path.c_str(), "wb");
    if (!file.f) {
        err = "Could not open file for writing: " + path;
        return false;
    }
    std::FILE* f = file.f;
    bool ok = true;
    auto w = [&](const void* p, size_t n) { ok = ok && std::fwrite(p, 1, n, f) == n; };
    const uint32_t magic = kMagic, version = 2, arch = static_cast<uint32_t>(desc.arch);
    w(&magic, 4);
    w(&version, 4);
    w(&arch, 4);
    w(&desc.vocab_size, 4);
    w(&desc.d_model, 4);
    w(&desc.num_layers, 4);
    w(&desc.num_heads, 4);
    w(&desc.max_len, 4);
    w(&desc.dropout_rate, 4);
    for (size_t i = 0; i < shapes.size(); i++) {
        const int32_t r = shapes[i].rows, c = shapes[i].cols;
        w(&r, 4);
        w(&c, 4);
        w(tensors[i], sizeof(float) * static_cast<size_t>(r) * static_cast<size_t>(c));
    }
    if (desc.has_fingerprint) {
        std::string t = "TKFP";
        put_le(t, 12, 4);
        put_le(t, desc.fingerprint_kind, 4);
        put_le(t, desc.fingerprint_hash, 8);
        w(t.data(), t.size());
    }
    ok = ok && std::fflush(f) == 0;
    const int rc = std::fclose(f);
    file.f = nullptr;
    if (!ok || rc != 0) {
        err = "writing checkpoint failed: " + path;
        return false;
    }
    return true;
}

}  // namespace gradb
