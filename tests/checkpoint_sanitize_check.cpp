// Host-side checkpoint code (csrc/checkpoint.cpp) under AddressSanitizer + UndefinedBehaviorSanitizer: the reference
// runs its own suite under both (.github/workflows/ci.yml:83-109). Every file given is read, rewritten and re-read;
// then the first file is damaged in many ways (cut at every 61st byte, every header field overwritten with extreme
// values, trailer lengths inflated) and each damaged copy is parsed. Parsing may succeed or throw; what must not
// happen is a sanitizer report (any report aborts with a non-zero exit status).
// Usage: checkpoint_sanitize_check <scratch path> <checkpoint>...
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iterator>
#include <string>
#include <vector>

#include "../grad.cpp_b200/csrc/checkpoint.h"

static std::vector<char> slurp(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
static void spit(const std::string& path, const std::vector<char>& bytes) {
    std::ofstream f(path, std::ios::binary);
    f.write(bytes.data(), (std::streamsize)bytes.size());
}

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const std::string scratch = argv[1];
    int parsed = 0, rejected = 0;
    for (int i = 2; i < argc; i++) {
        const gradb::Checkpoint ck = gradb::read_checkpoint(argv[i], true);
        std::vector<const float*> ptrs;
        for (const auto& t : ck.tensors) ptrs.push_back(t.data());
        std::string err;
        if (!gradb::write_checkpoint(scratch, ck.desc, ptrs.data(), (int)ptrs.size(), err)) {
            std::printf("FAIL write: %s\n", err.c_str());
            return 1;
        }
        const gradb::Checkpoint back = gradb::read_checkpoint(scratch, true);
        if (back.tensors.size() != ck.tensors.size() || back.desc.vocab_size != ck.desc.vocab_size) {
            std::printf("FAIL round trip of %s\n", argv[i]);
            return 1;
        }
        for (size_t t = 0; t < ck.tensors.size(); t++) {
            if (back.tensors[t] != ck.tensors[t]) {
                std::printf("FAIL tensor %zu of %s changed\n", t, argv[i]);
                return 1;
            }
        }
        (void)gradb::read_checkpoint(argv[i], false);
        parsed++;
    }
    const std::vector<char> good = slurp(argv[2]);
    auto attempt = [&](const std::vector<char>& bytes) {
        spit(scratch, bytes);
        try {
            (void)gradb::read_checkpoint(scratch, true);
            parsed++;
        } catch (const std::exception&) {
            rejected++;
        }
    };
    for (size_t cut = 0; cut < good.size(); cut += 61) attempt(std::vector<char>(good.begin(), good.begin() + (long)cut));
    const int32_t extremes[] = {0, -1, 1, 0x7fffffff, (int32_t)0x80000000, 16777216, 16777217, 65536, 65537, 1 << 20};
    for (size_t off = 0; off + 4 <= 44 && off + 4 <= good.size(); off += 4) {
        for (int32_t v : extremes) {
            std::vector<char> bad = good;
            std::memcpy(bad.data() + off, &v, 4);
            attempt(bad);
        }
    }
    for (uint32_t len : {0u, 1u, 11u, 12u, 13u, 1u << 20, (1u << 20) + 1u, 0xffffffffu}) {  // trailers after a whole file
        std::vector<char> bad = good;
        const char tag[4] = {'T', 'K', 'F', 'P'};
        bad.insert(bad.end(), tag, tag + 4);
        bad.insert(bad.end(), reinterpret_cast<const char*>(&len), reinterpret_cast<const char*>(&len) + 4);
        bad.insert(bad.end(), 16, '\x5a');
        attempt(bad);
    }
    std::printf("parsed %d rejected %d\n", parsed, rejected);
    return 0;
}
