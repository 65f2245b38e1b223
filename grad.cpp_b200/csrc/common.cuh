// Shared declarations of the decode engine's CUDA translation units.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/gradb.h"
#include "checkpoint.h"

namespace gradb {

struct Error : std::runtime_error {
    gradb_status status;
    Error(gradb_status s, const std::string& what) : std::runtime_error(what), status(s) {}
};

#define GRADB_CUDA(expr)                                                                          \
    do {                                                                                          \
        cudaError_t _e = (expr);                                                                  \
        if (_e != cudaSuccess) {                                                                  \
            throw ::gradb::Error(GRADB_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
        }                                                                                         \
    } while (0)

extern std::atomic<uint64_t> g_kernel_launches;
// Set by the thread that is capturing a CUDA graph.
extern thread_local bool g_capturing;
inline void count_launch(uint64_t n = 1) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }

// Programmatic dependent launch: a kernel launched with this attribute may start while its
// predecessor on the stream is still running; it must execute pdl_wait() before touching anything
// the predecessor produces (or still reads). Predecessors call pdl_trigger() as early as they can.
// Set by the session code around the launches that may overlap (g_pdl is per host thread).
extern thread_local bool g_pdl;

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    GRADB_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}
#endif

// Diagnostics build (-DGRADB_DIAGNOSTICS, libgradb_diag.so): device-side index checks that record a code in the
// session's status word instead of making the access, a scan of outputs for non-finite values, the stage trace of
// the single-sequence kernel, overrides of tile and split choices, and a hook that makes one bounded device wait
// expire. None of it is compiled into the product library.
#if defined(GRADB_DIAGNOSTICS)
#define GRADB_DIAG 1
#define GRADB_INDEX_OK(cond, status, code) ((cond) ? true : ((status) ? (atomicExch((status), (code)), false) : false))
#else
#define GRADB_DIAG 0
#define GRADB_INDEX_OK(cond, status, code) (true)
#endif
// Status-word codes from 900 up are failed index checks; below that, bounded waits that expired.
constexpr int kIndexCheckCodes = 900;

// Sequences whose current token id is negative take no part in a step.
constexpr int kSkip = -1;
// Width of the repetition-penalty window (text_gen.cpp:22).
constexpr int kPenaltyWindow = 50;

// Per-layer device pointers. fp32 masters are always present; the bf16 copies
// only in GRADB_BF16 mode. Linear weights are (in, out) row-major as in the
// checkpoint (inference.cpp:13).
struct LayerWeights {
    const float *wq, *wk, *wv, *wo, *bq, *bk, *bv, *bo;
    const float *gate, *w1, *b1, *w2, *b2;
    const float *n1g, *n1b, *n2g, *n2b;
    const __nv_bfloat16 *wq16, *wk16, *wv16, *wo16, *gate16, *w116, *w216;
    // Tensor-core path (BF16 mode): transposed (out, in) bf16 copies and their TMA descriptors.
    // qkvT: [3d][d]; upT: modern [2*dff][d] with 128-row gate/up tiles interleaved, GPT-2 [dff][d];
    // downT: [d][dff].
    __nv_bfloat16 *qkvT = nullptr, *oT = nullptr, *upT = nullptr, *downT = nullptr;
    CUtensorMap map_qkv, map_o, map_up, map_down;
    // Tensor-core path (FP32 mode): the same transposed matrices as fp32 TF32 hi/lo pairs, [2][rows][in];
    // the maps cover both halves (the lo half starts `rows` rows down).
    float *qkvS = nullptr, *oS = nullptr, *upS = nullptr, *downS = nullptr;
    CUtensorMap map_qkvS, map_oS, map_upS, map_downS;
    int up_rows = 0;  // rows of one half of upS / upT
};

struct B1Plan;

struct DeviceModel {
    gradb_model_desc desc{};
    int device = 0;
    int precision = GRADB_FP32;
    float* blob = nullptr;           // every tensor, file order, fp32
    std::vector<size_t> offsets;     // element offset of each tensor in blob
    __nv_bfloat16* blob16 = nullptr; // bf16 copies of the matrices (BF16 mode)
    const float *emb = nullptr, *pos = nullptr, *fng = nullptr, *fnb = nullptr;
    const __nv_bfloat16* emb16 = nullptr;
    float* embS = nullptr;  // FP32 mode: embedding table as a TF32 hi/lo pair [2][V][d] (logits GEMM)
    std::vector<LayerWeights> layers;
    float* rope_cos = nullptr;  // [max_len][hs/2], host-computed with the reference's expressions
    float* rope_sin = nullptr;
    int sm_count = 148;
    bool tc_ok = false;   // shapes fit the tensor-core kernels (BF16 mode, d and d_ff multiples of 64)
    CUtensorMap map_emb;  // (V, d) bf16 embedding table = the logits GEMM's A operand
    bool tc32_ok = false;  // FP32 mode: TF32 hi/lo operands built (d and d_ff multiples of 64)
    CUtensorMap map_embS;  // (2V, d) fp32 hi/lo embedding table
    B1Plan* b1 = nullptr; // per-CTA weight tiles for the single-sequence persistent kernel
};

DeviceModel* upload_model(const gradb_model_desc& desc, const float* const* tensors, int n_tensors, int device,
                          int precision);
void free_model(DeviceModel* m);

}  // namespace gradb
