// Places a model's weights in HBM.
#include <cmath>

#include "common.cuh"
#include "decode_b1.cuh"
#include "gemm_tc.cuh"

namespace gradb {

std::atomic<uint64_t> g_kernel_launches{0};
thread_local bool g_capturing = false;
thread_local bool g_pdl = false;

namespace {
__global__ void to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}
}  // namespace

DeviceModel* upload_model(const gradb_model_desc& desc_in, const float* const* tensors, int n_tensors, int device,
                          int precision) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        throw Error(GRADB_ERR_NO_DEVICE, "no CUDA device available; this library has no CPU path");
    }
    if (device < 0 || device >= ndev) throw Error(GRADB_ERR_INVALID, "device index out of range");
    if (precision != GRADB_FP32 && precision != GRADB_BF16) throw Error(GRADB_ERR_INVALID, "unknown precision mode");
    gradb_model_desc desc = desc_in;
    const bool modern = desc.arch == GRADB_ARCH_MODERN;
    desc.d_ff = resolve_d_ff(desc.d_model, modern);
    const int d = desc.d_model, hs = d / desc.num_heads;
    if (d % 4 != 0 || desc.d_ff % 4 != 0) throw Error(GRADB_ERR_INVALID, "d_model must be a multiple of 4");
    if (hs % 2 != 0 || hs > 256) throw Error(GRADB_ERR_INVALID, "head size must be even and at most 256");
    const std::vector<TensorShape> shapes = tensor_shapes(desc);
    if ((int)shapes.size() != n_tensors) throw Error(GRADB_ERR_INVALID, "wrong tensor count for this model shape");

    GRADB_CUDA(cudaSetDevice(device));
    auto* m = new DeviceModel();
    try {
        m->desc = desc;
        m->device = device;
        m->precision = precision;
        cudaDeviceProp prop{};
        GRADB_CUDA(cudaGetDeviceProperties(&prop, device));
        m->sm_count = prop.multiProcessorCount;

        // Every tensor starts on a 256-byte boundary so vector loads and bulk copies are aligned.
        size_t total = 0;
        m->offsets.resize(shapes.size());
        for (size_t i = 0; i < shapes.size(); i++) {
            m->offsets[i] = total;
            total += ((size_t)shapes[i].rows * shapes[i].cols + 63) / 64 * 64;
        }
        GRADB_CUDA(cudaMalloc(&m->blob, total * sizeof(float)));
        for (size_t i = 0; i < shapes.size(); i++) {
            GRADB_CUDA(cudaMemcpy(m->blob + m->offsets[i], tensors[i],
                                  sizeof(float) * (size_t)shapes[i].rows * shapes[i].cols, cudaMemcpyHostToDevice));
        }
        if (precision == GRADB_BF16) {
            GRADB_CUDA(cudaMalloc(&m->blob16, total * sizeof(__nv_bfloat16)));
            to_bf16_kernel<<<1024, 256>>>(m->blob, m->blob16, total);
            count_launch();
            GRADB_CUDA(cudaGetLastError());
        }
        const TensorIndex ix = tensor_index(desc);
        auto P = [&](int i) -> const float* { return i < 0 ? nullptr : m->blob + m->offsets[i]; };
        auto H = [&](int i) -> const __nv_bfloat16* {
            return (i < 0 || !m->blob16) ? nullptr : m->blob16 + m->offsets[i];
        };
        m->emb = P(ix.emb);
        m->emb16 = H(ix.emb);
        m->pos = P(ix.pos);
        m->fng = P(ix.final_g);
        m->fnb = P(ix.final_b);
        m->layers.resize(desc.num_layers);
        for (int l = 0; l < desc.num_layers; l++) {
            const int b = ix.layer0 + l * ix.per_layer;
            auto at = [&](int o) { return o < 0 ? -1 : b + o; };
            LayerWeights& w = m->layers[l];
            w.wq = P(at(ix.wq)); w.wk = P(at(ix.wk)); w.wv = P(at(ix.wv)); w.wo = P(at(ix.wo));
            w.bq = P(at(ix.bq)); w.bk = P(at(ix.bk)); w.bv = P(at(ix.bv)); w.bo = P(at(ix.bo));
            w.gate = P(at(ix.gate)); w.w1 = P(at(ix.w1)); w.b1 = P(at(ix.b1));
            w.w2 = P(at(ix.w2)); w.b2 = P(at(ix.b2));
            w.n1g = P(at(ix.n1g)); w.n1b = P(at(ix.n1b)); w.n2g = P(at(ix.n2g)); w.n2b = P(at(ix.n2b));
            w.wq16 = H(at(ix.wq)); w.wk16 = H(at(ix.wk)); w.wv16 = H(at(ix.wv)); w.wo16 = H(at(ix.wo));
            w.gate16 = H(at(ix.gate)); w.w116 = H(at(ix.w1)); w.w216 = H(at(ix.w2));
        }
        m->tc_ok = precision == GRADB_BF16 && d % 64 == 0 && desc.d_ff % 64 == 0;
        if (m->tc_ok) {
            const int f = desc.d_ff;
            for (int l = 0; l < desc.num_layers; l++) {
                LayerWeights& w = m->layers[l];
                const size_t up_rows = modern ? (size_t)((f + 127) / 128) * 256 : (size_t)f;
                GRADB_CUDA(cudaMalloc(&w.qkvT, (size_t)3 * d * d * 2));
                GRADB_CUDA(cudaMalloc(&w.oT, (size_t)d * d * 2));
                GRADB_CUDA(cudaMalloc(&w.upT, up_rows * d * 2));
                GRADB_CUDA(cudaMalloc(&w.downT, (size_t)d * f * 2));
                GRADB_CUDA(cudaMemset(w.upT, 0, up_rows * d * 2));
                launch_transpose_bf16(w.wq, w.qkvT, d, d, 0, false, nullptr);
                launch_transpose_bf16(w.wk, w.qkvT, d, d, d, false, nullptr);
                launch_transpose_bf16(w.wv, w.qkvT, d, d, 2 * d, false, nullptr);
                launch_transpose_bf16(w.wo, w.oT, d, d, 0, false, nullptr);
                if (modern) {
                    launch_transpose_bf16(w.gate, w.upT, d, f, 0, true, nullptr);
                    launch_transpose_bf16(w.w1, w.upT, d, f, 128, true, nullptr);
                } else {
                    launch_transpose_bf16(w.w1, w.upT, d, f, 0, false, nullptr);
                }
                launch_transpose_bf16(w.w2, w.downT, f, d, 0, false, nullptr);
                make_tensor_map_bf16(&w.map_qkv, w.qkvT, (uint64_t)3 * d, d, 128);
                make_tensor_map_bf16(&w.map_o, w.oT, d, d, 128);
                make_tensor_map_bf16(&w.map_up, w.upT, up_rows, d, 128);
                make_tensor_map_bf16(&w.map_down, w.downT, d, f, 128);
            }
            make_tensor_map_bf16(&m->map_emb, m->emb16, desc.vocab_size, d, 128);
        }
        m->tc32_ok = precision == GRADB_FP32 && d % 64 == 0 && desc.d_ff % 64 == 0;
        if (m->tc32_ok) {
            // fp32 mode on the tensor cores: every weight as a TF32 hi/lo pair, transposed like the bf16 copies
            const int f = desc.d_ff;
            for (int l = 0; l < desc.num_layers; l++) {
                LayerWeights& w = m->layers[l];
                const size_t up_rows = modern ? (size_t)((f + 127) / 128) * 256 : (size_t)f;
                w.up_rows = (int)up_rows;
                GRADB_CUDA(cudaMalloc(&w.qkvS, (size_t)2 * 3 * d * d * 4));
                GRADB_CUDA(cudaMalloc(&w.oS, (size_t)2 * d * d * 4));
                GRADB_CUDA(cudaMalloc(&w.upS, 2 * up_rows * d * 4));
                GRADB_CUDA(cudaMalloc(&w.downS, (size_t)2 * d * f * 4));
                GRADB_CUDA(cudaMemset(w.upS, 0, 2 * up_rows * d * 4));
                const size_t lo_qkv = (size_t)3 * d * d, lo_o = (size_t)d * d, lo_up = up_rows * d, lo_down = (size_t)d * f;
                launch_transpose_split(w.wq, w.qkvS, lo_qkv, d, d, 0, false, nullptr);
                launch_transpose_split(w.wk, w.qkvS, lo_qkv, d, d, d, false, nullptr);
                launch_transpose_split(w.wv, w.qkvS, lo_qkv, d, d, 2 * d, false, nullptr);
                launch_transpose_split(w.wo, w.oS, lo_o, d, d, 0, false, nullptr);
                if (modern) {
                    launch_transpose_split(w.gate, w.upS, lo_up, d, f, 0, true, nullptr);
                    launch_transpose_split(w.w1, w.upS, lo_up, d, f, 128, true, nullptr);
                } else {
                    launch_transpose_split(w.w1, w.upS, lo_up, d, f, 0, false, nullptr);
                }
                launch_transpose_split(w.w2, w.downS, lo_down, f, d, 0, false, nullptr);
                make_tensor_map_f32(&w.map_qkvS, w.qkvS, (uint64_t)2 * 3 * d, d, 128);
                make_tensor_map_f32(&w.map_oS, w.oS, (uint64_t)2 * d, d, 128);
                make_tensor_map_f32(&w.map_upS, w.upS, 2 * up_rows, d, 128);
                make_tensor_map_f32(&w.map_downS, w.downS, (uint64_t)2 * d, f, 128);
            }
            const size_t emb_elems = (size_t)desc.vocab_size * d;
            GRADB_CUDA(cudaMalloc(&m->embS, 2 * emb_elems * 4));
            launch_split_tf32(m->emb, m->embS, emb_elems, emb_elems, nullptr);
            make_tensor_map_f32(&m->map_embS, m->embS, (uint64_t)2 * desc.vocab_size, d, 128);
        }
        if (modern) {
            // RoPE angles, computed with the reference's own float expressions
            // (inference.cpp:169-175) on the host so that cos/sin bits are libm's.
            const int half = hs / 2;
            std::vector<float> c((size_t)desc.max_len * half), s((size_t)desc.max_len * half);
            for (int p = 0; p < desc.max_len; p++) {
                for (int j = 0; j < half; j++) {
                    const float theta = std::pow(10000.0f, -2.0f * static_cast<float>(j) / static_cast<float>(hs));
                    c[(size_t)p * half + j] = std::cos(static_cast<float>(p) * theta);
                    s[(size_t)p * half + j] = std::sin(static_cast<float>(p) * theta);
                }
            }
            GRADB_CUDA(cudaMalloc(&m->rope_cos, c.size() * sizeof(float)));
            GRADB_CUDA(cudaMalloc(&m->rope_sin, s.size() * sizeof(float)));
            GRADB_CUDA(cudaMemcpy(m->rope_cos, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice));
            GRADB_CUDA(cudaMemcpy(m->rope_sin, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice));
        }
        GRADB_CUDA(cudaDeviceSynchronize());
        m->b1 = b1_make_plan(m);
        return m;
    } catch (...) {
        free_model(m);
        throw;
    }
}

void free_model(DeviceModel* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    b1_free_plan(m->b1);
    cudaFree(m->blob);
    cudaFree(m->blob16);
    cudaFree(m->embS);
    for (LayerWeights& w : m->layers) {
        cudaFree(w.qkvS); cudaFree(w.oS); cudaFree(w.upS); cudaFree(w.downS);
        cudaFree(w.qkvT);
        cudaFree(w.oT);
        cudaFree(w.upT);
        cudaFree(w.downT);
    }
    cudaFree(m->rope_cos);
    cudaFree(m->rope_sin);
    delete m;
}

}  // namespace gradb
