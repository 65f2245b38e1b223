// extern "C" surface declared in include/gradb.h. Exceptions stop here and
// become status codes plus a thread-local message.
#include <cmath>
#include <cstring>

#include "session.cuh"
#include "attn_prefill.cuh"
#if GRADB_DIAG
#include "gradb_diag.h"
#endif

using namespace gradb;

namespace {
thread_local std::string g_error;

template <typename F>
gradb_status guarded(F&& f) {
    try {
        f();
        return GRADB_OK;
    } catch (const Error& e) {
        g_error = e.what();
        return e.status;
    } catch (const std::exception& e) {
        g_error = e.what();
        return GRADB_ERR_INVALID;
    }
}

}  // namespace

struct gradb_model {
    DeviceModel* impl;
};
struct gradb_session {
    Session* impl;
};

extern "C" {

const char* gradb_last_error(void) { return g_error.c_str(); }
const char* gradb_version(void) { return "gradb 0.1 (sm_100a)"; }

gradb_status gradb_device_count(int* count_out) {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (count_out) *count_out = e == cudaSuccess ? n : 0;
    if (e != cudaSuccess || n == 0) {
        g_error = "no CUDA device available; this library has no CPU path";
        return GRADB_ERR_NO_DEVICE;
    }
    return GRADB_OK;
}

gradb_status gradb_checkpoint_inspect(const char* path, gradb_model_desc* desc_out) {
    try {
        const Checkpoint ck = read_checkpoint(path, false);
        if (desc_out) *desc_out = ck.desc;
        return GRADB_OK;
    } catch (const std::exception& e) {
        g_error = e.what();
        return GRADB_ERR_CHECKPOINT;
    }
}

gradb_status gradb_tensor_count(const gradb_model_desc* desc, int* count_out) {
    return guarded([&] {
        if (!desc || !count_out) throw Error(GRADB_ERR_INVALID, "null argument");
        gradb_model_desc d = *desc;
        d.d_ff = resolve_d_ff(d.d_model, d.arch == GRADB_ARCH_MODERN);
        *count_out = tensor_index(d).count;
    });
}

gradb_status gradb_tensor_shape(const gradb_model_desc* desc, int index, int* rows_out, int* cols_out) {
    return guarded([&] {
        if (!desc) throw Error(GRADB_ERR_INVALID, "null argument");
        gradb_model_desc d = *desc;
        d.d_ff = resolve_d_ff(d.d_model, d.arch == GRADB_ARCH_MODERN);
        const auto shapes = tensor_shapes(d);
        if (index < 0 || index >= (int)shapes.size()) throw Error(GRADB_ERR_INVALID, "tensor index out of range");
        if (rows_out) *rows_out = shapes[index].rows;
        if (cols_out) *cols_out = shapes[index].cols;
    });
}

gradb_status gradb_checkpoint_write(const char* path, const gradb_model_desc* desc, const float* const* tensors_host,
                                    int n_tensors) {
    return guarded([&] {
        if (!path || !desc || !tensors_host) throw Error(GRADB_ERR_INVALID, "null argument");
        gradb_model_desc d = *desc;
        d.d_ff = resolve_d_ff(d.d_model, d.arch == GRADB_ARCH_MODERN);
        std::string err;
        if (!write_checkpoint(path, d, tensors_host, n_tensors, err)) throw Error(GRADB_ERR_IO, err);
    });
}

gradb_status gradb_model_load(const char* path, int device, int precision, gradb_model** model_out) {
    if (!path || !model_out) {
        g_error = "null argument";
        return GRADB_ERR_INVALID;
    }
    Checkpoint ck;
    try {
        ck = read_checkpoint(path, true);
    } catch (const std::exception& e) {
        g_error = e.what();
        return GRADB_ERR_CHECKPOINT;
    }
    return guarded([&] {
        std::vector<const float*> ptrs;
        for (const auto& t : ck.tensors) ptrs.push_back(t.data());
        DeviceModel* m = upload_model(ck.desc, ptrs.data(), (int)ptrs.size(), device, precision);
        *model_out = new gradb_model{m};
    });
}

gradb_status gradb_model_from_host(const gradb_model_desc* desc, const float* const* tensors_host, int n_tensors,
                                   int device, int precision, gradb_model** model_out) {
    return guarded([&] {
        if (!desc || !tensors_host || !model_out) throw Error(GRADB_ERR_INVALID, "null argument");
        DeviceModel* m = upload_model(*desc, tensors_host, n_tensors, device, precision);
        *model_out = new gradb_model{m};
    });
}

gradb_status gradb_model_save(const gradb_model* model, const char* path) {
    return guarded([&] {
        if (!model || !path) throw Error(GRADB_ERR_INVALID, "null argument");
        const DeviceModel* m = model->impl;
        GRADB_CUDA(cudaSetDevice(m->device));
        const auto shapes = tensor_shapes(m->desc);
        std::vector<std::vector<float>> host(shapes.size());
        std::vector<const float*> ptrs(shapes.size());
        for (size_t i = 0; i < shapes.size(); i++) {
            host[i].resize((size_t)shapes[i].rows * shapes[i].cols);
            GRADB_CUDA(cudaMemcpy(host[i].data(), m->blob + m->offsets[i], host[i].size() * sizeof(float),
                                  cudaMemcpyDeviceToHost));
            ptrs[i] = host[i].data();
        }
        std::string err;
        if (!write_checkpoint(path, m->desc, ptrs.data(), (int)ptrs.size(), err)) throw Error(GRADB_ERR_IO, err);
    });
}

gradb_status gradb_model_describe(const gradb_model* model, gradb_model_desc* desc_out) {
    if (!model || !desc_out) {
        g_error = "null argument";
        return GRADB_ERR_INVALID;
    }
    *desc_out = model->impl->desc;
    return GRADB_OK;
}

void gradb_model_free(gradb_model* model) {
    if (!model) return;
    free_model(model->impl);
    delete model;
}

gradb_status gradb_session_create(const gradb_model* model, int max_batch, int max_len, void* stream,
                                  gradb_session** session_out) {
    return guarded([&] {
        if (!model || !session_out) throw Error(GRADB_ERR_INVALID, "null argument");
        *session_out = new gradb_session{create_session(model->impl, max_batch, max_len, stream)};
    });
}

void gradb_session_free(gradb_session* session) {
    if (!session) return;
    destroy_session(session->impl);
    delete session;
}

gradb_status gradb_session_reset(gradb_session* session) {
    return guarded([&] {
        if (!session) throw Error(GRADB_ERR_INVALID, "null session");
        reset_session(session->impl);
        GRADB_CUDA(cudaStreamSynchronize(session->impl->stream));
    });
}

gradb_status gradb_session_position(const gradb_session* session, int seq, int* position_out) {
    if (!session || !position_out || seq < 0 || seq >= session->impl->B) {
        g_error = "bad argument";
        return GRADB_ERR_INVALID;
    }
    *position_out = session->impl->h_pos[seq];
    return GRADB_OK;
}
int gradb_session_capacity(const gradb_session* session) { return session ? session->impl->T : 0; }
int gradb_session_vocab(const gradb_session* session) { return session ? session->impl->V : 0; }
int gradb_session_max_batch(const gradb_session* session) { return session ? session->impl->B : 0; }

gradb_status gradb_step(gradb_session* session, const int32_t* tokens_host, int n_seq, float* logits_host) {
    return guarded([&] {
        if (!session || !tokens_host) throw Error(GRADB_ERR_INVALID, "null argument");
        session_step(session->impl, tokens_host, n_seq, logits_host);
    });
}

gradb_status gradb_prefill(gradb_session* session, const int32_t* tokens_host, const int32_t* offsets_host, int n_seq,
                           float* logits_host) {
    return guarded([&] {
        if (!session || !tokens_host || !offsets_host) throw Error(GRADB_ERR_INVALID, "null argument");
        session_prefill(session->impl, tokens_host, offsets_host, n_seq, logits_host);
    });
}

gradb_status gradb_select(gradb_session* session, const gradb_sampling* params, const float* uniforms_host, int n_seq,
                          int32_t* tokens_host) {
    return guarded([&] {
        if (!session || !params || !tokens_host) throw Error(GRADB_ERR_INVALID, "null argument");
        session_select(session->impl, *params, nullptr, uniforms_host, n_seq, tokens_host, nullptr);
    });
}

gradb_status gradb_generate_stream(gradb_session* session, const int32_t* prompts_host, const int32_t* offsets_host,
                                   int n_seq, const gradb_sampling* params, int max_new, gradb_draw_fn draw,
                                   gradb_token_fn on_token, void* user, int32_t* emitted_host) {
    return guarded([&] {
        if (!session || !prompts_host || !offsets_host || !params) throw Error(GRADB_ERR_INVALID, "null argument");
        session_generate_stream(session->impl, prompts_host, offsets_host, n_seq, *params, max_new, draw, on_token, user,
                                emitted_host);
    });
}

gradb_status gradb_session_admit(gradb_session* session, int n_admit, const int32_t* seqs_host,
                                 const int32_t* prompts_host, const int32_t* offsets_host,
                                 const int32_t* max_new_host, const float* const* uniforms_host, int reuse_prefix,
                                 int32_t* reused_host) {
    return guarded([&] {
        if (!session || !seqs_host || !prompts_host || !offsets_host || !max_new_host) {
            throw Error(GRADB_ERR_INVALID, "null argument");
        }
        session_admit(session->impl, n_admit, seqs_host, prompts_host, offsets_host, max_new_host, uniforms_host,
                      reuse_prefix, reused_host);
    });
}

gradb_status gradb_session_decode(gradb_session* session, const gradb_sampling* params, int n_steps,
                                  const int32_t* stop_ids_host, int n_stop, int32_t* out_ids_host, int out_stride,
                                  int32_t* out_count_host, int32_t* finished_host) {
    return guarded([&] {
        if (!session || !params || !out_ids_host || !out_count_host) throw Error(GRADB_ERR_INVALID, "null argument");
        session_decode(session->impl, *params, n_steps, stop_ids_host, n_stop, out_ids_host, out_stride, out_count_host,
                       finished_host);
    });
}

gradb_status gradb_session_release(gradb_session* session, int seq) {
    return guarded([&] {
        if (!session) throw Error(GRADB_ERR_INVALID, "null session");
        session_release(session->impl, seq);
    });
}

gradb_status gradb_session_slot_ids(const gradb_session* session, int seq, int32_t* ids_host, int capacity,
                                    int* count_out) {
    return guarded([&] {
        if (!session || !count_out || (capacity > 0 && !ids_host)) throw Error(GRADB_ERR_INVALID, "null argument");
        *count_out = session_slot_ids(session->impl, seq, ids_host, capacity);
    });
}

gradb_status gradb_score(gradb_session* session, const int32_t* inputs_host, const int32_t* targets_host, int n_windows,
                         int seq_len, float* row_logp_host, float* ms_out) {
    return guarded([&] {
        if (!session || !inputs_host || !targets_host || !row_logp_host) throw Error(GRADB_ERR_INVALID, "null argument");
        const float ms = session_score(session->impl, inputs_host, targets_host, n_windows, seq_len, row_logp_host);
        if (ms_out) *ms_out = ms;
    });
}

gradb_status gradb_mean_loss(gradb_session* session, const int32_t* inputs_host, const int32_t* targets_host,
                             int n_windows, int seq_len, int batch_windows, double* mean_loss_out,
                             float* batch_loss_host, float* ms_out) {
    return guarded([&] {
        if (!session || !mean_loss_out) throw Error(GRADB_ERR_INVALID, "null argument");
        if (batch_windows < 1) throw Error(GRADB_ERR_INVALID, "batch_windows must be positive");
        if (n_windows <= 0) {
            *mean_loss_out = -1.0;  // no batches: trainer.cpp:339
            if (ms_out) *ms_out = 0.f;
            return;
        }
        if (!inputs_host || !targets_host) throw Error(GRADB_ERR_INVALID, "null argument");
        std::vector<float> logp((size_t)n_windows * seq_len);
        const float ms = session_score(session->impl, inputs_host, targets_host, n_windows, seq_len, logp.data());
        double weighted = 0.0;
        size_t windows = 0;
        int batch = 0;
        for (int w0 = 0; w0 < n_windows; w0 += batch_windows, batch++) {
            const size_t nb = (size_t)std::min(batch_windows, n_windows - w0);
            const size_t rows = nb * (size_t)seq_len;
            const float* lp = logp.data() + (size_t)w0 * seq_len;
            float total = 0.0f;
            for (size_t r = 0; r < rows; r++) total -= lp[r];  // rows outside the vocabulary hold 0
            total /= static_cast<float>(rows);
            if (batch_loss_host) batch_loss_host[batch] = total;
            weighted += static_cast<double>(total) * static_cast<double>(nb);
            windows += nb;
        }
        *mean_loss_out = weighted / static_cast<double>(windows);
        if (ms_out) *ms_out = ms;
    });
}

gradb_status gradb_session_set_history(gradb_session* session, int seq, const int32_t* ids_host, int n) {
    return guarded([&] {
        if (!session || (!ids_host && n > 0)) throw Error(GRADB_ERR_INVALID, "null argument");
        session_set_history(session->impl, seq, ids_host, n);
    });
}

gradb_status gradb_select_from_logits(gradb_session* session, const gradb_sampling* params, const float* logits_host,
                                      const float* uniforms_host, int n_seq, int32_t* tokens_host, float* probs_host) {
    return guarded([&] {
        if (!session || !params || !logits_host || !tokens_host) throw Error(GRADB_ERR_INVALID, "null argument");
        session_select(session->impl, *params, logits_host, uniforms_host, n_seq, tokens_host, probs_host);
    });
}

gradb_status gradb_generate(gradb_session* session, const int32_t* prompts_host, const int32_t* offsets_host, int n_seq,
                            const gradb_sampling* params, int max_new, const float* uniforms_host,
                            int32_t* out_ids_host, int out_stride, int32_t* out_len_host, float* step_ms_host,
                            float* prefill_ms_host) {
    return guarded([&] {
        if (!session || !prompts_host || !offsets_host || !params || !out_ids_host || !out_len_host) {
            throw Error(GRADB_ERR_INVALID, "null argument");
        }
        session_generate(session->impl, prompts_host, offsets_host, n_seq, *params, max_new, uniforms_host,
                         out_ids_host, out_stride, out_len_host, step_ms_host, prefill_ms_host);
    });
}

gradb_status gradb_session_last_ms(const gradb_session* session, float* ms_out) {
    if (!session || !ms_out) {
        g_error = "null argument";
        return GRADB_ERR_INVALID;
    }
    *ms_out = session->impl->last_ms;
    return GRADB_OK;
}

gradb_status gradb_session_cache_row(gradb_session* session, int seq, int layer, int which, int pos, float* row_host) {
    return guarded([&] {
        if (!session || !row_host) throw Error(GRADB_ERR_INVALID, "null argument");
        session_cache_row(session->impl, seq, layer, which, pos, row_host);
    });
}

gradb_status gradb_attention_decode(const float* q_dev, const float* kcache_dev, const float* vcache_dev,
                                    const int32_t* pos_dev, int n_seq, int heads, int head_dim, int max_len,
                                    int splits, float* out_dev, void* stream) {
    return guarded([&] {
        if (!q_dev || !kcache_dev || !vcache_dev || !pos_dev || !out_dev) throw Error(GRADB_ERR_INVALID, "null argument");
        if (n_seq < 1 || heads < 1 || max_len < 1 || splits < 1 || splits > 64) {
            throw Error(GRADB_ERR_INVALID, "bad attention shape");
        }
        if (head_dim != 64) throw Error(GRADB_ERR_INVALID, "the stand-alone attention entry point supports head_dim 64");
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        float* partial = nullptr;
        int* counters = nullptr;
        const size_t units = (size_t)n_seq * heads;
        GRADB_CUDA(cudaMalloc(&partial, units * splits * (head_dim + 2) * sizeof(float)));
        if (cudaMalloc(&counters, units * sizeof(int)) != cudaSuccess) {
            cudaFree(partial);
            throw Error(GRADB_ERR_CUDA, "cudaMalloc failed");
        }
        try {
            GRADB_CUDA(cudaMemsetAsync(counters, 0, units * sizeof(int), st));
            AttnParams a{};
            a.q = q_dev; a.kcache = kcache_dev; a.vcache = vcache_dev;
            a.tok = pos_dev;  // every sequence takes part: positions are never negative
            a.pos = pos_dev;
            a.out = out_dev; a.out16 = nullptr; a.partial = partial; a.counters = counters;
            a.H = heads; a.hs = head_dim; a.T = max_len; a.d = heads * head_dim;
            a.scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
            launch_attention(a, n_seq, splits, st);
            GRADB_CUDA(cudaStreamSynchronize(st));
        } catch (...) {
            cudaFree(partial);
            cudaFree(counters);
            throw;
        }
        cudaFree(partial);
        cudaFree(counters);
    });
}

gradb_status gradb_attention_decode_static(const float* q_dev, const float* kcache_dev, const float* vcache_dev,
                                           const int32_t* pos_dev, int n_seq, int heads, int head_dim, int max_len,
                                           int splits, float* out_dev, void* stream) {
    return guarded([&] {
        if (!q_dev || !kcache_dev || !vcache_dev || !pos_dev || !out_dev) throw Error(GRADB_ERR_INVALID, "null argument");
        if (n_seq < 1 || heads < 1 || max_len < 1 || splits < 1 || splits > 64) {
            throw Error(GRADB_ERR_INVALID, "bad attention shape");
        }
        AttnParams a{};
        a.q = q_dev; a.kcache = kcache_dev; a.vcache = vcache_dev;
        a.tok = pos_dev;  // every sequence takes part: positions are never negative
        a.pos = pos_dev;
        a.out = out_dev; a.out16 = nullptr;
        a.H = heads; a.hs = head_dim; a.T = max_len; a.d = heads * head_dim;
        a.scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
        launch_attention_static(a, n_seq, splits, static_cast<cudaStream_t>(stream));
    });
}

int gradb_attention_static_capacity(void) { return static_attention_capacity(); }

gradb_status gradb_session_set_profiling(gradb_session* session, int on) {
    return guarded([&] {
        if (!session) throw Error(GRADB_ERR_INVALID, "null session");
        session_set_profiling(session->impl, on != 0);
    });
}

int gradb_kernel_class_count(void) { return kKernelClasses; }

const char* gradb_kernel_class_name(int cls) {
    static const char* const names[kKernelClasses] = {"embed",    "norm_qkv_rope", "attn_decode", "attn_out_proj", "norm_ffn_up",
                                                      "ffn_down", "norm_logits",   "advance",     "select",        "decode_step_b1",
                                                      "score_logp"};
    return cls >= 0 && cls < kKernelClasses ? names[cls] : "";
}

gradb_status gradb_session_profile(const gradb_session* session, double* ms_out, uint64_t* launches_out) {
    if (!session || !ms_out || !launches_out) {
        g_error = "null argument";
        return GRADB_ERR_INVALID;
    }
    for (int i = 0; i < kKernelClasses; i++) {
        ms_out[i] = session->impl->class_ms[i];
        launches_out[i] = session->impl->class_launches[i];
    }
    return GRADB_OK;
}

#if GRADB_DIAG
// ---- diagnostics build only (declared in csrc/gradb_diag.h) ------------------------------------------------------
gradb_status gradb_session_stage_trace(gradb_session* session, uint64_t* stamps_out, int capacity, int* count_out) {
    return guarded([&] {
        if (!session || !stamps_out || !count_out) throw Error(GRADB_ERR_INVALID, "null argument");
        Session* s = session->impl;
        *count_out = 0;
        if (!s->b1_trace) return;
        GRADB_CUDA(cudaSetDevice(s->m->device));
        GRADB_CUDA(cudaStreamSynchronize(s->stream));
        std::vector<unsigned long long> host(1024);
        GRADB_CUDA(cudaMemcpy(host.data(), s->b1_trace, host.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        int n = 0;
        while (n < 1024 && n < capacity && host[n] != 0) {
            stamps_out[n] = host[n];
            n++;
        }
        *count_out = n;
    });
}

gradb_status gradb_diag_attention_wait(gradb_session* session, unsigned spin_limit, int skip_tile) {
    return guarded([&] {
        if (!session) throw Error(GRADB_ERR_INVALID, "null session");
        session->impl->diag_spin_limit = spin_limit;
        session->impl->diag_skip_tile = skip_tile;
        // the decode graphs bake kernel parameters: drop them so that the next loop captures the new ones
        Session* s = session->impl;
        if (s->graph) {
            cudaGraphExecDestroy(s->graph);
            s->graph = nullptr;
        }
        if (s->serve_graph) {
            cudaGraphExecDestroy(s->serve_graph);
            s->serve_graph = nullptr;
        }
    });
}

gradb_status gradb_diag_count_nonfinite(gradb_session* session, int n_seq, long long* count_out) {
    return guarded([&] {
        if (!session || !count_out) throw Error(GRADB_ERR_INVALID, "null argument");
        Session* s = session->impl;
        if (n_seq < 1 || n_seq > s->B) throw Error(GRADB_ERR_INVALID, "n_seq out of range for this session");
        GRADB_CUDA(cudaSetDevice(s->m->device));
        *count_out = count_nonfinite(s->logits, (size_t)n_seq * s->V, s->stream) +
                     count_nonfinite(s->x, (size_t)n_seq * s->d, s->stream);
    });
}

gradb_status gradb_diag_wide_clocks(uint64_t* out128, int reset) {
    return guarded([&] {
        if (!out128) throw Error(GRADB_ERR_INVALID, "null argument");
        unsigned long long v[128];
        wide_clocks_read(v, reset != 0);
        for (int i = 0; i < 128; i++) out128[i] = v[i];
    });
}

gradb_status gradb_diag_attn_clocks(uint64_t* out16, int reset) {
    return guarded([&] {
        if (!out16) throw Error(GRADB_ERR_INVALID, "null argument");
        unsigned long long v[16];
        attn_clocks_read(v, reset != 0);
        for (int i = 0; i < 16; i++) out16[i] = v[i];
    });
}

gradb_status gradb_diag_select_clocks(uint64_t* out16, int reset) {
    return guarded([&] {
        if (!out16) throw Error(GRADB_ERR_INVALID, "null argument");
        unsigned long long v[16];
        select_clocks_read(v, reset != 0);
        for (int i = 0; i < 16; i++) out16[i] = v[i];
    });
}

gradb_status gradb_diag_poke_history(gradb_session* session, int seq, int index, int32_t id) {
    return guarded([&] {
        if (!session) throw Error(GRADB_ERR_INVALID, "null session");
        Session* s = session->impl;
        if (seq < 0 || seq >= s->B || index < 0 || index >= s->hist_stride) throw Error(GRADB_ERR_INVALID, "bad index");
        GRADB_CUDA(cudaSetDevice(s->m->device));
        GRADB_CUDA(cudaMemcpy(s->hist + (size_t)seq * s->hist_stride + index, &id, sizeof(int), cudaMemcpyHostToDevice));
    });
}
#endif  // GRADB_DIAG

uint64_t gradb_kernel_launches(void) { return g_kernel_launches.load(); }

}  // extern "C"
