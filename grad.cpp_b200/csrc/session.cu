#include "session.cuh"

#include "attn_prefill.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace gradb {

namespace {

template <typename T>
void dalloc(T** p, size_t n) {
    GRADB_CUDA(cudaMalloc(reinterpret_cast<void**>(p), std::max<size_t>(n, 1) * sizeof(T)));
}

size_t layer_cache_elems(const Session* s) { return (size_t)s->B * s->H * s->T * s->hs; }

// Brackets one launch with events when profiling is on.
struct Timed {
    Session* s;
    int idx = -1;
    Timed(Session* s_, int cls) : s(s_) {
        if (!s->profiling || g_capturing) return;
        auto take = [&] {
            cudaEvent_t e;
            if (s->event_pool.empty()) {
                GRADB_CUDA(cudaEventCreate(&e));
            } else {
                e = s->event_pool.back();
                s->event_pool.pop_back();
            }
            return e;
        };
        Session::Span sp{cls, take(), take()};
        cudaEventRecord(sp.a, s->stream);
        idx = (int)s->spans.size();
        s->spans.push_back(sp);
    }
    ~Timed() {
        if (idx >= 0) cudaEventRecord(s->spans[idx].b, s->stream);
    }
};

// After a stream synchronise: a kernel whose bounded wait expired left a code in the status word.
void check_status(Session* s) {
    int code = 0;
    GRADB_CUDA(cudaMemcpy(&code, s->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0) {
        // The kernels that gave up left their arrival tickets and barrier words half-way; start them afresh so the
        // session stays usable.
        cudaMemset(s->status, 0, sizeof(int));
        cudaMemset(s->attn_counters, 0, (size_t)s->B * s->H * sizeof(int));
        if (s->b1_ws) cudaMemset(s->b1_ws, 0, s->b1_ws_bytes);
        if (code >= kIndexCheckCodes) {
            throw Error(GRADB_ERR_INVALID, "a device-side index check failed (code " + std::to_string(code) + ")");
        }
        throw Error(GRADB_ERR_DEVICE_WAIT, "a device-side wait expired (code " + std::to_string(code) + ")");
    }
}

// After a stream synchronise: fold the recorded spans into per-class totals.
void collect_spans(Session* s) {
    for (const Session::Span& sp : s->spans) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) {
            s->class_ms[sp.cls] += ms;
            s->class_launches[sp.cls] += 1;
        }
        s->event_pool.push_back(sp.a);
        s->event_pool.push_back(sp.b);
    }
    s->spans.clear();
}

// Enqueues one decode step for rows 0..n_seq-1. tok_dev: current ids (<0 = skip row).
// logit_tok_dev: same convention, selects which rows get logits (the prompt feed
// only needs them at each sequence's last position).
// Tensor-core variant of a step: every projection is a TMA-fed tcgen05 GEMM over all
// sequences; norms produce the bf16 operand, attention stays the streaming kernel.
// Scope in which launches carry the programmatic-dependent-launch attribute.
struct PdlScope {
    bool prev;
    explicit PdlScope(bool on) : prev(g_pdl) { g_pdl = on; }
    ~PdlScope() { g_pdl = prev; }
};

void enqueue_step_tc(Session* s, int n_seq, const int* tok_dev, const int* logit_tok_dev, bool append_history) {
    const DeviceModel* m = s->m;
    const bool modern = m->desc.arch == GRADB_ARCH_MODERN;
    cudaStream_t st = s->stream;
    const int d = s->d, f = s->dff;
    const int want = m->sm_count * 3 / 4;
    auto tile_for = [&](int n_features) { return tc_token_tile(n_seq, (n_features + 127) / 128, want); };
    auto map_idx = [](int tn) { return tn == 32 ? 0 : (tn == 64 ? 1 : 2); };
    auto splits = [&](int n_features, int tn, int k_iters) {
        const int ctas = ((n_features + 127) / 128) * ((n_seq + tn - 1) / tn);
        int ks = 1;
        while (ks < 8 && ctas * ks * 2 <= m->sm_count * 3 / 2 && k_iters / (ks * 2) >= 2) ks *= 2;
        return ks;
    };
    {
        Timed t(s, KC_EMBED);
        launch_embed(m->emb, modern ? nullptr : m->pos, tok_dev, s->pos, s->x, d, n_seq, st);
    }
    // Every kernel of the step after the first may begin (its set-up, and for the GEMMs the weight
    // stream) while its predecessor drains; each waits for the predecessor before touching its data.
    PdlScope pdl(s->use_pdl && !s->profiling);
    // fp32 sessions run the same kernels on TF32 hi/lo operand pairs (three MMAs per product)
    const bool s32 = s->use_tc32;
    const int kind = s32 ? 1 : 0;
    const size_t lo_d = (size_t)s->split_rows * d, lo_f = (size_t)s->split_rows * f;
    auto norm_rows = [&](const float* g, const float* b, const int* tk) {
        if (s32) launch_norm_split(s->x, g, b, tk, s->hS, lo_d, d, modern, 1e-5f, n_seq, st);
        else launch_norm_bf16(s->x, g, b, tk, s->h16, d, modern, 1e-5f, n_seq, st);
    };
    TcGemmParams base{};
    base.B = n_seq; base.d = d; base.H = s->H; base.hs = s->hs; base.T = s->T;
    base.tok = tok_dev; base.pos = s->pos; base.status = s->status;
    base.b_lo_rows = s->split_rows;
    for (int l = 0; l < s->L; l++) {
        const LayerWeights& w = m->layers[l];
        float* kc = s->kcache + (size_t)l * layer_cache_elems(s);
        float* vc = s->vcache + (size_t)l * layer_cache_elems(s);
        {
            Timed t(s, KC_QKV);
            norm_rows(w.n1g, w.n1b, tok_dev);
            TcGemmParams g = base;
            g.K = d; g.N = 3 * d; g.ld_out = d; g.a_lo_rows = 3 * d;
            g.bias[0] = w.bq; g.bias[1] = w.bk; g.bias[2] = w.bv;
            g.rope_cos = modern ? m->rope_cos : nullptr;
            g.rope_sin = modern ? m->rope_sin : nullptr;
            g.out_f32 = s->q; g.kcache = kc; g.vcache = vc;
            const int tn = tile_for(3 * d);
            launch_tc_gemm(TC_QKV, s32 ? w.map_qkvS : w.map_qkv, s->map_h16[map_idx(tn)], g, tn, 1, st, kind);
        }
        {
            Timed t(s, KC_ATTN);
            AttnParams a{};
            a.q = s->q; a.kcache = kc; a.vcache = vc; a.tok = tok_dev; a.pos = s->pos;
            a.out = s->attn; a.out16 = s32 ? nullptr : s->attn16; a.partial = s->attn_partial; a.counters = s->attn_counters;
            a.status = s->status;
            a.H = s->H; a.hs = s->hs; a.T = s->T; a.d = d;
            a.scale = 1.0f / std::sqrt(static_cast<float>(s->hs));
            a.diag_spin_limit = s->diag_spin_limit; a.diag_skip_tile = s->diag_skip_tile;
            const bool split_inside = s32 && s->hs == 64;  // the pipelined kernel writes the hi/lo operand itself
            if (split_inside) { a.out_split = s->attnS; a.out_lo_elems = lo_d; }
            launch_attention(a, n_seq, s->attn_splits, st);
            if (s32 && !split_inside) launch_split_tf32(s->attn, s->attnS, lo_d, (size_t)n_seq * d, st);
        }
        {
            Timed t(s, KC_OPROJ);
            TcGemmParams g = base;
            g.K = d; g.N = d; g.ld_out = d; g.bias[0] = w.bo; g.out_f32 = s->x; g.a_lo_rows = d;
            const int tn = tile_for(d);
            launch_tc_gemm(TC_RESID, s32 ? w.map_oS : w.map_o, s->map_attn16[map_idx(tn)], g, tn,
                           splits(d, tn, d / (s32 ? 32 : 64)), st, kind);
        }
        {
            Timed t(s, KC_FFN_UP);
            norm_rows(w.n2g, w.n2b, tok_dev);
            TcGemmParams g = base;
            g.K = d; g.N = f; g.ld_out = f; g.out_bf16 = s->ffn16; g.out_split = s->ffnS; g.out_lo_elems = lo_f;
            g.a_lo_rows = w.up_rows;
            g.bias[0] = modern ? nullptr : w.b1;
            const int tn = tile_for(f);
            launch_tc_gemm(modern ? TC_SWIGLU : TC_GELU, s32 ? w.map_upS : w.map_up, s->map_h16[map_idx(tn)], g, tn, 1, st,
                           kind);
        }
        {
            Timed t(s, KC_FFN_DOWN);
            TcGemmParams g = base;
            g.K = f; g.N = d; g.ld_out = d; g.bias[0] = modern ? nullptr : w.b2; g.out_f32 = s->x; g.a_lo_rows = d;
            const int tn = tile_for(d);
            launch_tc_gemm(TC_RESID, s32 ? w.map_downS : w.map_down, s->map_ffn16[map_idx(tn)], g, tn,
                           splits(d, tn, f / (s32 ? 32 : 64)), st, kind);
        }
    }
    {
        Timed t(s, KC_LOGITS);
        norm_rows(m->fng, m->fnb, logit_tok_dev);
        TcGemmParams g = base;
        g.tok = logit_tok_dev;
        g.K = d; g.N = s->V; g.ld_out = s->V; g.out_f32 = s->logits; g.a_lo_rows = s->V;
        const int tn = tile_for(s->V);
        launch_tc_gemm(TC_LOGITS, s32 ? m->map_embS : m->map_emb, s->map_h16[map_idx(tn)], g, tn, 1, st, kind);
    }
    Timed t(s, KC_ADVANCE);
    launch_advance(tok_dev, s->pos, append_history ? s->hist : nullptr, s->hist_len, s->hist_stride, n_seq, st);
}

// The whole step of a single sequence as one persistent kernel.
void enqueue_step_b1(Session* s, const int* tok_dev, const int* logit_tok_dev, bool append_history) {
    const DeviceModel* m = s->m;
    const B1Plan* plan = m->b1;
    const bool modern = m->desc.arch == GRADB_ARCH_MODERN;
    B1Params p{};
    p.G = plan->G; p.d = s->d; p.dff = s->dff; p.H = s->H; p.hs = s->hs; p.V = s->V; p.L = s->L; p.T = s->T;
    p.modern = modern; p.wbytes = plan->wbytes;
    p.qkv = plan->qkv; p.o = plan->o; p.up = plan->up; p.down = plan->down;
    p.logit_rows_per_cta = plan->logit_rows_per_cta; p.logit_chunk_rows = plan->logit_chunk_rows;
    p.attn_splits = plan->attn_splits;
    p.layers = plan->layers_dev;
    p.emb32 = m->emb;
    p.emb_w = plan->wbytes == 2 ? (const void*)m->emb16 : (const void*)m->emb;
    p.pos_emb = modern ? nullptr : m->pos;
    p.fng = m->fng; p.fnb = m->fnb;
    p.rope_cos = modern ? m->rope_cos : nullptr;
    p.rope_sin = modern ? m->rope_sin : nullptr;
    p.kcache = s->kcache; p.vcache = s->vcache;
    p.layer_cache_stride = layer_cache_elems(s);
    b1_bind_workspace(p, s->b1_ws, m, plan);
    p.logits = s->logits;
    p.tok = tok_dev; p.logit_tok = logit_tok_dev;
    p.pos = s->pos; p.hist = s->hist; p.hist_len = s->hist_len;
    p.hist_stride = s->hist_stride; p.append_hist = append_history ? 1 : 0;
    p.status = s->status;
    p.trace = s->b1_trace;
    Timed t(s, KC_STEP_B1);
    launch_decode_b1(p, s->stream);
}

void enqueue_step(Session* s, int n_seq, const int* tok_dev, const int* logit_tok_dev, bool append_history) {
    if (s->use_b1 && n_seq == 1) {
        enqueue_step_b1(s, tok_dev, logit_tok_dev, append_history);
        return;
    }
    if ((s->use_tc || s->use_tc32) && n_seq >= 16) {
        enqueue_step_tc(s, n_seq, tok_dev, logit_tok_dev, append_history);
        return;
    }
    const DeviceModel* m = s->m;
    const bool modern = m->desc.arch == GRADB_ARCH_MODERN;
    const bool bf16 = m->precision == GRADB_BF16;
    cudaStream_t st = s->stream;
    {
        Timed t(s, KC_EMBED);
        launch_embed(m->emb, modern ? nullptr : m->pos, tok_dev, s->pos, s->x, s->d, n_seq, st);
    }
    const int pro = modern ? PRO_RMSNORM : PRO_LAYERNORM;
    for (int l = 0; l < s->L; l++) {
        const LayerWeights& w = m->layers[l];
        GemvParams g{};
        g.tok = tok_dev;
        g.pos = s->pos;
        g.B = n_seq;
        g.eps = 1e-5f;  // layer_norm.h:18
        // norm1 + Q/K/V projections (+ RoPE), K and V rows go straight into the cache
        g.X = s->x; g.ldx = s->d; g.K = s->d; g.N = s->d;
        g.W[0] = bf16 ? (const void*)w.wq16 : w.wq;
        g.W[1] = bf16 ? (const void*)w.wk16 : w.wk;
        g.W[2] = bf16 ? (const void*)w.wv16 : w.wv;
        g.bias[0] = w.bq; g.bias[1] = w.bk; g.bias[2] = w.bv;
        g.gamma = w.n1g; g.beta = w.n1b;
        g.Y = s->q; g.ldy = s->d;
        g.kcache = s->kcache + (size_t)l * layer_cache_elems(s);
        g.vcache = s->vcache + (size_t)l * layer_cache_elems(s);
        g.rope_cos = modern ? m->rope_cos : nullptr;
        g.rope_sin = modern ? m->rope_sin : nullptr;
        g.H = s->H; g.hs = s->hs; g.T = s->T;
        {
            Timed t(s, KC_QKV);
            launch_gemv(g, pro, EPI_QKV, bf16, m->sm_count, st);
        }

        AttnParams a{};
        a.q = s->q; a.kcache = g.kcache; a.vcache = g.vcache; a.tok = tok_dev; a.pos = s->pos;
        a.out = s->attn; a.out16 = nullptr; a.partial = s->attn_partial; a.counters = s->attn_counters;
        a.status = s->status;
        a.H = s->H; a.hs = s->hs; a.T = s->T; a.d = s->d;
        a.scale = 1.0f / std::sqrt(static_cast<float>(s->hs));  // inference.cpp:184
        a.diag_spin_limit = s->diag_spin_limit; a.diag_skip_tile = s->diag_skip_tile;
        {
            Timed t(s, KC_ATTN);
            launch_attention(a, n_seq, s->attn_splits, st);
        }

        // x += attn @ Wo + bo
        GemvParams o = g;
        o.X = s->attn; o.K = s->d; o.N = s->d;
        o.W[0] = bf16 ? (const void*)w.wo16 : w.wo;
        o.bias[0] = w.bo;
        o.Y = s->x; o.ldy = s->d;
        {
            Timed t(s, KC_OPROJ);
            launch_gemv(o, PRO_NONE, EPI_RESID, bf16, m->sm_count, st);
        }

        // norm2 + FFN
        GemvParams u = g;
        u.X = s->x; u.K = s->d; u.N = s->dff;
        u.gamma = w.n2g; u.beta = w.n2b;
        u.Y = s->ffn; u.ldy = s->dff;
        GemvParams dn = g;
        dn.X = s->ffn; dn.ldx = s->dff; dn.K = s->dff; dn.N = s->d;
        dn.W[0] = bf16 ? (const void*)w.w216 : w.w2;
        dn.Y = s->x; dn.ldy = s->d;
        if (modern) {
            u.W[0] = bf16 ? (const void*)w.gate16 : w.gate;
            u.W[1] = bf16 ? (const void*)w.w116 : w.w1;
            u.bias[0] = u.bias[1] = nullptr;
            {
                Timed t(s, KC_FFN_UP);
                launch_gemv(u, PRO_RMSNORM, EPI_SWIGLU, bf16, m->sm_count, st);
            }
            dn.bias[0] = nullptr;
        } else {
            u.W[0] = bf16 ? (const void*)w.w116 : w.w1;
            u.bias[0] = w.b1;
            {
                Timed t(s, KC_FFN_UP);
                launch_gemv(u, PRO_LAYERNORM, EPI_GELU, bf16, m->sm_count, st);
            }
            dn.bias[0] = w.b2;
        }
        {
            Timed t(s, KC_FFN_DOWN);
            launch_gemv(dn, PRO_NONE, EPI_RESID, bf16, m->sm_count, st);
        }
    }
    LogitsParams lp{};
    lp.X = s->x;
    lp.E = bf16 ? (const void*)m->emb16 : m->emb;
    lp.gamma = m->fng; lp.beta = m->fnb; lp.eps = 1e-5f; lp.rms = modern;
    lp.tok = logit_tok_dev; lp.logits = s->logits;
    lp.B = n_seq; lp.d = s->d; lp.V = s->V;
    {
        Timed t(s, KC_LOGITS);
        launch_logits(lp, bf16, st);
    }
    Timed t(s, KC_ADVANCE);
    launch_advance(tok_dev, s->pos, append_history ? s->hist : nullptr, s->hist_len, s->hist_stride, n_seq, st);
}

SelectParams make_select(Session* s, const gradb_sampling& sp) {
    SelectParams p{};
    p.logits = s->logits;
    p.V = s->V;
    p.greedy = sp.greedy;
    p.temperature = sp.temperature;
    p.penalty = sp.repetition_penalty;
    p.top_k = sp.top_k;
    p.top_p = sp.top_p;
    p.uniforms = s->uniforms;
    p.u_stride = 1;
    p.hist = s->hist;
    p.hist_stride = s->hist_stride;
    p.hist_len = s->hist_len;
    p.out_tok = s->out_tok;
    p.gen = s->gen;
    p.cur_tok = s->tok;
    p.done = s->done;
    p.pos = s->pos;
    p.capacity = s->T;
    p.status = s->status;
    if (!sp.greedy) {  // sampled selection keeps one row of global scratch per sequence
        if (!s->select_scratch) dalloc(&s->select_scratch, (size_t)s->B * select_scratch_floats(s->V));
        p.scratch = s->select_scratch;
    }
    return p;
}

void ensure_uniforms(Session* s, size_t n) {
    if (n > s->uniforms_cap) {
        cudaFree(s->uniforms);
        s->uniforms = nullptr;
        dalloc(&s->uniforms, n);
        s->uniforms_cap = n;
    }
}

// Checked before any state changes, so a call that cannot finish never feeds a prompt first.
void validate_sampling(const Session* s, const gradb_sampling& sp) {
    if (sp.greedy) return;
    if (!(sp.temperature > 0.0f)) throw Error(GRADB_ERR_INVALID, "temperature must be positive");
    if (!select_sampled_fits(s->V)) {
        throw Error(GRADB_ERR_INVALID,
                    "vocabulary too large for the on-device sampled selection stage (limit 47000 ids; greedy has none)");
    }
}

// Token matrix for the prompt feed: row t holds token t of every sequence (or
// kSkip once a prompt is exhausted), followed by the row that says which
// sequences need logits at step t (their last prompt position).
int upload_prompt_matrix(Session* s, const int32_t* tokens, const int32_t* offsets, int n_seq) {
    int steps = 0;
    for (int b = 0; b < n_seq; b++) {
        const int len = offsets[b + 1] - offsets[b];
        if (len < 0) throw Error(GRADB_ERR_INVALID, "prompt offsets must be non-decreasing");
        if (s->h_pos[b] + len > s->T) {
            throw Error(GRADB_ERR_CONTEXT_FULL, "InferenceSession: context exceeds max_len");
        }
        for (int i = offsets[b]; i < offsets[b + 1]; i++) {
            if (tokens[i] < 0 || tokens[i] >= s->V) {
                throw Error(GRADB_ERR_BAD_TOKEN, "InferenceSession: token id out of vocab range");
            }
        }
        steps = std::max(steps, len);
    }
    const size_t need = (size_t)steps * 2 * n_seq;
    if (need > s->tok_matrix_cap) {
        cudaFree(s->tok_matrix);
        s->tok_matrix = nullptr;
        dalloc(&s->tok_matrix, need);
        s->tok_matrix_cap = need;
    }
    // Pinned staging: the copy is asynchronous and the buffer is next written by a later call, after this call's
    // final stream synchronise.
    if (need > s->pin_tokmat_cap) {
        if (s->pin_tokmat) cudaFreeHost(s->pin_tokmat);
        s->pin_tokmat = nullptr;
        s->pin_tokmat_cap = 0;
        GRADB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&s->pin_tokmat), need * sizeof(int)));
        s->pin_tokmat_cap = need;
    }
    int* host = s->pin_tokmat;
    std::fill(host, host + need, kSkip);
    for (int b = 0; b < n_seq; b++) {
        const int len = offsets[b + 1] - offsets[b];
        for (int t = 0; t < len; t++) {
            host[(size_t)t * 2 * n_seq + b] = tokens[offsets[b] + t];
            if (t == len - 1) host[(size_t)t * 2 * n_seq + n_seq + b] = tokens[offsets[b] + t];
        }
    }
    if (need) {
        GRADB_CUDA(cudaMemcpyAsync(s->tok_matrix, host, need * sizeof(int), cudaMemcpyHostToDevice, s->stream));
    }
    return steps;
}

// Prompt tokens processed at once by the batched feed: everything the session can hold, between 8192 rows (the
// activations of a pass then stay in L2) and 65536 (long passes give the persistent GEMM tens of tiles per SM, so its
// prologue, its last un-overlapped epilogue and the partly filled last wave of tiles weigh little: scoring 65536 ids took
// 20.4 ms in passes of 8192 rows, 18.5 in 16384, 17.9 in 32768, 17.3 in one). fp32 sessions stop at 16384: their
// operands are twice as large and scoring keeps a pass's full logits. GRADB_FEED_ROWS overrides.
constexpr size_t kFeedRowsMin = 8192, kFeedRowsMax = 65536, kFeedRowsMaxFp32 = 16384;

size_t feed_rows_for(const Session* s) {
    const size_t most = s->use_tc ? kFeedRowsMax : kFeedRowsMaxFp32;
    size_t rows = std::min(most, std::max(kFeedRowsMin, (size_t)s->B * (size_t)s->T));
    if (const char* e = std::getenv("GRADB_FEED_ROWS")) {
        const long v = std::atol(e);
        if (v >= 1024 && v <= (1 << 18)) rows = (size_t)v;
    }
    return (rows + 255) / 256 * 256;
}

void ensure_feed_buffers(Session* s) {
    Session::Feed& f = s->feed;
    if (f.cap) return;
    const size_t R = feed_rows_for(s);
    dalloc(&f.x, R * s->d);
    dalloc(&f.q, R * s->d);
    dalloc(&f.attn, R * s->d);
    if (s->use_tc32) {
        dalloc(&f.hS, 2 * R * s->d);
        dalloc(&f.attnS, 2 * R * s->d);
        dalloc(&f.ffnS, 2 * R * s->dff);
    } else {
        dalloc(&f.h16, R * s->d);
        dalloc(&f.attn16, R * s->d);
        dalloc(&f.ffn16, R * s->dff);
    }
    dalloc(&f.row_tok, R);
    dalloc(&f.row_pos, R);
    dalloc(&f.row_seq, R);
    dalloc(&f.row_last, R);
    dalloc(&f.seq_count, (size_t)s->B);
    dalloc(&f.last_tok, (size_t)s->B);
    dalloc(&f.tiles, R);
    prefill_attention_configure();
    if (s->use_tc_attn) {
        prefill_attention_tc_configure();
        make_tensor_map_f32(&f.map_q, f.q, R, s->d, 128);
    }
    for (int i = 0; i < 3; i++) {
        const uint32_t tn = 32u << i;
        if (s->use_tc32) {
            make_tensor_map_f32(&f.map_h16[i], f.hS, 2 * R, s->d, tn);
            make_tensor_map_f32(&f.map_attn16[i], f.attnS, 2 * R, s->d, tn);
            make_tensor_map_f32(&f.map_ffn16[i], f.ffnS, 2 * R, s->dff, tn);
        } else {
            make_tensor_map_bf16(&f.map_h16[i], f.h16, R, s->d, tn);
            make_tensor_map_bf16(&f.map_attn16[i], f.attn16, R, s->d, tn);
            make_tensor_map_bf16(&f.map_ffn16[i], f.ffn16, R, s->dff, tn);
        }
    }
    f.cap = (int)R;
}

void ensure_score_buffers(Session* s) {
    ensure_feed_buffers(s);
    Session::Feed& f = s->feed;
    if (f.row_tgt) return;
    dalloc(&f.row_tgt, (size_t)f.cap);
    dalloc(&f.row_dst, (size_t)f.cap);
    dalloc(&f.lse_part, (size_t)f.cap * 2 * ((s->V + 127) / 128));
    dalloc(&f.lse_tgt, (size_t)f.cap);
}

// Batched prompt feed on the tensor-core path: every prompt token of a chunk of positions is one
// row, so each projection runs once per layer over all of them (M = rows) instead of once per
// position. Row r stands for (sequence row_seq[r], position row_pos[r]); K/V rows go to that
// sequence's cache slot and attention reads positions 0..row_pos[r] of it, which is the causal
// prompt attention. Leaves caches, positions, history and last-position logits exactly as the
// reference's step-by-step feed would (text_gen.cpp:44-46).
// With `score_targets` (one id per prompt token, laid out like `tokens`), every row's logits are
// also formed and the log-probability of its target is written to score_out[offsets[b] + j].
void enqueue_prompt_feed_batched(Session* s, const int32_t* tokens, const int32_t* offsets, int n_seq,
                                 const int32_t* score_targets = nullptr, float* score_out = nullptr) {
    const DeviceModel* m = s->m;
    const bool modern = m->desc.arch == GRADB_ARCH_MODERN;
    cudaStream_t st = s->stream;
    ensure_feed_buffers(s);
    Session::Feed& f = s->feed;
    const int d = s->d, ff = s->dff;
    int max_len = 0;
    for (int b = 0; b < n_seq; b++) max_len = std::max(max_len, offsets[b + 1] - offsets[b]);
    const int width = std::max(1, f.cap / n_seq);  // positions per chunk
    const int want = m->sm_count * 3 / 4;
    auto map_idx = [](int tn) { return tn == 32 ? 0 : (tn == 64 ? 1 : 2); };
    const char* no_tiled = std::getenv("GRADB_NO_TILED_ATTN");
    // fp32 sessions: TF32 hi/lo operands, three MMAs per product, in the GEMMs and in the tiled attention
    const bool s32 = s->use_tc32;
    const int kind = s32 ? 1 : 0;
    const bool tiled_ok = !(no_tiled && no_tiled[0] == '1');
    const char* no_tc_attn = std::getenv("GRADB_NO_TC_ATTN");
    const bool tc_attn = s->use_tc_attn && !(no_tc_attn && no_tc_attn[0] == '1');
    const int tile_rows = tc_attn ? 128 : 64;  // query positions per attention tile
    const size_t lo_d = (size_t)f.cap * d, lo_f = (size_t)f.cap * ff;
    auto norm_rows = [&](const float* x, const float* g, const float* b, const int* tk, int rows) {
        if (s32) launch_norm_split(x, g, b, tk, f.hS, lo_d, d, modern, 1e-5f, rows, st);
        else launch_norm_bf16(x, g, b, tk, f.h16, d, modern, 1e-5f, rows, st);
    };

    // per-sequence logits mask: id of the last prompt token, or skip
    // pinned staging: rows (4 x cap), per-sequence counts and last ids (2 x B), scoring targets (2 x cap), tiles (cap int4)
    if (!f.pin) {
        const size_t ints = (size_t)4 * f.cap + 2 * (size_t)s->B + 4 + (size_t)2 * f.cap + (size_t)4 * f.cap;
        GRADB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&f.pin), ints * sizeof(int)));
    }
    int* const h_rows = f.pin;
    int* const h_score = h_rows + (((size_t)4 * f.cap + 2 * (size_t)s->B + 3) & ~size_t(3));  // keeps the tiles 16-byte aligned
    int4* const h_tiles_pin = reinterpret_cast<int4*>(h_score + (size_t)2 * f.cap);
    if (score_targets) ensure_score_buffers(s);
    int* h_last = h_rows + (size_t)4 * f.cap + s->B;
    for (int b = 0; b < n_seq; b++) h_last[b] = offsets[b + 1] > offsets[b] ? tokens[offsets[b + 1] - 1] : kSkip;
    GRADB_CUDA(cudaMemcpyAsync(f.last_tok, h_last, n_seq * sizeof(int), cudaMemcpyHostToDevice, st));

    // Passes of at most f.cap rows. Whole sequences per pass when every prompt fits one (long runs of positions
    // make full 64-query attention tiles and share K/V tiles best); otherwise position ranges over all sequences.
    struct Pass { int b0, b1, p0, p1; };
    std::vector<Pass> passes;
    if (max_len <= f.cap) {
        int b0 = 0, rows = 0;
        for (int b = 0; b < n_seq; b++) {
            const int len = offsets[b + 1] - offsets[b];
            if (rows + len > f.cap) {
                passes.push_back({b0, b, 0, max_len});
                b0 = b;
                rows = 0;
            }
            rows += len;
        }
        passes.push_back({b0, n_seq, 0, max_len});
    } else {
        for (int p0 = 0; p0 < max_len; p0 += width) passes.push_back({0, n_seq, p0, std::min(max_len, p0 + width)});
    }
    for (const Pass& pass : passes) {
        const int p0 = pass.p0, p1 = pass.p1;
        // the staging area is rewritten per pass: wait for the previous pass's copies (rare: prompts beyond one pass)
        if (&pass != &passes.front()) GRADB_CUDA(cudaStreamSynchronize(st));
        int* h_tok = h_rows;
        int* h_pos = h_tok + f.cap;
        int* h_seq = h_pos + f.cap;
        int* h_lastrow = h_seq + f.cap;
        int* h_cnt = h_lastrow + f.cap;
        int R = 0;
        f.h_tiles.clear();
        for (int b = 0; b < n_seq; b++) h_cnt[b] = 0;
        for (int b = pass.b0; b < pass.b1; b++) {
            const int len = offsets[b + 1] - offsets[b];
            for (int j = p0; j < std::min(p1, len); j += tile_rows) {
                f.h_tiles.push_back(
                    make_int4(b, R + (j - p0), s->h_pos[b] + j, std::min(tile_rows, std::min(p1, len) - j)));
            }
            for (int j = p0; j < std::min(p1, len); j++) {
                h_tok[R] = tokens[offsets[b] + j];
                h_pos[R] = s->h_pos[b] + j;
                h_seq[R] = b;
                h_lastrow[R] = j == len - 1 ? h_tok[R] : kSkip;
                if (score_targets) {
                    h_score[R] = score_targets[offsets[b] + j];
                    h_score[(size_t)f.cap + R] = offsets[b] + j;
                }
                R++;
                h_cnt[b]++;
            }
        }
        if (R == 0) continue;
        GRADB_CUDA(cudaMemcpyAsync(f.row_tok, h_tok, R * sizeof(int), cudaMemcpyHostToDevice, st));
        GRADB_CUDA(cudaMemcpyAsync(f.row_pos, h_pos, R * sizeof(int), cudaMemcpyHostToDevice, st));
        GRADB_CUDA(cudaMemcpyAsync(f.row_seq, h_seq, R * sizeof(int), cudaMemcpyHostToDevice, st));
        GRADB_CUDA(cudaMemcpyAsync(f.row_last, h_lastrow, R * sizeof(int), cudaMemcpyHostToDevice, st));
        GRADB_CUDA(cudaMemcpyAsync(f.seq_count, h_cnt, n_seq * sizeof(int), cudaMemcpyHostToDevice, st));
        // Query-tiled attention when the rows form runs of consecutive positions; single positions per
        // sequence stream their prefix through the decode kernel instead. Longest prefixes first.
        const bool tiled = tiled_ok && (size_t)R >= 8 * f.h_tiles.size();
        if (tiled) {
            std::sort(f.h_tiles.begin(), f.h_tiles.end(),
                      [](const int4& a, const int4& b) { return a.z + a.w > b.z + b.w; });
            std::copy(f.h_tiles.begin(), f.h_tiles.end(), h_tiles_pin);
            GRADB_CUDA(cudaMemcpyAsync(f.tiles, h_tiles_pin, f.h_tiles.size() * sizeof(int4), cudaMemcpyHostToDevice, st));
        }
        if (score_targets) {
            GRADB_CUDA(cudaMemcpyAsync(f.row_tgt, h_score, R * sizeof(int), cudaMemcpyHostToDevice, st));
            GRADB_CUDA(cudaMemcpyAsync(f.row_dst, h_score + f.cap, R * sizeof(int), cudaMemcpyHostToDevice, st));
        }

        auto tile_for = [&](int n_features) { return tc_token_tile(R, (n_features + 127) / 128, want); };
        {
            Timed t(s, KC_EMBED);
            launch_embed(m->emb, modern ? nullptr : m->pos, f.row_tok, f.row_pos, f.x, d, R, st);
        }
        TcGemmParams base{};
        base.B = R; base.d = d; base.H = s->H; base.hs = s->hs; base.T = s->T;
        base.tok = f.row_tok; base.pos = f.row_pos; base.row_seq = f.row_seq; base.status = s->status;
        base.b_lo_rows = f.cap;
        for (int l = 0; l < s->L; l++) {
            const LayerWeights& w = m->layers[l];
            float* kc = s->kcache + (size_t)l * layer_cache_elems(s);
            float* vc = s->vcache + (size_t)l * layer_cache_elems(s);
            {
                Timed t(s, KC_QKV);
                norm_rows(f.x, w.n1g, w.n1b, f.row_tok, R);
                TcGemmParams g = base;
                g.K = d; g.N = 3 * d; g.ld_out = d; g.a_lo_rows = 3 * d;
                g.bias[0] = w.bq; g.bias[1] = w.bk; g.bias[2] = w.bv;
                g.rope_cos = modern ? m->rope_cos : nullptr;
                g.rope_sin = modern ? m->rope_sin : nullptr;
                g.out_f32 = f.q; g.kcache = kc; g.vcache = vc;
                const int tn = tile_for(3 * d);
                launch_tc_gemm(TC_QKV, s32 ? w.map_qkvS : w.map_qkv, f.map_h16[map_idx(tn)], g, tn, 1, st, kind);
            }
            {
                Timed t(s, KC_ATTN);
                if (tiled) {
                    PrefillAttnParams a{};
                    a.q = f.q; a.kcache = kc; a.vcache = vc; a.out = s32 ? f.attn : nullptr; a.out16 = s32 ? nullptr : f.attn16;
                    a.tiles = f.tiles; a.n_tiles = (int)f.h_tiles.size(); a.status = s->status;
                    a.H = s->H; a.T = s->T; a.d = d;
                    a.scale = 1.0f / std::sqrt(static_cast<float>(s->hs));
                    if (tc_attn) {
                        launch_prefill_attention_tc(a, f.map_q, s->map_kcache, s->map_vcache, (long long)l * s->B * s->H * s->T,
                                                    m->sm_count, st);
                    } else {
                        launch_prefill_attention(a, st, s32);
                    }
                    if (s32) launch_split_tf32(f.attn, f.attnS, lo_d, (size_t)R * d, st);
                } else {
                    AttnParams a{};
                    a.q = f.q; a.kcache = kc; a.vcache = vc; a.tok = f.row_tok; a.pos = f.row_pos; a.row_seq = f.row_seq;
                    a.out = f.attn; a.out16 = s32 ? nullptr : f.attn16; a.partial = nullptr; a.counters = nullptr;
                    a.status = s->status;
                    a.H = s->H; a.hs = s->hs; a.T = s->T; a.d = d;
                    a.scale = 1.0f / std::sqrt(static_cast<float>(s->hs));
                    launch_attention(a, R, 1, st);
                    if (s32) launch_split_tf32(f.attn, f.attnS, lo_d, (size_t)R * d, st);
                }
            }
            {
                Timed t(s, KC_OPROJ);
                TcGemmParams g = base;
                g.K = d; g.N = d; g.ld_out = d; g.bias[0] = w.bo; g.out_f32 = f.x; g.a_lo_rows = d;
                const int tn = tile_for(d);
                launch_tc_gemm(TC_RESID, s32 ? w.map_oS : w.map_o, f.map_attn16[map_idx(tn)], g, tn, 1, st, kind);
            }
            {
                Timed t(s, KC_FFN_UP);
                norm_rows(f.x, w.n2g, w.n2b, f.row_tok, R);
                TcGemmParams g = base;
                g.K = d; g.N = ff; g.ld_out = ff; g.out_bf16 = f.ffn16; g.out_split = f.ffnS; g.out_lo_elems = lo_f;
                g.a_lo_rows = w.up_rows;
                g.bias[0] = modern ? nullptr : w.b1;
                const int tn = tile_for(ff);
                launch_tc_gemm(modern ? TC_SWIGLU : TC_GELU, s32 ? w.map_upS : w.map_up, f.map_h16[map_idx(tn)], g, tn, 1,
                               st, kind);
            }
            {
                Timed t(s, KC_FFN_DOWN);
                TcGemmParams g = base;
                g.K = ff; g.N = d; g.ld_out = d; g.bias[0] = modern ? nullptr : w.b2; g.out_f32 = f.x; g.a_lo_rows = d;
                const int tn = tile_for(d);
                launch_tc_gemm(TC_RESID, s32 ? w.map_downS : w.map_down, f.map_ffn16[map_idx(tn)], g, tn, 1, st, kind);
            }
        }
        if (score_targets) {
            // every row's logits (final norm + tied-embedding GEMM), then the target's log-probability
            Timed t(s, KC_SCORE);
            norm_rows(f.x, m->fng, m->fnb, f.row_tok, R);
            TcGemmParams g = base;
            g.K = d; g.N = s->V; g.a_lo_rows = s->V;
            const int tn = tile_for(s->V);
            if (!s32 && tc_many_rows(g, tn)) {
                // logits never reach memory: every feature tile leaves (max, sum of exp) per row and the target's logit
                const int tiles = (s->V + 127) / 128;
                g.pos = f.row_tgt;  // this epilogue reads the rows' target ids where the others read positions
                g.out_f32 = f.lse_part; g.ld_out = 2 * tiles; g.lse_tgt = f.lse_tgt;
                launch_tc_gemm(TC_LSE, m->map_emb, f.map_h16[map_idx(tn)], g, tn, 1, st, 0);
                launch_lse_combine(f.lse_part, tiles, f.lse_tgt, f.row_tgt, s->V, f.row_dst, score_out, R, st);
            } else {
                if (!f.score_logits) dalloc(&f.score_logits, (size_t)f.cap * s->V);
                g.ld_out = s->V; g.out_f32 = f.score_logits;
                launch_tc_gemm(TC_LOGITS, s32 ? m->map_embS : m->map_emb, f.map_h16[map_idx(tn)], g, tn, 1, st, kind);
                launch_row_logp(f.score_logits, (size_t)s->V, s->V, f.row_tgt, f.row_dst, 0, 0, score_out, R, st);
            }
        }
        launch_gather_last_rows(f.x, f.row_last, f.row_seq, s->x, d, R, st);
        launch_feed_bookkeeping(f.row_tok, f.row_pos, f.row_seq, f.seq_count, s->pos, s->hist_len, s->hist, s->hist_stride,
                                R, n_seq, st);
    }
    // the host mirror of the positions is advanced by the callers

    // last-position logits: final norm + tied-embedding GEMM over the per-sequence rows
    {
        Timed t(s, KC_LOGITS);
        if (s32) launch_norm_split(s->x, m->fng, m->fnb, f.last_tok, s->hS, (size_t)s->split_rows * d, d, modern, 1e-5f, n_seq, st);
        else launch_norm_bf16(s->x, m->fng, m->fnb, f.last_tok, s->h16, d, modern, 1e-5f, n_seq, st);
        TcGemmParams g{};
        g.B = n_seq; g.d = d; g.H = s->H; g.hs = s->hs; g.T = s->T;
        g.tok = f.last_tok; g.pos = s->pos; g.status = s->status;
        g.K = d; g.N = s->V; g.ld_out = s->V; g.out_f32 = s->logits;
        g.a_lo_rows = s->V; g.b_lo_rows = s->split_rows;
        const int tn = tc_token_tile(n_seq, (s->V + 127) / 128, want);
        launch_tc_gemm(TC_LOGITS, s32 ? m->map_embS : m->map_emb, s->map_h16[map_idx(tn)], g, tn, 1, st, kind);
    }
}

bool batched_feed_available(const Session* s) {
    const char* off = std::getenv("GRADB_NO_BATCHED_FEED");
    return (s->use_tc || s->use_tc32) && s->hs == 64 && !(off && off[0] == '1');
}

// Generation keeps a small group of sequences on one family of kernels for the prompt and the
// decode steps; scoring has no decode steps and batches whenever the session can.
bool use_batched_feed(const Session* s, int n_seq) { return batched_feed_available(s) && n_seq >= 16; }

void enqueue_prompt_feed(Session* s, int steps, int n_seq) {
    for (int t = 0; t < steps; t++) {
        const int* row = s->tok_matrix + (size_t)t * 2 * n_seq;
        enqueue_step(s, n_seq, row, row + n_seq, true);
    }
}

}  // namespace

Session* create_session(const DeviceModel* m, int max_batch, int max_len, void* stream) {
    if (!m) throw Error(GRADB_ERR_INVALID, "null model");
    if (max_batch < 1 || max_batch > 65535) throw Error(GRADB_ERR_INVALID, "max_batch must be in [1, 65535]");
    if (max_len == 0) max_len = m->desc.max_len;
    if (max_len < 1 || max_len > m->desc.max_len) {
        throw Error(GRADB_ERR_INVALID, "session max_len must be in [1, model max_len]");
    }
    GRADB_CUDA(cudaSetDevice(m->device));
    auto* s = new Session();
    try {
        s->m = m;
        s->B = max_batch;
        s->T = max_len;
        s->V = m->desc.vocab_size;
        s->d = m->desc.d_model;
        s->H = m->desc.num_heads;
        s->hs = s->d / s->H;
        s->dff = m->desc.d_ff;
        s->L = m->desc.num_layers;
        s->hist_stride = s->T + 2;
        if (stream) {
            s->stream = static_cast<cudaStream_t>(stream);
        } else {
            GRADB_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
            s->own_stream = true;
        }
        const char* ng = std::getenv("GRADB_NO_GRAPH");
        s->use_graph = !(ng && ng[0] == '1');
        // Context splits: as many as still give every warp of the persistent attention kernel (seven per SM) at most
        // one (sequence, head, split) unit. Each warp keeps one 16 KB tile in flight, so the warps that have a unit
        // set the bandwidth; a split count that spills into a second round of units loses more than it gains
        // (32 sequences x 12 heads at contexts 1025..1280, attention per launch: 1 split 56 us, 2 splits 46, 3 splits
        // 59, 4 splits 50, 6 splits 57).
        const int want = (kAttnPipeWarps * m->sm_count) / (s->B * s->H);
        s->attn_splits = std::max(1, std::min({want, 16, (s->T + 31) / 32}));
#if GRADB_DIAG
        if (const char* sp = std::getenv("GRADB_ATTN_SPLITS")) {
            s->attn_splits = std::max(1, std::min({std::atoi(sp), 16, (s->T + 31) / 32}));
        }
#endif
        const size_t B = s->B;
        dalloc(&s->x, B * s->d);
        dalloc(&s->q, B * s->d);
        dalloc(&s->attn, B * s->d);
        dalloc(&s->ffn, B * s->dff);
        dalloc(&s->logits, B * s->V);
        const size_t cache = (size_t)s->L * layer_cache_elems(s);
        dalloc(&s->kcache, cache);
        dalloc(&s->vcache, cache);
        dalloc(&s->attn_partial, B * s->H * s->attn_splits * (s->hs + 2));
        dalloc(&s->attn_counters, B * s->H);
        dalloc(&s->tok, B);
        dalloc(&s->pos, B);
        dalloc(&s->hist, B * s->hist_stride);
        dalloc(&s->hist_len, B);
        dalloc(&s->gen, B);
        dalloc(&s->done, B);
        dalloc(&s->out_tok, B);
        dalloc(&s->status, 1);
        GRADB_CUDA(cudaMemsetAsync(s->status, 0, sizeof(int), s->stream));
        const char* nb1 = std::getenv("GRADB_NO_B1");
        s->use_b1 = s->B == 1 && m->b1 && m->b1->ok && !(nb1 && nb1[0] == '1');
        if (s->use_b1) {
            // exchange words, accumulators and step counters of the persistent kernel: all start at zero
            s->b1_ws_bytes = b1_workspace_bytes(m, m->b1);
            dalloc(&s->b1_ws, s->b1_ws_bytes);
            GRADB_CUDA(cudaMemsetAsync(s->b1_ws, 0, s->b1_ws_bytes, s->stream));
#if GRADB_DIAG
            const char* tr = std::getenv("GRADB_B1_TRACE");
            if (tr && tr[0] == '1') {
                dalloc(&s->b1_trace, 1024);
                GRADB_CUDA(cudaMemsetAsync(s->b1_trace, 0, 1024 * sizeof(unsigned long long), s->stream));
            }
#endif
        }
        const char* npdl = std::getenv("GRADB_NO_PDL");
        s->use_pdl = !(npdl && npdl[0] == '1');
        const char* ntc = std::getenv("GRADB_NO_TC");
        s->use_tc = m->tc_ok && s->B >= 16 && !(ntc && ntc[0] == '1');
        if (s->hs == 64) attention_configure();
        configure_select(s->V);
        const char* ntc32 = std::getenv("GRADB_NO_TC32");
        s->use_tc32 = m->tc32_ok && s->B >= 16 && !(ntc && ntc[0] == '1') && !(ntc32 && ntc32[0] == '1');
        if (s->use_tc32) {
            tc_configure_all();
            const size_t rows = (size_t)((s->B + 255) / 256) * 256;
            s->split_rows = (int)rows;
            dalloc(&s->hS, 2 * rows * s->d);
            dalloc(&s->attnS, 2 * rows * s->d);
            dalloc(&s->ffnS, 2 * rows * s->dff);
            GRADB_CUDA(cudaMemsetAsync(s->hS, 0, 2 * rows * s->d * 4, s->stream));
            GRADB_CUDA(cudaMemsetAsync(s->attnS, 0, 2 * rows * s->d * 4, s->stream));
            GRADB_CUDA(cudaMemsetAsync(s->ffnS, 0, 2 * rows * s->dff * 4, s->stream));
            for (int i = 0; i < 3; i++) {
                const uint32_t tn = 32u << i;
                make_tensor_map_f32(&s->map_h16[i], s->hS, 2 * rows, s->d, tn);
                make_tensor_map_f32(&s->map_attn16[i], s->attnS, 2 * rows, s->d, tn);
                make_tensor_map_f32(&s->map_ffn16[i], s->ffnS, 2 * rows, s->dff, tn);
            }
        }
        if (s->use_tc && s->hs == 64) {
            s->use_tc_attn = true;
            make_tensor_map_f32(&s->map_kcache, s->kcache, (uint64_t)s->L * B * s->H * s->T, 64, 128);
            make_tensor_map_f32(&s->map_vcache, s->vcache, (uint64_t)s->L * B * s->H * s->T, 64, 128, true);
        }
        if (s->use_tc) {
            tc_configure_all();
            // rows padded to a whole 256-token tile so a TMA box never starts outside the buffer
            const size_t rows = (size_t)((s->B + 255) / 256) * 256;
            dalloc(&s->h16, rows * s->d);
            dalloc(&s->attn16, rows * s->d);
            dalloc(&s->ffn16, rows * s->dff);
            GRADB_CUDA(cudaMemsetAsync(s->h16, 0, rows * s->d * 2, s->stream));
            GRADB_CUDA(cudaMemsetAsync(s->attn16, 0, rows * s->d * 2, s->stream));
            GRADB_CUDA(cudaMemsetAsync(s->ffn16, 0, rows * s->dff * 2, s->stream));
            for (int i = 0; i < 3; i++) {
                const uint32_t tn = 32u << i;
                make_tensor_map_bf16(&s->map_h16[i], s->h16, rows, s->d, tn);
                make_tensor_map_bf16(&s->map_attn16[i], s->attn16, rows, s->d, tn);
                make_tensor_map_bf16(&s->map_ffn16[i], s->ffn16, rows, s->dff, tn);
            }
        }
        GRADB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&s->h_stage), sizeof(int) * 4 * B));
        GRADB_CUDA(cudaEventCreate(&s->ev_begin));
        GRADB_CUDA(cudaEventCreate(&s->ev_end));
        s->h_pos.assign(B, 0);
        s->h_ids.assign(B, {});
        s->h_live.assign(B, 0);
        s->h_gen.assign(B, 0);
        // The reference zero-fills its caches at construction (inference.cpp:130-135).
        GRADB_CUDA(cudaMemsetAsync(s->kcache, 0, cache * sizeof(float), s->stream));
        GRADB_CUDA(cudaMemsetAsync(s->vcache, 0, cache * sizeof(float), s->stream));
        GRADB_CUDA(cudaMemsetAsync(s->attn_counters, 0, B * s->H * sizeof(int), s->stream));
        reset_session(s);
        return s;
    } catch (...) {
        destroy_session(s);
        throw;
    }
}

void destroy_session(Session* s) {
    if (!s) return;
    cudaSetDevice(s->m->device);
    if (s->stream) cudaStreamSynchronize(s->stream);
    if (s->graph) cudaGraphExecDestroy(s->graph);
    if (s->serve_graph) cudaGraphExecDestroy(s->serve_graph);
    if (s->stream_ring) cudaFreeHost(s->stream_ring);
    if (s->stream_u) cudaFreeHost(s->stream_u);
    cudaFree(s->max_new_seq); cudaFree(s->serve_u);
    for (cudaEvent_t e : s->step_events) cudaEventDestroy(e);
    for (cudaEvent_t e : s->event_pool) cudaEventDestroy(e);
    for (const Session::Span& sp : s->spans) {
        cudaEventDestroy(sp.a);
        cudaEventDestroy(sp.b);
    }
    if (s->ev_begin) cudaEventDestroy(s->ev_begin);
    if (s->ev_end) cudaEventDestroy(s->ev_end);
    cudaFree(s->x); cudaFree(s->q); cudaFree(s->attn); cudaFree(s->ffn); cudaFree(s->logits);
    cudaFree(s->kcache); cudaFree(s->vcache); cudaFree(s->attn_partial); cudaFree(s->attn_counters);
    cudaFree(s->tok); cudaFree(s->pos); cudaFree(s->hist); cudaFree(s->hist_len);
    cudaFree(s->gen); cudaFree(s->done); cudaFree(s->out_tok); cudaFree(s->tok_matrix);
    cudaFree(s->uniforms); cudaFree(s->probs); cudaFree(s->select_scratch);
    cudaFree(s->b1_ws); cudaFree(s->b1_trace);
    cudaFree(s->feed.hS); cudaFree(s->feed.attnS); cudaFree(s->feed.ffnS);
    cudaFree(s->feed.x); cudaFree(s->feed.q); cudaFree(s->feed.attn); cudaFree(s->feed.h16); cudaFree(s->feed.attn16);
    cudaFree(s->feed.ffn16); cudaFree(s->feed.row_tok); cudaFree(s->feed.row_pos); cudaFree(s->feed.row_seq);
    cudaFree(s->feed.row_last); cudaFree(s->feed.seq_count); cudaFree(s->feed.last_tok);
    cudaFree(s->feed.tiles); cudaFree(s->feed.score_logits); cudaFree(s->feed.lse_part); cudaFree(s->feed.lse_tgt); cudaFree(s->feed.row_tgt); cudaFree(s->feed.row_dst);
    cudaFree(s->score_out); cudaFree(s->score_tgt);
    cudaFree(s->h16); cudaFree(s->attn16); cudaFree(s->ffn16); cudaFree(s->status);
    cudaFree(s->hS); cudaFree(s->attnS); cudaFree(s->ffnS);
    if (s->h_stage) cudaFreeHost(s->h_stage);
    if (s->pin_tokmat) cudaFreeHost(s->pin_tokmat);
    if (s->feed.pin) cudaFreeHost(s->feed.pin);
    if (s->own_stream && s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

void reset_session(Session* s) {
    GRADB_CUDA(cudaSetDevice(s->m->device));
    const size_t B = s->B;
    GRADB_CUDA(cudaMemsetAsync(s->pos, 0, B * sizeof(int), s->stream));
    GRADB_CUDA(cudaMemsetAsync(s->hist_len, 0, B * sizeof(int), s->stream));
    GRADB_CUDA(cudaMemsetAsync(s->gen, 0, B * sizeof(int), s->stream));
    GRADB_CUDA(cudaMemsetAsync(s->done, 0, B * sizeof(int), s->stream));
    GRADB_CUDA(cudaMemsetAsync(s->tok, 0xff, B * sizeof(int), s->stream));
    std::fill(s->h_pos.begin(), s->h_pos.end(), 0);
    for (auto& ids : s->h_ids) ids.clear();
    std::fill(s->h_live.begin(), s->h_live.end(), 0);
    std::fill(s->h_gen.begin(), s->h_gen.end(), 0);
}

void session_step(Session* s, const int32_t* tokens, int n_seq, float* logits_host) {
    if (n_seq < 1 || n_seq > s->B) throw Error(GRADB_ERR_INVALID, "n_seq out of range for this session");
    GRADB_CUDA(cudaSetDevice(s->m->device));
    // Same order as the reference: context check, then the id range (inference.cpp:151-156).
    for (int b = 0; b < n_seq; b++) {
        if (tokens[b] < 0) continue;
        if (s->h_pos[b] >= s->T) throw Error(GRADB_ERR_CONTEXT_FULL, "InferenceSession: context exceeds max_len");
    }
    for (int b = 0; b < n_seq; b++) {
        if (tokens[b] >= s->V) throw Error(GRADB_ERR_BAD_TOKEN, "InferenceSession: token id out of vocab range");
    }
    for (int b = 0; b < n_seq; b++) s->h_stage[b] = tokens[b] < 0 ? kSkip : tokens[b];
    GRADB_CUDA(cudaEventRecord(s->ev_begin, s->stream));
    GRADB_CUDA(cudaMemcpyAsync(s->tok, s->h_stage, n_seq * sizeof(int), cudaMemcpyHostToDevice, s->stream));
    enqueue_step(s, n_seq, s->tok, s->tok, true);
    if (logits_host) {
        GRADB_CUDA(cudaMemcpyAsync(logits_host, s->logits, (size_t)n_seq * s->V * sizeof(float),
                                   cudaMemcpyDeviceToHost, s->stream));
    }
    GRADB_CUDA(cudaEventRecord(s->ev_end, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    GRADB_CUDA(cudaEventElapsedTime(&s->last_ms, s->ev_begin, s->ev_end));
    for (int b = 0; b < n_seq; b++) {
        if (tokens[b] >= 0) s->h_pos[b]++;
    }
}

void session_prefill(Session* s, const int32_t* tokens, const int32_t* offsets, int n_seq, float* logits_host) {
    if (n_seq < 1 || n_seq > s->B) throw Error(GRADB_ERR_INVALID, "n_seq out of range for this session");
    GRADB_CUDA(cudaSetDevice(s->m->device));
    const int steps = upload_prompt_matrix(s, tokens, offsets, n_seq);
    GRADB_CUDA(cudaEventRecord(s->ev_begin, s->stream));
    if (use_batched_feed(s, n_seq)) enqueue_prompt_feed_batched(s, tokens, offsets, n_seq);
    else enqueue_prompt_feed(s, steps, n_seq);
    GRADB_CUDA(cudaEventRecord(s->ev_end, s->stream));
    if (logits_host) {
        GRADB_CUDA(cudaMemcpyAsync(logits_host, s->logits, (size_t)n_seq * s->V * sizeof(float),
                                   cudaMemcpyDeviceToHost, s->stream));
    }
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    GRADB_CUDA(cudaEventElapsedTime(&s->last_ms, s->ev_begin, s->ev_end));
    for (int b = 0; b < n_seq; b++) s->h_pos[b] += offsets[b + 1] - offsets[b];
}

float session_score(Session* s, const int32_t* inputs, const int32_t* targets, int n_windows, int seq_len,
                    float* row_logp_host) {
    if (n_windows < 1) throw Error(GRADB_ERR_INVALID, "n_windows must be positive");
    if (seq_len < 1) throw Error(GRADB_ERR_INVALID, "seq_len must be positive");
    if (seq_len > s->T) throw Error(GRADB_ERR_CONTEXT_FULL, "InferenceSession: context exceeds max_len");
    for (size_t i = 0; i < (size_t)n_windows * seq_len; i++) {
        if (inputs[i] < 0 || inputs[i] >= s->V) {
            throw Error(GRADB_ERR_BAD_TOKEN, "InferenceSession: token id out of vocab range");
        }
    }
    GRADB_CUDA(cudaSetDevice(s->m->device));
    cudaStream_t st = s->stream;
    if (!s->score_out) {
        dalloc(&s->score_out, (size_t)s->B * s->T);
        dalloc(&s->score_tgt, (size_t)s->B * s->T);
    }
    const bool batched = batched_feed_available(s);
    if (batched) ensure_score_buffers(s);
    float total_ms = 0.f;
    std::vector<int> offsets, host;
    for (int w0 = 0; w0 < n_windows; w0 += s->B) {
        const int n = std::min(s->B, n_windows - w0);
        const int32_t* in = inputs + (size_t)w0 * seq_len;
        const int32_t* tg = targets + (size_t)w0 * seq_len;
        reset_session(s);
        if (batched) {
            offsets.resize(n + 1);
            for (int b = 0; b <= n; b++) offsets[b] = b * seq_len;
            GRADB_CUDA(cudaEventRecord(s->ev_begin, st));
            enqueue_prompt_feed_batched(s, in, offsets.data(), n, tg, s->score_out);
        } else {
            // position by position through the step kernels, logits for every sequence at every position
            const size_t need = (size_t)seq_len * 2 * n;
            if (need > s->tok_matrix_cap) {
                cudaFree(s->tok_matrix);
                s->tok_matrix = nullptr;
                dalloc(&s->tok_matrix, need);
                s->tok_matrix_cap = need;
            }
            host.resize(need + (size_t)seq_len * n);
            int* h_tgt = host.data() + need;
            for (int t = 0; t < seq_len; t++) {
                for (int b = 0; b < n; b++) {
                    const int id = in[(size_t)b * seq_len + t];
                    host[(size_t)t * 2 * n + b] = id;
                    host[(size_t)t * 2 * n + n + b] = id;
                    h_tgt[(size_t)t * n + b] = tg[(size_t)b * seq_len + t];
                }
            }
            GRADB_CUDA(cudaMemcpyAsync(s->tok_matrix, host.data(), need * sizeof(int), cudaMemcpyHostToDevice, st));
            GRADB_CUDA(cudaMemcpyAsync(s->score_tgt, h_tgt, (size_t)seq_len * n * sizeof(int),
                                       cudaMemcpyHostToDevice, st));
            GRADB_CUDA(cudaEventRecord(s->ev_begin, st));
            for (int t = 0; t < seq_len; t++) {
                const int* row = s->tok_matrix + (size_t)t * 2 * n;
                enqueue_step(s, n, row, row + n, true);
                Timed tm(s, KC_SCORE);
                launch_row_logp(s->logits, (size_t)s->V, s->V, s->score_tgt + (size_t)t * n, nullptr, seq_len, t,
                                s->score_out, n, st);
            }
        }
        GRADB_CUDA(cudaEventRecord(s->ev_end, st));
        GRADB_CUDA(cudaMemcpyAsync(row_logp_host + (size_t)w0 * seq_len, s->score_out,
                                   (size_t)n * seq_len * sizeof(float), cudaMemcpyDeviceToHost, st));
        GRADB_CUDA(cudaStreamSynchronize(st));
        collect_spans(s);
        check_status(s);
        float ms = 0.f;
        GRADB_CUDA(cudaEventElapsedTime(&ms, s->ev_begin, s->ev_end));
        total_ms += ms;
        for (int b = 0; b < n; b++) s->h_pos[b] += seq_len;
    }
    s->last_ms = total_ms;
    return total_ms;
}

void session_set_history(Session* s, int seq, const int32_t* ids, int n) {
    if (seq < 0 || seq >= s->B || n < 0 || n > s->hist_stride) throw Error(GRADB_ERR_INVALID, "bad history");
    for (int i = 0; i < n; i++) {  // the penalty indexes the logits with these ids
        if (ids[i] < 0 || ids[i] >= s->V) throw Error(GRADB_ERR_BAD_TOKEN, "InferenceSession: token id out of vocab range");
    }
    GRADB_CUDA(cudaSetDevice(s->m->device));
    GRADB_CUDA(cudaMemcpyAsync(s->hist + (size_t)seq * s->hist_stride, ids, n * sizeof(int), cudaMemcpyHostToDevice,
                               s->stream));
    GRADB_CUDA(cudaMemcpyAsync(s->hist_len + seq, &n, sizeof(int), cudaMemcpyHostToDevice, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
}

void session_select(Session* s, const gradb_sampling& sp, const float* logits_host, const float* uniforms,
                    int n_seq, int32_t* tokens_out, float* probs_host) {
    if (n_seq < 1 || n_seq > s->B) throw Error(GRADB_ERR_INVALID, "n_seq out of range for this session");
    validate_sampling(s, sp);
    if (!sp.greedy && !uniforms) throw Error(GRADB_ERR_INVALID, "sampling needs one uniform draw per sequence");
    GRADB_CUDA(cudaSetDevice(s->m->device));
    if (logits_host) {
        GRADB_CUDA(cudaMemcpyAsync(s->logits, logits_host, (size_t)n_seq * s->V * sizeof(float),
                                   cudaMemcpyHostToDevice, s->stream));
    }
    ensure_uniforms(s, n_seq);
    if (!sp.greedy) {
        GRADB_CUDA(cudaMemcpyAsync(s->uniforms, uniforms, n_seq * sizeof(float), cudaMemcpyHostToDevice, s->stream));
    }
    SelectParams p = make_select(s, sp);
    p.loop_mode = 0;
    if (probs_host && !sp.greedy) {
        if (!s->probs) dalloc(&s->probs, (size_t)s->B * s->V);
        p.probs_out = s->probs;
    }
    launch_select(p, n_seq, s->stream);
    GRADB_CUDA(cudaMemcpyAsync(tokens_out, s->out_tok, n_seq * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    if (p.probs_out) {
        GRADB_CUDA(cudaMemcpyAsync(probs_host, s->probs, (size_t)n_seq * s->V * sizeof(float), cudaMemcpyDeviceToHost,
                                   s->stream));
    }
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
}

void session_generate(Session* s, const int32_t* prompts, const int32_t* offsets, int n_seq,
                      const gradb_sampling& sp, int max_new, const float* uniforms, int32_t* out_ids,
                      int out_stride, int32_t* out_len, float* step_ms, float* prefill_ms) {
    if (n_seq < 1 || n_seq > s->B) throw Error(GRADB_ERR_INVALID, "n_seq out of range for this session");
    if (max_new < 0) throw Error(GRADB_ERR_INVALID, "max_new must not be negative");
    validate_sampling(s, sp);
    if (!sp.greedy && max_new > 0 && !uniforms) {
        throw Error(GRADB_ERR_INVALID, "sampling needs n_seq*max_new uniform draws");
    }
    GRADB_CUDA(cudaSetDevice(s->m->device));
    reset_session(s);
    // How many ids each sequence emits: max_new, or fewer when its context fills first; the id
    // chosen when the context is full is still emitted (text_gen.cpp:61-63).
    int emit_max = 0;
    std::vector<int> emit(n_seq, 0);
    for (int b = 0; b < n_seq; b++) {
        const int len = offsets[b + 1] - offsets[b];
        if (len <= 0) continue;  // empty prompt: nothing is generated (text_gen.cpp:40)
        emit[b] = std::min(max_new, s->T - len + 1);
        if (len + emit[b] > out_stride) throw Error(GRADB_ERR_INVALID, "out_stride too small for prompt + new ids");
        emit_max = std::max(emit_max, emit[b]);
    }
    const int steps = upload_prompt_matrix(s, prompts, offsets, n_seq);
    if (!sp.greedy && max_new > 0) {
        ensure_uniforms(s, (size_t)n_seq * max_new);
        GRADB_CUDA(cudaMemcpyAsync(s->uniforms, uniforms, (size_t)n_seq * max_new * sizeof(float),
                                   cudaMemcpyHostToDevice, s->stream));
    }
    // Sequences with an empty prompt never run.
    bool any_empty = false;
    for (int b = 0; b < n_seq; b++) {
        s->h_stage[b] = (offsets[b + 1] - offsets[b]) <= 0 ? 1 : 0;
        any_empty = any_empty || s->h_stage[b];
    }
    if (any_empty) {
        GRADB_CUDA(cudaMemcpyAsync(s->done, s->h_stage, n_seq * sizeof(int), cudaMemcpyHostToDevice, s->stream));
    }

    GRADB_CUDA(cudaEventRecord(s->ev_begin, s->stream));
    if (use_batched_feed(s, n_seq)) enqueue_prompt_feed_batched(s, prompts, offsets, n_seq);
    else enqueue_prompt_feed(s, steps, n_seq);
    GRADB_CUDA(cudaEventRecord(s->ev_end, s->stream));

    SelectParams p = make_select(s, sp);
    p.loop_mode = 1;
    p.u_stride = max_new;
    p.max_new = max_new;
    p.out_tok = nullptr;

    while ((int)s->step_events.size() < emit_max + 1) {
        cudaEvent_t e;
        GRADB_CUDA(cudaEventCreate(&e));
        s->step_events.push_back(e);
    }
    const bool graph_ok = s->use_graph && !s->profiling && emit_max > 1;
    if (graph_ok) {
        const bool same = s->graph && s->graph_nseq == n_seq && s->graph_max_new == max_new &&
                          std::memcmp(&s->graph_params, &sp, sizeof(sp)) == 0;
        if (!same) {
            if (s->graph) {
                cudaGraphExecDestroy(s->graph);
                s->graph = nullptr;
            }
            // One decode iteration = choose ids from the current logits, then feed them.
            // Everything it reads lives at fixed device addresses, so one graph serves every token.
            // The prompt feed has already run every step kernel eagerly, so their launch
            // attributes are in place before capture starts.
            cudaGraph_t g = nullptr;
            configure_select(s->V);
            GRADB_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
            g_capturing = true;
            try {
                launch_select(p, n_seq, s->stream);
                enqueue_step(s, n_seq, s->tok, s->tok, false);
            } catch (...) {
                g_capturing = false;
                cudaStreamEndCapture(s->stream, &g);
                if (g) cudaGraphDestroy(g);
                throw;
            }
            g_capturing = false;
            GRADB_CUDA(cudaStreamEndCapture(s->stream, &g));
            const cudaError_t e = cudaGraphInstantiate(&s->graph, g, 0);
            cudaGraphDestroy(g);
            if (e != cudaSuccess) throw Error(GRADB_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
            s->graph_params = sp;
            s->graph_nseq = n_seq;
            s->graph_max_new = max_new;
        }
    }
    for (int i = 0; i < emit_max; i++) {
        GRADB_CUDA(cudaEventRecord(s->step_events[i], s->stream));
        if (i == emit_max - 1) {
            Timed t(s, KC_SELECT);
            launch_select(p, n_seq, s->stream);  // the last ids need no further step
        } else if (graph_ok) {
            GRADB_CUDA(cudaGraphLaunch(s->graph, s->stream));
            count_launch(s->use_b1 && n_seq == 1 ? 2 : 4 + 5 * s->L);  // kernels inside the graph
        } else {
            {
                Timed t(s, KC_SELECT);
                launch_select(p, n_seq, s->stream);
            }
            enqueue_step(s, n_seq, s->tok, s->tok, false);
        }
    }
    GRADB_CUDA(cudaEventRecord(s->step_events[emit_max], s->stream));

    std::vector<int> lens(n_seq);
    GRADB_CUDA(cudaMemcpyAsync(lens.data(), s->hist_len, n_seq * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    std::vector<int> hist((size_t)n_seq * s->hist_stride);
    GRADB_CUDA(cudaMemcpyAsync(hist.data(), s->hist, hist.size() * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    for (int b = 0; b < n_seq; b++) {
        const int len = offsets[b + 1] - offsets[b];
        const int n = len <= 0 ? 0 : std::min(lens[b], out_stride);
        out_len[b] = n;
        std::memcpy(out_ids + (size_t)b * out_stride, hist.data() + (size_t)b * s->hist_stride, n * sizeof(int));
        s->h_pos[b] = len <= 0 ? 0 : std::min(s->T, len + std::max(0, emit[b] - 1));
    }
    float ms = 0.f;
    GRADB_CUDA(cudaEventElapsedTime(&ms, s->ev_begin, s->ev_end));
    if (prefill_ms) *prefill_ms = ms;
    float total = 0.f;
    for (int i = 0; i < emit_max; i++) {
        float t = 0.f;
        GRADB_CUDA(cudaEventElapsedTime(&t, s->step_events[i], s->step_events[i + 1]));
        if (step_ms) step_ms[i] = t;
        total += t;
    }
    s->last_ms = total;
}

// How many ids a sequence with a prompt of `len` ids emits: max_new, or fewer when its context fills first; the id
// chosen when the context is full is still emitted (text_gen.cpp:61-63). Empty prompts emit nothing (text_gen.cpp:40).
static int emit_count(const Session* s, int len, int max_new) { return len <= 0 ? 0 : std::min(max_new, s->T - len + 1); }

void session_generate_stream(Session* s, const int32_t* prompts, const int32_t* offsets, int n_seq,
                             const gradb_sampling& sp, int max_new, gradb_draw_fn draw, gradb_token_fn on_token,
                             void* user, int32_t* emitted) {
    if (n_seq < 1 || n_seq > s->B) throw Error(GRADB_ERR_INVALID, "n_seq out of range for this session");
    if (max_new < 0) throw Error(GRADB_ERR_INVALID, "max_new must not be negative");
    if (!on_token) throw Error(GRADB_ERR_INVALID, "streaming needs a token callback");
    validate_sampling(s, sp);
    if (!sp.greedy && max_new > 0 && !draw) throw Error(GRADB_ERR_INVALID, "sampling needs a draw callback");
    GRADB_CUDA(cudaSetDevice(s->m->device));
    reset_session(s);
    int emit_max = 0;
    std::vector<int> emit(n_seq, 0), given(n_seq, 0);
    std::vector<char> stopped(n_seq, 0);
    for (int b = 0; b < n_seq; b++) {
        emit[b] = emit_count(s, offsets[b + 1] - offsets[b], max_new);
        emit_max = std::max(emit_max, emit[b]);
    }
    const int steps = upload_prompt_matrix(s, prompts, offsets, n_seq);
    const size_t cap = (size_t)std::max(max_new, 1);
    if (cap > s->stream_cap) {
        if (s->stream_ring) cudaFreeHost(s->stream_ring);
        if (s->stream_u) cudaFreeHost(s->stream_u);
        s->stream_ring = nullptr;
        s->stream_u = nullptr;
        s->stream_cap = 0;
        GRADB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&s->stream_ring), (size_t)s->B * cap * sizeof(int),
                                 cudaHostAllocMapped));
        GRADB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&s->stream_u), (size_t)s->B * cap * sizeof(float),
                                 cudaHostAllocMapped));
        s->stream_cap = cap;
    }
    const size_t stride = s->stream_cap;
    std::memset(s->stream_ring, 0, (size_t)s->B * stride * sizeof(int));
    int* ring_dev = nullptr;
    float* u_dev = nullptr;
    GRADB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ring_dev), s->stream_ring, 0));
    GRADB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&u_dev), s->stream_u, 0));
    bool any_empty = false;
    for (int b = 0; b < n_seq; b++) {
        s->h_stage[b] = emit[b] == 0 ? 1 : 0;
        any_empty = any_empty || s->h_stage[b];
    }
    if (any_empty) {
        GRADB_CUDA(cudaMemcpyAsync(s->done, s->h_stage, n_seq * sizeof(int), cudaMemcpyHostToDevice, s->stream));
    }
    GRADB_CUDA(cudaEventRecord(s->ev_begin, s->stream));
    if (use_batched_feed(s, n_seq)) enqueue_prompt_feed_batched(s, prompts, offsets, n_seq);
    else enqueue_prompt_feed(s, steps, n_seq);
    GRADB_CUDA(cudaEventRecord(s->ev_end, s->stream));

    SelectParams p = make_select(s, sp);
    p.loop_mode = 1;
    p.uniforms = u_dev;
    p.u_stride = (int)stride;
    p.max_new = max_new;
    p.out_tok = nullptr;
    p.stream_ids = ring_dev;
    p.stream_stride = (int)stride;
    volatile const int* ring = s->stream_ring;
    int* h_flag = s->h_stage + 2 * s->B;  // pinned; [0] = 1, [1] = kSkip: the words that end a sequence on the device
    h_flag[0] = 1;
    h_flag[1] = kSkip;
    bool failed = false;
    for (int i = 0; i < emit_max && !failed; i++) {
        bool any = false;
        for (int b = 0; b < n_seq; b++) {
            if (stopped[b] || emit[b] <= i) continue;
            any = true;
            if (!sp.greedy) s->stream_u[(size_t)b * stride + i] = draw(user, b);
        }
        if (!any) break;
        {
            Timed t(s, KC_SELECT);
            launch_select(p, n_seq, s->stream);
        }
        if (i + 1 < emit_max) enqueue_step(s, n_seq, s->tok, s->tok, false);
        for (int b = 0; b < n_seq && !failed; b++) {
            if (stopped[b] || emit[b] <= i) continue;
            int v = 0;
            for (long spin = 0; (v = ring[(size_t)b * stride + i]) == 0; spin++) {
                if ((spin & 0xfff) == 0xfff && cudaStreamQuery(s->stream) != cudaErrorNotReady) {
                    v = ring[(size_t)b * stride + i];  // the stream drained: either the id is there or the step failed
                    if (v == 0) failed = true;
                    break;
                }
            }
            if (failed) break;
            given[b]++;
            if (on_token(user, b, i, v - 1) != 0) {
                // no further ids for this sequence: mark it done and take it out of the next step
                stopped[b] = 1;
                GRADB_CUDA(cudaMemcpyAsync(s->done + b, h_flag, sizeof(int), cudaMemcpyHostToDevice, s->stream));
                GRADB_CUDA(cudaMemcpyAsync(s->tok + b, h_flag + 1, sizeof(int), cudaMemcpyHostToDevice, s->stream));
            }
        }
    }
    GRADB_CUDA(cudaMemcpyAsync(s->h_stage, s->pos, n_seq * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    if (failed) throw Error(GRADB_ERR_CUDA, "the decode loop ended without producing the next id");
    for (int b = 0; b < n_seq; b++) {
        s->h_pos[b] = s->h_stage[b];
        if (emitted) emitted[b] = given[b];
    }
    GRADB_CUDA(cudaEventElapsedTime(&s->last_ms, s->ev_begin, s->ev_end));
}

// ------------------------------------------------------------------------------------------------ serving

static void ensure_serving(Session* s) {
    if (s->max_new_seq) return;
    dalloc(&s->max_new_seq, (size_t)s->B);
    dalloc(&s->serve_u, (size_t)s->B * (s->T + 2));
    GRADB_CUDA(cudaMemsetAsync(s->max_new_seq, 0, (size_t)s->B * sizeof(int), s->stream));
}

void session_admit(Session* s, int n_admit, const int32_t* seqs, const int32_t* prompts, const int32_t* offsets,
                   const int32_t* max_new, const float* const* uniforms, int reuse_prefix, int32_t* reused_out) {
    if (n_admit < 1 || n_admit > s->B) throw Error(GRADB_ERR_INVALID, "n_admit out of range for this session");
    GRADB_CUDA(cudaSetDevice(s->m->device));
    ensure_serving(s);
    // Everything is validated before any slot changes.
    int rows = 0;
    std::vector<char> seen(s->B, 0);
    for (int i = 0; i < n_admit; i++) {
        const int b = seqs[i], len = offsets[i + 1] - offsets[i];
        if (b < 0 || b >= s->B || seen[b]) throw Error(GRADB_ERR_INVALID, "slot index out of range or repeated");
        seen[b] = 1;
        if (len < 1) throw Error(GRADB_ERR_INVALID, "an admitted prompt must not be empty");
        if (len > s->T) throw Error(GRADB_ERR_CONTEXT_FULL, "InferenceSession: context exceeds max_len");
        if (max_new[i] < 0) throw Error(GRADB_ERR_INVALID, "max_new must not be negative");
        for (int j = offsets[i]; j < offsets[i + 1]; j++) {
            if (prompts[j] < 0 || prompts[j] >= s->V) {
                throw Error(GRADB_ERR_BAD_TOKEN, "InferenceSession: token id out of vocab range");
            }
        }
        rows = std::max(rows, b + 1);
    }
    // Per slot: how much of the cache stays, the slot's fresh loop state, the rest of the prompt as its feed.
    std::vector<int32_t> feed_tok, feed_off(rows + 1, 0);
    std::vector<int> keep(s->B, 0), first(s->B, -1);
    for (int i = 0; i < n_admit; i++) first[seqs[i]] = i;
    size_t total = 0;
    for (int b = 0; b < rows; b++) {
        feed_off[b] = (int32_t)feed_tok.size();
        const int i = first[b];
        if (i < 0) continue;
        const int32_t* pr = prompts + offsets[i];
        const int len = offsets[i + 1] - offsets[i];
        int k = 0;
        if (reuse_prefix) {
            const std::vector<int>& old = s->h_ids[b];
            const int lim = std::min({len - 1, s->h_pos[b], (int)old.size()});  // the last prompt id is always fed: its logits are needed
            while (k < lim && old[k] == pr[k]) k++;
        }
        keep[b] = k;
        if (reused_out) reused_out[i] = k;
        feed_tok.insert(feed_tok.end(), pr + k, pr + len);
        total += (size_t)(len - k);
    }
    feed_off[rows] = (int32_t)feed_tok.size();
    // device state of the admitted slots: position and history length = kept prefix, nothing emitted, not done
    std::vector<int> st(4 * (size_t)n_admit);
    for (int i = 0; i < n_admit; i++) {
        const int b = seqs[i];
        const int vals[5] = {keep[b], keep[b], 0, 0, kSkip};
        int* dst[5] = {s->pos + b, s->hist_len + b, s->gen + b, s->done + b, s->tok + b};
        for (int f = 0; f < 5; f++) {
            GRADB_CUDA(cudaMemcpyAsync(dst[f], &vals[f], sizeof(int), cudaMemcpyHostToDevice, s->stream));
        }
        GRADB_CUDA(cudaMemcpyAsync(s->max_new_seq + b, &max_new[i], sizeof(int), cudaMemcpyHostToDevice, s->stream));
        if (uniforms && uniforms[i] && max_new[i] > 0) {
            const int n = std::min(max_new[i], s->T + 2);
            GRADB_CUDA(cudaMemcpyAsync(s->serve_u + (size_t)b * (s->T + 2), uniforms[i], n * sizeof(float),
                                       cudaMemcpyHostToDevice, s->stream));
        }
        GRADB_CUDA(cudaStreamSynchronize(s->stream));  // `vals` and the caller's arrays are pageable
        s->h_pos[b] = keep[b];
        s->h_ids[b].assign(prompts + offsets[i], prompts + offsets[i + 1]);
        s->h_live[b] = 1;
        s->h_gen[b] = 0;
    }
    const int steps = upload_prompt_matrix(s, feed_tok.data(), feed_off.data(), rows);
    GRADB_CUDA(cudaEventRecord(s->ev_begin, s->stream));
    if (batched_feed_available(s) && total >= 16) enqueue_prompt_feed_batched(s, feed_tok.data(), feed_off.data(), rows);
    else enqueue_prompt_feed(s, steps, rows);
    GRADB_CUDA(cudaEventRecord(s->ev_end, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    GRADB_CUDA(cudaEventElapsedTime(&s->last_ms, s->ev_begin, s->ev_end));
    for (int b = 0; b < rows; b++) s->h_pos[b] += feed_off[b + 1] - feed_off[b];
}

void session_release(Session* s, int seq) {
    if (seq < 0 || seq >= s->B) throw Error(GRADB_ERR_INVALID, "slot index out of range");
    GRADB_CUDA(cudaSetDevice(s->m->device));
    const int one = 1, skip = kSkip;
    GRADB_CUDA(cudaMemcpyAsync(s->done + seq, &one, sizeof(int), cudaMemcpyHostToDevice, s->stream));
    GRADB_CUDA(cudaMemcpyAsync(s->tok + seq, &skip, sizeof(int), cudaMemcpyHostToDevice, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    s->h_live[seq] = 0;
}

int session_slot_ids(const Session* s, int seq, int32_t* ids_out, int capacity) {
    if (seq < 0 || seq >= s->B) throw Error(GRADB_ERR_INVALID, "slot index out of range");
    const std::vector<int>& ids = s->h_ids[seq];
    for (int i = 0; i < (int)ids.size() && i < capacity; i++) ids_out[i] = ids[i];
    return (int)ids.size();
}

void session_decode(Session* s, const gradb_sampling& sp, int n_steps, const int32_t* stop_ids, int n_stop,
                    int32_t* out_ids, int out_stride, int32_t* out_count, int32_t* finished) {
    if (n_steps < 1) throw Error(GRADB_ERR_INVALID, "n_steps must be positive");
    if (n_stop < 0 || n_stop > 8 || (n_stop > 0 && !stop_ids)) throw Error(GRADB_ERR_INVALID, "at most 8 stop ids");
    if (out_stride < n_steps) throw Error(GRADB_ERR_INVALID, "out_stride must hold n_steps ids");
    validate_sampling(s, sp);
    GRADB_CUDA(cudaSetDevice(s->m->device));
    ensure_serving(s);
    int rows = 0;
    for (int b = 0; b < s->B; b++) {
        if (s->h_live[b]) rows = b + 1;
    }
    for (int b = 0; b < s->B; b++) {
        out_count[b] = 0;
        if (finished) finished[b] = s->h_live[b] ? 0 : 1;
    }
    if (rows == 0) return;
    SelectParams p = make_select(s, sp);
    p.loop_mode = 1;
    p.uniforms = s->serve_u;
    p.u_stride = s->T + 2;
    p.max_new = 0;
    p.max_new_seq = s->max_new_seq;
    p.out_tok = nullptr;
    p.n_stop = n_stop;
    for (int i = 0; i < n_stop; i++) p.stop_ids[i] = stop_ids[i];
    // Vacant and finished slots below `rows` are marked done on the device, so neither kernel touches them.
    for (int b = 0; b < rows; b++) s->h_stage[b] = s->h_live[b] ? 0 : 1;
    GRADB_CUDA(cudaMemcpyAsync(s->done, s->h_stage, rows * sizeof(int), cudaMemcpyHostToDevice, s->stream));
    GRADB_CUDA(cudaEventRecord(s->ev_begin, s->stream));
    auto eager_iteration = [&] {
        {
            Timed t(s, KC_SELECT);
            launch_select(p, rows, s->stream);
        }
        enqueue_step(s, rows, s->tok, s->tok, false);
    };
    int i = 0;
    const bool graph_ok = s->use_graph && !s->profiling && n_steps > 2;
    if (graph_ok) {
        const bool same = s->serve_graph && s->serve_rows == rows && s->serve_n_stop == n_stop &&
                          std::memcmp(&s->serve_params, &sp, sizeof(sp)) == 0 &&
                          std::memcmp(s->serve_stop, p.stop_ids, sizeof(p.stop_ids)) == 0;
        if (!same) {
            if (s->serve_graph) {
                cudaGraphExecDestroy(s->serve_graph);
                s->serve_graph = nullptr;
            }
            // The first iteration runs eagerly, so every kernel of the step has its launch attributes before capture.
            eager_iteration();
            i = 1;
            cudaGraph_t g = nullptr;
            GRADB_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
            g_capturing = true;
            try {
                launch_select(p, rows, s->stream);
                enqueue_step(s, rows, s->tok, s->tok, false);
            } catch (...) {
                g_capturing = false;
                cudaStreamEndCapture(s->stream, &g);
                if (g) cudaGraphDestroy(g);
                throw;
            }
            g_capturing = false;
            GRADB_CUDA(cudaStreamEndCapture(s->stream, &g));
            const cudaError_t e = cudaGraphInstantiate(&s->serve_graph, g, 0);
            cudaGraphDestroy(g);
            if (e != cudaSuccess) throw Error(GRADB_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
            s->serve_params = sp;
            s->serve_rows = rows;
            s->serve_n_stop = n_stop;
            std::memcpy(s->serve_stop, p.stop_ids, sizeof(p.stop_ids));
        }
    }
    for (; i < n_steps; i++) {
        if (graph_ok) {
            GRADB_CUDA(cudaGraphLaunch(s->serve_graph, s->stream));
            count_launch(s->use_b1 && rows == 1 ? 2 : 4 + 5 * s->L);
        } else {
            eager_iteration();
        }
    }
    GRADB_CUDA(cudaEventRecord(s->ev_end, s->stream));
    std::vector<int> lens(rows), done(rows), pos(rows);
    std::vector<int> hist((size_t)rows * s->hist_stride);
    GRADB_CUDA(cudaMemcpyAsync(lens.data(), s->hist_len, rows * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    GRADB_CUDA(cudaMemcpyAsync(done.data(), s->done, rows * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    GRADB_CUDA(cudaMemcpyAsync(pos.data(), s->pos, rows * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    GRADB_CUDA(cudaMemcpyAsync(hist.data(), s->hist, hist.size() * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    GRADB_CUDA(cudaEventElapsedTime(&s->last_ms, s->ev_begin, s->ev_end));
    for (int b = 0; b < rows; b++) {
        if (!s->h_live[b]) continue;
        const int before = (int)s->h_ids[b].size();
        const int after = std::min(lens[b], s->hist_stride);
        const int* row = hist.data() + (size_t)b * s->hist_stride;
        int n = 0;
        for (int j = before; j < after; j++, n++) {
            if (n < out_stride) out_ids[(size_t)b * out_stride + n] = row[j];
            s->h_ids[b].push_back(row[j]);
        }
        out_count[b] = std::min(n, out_stride);
        s->h_gen[b] += n;
        s->h_pos[b] = pos[b];
        if (done[b]) s->h_live[b] = 0;
        if (finished) finished[b] = done[b] ? 1 : 0;
    }
}

void session_set_profiling(Session* s, bool on) {
    GRADB_CUDA(cudaSetDevice(s->m->device));
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
    collect_spans(s);
    check_status(s);
    s->profiling = on;
    for (int i = 0; i < kKernelClasses; i++) {
        s->class_ms[i] = 0.0;
        s->class_launches[i] = 0;
    }
}

void session_cache_row(Session* s, int seq, int layer, int which, int pos, float* row_host) {
    if (seq < 0 || seq >= s->B || layer < 0 || layer >= s->L || pos < 0 || pos >= s->T || which < 0 || which > 1) {
        throw Error(GRADB_ERR_INVALID, "cache row index out of range");
    }
    GRADB_CUDA(cudaSetDevice(s->m->device));
    const float* base = (which ? s->vcache : s->kcache) + (size_t)layer * layer_cache_elems(s);
    for (int h = 0; h < s->H; h++) {
        const float* src = base + (((size_t)seq * s->H + h) * s->T + pos) * s->hs;
        GRADB_CUDA(cudaMemcpyAsync(row_host + (size_t)h * s->hs, src, s->hs * sizeof(float), cudaMemcpyDeviceToHost,
                                   s->stream));
    }
    GRADB_CUDA(cudaStreamSynchronize(s->stream));
}

}  // namespace gradb
