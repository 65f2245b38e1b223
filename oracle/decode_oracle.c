/* CPU restatement of grad.cpp's KV-cached token loop. See decode_oracle.h:
 * TEST INFRASTRUCTURE ONLY; parity pinned against the compiled reference. */
#include "decode_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef GRO_REAL real;

/* ------------------------------------------------------------------ model */

typedef struct {
    const float *wq, *wk, *wv, *wo, *bq, *bk, *bv, *bo;
    const float *w1, *b1, *w2, *b2; /* GPT-2: W1 b1 W2 b2. Modern: w1 = up, w2 = down */
    const float* wgate;             /* Modern only */
    const float *n1g, *n1b, *n2g, *n2b;
} gro_layer;

struct gro_model {
    int vocab, d, layers, heads, max_len, arch, dff;
    int has_fp;
    uint32_t fp_kind;
    uint64_t fp_hash;
    float* blob; /* every tensor, in file order */
    const float *emb, *pos, *fng, *fnb;
    gro_layer* layer;
};

static void set_err(char* err, size_t cap, const char* path, const char* msg) {
    /* gpt_model.cpp:521-524 wraps every failure this way. */
    if (err && cap) snprintf(err, cap, "Failed to load model from %s: %s", path, msg);
}

typedef struct {
    FILE* f;
    char msg[256];
    int failed;
} reader;

static int rd(reader* r, void* out, size_t n, const char* what) {
    if (r->failed) return 0;
    if (fread(out, 1, n, r->f) != n) {
        snprintf(r->msg, sizeof r->msg, "file ends while reading %s", what);
        r->failed = 1;
        return 0;
    }
    return 1;
}

/* gpt_model.cpp:246-260: dims must equal the constructed parameter's. */
static const float* rd_tensor(reader* r, float** cursor, int rows, int cols, const char* what) {
    int fr = 0, fc = 0;
    if (!rd(r, &fr, 4, what) || !rd(r, &fc, 4, what)) return NULL;
    if (fr <= 0 || fc <= 0 || fr != rows || fc != cols) {
        snprintf(r->msg, sizeof r->msg, "%s is %dx%d, model expects %dx%d", what, fr, fc, rows, cols);
        r->failed = 1;
        return NULL;
    }
    float* dst = *cursor;
    size_t n = (size_t)rows * (size_t)cols;
    if (fread(dst, 4, n, r->f) != n) {
        snprintf(r->msg, sizeof r->msg, "file ends inside %s", what);
        r->failed = 1;
        return NULL;
    }
    *cursor += n;
    return dst;
}

static int in_range(reader* r, const char* name, int v, int lo, int hi) {
    if (v < lo || v > hi) {
        snprintf(r->msg, sizeof r->msg, "header field %s = %d is outside [%d, %d]", name, v, lo, hi);
        r->failed = 1;
        return 0;
    }
    return 1;
}

/* feedforward.h:24-28 */
static int resolve_dff(int d, int modern) {
    return modern ? ((8 * d / 3) + 63) / 64 * 64 : 4 * d;
}

gro_model* GRO(model_load)(const char* path, char* err, size_t err_cap) {
    FILE* f = fopen(path, "rb");
    if (!f) {
        if (err && err_cap) snprintf(err, err_cap, "Could not open checkpoint for reading: %s", path);
        return NULL;
    }
    reader r = {f, {0}, 0};
    gro_model* m = (gro_model*)calloc(1, sizeof *m);
    uint32_t magic = 0, version = 0, arch = 0;
    float dropout = 0;
    rd(&r, &magic, 4, "magic number");
    if (!r.failed && magic != 0x4750544Du) {
        snprintf(r.msg, sizeof r.msg, "not a grad.cpp checkpoint (wrong magic number)");
        r.failed = 1;
    }
    rd(&r, &version, 4, "format version");
    if (!r.failed && version != 1 && version != 2) {
        snprintf(r.msg, sizeof r.msg, "unsupported format version %u", version);
        r.failed = 1;
    }
    if (!r.failed && version == 2) {
        rd(&r, &arch, 4, "architecture tag");
        if (!r.failed && arch > 1) {
            snprintf(r.msg, sizeof r.msg, "unknown architecture tag %u", arch);
            r.failed = 1;
        }
    }
    rd(&r, &m->vocab, 4, "vocab_size");
    rd(&r, &m->d, 4, "d_model");
    rd(&r, &m->layers, 4, "num_layers");
    rd(&r, &m->heads, 4, "num_heads");
    rd(&r, &m->max_len, 4, "max_len");
    rd(&r, &dropout, 4, "dropout_rate");
    if (!r.failed) {
        (void)(in_range(&r, "vocab_size", m->vocab, 1, 1 << 24) && in_range(&r, "d_model", m->d, 1, 1 << 16) &&
               in_range(&r, "num_layers", m->layers, 1, 1 << 12) &&
               in_range(&r, "num_heads", m->heads, 1, m->d) &&
               in_range(&r, "max_len", m->max_len, 1, 1 << 20));
    }
    if (!r.failed && m->d % m->heads != 0) {
        snprintf(r.msg, sizeof r.msg, "d_model %d is not divisible by num_heads %d", m->d, m->heads);
        r.failed = 1;
    }
    if (!r.failed && !(dropout >= 0.0f && dropout < 1.0f)) {
        snprintf(r.msg, sizeof r.msg, "dropout_rate %f is outside [0, 1)", dropout);
        r.failed = 1;
    }
    if (r.failed) goto fail;

    m->arch = (int)arch;
    const int modern = m->arch == 1;
    const int d = m->d, V = m->vocab, L = m->layers;
    m->dff = resolve_dff(d, modern);
    const int dff = m->dff;
    size_t per_layer = 4 * (size_t)d * d + 4 * (size_t)d + 4 * (size_t)d;
    per_layer += modern ? 3 * (size_t)d * dff : 2 * (size_t)d * dff + dff + d;
    size_t total = (size_t)V * d + (modern ? 0 : (size_t)m->max_len * d) + L * per_layer + 2 * (size_t)d;
    m->blob = (float*)malloc(total * sizeof(float));
    m->layer = (gro_layer*)calloc((size_t)L, sizeof(gro_layer));
    float* cur = m->blob;

    m->emb = rd_tensor(&r, &cur, V, d, "token embedding");
    if (!modern) m->pos = rd_tensor(&r, &cur, m->max_len, d, "position embedding");
    for (int l = 0; l < L && !r.failed; l++) {
        gro_layer* y = &m->layer[l];
        char w[64];
#define NAME(s) (snprintf(w, sizeof w, "layer %d %s", l, s), w)
        y->wq = rd_tensor(&r, &cur, d, d, NAME("W_q"));
        y->wk = rd_tensor(&r, &cur, d, d, NAME("W_k"));
        y->wv = rd_tensor(&r, &cur, d, d, NAME("W_v"));
        y->wo = rd_tensor(&r, &cur, d, d, NAME("W_o"));
        y->bq = rd_tensor(&r, &cur, 1, d, NAME("b_q"));
        y->bk = rd_tensor(&r, &cur, 1, d, NAME("b_k"));
        y->bv = rd_tensor(&r, &cur, 1, d, NAME("b_v"));
        y->bo = rd_tensor(&r, &cur, 1, d, NAME("b_o"));
        if (modern) {
            y->wgate = rd_tensor(&r, &cur, d, dff, NAME("FFN gate"));
            y->w1 = rd_tensor(&r, &cur, d, dff, NAME("FFN up"));
            y->w2 = rd_tensor(&r, &cur, dff, d, NAME("FFN down"));
        } else {
            y->w1 = rd_tensor(&r, &cur, d, dff, NAME("FFN W1"));
            y->b1 = rd_tensor(&r, &cur, 1, dff, NAME("FFN b1"));
            y->w2 = rd_tensor(&r, &cur, dff, d, NAME("FFN W2"));
            y->b2 = rd_tensor(&r, &cur, 1, d, NAME("FFN b2"));
        }
        y->n1g = rd_tensor(&r, &cur, 1, d, NAME("norm1 gamma"));
        y->n1b = rd_tensor(&r, &cur, 1, d, NAME("norm1 beta"));
        y->n2g = rd_tensor(&r, &cur, 1, d, NAME("norm2 gamma"));
        y->n2b = rd_tensor(&r, &cur, 1, d, NAME("norm2 beta"));
#undef NAME
    }
    m->fng = rd_tensor(&r, &cur, 1, d, "final norm gamma");
    m->fnb = rd_tensor(&r, &cur, 1, d, "final norm beta");
    if (r.failed) goto fail;

    /* Trailer sections, gpt_model.cpp:489-515. */
    for (;;) {
        int c = fgetc(f);
        if (c == EOF) break;
        ungetc(c, f);
        unsigned char h[8];
        if (!rd(&r, h, 8, "trailer section header")) goto fail;
        uint32_t len = (uint32_t)h[4] | (uint32_t)h[5] << 8 | (uint32_t)h[6] << 16 | (uint32_t)h[7] << 24;
        if (len > (1u << 20)) {
            snprintf(r.msg, sizeof r.msg, "trailer section has an implausible length (%u bytes)", len);
            goto fail;
        }
        if (memcmp(h, "TKFP", 4) != 0) {
            for (uint32_t i = 0; i < len; i++) {
                if (fgetc(f) == EOF) {
                    snprintf(r.msg, sizeof r.msg, "file ends inside trailer section");
                    goto fail;
                }
            }
            continue;
        }
        if (len != 12) {
            snprintf(r.msg, sizeof r.msg, "tokenizer trailer has length %u, expected 12", len);
            goto fail;
        }
        unsigned char p[12];
        if (!rd(&r, p, 12, "tokenizer trailer")) goto fail;
        uint32_t kind = (uint32_t)p[0] | (uint32_t)p[1] << 8 | (uint32_t)p[2] << 16 | (uint32_t)p[3] << 24;
        if (kind != 1 && kind != 2) {
            snprintf(r.msg, sizeof r.msg, "unknown tokenizer kind %u", kind);
            goto fail;
        }
        uint64_t hash = 0;
        for (int i = 0; i < 8; i++) hash |= (uint64_t)p[4 + i] << (8 * i);
        m->has_fp = 1;
        m->fp_kind = kind;
        m->fp_hash = hash;
    }
    fclose(f);
    return m;

fail:
    set_err(err, err_cap, path, r.msg);
    fclose(f);
    GRO(model_free)(m);
    return NULL;
}

void GRO(model_free)(gro_model* m) {
    if (!m) return;
    free(m->blob);
    free(m->layer);
    free(m);
}

void GRO(model_dims)(const gro_model* m, int* dims) {
    dims[0] = m->vocab;
    dims[1] = m->d;
    dims[2] = m->layers;
    dims[3] = m->heads;
    dims[4] = m->max_len;
    dims[5] = m->arch;
    dims[6] = m->dff;
    dims[7] = m->has_fp;
    dims[8] = (int)m->fp_kind;
}

uint64_t GRO(model_fingerprint_hash)(const gro_model* m) { return m->fp_hash; }

/* ---------------------------------------------------------------- session */

struct gro_session {
    const gro_model* m;
    int pos;
    real **k, **v; /* per layer: (max_len, d) rows */
    real *x, *h, *q, *attn, *scores, *ffn, *gate, *cosv, *sinv, *logits;
};

gro_session* GRO(session_new)(const gro_model* m) {
    gro_session* s = (gro_session*)calloc(1, sizeof *s);
    s->m = m;
    const size_t d = (size_t)m->d;
    s->k = (real**)calloc((size_t)m->layers, sizeof(real*));
    s->v = (real**)calloc((size_t)m->layers, sizeof(real*));
    for (int l = 0; l < m->layers; l++) {
        s->k[l] = (real*)calloc((size_t)m->max_len * d, sizeof(real));
        s->v[l] = (real*)calloc((size_t)m->max_len * d, sizeof(real));
    }
    s->x = (real*)calloc(d, sizeof(real));
    s->h = (real*)calloc(d, sizeof(real));
    s->q = (real*)calloc(d, sizeof(real));
    s->attn = (real*)calloc(d, sizeof(real));
    s->scores = (real*)calloc((size_t)m->max_len, sizeof(real));
    s->ffn = (real*)calloc((size_t)m->dff, sizeof(real));
    s->gate = (real*)calloc((size_t)m->dff, sizeof(real));
    s->cosv = (real*)calloc(d, sizeof(real));
    s->sinv = (real*)calloc(d, sizeof(real));
    s->logits = (real*)calloc((size_t)m->vocab, sizeof(real));
    return s;
}

void GRO(session_free)(gro_session* s) {
    if (!s) return;
    for (int l = 0; l < s->m->layers; l++) {
        free(s->k[l]);
        free(s->v[l]);
    }
    free(s->k);
    free(s->v);
    free(s->x);
    free(s->h);
    free(s->q);
    free(s->attn);
    free(s->scores);
    free(s->ffn);
    free(s->gate);
    free(s->cosv);
    free(s->sinv);
    free(s->logits);
    free(s);
}

void GRO(session_reset)(gro_session* s) { s->pos = 0; }
int GRO(session_position)(const gro_session* s) { return s->pos; }

void GRO(session_cache_row)(const gro_session* s, int layer, int which, int pos, float* out) {
    const real* src = (which ? s->v[layer] : s->k[layer]) + (size_t)pos * s->m->d;
    for (int j = 0; j < s->m->d; j++) out[j] = (float)src[j];
}

/* y (=|+=) x @ W (+ b). W is (in, out) row-major. The reference issues an M=1
 * sgemm (inference.cpp:14-28, 94-96); the BLAS's blocking order is not part
 * of the algorithm, so rows are accumulated in index order here. */
static void matvec(const real* x, const float* W, const float* b, real* y, int in, int out, int accumulate) {
    if (!accumulate) {
        for (int j = 0; j < out; j++) y[j] = b ? (real)b[j] : (real)0;
    } else if (b) {
        for (int j = 0; j < out; j++) y[j] += (real)b[j];
    }
    for (int i = 0; i < in; i++) {
        const real xi = x[i];
        const float* row = W + (size_t)i * out;
        for (int j = 0; j < out; j++) y[j] += xi * (real)row[j];
    }
}

static real exp_r(real v) { return sizeof(real) == 4 ? (real)expf((float)v) : (real)exp((double)v); }
static real tanh_r(real v) { return sizeof(real) == 4 ? (real)tanhf((float)v) : (real)tanh((double)v); }
static real sqrt_r(real v) { return sizeof(real) == 4 ? (real)sqrtf((float)v) : (real)sqrt((double)v); }

/* inference.cpp:30-58 */
static void norm_row(const real* x, const float* g, const float* beta, int d, int rms, real* out) {
    const real eps = (real)1e-5f;
    if (rms) {
        real ms = 0;
        for (int j = 0; j < d; j++) ms += x[j] * x[j];
        const real r = (real)1 / sqrt_r(ms / (real)d + eps);
        for (int j = 0; j < d; j++) out[j] = (real)g[j] * x[j] * r;
        return;
    }
    real sum = 0;
    for (int j = 0; j < d; j++) sum += x[j];
    const real mean = sum / (real)d;
    real var = 0;
    for (int j = 0; j < d; j++) {
        const real diff = x[j] - mean;
        var += diff * diff;
    }
    var /= (real)d;
    const real inv_std = (real)1 / sqrt_r(var + eps);
    for (int j = 0; j < d; j++) out[j] = (real)g[j] * (x[j] - mean) * inv_std + (real)beta[j];
}


int GRO(session_step)(gro_session* s, int token, float* logits_out) {
    const gro_model* m = s->m;
    if (s->pos >= m->max_len) return 1;              /* inference.cpp:151-153 */
    if (token < 0 || token >= m->vocab) return 2;    /* inference.cpp:154-156 */
    const int d = m->d, H = m->heads, hs = d / H, dff = m->dff, pos = s->pos;
    const int modern = m->arch == 1;
    const float* e = m->emb + (size_t)token * d;

    /* inference.cpp:159-182 (embedding scale is 1.0, token_embedding.h:12) */
    if (modern) {
        for (int j = 0; j < d; j++) s->x[j] = (real)e[j] * (real)1.0f;
        const int half = hs / 2;
        for (int j = 0; j < half; j++) {
            if (sizeof(real) == 4) {
                const float theta = powf(10000.0f, -2.0f * (float)j / (float)hs);
                s->cosv[j] = (real)cosf((float)pos * theta);
                s->sinv[j] = (real)sinf((float)pos * theta);
            } else {
                const double theta = pow(10000.0, -2.0 * (double)j / (double)hs);
                s->cosv[j] = (real)cos((double)pos * theta);
                s->sinv[j] = (real)sin((double)pos * theta);
            }
        }
    } else {
        const float* p = m->pos + (size_t)pos * d;
        for (int j = 0; j < d; j++) s->x[j] = (real)e[j] * (real)1.0f + (real)p[j];
    }

    const real inv_sqrt_hs = (real)1 / sqrt_r((real)hs);
    const int ctx = pos + 1;

    for (int l = 0; l < m->layers; l++) {
        const gro_layer* y = &m->layer[l];
        norm_row(s->x, y->n1g, y->n1b, d, modern, s->h);                    /* :193 */
        real* krow = s->k[l] + (size_t)pos * d;
        real* vrow = s->v[l] + (size_t)pos * d;
        matvec(s->h, y->wq, y->bq, s->q, d, d, 0);                          /* :197-199 */
        matvec(s->h, y->wk, y->bk, krow, d, d, 0);
        matvec(s->h, y->wv, y->bv, vrow, d, d, 0);
        if (modern) {                                                       /* :101-115, 203-206 */
            for (int t = 0; t < 2; t++) {
                real* row = t ? krow : s->q;
                for (int hd = 0; hd < H; hd++) {
                    real* head = row + hd * hs;
                    for (int j = 0; j < hs / 2; j++) {
                        const real c = s->cosv[j], sn = s->sinv[j];
                        const real a = head[2 * j], b = head[2 * j + 1];
                        head[2 * j] = a * c - b * sn;
                        head[2 * j + 1] = a * sn + b * c;
                    }
                }
            }
        }
        for (int hd = 0; hd < H; hd++) {                                    /* :208-225 */
            const int off = hd * hs;
            for (int t = 0; t < ctx; t++) {
                const real* kt = s->k[l] + (size_t)t * d + off;
                real dot = 0;
                for (int j = 0; j < hs; j++) dot += s->q[off + j] * kt[j];
                s->scores[t] = dot * inv_sqrt_hs;
            }
            real mx = s->scores[0];                                          /* :60-67 */
            for (int t = 1; t < ctx; t++) mx = s->scores[t] > mx ? s->scores[t] : mx;
            real sum = 0;
            for (int t = 0; t < ctx; t++) {
                s->scores[t] = exp_r(s->scores[t] - mx);
                sum += s->scores[t];
            }
            const real inv_sum = (real)1 / sum;
            for (int t = 0; t < ctx; t++) s->scores[t] *= inv_sum;
            real* oh = s->attn + off;
            for (int j = 0; j < hs; j++) oh[j] = 0;
            for (int t = 0; t < ctx; t++) {
                const real* vt = s->v[l] + (size_t)t * d + off;
                const real w = s->scores[t];
                for (int j = 0; j < hs; j++) oh[j] += w * vt[j];
            }
        }
        matvec(s->attn, y->wo, y->bo, s->x, d, d, 1);                       /* :228 */
        norm_row(s->x, y->n2g, y->n2b, d, modern, s->h);                    /* :230 */
        if (modern) {                                                       /* :232-241 */
            matvec(s->h, y->wgate, NULL, s->gate, d, dff, 0);
            for (int j = 0; j < dff; j++) s->gate[j] = s->gate[j] / ((real)1 + exp_r(-s->gate[j]));
            matvec(s->h, y->w1, NULL, s->ffn, d, dff, 0);
            for (int j = 0; j < dff; j++) s->ffn[j] *= s->gate[j];
            matvec(s->ffn, y->w2, NULL, s->x, dff, d, 1);
        } else {                                                            /* :242-247, 69-80 */
            matvec(s->h, y->w1, y->b1, s->ffn, d, dff, 0);
            for (int j = 0; j < dff; j++) {
                const real v = s->ffn[j];
                const real t = tanh_r((real)0.79788456f * (v + (real)0.044715f * v * v * v));
                s->ffn[j] = (real)0.5f * v * ((real)1 + t);
            }
            matvec(s->ffn, y->w2, y->b2, s->x, dff, d, 1);
        }
    }

    norm_row(s->x, m->fng, m->fnb, d, modern, s->h);                        /* :251 */
    for (int v = 0; v < m->vocab; v++) {                                    /* :254 */
        const float* row = m->emb + (size_t)v * d;
        real acc = 0;
        for (int j = 0; j < d; j++) acc += s->h[j] * (real)row[j];
        s->logits[v] = acc;
    }
    if (logits_out) {
        for (int v = 0; v < m->vocab; v++) logits_out[v] = (float)s->logits[v];
    }
    s->pos++;
    return 0;
}

/* ---------------------------------------------------------------- sampler */
#ifndef GRO_SKIP_SAMPLER

/* text_gen.cpp:14-33: the last min(50, n) ids, one application per occurrence. */
void gro_apply_penalty(float* logits, int vocab, const int* tokens, int n_tokens, float penalty) {
    (void)vocab;
    if (penalty == 1.0f) return;
    const int window = n_tokens < 50 ? n_tokens : 50;
    for (int k = n_tokens - window; k < n_tokens; k++) {
        const int id = tokens[k];
        if (logits[id] > 0) {
            logits[id] /= penalty;
        } else {
            logits[id] *= penalty;
        }
    }
}

/* text_gen.cpp:52-60: first index of the maximum, strict >. */
int gro_argmax(const float* logits, int vocab) {
    int best = 0;
    float mx = logits[0];
    for (int j = 1; j < vocab; j++) {
        if (logits[j] > mx) {
            mx = logits[j];
            best = j;
        }
    }
    return best;
}

static int cmp_desc(const void* a, const void* b) {
    const float x = *(const float*)a, y = *(const float*)b;
    return (x < y) - (x > y);
}

/* text_gen.cpp:135-209. The reference sorts (value, index) pairs by value
 * only; every quantity it then uses depends on the sorted VALUES alone, so a
 * plain descending sort of the values is equivalent. */
int gro_sample(const float* logits, int vocab, float temperature, int top_k, float top_p, float u,
               float* probs_out) {
    const size_t n = (size_t)vocab;
    float* x = (float*)malloc(n * sizeof(float));
    float* sorted = (float*)malloc(n * sizeof(float));
    const float inv_t = 1.0f / temperature;                  /* :136 */
    for (size_t i = 0; i < n; i++) x[i] = logits[i] * inv_t;

    if (top_k > 0 && top_k < vocab) {                        /* :138-154 */
        memcpy(sorted, x, n * sizeof(float));
        qsort(sorted, n, sizeof(float), cmp_desc);
        const float kth = sorted[top_k - 1];
        for (size_t i = 0; i < n; i++) {
            if (x[i] < kth) x[i] = -1e10f;
        }
    }

    /* Tensor::softmax, tensor.cpp:421-452 */
    float mx = x[0];
    for (size_t i = 1; i < n; i++) mx = x[i] > mx ? x[i] : mx;
    for (size_t i = 0; i < n; i++) x[i] = expf(x[i] - mx);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) sum += x[i];
    const float inv_sum = 1.0f / sum;
    for (size_t i = 0; i < n; i++) x[i] *= inv_sum;

    if (top_p < 1.0f) {                                      /* :158-193 */
        memcpy(sorted, x, n * sizeof(float));
        qsort(sorted, n, sizeof(float), cmp_desc);
        float cumulative = 0.0f;
        size_t cutoff = 0;
        for (size_t i = 0; i < n; i++) {
            cumulative += sorted[i];
            if (cumulative >= top_p) {
                cutoff = i;
                break;
            }
        }
        const float cutoff_prob = sorted[cutoff];
        float kept = 0.0f;
        for (size_t i = 0; i < n; i++) {
            if (x[i] < cutoff_prob) {
                x[i] = 0.0f;
            } else {
                kept += x[i];
            }
        }
        if (kept > 0.0f) {
            for (size_t i = 0; i < n; i++) x[i] = x[i] / kept;
        }
    }

    int pick = vocab - 1;                                    /* :199-208 */
    float cumulative = 0.0f;
    for (size_t i = 0; i < n; i++) {
        cumulative += x[i];
        if (u <= cumulative) {
            pick = (int)i;
            break;
        }
    }
    if (probs_out) memcpy(probs_out, x, n * sizeof(float));
    free(x);
    free(sorted);
    return pick;
}
#endif

/* text_gen.cpp:37-91. No EOS stop; the id chosen when the context fills is
 * still emitted. */
int GRO(generate)(const gro_model* m, const int* prompt, int n_prompt, int max_tokens, int greedy,
                  float temperature, float repetition_penalty, int top_k, float top_p,
                  const float* draws, int* out, int cap) {
    if (n_prompt <= 0) return 0;
    gro_session* s = GRO(session_new)(m);
    const int V = m->vocab;
    float* logits = (float*)malloc((size_t)V * sizeof(float));
    float* work = (float*)malloc((size_t)V * sizeof(float));
    int* toks = (int*)malloc(((size_t)n_prompt + (size_t)max_tokens + 1) * sizeof(int));
    int n = 0, rc = 0;
    for (int i = 0; i < n_prompt && rc == 0; i++) {
        toks[n++] = prompt[i];
        rc = GRO(session_step)(s, prompt[i], logits);
    }
    for (int i = 0; i < max_tokens && rc == 0; i++) {
        memcpy(work, logits, (size_t)V * sizeof(float));
        gro_apply_penalty(work, V, toks, n, repetition_penalty);
        const int next = greedy ? gro_argmax(work, V)
                                : gro_sample(work, V, temperature, top_k, top_p, draws[i], NULL);
        toks[n++] = next;
        if (GRO(session_position)(s) >= m->max_len) break;
        rc = GRO(session_step)(s, next, logits);
    }
    const int total = rc == 0 ? n : -rc;
    for (int i = 0; i < n && i < cap; i++) out[i] = toks[i];
    free(logits);
    free(work);
    free(toks);
    GRO(session_free)(s);
    return total;
}

/* trainer.cpp:319-340 over variable.cpp:465-497 (log_softmax) and :533-556 (nll_loss). */
int GRO(mean_loss)(const gro_model* m, const int* inputs, const int* targets, int n_windows, int seq_len,
                   int batch_windows, double* mean_out, float* batch_loss_out, float* row_logp_out) {
    const int V = m->vocab;
    float* logits = (float*)malloc((size_t)V * sizeof(float));
    gro_session* s = GRO(session_new)(m);
    double weighted = 0.0;
    size_t rows = 0;
    int rc = 0, batch_index = 0;
    for (int w0 = 0; w0 < n_windows && rc == 0; w0 += batch_windows, batch_index++) {
        const int nb = batch_windows < n_windows - w0 ? batch_windows : n_windows - w0;
        float total = 0.0f; /* nll_loss keeps an fp32 running total */
        for (int b = 0; b < nb && rc == 0; b++) {
            GRO(session_reset)(s);
            for (int t = 0; t < seq_len && rc == 0; t++) {
                const size_t at = ((size_t)w0 + (size_t)b) * (size_t)seq_len + (size_t)t;
                rc = GRO(session_step)(s, inputs[at], logits);
                if (rc) break;
                real mx = logits[0];
                for (int j = 1; j < V; j++) mx = logits[j] > mx ? (real)logits[j] : mx;
                real sum = 0;
                for (int j = 0; j < V; j++) sum += exp_r((real)logits[j] - mx);
                const real log_sum = (sizeof(real) == 4 ? (real)logf((float)sum) : (real)log((double)sum));
                const int tg = targets[at];
                float logp = 0.0f;
                if (tg >= 0 && tg < V) {
                    logp = (float)(((real)logits[tg] - mx) - log_sum);
                    total -= logp;
                }
                if (row_logp_out) row_logp_out[at] = logp;
            }
        }
        total /= (float)((size_t)nb * (size_t)seq_len);
        if (batch_loss_out) batch_loss_out[batch_index] = total;
        weighted += (double)total * (double)nb;
        rows += (size_t)nb;
    }
    *mean_out = rows ? weighted / (double)rows : -1.0;
    free(logits);
    GRO(session_free)(s);
    return rc;
}
