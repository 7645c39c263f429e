/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement, in plain C, of the algorithm of Lighter++'s batch-1 decode step
 * (forward(token,pos) + sample).  Each function cites the reference lines it follows.
 * Arithmetic is scalar FP32 in the reference's own evaluation order, so for identical
 * inputs the results are bit-identical to the reference's CPU build; the only liberty
 * taken is that independent output rows of a matrix-vector product may be computed by
 * different OpenMP threads (each row's dot product keeps its sequential order).
 *
 * Pinning: tests/test_oracle.py checks this file against (a) the six known-answer tests of
 * the reference's src/runtests.cpp:87-306, (b) golden vectors under tests/golden/ produced
 * by the compiled reference (oracle/_ref/libref_cpu.so, see tests/golden/make_golden.py),
 * and (c) when oracle/_ref is present, bit-for-bit against the compiled reference on seeded
 * random models.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may
 * load the library built from this file.  Nothing under lighterpp_b200/ may.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_base;
    /* weights: caller-owned, per-layer tensors stacked [L][rows][cols] (model.h:34-53).  Matrices and
     * embedding are FP32, or (w_f16 != 0) IEEE binary16 that is widened exactly on use -- the values the
     * reference's GGUF loader produces with f16_to_f32 (loader.cpp:346-379) without holding them as FP32. */
    const float *tok_emb, *rms_att, *wq, *wk, *wv, *wo, *rms_ffn, *w1, *w2, *w3, *rms_final, *w_cls;
    int w_f16;
    /* run state (model.h:78-95) */
    float *x, *xb, *xb2, *hb, *he, *q, *k, *v, *att, *logits;
    float *key_cache, *value_cache; /* [L][KVH][seq_len][head_size] FP32 */
} oracle_model;

/* ops.cpp:9-17 -- out[i] = sum_k x[k]*w[i*d+k], k ascending, FP32. */
void oracle_matmul(float* out, const float* x, const float* w, int n, int d) {
#pragma omp parallel for schedule(static) if (((long)n * d) > 262144)
    for (int i = 0; i < n; i++) {
        float val = 0.0f;
        const float* row = w + (size_t)i * d;
        for (int k = 0; k < d; k++) val += x[k] * row[k];
        out[i] = val;
    }
}

/* Exact binary16 -> binary32 widening (every half is representable as a float). */
static inline float half_bits_to_float(uint16_t h) {
    uint32_t s = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, b;
    if (e == 0) {
        if (m == 0) {
            b = s;
        } else { /* subnormal: m * 2^-24 */
            int sh = 0;
            while (!(m & 1024u)) {
                m <<= 1;
                sh++;
            }
            b = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
        }
    } else if (e == 31) {
        b = s | 0x7f800000u | (m << 13);
    } else {
        b = s | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &b, 4);
    return f;
}

/* oracle_matmul on a binary16 matrix: the same sequential FP32 sum over the exactly widened weights. */
void oracle_matmul_f16(float* out, const float* x, const uint16_t* w, int n, int d) {
#pragma omp parallel for schedule(static) if (((long)n * d) > 262144)
    for (int i = 0; i < n; i++) {
        float val = 0.0f;
        const uint16_t* row = w + (size_t)i * d;
        for (int k = 0; k < d; k++) val += x[k] * half_bits_to_float(row[k]);
        out[i] = val;
    }
}

/* Matrix `w` (an oracle_model weight pointer) from element offset `off`, in the model's weight type. */
static void model_matmul(const oracle_model* m, float* out, const float* x, const float* w, size_t off, int n, int d) {
    if (m->w_f16)
        oracle_matmul_f16(out, x, (const uint16_t*)w + off, n, d);
    else
        oracle_matmul(out, x, w + off, n, d);
}

/* ops.cpp:20-32 */
void oracle_rmsnorm(float* out, const float* x, const float* weight, int n) {
    float ss = 0.0f;
    for (int i = 0; i < n; i++) ss += x[i] * x[i];
    ss /= n;
    ss += 1e-5f;
    ss = 1.0f / sqrtf(ss);
    for (int i = 0; i < n; i++) out[i] = x[i] * ss * weight[i];
}

/* ops.cpp:34-54 -- adjacent pairs (i, i+1); k rotated only for i < kv_dim. */
void oracle_rope(float* q, float* k, int pos, int dim, int kv_dim, int head_size, float rope_base) {
    for (int i = 0; i < dim; i += 2) {
        int head_dim = i % head_size;
        float freq = 1.0f / powf(rope_base, head_dim / (float)head_size);
        float val = pos * freq;
        float fcos = cosf(val);
        float fsin = sinf(val);
        float q0 = q[i], q1 = q[i + 1];
        q[i] = q0 * fcos - q1 * fsin;
        q[i + 1] = q0 * fsin + q1 * fcos;
        if (i < kv_dim) {
            float k0 = k[i], k1 = k[i + 1];
            k[i] = k0 * fcos - k1 * fsin;
            k[i + 1] = k0 * fsin + k1 * fcos;
        }
    }
}

/* The (cos, sin) pair rope() uses for pair index j = head_dim/2 at position pos (ops.cpp:36-40). */
void oracle_rope_cos_sin(int pos, int j, int head_size, float rope_base, float* c, float* s) {
    int head_dim = 2 * j;
    float freq = 1.0f / powf(rope_base, head_dim / (float)head_size);
    float val = pos * freq;
    *c = cosf(val);
    *s = sinf(val);
}

/* ops.cpp:56-75 */
void oracle_softmax(float* x, int size) {
    float max_val = x[0];
    for (int i = 1; i < size; i++)
        if (x[i] > max_val) max_val = x[i];
    float sum = 0.0f;
    for (int i = 0; i < size; i++) {
        x[i] = expf(x[i] - max_val);
        sum += x[i];
    }
    for (int i = 0; i < size; i++) x[i] = x[i] / sum;
}

/* ops.cpp:78-87 */
void oracle_swiglu(float* hb, const float* h1, const float* h3, int size) {
    for (int i = 0; i < size; i++) {
        float val = h1[i];
        float sig = 1.0f / (1.0f + expf(-val));
        hb[i] = (val * sig) * h3[i];
    }
}

/* The KV-cache element offset the reference writes k/v element `off` of kv head `h` at `pos` to:
 * model.cpp:173 (CPU) == scatter_kv.cu:15-16 (GPU). */
int64_t oracle_kv_index(int layer, int h, int pos, int off, int n_kv_heads, int head_size, int seq_len) {
    int64_t kv_dim = (int64_t)n_kv_heads * head_size;
    return (int64_t)layer * (kv_dim * seq_len) + (int64_t)h * ((int64_t)seq_len * head_size) +
           (int64_t)pos * head_size + off;
}

/* model.cpp:18-51 (host half) */
oracle_model* oracle_create(int dim, int hidden_dim, int n_layers, int n_heads, int n_kv_heads, int vocab_size,
                            int seq_len, float rope_base, const float* tok_emb, const float* rms_att,
                            const float* wq, const float* wk, const float* wv, const float* wo,
                            const float* rms_ffn, const float* w1, const float* w2, const float* w3,
                            const float* rms_final, const float* w_cls) {
    oracle_model* m = (oracle_model*)calloc(1, sizeof(oracle_model));
    m->dim = dim;
    m->hidden_dim = hidden_dim;
    m->n_layers = n_layers;
    m->n_heads = n_heads;
    m->n_kv_heads = n_kv_heads;
    m->vocab_size = vocab_size;
    m->seq_len = seq_len;
    m->rope_base = rope_base;
    m->tok_emb = tok_emb;
    m->rms_att = rms_att;
    m->wq = wq;
    m->wk = wk;
    m->wv = wv;
    m->wo = wo;
    m->rms_ffn = rms_ffn;
    m->w1 = w1;
    m->w2 = w2;
    m->w3 = w3;
    m->rms_final = rms_final;
    m->w_cls = w_cls ? w_cls : tok_emb;
    m->w_f16 = 0;
    int kv_dim = (dim * n_kv_heads) / n_heads;
    m->x = (float*)calloc(dim, sizeof(float));
    m->xb = (float*)calloc(dim, sizeof(float));
    m->xb2 = (float*)calloc(dim, sizeof(float));
    m->q = (float*)calloc(dim, sizeof(float));
    m->k = (float*)calloc(kv_dim, sizeof(float));
    m->v = (float*)calloc(kv_dim, sizeof(float));
    m->hb = (float*)calloc(hidden_dim, sizeof(float));
    m->he = (float*)calloc(hidden_dim, sizeof(float));
    m->att = (float*)calloc((size_t)n_heads * seq_len, sizeof(float));
    m->logits = (float*)calloc(vocab_size, sizeof(float));
    size_t kv = (size_t)n_layers * seq_len * kv_dim;
    m->key_cache = (float*)calloc(kv, sizeof(float));
    m->value_cache = (float*)calloc(kv, sizeof(float));
    return m;
}

/* The same model over binary16 matrices / embedding (norm weights stay FP32). */
oracle_model* oracle_create_f16(int dim, int hidden_dim, int n_layers, int n_heads, int n_kv_heads, int vocab_size,
                                int seq_len, float rope_base, const uint16_t* tok_emb, const float* rms_att,
                                const uint16_t* wq, const uint16_t* wk, const uint16_t* wv, const uint16_t* wo,
                                const float* rms_ffn, const uint16_t* w1, const uint16_t* w2, const uint16_t* w3,
                                const float* rms_final, const uint16_t* w_cls) {
    oracle_model* m = oracle_create(dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, rope_base,
                                    (const float*)tok_emb, rms_att, (const float*)wq, (const float*)wk,
                                    (const float*)wv, (const float*)wo, rms_ffn, (const float*)w1, (const float*)w2,
                                    (const float*)w3, rms_final, (const float*)w_cls);
    m->w_f16 = 1;
    return m;
}

void oracle_free(oracle_model* m) {
    if (!m) return;
    free(m->x);
    free(m->xb);
    free(m->xb2);
    free(m->q);
    free(m->k);
    free(m->v);
    free(m->hb);
    free(m->he);
    free(m->att);
    free(m->logits);
    free(m->key_cache);
    free(m->value_cache);
    free(m);
}

float* oracle_key_cache(oracle_model* m) { return m->key_cache; }
float* oracle_value_cache(oracle_model* m) { return m->value_cache; }
float* oracle_q(oracle_model* m) { return m->q; }
float* oracle_x(oracle_model* m) { return m->x; }
float* oracle_xb(oracle_model* m) { return m->xb; }

/* model.cpp:163-201 (CPU attention path) */
void oracle_attention(oracle_model* m, int layer, int pos) {
    int dim = m->dim;
    int kv_dim = (m->dim * m->n_kv_heads) / m->n_heads;
    int head_size = dim / m->n_heads;
    size_t off_q = (size_t)layer * dim * dim;
    size_t off_kv = (size_t)layer * kv_dim * dim;
    int gqa = m->n_heads / m->n_kv_heads;
    int cache_stride = m->seq_len * head_size;

    model_matmul(m, m->q, m->xb, m->wq, off_q, dim, dim);
    model_matmul(m, m->k, m->xb, m->wk, off_kv, kv_dim, dim);
    model_matmul(m, m->v, m->xb, m->wv, off_kv, kv_dim, dim);
    oracle_rope(m->q, m->k, pos, dim, kv_dim, head_size, m->rope_base);

    for (int h = 0; h < m->n_kv_heads; h++) {
        size_t dst = (size_t)layer * ((size_t)kv_dim * m->seq_len) + (size_t)h * cache_stride +
                     (size_t)pos * head_size;
        memcpy(m->key_cache + dst, m->k + h * head_size, head_size * sizeof(float));
        memcpy(m->value_cache + dst, m->v + h * head_size, head_size * sizeof(float));
    }

    float scale = 1.0f / sqrtf(head_size);
#pragma omp parallel for schedule(static) if (pos > 256)
    for (int h = 0; h < m->n_heads; h++) {
        float* qh = m->q + h * head_size;
        int kvh = h / gqa;
        size_t ho = (size_t)layer * ((size_t)kv_dim * m->seq_len) + (size_t)kvh * cache_stride;
        const float* kc = m->key_cache + ho;
        const float* vc = m->value_cache + ho;
        float* att = m->att + (size_t)h * m->seq_len;
        for (int t = 0; t <= pos; t++) { /* naive_matmul(att, q_head, k_cache_head, pos+1, head_size) */
            float val = 0.0f;
            const float* kr = kc + (size_t)t * head_size;
            for (int i = 0; i < head_size; i++) val += qh[i] * kr[i];
            att[t] = val;
        }
        for (int t = 0; t <= pos; t++) att[t] *= scale;
        oracle_softmax(att, pos + 1);
        float* xbh = m->xb + h * head_size;
        memset(xbh, 0, head_size * sizeof(float));
        for (int t = 0; t <= pos; t++) {
            float score = att[t];
            const float* vr = vc + (size_t)t * head_size;
            for (int i = 0; i < head_size; i++) xbh[i] += vr[i] * score;
        }
    }
    model_matmul(m, m->xb2, m->xb, m->wo, off_q, dim, dim);
}

/* model.cpp:229-239 (CPU transformer_block path) */
void oracle_transformer_block(oracle_model* m, int layer, int pos) {
    int dim = m->dim, hidden = m->hidden_dim;
    size_t off_ffn = (size_t)layer * hidden * dim;
    size_t off_norm = (size_t)layer * dim;
    oracle_rmsnorm(m->xb, m->x, m->rms_att + off_norm, dim);
    oracle_attention(m, layer, pos);
    for (int i = 0; i < dim; i++) m->x[i] += m->xb2[i];
    oracle_rmsnorm(m->xb, m->x, m->rms_ffn + off_norm, dim);
    model_matmul(m, m->hb, m->xb, m->w1, off_ffn, hidden, dim);
    model_matmul(m, m->he, m->xb, m->w3, off_ffn, hidden, dim);
    oracle_swiglu(m->hb, m->hb, m->he, hidden);
    model_matmul(m, m->xb2, m->hb, m->w2, off_ffn, dim, hidden);
    for (int i = 0; i < dim; i++) m->x[i] += m->xb2[i];
}

/* model.cpp:373-380: everything of forward() before sample(); logits copied out if asked. */
void oracle_step_logits(oracle_model* m, int token, int pos, float* logits_out) {
    int dim = m->dim;
    if (m->w_f16) {
        const uint16_t* row = (const uint16_t*)m->tok_emb + (size_t)token * dim;
        for (int i = 0; i < dim; i++) m->x[i] = half_bits_to_float(row[i]);
    } else {
        memcpy(m->x, m->tok_emb + (size_t)token * dim, dim * sizeof(float));
    }
    for (int l = 0; l < m->n_layers; l++) oracle_transformer_block(m, l, pos);
    oracle_rmsnorm(m->x, m->x, m->rms_final, dim);
    model_matmul(m, m->logits, m->x, m->w_cls, 0, m->vocab_size, dim);
    if (logits_out) memcpy(logits_out, m->logits, (size_t)m->vocab_size * sizeof(float));
}

/* model.cpp:256-303 with the random number passed in instead of drawn from rand()
 * (r = (float)rand()/(float)RAND_MAX at model.cpp:292), plain categorical branch only
 * (topp<=0 || topp>=1, model.cpp:294-303).  Mutates logits like the reference does. */
int oracle_sample(float* logits, int vocab_size, float temperature, float penalty, const int* history,
                  int history_len, float r) {
    if (penalty > 1.0f && history && history_len > 0) {
        for (int i = 0; i < history_len; i++) {
            int token = history[i];
            if (token >= 0 && token < vocab_size) {
                if (logits[token] > 0)
                    logits[token] /= penalty;
                else
                    logits[token] *= penalty;
            }
        }
    }
    if (temperature == 0.0f) {
        int max_idx = 0;
        float max_val = logits[0];
        for (int i = 1; i < vocab_size; i++) {
            if (logits[i] > max_val) {
                max_val = logits[i];
                max_idx = i;
            }
        }
        return max_idx;
    }
    for (int i = 0; i < vocab_size; i++) logits[i] /= temperature;
    oracle_softmax(logits, vocab_size);
    float cumulative = 0.0f;
    for (int i = 0; i < vocab_size; i++) {
        cumulative += logits[i];
        if (r < cumulative) return i;
    }
    return vocab_size - 1;
}

/* The reference's random stream: libc srand()/rand() (main.cpp:38, model.cpp:292). */
void oracle_srand(unsigned seed) { srand(seed); }
void oracle_rand_floats(float* out, int n) {
    for (int i = 0; i < n; i++) out[i] = (float)rand() / (float)RAND_MAX;
}

/* ---- CPU twin of the CUDA sampler's arithmetic (lighterpp_b200/csrc/common.cuh: exp_repro).
 * Same operations in the same order, IEEE double add/mul/fma only, so host and device agree bit for
 * bit.  Used to tell apart the two reasons a sampled id can differ from sample(): the summation
 * order of the kernel, and the last-bit difference between this exp and libm's expf. */
float oracle_exp_repro(float x) {
    if (!(x > -104.0f)) return (x != x) ? x : 0.0f;
    if (x > 88.8f) return INFINITY;
    const double kLog2e = 1.4426950408889634074;
    const double kLn2Hi = 6.93147180369123816490e-01;
    const double kLn2Lo = 1.90821492927058770002e-10;
    double xd = (double)x;
    double kd = rint(xd * kLog2e);
    double r = fma(-kd, kLn2Hi, xd);
    r = fma(-kd, kLn2Lo, r);
    double p = 1.0 / 6227020800.0;
    p = fma(p, r, 1.0 / 479001600.0);
    p = fma(p, r, 1.0 / 39916800.0);
    p = fma(p, r, 1.0 / 3628800.0);
    p = fma(p, r, 1.0 / 362880.0);
    p = fma(p, r, 1.0 / 40320.0);
    p = fma(p, r, 1.0 / 5040.0);
    p = fma(p, r, 1.0 / 720.0);
    p = fma(p, r, 1.0 / 120.0);
    p = fma(p, r, 1.0 / 24.0);
    p = fma(p, r, 1.0 / 6.0);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    long long k = (long long)kd;
    union {
        long long i;
        double d;
    } s;
    s.i = (k + 1023) << 52;
    return (float)(p * s.d);
}

/* sample() (src/model.cpp:256-303) with exp_repro in place of libm's expf and nothing else changed:
 * the sequential FP32 sums of softmax() and of the cumulative distribution are kept. */
int oracle_sample_exp_repro(float* logits, int vocab_size, float temperature, float penalty, const int* history,
                            int history_len, float r) {
    if (penalty > 1.0f && history && history_len > 0) {
        for (int i = 0; i < history_len; i++) {
            int token = history[i];
            if (token >= 0 && token < vocab_size) {
                if (logits[token] > 0)
                    logits[token] /= penalty;
                else
                    logits[token] *= penalty;
            }
        }
    }
    if (temperature == 0.0f) {
        int max_idx = 0;
        float max_val = logits[0];
        for (int i = 1; i < vocab_size; i++)
            if (logits[i] > max_val) {
                max_val = logits[i];
                max_idx = i;
            }
        return max_idx;
    }
    for (int i = 0; i < vocab_size; i++) logits[i] /= temperature;
    float max_val = logits[0];
    for (int i = 1; i < vocab_size; i++)
        if (logits[i] > max_val) max_val = logits[i];
    float sum = 0.0f;
    for (int i = 0; i < vocab_size; i++) {
        logits[i] = oracle_exp_repro(logits[i] - max_val);
        sum += logits[i];
    }
    for (int i = 0; i < vocab_size; i++) logits[i] = logits[i] / sum;
    float cumulative = 0.0f;
    for (int i = 0; i < vocab_size; i++) {
        cumulative += logits[i];
        if (r < cumulative) return i;
    }
    return vocab_size - 1;
}
