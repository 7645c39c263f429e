// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C-ABI harness around the UNMODIFIED Lighter++ reference CPU build.  This file is
// compiled together with the reference's own src/{model,ops,loader,gguf,tensor,
// tokenizer}.cpp (taken from where the reference checkout lies, never copied) into
// oracle/_ref/libref_cpu.so by oracle/Makefile.  It only *calls* reference functions:
//   forward body      model.cpp:372-380   (memcpy embedding, transformer_block per layer,
//                                           final RMSNorm, classifier matmul)
//   sample            model.cpp:256-340   (7-argument definition; model.h:148 declares 4)
//   loaders           loader.cpp:134-172 (.bin), loader.cpp:213-334 + 425-641 (GGUF)
//   primitive ops     ops.cpp:9-87
// Logits are copied out BEFORE sample() because sample() mutates them in place
// (model.cpp:259-290).
//
// Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may
// load the library built from this file.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <fcntl.h>
#include <unistd.h>

#include "model.h"
#include "ops.h"
#include "loader.h"
#include "gguf.h"

// model.cpp:256 defines this 7-argument form; the header only declares a 4-argument one.
int sample(float* logits, int vocab_size, float temperature, float topp, float penalty, int* history,
           int history_len);

struct ref_model {
    Config cfg;
    transformerWeights w;
    RunState s;
    bool state_ready;
    // ownership bookkeeping
    GGUFFile* gguf;
    float* bin_data;
    size_t bin_size;
    bool weights_owned_by_loader;  // gguf_init_weights malloc()s the FP32 stacks
};

static void silence_stdout(int* saved) {
    fflush(stdout);
    *saved = dup(1);
    int devnull = open("/dev/null", O_WRONLY);
    dup2(devnull, 1);
    close(devnull);
}
static void restore_stdout(int saved) {
    fflush(stdout);
    dup2(saved, 1);
    close(saved);
}

extern "C" {

// ---- model lifetime -------------------------------------------------------------------

// Load a llama2.c .bin or GGUF file with the reference's own loaders.  seq_len_override>0
// replaces Config.seq_len after config extraction (the GGUF path clamps to 16384,
// loader.cpp:328-331) and before malloc_run_state.
ref_model* ref_load(const char* path, int seq_len_override) {
    ref_model* m = (ref_model*)calloc(1, sizeof(ref_model));
    int saved;
    silence_stdout(&saved);
    bool ok = true;
    if (is_gguf_file(path)) {
        m->gguf = gguf_open(path);
        ok = m->gguf && gguf_extract_config(m->gguf, &m->cfg);
        if (ok) ok = gguf_init_weights(m->gguf, &m->w, &m->cfg);
        m->weights_owned_by_loader = true;
    } else {
        m->bin_data = load_model_file(path, &m->cfg, &m->bin_size);
        ok = m->bin_data != nullptr;
        if (ok) {
            m->cfg.weight_precision = WEIGHT_FP32;  // loader.cpp:158-159 copies 36 bytes of a 28-byte header
            checkpoint_init_weights(&m->w, &m->cfg, m->bin_data);
        }
    }
    if (ok) {
        if (seq_len_override > 0) m->cfg.seq_len = seq_len_override;
        malloc_run_state(&m->s, &m->cfg);
        m->state_ready = true;
    }
    restore_stdout(saved);
    if (!ok) {
        free(m);
        return nullptr;
    }
    return m;
}

// Build a model around caller-owned FP32 arrays laid out exactly as transformerWeights
// expects (model.h:34-53; per-layer tensors stacked [L][rows][cols]).  w_cls may be NULL
// for tied embeddings (loader.cpp:66, 471).
ref_model* ref_create(int dim, int hidden_dim, int n_layers, int n_heads, int n_kv_heads, int vocab_size,
                      int seq_len, float rope_base, float* tok_emb, float* rms_att, float* wq, float* wk,
                      float* wv, float* wo, float* rms_ffn, float* w1, float* w2, float* w3,
                      float* rms_final, float* w_cls) {
    ref_model* m = (ref_model*)calloc(1, sizeof(ref_model));
    m->cfg.dim = dim;
    m->cfg.hidden_dim = hidden_dim;
    m->cfg.n_layers = n_layers;
    m->cfg.n_heads = n_heads;
    m->cfg.n_kv_heads = n_kv_heads;
    m->cfg.vocab_size = vocab_size;
    m->cfg.seq_len = seq_len;
    m->cfg.rope_base = rope_base;
    m->cfg.weight_precision = WEIGHT_FP32;
    m->w.token_embedding_table = tok_emb;
    m->w.rms_att_weight = rms_att;
    m->w.wq = wq;
    m->w.wk = wk;
    m->w.wv = wv;
    m->w.wo = wo;
    m->w.rms_ffn_weight = rms_ffn;
    m->w.w1 = w1;
    m->w.w2 = w2;
    m->w.w3 = w3;
    m->w.rms_final_weight = rms_final;
    m->w.w_cls = w_cls ? w_cls : tok_emb;
    malloc_run_state(&m->s, &m->cfg);
    m->state_ready = true;
    return m;
}

void ref_free(ref_model* m) {
    if (!m) return;
    if (m->state_ready) free_run_state(&m->s);
    if (m->gguf) {
        if (m->w.w_cls != m->w.token_embedding_table) free(m->w.w_cls);
        free(m->w.token_embedding_table);
        free(m->w.rms_att_weight);
        free(m->w.wq);
        free(m->w.wk);
        free(m->w.wv);
        free(m->w.wo);
        free(m->w.rms_ffn_weight);
        free(m->w.w1);
        free(m->w.w2);
        free(m->w.w3);
        free(m->w.rms_final_weight);
        gguf_close(m->gguf);
    }
    if (m->bin_data) free_model_file(m->bin_data, m->bin_size);
    free(m);
}

// out[0..8] = dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, weight_precision
// rope_base returned separately.
void ref_get_config(ref_model* m, int* out8, float* rope_base) {
    out8[0] = m->cfg.dim;
    out8[1] = m->cfg.hidden_dim;
    out8[2] = m->cfg.n_layers;
    out8[3] = m->cfg.n_heads;
    out8[4] = m->cfg.n_kv_heads;
    out8[5] = m->cfg.vocab_size;
    out8[6] = m->cfg.seq_len;
    out8[7] = (int)m->cfg.weight_precision;
    *rope_base = m->cfg.rope_base;
}

// ---- the decode step -------------------------------------------------------------------

// forward()'s CPU body (model.cpp:373-380) without the trailing sample(): fills s.logits and
// copies them to logits_out (vocab_size floats) if non-NULL.
void ref_step_logits(ref_model* m, int token, int pos, float* logits_out) {
    Config* p = &m->cfg;
    int dim = p->dim;
    float* row = m->w.token_embedding_table + (size_t)token * dim;
    memcpy(m->s.x, row, dim * sizeof(float));
    for (int layer = 0; layer < p->n_layers; layer++) transformer_block(&m->s, &m->w, p, layer, pos);
    RMSNorm(m->s.x, m->s.x, m->w.rms_final_weight, dim);
    naive_matmul(m->s.logits, m->s.x, m->w.w_cls, p->vocab_size, dim);
    if (logits_out) memcpy(logits_out, m->s.logits, (size_t)p->vocab_size * sizeof(float));
}

// The reference entry point itself (model.cpp:342-384), rand() state as left by ref_srand.
int ref_forward(ref_model* m, int token, int pos, float temperature, float topp, float penalty, int* history,
                int history_len) {
    return forward(token, pos, &m->s, &m->w, &m->cfg, temperature, topp, penalty, history, history_len);
}

void ref_srand(unsigned seed) { srand(seed); }
// The value sample() will draw next is (float)rand()/(float)RAND_MAX (model.cpp:292); this
// peeks the stream by drawing n values, for feeding the same r to another implementation.
void ref_rand_floats(float* out, int n) {
    for (int i = 0; i < n; i++) out[i] = (float)rand() / (float)RAND_MAX;
}

// sample() on a caller buffer (mutated in place exactly as the reference does).  r comes from the
// process-global rand() stream like in the reference; call ref_srand first to fix it.
int ref_sample(float* logits, int vocab_size, float temperature, float topp, float penalty, int* history,
               int history_len) {
    return sample(logits, vocab_size, temperature, topp, penalty, history, history_len);
}

// ---- state inspection -------------------------------------------------------------------

float* ref_key_cache(ref_model* m) { return m->s.key_cache; }
float* ref_value_cache(ref_model* m) { return m->s.value_cache; }
float* ref_logits(ref_model* m) { return m->s.logits; }
float* ref_x(ref_model* m) { return m->s.x; }

// ---- primitive ops (ops.cpp) -------------------------------------------------------------

void ref_naive_matmul(float* out, float* x, float* w, int n, int d) { naive_matmul(out, x, w, n, d); }
void ref_rmsnorm(float* out, float* x, float* weight, int n) { RMSNorm(out, x, weight, n); }
void ref_rope(float* q, float* k, int pos, int dim, int kv_dim, int head_size, float rope_base) {
    rope(q, k, pos, dim, kv_dim, head_size, rope_base);
}
void ref_softmax(float* x, int size) { softmax(x, size); }
void ref_swiglu(float* hb, float* h1, float* h3, int size) { swiglu(hb, h1, h3, size); }
void ref_attention(ref_model* m, int layer, int pos) { attention(&m->s, &m->w, &m->cfg, layer, pos); }
void ref_transformer_block(ref_model* m, int layer, int pos) {
    transformer_block(&m->s, &m->w, &m->cfg, layer, pos);
}

// ---- timing helper for the CPU baseline -------------------------------------------------

// Runs n teacher-forced steps (tokens[i] at start_pos+i) through ref_step_logits + argmax
// sample, returns wall seconds.  Single-threaded like the reference (ops.cpp has no threading).
double ref_time_steps(ref_model* m, const int* tokens, int n, int start_pos, float temperature, float penalty,
                      int* history, int history_len) {
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < n; i++) {
        (void)forward(tokens[i], start_pos + i, &m->s, &m->w, &m->cfg, temperature, 1.0f, penalty, history,
                      history_len);
    }
    auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double>(t1 - t0).count();
}

}  // extern "C"
