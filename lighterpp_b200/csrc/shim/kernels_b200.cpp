// The reference's per-operator host wrappers (src/kernels.cuh:24-36) re-created on top of the C ABI
// of liblpp_b200.so, with the reference's exact C++ signatures, so that reference host code built
// with -DUSE_CUDA (model.cpp callers, loader.cpp, runtests.cpp) links against this library instead
// of the reference's eleven .cu files.  Errors keep the reference convention: print and exit(1)
// (src/kernels.cuh:14-21); the C ABI underneath never exits.
#include <cstdio>
#include <cstdlib>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "lpp_b200.h"

enum WeightPrecision : int;  // src/model.h:8-12 (0 = FP32, 1 = FP16: same values as lpp_dtype)

static void must(lpp_status s, const char* what) {
    if (s != LPP_OK) {
        printf("Error: %s: %s (%s)\n", what, lpp_strerror(s), lpp_last_error());
        exit(1);
    }
}

void cuda_convert_f32_to_f16(void* dst, float* src, int n) {
    must(lpp_op_convert_f32_to_f16(dst, src, n, nullptr), "cuda_convert_f32_to_f16");
}

void cuda_gemv(float* d_out, float* d_x, void* d_w, void* d_workspace, int n, int d, WeightPrecision precision) {
    (void)d_workspace;  // x is never rounded to FP16 here (the reference needs scratch for that, src/matmul.cu:136-141)
    must(lpp_op_gemv(d_out, d_x, d_w, n, d, (int)precision == 1 ? LPP_F16 : LPP_F32, nullptr), "cuda_gemv");
}

void cuda_rmsnorm(float* d_out, float* d_x, float* d_w, int n) { must(lpp_op_rmsnorm(d_out, d_x, d_w, n, nullptr), "cuda_rmsnorm"); }

void cuda_rope(float* d_q, float* d_k, int pos, int dim, int kv_dim, int head_size, float rope_base) {
    must(lpp_op_rope(d_q, d_k, pos, dim, kv_dim, head_size, rope_base, nullptr), "cuda_rope");
}

void cuda_swiglu(float* d_hb, float* d_h1, float* d_h3, int size) {
    must(lpp_op_swiglu(d_hb, d_h1, d_h3, size, nullptr), "cuda_swiglu");
}

void cuda_softmax_multihead(float* d_out, float* d_x, int n_heads, int seq_len, int att_stride) {
    must(lpp_op_softmax_multihead(d_out, d_x, n_heads, seq_len, att_stride, nullptr), "cuda_softmax_multihead");
}

void cuda_scale_multihead(float* d_att, float scale, int n_heads, int seq_len, int att_stride) {
    must(lpp_op_scale_multihead(d_att, scale, n_heads, seq_len, att_stride, nullptr), "cuda_scale_multihead");
}

void cuda_aggregation_multihead(float* d_out, const __half* d_v, const float* d_att, int n_heads, int seq_len,
                                int head_size, int gqa_factor, int att_stride) {
    must(lpp_op_aggregation_multihead(d_out, d_v, d_att, n_heads, seq_len, head_size, gqa_factor, att_stride, nullptr),
         "cuda_aggregation_multihead");
}

void cuda_residual_add(float* d_out, const float* d_a, const float* d_b, int n) {
    must(lpp_op_residual_add(d_out, d_a, d_b, n, nullptr), "cuda_residual_add");
}

void cuda_scatter_kv(__half* d_key_cache, __half* d_value_cache, const float* d_k, const float* d_v, int layer, int pos,
                     int n_kv_heads, int head_size, int seq_len) {
    must(lpp_op_scatter_kv(d_key_cache, d_value_cache, d_k, d_v, layer, pos, n_kv_heads, head_size, seq_len, nullptr),
         "cuda_scatter_kv");
}

void cuda_multihead_gemv(float* d_out, float* d_q, __half* d_k_cache, int layer, int pos, int n_heads, int n_kv_heads,
                         int head_size, int seq_len) {
    must(lpp_op_multihead_gemv(d_out, d_q, d_k_cache, layer, pos, n_heads, n_kv_heads, head_size, seq_len, nullptr),
         "cuda_multihead_gemv");
}

void cuda_sample(float* d_logits, int vocab_size, float temperature, float topp, float penalty, int* d_history,
                 int history_len, int* d_sampled_token, unsigned int* d_rng_state) {
    (void)topp;         // ignored by the reference kernel too (src/sample.cu:6)
    (void)d_rng_state;  // unused in the reference (nullptr at src/model.cpp:366)
    // the reference draws at every call, also at temperature 0 (src/sample.cu:211): keep its rand() stream
    const float r = (float)rand() / (float)RAND_MAX;
    must(lpp_op_sample(d_logits, vocab_size, temperature, penalty, d_history, history_len, r, d_sampled_token, nullptr),
         "cuda_sample");
}
