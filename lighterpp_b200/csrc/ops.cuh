// Standalone operator kernels behind the reference's per-op host wrappers (src/kernels.cuh:24-36).
// The decode step itself does not launch these -- it uses the fused kernels in gemv.cuh,
// attention.cuh and sampler.cuh -- but host code that calls the operators one by one (the
// reference's own runtests.cpp, or a partially ported model.cpp) gets the same results from them.
// All are element-wise or small reductions over L2-resident activations.
#pragma once
#include "common.cuh"

namespace lpp {

// src/matmul.cu:150-161
static __global__ void convert_f32_to_f16_kernel(__half* dst, const float* src, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long k = i; k < n; k += stride) dst[k] = __float2half_rn(src[k]);
}
static __global__ void convert_f16_to_f32_kernel(float* dst, const __half* src, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long k = i; k < n; k += stride) dst[k] = __half2float(src[k]);
}

// Strided 2-D repack with optional dtype conversion: dst[r*dst_pitch + c] = src[r*src_pitch + c]
// (pitches in elements).  Used to build the engine's fused weight layout from reference-layout
// tensors (row slices, column slices, gate/up interleave).
template <typename DT, typename ST>
static __global__ void repack_kernel(DT* dst, long long dst_pitch, const ST* src, long long src_pitch, int rows,
                              int cols) {
    const long long total = (long long)rows * cols;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < total; k += stride) {
        const long long r = k / cols, c = k % cols;
        const ST v = src[r * src_pitch + c];
        DT o;
        if constexpr (sizeof(DT) == 2 && sizeof(ST) == 4)
            o = __float2half_rn(v);
        else if constexpr (sizeof(DT) == 4 && sizeof(ST) == 2)
            o = __half2float(v);
        else
            o = v;
        dst[r * dst_pitch + c] = o;
    }
}

// src/RMSNorm.cu:11-71 -- one CTA; out = x * rsqrt(mean(x^2) + 1e-5) * w (src/ops.cpp:20-32)
static __global__ void __launch_bounds__(256) rmsnorm_kernel(float* out, const float* x, const float* w, int n) {
    __shared__ float red[8];
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += red[k];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)n), 1e-5f)));
    for (int i = threadIdx.x; i < n; i += 256) out[i] = __fmul_rn(__fmul_rn(x[i], scale), w[i]);
}

// (cos, sin) of pos / base^((2j)/hs) with the device's accurate powf/cosf/sinf.  The step path uses
// a host-built table instead (bit-identical to libm); this is for the stand-alone wrapper only.
__device__ __forceinline__ float2 rope_cos_sin(int pos, int j, int head_size, float rope_base) {
    const float freq = __fdiv_rn(1.0f, powf(rope_base, (float)(2 * j) / (float)head_size));
    const float val = (float)pos * freq;
    return make_float2(cosf(val), sinf(val));
}

// src/rope.cu:7-38 (in place, adjacent pairs, k rotated for i < kv_dim)
static __global__ void rope_kernel(float* q, float* k, int pos, int dim, int kv_dim, int head_size, float rope_base) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = 2 * p;
    if (i >= dim) return;
    const float2 cs = rope_cos_sin(pos, (i % head_size) >> 1, head_size, rope_base);
    const float q0 = q[i], q1 = q[i + 1];
    q[i] = __fsub_rn(__fmul_rn(q0, cs.x), __fmul_rn(q1, cs.y));
    q[i + 1] = __fadd_rn(__fmul_rn(q0, cs.y), __fmul_rn(q1, cs.x));
    if (i < kv_dim) {
        const float k0 = k[i], k1 = k[i + 1];
        k[i] = __fsub_rn(__fmul_rn(k0, cs.x), __fmul_rn(k1, cs.y));
        k[i + 1] = __fadd_rn(__fmul_rn(k0, cs.y), __fmul_rn(k1, cs.x));
    }
}

// src/scatter_kv.cu:6-26
static __global__ void scatter_kv_kernel(__half* kc, __half* vc, const float* k, const float* v, int layer, int pos,
                                  int n_kv_heads, int head_size, int seq_len) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int kv_dim = n_kv_heads * head_size;
    if (i >= kv_dim) return;
    const int h = i / head_size, off = i % head_size;
    const size_t idx = (size_t)layer * ((size_t)kv_dim * seq_len) + (size_t)h * ((size_t)seq_len * head_size) +
                       (size_t)pos * head_size + off;
    kc[idx] = __float2half_rn(k[i]);
    vc[idx] = __float2half_rn(v[i]);
}

// rope + scatter in one launch: q rotated in place; k rotated and written with v to the FP16 cache.
static __global__ void rope_scatter_kernel(float* q, const float* k, const float* v, __half* kc, __half* vc, int layer,
                                    int pos, int dim, int n_kv_heads, int head_size, int seq_len,
                                    float rope_base) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = 2 * p;
    if (i >= dim) return;
    const int kv_dim = n_kv_heads * head_size;
    const float2 cs = rope_cos_sin(pos, (i % head_size) >> 1, head_size, rope_base);
    const float q0 = q[i], q1 = q[i + 1];
    q[i] = __fsub_rn(__fmul_rn(q0, cs.x), __fmul_rn(q1, cs.y));
    q[i + 1] = __fadd_rn(__fmul_rn(q0, cs.y), __fmul_rn(q1, cs.x));
    if (i < kv_dim) {
        const float k0 = k[i], k1 = k[i + 1];
        const float r0 = __fsub_rn(__fmul_rn(k0, cs.x), __fmul_rn(k1, cs.y));
        const float r1 = __fadd_rn(__fmul_rn(k0, cs.y), __fmul_rn(k1, cs.x));
        const int h = i / head_size, off = i % head_size;
        const size_t idx = (size_t)layer * ((size_t)kv_dim * seq_len) +
                           (size_t)h * ((size_t)seq_len * head_size) + (size_t)pos * head_size + off;
        *reinterpret_cast<__half2*>(kc + idx) = __floats2half2_rn(r0, r1);
        *reinterpret_cast<__half2*>(vc + idx) = __floats2half2_rn(v[i], v[i + 1]);
    }
}

// src/swiglu.cu:6-33
static __global__ void swiglu_kernel(float* hb, const float* h1, const float* h3, int size) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= size) return;
    const float val = h1[i];
    const float sig = __fdiv_rn(1.0f, 1.0f + expf(-val));
    hb[i] = __fmul_rn(__fmul_rn(val, sig), h3[i]);
}

// src/residual.cu:5-31
static __global__ void residual_add_kernel(float* out, const float* a, const float* b, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

// src/scale.cu:6-21
static __global__ void scale_multihead_kernel(float* att, float scale, int seq_len, int att_stride) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < seq_len) att[(size_t)blockIdx.y * att_stride + t] *= scale;
}

// src/softmax.cu:5-125 -- one CTA per head, max / exp / sum / divide (src/ops.cpp:56-75)
static __global__ void __launch_bounds__(256) softmax_multihead_kernel(float* out, const float* x, int seq_len,
                                                                int att_stride) {
    __shared__ float red[8];
    const float* xi = x + (size_t)blockIdx.x * att_stride;
    float* oi = out + (size_t)blockIdx.x * att_stride;
    float m = -INFINITY;
    for (int t = threadIdx.x; t < seq_len; t += 256) m = fmaxf(m, xi[t]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int k = 1; k < 8; ++k) m = fmaxf(m, red[k]);
    __syncthreads();
    float s = 0.f;
    for (int t = threadIdx.x; t < seq_len; t += 256) {
        const float e = expf(xi[t] - m);
        oi[t] = e;
        s += e;
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += red[k];
    for (int t = threadIdx.x; t < seq_len; t += 256) oi[t] = __fdiv_rn(oi[t], tot);
}

// src/multihead_gemv.cu:6-68 -- att[h][t] = q_h . K[kv(h)][t] (unscaled), one warp per (h, t)
static __global__ void __launch_bounds__(128) multihead_gemv_kernel(float* att, const float* q, const __half* kc,
                                                             int layer, int pos, int n_heads, int n_kv_heads,
                                                             int head_size, int seq_len) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp, h = blockIdx.y;
    if (t > pos) return;
    const int kvh = h / (n_heads / n_kv_heads);
    const __half* kr = kc + (size_t)layer * ((size_t)n_kv_heads * head_size * seq_len) +
                       (size_t)kvh * ((size_t)seq_len * head_size) + (size_t)t * head_size;
    const float* qh = q + (size_t)h * head_size;
    float s = 0.f;
    for (int d = lane; d < head_size; d += 32) s = fmaf(qh[d], __half2float(kr[d]), s);
    s = warp_sum(s);
    if (lane == 0) att[(size_t)h * seq_len + t] = s;
}

// src/aggregation.cu:6-31 -- out[h][i] = sum_t V[kv(h)][t][i] * att[h][t]; V points at the layer
static __global__ void __launch_bounds__(128) aggregation_multihead_kernel(float* out, const __half* v,
                                                                    const float* att, int seq_len,
                                                                    int head_size, int gqa_factor,
                                                                    int att_stride) {
    // 4 warps split the positions, lanes split the head dimension; fixed-order merge
    __shared__ float part[4][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, kvh = h / gqa_factor;
    // cache stride per kv head is att_stride (= allocated seq_len) rows, as in the reference call
    const __half* vb = v + (size_t)kvh * ((size_t)att_stride * head_size);
    const float* ah = att + (size_t)h * att_stride;
    for (int d0 = 0; d0 < head_size; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.f;
        if (d < head_size)
            for (int t = warp; t < seq_len; t += 4) acc = fmaf(__half2float(vb[(size_t)t * head_size + d]), ah[t], acc);
        if (d < 128) part[warp][d] = acc;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < head_size; d += 128)
        out[(size_t)h * head_size + d] = part[0][d] + part[1][d] + part[2][d] + part[3][d];
}

}  // namespace lpp
