// C-ABI entry points for the stand-alone operators: one per host wrapper of the reference's
// src/kernels.cuh:24-36, same argument meaning, device pointers in and out, nothing synchronised
// (like the reference wrappers, callers order work through the stream).
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stddef.h>

#include <algorithm>

#include "../../include/lpp_b200.h"
#include "common.cuh"
#include "gemv.cuh"
#include "ops.cuh"
#include "sampler.cuh"
#include "sampler_exact.cuh"

using namespace lpp;

namespace {

inline lpp_status chk() { return cudaGetLastError() == cudaSuccess ? LPP_OK : LPP_ERR_CUDA; }
inline cudaStream_t S(void* s) { return (cudaStream_t)s; }
inline int blocks(long long n, int t) { return (int)std::max<long long>(1, (n + t - 1) / t); }

// Any-shape fallback for the stand-alone GEMV: one warp per row, scalar loads.
template <typename WT>
__global__ void gemv_generic_kernel(float* out, const float* x, const WT* w, int n, int d) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n) return;
    const WT* r = w + (size_t)row * d;
    float acc = 0.f;
    for (int k = lane; k < d; k += 32) {
        float wv;
        if constexpr (sizeof(WT) == 2)
            wv = __half2float(r[k]);
        else
            wv = r[k];
        acc = fmaf(wv, x[k], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc;
}

// Status word for stand-alone GEMV launches (their bounded waits need somewhere to report).
__device__ StepState g_op_state;

template <typename WT>
lpp_status op_gemv_t(float* out, const float* x, const void* w, int n, int d, cudaStream_t s) {
    const int vec = 16 / (int)sizeof(WT);
    const size_t smem = 128 + (((size_t)d * 4 + 127) & ~(size_t)127);
    // the vector kernel stages x with 16-byte loads, reads the rows with 16-byte loads and stores row pairs
    // with 8-byte stores: anything else (an offset sub-vector, say) takes the scalar kernel
    if ((n & 1) || (d % vec) || (((uintptr_t)w) & 15) || (((uintptr_t)x) & 15) || (((uintptr_t)out) & 7) ||
        smem > 200 * 1024) {
        gemv_generic_kernel<WT><<<blocks(n, 8), 256, 0, s>>>(out, x, (const WT*)w, n, d);
        return chk();
    }
    StepState* st = nullptr;
    if (cudaGetSymbolAddress((void**)&st, g_op_state) != cudaSuccess) return LPP_ERR_CUDA;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(gemv_ldg_kernel<WT, kEpiStore>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
        return LPP_ERR_CUDA;
    GemvArgs a = {};
    a.W = w;
    a.n_rows = n;
    a.K = d;
    a.x = x;
    a.out = out;
    a.st = st;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = std::max(1, std::min(n / kRowsPerGroup, sms * 4));
    gemv_ldg_kernel<WT, kEpiStore><<<grid, kGemvLdgThreads, smem, s>>>(a);
    return chk();
}

// ---- scratch layout of the stand-alone samplers: step state, per-block partials, ticket counter and barrier
//      words, then what the exact-order kernel adds (block sums, entry counts, scalars, entry lists).
//      `cap_blocks` sizes the areas: the blocks of this call (stream-ordered scratch) or of the largest
//      vocabulary the fixed array takes.
struct SampleScratch {
    size_t state, part, counters, sums, counts, scalars, entries, total;
};
constexpr SampleScratch sample_scratch_layout(int cap_blocks, bool exact) {
    SampleScratch L = {};
    size_t o = 0;
    L.state = o;
    o += (sizeof(StepState) + 255) & ~(size_t)255;
    L.part = o;
    o += ((size_t)cap_blocks * 12 + 255) & ~(size_t)255;
    L.counters = o;  // [0] ticket counter of the tree kernel; from +256: barrier counter and exit ticket of the exact kernel
    o += 512;
    if (exact) {
        L.sums = o;
        o += ((size_t)cap_blocks * sizeof(double) + 255) & ~(size_t)255;
        L.counts = o;
        o += ((size_t)cap_blocks * sizeof(int) + 255) & ~(size_t)255;
        L.scalars = o;
        o += 256;
        L.entries = o;
        o += (size_t)cap_blocks * kExactMaxEntries * sizeof(ExactEntry);
    }
    L.total = o;
    return L;
}

// Launches the sampler on logits with its scratch at `scratch` (laid out by sample_scratch_layout for
// cap_blocks >= the blocks of this vocabulary).  The step state at the head of the scratch and the zeroed
// counters are the caller's business.  The exact-order kernel (ids equal to the reference's sequential CPU
// sample()) needs all its blocks co-resident; a vocabulary beyond that takes the tree-sum kernel.
void launch_sampler_on_scratch(char* scratch, const SampleScratch& L, bool exact, float* d_logits, int vocab_size,
                               int nb, cudaStream_t s) {
    SampleArgs a = {};
    a.logits = d_logits;
    a.vocab = vocab_size;
    a.st = (StepState*)(scratch + L.state);
    a.part_max = (float*)(scratch + L.part);
    a.part_idx = (int*)(scratch + L.part + (size_t)nb * 4);
    a.part_sum = (float*)(scratch + L.part + (size_t)nb * 8);
    a.counter = (unsigned int*)(scratch + L.counters);
    if (exact) {
        SampleExactArgs ea = {};
        ea.base = a;
        ea.sync = (unsigned int*)(scratch + L.counters + 256);
        ea.block_sum = (double*)(scratch + L.sums);
        ea.entry_count = (int*)(scratch + L.counts);
        ea.scalars = (float*)(scratch + L.scalars);
        ea.entries = (ExactEntry*)(scratch + L.entries);
        sample_exact_kernel<<<nb, kSampleThreads, 0, s>>>(ea);
    } else {
        sample_kernel<<<nb, kSampleThreads, 0, s>>>(a);
    }
}

// ---- scratch for lpp_op_sample_static: lives in the library image, one copy per GPU that loads it
constexpr int kStaticSampleMaxVocab = 262144;  // 128 blocks of kSampleChunk logits
constexpr int kStaticSampleBlocks = kStaticSampleMaxVocab / kSampleChunk;
constexpr SampleScratch kStaticLayout = sample_scratch_layout(kStaticSampleBlocks, true);
static __device__ __align__(256) unsigned char g_sample_scratch[kStaticLayout.total];
// Device addresses of g_sample_scratch, one per CUDA device, filled in on first use.  In host code
// the name g_sample_scratch is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static unsigned char* g_sample_scratch_addr[64];

// Writes the step-state header the sampler reads, copies the history device-to-device and zeroes
// the ticket counter -- everything in the shared scratch that must not survive from the last call.
static __global__ void sample_static_setup_kernel(StepState* st, unsigned int* counters, float temperature,
                                                  float penalty, float r, const int* history, int history_len) {
    if (threadIdx.x == 0) {
        st->token = 0;
        st->pos = 0;
        st->history_len = history_len;
        st->history_window = 0;
        st->history_count = 0;
        st->step_idx = 0;
        st->advance = 0;
        st->temperature = temperature;
        st->penalty = penalty;
        st->r = r;
        st->out_token = -1;
        st->status = 0;
        st->wait_cycles = 0;
        st->tp_wait_cycles = 0;
    }
    if (threadIdx.x < 128) counters[threadIdx.x] = 0u;  // ticket counter, barrier counter, exit ticket
    if (threadIdx.x == 0) {
    }
    for (int i = threadIdx.x; i < history_len; i += blockDim.x) st->history[i] = history[i];
}
static __global__ void sample_static_publish_kernel(const StepState* st, int* dst) { *dst = st->out_token; }

}  // namespace

void lpp_internal_set_error(const char* msg);  // engine.cu: text behind lpp_last_error()

extern "C" {

lpp_status lpp_op_convert_f32_to_f16(void* d_dst, const float* d_src, int64_t n, void* stream) {
    if (!d_dst || !d_src || n < 0) return LPP_ERR_INVALID_ARG;
    if (n == 0) return LPP_OK;
    convert_f32_to_f16_kernel<<<(int)std::min<long long>(blocks(n, 256), 148 * 16), 256, 0, S(stream)>>>(
        (__half*)d_dst, d_src, n);
    return chk();
}

lpp_status lpp_op_gemv(float* d_out, const float* d_x, const void* d_w, int n, int d, int w_dtype, void* stream) {
    if (!d_out || !d_x || !d_w || n <= 0 || d <= 0) return LPP_ERR_INVALID_ARG;
    if (w_dtype == LPP_F16) return op_gemv_t<__half>(d_out, d_x, d_w, n, d, S(stream));
    if (w_dtype == LPP_F32) return op_gemv_t<float>(d_out, d_x, d_w, n, d, S(stream));
    return LPP_ERR_INVALID_ARG;
}

lpp_status lpp_op_rmsnorm(float* d_out, const float* d_x, const float* d_w, int n, void* stream) {
    if (!d_out || !d_x || !d_w || n <= 0) return LPP_ERR_INVALID_ARG;
    rmsnorm_kernel<<<1, 256, 0, S(stream)>>>(d_out, d_x, d_w, n);
    return chk();
}

lpp_status lpp_op_rope(float* d_q, float* d_k, int pos, int dim, int kv_dim, int head_size, float rope_base,
                       void* stream) {
    if (!d_q || !d_k || dim <= 0 || (dim & 1) || head_size <= 0 || (head_size & 1)) return LPP_ERR_INVALID_ARG;
    rope_kernel<<<blocks(dim / 2, 256), 256, 0, S(stream)>>>(d_q, d_k, pos, dim, kv_dim, head_size, rope_base);
    return chk();
}

lpp_status lpp_op_swiglu(float* d_hb, const float* d_h1, const float* d_h3, int size, void* stream) {
    if (!d_hb || !d_h1 || !d_h3 || size <= 0) return LPP_ERR_INVALID_ARG;
    swiglu_kernel<<<blocks(size, 256), 256, 0, S(stream)>>>(d_hb, d_h1, d_h3, size);
    return chk();
}

lpp_status lpp_op_softmax_multihead(float* d_out, const float* d_x, int n_heads, int seq_len, int att_stride,
                                    void* stream) {
    if (!d_out || !d_x || n_heads <= 0 || seq_len <= 0) return LPP_ERR_INVALID_ARG;
    softmax_multihead_kernel<<<n_heads, 256, 0, S(stream)>>>(d_out, d_x, seq_len, att_stride);
    return chk();
}

lpp_status lpp_op_scale_multihead(float* d_att, float scale, int n_heads, int seq_len, int att_stride, void* stream) {
    if (!d_att || n_heads <= 0 || seq_len <= 0) return LPP_ERR_INVALID_ARG;
    scale_multihead_kernel<<<dim3(blocks(seq_len, 256), n_heads), 256, 0, S(stream)>>>(d_att, scale, seq_len,
                                                                                        att_stride);
    return chk();
}

lpp_status lpp_op_aggregation_multihead(float* d_out, const void* d_v_f16, const float* d_att, int n_heads,
                                        int seq_len, int head_size, int gqa_factor, int att_stride, void* stream) {
    if (!d_out || !d_v_f16 || !d_att || n_heads <= 0 || seq_len <= 0 || head_size <= 0 || head_size > 128 ||
        gqa_factor <= 0)
        return LPP_ERR_INVALID_ARG;
    aggregation_multihead_kernel<<<n_heads, 128, 0, S(stream)>>>(d_out, (const __half*)d_v_f16, d_att, seq_len,
                                                                 head_size, gqa_factor, att_stride);
    return chk();
}

lpp_status lpp_op_residual_add(float* d_out, const float* d_a, const float* d_b, int n, void* stream) {
    if (!d_out || !d_a || !d_b || n <= 0) return LPP_ERR_INVALID_ARG;
    residual_add_kernel<<<blocks(n, 256), 256, 0, S(stream)>>>(d_out, d_a, d_b, n);
    return chk();
}

lpp_status lpp_op_scatter_kv(void* d_kc_f16, void* d_vc_f16, const float* d_k, const float* d_v, int layer, int pos,
                             int n_kv_heads, int head_size, int seq_len, void* stream) {
    if (!d_kc_f16 || !d_vc_f16 || !d_k || !d_v || layer < 0 || pos < 0 || pos >= seq_len || n_kv_heads <= 0 ||
        head_size <= 0)
        return LPP_ERR_INVALID_ARG;
    scatter_kv_kernel<<<blocks(n_kv_heads * head_size, 256), 256, 0, S(stream)>>>(
        (__half*)d_kc_f16, (__half*)d_vc_f16, d_k, d_v, layer, pos, n_kv_heads, head_size, seq_len);
    return chk();
}

lpp_status lpp_op_multihead_gemv(float* d_out, const float* d_q, const void* d_k_cache_f16, int layer, int pos,
                                 int n_heads, int n_kv_heads, int head_size, int seq_len, void* stream) {
    if (!d_out || !d_q || !d_k_cache_f16 || layer < 0 || pos < 0 || pos >= seq_len || n_heads <= 0 ||
        n_kv_heads <= 0 || n_heads % n_kv_heads)
        return LPP_ERR_INVALID_ARG;
    multihead_gemv_kernel<<<dim3(blocks(pos + 1, 4), n_heads), 128, 0, S(stream)>>>(
        d_out, d_q, (const __half*)d_k_cache_f16, layer, pos, n_heads, n_kv_heads, head_size, seq_len);
    return chk();
}

lpp_status lpp_op_rope_scatter(float* d_q, const float* d_k, const float* d_v, void* d_kc_f16, void* d_vc_f16,
                               int layer, int pos, int dim, int n_kv_heads, int head_size, int seq_len,
                               float rope_base, void* stream) {
    if (!d_q || !d_k || !d_v || !d_kc_f16 || !d_vc_f16 || layer < 0 || pos < 0 || pos >= seq_len || dim <= 0 ||
        (dim & 1) || (head_size & 1) || head_size <= 0)
        return LPP_ERR_INVALID_ARG;
    rope_scatter_kernel<<<blocks(dim / 2, 256), 256, 0, S(stream)>>>(d_q, d_k, d_v, (__half*)d_kc_f16,
                                                                    (__half*)d_vc_f16, layer, pos, dim, n_kv_heads,
                                                                    head_size, seq_len, rope_base);
    return chk();
}

lpp_status lpp_op_sample(float* d_logits, int vocab_size, float temperature, float penalty, const int* d_history,
                         int history_len, float r, int* d_sampled_token, void* stream) {
    if (!d_logits || !d_sampled_token || vocab_size <= 0 || history_len < 0 || history_len > kHistoryMax)
        return LPP_ERR_INVALID_ARG;
    cudaStream_t s = S(stream);
    const int nb = (vocab_size + kSampleChunk - 1) / kSampleChunk;
    if (nb > kSampleMaxBlocks) return LPP_ERR_TOO_LARGE;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return LPP_ERR_CUDA;
    const bool exact = nb <= sms;  // see launch_sampler_on_scratch
    const SampleScratch L = sample_scratch_layout(nb, exact);  // stream-ordered scratch, sized for this call
    char* scratch = nullptr;
    if (cudaMallocAsync((void**)&scratch, L.total, s) != cudaSuccess) return LPP_ERR_CUDA;
    StepState h = {};
    h.temperature = temperature;
    h.penalty = penalty;
    h.r = r;
    const bool use_hist = penalty > 1.0f && d_history && history_len > 0;
    h.history_len = use_hist ? history_len : 0;
    cudaMemcpyAsync(scratch + L.state, &h, offsetof(StepState, history), cudaMemcpyHostToDevice, s);
    if (use_hist)
        cudaMemcpyAsync(scratch + L.state + offsetof(StepState, history), d_history, (size_t)history_len * sizeof(int),
                        cudaMemcpyDeviceToDevice, s);
    cudaMemsetAsync(scratch + L.counters, 0, 512, s);
    launch_sampler_on_scratch(scratch, L, exact, d_logits, vocab_size, nb, s);
    cudaMemcpyAsync(d_sampled_token, scratch + offsetof(StepState, out_token), sizeof(int), cudaMemcpyDeviceToDevice, s);
    cudaFreeAsync(scratch, s);
    return chk();
}

lpp_status lpp_op_sample_static(float* d_logits, int vocab_size, float temperature, float penalty,
                                const int* d_history, int history_len, float r, int* d_sampled_token, void* stream) {
    if (!d_logits || !d_sampled_token || vocab_size <= 0 || history_len < 0) {
        lpp_internal_set_error("lpp_op_sample_static: null pointer or non-positive size");
        return LPP_ERR_INVALID_ARG;
    }
    if (vocab_size > kStaticSampleMaxVocab || history_len > kHistoryMax) {
        lpp_internal_set_error("lpp_op_sample_static: vocab_size > 262144 or history_len > 4096 exceeds the built-in "
                               "scratch; use lpp_op_sample, which sizes its scratch per call");
        return LPP_ERR_TOO_LARGE;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        lpp_internal_set_error("lpp_op_sample_static: no current CUDA device");
        return LPP_ERR_CUDA;
    }
    if (!g_sample_scratch_addr[dev]) {
        // one-time set-up for this device (it must be the current one): resolve where the symbol lives
        unsigned char* p = nullptr;
        const cudaError_t ge = cudaGetSymbolAddress((void**)&p, g_sample_scratch);
        if (ge != cudaSuccess || !p) {
            lpp_internal_set_error(cudaGetErrorString(ge));
            return LPP_ERR_CUDA;
        }
        g_sample_scratch_addr[dev] = p;
    }
    unsigned char* scratch = g_sample_scratch_addr[dev];
    cudaStream_t s = S(stream);
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return LPP_ERR_CUDA;
    const int nb = (vocab_size + kSampleChunk - 1) / kSampleChunk;
    const bool exact = nb <= sms;  // the same choice of kernel as lpp_op_sample
    const bool use_hist = penalty > 1.0f && d_history && history_len > 0;
    sample_static_setup_kernel<<<1, 256, 0, s>>>((StepState*)(scratch + kStaticLayout.state),
                                                 (unsigned int*)(scratch + kStaticLayout.counters), temperature, penalty, r,
                                                 use_hist ? d_history : nullptr, use_hist ? history_len : 0);
    launch_sampler_on_scratch((char*)scratch, kStaticLayout, exact, d_logits, vocab_size, nb, s);
    sample_static_publish_kernel<<<1, 1, 0, s>>>((const StepState*)(scratch + kStaticLayout.state), d_sampled_token);
    return chk();
}

}  // extern "C"
