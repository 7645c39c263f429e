// Batch-1 streaming GEMV family: out[n] = W[n,K] . x[K] with FP16 or FP32 weights, FP32 activations
// and FP32 accumulation.  One kernel template serves every matrix of the decode step; what differs
// is the prologue (plain vector, RMSNorm'd vector, embedding row) and the epilogue (store,
// residual add, SwiGLU, RoPE + KV-cache scatter).
//
// Replaces, from the reference tree: gemv_kernel / gemv_f16_kernel / convert_f32_to_f16_kernel
// (src/matmul.cu:9-161), rmsnorm (src/RMSNorm.cu:11-71, fused as prologue), swiglu_kernel
// (src/swiglu.cu:6-33) and residual_add_kernel (src/residual.cu:5-31) as epilogues, rope_kernel +
// scatter_kv_kernel (src/rope.cu:7-38, src/scatter_kv.cu:6-26) as the QKV epilogue.  Numerics
// follow the reference CPU path (src/ops.cpp): activations stay FP32 (the reference GPU kernel
// rounds x to FP16 and accumulates in half2, src/matmul.cu:85-99 -- deliberately not copied).
//
// Data movement, ring variant: each CTA owns a contiguous range of row pairs, dealt round-robin to
// eight consumer warps.  Every consumer warp has a private ring of shared-memory slots fed by its
// own lane of the producer warp with 1-D bulk async copies (completion counted in bytes on an
// mbarrier per slot): eight independent single-producer / single-consumer pipelines, so every
// barrier is visited phase by phase in order by exactly one waiter on each side, the main loop has
// no CTA-wide barrier, and the copy-issue work runs eight lanes wide instead of on one thread.
// The copy engine retires roughly one bulk copy per ~100 SM cycles whatever its size, so a stage is
// always ONE copy of ~8 KiB: several whole row pairs when rows are short, one K-chunk of one row
// when they are long.  The producer starts before the programmatic
// dependency wait -- weights do not depend on the previous kernel -- so the ring is already full
// when the activations arrive.  HBM traffic = the matrix once; x is re-read from L2 per CTA.
#pragma once
#include "common.cuh"

namespace lpp {

enum GemvEpi : int { kEpiStore = 0, kEpiResid = 1, kEpiSwiglu = 2, kEpiQkv = 3 };

constexpr int kGemvConsumerWarps = 8;
constexpr int kGemvRingThreads = (kGemvConsumerWarps + 1) * 32;  // + producer warp
constexpr int kGemvLdgThreads = 256;
constexpr int kGemvMaxStages = 16;  // ring slots per consumer warp
// per consumer warp: one "full" and one "empty" barrier per slot of its private ring
constexpr int kGemvBarrierBytes = 2 * kGemvConsumerWarps * kGemvMaxStages * 8;
constexpr int kRowsPerGroup = 2;                           // rows handled together by one warp

constexpr int kMaxTp = 8;  // ranks of a tensor-parallel group

struct GemvArgs {
    const void* W;  // [n_rows][K] row-major, element type WT
    int n_rows, K;
    // ---- prologue
    const float* x;       // input vector [K] (ignored when emb != nullptr)
    const float* norm_w;  // RMSNorm weight [K], nullptr = no normalisation
    const void* emb;      // embedding table [vocab][K] in the weight dtype, nullptr = use x
    float* x_store;       // CTA 0 stores the un-normalised input vector here (nullptr = don't)
    StepState* st;        // token / pos / status
    int vocab, seq_len;
    // ---- epilogue
    float* out;          // Store/Resid: [n_rows]; Swiglu: [n_rows/2]; Qkv: q vector [q_rows]
    const float* resid;  // Resid: added to the result when non-null
    int q_rows, kv_rows, head_size;  // Qkv: rows are q | k | v
    const float2* rope;              // Qkv: [seq_len][head_size/2] (cos, sin)
    void* k_cache;                   // Qkv: this layer's K cache [kv_heads][seq_len][head_size]
    void* v_cache;
    int kv_is_f32;
    // ---- ring geometry (host-computed)
    int pairs_per_stage;  // > 0: a stage holds this many whole row pairs (one contiguous copy);
                          // 0: rows are long, a stage holds one K-chunk (kc elements) of one row
    int kc;           // K elements per stage in long-row mode (multiple of 8)
    int n_stages;     // ring slots per consumer warp
    int stage_bytes;  // bytes per slot
    // ---- L2 prefetch of the weights the NEXT kernel of the step will stream (nullptr = none).  Used by tensor-
    // parallel engines only: there HBM idles while a consumer waits for its peers' rows, and pulling the next
    // matrix towards L2 in that time measured 45 us per token; on one GPU it made no difference and is off.
    const void* pf;
    unsigned int pf_bytes;
    int debug;        // timing experiments only: 1 = consumers skip the arithmetic, 2 = producer skips the copies
    int xs_bytes;     // shared-memory bytes reserved for the staged input (0 = K floats rounded up to 128)
    unsigned long long* trace;  // timing experiments only: [CTA][8] global-timer stamps, nullptr = none
    // ---- tensor-parallel exchange over peer memory (null pointers = not used).  (The same words used on ONE
    // GPU, so that a consumer starts on the arrival of its input instead of on the completion of the producing
    // grid, measured 45 us per token SLOWER than the programmatic kernel boundary: 1.4 us per exchange.)
    // Every result travels as one 64-bit word {value, flag}, flag = the step's epoch + 1, so a word is
    // either old or complete and no fence or counter is needed.  Residual epilogue: every rank stores its
    // partial rows into slot `rank` of the exchange's receive area on EVERY rank (plain peer stores over
    // NVLink).  Prologue of the next GEMV: polls the tp_size slots of its own receive area until the
    // words carry this step's flag and adds them in rank order, so all ranks go on with bit-identical
    // activations.  The epoch word is local to each rank and bumped once at the end of every step.
    unsigned long long* tp_out[kMaxTp];  // this rank's slot [n_rows] in rank p's receive area
    const unsigned long long* tp_in;     // local receive area [tp_size][K] of the exchange that produced the input
    const unsigned int* tp_epoch;        // local epoch word
    int tp_size;
    // Arrival hint: every CTA of a producing GEMV bumps (relaxed, unordered with the data) one counter per
    // rank and exchange when its rows are out, so that a consumer can sleep on a single word instead of
    // having all its threads poll the receive area; the flags in the data words stay the only proof of
    // arrival.  Counters only grow: an exchange is probably complete at (epoch + 1) * tp_hint_per_step.
    unsigned int* tp_hint_out[kMaxTp];   // rank p's hint counter of the exchange this GEMV produces
    const unsigned int* tp_hint_in;      // local hint counter of the exchange this GEMV consumes
    unsigned int tp_hint_per_step;       // tp_size * CTAs of the producing GEMV
    long long tp_wait_cycles;            // limit of a wait on a peer in SM clocks (a kernel argument: the poll loop must
                                         // not pay a global load for it)
};

// ------------------------------------------------------------------ x staging layouts
//
// FP16 weights: a lane multiplies 8 consecutive weights (one 16-byte vector) with 8 consecutive x.
// To keep both 16-byte x reads bank-conflict free the low and high halves of every 8-group live in
// two separate planes.  FP32 weights: one 16-byte vector = 4 weights, x is stored naturally.
template <typename WT>
__device__ __forceinline__ int xs_index(int k, int K);
template <>
__device__ __forceinline__ int xs_index<__half>(int k, int K) {
    return ((k >> 3) << 2) + (k & 3) + ((k & 4) ? (K >> 1) : 0);
}
template <>
__device__ __forceinline__ int xs_index<float>(int k, int /*K*/) {
    return k;
}

__device__ __forceinline__ void gemv_stamp(const GemvArgs& a, int k) {
    if (a.trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.trace[(size_t)blockIdx.x * 8 + k] = t;
    }
}

__device__ __forceinline__ void consumer_barrier(int nthreads) {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// Stores four consecutive inputs x[k..k+3] (k % 4 == 0) into the staging layout.
template <typename WT>
__device__ __forceinline__ void xs_store4(float* xs, int k, int K, float4 v) {
    if constexpr (sizeof(WT) == 2)
        *reinterpret_cast<float4*>(xs + ((k >> 3) << 2) + ((k & 4) ? (K >> 1) : 0)) = v;
    else
        *reinterpret_cast<float4*>(xs + k) = v;
}

// Address of the float4 holding inputs k..k+3 (k % 4 == 0) in the staging layout.
template <typename WT>
__device__ __forceinline__ float4* xs_ptr4(float* xs, int k, int K) {
    if constexpr (sizeof(WT) == 2)
        return reinterpret_cast<float4*>(xs + ((k >> 3) << 2) + ((k & 4) ? (K >> 1) : 0));
    else
        return reinterpret_cast<float4*>(xs + k);
}

// Input staging when the input vector arrives through the tensor-parallel exchange: the sum, in rank
// order, of the tp_size slots of the local receive area.  All words a thread needs from two ranks are
// requested together and only then checked for the step's flag (a failed check repeats the batch), so a
// slot costs one round trip to L2, not one per element.
template <typename WT, int NT>
__device__ __forceinline__ void stage_input_peers(const GemvArgs& a, float* xs, float* red, int tid) {
    const int K = a.K, nv4 = K >> 2;
    const unsigned int flag = *a.tp_epoch + 1u;
    if (a.tp_hint_in) {
        // one thread sleeps on the hint counter (bounded, then the data poll decides).  A wait that has already
        // run out on this engine is not repeated (the status is looked at once the counter has been slow for a
        // while, so that the ordinary case pays nothing for it), and one that runs out here sets the status bit,
        // which spares the data poll below and every later kernel of the step a second spin.
        if (tid == 0) {
            const unsigned int want = flag * a.tp_hint_per_step;
            const long long t0 = clock64();
            bool looked = false;
            while (true) {
                unsigned int v;
                asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(a.tp_hint_in) : "memory");
                if ((int)(v - want) >= 0) break;
                const long long waited = clock64() - t0;
                if (!looked && waited > (1 << 17)) {  // ~65 us: far beyond a healthy exchange
                    looked = true;
                    if (status_timed_out(a.st)) break;
                }
                if (waited > a.tp_wait_cycles) {
                    atomicOr(&a.st->status, kStatusBarrierTimeout);
                    break;
                }
                __nanosleep(20);
            }
        }
        consumer_barrier(NT);
    }
    if (tid == 0) gemv_stamp(a, 1);
    constexpr int kPer = 4, kRanks = 2;
    const bool store = a.x_store && blockIdx.x == 0;
    float ss = 0.f;
    for (int base = 0; base < nv4; base += kPer * NT) {
        float4 sum[kPer];
        for (int r0 = 0; r0 < a.tp_size; r0 += kRanks) {
            unsigned long long w[kRanks][kPer][4];
            long long t0 = 0;
            while (true) {
#pragma unroll
                for (int rr = 0; rr < kRanks; ++rr)
#pragma unroll
                    for (int j = 0; j < kPer; ++j) {
                        const int i = base + tid + j * NT;
                        if (r0 + rr < a.tp_size && i < nv4) {
                            const unsigned long long* p = a.tp_in + (size_t)(r0 + rr) * K + ((size_t)i << 2);
                            asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[rr][j][0]), "=l"(w[rr][j][1]) : "l"(p) : "memory");
                            asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[rr][j][2]), "=l"(w[rr][j][3]) : "l"(p + 2) : "memory");
                        }
                    }
                bool pending = false;
#pragma unroll
                for (int rr = 0; rr < kRanks; ++rr)
#pragma unroll
                    for (int j = 0; j < kPer; ++j)
                        if (r0 + rr < a.tp_size && base + tid + j * NT < nv4)
#pragma unroll
                            for (int q = 0; q < 4; ++q) pending |= (unsigned int)(w[rr][j][q] >> 32) != flag;
                if (!pending) break;
                if (t0 == 0) {
                    if (status_timed_out(a.st)) break;
                    t0 = clock64();
                } else if (clock64() - t0 > a.tp_wait_cycles) {
                    atomicOr(&a.st->status, kStatusBarrierTimeout);
                    break;
                }
                __nanosleep(20);
            }
#pragma unroll
            for (int rr = 0; rr < kRanks; ++rr)
#pragma unroll
                for (int j = 0; j < kPer; ++j)
                    if (r0 + rr < a.tp_size && base + tid + j * NT < nv4) {
                        const float4 u = make_float4(__uint_as_float((unsigned int)w[rr][j][0]), __uint_as_float((unsigned int)w[rr][j][1]),
                                                     __uint_as_float((unsigned int)w[rr][j][2]), __uint_as_float((unsigned int)w[rr][j][3]));
                        if (r0 + rr == 0) {
                            sum[j] = u;
                        } else {
                            sum[j].x = __fadd_rn(sum[j].x, u.x); sum[j].y = __fadd_rn(sum[j].y, u.y);
                            sum[j].z = __fadd_rn(sum[j].z, u.z); sum[j].w = __fadd_rn(sum[j].w, u.w);
                        }
                    }
        }
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = base + tid + j * NT;
            if (i < nv4) {
                ss = fmaf(sum[j].x, sum[j].x, fmaf(sum[j].y, sum[j].y, fmaf(sum[j].z, sum[j].z, fmaf(sum[j].w, sum[j].w, ss))));
                *xs_ptr4<WT>(xs, i << 2, K) = sum[j];
                if (store) reinterpret_cast<float4*>(a.x_store)[i] = sum[j];  // the residual stream
            }
        }
    }
    if (a.norm_w) {
        ss = warp_sum(ss);
        if ((tid & 31) == 0) red[tid >> 5] = ss;
        consumer_barrier(NT);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) tot += red[w];
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), 1e-5f)));
        for (int i = tid; i < nv4; i += NT) {  // the elements this thread staged itself
            float4* p = xs_ptr4<WT>(xs, i << 2, K);
            const float4 v = *p, g = __ldg(reinterpret_cast<const float4*>(a.norm_w) + i);
            *p = make_float4(__fmul_rn(__fmul_rn(v.x, scale), g.x), __fmul_rn(__fmul_rn(v.y, scale), g.y),
                             __fmul_rn(__fmul_rn(v.z, scale), g.z), __fmul_rn(__fmul_rn(v.w, scale), g.w));
        }
    }
    consumer_barrier(NT);
}

// Waits for the producing kernel, loads the input vector (embedding row or x), optionally
// RMS-normalises it (ss = 1/sqrt(mean(x^2) + 1e-5); out = x*ss*w, src/ops.cpp:20-32) and leaves it
// in shared memory in the layout xs_index<WT> describes.  Executed by `NT` threads (tid 0..NT-1).
// The norm weights are constants, so their loads are issued before the dependency wait.
template <typename WT, int NT>
__device__ __forceinline__ void stage_input(const GemvArgs& a, float* xs, float* red, int tid) {
    const int K = a.K;
    const int nv4 = K >> 2;
    constexpr int kPer = 4;  // float4 per thread and pass: one pass covers 4*4*NT inputs
    const bool one_pass = nv4 <= kPer * NT;
    float4 wr[kPer];
    if (a.norm_w && one_pass) {
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = tid + j * NT;
            if (i < nv4) wr[j] = __ldg(reinterpret_cast<const float4*>(a.norm_w) + i);
        }
    }
    // An input that arrives through the tensor-parallel exchange validates itself word by word (this
    // rank's own slot included): its flags can only be complete once every rank's producing GEMV has
    // stored all its rows, which in turn follows everything earlier in the step, so that case does not
    // wait for the local kernel to drain its peer stores and exit.
    if (a.tp_in != nullptr) {
        stage_input_peers<WT, NT>(a, xs, red, tid);
        return;
    }
    pdl_wait();  // activations / KV / step state come from the previous kernel
    if (tid == 0) gemv_stamp(a, 1);

    if (a.emb) {
        // first layer: the input is the embedding row of the device-resident token, widened exactly
        int tok = a.st->token;
        if (tok < 0 || tok >= a.vocab) {
            if (tid == 0) atomicOr(&a.st->status, kStatusBadToken);
            tok = 0;
        }
        const WT* erow = reinterpret_cast<const WT*>(a.emb) + (size_t)tok * K;
        const bool store = a.x_store && blockIdx.x == 0;
        float ss = 0.f;
        for (int k = tid; k < K; k += NT) {
            float v;
            if constexpr (sizeof(WT) == 2)
                v = __half2float(erow[k]);
            else
                v = erow[k];
            ss = fmaf(v, v, ss);
            if (store) a.x_store[k] = v;
            xs[xs_index<WT>(k, K)] = v;
        }
        if (a.norm_w) {
            ss = warp_sum(ss);
            if ((tid & 31) == 0) red[tid >> 5] = ss;
            consumer_barrier(NT);
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < NT / 32; ++w) tot += red[w];
            const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), 1e-5f)));
            for (int k = tid; k < K; k += NT) {
                const int i = xs_index<WT>(k, K);
                xs[i] = __fmul_rn(__fmul_rn(xs[i], scale), a.norm_w[k]);
            }
        }
        consumer_barrier(NT);
        return;
    }

    const float4* x4 = reinterpret_cast<const float4*>(a.x);
    auto load_x4 = [&](int i) -> float4 { return __ldcg(x4 + i); };
    if (!a.norm_w) {
        for (int i = tid; i < nv4; i += NT) xs_store4<WT>(xs, i << 2, K, load_x4(i));
        consumer_barrier(NT);
        return;
    }
    float ss = 0.f;
    float4 xr[kPer];
    if (one_pass) {
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = tid + j * NT;
            if (i < nv4) xr[j] = load_x4(i);
        }
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = tid + j * NT;
            if (i < nv4) ss = fmaf(xr[j].x, xr[j].x, fmaf(xr[j].y, xr[j].y, fmaf(xr[j].z, xr[j].z, fmaf(xr[j].w, xr[j].w, ss))));
        }
    } else {
        for (int i = tid; i < nv4; i += NT) {
            const float4 v = load_x4(i);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    consumer_barrier(NT);
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) tot += red[w];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), 1e-5f)));
    auto normed = [&](float4 v, float4 w) {
        return make_float4(__fmul_rn(__fmul_rn(v.x, scale), w.x), __fmul_rn(__fmul_rn(v.y, scale), w.y),
                           __fmul_rn(__fmul_rn(v.z, scale), w.z), __fmul_rn(__fmul_rn(v.w, scale), w.w));
    };
    if (one_pass) {
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = tid + j * NT;
            if (i < nv4) xs_store4<WT>(xs, i << 2, K, normed(xr[j], wr[j]));
        }
    } else {
        for (int i = tid; i < nv4; i += NT)
            xs_store4<WT>(xs, i << 2, K, normed(load_x4(i), __ldg(reinterpret_cast<const float4*>(a.norm_w) + i)));
    }
    consumer_barrier(NT);
}

__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

// Dot products of NR (1 or 2) weight rows (klen elements each, 16-byte aligned; in shared memory, or
// in global memory when kFromGlobal) with x[k0 .. k0+klen) from shared memory.  Lane-strided over
// 16-byte vectors; the x vectors are loaded once and used for both rows.
template <typename WT, int NR, bool kFromGlobal>
__device__ __forceinline__ void dot_rows(const unsigned char* row0, const unsigned char* row1, const float* xs,
                                         int K, int k0, int klen, int lane, float& acc0, float& acc1) {
    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
    const uint4* r0 = reinterpret_cast<const uint4*>(row0);
    const uint4* r1 = reinterpret_cast<const uint4*>(row1);
    const uint32_t s0 = kFromGlobal ? 0u : smem_u32(row0), s1 = (kFromGlobal || NR == 1) ? 0u : smem_u32(row1);
    if constexpr (sizeof(WT) == 2) {
        const int nvec = klen >> 3;
        const uint32_t xlo = smem_u32(xs) + (uint32_t)(k0 >> 3) * 16u;
        const uint32_t xhi = xlo + (uint32_t)K * 2u;  // second plane starts K/2 floats further on
#pragma unroll 4
        for (int v = lane; v < nvec; v += 32) {
            uint4 w0, w1 = make_uint4(0, 0, 0, 0);
            if constexpr (kFromGlobal) {
                w0 = ldg_stream_u4(r0 + v);
                if constexpr (NR == 2) w1 = ldg_stream_u4(r1 + v);
            } else {
                w0 = lds_u4(s0 + (uint32_t)v * 16u);
                if constexpr (NR == 2) w1 = lds_u4(s1 + (uint32_t)v * 16u);
            }
            const float4 xl = lds_f4(xlo + (uint32_t)v * 16u), xh = lds_f4(xhi + (uint32_t)v * 16u);
            float2 p;
            p = half2_bits_to_float2(w0.x); a0 = fmaf(p.x, xl.x, a0); b0 = fmaf(p.y, xl.y, b0);
            p = half2_bits_to_float2(w0.y); a0 = fmaf(p.x, xl.z, a0); b0 = fmaf(p.y, xl.w, b0);
            p = half2_bits_to_float2(w0.z); a0 = fmaf(p.x, xh.x, a0); b0 = fmaf(p.y, xh.y, b0);
            p = half2_bits_to_float2(w0.w); a0 = fmaf(p.x, xh.z, a0); b0 = fmaf(p.y, xh.w, b0);
            if constexpr (NR == 2) {
                p = half2_bits_to_float2(w1.x); a1 = fmaf(p.x, xl.x, a1); b1 = fmaf(p.y, xl.y, b1);
                p = half2_bits_to_float2(w1.y); a1 = fmaf(p.x, xl.z, a1); b1 = fmaf(p.y, xl.w, b1);
                p = half2_bits_to_float2(w1.z); a1 = fmaf(p.x, xh.x, a1); b1 = fmaf(p.y, xh.y, b1);
                p = half2_bits_to_float2(w1.w); a1 = fmaf(p.x, xh.z, a1); b1 = fmaf(p.y, xh.w, b1);
            }
        }
    } else {
        const int nvec = klen >> 2;
        const uint32_t x4 = smem_u32(xs) + (uint32_t)(k0 >> 2) * 16u;
#pragma unroll 4
        for (int v = lane; v < nvec; v += 32) {
            uint4 w0, w1 = make_uint4(0, 0, 0, 0);
            if constexpr (kFromGlobal) {
                w0 = ldg_stream_u4(r0 + v);
                if constexpr (NR == 2) w1 = ldg_stream_u4(r1 + v);
            } else {
                w0 = lds_u4(s0 + (uint32_t)v * 16u);
                if constexpr (NR == 2) w1 = lds_u4(s1 + (uint32_t)v * 16u);
            }
            const float4 xv = lds_f4(x4 + (uint32_t)v * 16u);
            a0 = fmaf(__uint_as_float(w0.x), xv.x, a0); b0 = fmaf(__uint_as_float(w0.y), xv.y, b0);
            a0 = fmaf(__uint_as_float(w0.z), xv.z, a0); b0 = fmaf(__uint_as_float(w0.w), xv.w, b0);
            if constexpr (NR == 2) {
                a1 = fmaf(__uint_as_float(w1.x), xv.x, a1); b1 = fmaf(__uint_as_float(w1.y), xv.y, b1);
                a1 = fmaf(__uint_as_float(w1.z), xv.z, a1); b1 = fmaf(__uint_as_float(w1.w), xv.w, b1);
            }
        }
    }
    acc0 += a0 + b0;
    if constexpr (NR == 2) acc1 += a1 + b1;
}

// Store of a finished row pair: locally, or as {value, flag} words into this rank's slot (residual GEMVs) or
// row range (vocabulary-sharded classifier) on every rank of the tensor-parallel group.
__device__ __forceinline__ void store_rows(const GemvArgs& a, int row, float v0, float v1) {
    if (a.tp_out[0]) {
        const unsigned long long flag = (unsigned long long)(*a.tp_epoch + 1u) << 32;
        const unsigned long long w0 = flag | __float_as_uint(v0), w1 = flag | __float_as_uint(v1);
#pragma unroll
        for (int p = 0; p < kMaxTp; ++p)
            if (p < a.tp_size)
                asm volatile("st.volatile.global.v2.u64 [%0], {%1,%2};" ::"l"(a.tp_out[p] + row), "l"(w0), "l"(w1) : "memory");
    } else {
        *reinterpret_cast<float2*>(a.out + row) = make_float2(v0, v1);
    }
}

// Writes the results of row pair `g` (rows 2g, 2g+1); called by one lane with the warp-reduced sums.
template <int EPI>
__device__ __forceinline__ void gemv_epilogue(const GemvArgs& a, int g, float v0, float v1) {
    const int row = g * kRowsPerGroup;
    if constexpr (EPI == kEpiStore) {
        store_rows(a, row, v0, v1);
    } else if constexpr (EPI == kEpiResid) {
        // x += W.xb (src/model.cpp:232, 239); under tensor parallelism only rank 0 passes resid
        if (a.resid) {
            const float2 r = __ldcg(reinterpret_cast<const float2*>(a.resid + row));  // written by an earlier phase
            v0 += r.x;
            v1 += r.y;
        }
        store_rows(a, row, v0, v1);
    } else if constexpr (EPI == kEpiSwiglu) {
        // rows are interleaved (gate_i, up_i); hb = (h1*sigmoid(h1))*h3 (src/ops.cpp:78-87)
        const float sig = __fdiv_rn(1.0f, 1.0f + expf(-v0));
        a.out[g] = __fmul_rn(__fmul_rn(v0, sig), v1);
    } else {  // kEpiQkv
        const int pos = a.st->pos;
        if (pos < 0 || pos >= a.seq_len) {
            atomicOr(&a.st->status, kStatusBadPos);
            return;
        }
        const int hs = a.head_size;
        if (row < a.q_rows + a.kv_rows) {
            // adjacent-pair rotation with the table entry for (pos, (row % hs)/2) (src/ops.cpp:34-54);
            // separate multiply and subtract/add, as the reference's scalar code rounds
            const float2 cs = __ldg(a.rope + (size_t)pos * (hs >> 1) + ((row % hs) >> 1));
            const float r0 = __fsub_rn(__fmul_rn(v0, cs.x), __fmul_rn(v1, cs.y));
            const float r1 = __fadd_rn(__fmul_rn(v0, cs.y), __fmul_rn(v1, cs.x));
            v0 = r0;
            v1 = r1;
        }
        if (row < a.q_rows) {
            *reinterpret_cast<float2*>(a.out + row) = make_float2(v0, v1);
        } else {
            const bool is_k = row < a.q_rows + a.kv_rows;
            const int r = row - a.q_rows - (is_k ? 0 : a.kv_rows);
            const int h = r / hs, off = r % hs;
            // cache index within the layer: h*(seq_len*hs) + pos*hs + off (src/scatter_kv.cu:15-16)
            const size_t idx = (size_t)h * ((size_t)a.seq_len * hs) + (size_t)pos * hs + off;
            void* base = is_k ? a.k_cache : a.v_cache;
            if (a.kv_is_f32)
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(base) + idx) = make_float2(v0, v1);
            else
                *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(base) + idx) = __floats2half2_rn(v0, v1);
        }
    }
}

// ------------------------------------------------------------------ ring (bulk async copy) variant

// Body of the ring kernel.  Returns true on the consumer threads once all of this CTA's rows are
// done (so a caller can append a CTA-level tail), false on the producer warp and after a timeout.
template <typename WT, int EPI>
__device__ __forceinline__ bool gemv_ring_body(const GemvArgs& a, unsigned char* smem) {
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                // [consumer warp][kGemvMaxStages]
    uint64_t* empty = full + kGemvConsumerWarps * kGemvMaxStages;      // [consumer warp][kGemvMaxStages]
    float* red = reinterpret_cast<float*>(smem + kGemvBarrierBytes);   // 8 floats
    float* xs = reinterpret_cast<float*>(smem + kGemvBarrierBytes + 128);
    const size_t xs_bytes = a.xs_bytes > 0 ? (size_t)a.xs_bytes : (((size_t)a.K * 4 + 127) & ~(size_t)127);
    unsigned char* ring = smem + kGemvBarrierBytes + 128 + xs_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = a.n_stages;  // slots per consumer warp
    const int groups = a.n_rows / kRowsPerGroup;
    // this CTA's row pairs, then this warp's (or producer lane's) contiguous share of them
    const int g0 = (int)(((long long)blockIdx.x * groups) / gridDim.x);
    const int g1 = (int)(((long long)(blockIdx.x + 1) * groups) / gridDim.x);
    const int ng = g1 - g0;
    const int w = (warp == kGemvConsumerWarps) ? lane : warp;  // pipeline index
    const int p0 = g0 + (w < kGemvConsumerWarps ? (ng * w) / kGemvConsumerWarps : 0);
    const int p1 = g0 + (w < kGemvConsumerWarps ? (ng * (w + 1)) / kGemvConsumerWarps : 0);
    const size_t row_bytes = (size_t)a.K * sizeof(WT);
    const int m = a.pairs_per_stage;
    const int nch = m > 0 ? 1 : (a.K + a.kc - 1) / a.kc;
    const int pstep = m > 0 ? m : 1;  // pairs advance by pstep from p0 to p1
    const int unit = m > 0 ? m : 1;

    if (tid == 0) gemv_stamp(a, 0);
    // The dependent kernel is released for launch at once: its CTAs take over an SM as soon as one of
    // this kernel's CTAs leaves it and start streaming their own weights while the rest of this grid
    // finishes (they still wait for this grid's completion before touching activations).
    if (tid == 0 && !(a.debug & 4)) pdl_launch_dependents();
    if (tid < kGemvConsumerWarps * NS) {
        const int bw = tid / NS, sl = tid - bw * NS;
        mbar_init(&full[bw * kGemvMaxStages + sl], 1);
        mbar_init(&empty[bw * kGemvMaxStages + sl], 1);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == kGemvConsumerWarps) {
        // ---------------- producer warp: lane w feeds consumer warp w through w's private ring
        if (lane < kGemvConsumerWarps) {
            const unsigned char* W = reinterpret_cast<const unsigned char*>(a.W);
            uint64_t* myfull = full + w * kGemvMaxStages;
            uint64_t* myempty = empty + w * kGemvMaxStages;
            unsigned char* myring = ring + (size_t)w * NS * a.stage_bytes;
            int slot = 0, pass = 0;  // pass = completed trips around the ring
            bool alive = true;
            // streamed weights are marked evict-first in L2: they are used once per token and would
            // otherwise push the K/V cache and the activations out (debug bit 8 turns the hint off)
            const unsigned long long policy = !(a.debug & 8) ? l2_policy_evict_first() : 0ull;
            auto issue = [&](const unsigned char* src, uint32_t bytes) -> bool {
                // trip p > 0 reuses a slot once its release number p-1 has happened
                if (pass > 0 && !mbar_wait_bounded(&myempty[slot], (uint32_t)(pass - 1) & 1u, a.st))
                    return false;
                if (a.debug & 2) {
                    mbar_arrive(&myfull[slot]);
                } else {
                    mbar_arrive_expect_tx(&myfull[slot], bytes);
                    if (!(a.debug & 8))
                        bulk_g2s_hint(myring + (size_t)slot * a.stage_bytes, src, bytes, &myfull[slot], policy);
                    else
                        bulk_g2s(myring + (size_t)slot * a.stage_bytes, src, bytes, &myfull[slot]);
                }
                if (++slot == NS) {
                    slot = 0;
                    ++pass;
                }
                return true;
            };
            if (lane == 0) gemv_stamp(a, 5);
            if (m > 0) {
                for (int p = p0; p < p1 && alive; p += pstep) {
                    const int cnt = min(unit, p1 - p);
                    alive = issue(W + (size_t)p * kRowsPerGroup * row_bytes, (uint32_t)(cnt * kRowsPerGroup * row_bytes));
                }
            } else {
                for (int p = p0; p < p1 && alive; p += pstep)
                    for (int r = 0; r < kRowsPerGroup && alive; ++r)
                        for (int c = 0; c < nch && alive; ++c) {
                            const int k0 = c * a.kc;
                            const int klen = min(a.kc, a.K - k0);
                            alive = issue(W + ((size_t)(p * kRowsPerGroup + r) * a.K + k0) * sizeof(WT),
                                          (uint32_t)(klen * sizeof(WT)));
                        }
            }
            if (lane == 0) gemv_stamp(a, 6);
            // this lane's HBM requests are all queued: pull its share of the next kernel's weights
            // towards L2 so the memory system stays busy across the kernel boundary
            if (a.pf && alive) {
                const unsigned int lanes = gridDim.x * kGemvConsumerWarps;
                unsigned int slice = (a.pf_bytes + lanes - 1) / lanes;
                slice = (slice + 15u) & ~15u;
                const unsigned long long off = (unsigned long long)(blockIdx.x * kGemvConsumerWarps + w) * slice;
                if (off < a.pf_bytes) {
                    const unsigned int n = (unsigned int)min((unsigned long long)slice, (unsigned long long)a.pf_bytes - off);
                    bulk_prefetch_l2(reinterpret_cast<const unsigned char*>(a.pf) + off, n & ~15u);
                }
            }
        }
        __syncwarp();
        // all of this CTA's copies are issued: the next kernel may start launching
        if (lane == 0 && (a.debug & 4)) pdl_launch_dependents();
        return false;
    }

    // ---------------- consumers
    if constexpr (EPI == kEpiQkv) {
        // The position is written by the previous step's sampler, which completed before this step
        // began, and the rotation table is constant: both are pulled into L1 before the dependency
        // wait so the epilogue of the first row pairs does not pay two L2 round trips in a row.
        const int pos = a.st->pos;
        if (pos >= 0 && pos < a.seq_len && tid < (a.head_size >> 1)) {
            const float2 cs = __ldg(a.rope + (size_t)pos * (a.head_size >> 1) + tid);
            asm volatile("" ::"f"(cs.x), "f"(cs.y));
        }
    }
    stage_input<WT, kGemvConsumerWarps * 32>(a, xs, red, tid);
    if (tid == 0) gemv_stamp(a, 2);

    uint64_t* myfull = full + w * kGemvMaxStages;
    uint64_t* myempty = empty + w * kGemvMaxStages;
    const unsigned char* myring = ring + (size_t)w * NS * a.stage_bytes;
    int slot = 0;
    uint32_t par = 0;
    // waits for this warp's next stage; warp-uniform outcome so a timed-out lane cannot strand the rest
    auto acquire = [&]() -> bool { return __all_sync(0xffffffffu, mbar_wait_bounded(&myfull[slot], par, a.st)); };
    auto release = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&myempty[slot]);
        if (++slot == NS) {
            slot = 0;
            par ^= 1u;
        }
    };
    // A warp whose wait runs out stops consuming but still returns through the common exit, so a
    // CTA-level tail (which uses CTA barriers) is never left waiting for it.
    bool ok = true;
    // Residual epilogue: the residual of this warp's first pair is requested now, so its L2 round
    // trip runs beside the dot product instead of after it (the weights are usually in the ring
    // already when the input arrives).  The producing kernel has completed: stage_input waited.
    float2 r_first = make_float2(0.f, 0.f);
    if (EPI == kEpiResid && a.resid && lane == 0 && p0 < p1)
        r_first = __ldcg(reinterpret_cast<const float2*>(a.resid + (size_t)p0 * kRowsPerGroup));
    if (m > 0) {
        for (int p = p0; p < p1 && ok; p += pstep) {
            const int cnt = min(unit, p1 - p);
            if (!acquire()) {
                ok = false;
                break;
            }
            if (tid == 0 && p == p0) gemv_stamp(a, 3);
            const unsigned char* st = myring + (size_t)slot * a.stage_bytes;
            for (int i = 0; i < cnt; ++i) {
                float acc0 = 0.f, acc1 = 0.f;
                const unsigned char* r0 = st + (size_t)i * kRowsPerGroup * row_bytes;
                if (!(a.debug & 1)) dot_rows<WT, 2, false>(r0, r0 + row_bytes, xs, a.K, 0, a.K, lane, acc0, acc1);
                acc0 = warp_sum(acc0);
                acc1 = warp_sum(acc1);
                if (lane == 0) {
                    if (EPI == kEpiResid && p + i == p0)
                        store_rows(a, p0 * kRowsPerGroup, acc0 + r_first.x, acc1 + r_first.y);
                    else
                        gemv_epilogue<EPI>(a, p + i, acc0, acc1);
                }
            }
            release();
        }
    } else {
        for (int p = p0; p < p1 && ok; p += pstep) {
            float acc[kRowsPerGroup] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < kRowsPerGroup; ++r)
                for (int c = 0; c < nch && ok; ++c) {
                    if (!acquire()) {
                        ok = false;
                        break;
                    }
                    const int k0 = c * a.kc;
                    const int klen = min(a.kc, a.K - k0);
                    const unsigned char* st = myring + (size_t)slot * a.stage_bytes;
                    float dummy = 0.f;
                    if (!(a.debug & 1)) dot_rows<WT, 1, false>(st, st, xs, a.K, k0, klen, lane, acc[r], dummy);
                    release();
                }
            if (!ok) break;
            const float v0 = warp_sum(acc[0]), v1 = warp_sum(acc[1]);
            if (lane == 0) {
                if (EPI == kEpiResid && p == p0)
                    store_rows(a, p0 * kRowsPerGroup, v0 + r_first.x, v1 + r_first.y);
                else
                    gemv_epilogue<EPI>(a, p, v0, v1);
            }
        }
    }
    if (tid == 0) gemv_stamp(a, 4);
    return true;
}

template <typename WT, int EPI>
__global__ void __launch_bounds__(kGemvRingThreads) gemv_ring_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const bool consumer = gemv_ring_body<WT, EPI>(a, smem);
    if constexpr (EPI == kEpiResid) {
        // tensor-parallel exchange: this CTA's rows are on their way, tell every rank (a hint, see GemvArgs)
        if (consumer && a.tp_size > 1 && a.tp_hint_out[0]) {
            consumer_barrier(kGemvConsumerWarps * 32);
            if (threadIdx.x == 0) gemv_stamp(a, 7);
            if ((int)threadIdx.x < a.tp_size)
                asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.tp_hint_out[threadIdx.x]) : "memory");
        }
    }
}

// ------------------------------------------------------------------ direct-load variant
//
// Same partition and epilogues; weights go global -> registers with 128-bit streaming loads.  Kept
// as the measured alternative to the ring (see profiles/).
template <typename WT, int EPI>
__global__ void __launch_bounds__(kGemvLdgThreads) gemv_ldg_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    float* red = reinterpret_cast<float*>(smem);
    float* xs = reinterpret_cast<float*>(smem + 128);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int groups = a.n_rows / kRowsPerGroup;
    const int g0 = (int)(((long long)blockIdx.x * groups) / gridDim.x);
    const int g1 = (int)(((long long)(blockIdx.x + 1) * groups) / gridDim.x);
    constexpr int NW = kGemvLdgThreads / 32;

    stage_input<WT, kGemvLdgThreads>(a, xs, red, tid);
    const unsigned char* W = reinterpret_cast<const unsigned char*>(a.W);
    const size_t row_bytes = (size_t)a.K * sizeof(WT);
    for (int g = g0 + warp; g < g1; g += NW) {
        float acc0 = 0.f, acc1 = 0.f;
        const unsigned char* r0 = W + (size_t)g * kRowsPerGroup * row_bytes;
        dot_rows<WT, 2, true>(r0, r0 + row_bytes, xs, a.K, 0, a.K, lane, acc0, acc1);
        acc0 = warp_sum(acc0);
        acc1 = warp_sum(acc1);
        if (lane == 0) gemv_epilogue<EPI>(a, g, acc0, acc1);
    }
    pdl_launch_dependents();
}

}  // namespace lpp
