// Multi-block fused sampler: repetition penalty -> temperature -> softmax -> categorical draw (or
// argmax at temperature 0) over up to 128K+ logits in ONE kernel launch.
//
// Replaces fused_sample_kernel / cuda_sample (src/sample.cu:6-214), which runs a single 256-thread
// block over the whole vocabulary, and follows the CPU sample() (src/model.cpp:256-303) where the
// two disagree: the penalty is applied once per history occurrence (src/model.cpp:259-270; the
// reference kernel races on duplicates, src/sample.cu:18-27), logits are divided by the
// temperature (src/model.cpp:286-288; the kernel multiplies by a reciprocal, src/sample.cu:29),
// argmax returns the first maximum (src/model.cpp:272-283; the kernel loses the index across
// warps, src/sample.cu:77-90), and no random number is consumed at temperature 0.  top-p is not
// implemented, as in the reference kernel.
//
// Structure: every block owns kSampleChunk consecutive logits: it applies penalty and temperature,
// writes them back (the reference kernel also mutates the logits in place), and publishes a
// partial (max, first index of max, sum of exp(v - block max)).  The last block to finish (ticket
// counter) reduces the partials in block order, locates the block in which the cumulative
// distribution passes r, and resolves the index inside it with a block-wide prefix sum.  All
// reductions have a fixed shape, so the result is a pure function of (logits, history, r).
#pragma once
#include "common.cuh"

namespace lpp {

constexpr int kSampleThreads = 512;
constexpr int kSamplePerThread = 4;
constexpr int kSampleChunk = kSampleThreads * kSamplePerThread;  // 2048 logits per block
constexpr int kSampleMaxBlocks = 512;  // vocabularies up to 1,048,576 entries

struct SampleArgs {
    float* logits;  // [vocab], modified in place (penalty, temperature)
    int vocab;
    StepState* st;
    float* part_max;  // [n_blocks]
    int* part_idx;    // [n_blocks]
    float* part_sum;  // [n_blocks]
    unsigned int* counter;  // zero between launches
    const float* r_values;  // free-running mode: one uniform draw per step
    int* out_tokens;        // free-running mode: sampled token per step
    unsigned int* zero;     // counters to clear once the step is over (grid-barrier tickets), may be null
    int zero_n;
    unsigned int* bump;     // word to increment once the step is over (tensor-parallel exchange epoch), may be null
};

struct MaxIdx {
    float v;
    int i;
};
// "first maximum": larger value wins, equal values keep the lower index
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ MaxIdx block_argmax(MaxIdx x, MaxIdx* s_red, int tid) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    if ((tid & 31) == 0) s_red[tid >> 5] = x;
    __syncthreads();
    MaxIdx r = s_red[0];
    for (int w = 1; w < kSampleThreads / 32; ++w) r = better(r, s_red[w]);
    __syncthreads();
    return r;
}
// Fixed-shape block sum: butterfly inside each warp, then warp totals added in warp order.
__device__ __forceinline__ float block_sum(float x, float* s_red, int tid) {
    x = warp_sum(x);
    if ((tid & 31) == 0) s_red[tid >> 5] = x;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) r += s_red[w];
    __syncthreads();
    return r;
}

static __global__ void __launch_bounds__(kSampleThreads) sample_kernel(const SampleArgs a) {
    __shared__ float s_val[kSampleChunk];
    __shared__ MaxIdx s_mi[kSampleThreads / 32];
    __shared__ float s_f[kSampleThreads / 32];
    __shared__ float s_wtot[kSampleThreads / 32];  // per-warp totals of the final prefix scan
    __shared__ float s_scaled[kSampleMaxBlocks];   // block partial sums rescaled to the global max
    __shared__ int s_flag;
    __shared__ int s_found;

    // the next token's step kernel may become resident and start streaming weights meanwhile; it
    // does not read anything this kernel writes before its own dependency wait
    pdl_launch_dependents();
    pdl_wait();
    StepState* st = a.st;
    const int tid = threadIdx.x;
    const int base = blockIdx.x * kSampleChunk;
    const int n = min(kSampleChunk, a.vocab - base);
    const float temperature = st->temperature;
    const float penalty = st->penalty;
    const int hist_len = min(st->history_len, kHistoryMax);

    for (int i = tid; i < n; i += kSampleThreads) s_val[i] = __ldcg(a.logits + base + i);
    __syncthreads();

    // repetition penalty, once per occurrence (order between different tokens is irrelevant and
    // repeated application to one token only depends on its own running value)
    if (penalty > 1.0f && hist_len > 0) {
        for (int i = tid; i < hist_len; i += kSampleThreads) {
            const int tok = st->history[i];
            if (tok < base || tok >= base + n) continue;
            bool first = true;
            for (int j = 0; j < i; ++j)
                if (st->history[j] == tok) {
                    first = false;
                    break;
                }
            if (!first) continue;
            int cnt = 1;
            for (int j = i + 1; j < hist_len; ++j) cnt += (st->history[j] == tok);
            float v = s_val[tok - base];
            for (int c = 0; c < cnt; ++c) v = (v > 0.f) ? __fdiv_rn(v, penalty) : __fmul_rn(v, penalty);
            s_val[tok - base] = v;
        }
        __syncthreads();
    }

    const bool greedy = (temperature == 0.0f);
    MaxIdx best = {-INFINITY, 0x7fffffff};
    for (int i = tid; i < n; i += kSampleThreads) {
        float v = s_val[i];
        if (!greedy) v = __fdiv_rn(v, temperature);
        s_val[i] = v;
        a.logits[base + i] = v;
        best = better(best, MaxIdx{v, base + i});
    }
    best = block_argmax(best, s_mi, tid);
    float bsum = 0.f;
    if (!greedy) {
        float e = 0.f;
        for (int i = tid; i < n; i += kSampleThreads) e += exp_repro(s_val[i] - best.v);
        bsum = block_sum(e, s_f, tid);
    }
    if (tid == 0) {
        __stcg(a.part_max + blockIdx.x, best.v);
        __stcg(a.part_idx + blockIdx.x, best.i);
        __stcg(a.part_sum + blockIdx.x, bsum);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(a.counter, 1u);
        s_flag = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();

    // ---------------- last block: global decision
    const int nb = gridDim.x;
    MaxIdx g = {-INFINITY, 0x7fffffff};
    for (int b = tid; b < nb; b += kSampleThreads)
        g = better(g, MaxIdx{__ldcg(a.part_max + b), __ldcg(a.part_idx + b)});
    g = block_argmax(g, s_mi, tid);
    int token = g.i;

    if (!greedy) {
        const float r = st->advance ? a.r_values[st->step_idx] : st->r;
        // block partial b scaled to the global maximum: s_b * exp(m_b - M), one thread per block
        // (kSampleMaxBlocks bounds the vocabulary this kernel serves)
        for (int b = tid; b < nb; b += kSampleThreads)
            s_scaled[b] = __ldcg(a.part_sum + b) * exp_repro(__ldcg(a.part_max + b) - g.v);
        __syncthreads();
        // thread 0 walks the blocks in order: Z, then the block in which r*Z is passed
        if (tid == 0) {
            float Z = 0.f;
            for (int b = 0; b < nb; ++b) Z += s_scaled[b];
            const float u = r * Z;
            float c = 0.f;
            int bsel = nb - 1;
            float cprev = 0.f;
            for (int b = 0; b < nb; ++b) {
                const float cn = c + s_scaled[b];
                if (u < cn) {
                    bsel = b;
                    cprev = c;
                    break;
                }
                cprev = c;
                c = cn;
            }
            s_flag = bsel;
            s_f[0] = cprev;
            s_f[1] = u;
            s_found = 0x7fffffff;
        }
        __syncthreads();
        const int bsel = s_flag;
        const float cprev = s_f[0], u = s_f[1];
        __syncthreads();
        const int sb = bsel * kSampleChunk;
        const int sn = min(kSampleChunk, a.vocab - sb);
        // thread t owns elements 4t..4t+3 of the selected block: local prefix, then block scan
        float e[kSamplePerThread];
        float tsum = 0.f;
#pragma unroll
        for (int k = 0; k < kSamplePerThread; ++k) {
            const int i = tid * kSamplePerThread + k;
            e[k] = (i < sn) ? exp_repro(__ldcg(a.logits + sb + i) - g.v) : 0.f;
            tsum += e[k];
        }
        // exclusive scan of tsum over threads: warp scan + warp totals in order
        float incl = tsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, incl, o);
            if ((tid & 31) >= o) incl += y;
        }
        if ((tid & 31) == 31) s_wtot[tid >> 5] = incl;
        __syncthreads();
        float woff = 0.f;
        for (int w = 0; w < (tid >> 5); ++w) woff += s_wtot[w];
        float run = cprev + woff + (incl - tsum);
#pragma unroll
        for (int k = 0; k < kSamplePerThread; ++k) {
            run += e[k];
            const int i = tid * kSamplePerThread + k;
            if (i < sn && u < run) atomicMin(&s_found, sb + i);
        }
        __syncthreads();
        token = (s_found != 0x7fffffff) ? s_found : (sb + sn - 1);
    }

    if (tid == 0) {
        st->out_token = token;
        if (st->advance) {
            const int k = st->step_idx;
            a.out_tokens[k] = token;
            st->token = token;
            st->pos = st->pos + 1;
            st->step_idx = k + 1;
            const int w = st->history_window;
            if (w > 0) {
                // ring of the last w tokens (src/main.cpp:203-208 keeps the same set by shifting)
                st->history[st->history_count % w] = token;
                st->history_count = st->history_count + 1;
                st->history_len = min(st->history_count, w);
            }
        }
        *a.counter = 0u;
    }
    // every kernel of this step has completed: reset the step kernels' grid-barrier counters
    for (int i = tid; i < a.zero_n; i += kSampleThreads) a.zero[i] = 0u;
    if (a.bump && tid == 0) *a.bump = *a.bump + 1u;
}

}  // namespace lpp
