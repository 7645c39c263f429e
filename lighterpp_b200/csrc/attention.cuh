// Split-KV GQA flash-decode attention for one query token.
//
// Replaces the reference's four attention kernels -- multihead_gemv_kernel_optimized
// (src/multihead_gemv.cu:6-68), scale_kernel_multihead (src/scale.cu:6-21), softmax_multihead
// (src/softmax.cu:5-125) and aggregation_kernel_multihead (src/aggregation.cu:6-31) -- and the
// att[n_heads][seq_len] buffer they pass through HBM.  Semantics follow the CPU path
// (src/model.cpp:178-199): score = (q.k)*1/sqrt(hs) (scale after the dot product), softmax over
// t = 0..pos, out = sum_t p_t v_t, kv_head = h / (n_heads/n_kv_heads).
//
// Grid (n_splits, kv_heads, gqa/GB).  A CTA owns one KV head, GB of its query heads and one slice
// of the positions 0..pos; K/V rows are read once per CTA straight from global memory with fully
// coalesced 16-byte loads (8 lanes cover one row, 4 rows per warp instruction), so all GB query
// heads share every K/V byte.  Each 8-lane group keeps an online-softmax state (m, l, acc) for its
// positions; states merge across groups, warps and finally across splits by the last CTA to
// finish (ticket counter), in a fixed order, so results do not depend on scheduling.
// HBM traffic: K and V rows 0..pos of the layer once (twice when gqa > 4).
#pragma once
#include "common.cuh"

namespace lpp {

constexpr int kAttnThreads = 128;        // a team inside the persistent step kernel
constexpr int kAttnKernelThreads = 256;  // the stand-alone kernel: 32 position groups, 128 positions in flight
constexpr int kAttnGroups = kAttnThreads / 8;  // position groups per CTA
constexpr int kAttnMinChunk = 128;             // fewest positions worth a CTA of its own

// Number of KV splits actually used at sequence length T: short contexts use few CTAs (a split
// with a handful of positions costs more in the final combine than it saves), long ones all of
// them.  Every CTA evaluates this identically from the device-resident position.
__host__ __device__ inline int attn_effective_splits(int T, int max_splits, int min_chunk = kAttnMinChunk) {
    if (min_chunk < 1) min_chunk = kAttnMinChunk;
    int n = (T + min_chunk - 1) / min_chunk;
    n = n < 1 ? 1 : n;
    return n < max_splits ? n : max_splits;
}

struct AttnArgs {
    const float* q;       // [n_heads_local][head_size]
    const void* k_cache;  // this layer: [kv_heads_local][seq_len][head_size]
    const void* v_cache;
    float* out;           // [n_heads_local][head_size]
    float* part;          // [kv_heads*gqa][n_splits][head_size+2]  (acc..., m, l)
    unsigned int* counters;  // [kv_heads * gqa/GB], zero between launches
    const StepState* st;
    int seq_len, head_size, gqa, n_splits;
    int n_kv_heads;  // KV heads on this rank
    int min_chunk;   // fewest positions per split (0 = kAttnMinChunk)
    unsigned long long* trace;  // timing experiments only: [CTA y*z][8] global-timer stamps of split 0
};

template <typename KT, int DPL>
__device__ __forceinline__ void load_row_slice(const KT* p, float (&dst)[DPL]) {
    if constexpr (sizeof(KT) == 2) {
        if constexpr (DPL % 8 == 0) {
#pragma unroll
            for (int i = 0; i < DPL / 8; ++i) {
                const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p) + i);
                float2 f;
                f = half2_bits_to_float2(u.x); dst[8 * i + 0] = f.x; dst[8 * i + 1] = f.y;
                f = half2_bits_to_float2(u.y); dst[8 * i + 2] = f.x; dst[8 * i + 3] = f.y;
                f = half2_bits_to_float2(u.z); dst[8 * i + 4] = f.x; dst[8 * i + 5] = f.y;
                f = half2_bits_to_float2(u.w); dst[8 * i + 6] = f.x; dst[8 * i + 7] = f.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < DPL / 2; ++i) {
                const unsigned int u = __ldcg(reinterpret_cast<const unsigned int*>(p) + i);
                const float2 f = half2_bits_to_float2(u);
                dst[2 * i] = f.x;
                dst[2 * i + 1] = f.y;
            }
        }
    } else {
        if constexpr (DPL % 4 == 0) {
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 f = __ldcg(reinterpret_cast<const float4*>(p) + i);
                dst[4 * i] = f.x; dst[4 * i + 1] = f.y; dst[4 * i + 2] = f.z; dst[4 * i + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < DPL / 2; ++i) {
                const float2 f = __ldcg(reinterpret_cast<const float2*>(p) + i);
                dst[2 * i] = f.x;
                dst[2 * i + 1] = f.y;
            }
        }
    }
}

// Merge online-softmax state (m2, l2, acc2) into (m, l, acc).
template <int DPL>
__device__ __forceinline__ void merge_state(float& m, float& l, float (&acc)[DPL], float m2, float l2,
                                            const float (&acc2)[DPL]) {
    const float mn = fmaxf(m, m2);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - mn);
    const float b = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
    l = l * a + l2 * b;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[d] = acc[d] * a + acc2[d] * b;
    m = mn;
}

__device__ __forceinline__ void attn_stamp(const AttnArgs& a, int tid, int k) {
    if (a.trace && tid == 0 && blockIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.trace[(size_t)(blockIdx.y * gridDim.z + blockIdx.z) * 8 + k] = t;
    }
}

__device__ __forceinline__ void team_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Second half of a work item.  `scratch` holds one online-softmax state per warp of the team,
// [NT/32][GB][HS+2] floats (HS accumulated values, then the running maximum and the running sum); the team
// has passed a barrier since they were written.  Merges them, writes the result (one split) or this
// split's partial, and lets the last team of the (kv head, head batch) combine the partials.
template <int HS, int GB, int NT>
__device__ __forceinline__ void attn_merge_and_combine(const AttnArgs& a, float* scratch, int split, int kvh, int hz, int n_z,
                                                       int n_eff, int* s_last, int tid, int bar) {
    float (*s_state)[GB][HS + 2] = reinterpret_cast<float (*)[GB][HS + 2]>(scratch);
    const int hbase = kvh * a.gqa + hz * GB;
    // merge the warps; with a single split the result is final, otherwise it is this split's partial
    constexpr int NW = NT / 32;
    float* part = a.part;
    const int PS = HS + 2;
    for (int idx = tid; idx < GB * HS; idx += NT) {
        const int h = idx / HS, d = idx % HS;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) mm = fmaxf(mm, s_state[w][h][HS]);
        float av = 0.f, lv = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = s_state[w][h][HS];
            const float f = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
            av += s_state[w][h][d] * f;
            lv += s_state[w][h][HS + 1] * f;
        }
        if (n_eff == 1) {
            a.out[(size_t)(hbase + h) * HS + d] = (lv > 0.f) ? __fdiv_rn(av, lv) : 0.f;
        } else {
            float* p = part + ((size_t)(hbase + h) * a.n_splits + split) * PS;
            __stcg(p + d, av);
            if (d == 0) {
                __stcg(p + HS, mm);
                __stcg(p + HS + 1, lv);
            }
        }
    }
    if (n_eff == 1) {
        team_barrier(bar, NT);  // scratch may be reused by the team's next item
        return;  // short context: no partials, no ticket, no second pass
    }
    __threadfence();
    team_barrier(bar, NT);
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&a.counters[kvh * n_z + hz], 1u);
        *s_last = (ticket == (unsigned int)n_eff - 1);
    }
    team_barrier(bar, NT);
    if (!*s_last) return;
    __threadfence();

    // last team of this (kv head, head batch): combine the splits in index order.  Loads are issued
    // in batches of eight before they are consumed; up to eight splits need a single round trip.
    for (int idx = tid; idx < GB * HS; idx += NT) {
        const int h = idx / HS, d = idx % HS;
        const float* p = part + (size_t)(hbase + h) * a.n_splits * PS;
        float mm = -INFINITY, av = 0.f, lv = 0.f;
        for (int s0 = 0; s0 < n_eff; s0 += 8) {
            float ms[8], ls[8], as[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool ok = s0 + i < n_eff;
                const float* ps = p + (size_t)(s0 + i) * PS;
                ms[i] = ok ? __ldcg(ps + HS) : -INFINITY;
                ls[i] = ok ? __ldcg(ps + HS + 1) : 0.f;
                as[i] = ok ? __ldcg(ps + d) : 0.f;
            }
            float mb = mm;
#pragma unroll
            for (int i = 0; i < 8; ++i) mb = fmaxf(mb, ms[i]);
            // rescale what has been accumulated so far to the new running maximum (fixed order)
            const float fo = (mm == -INFINITY) ? 0.f : __expf(mm - mb);
            av *= fo;
            lv *= fo;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float f = (ms[i] == -INFINITY) ? 0.f : __expf(ms[i] - mb);
                av = fmaf(as[i], f, av);
                lv = fmaf(ls[i], f, lv);
            }
            mm = mb;
        }
        a.out[(size_t)(hbase + h) * HS + d] = (lv > 0.f) ? __fdiv_rn(av, lv) : 0.f;
    }
    if (tid == 0) a.counters[kvh * n_z + hz] = 0u;
}

// One work item = (split, kv head, batch hz of GB query heads) at sequence length T with n_eff
// splits in use, executed by a team of 128 threads (tid 0..127) that synchronise on named barrier
// `bar`.  `scratch` holds [NT/32 warps][GB][HS+2] floats of shared memory, `s_last` one int.
// DPL = head_size / 8 (dims per lane), GB = query heads per item (divides gqa), n_z = gqa / GB,
// NT = threads in the team (128 for the stand-alone kernel, 256 when a GEMV CTA's consumers run it).
template <typename KT, int DPL, int GB, int NT = kAttnThreads>
__device__ __forceinline__ void attn_item(const AttnArgs& a, int split, int kvh, int hz, int n_z, int T, int n_eff,
                                          float* scratch, int* s_last, int tid, int bar, int pos_cur) {
    constexpr int HS = DPL * 8;
    float (*s_state)[GB][HS + 2] = reinterpret_cast<float (*)[GB][HS + 2]>(scratch);
    const int warp = tid >> 5, lane = tid & 31;
    const int sub = lane & 7, grp = warp * 4 + (lane >> 3);
    const int chunk = (T + n_eff - 1) / n_eff;
    const int t0 = split * chunk;
    const int t1 = min(T, t0 + chunk);
    const int hbase = kvh * a.gqa + hz * GB;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)HS));

    float q[GB][DPL], acc[GB][DPL], m[GB], l[GB];
#pragma unroll
    for (int h = 0; h < GB; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
    }
    // Rows of positions before `pos_cur` were written by earlier steps and are requested before the
    // dependency wait; q and the row of pos_cur come from the preceding kernel and follow it.
    bool waited = false;
    auto wait_and_load_q = [&]() {
        pdl_wait();
        attn_stamp(a, tid, 1);
#pragma unroll
        for (int h = 0; h < GB; ++h) {
            const float* qp = a.q + (size_t)(hbase + h) * HS + sub * DPL;
            if constexpr (DPL % 4 == 0) {
#pragma unroll
                for (int d = 0; d < DPL; d += 4) {
                    const float4 f = __ldcg(reinterpret_cast<const float4*>(qp + d));
                    q[h][d] = f.x; q[h][d + 1] = f.y; q[h][d + 2] = f.z; q[h][d + 3] = f.w;
                }
            } else {
#pragma unroll
                for (int d = 0; d < DPL; d += 2) {
                    const float2 f = __ldcg(reinterpret_cast<const float2*>(qp + d));
                    q[h][d] = f.x; q[h][d + 1] = f.y;
                }
            }
        }
        waited = true;
    };

    const KT* kbase = reinterpret_cast<const KT*>(a.k_cache) + (size_t)kvh * a.seq_len * HS + sub * DPL;
    const KT* vbase = reinterpret_cast<const KT*>(a.v_cache) + (size_t)kvh * a.seq_len * HS + sub * DPL;

    // U positions per 8-lane group and iteration: all their K and V loads (2*U independent 16-byte
    // loads per lane) are issued before any is used, so a chunk of up to U*16 positions costs one
    // memory round trip.  The trip count depends only on (t0, t1) and is therefore the same for every
    // lane: the shuffles below need all 32 lanes, so lanes whose position is past the end run the
    // iteration with zeros and are masked out of the softmax update.
    constexpr int U = (DPL <= 8) ? 4 : 2;
    for (int base = t0; base < t1; base += U * (NT / 8)) {
        float kk[U][DPL], vv[U][DPL];
        bool has[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = base + u * (NT / 8) + grp;
            has[u] = t < t1;
            if (has[u] && t < pos_cur) {
                load_row_slice<KT, DPL>(kbase + (size_t)t * HS, kk[u]);
                load_row_slice<KT, DPL>(vbase + (size_t)t * HS, vv[u]);
            } else {
#pragma unroll
                for (int d = 0; d < DPL; ++d) kk[u][d] = vv[u][d] = 0.f;
            }
        }
        if (!waited) wait_and_load_q();
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = base + u * (NT / 8) + grp;
            if (has[u] && t >= pos_cur) {
                load_row_slice<KT, DPL>(kbase + (size_t)t * HS, kk[u]);
                load_row_slice<KT, DPL>(vbase + (size_t)t * HS, vv[u]);
            }
        }
#pragma unroll
        for (int h = 0; h < GB; ++h) {
            float sc[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float x = 0.f;
#pragma unroll
                for (int d = 0; d < DPL; ++d) x = fmaf(q[h][d], kk[u][d], x);
                sc[u] = x;
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
                for (int u = 0; u < U; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
            }
            float mn = m[h];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                sc[u] = has[u] ? sc[u] * scale : -INFINITY;
                mn = fmaxf(mn, sc[u]);
            }
            if (mn != -INFINITY) {  // per-lane predicate; no warp-collective inside
                const float alpha = (m[h] == -INFINITY) ? 0.f : __expf(m[h] - mn);
                float pu[U], ls = 0.f;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    pu[u] = has[u] ? __expf(sc[u] - mn) : 0.f;
                    ls += pu[u];
                }
                l[h] = l[h] * alpha + ls;
#pragma unroll
                for (int d = 0; d < DPL; ++d) {
                    float x = acc[h][d] * alpha;
#pragma unroll
                    for (int u = 0; u < U; ++u) x = fmaf(pu[u], vv[u][d], x);
                    acc[h][d] = x;
                }
                m[h] = mn;
            }
        }
    }

    if (!waited) wait_and_load_q();
    attn_stamp(a, tid, 2);
    // merge the four position groups of a warp (lanes differing in bits 3 and 4)
#pragma unroll
    for (int h = 0; h < GB; ++h) {
#pragma unroll
        for (int o = 8; o < 32; o <<= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m[h], o);
            const float l2 = __shfl_xor_sync(0xffffffffu, l[h], o);
            float acc2[DPL];
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc2[d] = __shfl_xor_sync(0xffffffffu, acc[h][d], o);
            merge_state<DPL>(m[h], l[h], acc[h], m2, l2, acc2);
        }
        if (lane < 8) {
#pragma unroll
            for (int d = 0; d < DPL; ++d) s_state[warp][h][sub * DPL + d] = acc[h][d];
            if (sub == 0) {
                s_state[warp][h][HS] = m[h];
                s_state[warp][h][HS + 1] = l[h];
            }
        }
    }
    team_barrier(bar, NT);
    attn_stamp(a, tid, 3);

    attn_merge_and_combine<HS, GB, NT>(a, scratch, split, kvh, hz, n_z, n_eff, s_last, tid, bar);
}

template <typename KT, int DPL, int GB>
__global__ void __launch_bounds__(kAttnKernelThreads) attn_decode_kernel(const AttnArgs a) {
    __shared__ float s_scratch[(kAttnKernelThreads / 32) * GB * (DPL * 8 + 2)];
    __shared__ int s_last;
    auto stamp = [&](int k) {
        if (a.trace && threadIdx.x == 0 && blockIdx.x == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            a.trace[(size_t)(blockIdx.y * gridDim.z + blockIdx.z) * 8 + k] = t;
        }
    };
    stamp(0);
    pdl_launch_dependents();  // the next GEMV may start streaming its weights now
    // The position was written by the previous step's sampler, which completed before this step began,
    // and the cache rows of earlier positions by earlier steps: both may be touched before the wait.
    const int pos = a.st->pos;
    const int T = (pos < 0 || pos >= a.seq_len) ? 0 : pos + 1;
    const int n_eff = attn_effective_splits(T, a.n_splits, a.min_chunk);
    if ((int)blockIdx.x >= n_eff) return;  // surplus CTA at this sequence length: no work, no ticket
    {
        // pull this CTA's share of the K and V rows of positions < pos towards L2 while the QKV kernel
        // is still running; only q and the row of position pos are read after the wait
        constexpr int HS = DPL * 8;
        constexpr int kLines = (HS * (int)sizeof(KT) + 127) / 128;  // 128-byte lines per row (<= 4)
        const int chunk = (T + n_eff - 1) / n_eff;
        const int t0 = blockIdx.x * chunk;
        const int t1 = min(min(T, t0 + chunk), pos);
        const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
        const char* base = reinterpret_cast<const char*>(sub < 4 ? a.k_cache : a.v_cache) +
                           (size_t)blockIdx.y * a.seq_len * HS * sizeof(KT) + (size_t)(sub & 3) * 128;
        if ((sub & 3) < kLines)
            for (int t = t0 + grp; t < t1; t += kAttnKernelThreads / 8)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (size_t)t * HS * sizeof(KT)));
    }
    attn_item<KT, DPL, GB, kAttnKernelThreads>(a, blockIdx.x, blockIdx.y, blockIdx.z, gridDim.z, T, n_eff, s_scratch, &s_last,
                                               threadIdx.x, 0, pos);
    stamp(4);
}

// ------------------------------------------------------------------ tensor-core variant (FP16 cache)
//
// The kernel above spends its time in FP32 shuffles and exponentials (1.7 TB/s at 32 K positions, and
// slower than this one from a few dozen positions on).  Here the scores q.K^T and the product P.V run
// as mma.sync.m16n8k16 (FP16 operands, FP32 accumulators): the up to 8 query heads of a KV head are the
// rows of the 16-row operand (the rest is zero), a warp handles 16 positions per step and keeps the rows
// of its next step in flight.  No shared memory is involved in the operands: the dot product over head
// dimensions and the sum over positions do not care about order, so the dimension / position that an
// operand register stands for is chosen such that every lane reads whole 16-byte pieces of the rows
// straight from global memory (a quad of lanes covers one K row; lane quad-row g owns head dims
// [g*HS/8, (g+1)*HS/8) of its V rows).  Same splits, partials and combine as above.  As there, the
// position and the rows of earlier positions are read before the dependency wait.
__device__ __forceinline__ void mma_16816(float (&d)[4], unsigned int a0, unsigned int a1, unsigned int a2, unsigned int a3,
                                          unsigned int b0, unsigned int b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned int pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned int*>(&h);
}

constexpr int kAttnPrefetchSteps = 1;  // how many steps past the next one the L2 prefetch runs ahead

template <int HS, int GQA>
__global__ void __launch_bounds__(kAttnKernelThreads) attn_mma_kernel(const AttnArgs a) {
    static_assert(HS == 64 || HS == 128, "head size");
    static_assert(GQA >= 1 && GQA <= 8, "query heads per KV head");
    constexpr int NT = kAttnKernelThreads, NW = NT / 32;
    constexpr int KS = HS / 16;   // k-steps of the score product; a lane owns HS/4 dims of its K row = 2*KS registers
    constexpr int NTL = HS / 8;   // n-tiles of the output; a lane owns NTL dims of its V rows = NTL/2 registers
    __shared__ float s_scratch[NW * GQA * (HS + 2)];
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, j = lane & 3;
    pdl_launch_dependents();
    // the position was written by the previous step's sampler, which completed before this step began
    const int pos = a.st->pos;
    const int T = (pos < 0 || pos >= a.seq_len) ? 0 : pos + 1;
    // one CTA per KV head up to two chunks of positions: below that a second split costs more in the
    // combine (partials, ticket, second pass) than it saves (measured: 602 against 620 us/token at 180-243)
    const int min_chunk = a.min_chunk > 0 ? a.min_chunk : kAttnMinChunk;
    const int n_eff = (T <= 2 * min_chunk) ? 1 : attn_effective_splits(T, a.n_splits, min_chunk);
    const int split = blockIdx.x, kvh = blockIdx.y;
    if (split >= n_eff) return;
    const int chunk = (T + n_eff - 1) / n_eff;
    const int t0 = split * chunk;
    const int t1 = min(T, t0 + chunk);
    const __half* kb = reinterpret_cast<const __half*>(a.k_cache) + (size_t)kvh * a.seq_len * HS;
    const __half* vb = reinterpret_cast<const __half*>(a.v_cache) + (size_t)kvh * a.seq_len * HS;
    const int hbase = kvh * a.gqa;

    float o[NTL][4];
#pragma unroll
    for (int t = 0; t < NTL; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
    float m = -INFINITY, l = 0.f;  // running maximum / sum of head g (identical on the 4 lanes of a quad)

    // K rows of one step: group 0 = positions base..base+7, group 1 = base+8..base+15; this lane reads the
    // piece [j*HS/4, (j+1)*HS/4) of the rows base+g and base+8+g
    auto load_k = [&](int base, unsigned int (&kr)[2][2 * KS], int lim) {
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            const int t = base + grp * 8 + g;
            if (t < lim) {
                const uint4* p = reinterpret_cast<const uint4*>(kb + (size_t)t * HS + j * (HS / 4));
#pragma unroll
                for (int i = 0; i < KS / 2; ++i) {
                    const uint4 u = __ldcg(p + i);
                    kr[grp][4 * i] = u.x; kr[grp][4 * i + 1] = u.y; kr[grp][4 * i + 2] = u.z; kr[grp][4 * i + 3] = u.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 2 * KS; ++i) kr[grp][i] = 0u;
            }
        }
    };
    // V rows of one step: positions base+2j, base+2j+1, base+8+2j, base+8+2j+1 (the order in which the
    // probabilities sit in the A operand below), head dims [g*NTL, (g+1)*NTL)
    auto load_v = [&](int base, unsigned int (&vr)[4][NTL / 2], int lim) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int t = base + (r >> 1) * 8 + 2 * j + (r & 1);
            if (t < lim) {
                const uint4* p = reinterpret_cast<const uint4*>(vb + (size_t)t * HS + g * NTL);
#pragma unroll
                for (int i = 0; i < NTL / 8; ++i) {
                    const uint4 u = __ldcg(p + i);
                    vr[r][4 * i] = u.x; vr[r][4 * i + 1] = u.y; vr[r][4 * i + 2] = u.z; vr[r][4 * i + 3] = u.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < NTL / 2; ++i) vr[r][i] = 0u;
            }
        }
    };
    unsigned int kr[2][2 * KS], vr[4][NTL / 2];
    int base = t0 + warp * 16;
    // first step: rows of earlier positions (written by earlier steps) are requested before the wait; the
    // row of the current position, like q, comes from the QKV kernel of this step and follows it
    const int stable = min(t1, pos);
    if (base < t1) {
        load_k(base, kr, stable);
        load_v(base, vr, stable);
    }
    pdl_wait();
    // A operand of the score product: row g = head g (zero from GQA on), this lane's HS/4 dims, pre-scaled
    unsigned int qa[KS][2];
    {
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)HS));
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < GQA) v = __ldcg(reinterpret_cast<const float4*>(a.q + (size_t)(hbase + g) * HS + j * (HS / 4) + 4 * s));
            qa[s][0] = pack_half2(v.x * scale, v.y * scale);
            qa[s][1] = pack_half2(v.z * scale, v.w * scale);
        }
    }
    if (pos < t1 && pos >= base && pos < base + 16) {
#pragma unroll
        for (int grp = 0; grp < 2; ++grp)
            if (base + grp * 8 + g == pos) {
                const uint4* p = reinterpret_cast<const uint4*>(kb + (size_t)pos * HS + j * (HS / 4));
#pragma unroll
                for (int i = 0; i < KS / 2; ++i) {
                    const uint4 u = __ldcg(p + i);
                    kr[grp][4 * i] = u.x; kr[grp][4 * i + 1] = u.y; kr[grp][4 * i + 2] = u.z; kr[grp][4 * i + 3] = u.w;
                }
            }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (base + (r >> 1) * 8 + 2 * j + (r & 1) == pos) {
                const uint4* p = reinterpret_cast<const uint4*>(vb + (size_t)pos * HS + g * NTL);
#pragma unroll
                for (int i = 0; i < NTL / 8; ++i) {
                    const uint4 u = __ldcg(p + i);
                    vr[r][4 * i] = u.x; vr[r][4 * i + 1] = u.y; vr[r][4 * i + 2] = u.z; vr[r][4 * i + 3] = u.w;
                }
            }
    }
    for (; base < t1; base += NW * 16) {
        // the rows of this warp's next step are requested before this step is computed
        unsigned int krn[2][2 * KS], vrn[4][NTL / 2];
        const int nbase = base + NW * 16;
        if (nbase < t1) {
            load_k(nbase, krn, t1);
            load_v(nbase, vrn, t1);
        }
        // the rows of the step after that are pulled towards L2 (no registers to hold them yet), so that
        // their loads, one iteration from now, take an L2 round trip instead of an HBM one
        {
            const int pbase = nbase + kAttnPrefetchSteps * NW * 16;
#pragma unroll
            for (int grp = 0; grp < 2; ++grp)
                if (pbase + grp * 8 + g < t1)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(kb + (size_t)(pbase + grp * 8 + g) * HS + j * (HS / 4)));
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (pbase + (r >> 1) * 8 + 2 * j + (r & 1) < t1)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(vb + (size_t)(pbase + (r >> 1) * 8 + 2 * j + (r & 1)) * HS + g * NTL));
        }
        // scores of the two groups
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            mma_16816(s0, qa[s][0], 0u, qa[s][1], 0u, kr[0][2 * s], kr[0][2 * s + 1]);
            mma_16816(s1, qa[s][0], 0u, qa[s][1], 0u, kr[1][2 * s], kr[1][2 * s + 1]);
        }
        // row g of s0 / s1: positions base+2j, base+2j+1 / base+8+2j, base+8+2j+1
        float sc[4] = {s0[0], s0[1], s1[0], s1[1]};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = base + (i >> 1) * 8 + 2 * j + (i & 1);
            if (t >= t1) sc[i] = -INFINITY;
        }
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m, mx);  // finite: position `base` is valid for every row
        const float alpha = (m == -INFINITY) ? 0.f : __expf(m - mn);
        float p[4], ps = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            p[i] = (sc[i] == -INFINITY) ? 0.f : __expf(sc[i] - mn);
            ps += p[i];
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l = l * alpha + ps;
        m = mn;
        const unsigned int pa0 = pack_half2(p[0], p[1]), pa2 = pack_half2(p[2], p[3]);
#pragma unroll
        for (int t = 0; t < NTL; ++t) {
            o[t][0] *= alpha;
            o[t][1] *= alpha;
            // B operand of n-tile t: column g = head dim g*NTL + t, rows = the four positions above
            const unsigned int sel = (t & 1) ? 0x7632u : 0x5410u;
            const unsigned int b0 = __byte_perm(vr[0][t >> 1], vr[1][t >> 1], sel);
            const unsigned int b1 = __byte_perm(vr[2][t >> 1], vr[3][t >> 1], sel);
            mma_16816(o[t], pa0, 0u, pa2, 0u, b0, b1);
        }
        if (nbase < t1) {
#pragma unroll
            for (int i = 0; i < 2 * KS; ++i) kr[0][i] = krn[0][i], kr[1][i] = krn[1][i];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < NTL / 2; ++i) vr[r][i] = vrn[r][i];
        }
    }
    // this warp's state: row g of n-tile t, columns 2j and 2j+1 = head dims (2j)*NTL + t and (2j+1)*NTL + t
    float (*s_state)[GQA][HS + 2] = reinterpret_cast<float (*)[GQA][HS + 2]>(s_scratch);
    if (g < GQA) {
#pragma unroll
        for (int t = 0; t < NTL; ++t) {
            s_state[warp][g][(2 * j) * NTL + t] = o[t][0];
            s_state[warp][g][(2 * j + 1) * NTL + t] = o[t][1];
        }
        if (j == 0) {
            s_state[warp][g][HS] = m;
            s_state[warp][g][HS + 1] = l;
        }
    }
    __syncthreads();
    attn_merge_and_combine<HS, GQA, NT>(a, s_scratch, split, kvh, 0, 1, n_eff, &s_last, tid, 0);
}

}  // namespace lpp
