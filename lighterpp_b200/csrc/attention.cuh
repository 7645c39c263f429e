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

constexpr int kAttnThreads = 128;
constexpr int kAttnGroups = kAttnThreads / 8;  // position groups per CTA
constexpr int kAttnMinChunk = 64;              // fewest positions worth a CTA of its own

// Number of KV splits actually used at sequence length T: short contexts use few CTAs (a split
// with a handful of positions costs more in the final combine than it saves), long ones all of
// them.  Every CTA evaluates this identically from the device-resident position.
__host__ __device__ inline int attn_effective_splits(int T, int max_splits) {
    int n = (T + kAttnMinChunk - 1) / kAttnMinChunk;
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

// DPL = head_size / 8 (dims per lane), GB = query heads handled per CTA (divides gqa).
template <typename KT, int DPL, int GB>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnArgs a) {
    constexpr int HS = DPL * 8;
    __shared__ float s_state[kAttnThreads / 32][GB][HS + 2];
    __shared__ int s_last;

    pdl_launch_dependents();  // the next GEMV may start streaming its weights now
    pdl_wait();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sub = lane & 7, grp = warp * 4 + (lane >> 3);
    const int split = blockIdx.x, kvh = blockIdx.y, hz = blockIdx.z;
    const int pos = a.st->pos;
    const int T = (pos < 0 || pos >= a.seq_len) ? 0 : pos + 1;
    const int n_eff = attn_effective_splits(T, a.n_splits);
    if (split >= n_eff) return;  // surplus CTA at this sequence length: no work, no ticket
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
        for (int d = 0; d < DPL; ++d) {
            q[h][d] = __ldcg(a.q + (size_t)(hbase + h) * HS + sub * DPL + d);
            acc[h][d] = 0.f;
        }
    }

    const KT* kbase = reinterpret_cast<const KT*>(a.k_cache) + (size_t)kvh * a.seq_len * HS + sub * DPL;
    const KT* vbase = reinterpret_cast<const KT*>(a.v_cache) + (size_t)kvh * a.seq_len * HS + sub * DPL;

    // Two positions per 8-lane group and iteration, so four independent 16-byte loads are in flight
    // per lane.  The trip count depends only on (t0, t1) and is therefore the same for every lane:
    // the shuffles below need all 32 lanes, so lanes whose position is past the end run the
    // iteration with zeros and are masked out of the softmax update.
    for (int base = t0; base < t1; base += 2 * kAttnGroups) {
        const int ta = base + grp, tb = ta + kAttnGroups;
        const bool has_a = ta < t1, has_b = tb < t1;
        float ka[DPL], va[DPL], kb[DPL], vb[DPL];
        if (has_a) {
            load_row_slice<KT, DPL>(kbase + (size_t)ta * HS, ka);
            load_row_slice<KT, DPL>(vbase + (size_t)ta * HS, va);
        } else {
#pragma unroll
            for (int d = 0; d < DPL; ++d) ka[d] = va[d] = 0.f;
        }
        if (has_b) {
            load_row_slice<KT, DPL>(kbase + (size_t)tb * HS, kb);
            load_row_slice<KT, DPL>(vbase + (size_t)tb * HS, vb);
        } else {
#pragma unroll
            for (int d = 0; d < DPL; ++d) kb[d] = vb[d] = 0.f;
        }
#pragma unroll
        for (int h = 0; h < GB; ++h) {
            float sa = 0.f, sb = 0.f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) {
                sa = fmaf(q[h][d], ka[d], sa);
                sb = fmaf(q[h][d], kb[d], sb);
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                sa += __shfl_xor_sync(0xffffffffu, sa, o);
                sb += __shfl_xor_sync(0xffffffffu, sb, o);
            }
            sa = has_a ? sa * scale : -INFINITY;
            sb = has_b ? sb * scale : -INFINITY;
            const float mn = fmaxf(m[h], fmaxf(sa, sb));
            if (mn != -INFINITY) {  // per-lane predicate; no warp-collective inside
                const float alpha = (m[h] == -INFINITY) ? 0.f : __expf(m[h] - mn);
                const float pa = has_a ? __expf(sa - mn) : 0.f;
                const float pb = has_b ? __expf(sb - mn) : 0.f;
                l[h] = l[h] * alpha + pa + pb;
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[h][d] = fmaf(pb, vb[d], fmaf(pa, va[d], acc[h][d] * alpha));
                m[h] = mn;
            }
        }
    }

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
    __syncthreads();

    // merge the warps; with a single split the result is final, otherwise it is this split's partial
    constexpr int NW = kAttnThreads / 32;
    float* part = a.part;
    const int PS = HS + 2;
    for (int idx = tid; idx < GB * HS; idx += kAttnThreads) {
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
    if (n_eff == 1) return;  // short context: no partials, no ticket, no second pass
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&a.counters[kvh * gridDim.z + hz], 1u);
        s_last = (ticket == (unsigned int)n_eff - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // last CTA of this (kv head, head batch): combine the splits in index order.  Loads are issued
    // in batches of eight before they are consumed so the L2 latency is paid once per batch.
    for (int idx = tid; idx < GB * HS; idx += kAttnThreads) {
        const int h = idx / HS, d = idx % HS;
        const float* p = part + (size_t)(hbase + h) * a.n_splits * PS;
        float mm = -INFINITY;
        for (int s0 = 0; s0 < n_eff; s0 += 8) {
            float ms[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ms[i] = (s0 + i < n_eff) ? __ldcg(p + (size_t)(s0 + i) * PS + HS) : -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) mm = fmaxf(mm, ms[i]);
        }
        float av = 0.f, lv = 0.f;
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
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float f = (ms[i] == -INFINITY) ? 0.f : __expf(ms[i] - mm);
                av = fmaf(as[i], f, av);
                lv = fmaf(ls[i], f, lv);
            }
        }
        a.out[(size_t)(hbase + h) * HS + d] = (lv > 0.f) ? __fdiv_rn(av, lv) : 0.f;
    }
    if (tid == 0) a.counters[kvh * gridDim.z + hz] = 0u;
}

}  // namespace lpp
