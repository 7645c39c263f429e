// Batched prompt path ("prefill"): the K/V cache rows of up to kPrefillTokens prompt positions in one pass over
// the weights, instead of one pass per token.
//
// The reference feeds a prompt through forward() token by token (src/main.cpp:163-179): every prompt token
// streams all weights once.  Here the layer's matrices are streamed ONCE for the whole block of tokens: the
// four projections become small GEMMs  C[tokens][rows] = X[tokens][K] . W[rows][K]^T  that are still bound by
// the weight stream (2 FLOP per weight byte and token: far below the tensor cores' ridge for a few dozen
// tokens), so the kernel is organised around that stream exactly like the decode GEMV -- a producer warp,
// a ring of shared-memory stages, mbarrier hand-over -- only that a stage is a set of 2-D tiles fetched by the
// tensor memory accelerator (cp.async.bulk.tensor.2d with the 128-byte swizzle: 32 or 64 weight rows x 128 inputs
// and the matching 64 tokens x 128 inputs of the activations) and the arithmetic is warp-level tensor-core MMA
// (ldmatrix + m16n8k16, FP16 operands, FP32 accumulation).  The two matrices with few rows and a plain residual
// epilogue (o_proj, down) are also cut along K so that every SM streams a share; their partial sums are added to
// the residual stream in a fixed order by the next kernel.  Activations are rounded to FP16 as MMA operands; everything between the GEMMs (residual
// stream, RMSNorm, RoPE, softmax) stays FP32, following src/ops.cpp like the decode path.
//
// Tensor maps cover this GPU's own memory only; no cluster multicast is used anywhere.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace lpp {

constexpr int kPrefillTokens = 64;   // tokens per pass (rows of the activation tiles)
constexpr int kPfKc = 128;           // inputs per stage: two 64-wide (128-byte) swizzled sub-tiles per operand
constexpr int kPfConsumerWarps = 8;
constexpr int kPfThreads = (kPfConsumerWarps + 1) * 32;
constexpr int kPfSubBytesX = kPrefillTokens * 128;  // one activation sub-tile: 64 tokens x 64 inputs
constexpr int kPfMaxSplits = 8;
constexpr int kPfRingBytes = 192 * 1024;
constexpr int kPfSmemBytes = 1024 /*barriers*/ + 1024 /*alignment slack*/ + kPfRingBytes;
template <int M>
struct PfGeom {
    static constexpr int kSubW = M * 128;                         // one weight sub-tile: M rows x 64 inputs
    static constexpr int kStage = 2 * kSubW + 2 * kPfSubBytesX;   // 32 KiB (M = 64) / 24 KiB (M = 32)
    static constexpr int kStages = kPfRingBytes / kStage;         // 6 / 8
    static constexpr int kRowTiles = M / 16;                      // 16-row MMA tiles per CTA tile
    static constexpr int kTokGroups = kPfConsumerWarps / kRowTiles;
    static constexpr int kTokPerWarp = kPrefillTokens / kTokGroups;  // 32 / 16
    static constexpr int kNT = kTokPerWarp / 8;                   // 8-token MMA tiles per warp
};

enum PfEpi : int { kPfQkv = 0, kPfResid = 1, kPfSwiglu = 2 };

struct PrefillGemmArgs {
    int n_rows, K;        // rows of the weight matrix, inputs per row
    int row0;             // first row of this layer's matrix inside the tensor map (layers are stacked)
    int n_tokens;         // valid tokens (<= kPrefillTokens)
    int start_pos;        // position of token 0
    int epi;
    int splits;           // K is cut into this many ranges (kPfResid only when > 1): work item = (row tile, range)
    StepState* st;
    // kPfResid: x[t][row] += c (x: [kPrefillTokens][n_rows] FP32) when splits == 1; else the partial sums go to
    // part[split][t][row] and the next kernel (prefill_norm_kernel) adds them to x in split order
    float* x;
    float* part;
    // kPfSwiglu: hb[t][row/2] = silu(gate) * up   (rows interleaved gate, up; hb: FP16 [kPrefillTokens][n_rows/2])
    __half* hb;
    // kPfQkv: rows are q | k | v; RoPE on q and k, q -> FP32 [kPrefillTokens][q_rows], k/v -> cache at start_pos + t
    float* q;
    int q_rows, kv_rows, head_size, seq_len;
    const float2* rope;   // [seq_len][head_size/2]
    __half* k_cache;      // this layer: [kv_heads][seq_len][head_size]
    __half* v_cache;
};

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_dst),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// Address of 16-byte chunk `chunk` (0..7) of row `row` in a sub-tile written by the tensor memory accelerator with
// the 128-byte swizzle (rows of 128 bytes, chunk index XOR row % 8; the sub-tile starts on a 1024-byte boundary).
__device__ __forceinline__ uint32_t swz(uint32_t base, int row, int chunk) {
    return base + (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// One value of the finished tile: row `row` (and its pair partner `other`, the value of row ^ 1), token t.
__device__ __forceinline__ void pf_epilogue(const PrefillGemmArgs& a, int split, int row, int t, float v, float other) {
    if (row >= a.n_rows || t >= a.n_tokens) return;
    if (a.epi == kPfResid) {
        if (a.splits > 1) {
            a.part[((size_t)split * kPrefillTokens + t) * a.n_rows + row] = v;
        } else {
            float* p = a.x + (size_t)t * a.n_rows + row;
            *p = *p + v;  // x += W.xb (src/model.cpp:232, 239)
        }
    } else if (a.epi == kPfSwiglu) {
        // rows are interleaved (gate_i, up_i); hb = (h1*sigmoid(h1))*h3 (src/ops.cpp:78-87): the even row writes
        if ((row & 1) == 0) {
            const float sig = __fdiv_rn(1.0f, 1.0f + expf(-v));
            a.hb[(size_t)t * (a.n_rows >> 1) + (row >> 1)] = __float2half_rn(__fmul_rn(__fmul_rn(v, sig), other));
        }
    } else {  // kPfQkv
        const int pos = a.start_pos + t;
        if (pos < 0 || pos >= a.seq_len) {
            atomicOr(&a.st->status, kStatusBadPos);
            return;
        }
        const int hs = a.head_size;
        float r = v;
        if (row < a.q_rows + a.kv_rows) {
            // adjacent-pair rotation with the table entry for (pos, (row % hs)/2) (src/ops.cpp:34-54)
            const float2 cs = __ldg(a.rope + (size_t)pos * (hs >> 1) + ((row % hs) >> 1));
            r = (row & 1) ? __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(v, cs.x))   // v1' = v0*sin + v1*cos
                          : __fsub_rn(__fmul_rn(v, cs.x), __fmul_rn(other, cs.y));  // v0' = v0*cos - v1*sin
        }
        if (row < a.q_rows) {
            a.q[(size_t)t * a.q_rows + row] = r;
        } else {
            const bool is_k = row < a.q_rows + a.kv_rows;
            const int rr = row - a.q_rows - (is_k ? 0 : a.kv_rows);
            const int h = rr / hs, off = rr % hs;
            // cache index within the layer: h*(seq_len*hs) + pos*hs + off (src/scatter_kv.cu:15-16)
            const size_t idx = (size_t)h * ((size_t)a.seq_len * hs) + (size_t)pos * hs + off;
            (is_k ? a.k_cache : a.v_cache)[idx] = __float2half_rn(r);
        }
    }
}

// C[t][row] = sum_k X[t][k] * W[row][k] for t < 64, fused with the epilogue.  A work item is (tile of M rows, K
// range); CTA b takes items b, b + grid, ...; the ring runs across item boundaries.  M = 32 for the matrices with
// few rows per SM and an epilogue that needs the whole sum (QKV), 64 otherwise.
template <int M>
static __global__ void __launch_bounds__(kPfThreads) prefill_gemm_kernel(const __grid_constant__ CUtensorMap w_map,
                                                                          const __grid_constant__ CUtensorMap x_map,
                                                                          const PrefillGemmArgs a) {
    using G = PfGeom<M>;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // [kStages]
    uint64_t* empty = full + G::kStages;                 // [kStages]
    const uint32_t ring = (smem_u32(smem) + 1024u + 1023u) & ~1023u;  // swizzled sub-tiles start on 1024-byte boundaries
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = (a.n_rows + M - 1) / M;
    const int n_kc = (a.K + kPfKc - 1) / kPfKc;
    const int S = a.splits;
    const int n_items = n_tiles * S;
    pdl_launch_dependents();
    if (tid < G::kStages) {
        mbar_init(&full[tid], 1);
        mbar_init(&empty[tid], kPfConsumerWarps);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == kPfConsumerWarps) {
        // ---------------- producer: one lane issues the four sub-tile copies of every stage
        if (lane == 0) {
            pdl_wait();  // the activation tile comes from the previous kernel (the weights do not, but share the stage)
            int slot = 0, pass = 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
                const int tile = item / S, split = item - tile * S;
                const int kc0 = (split * n_kc) / S, kc1 = ((split + 1) * n_kc) / S;
                for (int kc = kc0; kc < kc1; ++kc) {
                    if (pass > 0 && !mbar_wait_bounded(&empty[slot], (uint32_t)(pass - 1) & 1u, a.st)) return;
                    const uint32_t dst = ring + (uint32_t)slot * G::kStage;
                    mbar_arrive_expect_tx(&full[slot], G::kStage);
                    tma_load_2d(dst, &w_map, kc * kPfKc, a.row0 + tile * M, &full[slot]);
                    tma_load_2d(dst + G::kSubW, &w_map, kc * kPfKc + 64, a.row0 + tile * M, &full[slot]);
                    tma_load_2d(dst + 2 * G::kSubW, &x_map, kc * kPfKc, 0, &full[slot]);
                    tma_load_2d(dst + 2 * G::kSubW + kPfSubBytesX, &x_map, kc * kPfKc + 64, 0, &full[slot]);
                    if (++slot == G::kStages) {
                        slot = 0;
                        ++pass;
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers: warp = (16-row tile rt of the CTA tile, token group tg)
    const int rt = warp % G::kRowTiles, tg = warp / G::kRowTiles;
    const int g = lane >> 2, j = lane & 3;
    // ldmatrix source rows of this lane.  A (x4): matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15),
    // (rows 8-15, k 8-15) = a0..a3.  B (x4): (tokens 0-7, k 0-7), (tokens 0-7, k 8-15), (tokens 8-15, k 0-7),
    // (tokens 8-15, k 8-15) = b0, b1 of two 8-token tiles.
    const int a_row = rt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_chunk = lane >> 4;
    const int b_row = tg * G::kTokPerWarp + (lane & 7) + ((lane >> 4) & 1) * 8, b_chunk = (lane >> 3) & 1;
    int slot = 0;
    uint32_t par = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int tile = item / S, split = item - tile * S;
        const int kc0 = (split * n_kc) / S, kc1 = ((split + 1) * n_kc) / S;
        float acc[G::kNT][4];
#pragma unroll
        for (int nt = 0; nt < G::kNT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        for (int kc = kc0; kc < kc1; ++kc) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full[slot], par, a.st))) return;
            const uint32_t st = ring + (uint32_t)slot * G::kStage;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                const uint32_t wt = st + sub * G::kSubW, xt = st + 2 * G::kSubW + sub * kPfSubBytesX;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {  // four 16-input steps per 64-wide sub-tile
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(swz(wt, a_row, 2 * ks + a_chunk), a0, a1, a2, a3);
#pragma unroll
                    for (int np = 0; np < G::kNT / 2; ++np) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(swz(xt, b_row + np * 16, 2 * ks + b_chunk), b0, b1, b2, b3);
                        mma_f16_16816(acc[2 * np], a0, a1, a2, a3, b0, b1);
                        mma_f16_16816(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
            if (++slot == G::kStages) {
                slot = 0;
                par ^= 1u;
            }
        }
        // acc[nt]: rows g (c0, c1) and g + 8 (c2, c3), tokens tg*kTokPerWarp + nt*8 + 2j (c0, c2) and + 1 (c1, c3)
        const int row_lo = tile * M + rt * 16 + g;
#pragma unroll
        for (int nt = 0; nt < G::kNT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float v = acc[nt][c];
                const float other = __shfl_xor_sync(0xffffffffu, v, 4);  // the same token, row g ^ 1
                pf_epilogue(a, split, row_lo + (c >> 1) * 8, tg * G::kTokPerWarp + nt * 8 + 2 * j + (c & 1), v, other);
            }
    }
}

// Rows of the residual stream -> RMS-normalised FP16 rows (MMA operands).  Layer 0 takes the embedding rows of
// the prompt tokens and also writes them out as the FP32 residual stream.  grid: tokens.
static __global__ void __launch_bounds__(256) prefill_norm_kernel(float* x, const int* tokens, const __half* emb, int vocab,
                                                                  const float* norm_w, __half* out, int D, int n_tokens,
                                                                  const float* part, int splits, StepState* st) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    float* xr = x + (size_t)t * D;
    if (emb) {
        int tok = tokens[t];
        if (tok < 0 || tok >= vocab) {
            if (threadIdx.x == 0) atomicOr(&st->status, kStatusBadToken);
            tok = 0;
        }
        const __half* er = emb + (size_t)tok * D;
        for (int i = threadIdx.x; i < D; i += 256) xr[i] = __half2float(er[i]);
    } else if (splits > 1) {
        // the preceding residual GEMM left its K-range partial sums: x += p_0 + p_1 + ... in range order
        for (int i = threadIdx.x; i < D; i += 256) {
            float v = xr[i];
            for (int s = 0; s < splits; ++s) v += part[((size_t)s * kPrefillTokens + t) * D + i];
            xr[i] = v;
        }
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += 256) ss = fmaf(xr[i], xr[i], ss);  // every thread reads back what it wrote
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += red[k];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)D), 1e-5f)));
    for (int i = threadIdx.x; i < D; i += 256) out[(size_t)t * D + i] = __float2half_rn(__fmul_rn(__fmul_rn(xr[i], scale), norm_w[i]));
}

// Causal attention of the prompt block: query token t (position start_pos + t) over cache rows 0..start_pos + t,
// scores scaled after the dot product, softmax, weighted sum of V (src/model.cpp:178-199); one warp per query head,
// lanes over positions with an online softmax, FP32 throughout.  grid: (tokens, kv heads), block: gqa warps.
static __global__ void __launch_bounds__(256) prefill_attention_kernel(const float* q, const __half* k_cache, const __half* v_cache,
                                                                       __half* out, int n_tokens, int start_pos, int seq_len,
                                                                       int head_size, int gqa, int q_rows) {
    extern __shared__ float sm[];  // [gqa][head_size] query rows, then [gqa warps][32 lanes][head_size] is too much: V sums go through registers
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = kvh * gqa + warp;
    const int hs = head_size;
    float* qs = sm + warp * hs;
    for (int d = lane; d < hs; d += 32) qs[d] = q[(size_t)t * q_rows + (size_t)h * hs + d];
    __syncwarp();
    const int T = start_pos + t + 1;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hs));
    const __half* kb = k_cache + (size_t)kvh * seq_len * hs;
    const __half* vb = v_cache + (size_t)kvh * seq_len * hs;
    // pass 1: scores of this lane's positions, maximum
    float m = -INFINITY;
    for (int p = lane; p < T; p += 32) {
        const __half2* kr = reinterpret_cast<const __half2*>(kb + (size_t)p * hs);
        float s = 0.f;
        for (int d = 0; d < hs / 2; ++d) {
            const float2 kk = __half22float2(kr[d]);
            s = fmaf(qs[2 * d], kk.x, s);
            s = fmaf(qs[2 * d + 1], kk.y, s);
        }
        m = fmaxf(m, s * scale);
    }
    m = warp_max(m);
    // pass 2: every lane owns head dims lane, lane + 32, ...; positions in order
    float l = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // head_size <= 128
    for (int p0 = 0; p0 < T; p0 += 32) {
        const int p = p0 + lane;
        float e = 0.f;
        if (p < T) {
            const __half2* kr = reinterpret_cast<const __half2*>(kb + (size_t)p * hs);
            float s = 0.f;
            for (int d = 0; d < hs / 2; ++d) {
                const float2 kk = __half22float2(kr[d]);
                s = fmaf(qs[2 * d], kk.x, s);
                s = fmaf(qs[2 * d + 1], kk.y, s);
            }
            e = __expf(s * scale - m);
        }
        l += e;
        const int cnt = min(32, T - p0);
        for (int i = 0; i < cnt; ++i) {
            const float ei = __shfl_sync(0xffffffffu, e, i);
            const __half* vr = vb + (size_t)(p0 + i) * hs;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (lane + 32 * c < hs) acc[c] = fmaf(ei, __half2float(vr[lane + 32 * c]), acc[c]);
        }
    }
    l = warp_sum(l);
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (lane + 32 * c < hs) out[(size_t)t * q_rows + (size_t)h * hs + lane + 32 * c] = __float2half_rn(__fdiv_rn(acc[c], l));
}

}  // namespace lpp
