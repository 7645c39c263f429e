// Batched prompt path ("prefill"): the K/V cache rows of up to kPrefillTokens prompt positions in one pass over
// the weights, instead of one pass per token.
//
// The reference feeds a prompt through forward() token by token (src/main.cpp:163-179): every prompt token
// streams all weights once.  Here the layer's matrices are streamed ONCE for the whole block of tokens: the
// four projections become small GEMMs  C[tokens][rows] = X[tokens][K] . W[rows][K]^T  that are still bound by
// the weight stream (2 FLOP per weight byte and token: far below the tensor cores' ridge for 64 tokens), so the
// kernels are organised around that stream like the decode GEMV -- a producer thread, a ring of shared-memory
// stages, mbarrier hand-over -- only that a stage is a pair of tiles fetched by the tensor memory accelerator
// (cp.async.bulk.tensor with the 128-byte swizzle, one copy per operand and stage: 128 weight rows x 128 inputs
// through a 3-D map, the matching 64 tokens x 128 inputs of the activations, hi and lo plane, through a 4-D map;
// the weight tiles of the first ring pass are requested before the dependency wait) and the arithmetic runs on
// the tensor cores: prefill_gemm_umma_kernel issues tcgen05.mma reading both operands from shared memory through
// matrix descriptors, FP32 accumulators in tensor memory, epilogue warps that read them back with tcgen05.ld.
// (An earlier kernel that consumed the same ring with ldmatrix + mma.sync.m16n8k16 in eight warps measured 1.17 ms
// against 0.83 ms for a 64-token pass of the Llama-3.2-1B shape and was removed.)
// Matrices whose row tiles do not fill the GPU (QKV, o_proj, down) are also cut along K so that every SM streams
// a share; partial sums are added in a fixed order by the next kernel (the norm kernel for the residual
// projections, prefill_qkv_finish_kernel for QKV).  Activations reach the MMAs as hi + lo FP16 pairs (see
// split_half); everything between the GEMMs (residual stream, RMSNorm, RoPE, softmax) stays FP32, following
// src/ops.cpp like the decode path.  The causal attention of the block (prefill_attention_mma_kernel) is a
// tensor-core flash attention over the cache.
//
// Tensor maps cover this GPU's own memory only; no cluster multicast is used anywhere.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace lpp {

constexpr int kPrefillTokens = 64;   // tokens per pass (rows of the activation tiles)
constexpr int kPfKc = 128;           // inputs per stage: two 64-wide (128-byte) swizzled sub-tiles per operand
constexpr int kPfSubBytesX = kPrefillTokens * 128;  // one activation sub-tile: 64 tokens x 64 inputs
constexpr int kPfMaxSplits = 8;
constexpr int kPfRingBytes = 192 * 1024;
constexpr int kPfSmemBytes = 1024 /*barriers*/ + 1024 /*alignment slack*/ + kPfRingBytes;

enum PfEpi : int { kPfQkv = 0, kPfResid = 1, kPfSwiglu = 2 };

// An activation x is handed to the tensor cores as two FP16 numbers, hi = fp16(x) and lo = fp16(x - hi): the MMA
// accumulates W.hi + W.lo in FP32, which keeps about 22 bits of x, so the batched pass carries FP32 activations
// through FP16-operand MMAs like the token loop carries them through its FP32 arithmetic.  Every activation buffer
// holds the hi plane [kPrefillTokens][cols] followed by the lo plane; one 4-D tensor map covers both.
__device__ __forceinline__ void split_half(float x, __half& hi, __half& lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}

struct PrefillGemmArgs {
    int n_rows, K;        // rows of the weight matrix, inputs per row
    int row0;             // first row of this layer's matrix inside the tensor map (layers are stacked)
    int n_tokens;         // valid tokens (<= kPrefillTokens)
    int start_pos;        // position of token 0
    int epi;
    int splits;           // K is cut into this many ranges (kPfResid and kPfQkv): work item = (row tile, range)
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

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                     smem_dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_addr)
                 : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, int z, int w, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                     smem_dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar_addr)
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
// QKV epilogue of one value: row `row` (and its pair partner `other`, the value of row ^ 1), token t: rotation of
// q and k pairs, q -> FP32 rows, k / v -> cache rows at the reference index.
__device__ __forceinline__ void pf_qkv_store(const PrefillGemmArgs& a, int row, int t, float v, float other) {
    if (row >= a.n_rows || t >= a.n_tokens) return;
    {  // (one scope: the body reads like the decode epilogue it mirrors, gemv.cuh)
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

// ---- the GEMM on the fifth-generation tensor cores (tcgen05), accumulators in tensor memory
//
// A work item is (tile of 128 weight rows, K range).  Per stage the tensor memory accelerator delivers the two
// 128-row x 64-input weight sub-tiles and, per 64-input piece, the 64 hi rows followed by the 64 lo rows of the
// activations, all in the 128-byte swizzled K-major layout that the MMA reads straight from shared memory through
// matrix descriptors: one elected thread issues eight 128 x 128 x 16 MMAs per stage (D[128 rows][hi tokens | lo
// tokens] += W . X^T) into one of two 128-column accumulators in tensor memory, commits the stage back to the
// producer, and after the last stage of the item commits the accumulator to the eight epilogue warps; these read
// their 32 lanes (rows) x 32 token columns of both halves with tcgen05.ld, add them, release the accumulator and
// run the epilogue from registers while the next item's MMAs already fill the other accumulator.  Warp roles: 0
// producer, 1 MMA issue and tensor-memory allocation, 2..9 epilogue (a warp may only read the tensor-memory lanes
// of its quarter, warp index modulo 4; two warps share a quarter and take 32 tokens each).  An epilogue thread owns
// one weight row and walks its tokens, so everything that depends on the row alone (which of q/k/v, head,
// rotation-table column) is computed once.
// Every wait is bounded; every path, also a failed one, reaches the common exit, which lets copies in flight land
// (bounded) and frees the tensor memory.
constexpr int kUmmaM = 128;
constexpr int kUmmaSubW = kUmmaM * 128;                            // 16 KiB
constexpr int kUmmaStage = 2 * kUmmaSubW + 4 * kPfSubBytesX;       // 64 KiB: weights, activations hi, activations lo
constexpr int kUmmaStages = kPfRingBytes / kUmmaStage;             // 3
constexpr int kUmmaEpiWarps = 8;                                   // two per tensor-memory lane quarter: 32 tokens each
constexpr int kUmmaThreads = (2 + kUmmaEpiWarps) * 32;
constexpr int kUmmaN = 2 * kPrefillTokens;                         // MMA N: the 64 hi rows and the 64 lo rows of the activation tile
constexpr int kUmmaAccCols = kUmmaN;                               // FP32 columns of one accumulator: W.hi | W.lo
constexpr int kUmmaTmemCols = 2 * kUmmaAccCols;                    // power of two >= 32
// Instruction descriptor: D = F32 (bits 4-5 = 1), A = B = F16 (0), both K-major (bits 15, 16 = 0),
// N / 8 in bits 17-22, M / 16 in bits 24-28.
constexpr uint32_t kUmmaIdesc = (1u << 4) | ((uint32_t)(kUmmaN >> 3) << 17) | ((uint32_t)(kUmmaM >> 4) << 24);

// Shared-memory matrix descriptor of a K-major operand tile with the 128-byte swizzle: start address / 16 in bits
// 0-13, leading byte offset (unused for swizzled K-major, set to 1) in bits 16-29, stride between 8-row groups
// (1024 bytes) / 16 in bits 32-45, descriptor version 1 in bits 46-47, layout type 2 (128-byte swizzle) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tc_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (quarter base + i), columns c .. c+31
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Epilogue of one thread: weight row `row`, tokens t0 .. t0+31 with the sums v[0..31].  Lanes are consecutive rows,
// so for a fixed token a warp's stores are contiguous; the partner row (row ^ 1) of the rotation and SwiGLU pairs
// is the neighbouring lane.  The rotation rounds like pf_qkv_store.
template <int EPI>
__device__ __forceinline__ void umma_epilogue(const PrefillGemmArgs& a, int split, int row, int t0, const float (&v)[32],
                                              int lane) {
    const bool row_ok = row < a.n_rows;
    const int nt = min(32, a.n_tokens - t0);  // valid tokens of this half (may be <= 0)
    if constexpr (EPI == kPfResid) {
        if (a.splits > 1) {
            float* p = a.part + ((size_t)split * kPrefillTokens + t0) * a.n_rows + row;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (row_ok && i < nt) p[(size_t)i * a.n_rows] = v[i];
        } else {
            float* p = a.x + (size_t)t0 * a.n_rows + row;
            float old[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) old[i] = (row_ok && i < nt) ? p[(size_t)i * a.n_rows] : 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (row_ok && i < nt) p[(size_t)i * a.n_rows] = old[i] + v[i];  // x += W.xb (src/model.cpp:232, 239)
        }
    } else if constexpr (EPI == kPfSwiglu) {
        // rows interleaved (gate_i, up_i): the even lane finishes tokens 0..15 of the pair, the odd lane tokens 16..31;
        // each sends the partner the half it does not finish itself.  hb = (h1*sigmoid(h1))*h3 (src/ops.cpp:78-87)
        // with the fast exponential and division (relative error ~1e-6, far below the FP16 weights' own rounding).
        const bool even = (lane & 1) == 0;
        __half* hb = a.hb + (size_t)(t0 + (even ? 0 : 16)) * (a.n_rows >> 1) + (row >> 1);
        const int nt_mine = nt - (even ? 0 : 16);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float keep = even ? v[k] : v[k + 16], send = even ? v[k + 16] : v[k];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
            const float g = even ? keep : recv, u = even ? recv : keep;
            const float r = __fdividef(g, 1.0f + __expf(-g)) * u;
            __half hi, lo;
            split_half(r, hi, lo);
            if (row_ok && k < nt_mine) {
                hb[(size_t)k * (a.n_rows >> 1)] = hi;
                hb[(size_t)(kPrefillTokens + k) * (a.n_rows >> 1)] = lo;
            }
        }
    } else if (a.splits > 1) {  // kPfQkv cut along K: partial sums, finished by prefill_qkv_finish_kernel
        float* p = a.part + ((size_t)split * kPrefillTokens + t0) * a.n_rows + row;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (row_ok && i < nt) p[(size_t)i * a.n_rows] = v[i];
    } else {  // kPfQkv
        const int hs = a.head_size;
        const bool pos_ok = a.start_pos >= 0 && a.start_pos + a.n_tokens <= a.seq_len;
        if (!pos_ok && lane == 0) atomicOr(&a.st->status, kStatusBadPos);
        const bool rot = row < a.q_rows + a.kv_rows;   // q and k rows rotate, v rows do not
        const bool is_q = row < a.q_rows, is_k = rot && !is_q;
        const int rr = is_q ? row : row - a.q_rows - (is_k ? 0 : a.kv_rows);
        const int head = rr / hs, off = rr - head * hs;
        const float2* rope = a.rope + (off >> 1);       // + pos * (hs / 2)
        float* qp = a.q + row;                          // + t * q_rows
        // cache index within the layer: h*(seq_len*hs) + pos*hs + off (src/scatter_kv.cu:15-16)
        __half* cp = (is_k ? a.k_cache : a.v_cache) + (size_t)head * ((size_t)a.seq_len * hs) + off;
        const bool odd = row & 1;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);
            if (!(row_ok && pos_ok && i < nt)) continue;
            const int t = t0 + i, pos = a.start_pos + t;
            float r = v[i];
            if (rot) {
                // adjacent-pair rotation with the table entry for (pos, off/2) (src/ops.cpp:34-54)
                const float2 cs = __ldg(rope + (size_t)pos * (hs >> 1));
                r = odd ? __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(v[i], cs.x))   // v1' = v0*sin + v1*cos
                        : __fsub_rn(__fmul_rn(v[i], cs.x), __fmul_rn(other, cs.y));  // v0' = v0*cos - v1*sin
            }
            if (is_q)
                qp[(size_t)t * a.q_rows] = r;
            else
                cp[(size_t)pos * hs] = __float2half_rn(r);
        }
    }
}

#ifdef LPP_TIMING_AIDS
// timing aid: global-timer stamps [cta][slot] of the last gate|up launch
__device__ unsigned long long g_pf_trace[160][48];
#define PF_STAMP(k)                                                                      \
    do {                                                                                 \
        if (EPI == kPfSwiglu && (k) < 48) {                                              \
            unsigned long long t_;                                                       \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                       \
            g_pf_trace[blockIdx.x][k] = t_;                                              \
        }                                                                                \
    } while (0)
#else
#define PF_STAMP(k) \
    do {            \
    } while (0)
#endif

template <int EPI>
static __global__ void __launch_bounds__(kUmmaThreads, 1) prefill_gemm_umma_kernel(const __grid_constant__ CUtensorMap w_map,
                                                                                   const __grid_constant__ CUtensorMap x_map,
                                                                                   const PrefillGemmArgs a) {
    constexpr int kStages = kUmmaStages, kStage = kUmmaStage, kSubX = kPfSubBytesX;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // [kStages]
    uint64_t* empty = full + kStages;                    // [kStages]
    uint64_t* acc_full = empty + kStages;                // [2]
    uint64_t* acc_empty = acc_full + 2;                  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* s_fail = reinterpret_cast<int*>(tmem_slot + 1);  // set by a role whose wait ran out
    const uint32_t ring = (smem_u32(smem) + 1024u + 1023u) & ~1023u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit = blockIdx.x, n_units = gridDim.x;
    const int n_tiles = (a.n_rows + kUmmaM - 1) / kUmmaM;  // items along the rows
    const int n_kc = (a.K + kPfKc - 1) / kPfKc;
    const int S = a.splits;
    const int n_items = n_tiles * S;
    pdl_launch_dependents();
    if (tid == 0) {
        *s_fail = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], kUmmaEpiWarps);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tc_alloc(tmem_slot, kUmmaTmemCols);
        tc_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == 0) {
        // ---------------- producer
        if (lane == 0) {
            PF_STAMP(0);
            // The weight sub-tiles of the first ring pass do not depend on the previous kernel: they are requested
            // before the dependency wait, the activation sub-tiles of the same stages right after it.
            int slot = 0, pass = 0;
            bool ok = true, waited = false;
            int early = 0;  // stages whose weights are already in flight
            // one copy per operand and stage: both 64-input weight sub-tiles / the four activation sub-tiles (hi, lo)
            auto load_w = [&](uint32_t dst, int kc, int wrow, int sl) { tma_load_3d(dst, &w_map, 0, wrow, 2 * kc, smem_u32(&full[sl])); };
            auto load_x = [&](uint32_t dst, int kc, int sl) { tma_load_4d(dst, &x_map, 0, 0, 0, 2 * kc, smem_u32(&full[sl])); };
            auto expect = [&](int sl) { mbar_arrive_expect_tx(&full[sl], kStage); };
            for (int item = unit; item < n_items && ok; item += n_units) {
                const int tile = item / S, split = item - tile * S;
                const int kc0 = (split * n_kc) / S, kc1 = ((split + 1) * n_kc) / S;
                const int wrow = a.row0 + tile * kUmmaM;
                if (!waited) {
                    early = min(kc1 - kc0, kStages);
                    for (int i = 0; i < early; ++i) {
                        const uint32_t dst = ring + (uint32_t)i * kStage;
                        expect(i);
                        load_w(dst, kc0 + i, wrow, i);
                    }
                    pdl_wait();
                    PF_STAMP(1);
                    waited = true;
                }
                for (int kc = kc0; kc < kc1; ++kc) {
                    const uint32_t dst = ring + (uint32_t)slot * kStage;
                    if (early > 0) {
                        --early;  // first pass of the first item: only the activations are missing
                    } else {
                        if (pass > 0 && !mbar_wait_bounded(&empty[slot], (uint32_t)(pass - 1) & 1u, a.st)) {
                            *s_fail = 1;
                            ok = false;
                            break;
                        }
                        expect(slot);
                        load_w(dst, kc, wrow, slot);
                    }
                    PF_STAMP(2 + kc - kc0);
                    load_x(dst + 2 * kUmmaSubW, kc, slot);
                    if (++slot == kStages) {
                        slot = 0;
                        ++pass;
                    }
                }
            }
            if (!waited) pdl_wait();
        }
    } else if (warp == 1) {
        // ---------------- MMA issue
        if (lane == 0) {
            int slot = 0;
            uint32_t par = 0;
            bool ok = true;
            int it = 0;
            for (int item = unit; item < n_items && ok; item += n_units, ++it) {
                const int tile = item / S, split = item - tile * S;
                const int kc0 = (split * n_kc) / S, kc1 = ((split + 1) * n_kc) / S;
                const int b = it & 1, use = it >> 1;
                (void)tile;
                if (use > 0 && !mbar_wait_bounded(&acc_empty[b], (uint32_t)(use - 1) & 1u, a.st)) {
                    *s_fail = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem + (uint32_t)(b * kUmmaAccCols);
                for (int kc = kc0; kc < kc1; ++kc) {
                    if (!mbar_wait_bounded(&full[slot], par, a.st)) {
                        *s_fail = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    PF_STAMP(18 + kc - kc0);
                    const uint32_t st = ring + (uint32_t)slot * kStage;
#pragma unroll
                    for (int sub = 0; sub < 2; ++sub) {
                        // the activation sub-tile holds the hi rows followed by the lo rows: one MMA covers both (N = 128)
                        const uint32_t wt = st + sub * kUmmaSubW, xt = st + 2 * kUmmaSubW + sub * 2 * kSubX;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {  // 16 inputs = 32 bytes along the swizzled row per step
                            const uint32_t acc = (kc > kc0 || sub > 0 || ks > 0) ? 1u : 0u;
                            tc_mma_f16(d_tmem, umma_desc(wt + ks * 32), umma_desc(xt + ks * 32), kUmmaIdesc, acc);
                        }
                    }
                    tc_commit(&empty[slot]);  // arrives once the MMAs issued so far have read this stage
                    if (++slot == kStages) {
                        slot = 0;
                        par ^= 1u;
                    }
                }
                if (ok) tc_commit(&acc_full[b]);
            }
        }
    } else {
        // ---------------- epilogue: this warp owns tensor-memory lanes 32 * (warp % 4) .. + 31 = rows of the tile,
        // and the first or second 32 columns (tokens) of the accumulator
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        int it = 0;
        for (int item = unit; item < n_items; item += n_units, ++it) {
            const int tile = item / S, split = item - tile * S;
            const int b = it & 1, use = it >> 1;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(&acc_full[b], (uint32_t)use & 1u, a.st))) {
                *s_fail = 1;
                break;
            }
            tc_fence_after();
            if (tid == 64) PF_STAMP(34);
            float v[32], vlo[32];
            const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * kUmmaAccCols);
            tc_ld32(taddr + half * 32, v);                     // W.hi of this warp's 32 tokens
            tc_ld32(taddr + kPrefillTokens + half * 32, vlo);  // W.lo
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += vlo[i];
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
            if (tid == 64) PF_STAMP(35);
            umma_epilogue<EPI>(a, split, tile * kUmmaM + quarter * 32 + lane, half * 32, v, lane);
            if (tid == 64) PF_STAMP(36);
        }
    }
    // ---------------- common exit
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    // A wait that ran out has set the status word (mbar_wait_bounded) and this CTA's flag.  Copies may then still be in
    // flight towards its shared memory: give them a bounded time to land before the CTA leaves (a tile copy takes a
    // few microseconds; nobody reads the tiles any more).
    if (tid == 0 && *reinterpret_cast<volatile int*>(s_fail) != 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < (1 << 17)) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) tc_dealloc(tmem, kUmmaTmemCols);
}

// Finishes a QKV GEMM that was cut along K: adds the partial sums of a row pair in range order and applies the
// QKV epilogue (rotation of q and k pairs, q -> FP32 rows, k/v -> cache rows at the reference index).
// grid: (tokens, ceil(row pairs / 256)).
static __global__ void __launch_bounds__(256) prefill_qkv_finish_kernel(const PrefillGemmArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, pr = blockIdx.y * 256 + threadIdx.x;
    const int row = 2 * pr;
    if (row >= a.n_rows) return;
    float2 v = make_float2(0.f, 0.f);
    float2 p[kPfMaxSplits];
#pragma unroll
    for (int s0 = 0; s0 < kPfMaxSplits; ++s0)
        if (s0 < a.splits) p[s0] = *reinterpret_cast<const float2*>(a.part + ((size_t)s0 * kPrefillTokens + t) * a.n_rows + row);
#pragma unroll
    for (int s0 = 0; s0 < kPfMaxSplits; ++s0)
        if (s0 < a.splits) {
            v.x += p[s0].x;
            v.y += p[s0].y;
        }
    pf_qkv_store(a, row, t, v.x, v.y);
    pf_qkv_store(a, row + 1, t, v.y, v.x);
}

// Rows of the residual stream -> RMS-normalised FP16 rows (MMA operands).  Layer 0 takes the embedding rows of
// the prompt tokens and also writes them out as the FP32 residual stream.  grid: tokens.
constexpr int kPfNormThreads = 512;
// Only the weights (emb, norm_w) are marked read-only: a pointer to data the preceding kernel produced must not be
// `const __restrict__`, or its loads become invariant loads that the compiler may move above the dependency wait.
static __global__ void __launch_bounds__(kPfNormThreads) prefill_norm_kernel(float* x, const int* tokens,
                                                                            const __half* __restrict__ emb, int vocab,
                                                                            const float* __restrict__ norm_w, __half* out,
                                                                            int D, int n_tokens, const float* part,
                                                                            int splits, StepState* st) {
    __shared__ float red[kPfNormThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)t * D);
    const int nv4 = D >> 2;  // D is a multiple of 8
    constexpr int kMaxPer = 4;  // float4 per thread kept in registers for the second pass: rows up to 8192 wide
    float4 v[kMaxPer];
    int tok = 0;
    if (emb) {
        tok = tokens[t];
        if (tok < 0 || tok >= vocab) {
            if (tid == 0) atomicOr(&st->status, kStatusBadToken);
            tok = 0;
        }
    }
    const bool add_parts = !emb && splits > 1;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPer; ++k) {
        const int i = tid + k * kPfNormThreads;
        if (i < nv4) {
            // every load of this piece (the row and all partial sums) is issued before the first is used
            float4 p[kPfMaxSplits];
            if (emb) {
                const uint2 h = *reinterpret_cast<const uint2*>(emb + (size_t)tok * D + 4 * (size_t)i);
                const float2 lo = half2_bits_to_float2(h.x), hi = half2_bits_to_float2(h.y);
                v[k] = make_float4(lo.x, lo.y, hi.x, hi.y);
            } else {
                v[k] = xr[i];
            }
            if (add_parts) {
#pragma unroll
                for (int s0 = 0; s0 < kPfMaxSplits; ++s0)
                    if (s0 < splits) p[s0] = reinterpret_cast<const float4*>(part + ((size_t)s0 * kPrefillTokens + t) * D)[i];
                // x += p_0 + p_1 + ... in range order
#pragma unroll
                for (int s0 = 0; s0 < kPfMaxSplits; ++s0)
                    if (s0 < splits) {
                        v[k].x += p[s0].x; v[k].y += p[s0].y; v[k].z += p[s0].z; v[k].w += p[s0].w;
                    }
            }
            if (emb || add_parts) xr[i] = v[k];  // the residual stream as the next residual GEMM reads it
            ss = fmaf(v[k].x, v[k].x, fmaf(v[k].y, v[k].y, fmaf(v[k].z, v[k].z, fmaf(v[k].w, v[k].w, ss))));
        }
    }
    // rows wider than kMaxPer * kPfNormThreads * 4: the rest without register caching
    for (int i = tid + kMaxPer * kPfNormThreads; i < nv4; i += kPfNormThreads) {
        float4 w;
        if (emb) {
            const uint2 h = *reinterpret_cast<const uint2*>(emb + (size_t)tok * D + 4 * (size_t)i);
            const float2 lo = half2_bits_to_float2(h.x), hi = half2_bits_to_float2(h.y);
            w = make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            w = xr[i];
        }
        if (add_parts)
            for (int s0 = 0; s0 < splits; ++s0) {
                const float4 q = reinterpret_cast<const float4*>(part + ((size_t)s0 * kPrefillTokens + t) * D)[i];
                w.x += q.x; w.y += q.y; w.z += q.z; w.w += q.w;
            }
        if (emb || add_parts) xr[i] = w;
        ss = fmaf(w.x, w.x, fmaf(w.y, w.y, fmaf(w.z, w.z, fmaf(w.w, w.w, ss))));
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < kPfNormThreads / 32; ++k) tot += red[k];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)D), 1e-5f)));
    auto emit = [&](int i, const float4& xv) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(norm_w) + i);
        const float y[4] = {__fmul_rn(__fmul_rn(xv.x, scale), w.x), __fmul_rn(__fmul_rn(xv.y, scale), w.y),
                            __fmul_rn(__fmul_rn(xv.z, scale), w.z), __fmul_rn(__fmul_rn(xv.w, scale), w.w)};
        __align__(8) __half hi[4], lo[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) split_half(y[c], hi[c], lo[c]);
        *reinterpret_cast<uint2*>(out + (size_t)t * D + 4 * (size_t)i) = *reinterpret_cast<const uint2*>(hi);
        *reinterpret_cast<uint2*>(out + (size_t)(kPrefillTokens + t) * D + 4 * (size_t)i) = *reinterpret_cast<const uint2*>(lo);
    };
#pragma unroll
    for (int k = 0; k < kMaxPer; ++k) {
        const int i = tid + k * kPfNormThreads;
        if (i < nv4) emit(i, v[k]);
    }
    for (int i = tid + kMaxPer * kPfNormThreads; i < nv4; i += kPfNormThreads) emit(i, xr[i]);  // re-read what this thread wrote
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
    // one position's score: the K row in 16-byte pieces, all requested before the first is used
    auto score = [&](int p) -> float {
        const uint4* kr = reinterpret_cast<const uint4*>(kb + (size_t)p * hs);
        float s = 0.f;
        for (int d0 = 0; d0 < hs / 8; d0 += 8) {
            uint4 u[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (d0 + i < hs / 8) u[i] = __ldcg(kr + d0 + i);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (d0 + i < hs / 8) {
                    const float* qq = qs + 8 * (d0 + i);
                    float2 f;
                    f = half2_bits_to_float2(u[i].x); s = fmaf(qq[0], f.x, s); s = fmaf(qq[1], f.y, s);
                    f = half2_bits_to_float2(u[i].y); s = fmaf(qq[2], f.x, s); s = fmaf(qq[3], f.y, s);
                    f = half2_bits_to_float2(u[i].z); s = fmaf(qq[4], f.x, s); s = fmaf(qq[5], f.y, s);
                    f = half2_bits_to_float2(u[i].w); s = fmaf(qq[6], f.x, s); s = fmaf(qq[7], f.y, s);
                }
        }
        return s * scale;
    };
    // pass 1: scores of this lane's positions, maximum
    float m = -INFINITY;
    for (int p = lane; p < T; p += 32) m = fmaxf(m, score(p));
    m = warp_max(m);
    // pass 2: every lane owns head dims lane, lane + 32, ...; positions in order, eight V rows in flight
    float l = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // head_size <= 128
    for (int p0 = 0; p0 < T; p0 += 32) {
        const int p = p0 + lane;
        const float e = (p < T) ? __expf(score(p) - m) : 0.f;
        l += e;
        const int cnt = min(32, T - p0);
        for (int i0 = 0; i0 < cnt; i0 += 8) {
            __half vv[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (i0 + i < cnt && lane + 32 * c < hs) vv[i][c] = vb[(size_t)(p0 + i0 + i) * hs + lane + 32 * c];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float ei = __shfl_sync(0xffffffffu, e, (i0 + i) & 31);
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (i0 + i < cnt && lane + 32 * c < hs) acc[c] = fmaf(ei, __half2float(vv[i][c]), acc[c]);
            }
        }
    }
    l = warp_sum(l);
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (lane + 32 * c < hs) {
            __half hi, lo;
            split_half(__fdiv_rn(acc[c], l), hi, lo);
            out[(size_t)t * q_rows + (size_t)h * hs + lane + 32 * c] = hi;
            out[(size_t)(kPrefillTokens + t) * q_rows + (size_t)h * hs + lane + 32 * c] = lo;
        }
}

// Causal attention of the prompt block on the tensor cores: CTA (query tile of 16 tokens, KV head), one warp per
// query head of the group.  K and V rows stream through shared memory 64 positions at a time (16-byte asynchronous
// copies, double buffered, rows padded by 16 bytes so that the 8-row matrix loads do not collide on banks); every
// warp keeps its 16 x head_size query tile as A fragments, forms the 16 x 64 scores with mma.sync m16n8k16, masks
// them causally, runs the online softmax in FP32 on the accumulator layout, and feeds the probabilities back as A
// fragments of the P x V product (V read through transposing matrix loads).  Same mathematics as
// prefill_attention_kernel (src/model.cpp:178-199), FP16 operands with FP32 accumulation.
constexpr int kPfAttnTile = 64;   // positions per shared-memory tile
constexpr int kPfAttnRows = 16;   // query tokens per CTA
template <int HS>
constexpr int pf_attn_smem() {
    return 2 /*buffers*/ * 2 /*K, V*/ * kPfAttnTile * (HS * 2 + 16);
}

__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src, bool valid) {
    const uint32_t d = smem_u32(dst_smem);
    const int n = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
template <int HS>
static __global__ void __launch_bounds__(256) prefill_attention_mma_kernel(const float* q, const __half* k_cache,
                                                                           const __half* v_cache, __half* out, int n_tokens,
                                                                           int start_pos, int seq_len, int gqa, int q_rows) {
    constexpr int kStride = HS * 2 + 16;              // bytes per padded row
    constexpr int kMat = kPfAttnTile * kStride;       // bytes of one K or V tile
    constexpr int kChunks = kPfAttnTile * (HS / 8);   // 16-byte pieces of one tile
    extern __shared__ __align__(128) unsigned char at_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * kPfAttnRows, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int h = kvh * gqa + warp;
    const int rows_here = min(kPfAttnRows, n_tokens - t0);
    const int t_max = start_pos + t0 + rows_here;  // positions 0 .. t_max - 1 are visible to the last token of the tile
    const int n_tiles = (t_max + kPfAttnTile - 1) / kPfAttnTile;
    const unsigned char* kb = reinterpret_cast<const unsigned char*>(k_cache + (size_t)kvh * seq_len * HS);
    const unsigned char* vb = reinterpret_cast<const unsigned char*>(v_cache + (size_t)kvh * seq_len * HS);

    auto load_tile = [&](int tile, int buf) {
        unsigned char* ks = at_smem + (size_t)buf * 2 * kMat;
        unsigned char* vs = ks + kMat;
        const int p0 = tile * kPfAttnTile;
        for (int c = threadIdx.x; c < kChunks; c += blockDim.x) {
            const int row = c / (HS / 8), col = c % (HS / 8);
            const bool ok = p0 + row < t_max;
            const size_t src = ok ? ((size_t)(p0 + row) * HS * 2 + (size_t)col * 16) : 0;
            cp_async_16(ks + row * kStride + col * 16, kb + src, ok);
            cp_async_16(vs + row * kStride + col * 16, vb + src, ok);
        }
    };

    // the query tile of this warp's head as A fragments
    uint32_t qa[HS / 16][4];
    {
        const int r0 = t0 + g, r1 = t0 + g + 8;
        const float* q0 = q + (size_t)r0 * q_rows + (size_t)h * HS;
        const float* q1 = q + (size_t)r1 * q_rows + (size_t)h * HS;
#pragma unroll
        for (int kk = 0; kk < HS / 16; ++kk) {
            const int c0 = kk * 16 + 2 * tq;
            const float2 z = make_float2(0.f, 0.f);
            const float2 a0 = (r0 < n_tokens) ? *reinterpret_cast<const float2*>(q0 + c0) : z;
            const float2 a1 = (r1 < n_tokens) ? *reinterpret_cast<const float2*>(q1 + c0) : z;
            const float2 a2 = (r0 < n_tokens) ? *reinterpret_cast<const float2*>(q0 + c0 + 8) : z;
            const float2 a3 = (r1 < n_tokens) ? *reinterpret_cast<const float2*>(q1 + c0 + 8) : z;
            qa[kk][0] = pack_half2(a0.x, a0.y);
            qa[kk][1] = pack_half2(a1.x, a1.y);
            qa[kk][2] = pack_half2(a2.x, a2.y);
            qa[kk][3] = pack_half2(a3.x, a3.y);
        }
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)HS));
    const int lim0 = (t0 + g < n_tokens) ? start_pos + t0 + g : -1;          // last visible position of row g
    const int lim1 = (t0 + g + 8 < n_tokens) ? start_pos + t0 + g + 8 : -1;  // ... of row g + 8
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[HS / 8][4];
#pragma unroll
    for (int i = 0; i < HS / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    load_tile(0, 0);
    cp_async_commit();
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < n_tiles) {
            load_tile(tile + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t ks = smem_u32(at_smem + (size_t)buf * 2 * kMat);
        const uint32_t vs = ks + kMat;
        const int p0 = tile * kPfAttnTile;
        // scores of 16 rows x 64 positions
        float c[kPfAttnTile / 8][4];
#pragma unroll
        for (int j = 0; j < kPfAttnTile / 8; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
        const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
        for (int jp = 0; jp < kPfAttnTile / 16; ++jp) {
#pragma unroll
            for (int kk = 0; kk < HS / 16; ++kk) {
                uint32_t b[4];
                ldmatrix_x4(ks + (uint32_t)((jp * 16 + (mi >> 1) * 8 + mr) * kStride + (kk * 16 + (mi & 1) * 8) * 2), b[0], b[1],
                            b[2], b[3]);
                mma_f16_16816(c[2 * jp], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b[0], b[1]);
                mma_f16_16816(c[2 * jp + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b[2], b[3]);
            }
        }
        // scale, causal mask, online softmax (rows g and g + 8; a row's 64 scores lie on the four lanes of a quad)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < kPfAttnTile / 8; ++j) {
            const int p = p0 + 8 * j + 2 * tq;
            c[j][0] = (p <= lim0) ? c[j][0] * scale : -INFINITY;
            c[j][1] = (p + 1 <= lim0) ? c[j][1] * scale : -INFINITY;
            c[j][2] = (p <= lim1) ? c[j][2] * scale : -INFINITY;
            c[j][3] = (p + 1 <= lim1) ? c[j][3] * scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(c[j][0], c[j][1]));
            mx1 = fmaxf(mx1, fmaxf(c[j][2], c[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float u0 = (n0 == -INFINITY) ? 0.f : n0, u1 = (n1 == -INFINITY) ? 0.f : n1;  // nothing visible yet
        const float f0 = __expf(m0 - u0), f1 = __expf(m1 - u1);  // exp(-inf) = 0 on the first visible tile
        m0 = n0;
        m1 = n1;
        l0 *= f0;
        l1 *= f1;
#pragma unroll
        for (int i = 0; i < HS / 8; ++i) {
            o[i][0] *= f0;
            o[i][1] *= f0;
            o[i][2] *= f1;
            o[i][3] *= f1;
        }
        uint32_t pa[kPfAttnTile / 16][4];
#pragma unroll
        for (int j = 0; j < kPfAttnTile / 8; ++j) {
            const float e0 = __expf(c[j][0] - u0), e1 = __expf(c[j][1] - u0);
            const float e2 = __expf(c[j][2] - u1), e3 = __expf(c[j][3] - u1);
            l0 += e0 + e1;
            l1 += e2 + e3;
            pa[j >> 1][(j & 1) * 2 + 0] = pack_half2(e0, e1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_half2(e2, e3);
        }
        // o += P x V
#pragma unroll
        for (int kk = 0; kk < kPfAttnTile / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < HS / 16; ++dp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vs + (uint32_t)((kk * 16 + (mi & 1) * 8 + mr) * kStride + (dp * 16 + (mi >> 1) * 8) * 2));
                mma_f16_16816(o[2 * dp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[0], b[1]);
                mma_f16_16816(o[2 * dp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[2], b[3]);
            }
        }
        __syncthreads();  // the buffer is refilled two iterations from now, by the copy issued in the next one
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int r0 = t0 + g, r1 = t0 + g + 8;
#pragma unroll
    for (int i = 0; i < HS / 8; ++i) {
        const int d = 8 * i + 2 * tq;
        auto put = [&](int r, float a0, float a1) {
            __align__(4) __half hi[2], lo[2];
            split_half(a0, hi[0], lo[0]);
            split_half(a1, hi[1], lo[1]);
            *reinterpret_cast<uint32_t*>(out + (size_t)r * q_rows + (size_t)h * HS + d) = *reinterpret_cast<const uint32_t*>(hi);
            *reinterpret_cast<uint32_t*>(out + (size_t)(kPrefillTokens + r) * q_rows + (size_t)h * HS + d) =
                *reinterpret_cast<const uint32_t*>(lo);
        };
        if (r0 < n_tokens) put(r0, __fdiv_rn(o[i][0], l0), __fdiv_rn(o[i][1], l0));
        if (r1 < n_tokens) put(r1, __fdiv_rn(o[i][2], l1), __fdiv_rn(o[i][3], l1));
    }
}

}  // namespace lpp
