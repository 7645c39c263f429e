// Shared device helpers for the sm_100a decode kernels: PTX wrappers for mbarrier / bulk async
// copies / programmatic dependent launch, warp reductions, an exp() that is bit-reproducible on
// the host, and the device-resident per-step state.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <math.h>

namespace lpp {

// ------------------------------------------------------------------ device-resident step state

constexpr int kHistoryMax = 4096;  // capacity of the repetition-penalty history on the device

// Device status bits (StepState::status); any non-zero value makes the host call fail with
// LPP_ERR_DEVICE_STATUS instead of hanging or trapping.
enum : int {
    kStatusOk = 0,
    kStatusBarrierTimeout = 1,  // a bounded mbarrier wait ran out
    kStatusBadToken = 2,        // token id outside [0, vocab)
    kStatusBadPos = 4           // pos outside [0, seq_len)
};

// Everything a step needs that changes from token to token lives here, so one captured graph
// serves every position: forward()'s scalar arguments (src/model.cpp:342) become fields.
struct StepState {
    int token;         // input token of this step
    int pos;           // position of this step
    int history_len;   // valid entries in history[]
    int history_window;  // free-running mode: ring capacity (src/main.cpp:158 uses 64); 0 = host-managed
    int history_count; // free-running mode: tokens pushed so far (ring cursor)
    int step_idx;      // free-running mode: index into r_values / out_tokens
    int advance;       // 1 = sampler feeds its token back (token=sampled, pos+1, push history)
    float temperature;
    float penalty;
    float r;           // uniform draw for teacher-forced steps (advance == 0)
    int out_token;     // sampled token of the last step
    int status;        // kStatus* bits, sticky until the host clears them
    long long wait_cycles;     // limit of a wait on this GPU's own work in SM clocks (0 = kWaitCycles)
    long long tp_wait_cycles;  // limit of a wait on a tensor-parallel peer in SM clocks (0 = kTpWaitCycles)
    int history[kHistoryMax];
};

// ------------------------------------------------------------------ small utilities

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 128-bit streaming load that does not pollute L1 (weights are read exactly once per token).
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}

// ------------------------------------------------------------------ programmatic dependent launch

// Block until every grid this one programmatically depends on has completed and its writes are
// visible.  A no-op when the launch carried no programmatic dependency.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allow the dependent grid to start launching (it still waits in pdl_wait for our completion).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------ mbarrier + bulk async copy

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    // make the initialised barriers visible to the async proxy (the bulk-copy engine)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a barrier phase (try_wait may suspend the whole warp for a while, which a warp whose
// lanes watch DIFFERENT barriers cannot afford).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Limits of device-side waits, in SM clocks.  A wait on this GPU's own work (a bulk copy, a grid barrier)
// gives up after tens of milliseconds.  The ranks of a tensor-parallel group are separate processes whose
// launches may be skewed by host-side delays, so the limit of a wait on a peer is seconds.  Both can be
// shortened per engine (lpp_config.wait_ms / tp_wait_ms; the first is read from StepState only once a wait
// has lasted unusually long, the second travels as a kernel argument); once a wait has run out the status
// bit is set and no later wait of the step spins again.
constexpr long long kWaitCycles = 100ll * 1000 * 1000;
constexpr long long kTpWaitCycles = 8ll * 1000 * 1000 * 1000;
__device__ __forceinline__ long long wait_limit(const StepState* st) {
    const long long v = st ? *reinterpret_cast<const volatile long long*>(&st->wait_cycles) : 0;
    return v > 0 ? v : kWaitCycles;
}
__device__ __forceinline__ bool status_timed_out(const StepState* st) {
    return (*reinterpret_cast<const volatile int*>(&st->status) & kStatusBarrierTimeout) != 0;
}

// Bounded wait: polls until the phase completes or the limit has passed, then records the timeout in
// st->status and returns false.  Callers stop consuming and fall through to the kernel's end, so a lost
// copy cannot hang the GPU; the host sees the status (LPP_ERR_DEVICE_STATUS).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, StepState* st) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    // The engine's limit lives in global memory; fetching it costs an L2 round trip, which an ordinary wait
    // for a copy in flight must not pay.  It is read once the wait has lasted longer than any normal one.
    long long limit = 1 << 17;  // ~65 us, below every configurable limit
    bool fetched = false;
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > limit) {
            if (!fetched) {
                limit = wait_limit(st);
                fetched = true;
                continue;
            }
            if (st) atomicOr(&st->status, kStatusBarrierTimeout);
            return false;
        }
    }
    return true;
}

// One-dimensional bulk copy global -> this CTA's shared memory, completion counted in bytes on
// an mbarrier.  dst/src 16-byte aligned, bytes a multiple of 16.  No cluster qualifier: every
// CTA fetches its own data.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// The same copy with an L2 cache policy (from l2_policy_evict_first): streamed weights are used once per
// token and should not push the K/V cache and the activations out of L2.
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar,
                                              unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Asks the copy engine to pull [gsrc, gsrc+bytes) into L2 (no shared-memory destination, no
// completion to wait for).  gsrc 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}

// ------------------------------------------------------------------ reproducible expf

// exp(x) for float x, evaluated in double with only IEEE add/mul/fma, so the host twin (same
// source, compiled by the host compiler) returns the same bits as the device.  Relative error of
// the double intermediate is < 1e-13, so the float result is the correctly rounded exp(x) except
// when exp(x) lies within that distance of a rounding boundary.
__host__ __device__ inline float exp_repro(float x) {
    if (!(x > -104.0f)) return (x != x) ? x : 0.0f;
    if (x > 88.8f) return INFINITY;
    const double kLog2e = 1.4426950408889634074;
    const double kLn2Hi = 6.93147180369123816490e-01;  // ln2 split so k*kLn2Hi is exact for |k| < 2^10
    const double kLn2Lo = 1.90821492927058770002e-10;
    double xd = (double)x;
    double kd = rint(xd * kLog2e);
    double r = fma(-kd, kLn2Hi, xd);
    r = fma(-kd, kLn2Lo, r);
    // Taylor series to degree 13 on |r| <= 0.3466: remainder < 3e-18 relative
    double p = 1.0 / 6227020800.0;
    p = fma(p, r, 1.0 / 479001600.0);
    p = fma(p, r, 1.0 / 39916800.0);
    p = fma(p, r, 1.0 / 3628800.0);
    p = fma(p, r, 1.0 / 362880.0);
    p = fma(p, r, 1.0 / 40320.0);
    p = fma(p, r, 1.0 / 5040.0);
    p = fma(p, r, 1.0 / 720.0);
    p = fma(p, r, 1.0 / 120.0);
    p = fma(p, r, 1.0 / 24.0);
    p = fma(p, r, 1.0 / 6.0);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    long long k = (long long)kd;
    union {
        long long i;
        double d;
    } s;
    s.i = (k + 1023) << 52;  // k in [-151, 128]: always a normal double
    return (float)(p * s.d);
}

}  // namespace lpp
