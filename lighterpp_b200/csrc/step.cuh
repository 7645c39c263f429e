// Persistent decode-step kernel: a run of consecutive phases of one step (fused GEMVs and the
// flash-decode attention between them) executed by ONE launch of one CTA per SM, with grid-wide
// barriers where a phase consumes what the previous one produced.
//
// Why: as separate launches every GEMV pays launch, barrier set-up, input staging, first-copy
// latency and tail drain (~3-4 us during which HBM idles); with 80 such boundaries per token that is
// as much as the weight streaming itself.  Here the producer warp never waits for a phase boundary:
// weights do not depend on activations, so each producer lane keeps issuing bulk copies for the next
// phase into its consumer's ring while the consumers sit in the grid barrier and stage the next
// input vector.  The rings (128 KiB per SM, ~19 MB per GPU) cover about 3 us of HBM time, more than
// a barrier plus the staging costs.
//
// The phases replace the same reference calls as the stand-alone kernels: attention() and
// transformer_block() of src/model.cpp:121-241 (USE_CUDA branches) for all layers, plus the final
// RMSNorm + classifier of src/model.cpp:357-358.  Under tensor parallelism the run is cut at the two
// all-reduce points of each layer.
#pragma once
#include "attention.cuh"
#include "common.cuh"
#include "gemv.cuh"

namespace lpp {

enum StepPhaseType : int { kPhaseGemv = 0, kPhaseAttn = 1 };

struct StepPhase {
    int type;  // StepPhaseType
    int epi;   // GemvEpi for kPhaseGemv
    GemvArgs g;
    AttnArgs at;
};

struct StepArgs {
    const StepPhase* phases;  // device array
    int first, count;         // phases [first, first+count) run in this launch
    unsigned int* gbar;       // grid-barrier counter of this launch (zero at launch, zeroed again by the sampler)
    StepState* st;
    int n_slots;     // ring slots per consumer warp
    int slot_bytes;  // bytes per slot (>= every phase's stage_bytes)
    int xs_bytes;    // bytes reserved for the staged input vector / attention scratch
    unsigned long long* trace;  // timing aid: [cta][phase][4] global-timer stamps, or nullptr
};

constexpr int kStepConsumerThreads = kGemvConsumerWarps * 32;

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid-wide barrier among the consumer halves of all CTAs (the producer warps never take part).
// Every CTA adds one to a monotonically growing counter and waits until it reaches `target`.  The
// wait is bounded; on timeout, or when another CTA already reported a failure, the kernel is
// abandoned (returns false on every thread of the CTA) and the host sees StepState.status.
__device__ __forceinline__ bool grid_barrier(unsigned int* gbar, unsigned int target, StepState* st, int* s_flag,
                                             int tid) {
    consumer_barrier(kStepConsumerThreads);  // all of this CTA's results of the phase are written
    if (tid == 0) {
        // release at GPU scope: everything this CTA wrote (ordered before by the CTA barrier) is visible
        // to whoever acquires the counter afterwards
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gbar) : "memory");
        bool ok = s_flag[3] == 0;  // s_flag[3]: a consumer warp of this CTA gave up on its ring
        if (!ok) atomicOr(&st->status, kStatusBarrierTimeout);
        if (ok && ld_acquire_u32(gbar) < target) {
            const long long t0 = clock64();
            while (ld_acquire_u32(gbar) < target) {
                if (clock64() - t0 > kWaitCycles || ld_acquire_u32(reinterpret_cast<unsigned int*>(&st->status)) != 0u) {
                    atomicOr(&st->status, kStatusBarrierTimeout);
                    ok = false;
                    break;
                }
            }
        }
        *s_flag = ok ? 1 : 0;
    }
    consumer_barrier(kStepConsumerThreads);
    return *s_flag != 0;
}

// This CTA's row pairs of a GEMV phase, then pipeline w's contiguous share [p0, p1).
__device__ __forceinline__ void gemv_share(const GemvArgs& a, int w, int& p0, int& p1) {
    const int groups = a.n_rows / kRowsPerGroup;
    const int g0 = (int)(((long long)blockIdx.x * groups) / gridDim.x);
    const int g1 = (int)(((long long)(blockIdx.x + 1) * groups) / gridDim.x);
    const int ng = g1 - g0;
    p0 = g0 + (ng * w) / kGemvConsumerWarps;
    p1 = g0 + (ng * (w + 1)) / kGemvConsumerWarps;
}

// Per-pipeline ring state that survives from phase to phase.
struct PipeState {
    uint64_t* full;
    uint64_t* empty;
    unsigned char* ring;
    int slot;
    int pass;  // producer: completed trips; consumer: parity in bit 0
};

template <typename WT>
__device__ __forceinline__ bool produce_phase(const GemvArgs& a, PipeState& ps, int w, int NS, int slot_bytes,
                                              StepState* st) {
    int p0, p1;
    gemv_share(a, w, p0, p1);
    const unsigned char* W = reinterpret_cast<const unsigned char*>(a.W);
    const size_t row_bytes = (size_t)a.K * sizeof(WT);
    const int m = a.pairs_per_stage;
    auto issue = [&](const unsigned char* src, uint32_t bytes) -> bool {
        if (ps.pass > 0 && !mbar_wait_bounded(&ps.empty[ps.slot], (uint32_t)(ps.pass - 1) & 1u, &st->status))
            return false;
        mbar_arrive_expect_tx(&ps.full[ps.slot], bytes);
        bulk_g2s(ps.ring + (size_t)ps.slot * slot_bytes, src, bytes, &ps.full[ps.slot]);
        if (++ps.slot == NS) {
            ps.slot = 0;
            ++ps.pass;
        }
        return true;
    };
    if (m > 0) {
        for (int p = p0; p < p1; p += m) {
            const int cnt = min(m, p1 - p);
            if (!issue(W + (size_t)p * kRowsPerGroup * row_bytes, (uint32_t)(cnt * kRowsPerGroup * row_bytes)))
                return false;
        }
    } else {
        const int nch = (a.K + a.kc - 1) / a.kc;
        for (int p = p0; p < p1; ++p)
            for (int r = 0; r < kRowsPerGroup; ++r)
                for (int c = 0; c < nch; ++c) {
                    const int k0 = c * a.kc;
                    const int klen = min(a.kc, a.K - k0);
                    if (!issue(W + ((size_t)(p * kRowsPerGroup + r) * a.K + k0) * sizeof(WT), (uint32_t)(klen * sizeof(WT))))
                        return false;
                }
    }
    return true;
}

template <typename WT, int EPI>
__device__ __forceinline__ bool consume_phase(const GemvArgs& a, PipeState& ps, int w, int lane, int NS, int slot_bytes,
                                              const float* xs, StepState* st) {
    int p0, p1;
    gemv_share(a, w, p0, p1);
    const size_t row_bytes = (size_t)a.K * sizeof(WT);
    const int m = a.pairs_per_stage;
    auto acquire = [&]() -> bool {
        return __all_sync(0xffffffffu, mbar_wait_bounded(&ps.full[ps.slot], (uint32_t)ps.pass & 1u, &st->status));
    };
    auto release = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps.empty[ps.slot]);
        if (++ps.slot == NS) {
            ps.slot = 0;
            ps.pass ^= 1;
        }
    };
    if (m > 0) {
        for (int p = p0; p < p1; p += m) {
            const int cnt = min(m, p1 - p);
            // the residual value of the first pair is fetched before waiting for the weights, so its L2
            // round trip overlaps the wait instead of following the reduction
            float2 r_first = make_float2(0.f, 0.f);
            if (EPI == kEpiResid && a.resid && lane == 0)
                r_first = __ldcg(reinterpret_cast<const float2*>(a.resid + (size_t)p * kRowsPerGroup));
            if (!acquire()) return false;
            const unsigned char* stg = ps.ring + (size_t)ps.slot * slot_bytes;
            for (int i = 0; i < cnt; ++i) {
                float acc0 = 0.f, acc1 = 0.f;
                const unsigned char* r0 = stg + (size_t)i * kRowsPerGroup * row_bytes;
                dot_rows<WT, 2, false>(r0, r0 + row_bytes, xs, a.K, 0, a.K, lane, acc0, acc1);
                acc0 = warp_sum(acc0);
                acc1 = warp_sum(acc1);
                if (lane == 0) {
                    if (EPI == kEpiResid && i == 0) {
                        *reinterpret_cast<float2*>(a.out + (size_t)p * kRowsPerGroup) =
                            make_float2(acc0 + r_first.x, acc1 + r_first.y);
                    } else {
                        gemv_epilogue<EPI>(a, p + i, acc0, acc1);
                    }
                }
            }
            release();
        }
    } else {
        const int nch = (a.K + a.kc - 1) / a.kc;
        for (int p = p0; p < p1; ++p) {
            float acc[kRowsPerGroup] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < kRowsPerGroup; ++r)
                for (int c = 0; c < nch; ++c) {
                    if (!acquire()) return false;
                    const int k0 = c * a.kc;
                    const int klen = min(a.kc, a.K - k0);
                    const unsigned char* stg = ps.ring + (size_t)ps.slot * slot_bytes;
                    float dummy = 0.f;
                    dot_rows<WT, 1, false>(stg, stg, xs, a.K, k0, klen, lane, acc[r], dummy);
                    release();
                }
            const float v0 = warp_sum(acc[0]), v1 = warp_sum(acc[1]);
            if (lane == 0) gemv_epilogue<EPI>(a, p, v0, v1);
        }
    }
    return true;
}

template <typename WT, typename KT, int DPL, int GB>
__global__ void __launch_bounds__(kGemvRingThreads) step_kernel(const StepArgs sa) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kGemvConsumerWarps * kGemvMaxStages;
    float* red = reinterpret_cast<float*>(smem + kGemvBarrierBytes);  // 8 floats + barrier flag + attention flags
    int* s_flag = reinterpret_cast<int*>(smem + kGemvBarrierBytes + 64);
    float* xs = reinterpret_cast<float*>(smem + kGemvBarrierBytes + 128);
    unsigned char* ring = smem + kGemvBarrierBytes + 128 + sa.xs_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = sa.n_slots;
    if (tid == 0) s_flag[3] = 0;
    if (tid < kGemvConsumerWarps * NS) {
        const int bw = tid / NS, sl = tid - bw * NS;
        mbar_init(&full[bw * kGemvMaxStages + sl], 1);
        mbar_init(&empty[bw * kGemvMaxStages + sl], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int w = (warp == kGemvConsumerWarps) ? lane : warp;
    PipeState ps;
    if (w < kGemvConsumerWarps) {
        ps.full = full + w * kGemvMaxStages;
        ps.empty = empty + w * kGemvMaxStages;
        ps.ring = ring + (size_t)w * NS * sa.slot_bytes;
    }
    ps.slot = 0;
    ps.pass = 0;

    if (warp == kGemvConsumerWarps) {
        // ---------------- producer warp: streams the weights of every GEMV phase, back to back
        if (lane < kGemvConsumerWarps) {
            for (int i = 0; i < sa.count; ++i) {
                const StepPhase& ph = sa.phases[sa.first + i];
                if (ph.type != kPhaseGemv) continue;
                if (!produce_phase<WT>(ph.g, ps, w, NS, sa.slot_bytes, sa.st)) break;
            }
        }
        __syncwarp();
        if (lane == 0) pdl_launch_dependents();
        return;
    }

    // ---------------- consumers
    for (int i = 0; i < sa.count; ++i) {
        const StepPhase& ph = sa.phases[sa.first + i];
        unsigned long long* tr = (sa.trace && tid == 0) ? sa.trace + ((size_t)blockIdx.x * sa.count + i) * 4 : nullptr;
        if (tr) tr[0] = global_timer_ns();
        // phase i consumes what phase i-1 wrote (the first phase consumes the previous kernel's
        // output: stage_input / the attention body wait for that with griddepcontrol.wait)
        if (i > 0 && !grid_barrier(sa.gbar, (unsigned int)i * gridDim.x, sa.st, s_flag, tid)) return;
        if (tr) tr[1] = global_timer_ns();
        if (ph.type == kPhaseGemv) {
            stage_input<WT, kStepConsumerThreads>(ph.g, xs, red, tid);
            if (tr) tr[2] = global_timer_ns();
            bool ok;
            switch (ph.epi) {
                case kEpiStore: ok = consume_phase<WT, kEpiStore>(ph.g, ps, w, lane, NS, sa.slot_bytes, xs, sa.st); break;
                case kEpiResid: ok = consume_phase<WT, kEpiResid>(ph.g, ps, w, lane, NS, sa.slot_bytes, xs, sa.st); break;
                case kEpiSwiglu: ok = consume_phase<WT, kEpiSwiglu>(ph.g, ps, w, lane, NS, sa.slot_bytes, xs, sa.st); break;
                default: ok = consume_phase<WT, kEpiQkv>(ph.g, ps, w, lane, NS, sa.slot_bytes, xs, sa.st); break;
            }
            // a warp whose wait ran out keeps taking part in the CTA's barriers (leaving would strand the
            // others in bar.sync); it raises the abort flag and the next grid barrier ends the kernel
            if (!ok) s_flag[3] = 1;
            if (tr) tr[3] = global_timer_ns();
        } else {
            pdl_wait();
            // two teams of 128 threads share out the (split, kv head, head batch) items
            const AttnArgs& at = ph.at;
            const int team = tid >> 7, t128 = tid & 127;
            const int pos = at.st->pos;
            const int T = (pos < 0 || pos >= at.seq_len) ? 0 : pos + 1;
            const int n_eff = attn_effective_splits(T, at.n_splits, at.min_chunk);
            const int n_z = at.gqa / GB;
            const int items = n_eff * at.n_kv_heads * n_z;
            float* scratch = xs + (size_t)team * (kAttnThreads / 32) * GB * (DPL * 8 + 2);
            for (int it = blockIdx.x * 2 + team; it < items; it += gridDim.x * 2) {
                const int split = it % n_eff;
                const int rest = it / n_eff;
                attn_item<KT, DPL, GB>(at, split, rest / n_z, rest % n_z, n_z, T, n_eff, scratch, s_flag + 1 + team, t128,
                                       2 + team, pos);
            }
            if (tr) tr[2] = tr[3] = global_timer_ns();
        }
    }
}

}  // namespace lpp
