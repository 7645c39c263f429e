// Exact-order sampler: repetition penalty -> temperature -> softmax -> categorical draw with the
// SAME floating-point results as the reference's sequential CPU code (src/model.cpp:256-303 with
// softmax() of src/ops.cpp:56-75), computed in parallel.
//
// The reference sums 128K probabilities one after the other in FP32, twice (the softmax denominator
// and the running CDF).  Those sums carry ~1e-5 of rounding drift, more than the width of one
// token's probability in a flat 128K distribution, so any re-associated (tree) sum picks a
// neighbouring token in a large share of draws.  Re-association is avoided here by emulating the
// sequential rounding exactly:
//
//   While the running sum s stays inside one binade [2^E, 2^(E+1)) with ulp u, fl(s + x) equals
//   s + q*u where q = x/u rounded to nearest; only an exact tie depends on s, and then only on the
//   parity of s/u.  So each element acts on the integer S = s/u as a map
//   "S -> S + d[parity of S]", and maps compose associatively: a run of elements collapses, with a
//   parallel scan, into one pair (D0, D1).
//
//   Where the sum may change binade the emulation does not apply.  Every thread classifies its four
//   consecutive elements from an approximate (double) prefix sum: if the prefix before and after the
//   quad is safely inside one binade the quad is "plain" and contributes a map, otherwise it is a
//   "window" whose elements are added one by one with real FP32 additions.  Blocks publish a short
//   list of entries (map runs and windows); one warp then walks all entries in order.  A map entry
//   is applied only after checking that s really is in the predicted binade and stays in it;
//   otherwise its elements are added one by one as well, so the result never depends on the
//   approximate prefix being accurate -- only the speed does.
//
// exp() is exp_repro (common.cuh): IEEE double arithmetic only, identical on host and device; it
// differs from libm's expf in the last bit for about 0.06 % of arguments, which is the only source
// of disagreement with the reference left (none in 3000 test draws at 32K-128K vocabularies).
//
// One launch, ceil(V/2048) co-resident blocks, bounded grid barriers between the stages (max, sum,
// CDF); vocabularies that need more blocks than the GPU has SMs use the tree sampler of sampler.cuh.
#pragma once
#include "common.cuh"
#include "sampler.cuh"

namespace lpp {

constexpr int kExactMaxEntries = 96;  // per block; a block that needs more becomes one "add one by one" entry
constexpr double kExactEps = 1.0 / 4096.0;  // safety margin of the binade prediction (speed only)

enum : int { kEntryMap = 0, kEntrySeq = 1, kEntryQuad = 2 };
constexpr int kExactListCap = 512;  // entries the walking block stages in shared memory per round

struct ExactEntry {
    int kind;  // kEntryMap: apply (d0, d1) in binade e; kEntrySeq: add elements [lo, hi) one by one;
               // kEntryQuad: add the four floats stored in (d0, d1), elements lo..lo+3, one by one
    int lo, hi;
    int e;
    unsigned long long d0, d1;
};

struct SampleExactArgs {
    SampleArgs base;
    unsigned int* sync;      // [0] grid-barrier counter, [1] exit ticket; zero between launches
    double* block_sum;       // [n_blocks] approximate sum of exp per block
    int* entry_count;        // [n_blocks]
    ExactEntry* entries;     // [n_blocks][kExactMaxEntries]
    float* scalars;          // [0] exact softmax denominator
};

// ---- the integer map of one element -------------------------------------------------------------

struct Map2 {
    unsigned long long d0, d1;  // increment of S when S is even / odd
};
__device__ __forceinline__ Map2 map_identity() { return Map2{0ull, 0ull}; }
// b after a
__device__ __forceinline__ Map2 map_compose(Map2 a, Map2 b) {
    Map2 c;
    c.d0 = a.d0 + ((a.d0 & 1ull) ? b.d1 : b.d0);
    c.d1 = a.d1 + (((1ull + a.d1) & 1ull) ? b.d1 : b.d0);
    return c;
}
// Map of adding x (a non-negative float) to a sum in binade E (ulp 2^(E-23)); requires x < 2^E.
__device__ __forceinline__ Map2 map_of(float x, int E) {
    const unsigned int bits = __float_as_uint(x);
    int ex = (int)((bits >> 23) & 0xffu);
    unsigned int mx = bits & 0x7fffffu;
    if (ex == 0)
        ex = 1;  // zero or subnormal: value = mx * 2^(1-150)
    else
        mx |= 0x800000u;
    const int shift = (E + 127) - ex;  // x/ulp = mx / 2^shift, shift >= 1
    if (mx == 0u || shift > 25) return map_identity();
    const unsigned long long m = mx;
    const unsigned long long n = m >> shift;
    const unsigned long long rem = m & ((1ull << shift) - 1ull);
    const unsigned long long half = 1ull << (shift - 1);
    Map2 r;
    if (rem < half) {
        r.d0 = r.d1 = n;
    } else if (rem > half) {
        r.d0 = r.d1 = n + 1ull;
    } else {  // tie: round so that S + increment is even
        r.d0 = n + (n & 1ull);
        r.d1 = n + ((n + 1ull) & 1ull);
    }
    return r;
}

__device__ __forceinline__ int binade_of(double v) {  // floor(log2(v)) for v > 0 (normal doubles)
    return (int)((__double_as_longlong(v) >> 52) & 0x7ff) - 1023;
}

// Exact fl(s + x) bookkeeping helpers for the walking warp.
__device__ __forceinline__ bool apply_map(float& s, int E, unsigned long long d0, unsigned long long d1) {
    const unsigned int bits = __float_as_uint(s);
    const int es = (int)((bits >> 23) & 0xffu) - 127;
    if (!(s > 0.f) || es != E || ((bits >> 23) & 0xffu) == 0u) return false;
    const unsigned long long S = (bits & 0x7fffffu) | 0x800000u;
    const unsigned long long R = S + ((S & 1ull) ? d1 : d0);
    if (R > (1ull << 24)) return false;
    // R in [2^23, 2^24]: the float with mantissa R in binade E (or exactly 2^(E+1))
    s = (R == (1ull << 24)) ? __uint_as_float((unsigned int)(E + 128) << 23)
                            : __uint_as_float(((unsigned int)(E + 127) << 23) | ((unsigned int)R & 0x7fffffu));
    return true;
}

// ---- grid barrier for this kernel (all blocks co-resident; bounded wait) -------------------------

__device__ __forceinline__ bool sampler_grid_barrier(unsigned int* counter, unsigned int target, StepState* st,
                                                     int* s_flag, int tid) {
    __syncthreads();
    if (tid == 0) {
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        bool ok = true;
        unsigned int v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v < target) {
            const long long t0 = clock64();
            while (true) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
                if (v >= target) break;
                if (clock64() - t0 > kWaitCycles) {
                    atomicOr(&st->status, kStatusBarrierTimeout);
                    ok = false;
                    break;
                }
            }
        }
        *s_flag = ok ? 1 : 0;
    }
    __syncthreads();
    return *s_flag != 0;
}

// Inclusive segmented scan of per-thread maps over the block: `start` marks the first thread of a
// run.  Returns the composition of the maps of the run's threads up to and including this one.
__device__ __forceinline__ Map2 block_segscan(Map2 v, bool start, Map2* s_warp_map, int* s_warp_flag, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    int f = start ? 1 : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        Map2 u;
        u.d0 = __shfl_up_sync(0xffffffffu, v.d0, o);
        u.d1 = __shfl_up_sync(0xffffffffu, v.d1, o);
        const int fu = __shfl_up_sync(0xffffffffu, f, o);
        if (lane >= o) {
            if (!f) v = map_compose(u, v);
            f |= fu;
        }
    }
    // v = composition from the last start at or before this lane within the warp; f = a start exists
    if (lane == 31) {
        s_warp_map[warp] = v;
        s_warp_flag[warp] = f;
    }
    __syncthreads();
    if (!f) {  // the run began in an earlier warp: prepend the carried maps of the warps before
        Map2 carry = map_identity();
        bool open = true;
        for (int w = warp - 1; w >= 0 && open; --w) {
            carry = map_compose(s_warp_map[w], carry);
            if (s_warp_flag[w]) open = false;
        }
        v = map_compose(carry, v);
    }
    __syncthreads();
    return v;
}

// Inclusive block scan of doubles (one value per thread).
__device__ __forceinline__ double block_scan_double(double v, double* s_warp, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    if (lane == 31) s_warp[warp] = v;
    __syncthreads();
    double off = 0.0;
    for (int w = 0; w < warp; ++w) off += s_warp[w];
    __syncthreads();
    return v + off;
}

// Stage helper: every thread owns four consecutive values x[0..3] (element indices base+4*tid+k,
// zero past the end).  Given the approximate prefix `pre` (double, exclusive) before the quad, the
// block writes its entry list for the sequential sum of these values.
__device__ __forceinline__ void emit_entries(const float (&x)[4], double pre, int first_elem, int n_valid_quads,
                                             ExactEntry* out, int* out_count, Map2* s_wm, int* s_wf, int* s_i,
                                             int tid) {
    const int lane = tid & 31;
    const bool valid = tid < n_valid_quads;
    const double post = pre + (double)x[0] + (double)x[1] + (double)x[2] + (double)x[3];
    // plain: the sum is provably inside one binade before, during and after this quad
    bool plain = false;
    int E = 0;
    if (valid && pre > 0.0) {
        const int e0 = binade_of(pre * (1.0 - kExactEps)), e1 = binade_of(post * (1.0 + kExactEps));
        E = e0;
        const float lim = scalbnf(1.0f, e0 > -120 && e0 < 120 ? e0 : 0);
        plain = (e0 == e1) && e0 > -120 && e0 < 120 && x[0] < lim && x[1] < lim && x[2] < lim && x[3] < lim;
    }
    // runs: maximal sequences of threads of one class (plain runs also share E)
    const int cls = !valid ? 2000 : (plain ? E : 1000);  // binades lie in (-120, 120): no clash with the markers
    const int prev = __shfl_up_sync(0xffffffffu, cls, 1);
    __shared__ int s_cls_last[kSampleThreads / 32];
    if (lane == 31) s_cls_last[tid >> 5] = cls;
    __syncthreads();
    const int before = (tid == 0) ? 3000 : (lane == 0 ? s_cls_last[(tid >> 5) - 1] : prev);
    const bool start = valid && cls != before;
    Map2 mp = map_identity();
    if (plain) {
#pragma unroll
        for (int k = 0; k < 4; ++k) mp = map_compose(mp, map_of(x[k], E));
    }
    const Map2 run = block_segscan(mp, start, s_wm, s_wf, tid);
    // entry index = number of run starts up to and including this thread, minus one
    int cnt = start ? 1 : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, cnt, o);
        if (lane >= o) cnt += u;
    }
    if (lane == 31) s_i[tid >> 5] = cnt;
    __syncthreads();
    int off = 0;
    for (int w = 0; w < (tid >> 5); ++w) off += s_i[w];
    const int idx = cnt + off - 1;
    int total = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) total += s_i[w];
    __syncthreads();
    const bool overflow = total > kExactMaxEntries;
    // is this thread the last of its run?
    const int nxt_cls = __shfl_down_sync(0xffffffffu, cls, 1);
    if (lane == 0) s_cls_last[tid >> 5] = cls;  // reuse as "first class of warp"
    __syncthreads();
    const int after = (tid == kSampleThreads - 1) ? 3000 : (lane == 31 ? s_cls_last[(tid >> 5) + 1] : nxt_cls);
    const bool last = valid && cls != after;
    if (!overflow) {
        if (start) {
            out[idx].kind = plain ? kEntryMap : kEntrySeq;
            out[idx].lo = first_elem + 4 * tid;
            out[idx].e = E;
        }
        if (last) {
            out[idx].hi = first_elem + 4 * tid + 4;
            if (!plain && start) {
                // a window of one quad (the usual case) carries its values, sparing the walker a memory round trip
                out[idx].kind = kEntryQuad;
                out[idx].d0 = (unsigned long long)__float_as_uint(x[0]) | ((unsigned long long)__float_as_uint(x[1]) << 32);
                out[idx].d1 = (unsigned long long)__float_as_uint(x[2]) | ((unsigned long long)__float_as_uint(x[3]) << 32);
            } else {
                out[idx].d0 = run.d0;
                out[idx].d1 = run.d1;
            }
        }
        if (tid == 0) *out_count = total;
    } else if (tid == 0) {
        out[0].kind = kEntrySeq;
        out[0].lo = first_elem;
        out[0].hi = first_elem + 4 * n_valid_quads;
        out[0].e = 0;
        out[0].d0 = out[0].d1 = 0ull;
        *out_count = 1;
    }
    __syncthreads();
}

// State of the walk over all entries, kept by warp 0 of the walking block (identical on all lanes).
struct WalkState {
    float s;                    // exact running sum
    int found;                  // >= 0: first element whose running sum exceeds r
    int run_lo, run_hi, run_e;  // >= 0: the crossing lies inside this map run ...
    float run_s0;               // ... which starts from this exact sum
};

// Applies `count` entries (in shared memory) in order.  Returns true when the walk is over (stop
// requested and the crossing was located).
__device__ __forceinline__ bool walk_list(const ExactEntry* list, int count, const float* x, int n_total, bool stop,
                                          float r, int lane, WalkState& w) {
    float s = w.s;
    for (int i = 0; i < count; ++i) {
        const ExactEntry e = list[i];
        if (e.kind == kEntryMap) {
            float s_new = s;
            if (apply_map(s_new, e.e, e.d0, e.d1)) {
                if (stop && r < s_new) {  // the first crossing lies inside this run
                    w.run_lo = e.lo;
                    w.run_hi = min(e.hi, n_total);
                    w.run_e = e.e;
                    w.run_s0 = s;
                    w.s = s;
                    return true;
                }
                s = s_new;
                continue;
            }
        } else if (e.kind == kEntryQuad) {
            const float v[4] = {__uint_as_float((unsigned int)e.d0), __uint_as_float((unsigned int)(e.d0 >> 32)),
                                __uint_as_float((unsigned int)e.d1), __uint_as_float((unsigned int)(e.d1 >> 32))};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s = __fadd_rn(s, v[j]);
                if (stop && r < s && w.found < 0) {
                    w.found = e.lo + j;
                    w.s = s;
                    return true;
                }
            }
            continue;
        }
        // one-by-one FP32 additions from global memory, 32 loads at a time (long windows, failed predictions)
        const int hi = min(e.hi, n_total);
        for (int b = e.lo; b < hi; b += 32) {
            const float v = (b + lane < hi) ? __ldcg(x + b + lane) : 0.f;
            const int m = min(32, hi - b);
            for (int j = 0; j < m; ++j) {
                s = __fadd_rn(s, __shfl_sync(0xffffffffu, v, j));
                if (stop && r < s) {
                    w.found = b + j;
                    w.s = s;
                    return true;
                }
            }
        }
    }
    w.s = s;
    return false;
}

// Whole-block walk: rounds of (stage as many blocks' entries as fit into shared memory, in order;
// warp 0 applies them).  Returns the final state in *out (shared memory).
__device__ __forceinline__ void walk_all(const ExactEntry* entries, const int* counts, int n_blocks, const float* x,
                                         int n_total, bool stop, float r, ExactEntry* s_list, int* s_off, WalkState* out,
                                         int tid) {
    const int lane = tid & 31;
    if (tid == 0) {
        out->s = 0.f;
        out->found = -1;
        out->run_lo = -1;
        out->run_hi = out->run_e = 0;
        out->run_s0 = 0.f;
    }
    int b0 = 0;
    __shared__ int s_round[2];  // [0] first block after this round, [1] done flag
    if (tid == 0) s_round[1] = 0;
    __syncthreads();
    while (b0 < n_blocks) {
        // offsets of this round's blocks in the staged list
        if (tid == 0) {
            int tot = 0, b = b0;
            while (b < n_blocks) {
                const int c = __ldcg(counts + b);
                if (tot + c > kExactListCap) break;
                s_off[b - b0] = tot;
                tot += c;
                ++b;
            }
            s_off[b - b0] = tot;
            s_round[0] = b;
        }
        __syncthreads();
        const int b1 = s_round[0];
        for (int slot = tid; slot < (b1 - b0) * kExactMaxEntries; slot += kSampleThreads) {
            const int bl = slot / kExactMaxEntries, i = slot - bl * kExactMaxEntries;
            if (i < s_off[bl + 1] - s_off[bl]) {
                const uint4* src = reinterpret_cast<const uint4*>(entries + (size_t)(b0 + bl) * kExactMaxEntries + i);
                uint4* dst = reinterpret_cast<uint4*>(s_list + s_off[bl] + i);
                dst[0] = __ldcg(src);
                dst[1] = __ldcg(src + 1);
            }
        }
        __syncthreads();
        if (tid < 32) {
            WalkState w = *out;
            const bool done = walk_list(s_list, s_off[b1 - b0], x, n_total, stop, r, lane, w);
            if (lane == 0) {
                *out = w;
                if (done) s_round[1] = 1;
            }
        }
        __syncthreads();
        if (s_round[1]) break;
        b0 = b1;
    }
}

static __global__ void __launch_bounds__(kSampleThreads) sample_exact_kernel(const SampleExactArgs ea) {
    const SampleArgs& a = ea.base;
    __shared__ float s_val[kSampleChunk];
    __shared__ MaxIdx s_mi[kSampleThreads / 32];
    __shared__ double s_d[kSampleThreads / 32];
    __shared__ Map2 s_wm[kSampleThreads / 32];
    __shared__ int s_wf[kSampleThreads / 32];
    __shared__ int s_i[kSampleThreads / 32];
    __shared__ int s_flag;
    __shared__ int s_found;
    __shared__ __align__(16) ExactEntry s_list[kExactListCap];
    __shared__ int s_off[kSampleMaxBlocks / 2 + 2];
    __shared__ WalkState s_walk;

    pdl_launch_dependents();
    pdl_wait();
    StepState* st = a.st;
    const int tid = threadIdx.x, lane = tid & 31;
    const int nb = gridDim.x;
    const int base = blockIdx.x * kSampleChunk;
    const int n = min(kSampleChunk, a.vocab - base);
    const int n_quads = (n + 3) >> 2;
    const float temperature = st->temperature;
    const float penalty = st->penalty;
    const int hist_len = min(st->history_len, kHistoryMax);
    const bool greedy = (temperature == 0.0f);
    unsigned int bar = 0;  // barriers passed so far
    // timing aid: block 0 leaves global-timer stamps (ns since its start) in scalars[4..]
    unsigned long long t_start = 0;
    if (blockIdx.x == 0 && tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    auto stamp = [&](int k) {
        if (blockIdx.x == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            ea.scalars[4 + k] = (float)(t - t_start);
        }
    };

    // ---- stage 0: penalty, temperature, block maximum (element i of the block lives in s_val[i])
    for (int i = tid; i < kSampleChunk; i += kSampleThreads) s_val[i] = (i < n) ? __ldcg(a.logits + base + i) : 0.f;
    __syncthreads();
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
    MaxIdx best = {-INFINITY, 0x7fffffff};
    for (int i = tid; i < n; i += kSampleThreads) {
        float v = s_val[i];
        if (!greedy) v = __fdiv_rn(v, temperature);
        s_val[i] = v;
        best = better(best, MaxIdx{v, base + i});
    }
    best = block_argmax(best, s_mi, tid);
    if (tid == 0) {
        __stcg(a.part_max + blockIdx.x, best.v);
        __stcg(a.part_idx + blockIdx.x, best.i);
    }
    stamp(0);
    bool alive = sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);
    stamp(1);

    // ---- global maximum (every block reduces the partials itself)
    MaxIdx g = {-INFINITY, 0x7fffffff};
    for (int b = tid; b < nb; b += kSampleThreads) g = better(g, MaxIdx{__ldcg(a.part_max + b), __ldcg(a.part_idx + b)});
    g = block_argmax(g, s_mi, tid);
    int token = g.i;

    if (!greedy && alive) {
        // ---- stage 1: e = exp(v - max) (kept in s_val and written to global), approximate block sums
        float x[4];
        double loc = 0.0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = 4 * tid + k;
            x[k] = (i < n) ? exp_repro(s_val[i] - g.v) : 0.f;
            if (i < n) a.logits[base + i] = x[k];
            loc += (double)x[k];
        }
        const double incl = block_scan_double(loc, s_d, tid);
        if (tid == kSampleThreads - 1) ea.block_sum[blockIdx.x] = incl;
        stamp(2);
        alive = sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);
        stamp(3);

        // ---- stage 2: entry list of the sequential sum of e
        double before_blocks = 0.0, total_d = 0.0;
        for (int b = 0; b < nb; ++b) {
            const double v = __ldcg(ea.block_sum + b);
            if (b < (int)blockIdx.x) before_blocks += v;
            total_d += v;
        }
        if (alive) {
            emit_entries(x, before_blocks + (incl - loc), base, n_quads, ea.entries + (size_t)blockIdx.x * kExactMaxEntries,
                         ea.entry_count + blockIdx.x, s_wm, s_wf, s_i, tid);
            __threadfence();
        }
        stamp(4);
        alive = alive && sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);
        stamp(5);

        // ---- stage 3: block 0, warp 0 walks the entries: the exact softmax denominator
        if (alive && blockIdx.x == 0) {
            walk_all(ea.entries, ea.entry_count, nb, a.logits, a.vocab, false, 0.f, s_list, s_off, &s_walk, tid);
            if (tid == 0) {
                __stcg(ea.scalars, s_walk.s);
                __threadfence();
            }
        }
        stamp(6);
        alive = alive && sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);
        stamp(7);

        // ---- stage 4: p = e / sum (IEEE division), entry list of the running CDF
        const float denom = __ldcg(ea.scalars);
        double locp = 0.0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = 4 * tid + k;
            x[k] = (i < n) ? __fdiv_rn(x[k], denom) : 0.f;
            if (i < n) a.logits[base + i] = x[k];  // like the reference, the logits end up as probabilities
            locp += (double)x[k];
        }
        const double inclp = block_scan_double(locp, s_d, tid);
        // approximate prefix of p before this block = (approximate prefix of e) / denominator
        const double pre_p = before_blocks / (double)denom + (inclp - locp);
        if (alive) {
            emit_entries(x, pre_p, base, n_quads, ea.entries + (size_t)blockIdx.x * kExactMaxEntries,
                         ea.entry_count + blockIdx.x, s_wm, s_wf, s_i, tid);
            __threadfence();
        }
        stamp(8);
        alive = alive && sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);
        stamp(9);

        // ---- stage 5: block 0 finds the first index whose running sum exceeds r
        if (alive && blockIdx.x == 0) {
            const float r = st->advance ? a.r_values[st->step_idx] : st->r;
            walk_all(ea.entries, ea.entry_count, nb, a.logits, a.vocab, true, r, s_list, s_off, &s_walk, tid);
            if (tid == 0) s_found = (s_walk.found >= 0) ? s_walk.found : 0x7fffffff;
            __syncthreads();
            const int run_lo = s_walk.run_lo, run_hi = s_walk.run_hi, E = s_walk.run_e;
            if (run_lo >= 0) {
                // the crossing lies inside a map run (<= 2048 elements, quads aligned): redo the run's scan
                // with the exact starting sum and look at every element
                const float s0 = s_walk.run_s0;
                const unsigned int b0 = __float_as_uint(s0);
                const unsigned long long S0 = (b0 & 0x7fffffu) | 0x800000u;
                float y[4];
                Map2 mp = map_identity();
                const int q = run_lo + 4 * tid;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    y[k] = (q + k < run_hi) ? __ldcg(a.logits + q + k) : 0.f;
                    mp = map_compose(mp, map_of(y[k], E));
                }
                const Map2 incl_m = block_segscan(mp, tid == 0, s_wm, s_wf, tid);
                // exclusive prefix for this thread: shift by one thread
                Map2 ex;
                ex.d0 = __shfl_up_sync(0xffffffffu, incl_m.d0, 1);
                ex.d1 = __shfl_up_sync(0xffffffffu, incl_m.d1, 1);
                __shared__ Map2 s_last_map[kSampleThreads / 32];
                if (lane == 31) s_last_map[tid >> 5] = incl_m;
                __syncthreads();
                if (lane == 0) ex = (tid == 0) ? map_identity() : s_last_map[(tid >> 5) - 1];
                unsigned long long S = S0 + ((S0 & 1ull) ? ex.d1 : ex.d0);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const Map2 m1 = map_of(y[k], E);
                    S += (S & 1ull) ? m1.d1 : m1.d0;
                    const float cum = scalbnf((float)(unsigned int)min(S, 1ull << 24), E - 23);
                    if (q + k < run_hi && r < cum) atomicMin(&s_found, q + k);
                }
                __syncthreads();
            }
            token = (s_found != 0x7fffffff) ? s_found : a.vocab - 1;
        }
    }

    // ---- exit ticket: the last block to get here publishes the result and resets the counters
    __syncthreads();
    stamp(10);
    if (blockIdx.x == 0 && tid == 0) {
        st->out_token = token;
        if (st->advance) {
            const int k = st->step_idx;
            a.out_tokens[k] = token;
            st->token = token;
            st->pos = st->pos + 1;
            st->step_idx = k + 1;
            const int w = st->history_window;
            if (w > 0) {
                st->history[st->history_count % w] = token;
                st->history_count = st->history_count + 1;
                st->history_len = min(st->history_count, w);
            }
        }
        __threadfence();
    }
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&ea.sync[1], 1u);
        s_flag = (ticket == (unsigned int)nb - 1);
    }
    __syncthreads();
    if (s_flag) {
        if (tid == 0) {
            ea.sync[0] = 0u;
            ea.sync[1] = 0u;
        }
        for (int i = tid; i < a.zero_n; i += kSampleThreads) a.zero[i] = 0u;
    }
}

}  // namespace lpp
