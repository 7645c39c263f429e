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
            long long limit = 1 << 17;  // the engine's limit is fetched from global memory only after ~65 us
            bool fetched = false;
            while (true) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
                if (v >= target) break;
                if (clock64() - t0 > limit) {
                    if (!fetched) {
                        limit = wait_limit(st);
                        fetched = true;
                        continue;
                    }
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

// Sum of one double per thread over the block, returned to every thread.
__device__ __forceinline__ double block_sum_double(double v, double* s_warp, int tid) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((tid & 31) == 0) s_warp[tid >> 5] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < kSampleThreads / 32; ++w) t += s_warp[w];
    __syncthreads();
    return t;
}

// Stage helper: every thread owns four consecutive values x[0..3] (element indices base+4*tid+k,
// zero past the end).  Given the approximate prefix `pre` (double, exclusive) before the quad, the
// block writes its entry list for the sequential sum of these values.
static __device__ __noinline__ void emit_entries(const float (&x)[4], double pre, int first_elem, int n_valid_quads,
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
        const float lim = __uint_as_float((unsigned int)((e0 > -120 && e0 < 120 ? e0 : 0) + 127) << 23);  // 2^e0
        plain = (e0 == e1) && e0 > -120 && e0 < 120 && x[0] < lim && x[1] < lim && x[2] < lim && x[3] < lim;
    }
    // runs: maximal sequences of threads of one class (plain runs also share E)
    const int cls = !valid ? 2000 : (plain ? E : 1000);  // binades lie in (-120, 120): no clash with the markers
    const int prev = __shfl_up_sync(0xffffffffu, cls, 1);
    __shared__ int s_cls_last[kSampleThreads / 32];
    if (lane == 31) s_cls_last[tid >> 5] = cls;
    __syncthreads();
    const int before = (tid == 0) ? 3000 : (lane == 0 ? s_cls_last[(tid >> 5) - 1] : prev);
    // a quad outside the plain class is an entry of its own: it travels with its four values
    const bool start = valid && (cls != before || !plain);
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
    const bool last = valid && (cls != after || !plain);
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
// requested and the crossing was located).  A map moves the sum by an integer number of ulps inside
// one binade (or exactly onto the next power of two), which on the bit pattern of a positive float
// is a plain integer addition.
static __device__ __noinline__ bool walk_list(const ExactEntry* list, int count, const float* x, int n_total,
                                          const bool kStop, float r, int lane, WalkState& w) {
    unsigned int bits = __float_as_uint(w.s);
    int4 nh = *reinterpret_cast<const int4*>(&list[0]);
    ulonglong2 nd = *reinterpret_cast<const ulonglong2*>(&list[0].d0);
    for (int i = 0; i < count; ++i) {
        const int4 h = nh;  // kind, lo, hi, e
        const ulonglong2 d = nd;
        const int nx = min(i + 1, count - 1);  // fetched while this entry is applied
        nh = *reinterpret_cast<const int4*>(&list[nx]);
        nd = *reinterpret_cast<const ulonglong2*>(&list[nx].d0);
        if (h.x == kEntryMap) {
            const unsigned int ebase = (unsigned int)(h.w + 127) << 23;
            const unsigned long long dd = (bits & 1u) ? d.y : d.x;
            const unsigned int nb = bits + (unsigned int)dd;
            // sum inside binade e before, and inside it or exactly on its upper end after
            if (bits - ebase < 0x800000u && dd <= 0x800000ull && nb - ebase <= 0x800000u) {
                if (kStop && r < __uint_as_float(nb)) {  // the first crossing lies inside this run
                    w.run_lo = h.y;
                    w.run_hi = min(h.z, n_total);
                    w.run_e = h.w;
                    w.run_s0 = __uint_as_float(bits);
                    w.s = __uint_as_float(bits);
                    return true;
                }
                bits = nb;
                continue;
            }
        } else if (h.x == kEntryQuad) {
            const float v[4] = {__uint_as_float((unsigned int)d.x), __uint_as_float((unsigned int)(d.x >> 32)),
                                __uint_as_float((unsigned int)d.y), __uint_as_float((unsigned int)(d.y >> 32))};
            float s = __uint_as_float(bits);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s = __fadd_rn(s, v[j]);
                if (kStop && r < s) {
                    w.found = h.y + j;
                    w.s = s;
                    return true;
                }
            }
            bits = __float_as_uint(s);
            continue;
        }
        // one-by-one FP32 additions from global memory, 32 loads at a time (oversized blocks, failed predictions)
        float s = __uint_as_float(bits);
        const int hi = min(h.z, n_total);
        for (int b = h.y; b < hi; b += 32) {
            const float v = (b + lane < hi) ? __ldcg(x + b + lane) : 0.f;
            const int m = min(32, hi - b);
            for (int j = 0; j < m; ++j) {
                s = __fadd_rn(s, __shfl_sync(0xffffffffu, v, j));
                if (kStop && r < s) {
                    w.found = b + j;
                    w.s = s;
                    return true;
                }
            }
        }
        bits = __float_as_uint(s);
    }
    w.s = __uint_as_float(bits);
    return false;
}

// Whole-block walk.  The blocks' entry lists are concatenated in block order (a prefix sum of the
// counts gives every entry its place), staged into shared memory kExactListCap at a time, and
// applied by warp 0.  Returns the final state in *out (shared memory).
static __device__ __noinline__ void walk_all(const ExactEntry* entries, const int* counts, int n_blocks, const float* x,
                                         int n_total, bool stop, float r, ExactEntry* s_list, int* s_pref, int* s_i,
                                         WalkState* out, int tid) {
    static_assert(kSampleMaxBlocks <= kSampleThreads, "one thread per block's count");
    const int lane = tid & 31;
    __shared__ int s_done;
    __shared__ int s_ctl[2];                          // first failed entry, first crossing entry
    __shared__ unsigned int s_before[kExactListCap + 1];  // bit pattern of the sum before every staged entry
    // inclusive prefix of the counts: thread t owns block t
    int c = (tid < n_blocks) ? __ldcg(counts + tid) : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, c, o);
        if (lane >= o) c += u;
    }
    if (lane == 31) s_i[tid >> 5] = c;
    if (tid == 0) {
        out->s = 0.f;
        out->found = -1;
        out->run_lo = -1;
        out->run_hi = out->run_e = 0;
        out->run_s0 = 0.f;
        s_done = 0;
        s_pref[0] = 0;
    }
    __syncthreads();
    int off = 0;
    for (int w = 0; w < (tid >> 5); ++w) off += s_i[w];
    s_pref[tid + 1] = c + off;
    __syncthreads();
    const int tot = s_pref[n_blocks];
    for (int base = 0; base < tot; base += kExactListCap) {
        const int m = min(kExactListCap, tot - base);
        for (int j = tid; j < m; j += kSampleThreads) {
            const int g = base + j;
            int lo = 0, hi = n_blocks;  // s_pref[lo] <= g < s_pref[hi]: entry g belongs to block lo
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (s_pref[mid] <= g)
                    lo = mid;
                else
                    hi = mid;
            }
            const uint4* src = reinterpret_cast<const uint4*>(entries + (size_t)lo * kExactMaxEntries + (g - s_pref[lo]));
            uint4* dst = reinterpret_cast<uint4*>(s_list + j);
            const uint4 v0 = __ldcg(src), v1 = __ldcg(src + 1);
            dst[0] = v0;
            dst[1] = v1;
        }
        __syncthreads();
        // pass 1 (warp 0, every lane the same): apply the entries speculatively without a branch, keeping the
        // sum before every entry; the first entry whose prediction fails (or that needs the one-by-one path)
        // is remembered
        if (tid < 32) {
            unsigned int bits = __float_as_uint(out->s);
            int bad = 0x7fffffff;
#pragma unroll 4
            for (int i = 0; i < m; ++i) {
                const int4 h = *reinterpret_cast<const int4*>(&s_list[i]);  // kind, lo, hi, e
                const ulonglong2 d = *reinterpret_cast<const ulonglong2*>(&s_list[i].d0);
                s_before[i] = bits;
                // as a map
                const unsigned int ebase = (unsigned int)(h.w + 127) << 23;
                const unsigned long long dd = (bits & 1u) ? d.y : d.x;
                const unsigned int nb = bits + (unsigned int)dd;
                const bool map_ok = bits - ebase < 0x800000u && dd <= 0x800000ull && nb - ebase <= 0x800000u;
                // as four values
                float q = __uint_as_float(bits);
                q = __fadd_rn(q, __uint_as_float((unsigned int)d.x));
                q = __fadd_rn(q, __uint_as_float((unsigned int)(d.x >> 32)));
                q = __fadd_rn(q, __uint_as_float((unsigned int)d.y));
                q = __fadd_rn(q, __uint_as_float((unsigned int)(d.y >> 32)));
                const bool is_map = h.x == kEntryMap;
                const bool fine = is_map ? map_ok : (h.x == kEntryQuad);
                bad = (!fine && bad == 0x7fffffff) ? i : bad;
                bits = is_map ? nb : __float_as_uint(q);
            }
            s_before[m] = bits;
            if (lane == 0) {
                s_ctl[0] = bad;
                s_ctl[1] = 0x7fffffff;
            }
        }
        __syncthreads();
        const int bad = s_ctl[0];
        const int good = min(m, bad);  // entries [0, good) were applied exactly
        // pass 2: the first entry after which the running sum exceeds r (sums never decrease)
        if (stop) {
            for (int i = tid; i < good; i += kSampleThreads)
                if (r < __uint_as_float(s_before[i + 1])) atomicMin(&s_ctl[1], i);
            __syncthreads();
        }
        const int cross = stop ? s_ctl[1] : 0x7fffffff;
        if (cross < good) {
            if (tid == 0) {
                const ExactEntry e = s_list[cross];
                float sum = __uint_as_float(s_before[cross]);
                if (e.kind == kEntryQuad) {
                    const float v[4] = {__uint_as_float((unsigned int)e.d0), __uint_as_float((unsigned int)(e.d0 >> 32)),
                                        __uint_as_float((unsigned int)e.d1), __uint_as_float((unsigned int)(e.d1 >> 32))};
                    int j = 0;
                    for (; j < 3; ++j) {
                        sum = __fadd_rn(sum, v[j]);
                        if (r < sum) break;
                    }
                    out->found = e.lo + j;
                } else {  // inside a map run: the caller redoes the run element by element
                    out->run_lo = e.lo;
                    out->run_hi = min(e.hi, n_total);
                    out->run_e = e.e;
                    out->run_s0 = sum;
                }
                out->s = sum;
                s_done = 1;
            }
        } else if (bad < m) {
            // a prediction failed: warp 0 goes on from that entry with the checked walk
            if (tid < 32) {
                WalkState w = *out;
                w.s = __uint_as_float(s_before[bad]);
                const bool done = walk_list(s_list + bad, m - bad, x, n_total, stop, r, lane, w);
                if (lane == 0) {
                    *out = w;
                    if (done) s_done = 1;
                }
            }
        } else if (tid == 0) {
            out->s = __uint_as_float(s_before[m]);
        }
        __syncthreads();
        if (s_done) break;
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
    __shared__ int s_pref[kSampleThreads + 1];
    __shared__ WalkState s_walk;
    __shared__ int s_hist[kHistoryMax];

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
    // ---- stage 0: penalty, temperature, block maximum (element i of the block lives in s_val[i])
    for (int i = tid; i < kSampleChunk; i += kSampleThreads) s_val[i] = (i < n) ? __ldcg(a.logits + base + i) : 0.f;
    __syncthreads();
    if (penalty > 1.0f && hist_len > 0) {
        // the history is scanned by every thread that owns one of its entries: keep it in shared memory
        for (int i = tid; i < hist_len; i += kSampleThreads) s_hist[i] = st->history[i];
        __syncthreads();
        for (int i = tid; i < hist_len; i += kSampleThreads) {
            const int tok = s_hist[i];
            if (tok < base || tok >= base + n) continue;
            bool first = true;
            for (int j = 0; j < i; ++j)
                if (s_hist[j] == tok) {
                    first = false;
                    break;
                }
            if (!first) continue;
            int cnt = 1;
            for (int j = i + 1; j < hist_len; ++j) cnt += (s_hist[j] == tok);
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
    bool alive = sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);

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
        alive = sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);

        // ---- stage 2: entry list of the sequential sum of e
        // approximate sum of e over the blocks before this one (loads in parallel, then a block reduction)
        double mine = 0.0;
        for (int b = tid; b < (int)blockIdx.x; b += kSampleThreads) mine += __ldcg(ea.block_sum + b);
        const double before_blocks = block_sum_double(mine, s_d, tid);
        if (alive) {
            emit_entries(x, before_blocks + (incl - loc), base, n_quads, ea.entries + (size_t)blockIdx.x * kExactMaxEntries,
                         ea.entry_count + blockIdx.x, s_wm, s_wf, s_i, tid);
            __threadfence();
        }
        alive = alive && sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);

        // ---- stage 3: block 0, warp 0 walks the entries: the exact softmax denominator
        if (alive && blockIdx.x == 0) {
            walk_all(ea.entries, ea.entry_count, nb, a.logits, a.vocab, false, 0.f, s_list, s_pref, s_i, &s_walk, tid);
            if (tid == 0) {
                __stcg(ea.scalars, s_walk.s);
                __threadfence();
            }
        }
        alive = alive && sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);

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
        alive = alive && sampler_grid_barrier(&ea.sync[0], ++bar * nb, st, &s_flag, tid);

        // ---- stage 5: block 0 finds the first index whose running sum exceeds r
        if (alive && blockIdx.x == 0) {
            const float r = st->advance ? a.r_values[st->step_idx] : st->r;
            walk_all(ea.entries, ea.entry_count, nb, a.logits, a.vocab, true, r, s_list, s_pref, s_i, &s_walk, tid);
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
                    const float cum = (S >= (1ull << 24))
                                          ? __uint_as_float((unsigned int)(E + 128) << 23)
                                          : __uint_as_float(((unsigned int)(E + 127) << 23) | ((unsigned int)S & 0x7fffffu));
                    if (q + k < run_hi && r < cum) atomicMin(&s_found, q + k);
                }
                __syncthreads();
            }
            token = (s_found != 0x7fffffff) ? s_found : a.vocab - 1;
        }
    }

    // ---- exit ticket: the last block to get here publishes the result and resets the counters
    __syncthreads();
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
        if (a.bump && tid == 0) *a.bump = *a.bump + 1u;
    }
}

}  // namespace lpp
