// Host side of the B200 decode engine: device memory layout, weight repacking, the per-token
// CUDA graph and the C ABI declared in include/lpp_b200.h.
//
// Stands in for the device halves of malloc_run_state / free_run_state (src/model.cpp:18-118),
// attention / transformer_block / forward (src/model.cpp:121-384, USE_CUDA branches) and the upload
// code of the loaders (src/loader.cpp:73-131, 543-637) of the reference tree.
//
// Device layout (per tensor-parallel rank; Dq = local query rows, KVd = local kv rows, Fl = local
// FFN columns):
//   wqkv [L][Dq + 2*KVd][D]   rows q | k | v of one layer back to back  -> one fused GEMV
//   wo   [L][D][Dq]           column slice of the reference wo, repacked contiguous
//   w13  [L][2*Fl][D]         gate row i and up row i interleaved         -> SwiGLU in the epilogue
//   w2   [L][D][Fl]           column slice of the reference w2
//   emb / wcls [V][D]         weight dtype; wcls aliases emb when the classifier is tied
//   K, V cache [L][KVHl][S][hs]   FP16 (or FP32), the reference's index order
//   rope [S][hs/2] (cos, sin)     built on the host with libm so rotations match the CPU path bit
//                                 for bit
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../include/lpp_b200.h"
#include "attention.cuh"
#include "common.cuh"
#include "gemv.cuh"
#include "ops.cuh"
#include "prefill.cuh"
#include "sampler.cuh"
#include "sampler_exact.cuh"

using namespace lpp;

// ------------------------------------------------------------------ error plumbing

static thread_local std::string g_err;
static lpp_status fail(lpp_status s, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return s;
}
void lpp_internal_set_error(const char* msg) { g_err = msg ? msg : ""; }
#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess)                                                                     \
            return fail(LPP_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)
#define TRY(call)                      \
    do {                               \
        lpp_status s_ = (call);        \
        if (s_ != LPP_OK) return s_;   \
    } while (0)

// Timing aids: environment switches that change what a step launches (kernel kinds left out, arithmetic
// skipped, stage sizes, prefetch depth ...).  Some make the results meaningless, so they exist only in
// builds made with -DLPP_TIMING_AIDS; the product build never looks at them.
#ifdef LPP_TIMING_AIDS
static const char* aid_env(const char* name) { return getenv(name); }
#else
static const char* aid_env(const char*) { return nullptr; }
#endif

// LPP_TRACE=1 in the environment prints one line per host-side phase and synchronises after every
// launch of an un-graphed step, to localise a failing kernel.
static bool tracing() {
    static int t = -1;
    if (t < 0) t = getenv("LPP_TRACE") ? 1 : 0;
    return t == 1;
}
#define TRACE(...)                        \
    do {                                  \
        if (tracing()) {                  \
            fprintf(stderr, "[lpp] " __VA_ARGS__); \
            fprintf(stderr, "\n");        \
            fflush(stderr);               \
        }                                 \
    } while (0)

// ------------------------------------------------------------------ NCCL through dlopen
// Only tensor-parallel engines need NCCL, so it is bound at run time; a single-GPU process never
// loads it.  The handful of prototypes below follow nccl.h.

namespace nccl {
typedef struct ncclComm* comm_t;
typedef struct { char internal[128]; } unique_id;
typedef int result_t;
static void* lib = nullptr;
static result_t (*GetUniqueId)(unique_id*);
static result_t (*CommInitRank)(comm_t*, int, unique_id, int);
static result_t (*CommDestroy)(comm_t);
static result_t (*AllReduce)(const void*, void*, size_t, int /*dtype*/, int /*op*/, comm_t, cudaStream_t);
static const char* (*GetErrorString)(result_t);
constexpr int kFloat32 = 7, kSum = 0;
static bool load() {
    if (lib) return true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) return false;
    GetUniqueId = (decltype(GetUniqueId))dlsym(lib, "ncclGetUniqueId");
    CommInitRank = (decltype(CommInitRank))dlsym(lib, "ncclCommInitRank");
    CommDestroy = (decltype(CommDestroy))dlsym(lib, "ncclCommDestroy");
    AllReduce = (decltype(AllReduce))dlsym(lib, "ncclAllReduce");
    GetErrorString = (decltype(GetErrorString))dlsym(lib, "ncclGetErrorString");
    return GetUniqueId && CommInitRank && CommDestroy && AllReduce && GetErrorString;
}
}  // namespace nccl

// ------------------------------------------------------------------ engine

enum Kind { kQkv = 0, kAttn = 1, kOproj = 2, kGateUp = 3, kDown = 4, kLmHead = 5, kSampler = 6, kAllReduce = 7, kKinds = 10 };

struct lpp_engine {
    lpp_config c;
    int hs, Hl, KVHl, Dq, KVd, Fl, gqa;
    int esz, kvesz;
    int num_sms;
    int attn_splits, attn_gb, attn_z;
    int attn_splits_long;  // splits of the tensor-core kernel: one CTA per SM, one wave
    int sample_blocks;
    size_t smem_optin;
    cudaStream_t stream = nullptr;
    // weights
    void *wqkv = nullptr, *wo = nullptr, *w13 = nullptr, *w2 = nullptr, *emb = nullptr, *wcls = nullptr;
    float *rms_att = nullptr, *rms_ffn = nullptr, *rms_final = nullptr;
    bool wcls_owned = false;
    bool wcls_shard_only = false;  // an untied classifier of a tensor-parallel rank holds this rank's vocabulary rows only
    std::vector<unsigned char> got;  // upload bookkeeping: [tensor][layer]
    // state
    void *kcache = nullptr, *vcache = nullptr;
    float *xa = nullptr, *xb = nullptr, *q = nullptr, *att_out = nullptr, *hb = nullptr, *logits = nullptr;
    float *attn_part = nullptr, *samp_max = nullptr, *samp_sum = nullptr, *r_values = nullptr;
    int *samp_idx = nullptr, *out_tokens = nullptr;
    unsigned int *attn_counters = nullptr, *samp_counter = nullptr;
    // exact-order sampler scratch
    bool exact_sampler = false;
    unsigned int* ex_sync = nullptr;
    double* ex_block_sum = nullptr;
    int* ex_entry_count = nullptr;
    ExactEntry* ex_entries = nullptr;
    float* ex_scalars = nullptr;
    float2* rope = nullptr;
    StepState* st = nullptr;
    int run_cap = 0;  // capacity of r_values / out_tokens
    // host staging (pinned)
    StepState* h_st = nullptr;
    int* h_out = nullptr;  // out_token, status
    // upload staging
    void* stage = nullptr;
    size_t stage_bytes = 0;
    // tensor-parallel exchange over peer memory: per exchange (2 per layer) a receive area [tp][dim] floats
    // and two counters; peer_base[p] = rank p's buffer as mapped into this process (own buffer for p == rank)
    unsigned char* tp_buf = nullptr;
    size_t tp_buf_bytes = 0;
    unsigned char* peer_base[kMaxTp] = {};
    bool peer_ready = false;
    unsigned char* absent_peer = nullptr;  // test aid: where stores to ranks that do not exist go (lpp_debug_tp_absent_peers)
    unsigned long long* gtrace = nullptr;  // LPP_GEMV_TRACE: per-launch per-CTA time stamps of the ring GEMV
    // graphs
    // graph variants by context length; only [0] is used at present
    cudaGraphExec_t g_full[2] = {nullptr, nullptr}, g_logits[2] = {nullptr, nullptr};

    // batched prompt path (allocated by the first lpp_prefill)
    float *pf_x = nullptr, *pf_q = nullptr, *pf_part = nullptr;
    __half *pf_xn = nullptr, *pf_att = nullptr, *pf_hb = nullptr;
    int* pf_tokens = nullptr;
    CUtensorMap pf_map_wqkv, pf_map_wo, pf_map_w13, pf_map_w2, pf_map_xn, pf_map_att, pf_map_hb;
    bool pf_ready = false;

    bool finalized = false;
    int kernels_full = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // NCCL
    nccl::comm_t comm = nullptr;
    // profiling hooks
    bool profiling = false;
    bool profiling_capture = false;
    int only_kind = -1;  // lpp_profile_kind: the one kind recorded
    std::vector<cudaEvent_t> prof_events;
    std::vector<int> prof_kinds;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <typename... KArgs, typename... Args>
static cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// ---- GEMV dispatch

struct GemvPlan {
    dim3 grid;
    int threads;
    size_t smem;
};

constexpr int kStageTarget = 8192;  // bytes per bulk copy / ring slot (see gemv.cuh)

// A stage is one bulk copy of about stage_target bytes: whole row pairs when they fit, else one
// K-chunk of one row.
static void gemv_geometry(GemvArgs& a, int esz, int stage_target) {
    const int pair_bytes = kRowsPerGroup * a.K * esz;
    if (pair_bytes <= stage_target) {
        a.pairs_per_stage = stage_target / pair_bytes;
        a.kc = a.K;
        a.stage_bytes = a.pairs_per_stage * pair_bytes;
    } else {
        a.pairs_per_stage = 0;
        a.kc = std::max(8, std::min(a.K, stage_target / esz) / 8 * 8);
        a.stage_bytes = a.kc * esz;
    }
}

template <typename WT, int EPI>
static cudaError_t launch_gemv_t(lpp_engine* e, GemvArgs& a, bool pdl, cudaStream_t s) {
    const int esz = sizeof(WT);
    const int groups = a.n_rows / kRowsPerGroup;
    const size_t xbytes = align_up((size_t)a.K * 4, 128);
    if (e->c.flags & LPP_FLAG_GEMV_LDG) {
        const size_t smem = 128 + xbytes;
        static bool attr_done[64] = {};
        if (!attr_done[e->c.device & 63]) {
            cudaError_t r = cudaFuncSetAttribute(gemv_ldg_kernel<WT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)e->smem_optin);
            if (r != cudaSuccess) return r;
            attr_done[e->c.device & 63] = true;
        }
        const int grid = std::max(1, std::min(groups, e->num_sms * 4));
        return launch_kernel(gemv_ldg_kernel<WT, EPI>, dim3(grid), dim3(kGemvLdgThreads), smem, s, pdl, a);
    }
    // LPP_STAGE_KB (timing experiments) overrides the 8 KiB stage size.
    int stage_target = kStageTarget;
    if (const char* sk = aid_env("LPP_STAGE_KB")) stage_target = std::max(1, atoi(sk)) * 1024;
    gemv_geometry(a, esz, stage_target);
    const size_t fixed = kGemvBarrierBytes + 128 + xbytes;
    size_t ring = (size_t)(e->c.ring_kb > 0 ? e->c.ring_kb : 128) * 1024;
    if (fixed + ring > e->smem_optin) ring = e->smem_optin - fixed;
    int ns = (int)(ring / ((size_t)kGemvConsumerWarps * a.stage_bytes));  // slots per consumer warp
    ns = std::max(2, std::min(ns, kGemvMaxStages));
    const int grid = std::max(1, std::min(groups, e->num_sms));
    a.n_stages = ns;
    const size_t smem = fixed + (size_t)kGemvConsumerWarps * ns * a.stage_bytes;
    if (smem > e->smem_optin) return cudaErrorInvalidValue;
    static bool attr_done[64] = {};
    if (!attr_done[e->c.device & 63]) {
        cudaError_t r = cudaFuncSetAttribute(gemv_ring_kernel<WT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)e->smem_optin);
        if (r != cudaSuccess) return r;
        attr_done[e->c.device & 63] = true;
    }
    return launch_kernel(gemv_ring_kernel<WT, EPI>, dim3(grid), dim3(kGemvRingThreads), smem, s, pdl, a);
}

static cudaError_t launch_gemv(lpp_engine* e, int epi, int w_dtype, GemvArgs& a, bool pdl, cudaStream_t s) {
#define LPP_GEMV_CASE(E)                                                          \
    case E:                                                                       \
        return w_dtype == LPP_F16 ? launch_gemv_t<__half, E>(e, a, pdl, s)        \
                                  : launch_gemv_t<float, E>(e, a, pdl, s);
    switch (epi) {
        LPP_GEMV_CASE(kEpiStore)
        LPP_GEMV_CASE(kEpiResid)
        LPP_GEMV_CASE(kEpiSwiglu)
        LPP_GEMV_CASE(kEpiQkv)
    }
#undef LPP_GEMV_CASE
    return cudaErrorInvalidValue;
}

// ---- attention dispatch

template <typename KT, int DPL>
static cudaError_t launch_attn_d(lpp_engine* e, const AttnArgs& a, dim3 grid, bool pdl, cudaStream_t s) {
    switch (e->attn_gb) {
        case 4:
            return launch_kernel(attn_decode_kernel<KT, DPL, 4>, grid, dim3(kAttnKernelThreads), 0, s, pdl, a);
        case 2:
            return launch_kernel(attn_decode_kernel<KT, DPL, 2>, grid, dim3(kAttnKernelThreads), 0, s, pdl, a);
        default:
            return launch_kernel(attn_decode_kernel<KT, DPL, 1>, grid, dim3(kAttnKernelThreads), 0, s, pdl, a);
    }
}
template <typename KT>
static cudaError_t launch_attn_t(lpp_engine* e, const AttnArgs& a, dim3 grid, bool pdl, cudaStream_t s) {
    switch (e->hs / 8) {
        case 2: return launch_attn_d<KT, 2>(e, a, grid, pdl, s);
        case 4: return launch_attn_d<KT, 4>(e, a, grid, pdl, s);
        case 6: return launch_attn_d<KT, 6>(e, a, grid, pdl, s);
        case 8: return launch_attn_d<KT, 8>(e, a, grid, pdl, s);
        case 12: return launch_attn_d<KT, 12>(e, a, grid, pdl, s);
        case 16: return launch_attn_d<KT, 16>(e, a, grid, pdl, s);
    }
    return cudaErrorInvalidValue;
}

// Attention with the scores and P.V on the tensor cores (FP16 cache, head size 64 or 128, 1/2/4/8 query heads
// per KV head); other shapes keep the CUDA-core kernel.
static cudaError_t launch_attn_mma(lpp_engine* e, const AttnArgs& a, bool pdl, cudaStream_t s) {
    if (e->c.kv_dtype != LPP_F16) return cudaErrorNotSupported;
    const dim3 grid(a.n_splits, e->KVHl, 1), block(kAttnKernelThreads);
#define LPP_MMA_CASE(HS_, G_) \
    if (e->hs == HS_ && e->gqa == G_) return launch_kernel(attn_mma_kernel<HS_, G_>, grid, block, 0, s, pdl, a);
    LPP_MMA_CASE(64, 1) LPP_MMA_CASE(64, 2) LPP_MMA_CASE(64, 4) LPP_MMA_CASE(64, 8)
    LPP_MMA_CASE(128, 1) LPP_MMA_CASE(128, 2) LPP_MMA_CASE(128, 4) LPP_MMA_CASE(128, 8)
#undef LPP_MMA_CASE
    return cudaErrorNotSupported;
}
static bool attn_mma_supported(const lpp_engine* e) {
    return e->c.kv_dtype == LPP_F16 && (e->hs == 64 || e->hs == 128) && (e->gqa == 1 || e->gqa == 2 || e->gqa == 4 || e->gqa == 8);
}

// ---- one decode step as a sequence of launches (captured into the graph, or run directly)

struct Recorder {
    lpp_engine* e;
    cudaStream_t s;
    bool prev_kernel = false;  // previous stream item was one of our kernels -> PDL edge allowed
    int kernels = 0;
    bool long_ctx = false;  // record the long-context variant of the step (tensor-core attention kernel)
    cudaError_t err = cudaSuccess;
    std::string where;

    bool pdl() const { return prev_kernel && !(e->c.flags & LPP_FLAG_NO_PDL) && !e->profiling; }
    void mark(int kind) {
        if (!e->profiling) return;
        cudaEvent_t ev;
        cudaEventCreate(&ev);
        if (e->profiling_capture)
            cudaEventRecordWithFlags(ev, s, cudaEventRecordExternal);  // becomes an event-record graph node
        else
            cudaEventRecord(ev, s);
        e->prof_events.push_back(ev);
        e->prof_kinds.push_back(kind);
    }
    void check(cudaError_t r, const char* what) {
        if (r != cudaSuccess && err == cudaSuccess) {
            err = r;
            where = what;
        }
        if (tracing() && (e->c.flags & LPP_FLAG_NO_GRAPH)) {
            TRACE("launched %s #%d -> %s; syncing", what, kernels, cudaGetErrorString(r));
            cudaError_t se = cudaStreamSynchronize(s);
            TRACE("  sync -> %s", cudaGetErrorString(se));
        }
    }
};

// LPP_DEBUG_SKIP=<bitmask of Kind> leaves those kernels out of the step (results become
// meaningless): a timing aid that shows what each kernel kind costs inside the replayed graph.
static unsigned skip_mask() {
    const char* v = aid_env("LPP_DEBUG_SKIP");
    return v ? (unsigned)strtol(v, nullptr, 0) : 0u;
}
// only_kind >= 0 (lpp_profile_kind): every other kind is left out of the recorded sequence.
static bool kind_skipped(const lpp_engine* e, int kind) {
    return (skip_mask() & (1u << kind)) || (e->only_kind >= 0 && kind != e->only_kind);
}

static void record_gemv(Recorder& R, int kind, int epi, GemvArgs a) {
    lpp_engine* e = R.e;
    if (kind_skipped(e, kind)) return;
    a.st = e->st;
    if (const char* dbg = aid_env("LPP_DEBUG_GEMV")) a.debug = (int)strtol(dbg, nullptr, 0);
    if (aid_env("LPP_GEMV_TRACE")) {
        if (e->gtrace && R.kernels < 256) a.trace = e->gtrace + (size_t)R.kernels * e->num_sms * 8;
    }
    a.vocab = e->c.vocab_size;
    a.seq_len = e->c.seq_len;
    R.mark(kind);
    R.check(launch_gemv(e, epi, e->c.weight_dtype, a, R.pdl(), R.s), "gemv launch");
    R.mark(-1);
    R.prev_kernel = true;
    R.kernels++;
}

static void record_allreduce(Recorder& R, float* buf, int n) {
    lpp_engine* e = R.e;
    if (kind_skipped(e, kAllReduce)) return;
    R.mark(kAllReduce);
    nccl::result_t r = nccl::AllReduce(buf, buf, (size_t)n, nccl::kFloat32, nccl::kSum, e->comm, R.s);
    if (r != 0 && R.err == cudaSuccess) {
        R.err = cudaErrorUnknown;
        R.where = std::string("ncclAllReduce: ") + nccl::GetErrorString(r);
    }
    R.mark(-1);
    R.prev_kernel = false;
}

static bool tp_peer_path(const lpp_engine* e);
static bool tp_cls_sharded(const lpp_engine* e);
static unsigned int* tp_epoch_word(const lpp_engine* e);

// The fused sampler: exact-order kernel by default, tree kernel when asked for or when the vocabulary
// needs more blocks than can be co-resident.
static cudaError_t launch_sampler(lpp_engine* e, cudaStream_t s, bool pdl, bool end_of_step = false) {
    SampleArgs a = {};
    a.logits = e->logits;
    a.vocab = e->c.vocab_size;
    a.st = e->st;
    a.part_max = e->samp_max;
    a.part_idx = e->samp_idx;
    a.part_sum = e->samp_sum;
    a.counter = e->samp_counter;
    a.r_values = e->r_values;
    a.out_tokens = e->out_tokens;
    a.bump = (end_of_step && tp_peer_path(e)) ? tp_epoch_word(e) : nullptr;
    if (e->exact_sampler) {
        SampleExactArgs ea = {};
        ea.base = a;
        ea.sync = e->ex_sync;
        ea.block_sum = e->ex_block_sum;
        ea.entry_count = e->ex_entry_count;
        ea.entries = e->ex_entries;
        ea.scalars = e->ex_scalars;
        return launch_kernel(sample_exact_kernel, dim3(e->sample_blocks), dim3(kSampleThreads), 0, s, pdl, ea);
    }
    return launch_kernel(sample_kernel, dim3(e->sample_blocks), dim3(kSampleThreads), 0, s, pdl, a);
}

// Start and size of the weight matrix a GEMV kind streams in layer l (this rank's share).
static void matrix_span(const lpp_engine* e, int kind, int l, const void** ptr, size_t* bytes) {
    const size_t D = e->c.dim, esz = e->esz;
    const size_t qkv_rows = e->Dq + 2 * (size_t)e->KVd;
    switch (kind) {
        case kQkv: *bytes = qkv_rows * D * esz; *ptr = (const char*)e->wqkv + l * *bytes; break;
        case kOproj: *bytes = D * e->Dq * esz; *ptr = (const char*)e->wo + l * *bytes; break;
        case kGateUp: *bytes = 2 * (size_t)e->Fl * D * esz; *ptr = (const char*)e->w13 + l * *bytes; break;
        case kDown: *bytes = D * e->Fl * esz; *ptr = (const char*)e->w2 + l * *bytes; break;
        default:
            *bytes = (size_t)e->c.vocab_size * D * esz;
            *ptr = e->wcls;
            if (tp_cls_sharded(e)) {  // this rank's vocabulary rows
                *bytes /= e->c.tp_size;
                if (!e->wcls_shard_only) *ptr = (const char*)e->wcls + (size_t)e->c.tp_rank * *bytes;
            }
            break;
    }
}
// What the GEMV (kind, l) should pull towards L2 for its successor in the step: the next matrix, or
// its first LPP_PF_MB MiB (default 8) when it is larger.  The classifier's successor is the first
// layer's QKV matrix of the next token.
static void set_prefetch(const lpp_engine* e, GemvArgs& a, int kind, int l) {
    int nk, nl = l;
    switch (kind) {
        case kQkv: nk = kOproj; break;
        case kOproj: nk = kGateUp; break;
        case kGateUp: nk = kDown; break;
        case kDown: nk = (l + 1 < e->c.n_layers) ? kQkv : kLmHead; nl = l + 1; break;
        default: nk = kQkv; nl = 0; break;
    }
    if (e->c.tp_size < 2) return;  // one GPU: no measurable effect, so a launch's DRAM traffic stays its matrix once
    size_t cap = 8;
    if (const char* v = aid_env("LPP_PF_MB")) cap = (size_t)std::max(0, atoi(v));
    const void* p;
    size_t bytes;
    matrix_span(e, nk, nl, &p, &bytes);
    bytes = std::min(bytes, cap << 20) & ~(size_t)15;
    a.pf = bytes ? p : nullptr;
    a.pf_bytes = (unsigned int)bytes;
}

// ---- tensor-parallel exchange buffer layout: [epoch word, padded to 256 B][2 * n_layers receive areas],
//      a receive area = [tp][dim] 64-bit {value, flag} words
static size_t tp_header_bytes() { return 1024; }  // epoch word at 0, hint counters (one per exchange) from byte 256
static size_t tp_area_bytes(const lpp_engine* e) { return (size_t)e->c.tp_size * e->c.dim * sizeof(unsigned long long); }
static unsigned long long* tp_area(const lpp_engine* e, int p, int ex) {
    return reinterpret_cast<unsigned long long*>(e->peer_base[p] + tp_header_bytes() + (size_t)ex * tp_area_bytes(e));
}
static unsigned int* tp_epoch_word(const lpp_engine* e) { return reinterpret_cast<unsigned int*>(e->tp_buf); }
static unsigned int* tp_hint(const lpp_engine* e, int p, int ex) { return reinterpret_cast<unsigned int*>(e->peer_base[p] + 256) + ex; }
// The arrival hint spares the receive area the polling of every thread of every CTA; with two ranks that
// polling is light and measured faster (2051 against 2078 us/step on the 8B shape), so the hint is used from
// three ranks on (LPP_TP_HINT=0/1 overrides).
static bool tp_use_hint(const lpp_engine* e) {
    if (2 * e->c.n_layers > 192) return false;
    if (const char* v = aid_env("LPP_TP_HINT")) return atoi(v) != 0;
    return e->c.tp_size > 2;
}
static unsigned int tp_hint_per_step(const lpp_engine* e) {
    const int groups = e->c.dim / kRowsPerGroup;  // the producing GEMVs have dim rows
    return (unsigned int)(e->c.tp_size * std::max(1, std::min(groups, e->num_sms)));
}
// (a single-kind timing run must not take part in exchanges: its producers would have no consumers)
static bool tp_peer_path(const lpp_engine* e) {
    return e->c.tp_size > 1 && e->peer_ready && e->only_kind < 0 &&
           !(e->c.flags & (LPP_FLAG_GEMV_LDG | LPP_FLAG_TP_NCCL));
}
// producer side: exchange `ex` takes the rows of this residual GEMV
static void tp_set_producer(const lpp_engine* e, GemvArgs& a, int ex) {
    const bool use_hint = tp_use_hint(e);
    a.tp_size = e->c.tp_size;
    a.tp_epoch = tp_epoch_word(e);
    for (int p = 0; p < e->c.tp_size; ++p) {
        a.tp_out[p] = tp_area(e, p, ex) + (size_t)e->c.tp_rank * e->c.dim;
        a.tp_hint_out[p] = use_hint ? tp_hint(e, p, ex) : nullptr;
    }
}
// consumer side: this GEMV's input is the sum of the slots of exchange `ex`
static void tp_set_consumer(const lpp_engine* e, GemvArgs& a, int ex, float* x_store) {
    a.tp_size = e->c.tp_size;
    a.tp_epoch = tp_epoch_word(e);
    a.tp_in = tp_area(e, e->c.tp_rank, ex);
    a.tp_hint_in = tp_use_hint(e) ? tp_hint(e, e->c.tp_rank, ex) : nullptr;
    a.tp_wait_cycles = e->h_st->tp_wait_cycles > 0 ? e->h_st->tp_wait_cycles : kTpWaitCycles;
    a.tp_hint_per_step = tp_hint_per_step(e);
    a.x = nullptr;
    a.x_store = x_store;
}

// The classifier is sharded by vocabulary rows when the peers are mapped: every rank computes
// vocab/tp logits and stores them, as flagged words, into every rank's logits area (after the
// exchange areas of the buffer); a small kernel turns the words into the float logits the sampler reads.
static bool tp_cls_sharded(const lpp_engine* e) {
    return e->c.tp_size > 1 && tp_peer_path(e) && e->c.vocab_size % (kRowsPerGroup * e->c.tp_size) == 0 && !aid_env("LPP_TP_FULL_CLS");
}
static unsigned long long* tp_logits_area(const lpp_engine* e, int p) {
    return reinterpret_cast<unsigned long long*>(e->peer_base[p] + tp_header_bytes() + (size_t)2 * e->c.n_layers * tp_area_bytes(e));
}

// words [0, n) = {logit, flag}: waits for the local classifier kernel (so that its CTAs, which this kernel's
// CTAs would otherwise sit beside, are not slowed by polling), then polls until every word, local or from a
// peer, carries this step's flag (bounded) and writes the floats.
static __global__ void __launch_bounds__(256) tp_unpack_logits_kernel(const unsigned long long* words, float* logits, int n,
                                                                    const unsigned int* epoch, StepState* st, long long limit) {
    pdl_launch_dependents();
    pdl_wait();
    const unsigned int flag = *epoch + 1u;
    const int i = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (i >= n) return;
    unsigned long long w[4];
    long long t0 = 0;
    while (true) {
        asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[0]), "=l"(w[1]) : "l"(words + i) : "memory");
        asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[2]), "=l"(w[3]) : "l"(words + i + 2) : "memory");
        bool pending = false;
#pragma unroll
        for (int q = 0; q < 4; ++q) pending |= (i + q < n) && (unsigned int)(w[q] >> 32) != flag;
        if (!pending) break;
        if (t0 == 0) {
            if (status_timed_out(st)) break;
            t0 = clock64();
        } else if (clock64() - t0 > limit) {
            atomicOr(&st->status, kStatusBarrierTimeout);
            break;
        }
        __nanosleep(40);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
        if (i + q < n) logits[i + q] = __uint_as_float((unsigned int)w[q]);
}

// Ends a step that has no sampler kernel: bumps the exchange epoch.
static __global__ void tp_bump_kernel(unsigned int* epoch) {
    pdl_wait();
    *epoch = *epoch + 1u;
}

static void record_step(Recorder& R, bool with_sampler) {
    lpp_engine* e = R.e;
    const lpp_config& c = e->c;
    const int D = c.dim, L = c.n_layers;
    const size_t esz = e->esz;
    const int qkv_rows = e->Dq + 2 * e->KVd;
    const bool tp = c.tp_size > 1;
    const bool peers = tp_peer_path(e);  // fused exchange over peer memory instead of an NCCL all-reduce
    float* cur = e->xa;
    float* oth = e->xb;
    for (int l = 0; l < L; ++l) {
        {  // fused RMSNorm + QKV GEMV + RoPE + KV scatter
            GemvArgs a = {};
            a.W = (const char*)e->wqkv + (size_t)l * qkv_rows * D * esz;
            a.n_rows = qkv_rows;
            a.K = D;
            a.norm_w = e->rms_att + (size_t)l * D;
            if (l == 0) {
                a.emb = e->emb;
                a.x_store = cur;
            } else {
                a.x = cur;
                if (peers) tp_set_consumer(e, a, 2 * (l - 1) + 1, cur);  // the previous layer's down exchange
            }
            a.out = e->q;
            a.q_rows = e->Dq;
            a.kv_rows = e->KVd;
            a.head_size = e->hs;
            a.rope = e->rope;
            const size_t lofs = (size_t)l * e->KVHl * c.seq_len * e->hs * e->kvesz;
            a.k_cache = (char*)e->kcache + lofs;
            a.v_cache = (char*)e->vcache + lofs;
            a.kv_is_f32 = c.kv_dtype == LPP_F32;
            // split-KV flash decode
            AttnArgs at = {};
            at.q = e->q;
            at.k_cache = a.k_cache;
            at.v_cache = a.v_cache;
            at.out = e->att_out;
            at.part = e->attn_part;
            at.counters = e->attn_counters;
            at.st = e->st;
            at.seq_len = c.seq_len;
            at.head_size = e->hs;
            at.gqa = e->gqa;
            at.n_splits = e->attn_splits;
            at.n_kv_heads = e->KVHl;
            if (const char* mc = aid_env("LPP_ATTN_CHUNK")) at.min_chunk = atoi(mc);  // timing experiments
            {
                set_prefetch(e, a, kQkv, l);
                record_gemv(R, kQkv, kEpiQkv, a);
                dim3 grid(e->attn_splits, e->KVHl, e->attn_z);
                if (!kind_skipped(e, kAttn)) {
                    if (e->gtrace && R.kernels < 256) at.trace = e->gtrace + (size_t)R.kernels * e->num_sms * 8;
                    R.mark(kAttn);
                    if (attn_mma_supported(e) && !aid_env("LPP_ATTN_CUDA_CORES")) {
                        at.n_splits = e->attn_splits_long;
                        R.check(launch_attn_mma(e, at, R.pdl(), R.s), "attention (tensor-core) launch");
                    } else {
                        R.check(c.kv_dtype == LPP_F32 ? launch_attn_t<float>(e, at, grid, R.pdl(), R.s)
                                                      : launch_attn_t<__half>(e, at, grid, R.pdl(), R.s),
                                "attention launch");
                    }
                    R.mark(-1);
                    R.prev_kernel = true;
                    R.kernels++;
                }
            }
        }
        {  // o_proj + residual
            GemvArgs a = {};
            a.W = (const char*)e->wo + (size_t)l * D * e->Dq * esz;
            a.n_rows = D;
            a.K = e->Dq;
            a.x = e->att_out;
            a.resid = (!tp || c.tp_rank == 0) ? cur : nullptr;
            a.out = tp ? oth : cur;
            if (peers) tp_set_producer(e, a, 2 * l);
            set_prefetch(e, a, kOproj, l);
            record_gemv(R, kOproj, kEpiResid, a);
            if (tp && !peers) {
                record_allreduce(R, oth, D);
                std::swap(cur, oth);
            }
        }
        {  // fused RMSNorm + gate|up GEMV + SwiGLU
            GemvArgs a = {};
            a.W = (const char*)e->w13 + (size_t)l * 2 * e->Fl * D * esz;
            a.n_rows = 2 * e->Fl;
            a.K = D;
            a.x = cur;
            if (peers) tp_set_consumer(e, a, 2 * l, cur);
            a.norm_w = e->rms_ffn + (size_t)l * D;
            a.out = e->hb;
            set_prefetch(e, a, kGateUp, l);
            record_gemv(R, kGateUp, kEpiSwiglu, a);
        }
        {  // down + residual
            GemvArgs a = {};
            a.W = (const char*)e->w2 + (size_t)l * D * e->Fl * esz;
            a.n_rows = D;
            a.K = e->Fl;
            a.x = e->hb;
            a.resid = (!tp || c.tp_rank == 0) ? cur : nullptr;
            a.out = tp ? oth : cur;
            if (peers) tp_set_producer(e, a, 2 * l + 1);
            set_prefetch(e, a, kDown, l);
            record_gemv(R, kDown, kEpiResid, a);
            if (tp && !peers) {
                record_allreduce(R, oth, D);
                std::swap(cur, oth);
            }
        }
    }
    {  // final RMSNorm + classifier
        GemvArgs a = {};
        a.W = e->wcls;
        a.n_rows = c.vocab_size;
        a.K = D;
        a.x = cur;
        if (peers) tp_set_consumer(e, a, 2 * (L - 1) + 1, cur);
        a.norm_w = e->rms_final;
        a.out = e->logits;
        const bool sharded = tp_cls_sharded(e);
        if (sharded) {
            const int Vl = c.vocab_size / c.tp_size, r0 = c.tp_rank * Vl;
            a.W = e->wcls_shard_only ? (const char*)e->wcls : (const char*)e->wcls + (size_t)r0 * D * esz;
            a.n_rows = Vl;
            for (int p = 0; p < c.tp_size; ++p) a.tp_out[p] = tp_logits_area(e, p) + r0;
        }
        set_prefetch(e, a, kLmHead, 0);
        record_gemv(R, kLmHead, kEpiStore, a);
        if (sharded && !kind_skipped(e, kLmHead)) {
            const int V = c.vocab_size;
            R.check(launch_kernel(tp_unpack_logits_kernel, dim3((V + 1023) / 1024), dim3(256), 0, R.s, R.pdl(),
                                  (const unsigned long long*)tp_logits_area(e, c.tp_rank), e->logits, V,
                                  (const unsigned int*)tp_epoch_word(e), e->st,
                                  (long long)(e->h_st->tp_wait_cycles > 0 ? e->h_st->tp_wait_cycles : kTpWaitCycles)),
                    "logits unpack launch");
            R.prev_kernel = true;
            R.kernels++;
        }
    }
    if (!with_sampler && tp_peer_path(e)) {
        // no sampler in this graph to end the step: a one-thread kernel bumps the exchange epoch
        R.check(launch_kernel(tp_bump_kernel, dim3(1), dim3(1), 0, R.s, R.pdl(), tp_epoch_word(e)), "epoch bump launch");
        R.prev_kernel = true;
    }
    if (with_sampler && !kind_skipped(e, kSampler)) {
        R.mark(kSampler);
        R.check(launch_sampler(e, R.s, R.pdl(), true), "sampler launch");
        R.mark(-1);
        R.prev_kernel = true;
        R.kernels++;
    }
}

static lpp_status capture(lpp_engine* e, bool with_sampler, bool long_ctx, cudaGraphExec_t* out, int* kernels) {
    cudaGraph_t g = nullptr;
    CU(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    Recorder R{e, e->stream};
    R.long_ctx = long_ctx;
    record_step(R, with_sampler);
    cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
    if (R.err != cudaSuccess) {
        if (g) cudaGraphDestroy(g);
        (void)cudaGetLastError();
        return fail(LPP_ERR_CUDA, "%s: %s", R.where.c_str(), cudaGetErrorString(R.err));
    }
    if (ce != cudaSuccess) return fail(LPP_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(ce));
    cudaError_t ie = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (ie != cudaSuccess) return fail(LPP_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(ie));
    if (kernels) *kernels = R.kernels;
    return LPP_OK;
}

// pos: the position this step runs at (known to the host in every mode); it selects the variant.
static lpp_status run_step(lpp_engine* e, bool with_sampler, int pos) {
    const int v = 0;  // a single graph variant serves every position
    (void)pos;
    if (e->c.flags & LPP_FLAG_NO_GRAPH) {
        Recorder R{e, e->stream};
        R.long_ctx = v == 1;
        record_step(R, with_sampler);
        if (R.err != cudaSuccess) return fail(LPP_ERR_CUDA, "%s: %s", R.where.c_str(), cudaGetErrorString(R.err));
        return LPP_OK;
    }
    CU(cudaGraphLaunch(with_sampler ? e->g_full[v] : e->g_logits[v], e->stream));
    return LPP_OK;
}

// ------------------------------------------------------------------ create / destroy

static bool dpl_supported(int hs) {
    const int d = hs / 8;
    return hs % 8 == 0 && (d == 2 || d == 4 || d == 6 || d == 8 || d == 12 || d == 16);
}

extern "C" lpp_status lpp_engine_create(const lpp_config* cfg, const void* nccl_id, lpp_engine** out) {
    if (!cfg || !out) return fail(LPP_ERR_INVALID_ARG, "null argument");
    *out = nullptr;
    const lpp_config& c = *cfg;
    if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 ||
        c.vocab_size <= 0 || c.seq_len <= 0)
        return fail(LPP_ERR_INVALID_ARG, "non-positive model dimension");
    if (c.dim % c.n_heads || c.n_heads % c.n_kv_heads)
        return fail(LPP_ERR_INVALID_ARG, "dim %% n_heads or n_heads %% n_kv_heads != 0");
    if (c.weight_dtype != LPP_F16 && c.weight_dtype != LPP_F32) return fail(LPP_ERR_INVALID_ARG, "bad weight_dtype");
    if (c.kv_dtype != LPP_F16 && c.kv_dtype != LPP_F32) return fail(LPP_ERR_INVALID_ARG, "bad kv_dtype");
    if (c.tp_size < 1 || c.tp_rank < 0 || c.tp_rank >= c.tp_size) return fail(LPP_ERR_INVALID_ARG, "bad tp rank/size");
    if (c.n_kv_heads % c.tp_size || c.hidden_dim % c.tp_size)
        return fail(LPP_ERR_INVALID_ARG, "tp_size %d must divide n_kv_heads %d and hidden_dim %d", c.tp_size,
                    c.n_kv_heads, c.hidden_dim);
    const int hs = c.dim / c.n_heads;
    if (!dpl_supported(hs)) return fail(LPP_ERR_INVALID_ARG, "head_size %d unsupported (16,32,48,64,96,128)", hs);
    const int vec = c.weight_dtype == LPP_F16 ? 8 : 4;
    const int Fl = c.hidden_dim / c.tp_size;
    const int Dq = c.dim / c.tp_size;
    if (c.dim % vec || Fl % vec || Dq % vec || (c.vocab_size & 1) || (Fl & 1))
        return fail(LPP_ERR_INVALID_ARG, "dim/hidden/vocab not multiples of the vector width");
    if (c.tp_size > 1 && !nccl_id && !(c.flags & LPP_FLAG_TP_LOCAL))
        return fail(LPP_ERR_INVALID_ARG, "tp_size > 1 needs an nccl id (or LPP_FLAG_TP_LOCAL)");
    if ((c.flags & LPP_FLAG_TP_LOCAL) && c.tp_size > kMaxTp)
        return fail(LPP_ERR_INVALID_ARG, "LPP_FLAG_TP_LOCAL supports at most %d ranks", kMaxTp);

    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        (void)cudaGetLastError();
        return fail(LPP_ERR_NO_DEVICE, "no CUDA device");
    }
    if (c.device < 0 || c.device >= ndev) return fail(LPP_ERR_INVALID_ARG, "device %d out of range", c.device);
    CU(cudaSetDevice(c.device));
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, c.device));
    if (prop.major < 10) return fail(LPP_ERR_NO_DEVICE, "device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);

    TRACE("create: device %d ok (%s, %d SMs)", c.device, prop.name, prop.multiProcessorCount);
    lpp_engine* e = new lpp_engine();
    e->c = c;
    e->hs = hs;
    e->Hl = c.n_heads / c.tp_size;
    e->KVHl = c.n_kv_heads / c.tp_size;
    e->Dq = Dq;
    e->KVd = e->KVHl * hs;
    e->Fl = Fl;
    e->gqa = c.n_heads / c.n_kv_heads;
    e->esz = c.weight_dtype == LPP_F16 ? 2 : 4;
    e->kvesz = c.kv_dtype == LPP_F16 ? 2 : 4;
    e->num_sms = prop.multiProcessorCount;
    e->smem_optin = prop.sharedMemPerBlockOptin;
    e->attn_gb = (e->gqa % 4 == 0) ? 4 : (e->gqa % 2 == 0 ? 2 : 1);  // query heads per attention CTA
    e->attn_z = e->gqa / e->attn_gb;
    int splits = c.attn_splits > 0 ? c.attn_splits : (2 * e->num_sms + e->KVHl * e->attn_z - 1) / (e->KVHl * e->attn_z);
    e->attn_splits = std::max(1, std::min(splits, 64));
    e->attn_splits_long = std::max(1, std::min(e->attn_splits, e->num_sms / std::max(1, e->KVHl)));
    e->sample_blocks = (c.vocab_size + kSampleChunk - 1) / kSampleChunk;
    if (e->sample_blocks > kSampleMaxBlocks) {
        delete e;
        return fail(LPP_ERR_TOO_LARGE, "vocab_size %d exceeds the sampler's %d", c.vocab_size, kSampleMaxBlocks * kSampleChunk);
    }
    e->got.assign((size_t)LPP_T_COUNT * c.n_layers, 0);

    auto bail = [&](lpp_status s) {
        lpp_engine_destroy(e);
        return s;
    };
#define CUB(call)                                                                                              \
    do {                                                                                                       \
        cudaError_t e_ = (call);                                                                               \
        if (e_ != cudaSuccess)                                                                                 \
            return bail(fail(LPP_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__)); \
    } while (0)
    CUB(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    CUB(cudaEventCreate(&e->ev0));
    CUB(cudaEventCreate(&e->ev1));
    const size_t D = c.dim, L = c.n_layers, V = c.vocab_size, S = c.seq_len;
    const size_t esz = e->esz;
    CUB(cudaMalloc(&e->wqkv, L * (e->Dq + 2 * (size_t)e->KVd) * D * esz));
    CUB(cudaMalloc(&e->wo, L * D * e->Dq * esz));
    CUB(cudaMalloc(&e->w13, L * 2 * e->Fl * D * esz));
    CUB(cudaMalloc(&e->w2, L * D * e->Fl * esz));
    CUB(cudaMalloc(&e->emb, V * D * esz));
    CUB(cudaMalloc(&e->rms_att, L * D * 4));
    CUB(cudaMalloc(&e->rms_ffn, L * D * 4));
    CUB(cudaMalloc(&e->rms_final, D * 4));
    const size_t kvbytes = L * e->KVHl * S * hs * e->kvesz;
    CUB(cudaMalloc(&e->kcache, kvbytes));
    CUB(cudaMalloc(&e->vcache, kvbytes));
    CUB(cudaMemsetAsync(e->kcache, 0, kvbytes, e->stream));
    CUB(cudaMemsetAsync(e->vcache, 0, kvbytes, e->stream));
    CUB(cudaMalloc(&e->xa, D * 4));
    CUB(cudaMalloc(&e->xb, D * 4));
    CUB(cudaMalloc(&e->q, (size_t)e->Dq * 4));
    CUB(cudaMalloc(&e->att_out, (size_t)e->Dq * 4));
    CUB(cudaMalloc(&e->hb, (size_t)e->Fl * 4));
    CUB(cudaMalloc(&e->logits, V * 4));
    CUB(cudaMalloc(&e->attn_part, (size_t)e->Hl * e->attn_splits * (hs + 2) * 4));
    CUB(cudaMalloc(&e->attn_counters, (size_t)e->KVHl * e->attn_z * 4));
    CUB(cudaMemsetAsync(e->attn_counters, 0, (size_t)e->KVHl * e->attn_z * 4, e->stream));
    CUB(cudaMalloc(&e->samp_max, e->sample_blocks * 4));
    CUB(cudaMalloc(&e->samp_sum, e->sample_blocks * 4));
    CUB(cudaMalloc(&e->samp_idx, e->sample_blocks * 4));
    CUB(cudaMalloc(&e->samp_counter, 4));
    CUB(cudaMemsetAsync(e->samp_counter, 0, 4, e->stream));
    e->exact_sampler = !(c.flags & LPP_FLAG_FAST_SAMPLER) && e->sample_blocks <= e->num_sms;
    if (e->exact_sampler) {
        CUB(cudaMalloc(&e->ex_sync, 2 * sizeof(unsigned int)));
        CUB(cudaMemsetAsync(e->ex_sync, 0, 2 * sizeof(unsigned int), e->stream));
        CUB(cudaMalloc(&e->ex_block_sum, e->sample_blocks * sizeof(double)));
        CUB(cudaMalloc(&e->ex_entry_count, e->sample_blocks * sizeof(int)));
        CUB(cudaMalloc(&e->ex_entries, (size_t)e->sample_blocks * kExactMaxEntries * sizeof(ExactEntry)));
        CUB(cudaMalloc(&e->ex_scalars, 64 * sizeof(float)));
    }
    e->run_cap = std::max<int>(4096, c.seq_len);
    CUB(cudaMalloc(&e->r_values, (size_t)e->run_cap * 4));
    CUB(cudaMalloc(&e->out_tokens, (size_t)e->run_cap * 4));
    CUB(cudaMalloc(&e->st, sizeof(StepState)));
    CUB(cudaMemsetAsync(e->st, 0, sizeof(StepState), e->stream));
    CUB(cudaMallocHost(&e->h_st, sizeof(StepState)));
    memset(e->h_st, 0, sizeof(StepState));
    {
        int khz = 0;  // SM clock in kHz = clocks per millisecond
        CUB(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c.device));
        e->h_st->wait_cycles = c.wait_ms > 0 ? (long long)c.wait_ms * khz : 0;
        e->h_st->tp_wait_cycles = c.tp_wait_ms > 0 ? (long long)c.tp_wait_ms * khz : 0;
    }
    CUB(cudaMallocHost(&e->h_out, 16));

    TRACE("create: buffers allocated");
    // rope table with libm, evaluated exactly like the reference loop (src/ops.cpp:36-40)
    {
        const int half = hs / 2;
        std::vector<float> freq(half);
        for (int j = 0; j < half; ++j) {
            const int head_dim = 2 * j;
            freq[j] = 1.0f / powf(c.rope_base, head_dim / (float)hs);
        }
        std::vector<float2> tab((size_t)S * half);
        for (size_t p = 0; p < S; ++p)
            for (int j = 0; j < half; ++j) {
                const float val = (int)p * freq[j];
                tab[p * half + j] = make_float2(cosf(val), sinf(val));
            }
        CUB(cudaMalloc(&e->rope, tab.size() * sizeof(float2)));
        CUB(cudaMemcpy(e->rope, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice));
    }

    if (c.tp_size > 1 && !(c.flags & LPP_FLAG_TP_LOCAL)) {
        if (!nccl::load()) return bail(fail(LPP_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror()));
        nccl::unique_id id;
        memcpy(&id, nccl_id, sizeof id);
        nccl::result_t r = nccl::CommInitRank(&e->comm, c.tp_size, id, c.tp_rank);
        if (r != 0) return bail(fail(LPP_ERR_NCCL, "ncclCommInitRank: %s", nccl::GetErrorString(r)));
    }
    if (c.tp_size > 1 && c.tp_size <= kMaxTp) {
        // receive areas and counters of the peer-memory exchange (used once lpp_tp_connect has mapped the peers)
        // and the logits area of the vocabulary-sharded classifier
        e->tp_buf_bytes = tp_header_bytes() + (size_t)2 * c.n_layers * tp_area_bytes(e) +
                          (size_t)c.vocab_size * sizeof(unsigned long long);
        CUB(cudaMalloc(&e->tp_buf, e->tp_buf_bytes));
        CUB(cudaMemset(e->tp_buf, 0, e->tp_buf_bytes));
        e->peer_base[c.tp_rank] = e->tp_buf;
    }
    CUB(cudaStreamSynchronize(e->stream));
#undef CUB
    TRACE("create: done");
    *out = e;
    return LPP_OK;
}

extern "C" lpp_status lpp_engine_destroy(lpp_engine* e) {
    if (!e) return LPP_OK;
    cudaSetDevice(e->c.device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (int v = 0; v < 2; ++v) {
        if (e->g_full[v]) cudaGraphExecDestroy(e->g_full[v]);
        if (e->g_logits[v]) cudaGraphExecDestroy(e->g_logits[v]);
    }
    if (e->comm) nccl::CommDestroy(e->comm);
    for (int p = 0; p < kMaxTp; ++p)
        if (e->peer_base[p] && p != e->c.tp_rank && e->peer_base[p] != e->absent_peer) cudaIpcCloseMemHandle(e->peer_base[p]);
    if (e->absent_peer) cudaFree(e->absent_peer);
    if (e->tp_buf) cudaFree(e->tp_buf);
    void* bufs[] = {e->wqkv, e->wo, e->w13, e->w2, e->emb, e->wcls_owned ? e->wcls : nullptr, e->rms_att, e->rms_ffn,
                    e->rms_final, e->kcache, e->vcache, e->xa, e->xb, e->q, e->att_out, e->hb, e->logits,
                    e->attn_part, e->attn_counters, e->samp_max, e->samp_sum, e->samp_idx, e->samp_counter,
                    e->r_values, e->out_tokens, e->st, e->rope, e->stage, e->gtrace, e->pf_x, e->pf_q, e->pf_part, e->pf_xn, e->pf_att, e->pf_hb,
                    e->pf_tokens, e->ex_sync, e->ex_block_sum, e->ex_entry_count, e->ex_entries, e->ex_scalars};
    for (void* p : bufs)
        if (p) cudaFree(p);
    if (e->h_st) cudaFreeHost(e->h_st);
    if (e->h_out) cudaFreeHost(e->h_out);
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
    return LPP_OK;
}

extern "C" lpp_status lpp_nccl_unique_id(void* out128) {
    if (!out128) return fail(LPP_ERR_INVALID_ARG, "null argument");
    if (!nccl::load()) return fail(LPP_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror());
    nccl::unique_id id;
    nccl::result_t r = nccl::GetUniqueId(&id);
    if (r != 0) return fail(LPP_ERR_NCCL, "ncclGetUniqueId: %s", nccl::GetErrorString(r));
    memcpy(out128, &id, sizeof id);
    return LPP_OK;
}

// ------------------------------------------------------------------ weight upload

static lpp_status ensure_stage(lpp_engine* e, size_t bytes) {
    if (bytes <= e->stage_bytes) return LPP_OK;
    if (e->stage) CU(cudaFree(e->stage));
    e->stage = nullptr;
    e->stage_bytes = 0;
    CU(cudaMalloc(&e->stage, bytes));
    e->stage_bytes = bytes;
    return LPP_OK;
}

// dst[r*dst_pitch + c] (dst_dtype) = src[(r0 + r)*src_pitch + c0 + c] (src_dtype), r < rows, c < cols
static lpp_status put_block(lpp_engine* e, void* dst, size_t dst_pitch, int dst_dtype, const void* src,
                            size_t src_pitch, size_t r0, size_t c0, int rows, int cols, int src_dtype, int memkind) {
    const size_t sesz = src_dtype == LPP_F16 ? 2 : 4;
    const char* s = (const char*)src + (r0 * src_pitch + c0) * sesz;
    size_t spitch = src_pitch;
    if (memkind == LPP_MEM_HOST) {
        TRY(ensure_stage(e, (size_t)rows * cols * sesz));
        CU(cudaMemcpy2DAsync(e->stage, (size_t)cols * sesz, s, src_pitch * sesz, (size_t)cols * sesz, rows,
                             cudaMemcpyHostToDevice, e->stream));
        s = (const char*)e->stage;
        spitch = cols;
    }
    const long long total = (long long)rows * cols;
    const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
    if (dst_dtype == LPP_F16 && src_dtype == LPP_F16)
        repack_kernel<__half, __half><<<grid, 256, 0, e->stream>>>((__half*)dst, dst_pitch, (const __half*)s, spitch, rows, cols);
    else if (dst_dtype == LPP_F16 && src_dtype == LPP_F32)
        repack_kernel<__half, float><<<grid, 256, 0, e->stream>>>((__half*)dst, dst_pitch, (const float*)s, spitch, rows, cols);
    else if (dst_dtype == LPP_F32 && src_dtype == LPP_F16)
        repack_kernel<float, __half><<<grid, 256, 0, e->stream>>>((float*)dst, dst_pitch, (const __half*)s, spitch, rows, cols);
    else
        repack_kernel<float, float><<<grid, 256, 0, e->stream>>>((float*)dst, dst_pitch, (const float*)s, spitch, rows, cols);
    CU(cudaGetLastError());
    // the staging buffer is reused by the next call and host memory may be freed by the caller
    CU(cudaStreamSynchronize(e->stream));
    return LPP_OK;
}

extern "C" lpp_status lpp_upload_tensor(lpp_engine* e, int which, int layer, const void* src, int src_dtype,
                                        int memkind) {
    if (!e || !src) return fail(LPP_ERR_INVALID_ARG, "null argument");
    if (which < 0 || which >= LPP_T_COUNT) return fail(LPP_ERR_INVALID_ARG, "unknown tensor id %d", which);
    if (src_dtype != LPP_F16 && src_dtype != LPP_F32) return fail(LPP_ERR_INVALID_ARG, "bad src_dtype");
    if (memkind != LPP_MEM_HOST && memkind != LPP_MEM_DEVICE) return fail(LPP_ERR_INVALID_ARG, "bad memkind");
    const lpp_config& c = e->c;
    const bool stacked = !(which == LPP_T_TOK_EMB || which == LPP_T_RMS_FINAL || which == LPP_T_W_CLS);
    if (stacked && (layer < 0 || layer >= c.n_layers)) return fail(LPP_ERR_INVALID_ARG, "layer %d out of range", layer);
    if (!stacked) layer = 0;
    CU(cudaSetDevice(c.device));
    TRACE("upload tensor %d layer %d", which, layer);
    const size_t D = c.dim, F = c.hidden_dim, V = c.vocab_size, esz = e->esz;
    const size_t l = layer, r = c.tp_rank;
    const size_t qkv_rows = e->Dq + 2 * (size_t)e->KVd;
    const int wd = c.weight_dtype;
    char* wqkv_l = (char*)e->wqkv + l * qkv_rows * D * esz;
    char* w13_l = (char*)e->w13 + l * 2 * e->Fl * D * esz;
    lpp_status s = LPP_OK;
    switch (which) {
        case LPP_T_TOK_EMB:
            s = put_block(e, e->emb, D, wd, src, D, 0, 0, (int)V, (int)D, src_dtype, memkind);
            break;
        case LPP_T_W_CLS:
            // With the peers mapped (lpp_tp_connect comes before the uploads in that case) the classifier is
            // sharded by vocabulary rows and this rank never reads another rank's rows: it keeps V/tp rows.
            if (!e->wcls_owned) {
                e->wcls_shard_only = tp_cls_sharded(e);
                CU(cudaMalloc(&e->wcls, (e->wcls_shard_only ? V / c.tp_size : V) * D * esz));
                e->wcls_owned = true;
            }
            if (e->wcls_shard_only)
                s = put_block(e, e->wcls, D, wd, src, D, r * (V / c.tp_size), 0, (int)(V / c.tp_size), (int)D, src_dtype, memkind);
            else
                s = put_block(e, e->wcls, D, wd, src, D, 0, 0, (int)V, (int)D, src_dtype, memkind);
            break;
        case LPP_T_RMS_ATT:
            s = put_block(e, e->rms_att + l * D, D, LPP_F32, src, D, 0, 0, 1, (int)D, src_dtype, memkind);
            break;
        case LPP_T_RMS_FFN:
            s = put_block(e, e->rms_ffn + l * D, D, LPP_F32, src, D, 0, 0, 1, (int)D, src_dtype, memkind);
            break;
        case LPP_T_RMS_FINAL:
            s = put_block(e, e->rms_final, D, LPP_F32, src, D, 0, 0, 1, (int)D, src_dtype, memkind);
            break;
        case LPP_T_WQ:  // row slice of [D][D]
            s = put_block(e, wqkv_l, D, wd, src, D, r * e->Dq, 0, e->Dq, (int)D, src_dtype, memkind);
            break;
        case LPP_T_WK:  // row slice of [KV][D]
            s = put_block(e, wqkv_l + (size_t)e->Dq * D * esz, D, wd, src, D, r * e->KVd, 0, e->KVd, (int)D, src_dtype, memkind);
            break;
        case LPP_T_WV:
            s = put_block(e, wqkv_l + ((size_t)e->Dq + e->KVd) * D * esz, D, wd, src, D, r * e->KVd, 0, e->KVd, (int)D, src_dtype, memkind);
            break;
        case LPP_T_WO:  // column slice of [D][D] (columns = this rank's heads), repacked contiguous
            s = put_block(e, (char*)e->wo + l * D * e->Dq * esz, e->Dq, wd, src, D, 0, r * e->Dq, (int)D, e->Dq, src_dtype, memkind);
            break;
        case LPP_T_W1:  // gate rows -> even rows of w13
            s = put_block(e, w13_l, 2 * D, wd, src, D, r * e->Fl, 0, e->Fl, (int)D, src_dtype, memkind);
            break;
        case LPP_T_W3:  // up rows -> odd rows of w13
            s = put_block(e, w13_l + D * esz, 2 * D, wd, src, D, r * e->Fl, 0, e->Fl, (int)D, src_dtype, memkind);
            break;
        case LPP_T_W2:  // column slice of [D][F]
            s = put_block(e, (char*)e->w2 + l * D * e->Fl * esz, e->Fl, wd, src, F, 0, r * e->Fl, (int)D, e->Fl, src_dtype, memkind);
            break;
    }
    TRY(s);
    e->got[(size_t)which * c.n_layers + layer] = 1;
    e->finalized = false;
    return LPP_OK;
}

extern "C" lpp_status lpp_finalize(lpp_engine* e) {
    if (!e) return fail(LPP_ERR_INVALID_ARG, "null argument");
    const lpp_config& c = e->c;
    CU(cudaSetDevice(c.device));
    static const char* names[LPP_T_COUNT] = {"tok_emb", "rms_att", "wq", "wk", "wv", "wo", "rms_ffn", "w1", "w2", "w3", "rms_final", "w_cls"};
    for (int t = 0; t < LPP_T_COUNT; ++t) {
        if (t == LPP_T_W_CLS) continue;
        const bool stacked = !(t == LPP_T_TOK_EMB || t == LPP_T_RMS_FINAL);
        const int n = stacked ? c.n_layers : 1;
        for (int l = 0; l < n; ++l)
            if (!e->got[(size_t)t * c.n_layers + l])
                return fail(LPP_ERR_NOT_READY, "tensor %s (layer %d) was never uploaded", names[t], l);
    }
    if (c.tp_size > 1 && !e->comm && !tp_peer_path(e))
        return fail(LPP_ERR_NOT_READY, "a tensor-parallel engine without NCCL (LPP_FLAG_TP_LOCAL) needs lpp_tp_connect");
    if (e->wcls_shard_only && !tp_cls_sharded(e))
        return fail(LPP_ERR_NOT_READY, "the classifier was uploaded as a vocabulary shard but the engine no longer shards it");
    if (!e->wcls_owned) e->wcls = e->emb;  // tied classifier (src/loader.cpp:66, 471)
    if (e->stage) {
        cudaFree(e->stage);
        e->stage = nullptr;
        e->stage_bytes = 0;
    }
    for (int v = 0; v < 2; ++v) {
        if (e->g_full[v]) cudaGraphExecDestroy(e->g_full[v]), e->g_full[v] = nullptr;
        if (e->g_logits[v]) cudaGraphExecDestroy(e->g_logits[v]), e->g_logits[v] = nullptr;
    }
    TRACE("finalize: weights complete");
    if (aid_env("LPP_GEMV_TRACE") && !e->gtrace) {
        CU(cudaMalloc(&e->gtrace, (size_t)256 * e->num_sms * 8 * sizeof(unsigned long long)));
        CU(cudaMemset(e->gtrace, 0, (size_t)256 * e->num_sms * 8 * sizeof(unsigned long long)));
    }
    if (!(c.flags & LPP_FLAG_NO_GRAPH)) {
        for (int v = 0; v < 1; ++v) {
            TRY(capture(e, true, v == 1, &e->g_full[v], v == 0 ? &e->kernels_full : nullptr));
            TRY(capture(e, false, v == 1, &e->g_logits[v], nullptr));
        }
        TRACE("finalize: graphs captured (%d kernels per long-context step)", e->kernels_full);
    } else {
        e->kernels_full = 5 * c.n_layers + 2 + (tp_cls_sharded(e) ? 1 : 0);
    }
    e->finalized = true;
    return LPP_OK;
}

// ------------------------------------------------------------------ stepping

static lpp_status push_state(lpp_engine* e, int token, int pos, const lpp_sample_params* sp, const int* hist,
                             int hist_len, float r, int advance, int window) {
    const lpp_config& c = e->c;
    if (token < 0 || token >= c.vocab_size) return fail(LPP_ERR_INVALID_ARG, "token %d outside [0, %d)", token, c.vocab_size);
    if (pos < 0 || pos >= c.seq_len) return fail(LPP_ERR_INVALID_ARG, "pos %d outside [0, %d)", pos, c.seq_len);
    if (hist_len < 0 || hist_len > kHistoryMax) return fail(LPP_ERR_TOO_LARGE, "history_len %d > %d", hist_len, kHistoryMax);
    StepState* h = e->h_st;
    h->token = token;
    h->pos = pos;
    const bool use_hist = sp && sp->penalty > 1.0f && hist && hist_len > 0;
    h->history_len = use_hist || advance ? (hist ? hist_len : 0) : 0;
    h->history_window = window;
    h->history_count = h->history_len;
    h->step_idx = 0;
    h->advance = advance;
    h->temperature = sp ? sp->temperature : 0.f;
    h->penalty = sp ? sp->penalty : 1.f;
    h->r = r;
    h->out_token = -1;
    h->status = 0;
    if (h->history_len > 0) memcpy(h->history, hist, (size_t)h->history_len * sizeof(int));
    const size_t bytes = offsetof(StepState, history) + (size_t)h->history_len * sizeof(int);
    CU(cudaMemcpyAsync(e->st, h, bytes, cudaMemcpyHostToDevice, e->stream));
    return LPP_OK;
}

static lpp_status pull_result(lpp_engine* e, int* token) {
    TRACE("pull_result: waiting for the stream");
    CU(cudaMemcpyAsync(e->h_out, &e->st->out_token, 2 * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    if (e->h_out[1] != 0) return fail(LPP_ERR_DEVICE_STATUS, "device status 0x%x (1=barrier timeout, 2=bad token, 4=bad pos)", e->h_out[1]);
    if (token) *token = e->h_out[0];
    return LPP_OK;
}

#define NEED_READY(e)                                                              \
    do {                                                                           \
        if (!(e)) return fail(LPP_ERR_INVALID_ARG, "null engine");                 \
        if (!(e)->finalized) return fail(LPP_ERR_NOT_READY, "lpp_finalize not called"); \
        CU(cudaSetDevice((e)->c.device));                                          \
    } while (0)

extern "C" lpp_status lpp_step(lpp_engine* e, int token, int pos, const lpp_sample_params* sp, const int* h_history,
                               int history_len, float r, int* next_token) {
    NEED_READY(e);
    if (!sp || !next_token) return fail(LPP_ERR_INVALID_ARG, "null argument");
    TRY(push_state(e, token, pos, sp, h_history, history_len, r, 0, 0));
    TRY(run_step(e, true, pos));
    return pull_result(e, next_token);
}

extern "C" lpp_status lpp_step_logits(lpp_engine* e, int token, int pos, float* h_logits) {
    NEED_READY(e);
    if (!h_logits) return fail(LPP_ERR_INVALID_ARG, "null argument");
    TRY(push_state(e, token, pos, nullptr, nullptr, 0, 0.f, 0, 0));
    TRY(run_step(e, false, pos));
    CU(cudaMemcpyAsync(h_logits, e->logits, (size_t)e->c.vocab_size * 4, cudaMemcpyDeviceToHost, e->stream));
    return pull_result(e, nullptr);
}

extern "C" lpp_status lpp_decode(lpp_engine* e, int first_token, int start_pos, int n, const lpp_sample_params* sp,
                                 const int* h_history, int history_len, int history_window, const float* h_r,
                                 int* h_out_tokens, float* device_ms) {
    NEED_READY(e);
    if (!sp || !h_out_tokens || n <= 0) return fail(LPP_ERR_INVALID_ARG, "bad argument");
    if (n > e->run_cap) return fail(LPP_ERR_TOO_LARGE, "n %d > capacity %d", n, e->run_cap);
    if (start_pos + n > e->c.seq_len) return fail(LPP_ERR_INVALID_ARG, "start_pos + n exceeds seq_len %d", e->c.seq_len);
    if (history_window < 0 || history_window > kHistoryMax || history_len > std::max(history_window, 0))
        return fail(LPP_ERR_INVALID_ARG, "history_len %d / window %d invalid", history_len, history_window);
    if (sp->temperature != 0.0f && !h_r) return fail(LPP_ERR_INVALID_ARG, "temperature > 0 needs h_r");
    TRY(push_state(e, first_token, start_pos, sp, h_history, history_len, 0.f, 1, history_window));
    if (h_r) CU(cudaMemcpyAsync(e->r_values, h_r, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaEventRecord(e->ev0, e->stream));
    for (int i = 0; i < n; ++i) TRY(run_step(e, true, start_pos + i));
    CU(cudaEventRecord(e->ev1, e->stream));
    CU(cudaMemcpyAsync(h_out_tokens, e->out_tokens, (size_t)n * 4, cudaMemcpyDeviceToHost, e->stream));
    TRY(pull_result(e, nullptr));
    if (device_ms) CU(cudaEventElapsedTime(device_ms, e->ev0, e->ev1));
    return LPP_OK;
}

extern "C" lpp_status lpp_sample_logits(lpp_engine* e, const float* h_logits, const lpp_sample_params* sp,
                                        const int* h_history, int history_len, float r, int* token) {
    NEED_READY(e);
    if (!h_logits || !sp || !token) return fail(LPP_ERR_INVALID_ARG, "null argument");
    TRY(push_state(e, 0, 0, sp, h_history, history_len, r, 0, 0));
    CU(cudaMemcpyAsync(e->logits, h_logits, (size_t)e->c.vocab_size * 4, cudaMemcpyHostToDevice, e->stream));
    CU(launch_sampler(e, e->stream, false));
    return pull_result(e, token);
}

// ------------------------------------------------------------------ batched prompt path

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn tensor_map_encoder() {
    static encode_tiled_fn encode = nullptr;
    if (!encode) {
        cudaDriverEntryPointQueryResult qr;
        void* fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && fn &&
            qr == cudaDriverEntryPointSuccess)
            encode = (encode_tiled_fn)fn;
    }
    return encode;
}

// Tensor maps over row-major FP16 matrices of THIS GPU's memory, cut into pieces of 64 inputs (128 bytes, stored with
// the 128-byte swizzle: the K-major operand layout of the MMA descriptors).  cols must be a multiple of 64; elements
// outside the matrix read as zero.
//
// Weights [rows][cols] seen as (64 inputs, rows, cols / 64): a box is 64 inputs x box_rows rows x 2 pieces, i.e. one
// copy delivers both 64-input sub-tiles of a stage, sub-tile after sub-tile.
static lpp_status make_weight_map(CUtensorMap* m, const void* base, size_t rows, size_t cols, int box_rows) {
    encode_tiled_fn encode = tensor_map_encoder();
    if (!encode) return fail(LPP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 2u};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LPP_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a %zu x %zu matrix", (int)r, rows, cols);
    return LPP_OK;
}
// Activations: hi plane [tokens][cols] followed by the lo plane, seen as (64 inputs, tokens, 2 planes, cols / 64): a
// box is 64 inputs x box_tokens x 2 planes x 2 pieces, i.e. one copy delivers, per 64-input piece, the hi rows
// followed by the lo rows: one K-major operand tile of 2 x box_tokens rows (the MMA's N) per piece.
static lpp_status make_activation_map(CUtensorMap* m, const void* base, size_t tokens, size_t cols, int box_tokens) {
    encode_tiled_fn encode = tensor_map_encoder();
    if (!encode) return fail(LPP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[4] = {64, (cuuint64_t)tokens, 2, (cuuint64_t)(cols / 64)};
    const cuuint64_t strides[3] = {(cuuint64_t)cols * 2, (cuuint64_t)tokens * cols * 2, 128};
    const cuuint32_t box[4] = {64u, (cuuint32_t)box_tokens, 2u, 2u};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LPP_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a %zu x %zu activation block", (int)r, tokens, cols);
    return LPP_OK;
}

// The tensor-core path takes FP16 weights, an FP16 cache and a single GPU; everything else is fed token by token.
static bool prefill_batched(const lpp_engine* e) {
    return e->c.tp_size == 1 && e->c.weight_dtype == LPP_F16 && e->c.kv_dtype == LPP_F16 && e->hs <= 128 && e->gqa <= 8 &&
           e->c.dim % 64 == 0 && e->Dq % 64 == 0 && e->Fl % 64 == 0 && !(e->c.flags & LPP_FLAG_NO_PREFILL_GEMM);
}

static lpp_status prefill_setup(lpp_engine* e) {
    if (e->pf_ready) return LPP_OK;
    const lpp_config& c = e->c;
    const size_t D = c.dim, L = c.n_layers, T = kPrefillTokens;
    const size_t qkv_rows = e->Dq + 2 * (size_t)e->KVd;
    CU(cudaMalloc(&e->pf_x, T * D * 4));
    CU(cudaMalloc(&e->pf_q, T * e->Dq * 4));
    CU(cudaMalloc(&e->pf_xn, 2 * T * D * 2));  // hi plane, lo plane
    CU(cudaMalloc(&e->pf_att, 2 * T * e->Dq * 2));  // hi plane, lo plane
    CU(cudaMalloc(&e->pf_hb, 2 * T * e->Fl * 2));  // hi plane, lo plane
    CU(cudaMalloc(&e->pf_part, (size_t)kPfMaxSplits * T * std::max<size_t>(D, qkv_rows) * 4));
    CU(cudaMalloc(&e->pf_tokens, T * sizeof(int)));
    CU(cudaMemsetAsync(e->pf_x, 0, T * D * 4, e->stream));
    CU(cudaMemsetAsync(e->pf_xn, 0, 2 * T * D * 2, e->stream));
    CU(cudaMemsetAsync(e->pf_att, 0, 2 * T * e->Dq * 2, e->stream));
    CU(cudaMemsetAsync(e->pf_hb, 0, 2 * T * e->Fl * 2, e->stream));
    CU(cudaMemsetAsync(e->pf_tokens, 0, T * sizeof(int), e->stream));
    TRY(make_weight_map(&e->pf_map_wqkv, e->wqkv, L * qkv_rows, D, kUmmaM));
    TRY(make_weight_map(&e->pf_map_wo, e->wo, L * D, e->Dq, kUmmaM));
    TRY(make_weight_map(&e->pf_map_w13, e->w13, L * 2 * e->Fl, D, kUmmaM));
    TRY(make_weight_map(&e->pf_map_w2, e->w2, L * D, e->Fl, kUmmaM));
    TRY(make_activation_map(&e->pf_map_xn, e->pf_xn, T, D, kPrefillTokens));
    TRY(make_activation_map(&e->pf_map_att, e->pf_att, T, e->Dq, kPrefillTokens));
    TRY(make_activation_map(&e->pf_map_hb, e->pf_hb, T, e->Fl, kPrefillTokens));
    CU(cudaFuncSetAttribute(prefill_gemm_umma_kernel<kPfQkv>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmemBytes));
    CU(cudaFuncSetAttribute(prefill_gemm_umma_kernel<kPfResid>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmemBytes));
    CU(cudaFuncSetAttribute(prefill_gemm_umma_kernel<kPfSwiglu>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmemBytes));
    CU(cudaFuncSetAttribute(prefill_attention_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_attn_smem<64>()));
    CU(cudaFuncSetAttribute(prefill_attention_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_attn_smem<128>()));
    e->pf_ready = true;
    return LPP_OK;
}

// Work items are tiles of 128 weight rows (the weight maps' box).  A GEMM whose row tiles do not fill the GPU is also
// cut along K; its partial sums go to pf_part and are added up by the next prefill_norm_kernel (residual projections)
// or by prefill_qkv_finish_kernel (QKV).
static cudaError_t launch_prefill_gemm(lpp_engine* e, const CUtensorMap& wm, const CUtensorMap& xm, PrefillGemmArgs a) {
    const int tiles = (a.n_rows + kUmmaM - 1) / kUmmaM;
    const int n_kc = (a.K + kPfKc - 1) / kPfKc;
    a.st = e->st;
    a.splits = 1;
    // QKV is cut too: its partial sums are finished by prefill_qkv_finish_kernel
    if ((a.epi == kPfResid || a.epi == kPfQkv) && tiles < e->num_sms)
        a.splits = std::max(1, std::min({kPfMaxSplits, n_kc, (e->num_sms + tiles - 1) / tiles}));
    a.part = e->pf_part;
    const dim3 g(std::min(tiles * a.splits, e->num_sms)), b(kUmmaThreads);
    const size_t sm = (size_t)kPfSmemBytes;
    if (a.epi == kPfResid) return launch_kernel(prefill_gemm_umma_kernel<kPfResid>, g, b, sm, e->stream, true, wm, xm, a);
    if (a.epi == kPfSwiglu) return launch_kernel(prefill_gemm_umma_kernel<kPfSwiglu>, g, b, sm, e->stream, true, wm, xm, a);
    const cudaError_t err = launch_kernel(prefill_gemm_umma_kernel<kPfQkv>, g, b, sm, e->stream, true, wm, xm, a);
    if (err != cudaSuccess || a.splits == 1) return err;
    return launch_kernel(prefill_qkv_finish_kernel, dim3(a.n_tokens, (a.n_rows / 2 + 255) / 256), dim3(256), 0, e->stream, true, a);
}
static int prefill_splits(const lpp_engine* e, int n_rows, int K) {  // what launch_prefill_gemm chooses for a residual GEMM
    const int tiles = (n_rows + kUmmaM - 1) / kUmmaM, n_kc = (K + kPfKc - 1) / kPfKc;
    return tiles < e->num_sms ? std::max(1, std::min({kPfMaxSplits, n_kc, (e->num_sms + tiles - 1) / tiles})) : 1;
}

// One block of n <= kPrefillTokens prompt tokens at positions start_pos ..: seven kernels per layer; the last layer
// stops after its K/V rows are written (nothing downstream of them is needed: the call produces no logits).
static lpp_status prefill_block(lpp_engine* e, const int* h_tokens, int n, int start_pos) {
    const lpp_config& c = e->c;
    const int D = c.dim, L = c.n_layers;
    const int qkv_rows = e->Dq + 2 * e->KVd;
    const int s_o = prefill_splits(e, D, e->Dq), s_d = prefill_splits(e, D, e->Fl);
    CU(cudaMemcpyAsync(e->pf_tokens, h_tokens, (size_t)n * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    for (int l = 0; l < L; ++l) {
        // layer 0 takes the embedding rows; later layers first add the previous down projection's partial sums
        CU(launch_kernel(prefill_norm_kernel, dim3(n), dim3(kPfNormThreads), 0, e->stream, l > 0, e->pf_x, (const int*)e->pf_tokens,
                         (const __half*)(l == 0 ? e->emb : nullptr), c.vocab_size, (const float*)(e->rms_att + (size_t)l * D),
                         e->pf_xn, D, n, (const float*)e->pf_part, l == 0 ? 1 : s_d, e->st));
        const size_t lofs = (size_t)l * e->KVHl * c.seq_len * e->hs;
        PrefillGemmArgs g = {};
        g.n_tokens = n;
        g.start_pos = start_pos;
        g.n_rows = qkv_rows;
        g.K = D;
        g.row0 = l * qkv_rows;
        g.epi = kPfQkv;
        g.q = e->pf_q;
        g.q_rows = e->Dq;
        g.kv_rows = e->KVd;
        g.head_size = e->hs;
        g.seq_len = c.seq_len;
        g.rope = e->rope;
        g.k_cache = (__half*)e->kcache + lofs;
        g.v_cache = (__half*)e->vcache + lofs;
        CU(launch_prefill_gemm(e, e->pf_map_wqkv, e->pf_map_xn, g));
        if (l == L - 1) break;
        const dim3 agrid((n + kPfAttnRows - 1) / kPfAttnRows, e->KVHl);
        const bool pf_mma = !aid_env("LPP_ATTN_CUDA_CORES");
        if (pf_mma && e->hs == 64 && e->gqa <= 8)
            CU(launch_kernel(prefill_attention_mma_kernel<64>, agrid, dim3(32 * e->gqa), pf_attn_smem<64>(), e->stream, true,
                             (const float*)e->pf_q, (const __half*)g.k_cache, (const __half*)g.v_cache, e->pf_att, n, start_pos,
                             c.seq_len, e->gqa, e->Dq));
        else if (pf_mma && e->hs == 128 && e->gqa <= 8)
            CU(launch_kernel(prefill_attention_mma_kernel<128>, agrid, dim3(32 * e->gqa), pf_attn_smem<128>(), e->stream, true,
                             (const float*)e->pf_q, (const __half*)g.k_cache, (const __half*)g.v_cache, e->pf_att, n, start_pos,
                             c.seq_len, e->gqa, e->Dq));
        else
            CU(launch_kernel(prefill_attention_kernel, dim3(n, e->KVHl), dim3(32 * e->gqa),
                             (size_t)e->gqa * e->hs * sizeof(float), e->stream, true, (const float*)e->pf_q,
                             (const __half*)g.k_cache, (const __half*)g.v_cache, e->pf_att, n, start_pos, c.seq_len, e->hs,
                             e->gqa, e->Dq));
        PrefillGemmArgs o = {};
        o.n_tokens = n;
        o.start_pos = start_pos;
        o.n_rows = D;
        o.K = e->Dq;
        o.row0 = l * D;
        o.epi = kPfResid;
        o.x = e->pf_x;
        CU(launch_prefill_gemm(e, e->pf_map_wo, e->pf_map_att, o));
        CU(launch_kernel(prefill_norm_kernel, dim3(n), dim3(kPfNormThreads), 0, e->stream, true, e->pf_x, (const int*)e->pf_tokens,
                         (const __half*)nullptr, c.vocab_size, (const float*)(e->rms_ffn + (size_t)l * D), e->pf_xn, D, n,
                         (const float*)e->pf_part, s_o, e->st));
        PrefillGemmArgs u = {};
        u.n_tokens = n;
        u.start_pos = start_pos;
        u.n_rows = 2 * e->Fl;
        u.K = D;
        u.row0 = l * 2 * e->Fl;
        u.epi = kPfSwiglu;
        u.hb = e->pf_hb;
        CU(launch_prefill_gemm(e, e->pf_map_w13, e->pf_map_xn, u));
        PrefillGemmArgs d = {};
        d.n_tokens = n;
        d.start_pos = start_pos;
        d.n_rows = D;
        d.K = e->Fl;
        d.row0 = l * D;
        d.epi = kPfResid;
        d.x = e->pf_x;
        CU(launch_prefill_gemm(e, e->pf_map_w2, e->pf_map_hb, d));
    }
    return LPP_OK;
}

extern "C" lpp_status lpp_prefill(lpp_engine* e, const int* h_tokens, int n, int start_pos, float* device_ms) {
    NEED_READY(e);
    if (!h_tokens || n <= 0) return fail(LPP_ERR_INVALID_ARG, "bad argument");
    if (start_pos < 0 || start_pos + n > e->c.seq_len) return fail(LPP_ERR_INVALID_ARG, "positions %d..%d outside [0, %d)", start_pos, start_pos + n - 1, e->c.seq_len);
    for (int i = 0; i < n; ++i)
        if (h_tokens[i] < 0 || h_tokens[i] >= e->c.vocab_size) return fail(LPP_ERR_INVALID_ARG, "token %d outside [0, %d)", h_tokens[i], e->c.vocab_size);
    TRY(push_state(e, h_tokens[0], start_pos, nullptr, nullptr, 0, 0.f, 0, 0));  // clears the device status
    if (prefill_batched(e)) {
        TRY(prefill_setup(e));
        CU(cudaEventRecord(e->ev0, e->stream));
        for (int i = 0; i < n; i += kPrefillTokens) TRY(prefill_block(e, h_tokens + i, std::min(kPrefillTokens, n - i), start_pos + i));
        CU(cudaEventRecord(e->ev1, e->stream));
    } else {
        // token by token through the step graph without its sampler, like the reference's prompt loop
        CU(cudaEventRecord(e->ev0, e->stream));
        for (int i = 0; i < n; ++i) {
            TRY(push_state(e, h_tokens[i], start_pos + i, nullptr, nullptr, 0, 0.f, 0, 0));
            TRY(run_step(e, false, start_pos + i));
            // the pinned staging block of push_state is rewritten by the next token: the copy must have run
            if (i + 1 < n) CU(cudaStreamSynchronize(e->stream));
        }
        CU(cudaEventRecord(e->ev1, e->stream));
    }
    TRY(pull_result(e, nullptr));
    if (device_ms) CU(cudaEventElapsedTime(device_ms, e->ev0, e->ev1));
    return LPP_OK;
}

// ------------------------------------------------------------------ KV cache access

extern "C" int64_t lpp_kv_index(const lpp_engine* e, int layer, int kv_head, int pos, int off) {
    if (!e) return -1;
    const int64_t kvd = (int64_t)e->KVHl * e->hs, S = e->c.seq_len;
    return (int64_t)layer * (kvd * S) + (int64_t)kv_head * (S * e->hs) + (int64_t)pos * e->hs + off;
}

extern "C" lpp_status lpp_kv_prefill(lpp_engine* e, int layer, const void* k, const void* v, int n_pos, int src_dtype,
                                     int memkind) {
    if (!e || !k || !v) return fail(LPP_ERR_INVALID_ARG, "null argument");
    const lpp_config& c = e->c;
    if (layer < 0 || layer >= c.n_layers || n_pos < 0 || n_pos > c.seq_len) return fail(LPP_ERR_INVALID_ARG, "layer/n_pos out of range");
    if (src_dtype != LPP_F16 && src_dtype != LPP_F32) return fail(LPP_ERR_INVALID_ARG, "bad src_dtype");
    CU(cudaSetDevice(c.device));
    const int hs = e->hs;
    for (int h = 0; h < e->KVHl; ++h) {
        const size_t gh = (size_t)c.tp_rank * e->KVHl + h;  // global kv head
        const size_t dst = (size_t)lpp_kv_index(e, layer, h, 0, 0) * e->kvesz;
        // source rows [gh][0..n_pos) are contiguous: one block of n_pos rows x hs columns
        TRY(put_block(e, (char*)e->kcache + dst, hs, c.kv_dtype, k, hs, gh * n_pos, 0, n_pos, hs, src_dtype, memkind));
        TRY(put_block(e, (char*)e->vcache + dst, hs, c.kv_dtype, v, hs, gh * n_pos, 0, n_pos, hs, src_dtype, memkind));
    }
    if (e->stage && e->finalized) {
        cudaFree(e->stage);
        e->stage = nullptr;
        e->stage_bytes = 0;
    }
    return LPP_OK;
}

extern "C" lpp_status lpp_kv_read(lpp_engine* e, int layer, int kv_head, int pos, float* h_k, float* h_v) {
    if (!e || !h_k || !h_v) return fail(LPP_ERR_INVALID_ARG, "null argument");
    const lpp_config& c = e->c;
    if (layer < 0 || layer >= c.n_layers || kv_head < 0 || kv_head >= e->KVHl || pos < 0 || pos >= c.seq_len)
        return fail(LPP_ERR_INVALID_ARG, "index out of range");
    CU(cudaSetDevice(c.device));
    const size_t off = (size_t)lpp_kv_index(e, layer, kv_head, pos, 0) * e->kvesz;
    const int hs = e->hs;
    CU(cudaStreamSynchronize(e->stream));
    if (c.kv_dtype == LPP_F32) {
        CU(cudaMemcpy(h_k, (char*)e->kcache + off, hs * 4, cudaMemcpyDeviceToHost));
        CU(cudaMemcpy(h_v, (char*)e->vcache + off, hs * 4, cudaMemcpyDeviceToHost));
    } else {
        std::vector<__half> tk(hs), tv(hs);
        CU(cudaMemcpy(tk.data(), (char*)e->kcache + off, hs * 2, cudaMemcpyDeviceToHost));
        CU(cudaMemcpy(tv.data(), (char*)e->vcache + off, hs * 2, cudaMemcpyDeviceToHost));
        for (int i = 0; i < hs; ++i) {
            h_k[i] = __half2float(tk[i]);
            h_v[i] = __half2float(tv[i]);
        }
    }
    return LPP_OK;
}

// ------------------------------------------------------------------ introspection

// ---- tensor-parallel peer mapping ---------------------------------------------------------------

static_assert(sizeof(cudaIpcMemHandle_t) == LPP_TP_HANDLE_BYTES, "IPC handle size");

extern "C" lpp_status lpp_tp_export(lpp_engine* e, void* handle, size_t handle_bytes) {
    if (!e || !handle) return fail(LPP_ERR_INVALID_ARG, "null argument");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return fail(LPP_ERR_INVALID_ARG, "handle buffer needs %zu bytes", sizeof(cudaIpcMemHandle_t));
    if (!e->tp_buf || e->c.tp_size < 2) return fail(LPP_ERR_INVALID_ARG, "engine has no tensor-parallel exchange buffer (tp_size 1 or > %d)", kMaxTp);
    CU(cudaSetDevice(e->c.device));
    cudaIpcMemHandle_t h;
    CU(cudaIpcGetMemHandle(&h, e->tp_buf));
    memcpy(handle, &h, sizeof h);
    return LPP_OK;
}

extern "C" lpp_status lpp_tp_connect(lpp_engine* e, const void* handles, size_t handle_bytes) {
    if (!e || !handles) return fail(LPP_ERR_INVALID_ARG, "null argument");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return fail(LPP_ERR_INVALID_ARG, "handles are %zu bytes each", sizeof(cudaIpcMemHandle_t));
    if (!e->tp_buf || e->c.tp_size < 2) return fail(LPP_ERR_INVALID_ARG, "engine has no tensor-parallel exchange buffer");
    if (e->finalized) return fail(LPP_ERR_INVALID_ARG, "lpp_tp_connect must precede lpp_finalize");
    CU(cudaSetDevice(e->c.device));
    for (int p = 0; p < e->c.tp_size; ++p) {
        if (p == e->c.tp_rank || e->peer_base[p]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)p * handle_bytes, sizeof h);
        void* ptr = nullptr;
        cudaError_t r = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (r != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(LPP_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d: %s", p, cudaGetErrorString(r));
        }
        e->peer_base[p] = (unsigned char*)ptr;
    }
    e->peer_ready = true;
    return LPP_OK;
}

// Test aid (not part of the public header): lets ONE rank of a tensor-parallel group run without its peers.
// Stores to the other ranks land in a private scratch buffer and nobody ever fills this rank's receive slots,
// so the first consuming GEMV's wait on its peers runs out after lpp_config.tp_wait_ms and the step ends
// with LPP_ERR_DEVICE_STATUS: the one way to see that path on a single GPU without a fault or a hang.
extern "C" lpp_status lpp_debug_tp_absent_peers(lpp_engine* e) {
    if (!e) return fail(LPP_ERR_INVALID_ARG, "null argument");
    if (!e->tp_buf || e->c.tp_size < 2) return fail(LPP_ERR_INVALID_ARG, "engine has no tensor-parallel exchange buffer");
    if (e->finalized) return fail(LPP_ERR_INVALID_ARG, "must precede lpp_finalize");
    CU(cudaSetDevice(e->c.device));
    if (!e->absent_peer) {
        CU(cudaMalloc(&e->absent_peer, e->tp_buf_bytes));
        CU(cudaMemset(e->absent_peer, 0, e->tp_buf_bytes));
    }
    for (int p = 0; p < e->c.tp_size; ++p)
        if (p != e->c.tp_rank && !e->peer_base[p]) e->peer_base[p] = e->absent_peer;
    e->peer_ready = true;
    return LPP_OK;
}

// Test aid (not part of the public header): one warp waits, with the engine's wait limit, on a shared-memory
// barrier that nothing ever arrives on.  The wait must run out, the kernel must return normally, and the
// call must fail with LPP_ERR_DEVICE_STATUS like a step whose copy never completed.
static __global__ void wait_probe_kernel(StepState* st) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar, 0u, st));
    if (!ok && threadIdx.x == 0) st->out_token = -2;
}
extern "C" lpp_status lpp_debug_wait_probe(lpp_engine* e) {
    NEED_READY(e);
    TRY(push_state(e, 0, 0, nullptr, nullptr, 0, 0.f, 0, 0));
    wait_probe_kernel<<<1, 32, 0, e->stream>>>(e->st);
    CU(cudaGetLastError());
    return pull_result(e, nullptr);
}

// Debugging aid (not part of the public header): per-CTA time stamps of the ring GEMV launches of one step.
extern "C" int lpp_debug_gemv_trace(lpp_engine* e, unsigned long long* out, int max_values) {
    if (!e || !e->gtrace || !out) return -1;
    const size_t n = (size_t)256 * e->num_sms * 8;
    if ((size_t)max_values < n) return -2;
    cudaStreamSynchronize(e->stream);
    if (cudaMemcpy(out, e->gtrace, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -3;
    return e->num_sms;
}

// Debugging aid (not part of the public header): the exact sampler's entry lists of its last stage.
extern "C" int lpp_debug_sampler_entries(lpp_engine* e, int* counts, void* entries, float* scalars) {
    if (!e || !e->exact_sampler) return -1;
    cudaStreamSynchronize(e->stream);
    cudaMemcpy(counts, e->ex_entry_count, e->sample_blocks * sizeof(int), cudaMemcpyDeviceToHost);
    cudaMemcpy(entries, e->ex_entries, (size_t)e->sample_blocks * kExactMaxEntries * sizeof(ExactEntry), cudaMemcpyDeviceToHost);
    cudaMemcpy(scalars, e->ex_scalars, 64 * sizeof(float), cudaMemcpyDeviceToHost);
    return e->sample_blocks;
}

#ifdef LPP_TIMING_AIDS
extern "C" int lpp_debug_pf_trace(lpp_engine* e, unsigned long long* out) {
    if (!e) return -1;
    cudaStreamSynchronize(e->stream);
    return (int)cudaMemcpyFromSymbol(out, g_pf_trace, sizeof(unsigned long long) * 160 * 48);
}
#endif

extern "C" const char* lpp_strerror(int s) {
    switch (s) {
        case LPP_OK: return "ok";
        case LPP_ERR_INVALID_ARG: return "invalid argument";
        case LPP_ERR_CUDA: return "CUDA error";
        case LPP_ERR_NOT_READY: return "engine not ready";
        case LPP_ERR_NCCL: return "NCCL error";
        case LPP_ERR_DEVICE_STATUS: return "device reported an error status";
        case LPP_ERR_TOO_LARGE: return "request exceeds capacity";
        case LPP_ERR_NO_DEVICE: return "no usable CUDA device";
    }
    return "unknown status";
}
extern "C" const char* lpp_last_error(void) { return g_err.c_str(); }
extern "C" void* lpp_engine_stream(lpp_engine* e) { return e ? (void*)e->stream : nullptr; }
extern "C" int lpp_kernels_per_step(const lpp_engine* e) { return e ? e->kernels_full : 0; }

static void kind_bytes(const lpp_engine* e, int pos, int64_t* b) {
    const lpp_config& c = e->c;
    const int64_t D = c.dim, L = c.n_layers, V = c.vocab_size, esz = e->esz;
    for (int k = 0; k < kKinds; ++k) b[k] = 0;
    b[kQkv] = L * ((int64_t)(e->Dq + 2 * e->KVd) * D * esz + 4 * D) + 4 * D;  // + att norms + embedding row
    b[kAttn] = L * (int64_t)e->kvesz * 2 * e->KVd * ((int64_t)pos + 1) + L * (int64_t)e->kvesz * 2 * e->KVd;
    b[kOproj] = L * D * e->Dq * esz;
    b[kGateUp] = L * ((int64_t)2 * e->Fl * D * esz + 4 * D);
    b[kDown] = L * D * e->Fl * esz;
    b[kLmHead] = (tp_cls_sharded(e) ? V / c.tp_size : V) * D * esz + 4 * D;
}
extern "C" int64_t lpp_step_bytes(const lpp_engine* e, int pos) {
    if (!e) return 0;
    int64_t b[kKinds], t = 0;
    kind_bytes(e, pos, b);
    for (int k = 0; k < kKinds; ++k) t += b[k];
    return t;
}

// Average duration of one launch of `kind` when all of the step's launches of that kind run back to
// back, with the launch attributes the step uses (programmatic dependent launch between them) and one
// CUDA event pair on the engine stream around the whole sequence.  Every launch streams its own
// layer's weights, so consecutive launches never find them in L2.  Activations are whatever the
// buffers hold: the results are meaningless and the next real step overwrites them.
extern "C" lpp_status lpp_profile_kind(lpp_engine* e, int pos, int kind, int iters, float* ms_per_launch, int* launches) {
    NEED_READY(e);
    if (!ms_per_launch || !launches || iters <= 0 || kind < 0 || kind >= kKinds) return fail(LPP_ERR_INVALID_ARG, "bad argument");
    if (pos < 0 || pos >= e->c.seq_len) return fail(LPP_ERR_INVALID_ARG, "pos out of range");
    *ms_per_launch = 0.f;
    *launches = 0;
    lpp_sample_params sp = {0.8f, 1.1f};
    cudaGraphExec_t gx = nullptr;
    int n_kernels = 0;
    e->only_kind = kind;
    lpp_status rs = capture(e, true, false, &gx, &n_kernels);
    e->only_kind = -1;
    if (rs != LPP_OK) return rs;
    if (n_kernels == 0 && kind != kAllReduce) {
        cudaGraphExecDestroy(gx);
        return LPP_OK;
    }
    float total = 0.f;
    for (int it = 0; it < iters + 2 && rs == LPP_OK; ++it) {  // two warm-up rounds
        rs = push_state(e, 0, pos, &sp, nullptr, 0, 0.5f, 0, 0);
        if (rs != LPP_OK) break;
        cudaEventRecord(e->ev0, e->stream);
        cudaError_t le = cudaGraphLaunch(gx, e->stream);
        cudaEventRecord(e->ev1, e->stream);
        cudaError_t se = cudaStreamSynchronize(e->stream);
        if (le != cudaSuccess || se != cudaSuccess) {
            rs = fail(LPP_ERR_CUDA, "profile kind: %s", cudaGetErrorString(le != cudaSuccess ? le : se));
            break;
        }
        float t = 0.f;
        cudaEventElapsedTime(&t, e->ev0, e->ev1);
        if (it >= 2) total += t;
    }
    cudaGraphExecDestroy(gx);
    if (rs == LPP_OK) {
        *launches = n_kernels;
        *ms_per_launch = n_kernels > 0 ? total / iters / n_kernels : total / iters;
    }
    return rs;
}

extern "C" lpp_status lpp_profile_step(lpp_engine* e, int pos, int iters, const lpp_sample_params* spp, float* ms,
                                       int* launches, int64_t* bytes) {
    NEED_READY(e);
    if (!ms || !launches || !bytes || iters <= 0) return fail(LPP_ERR_INVALID_ARG, "bad argument");
    if (pos < 0 || pos >= e->c.seq_len) return fail(LPP_ERR_INVALID_ARG, "pos out of range");
    for (int k = 0; k < kKinds; ++k) ms[k] = 0.f, launches[k] = 0;
    kind_bytes(e, pos, bytes);
    // the sampler that is timed is the one the caller's workload runs (argmax and categorical paths differ)
    const lpp_sample_params sp = spp ? *spp : lpp_sample_params{0.f, 1.f};
    const int hist[3] = {1, 2, 3};
    // The step is captured once more with an event-record node before and after every kernel and
    // replayed as a graph, so the durations carry no host launch latency.  Event nodes sit between
    // the kernels, hence no programmatic overlap: these are isolated per-kernel times.
    cudaGraphExec_t gx = nullptr;
    lpp_status rs = LPP_OK;
    {
        cudaGraph_t g = nullptr;
        CU(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
        e->profiling = e->profiling_capture = true;
        Recorder R{e, e->stream};
        record_step(R, true);
        e->profiling = e->profiling_capture = false;
        cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
        if (R.err != cudaSuccess || ce != cudaSuccess) {
            rs = fail(LPP_ERR_CUDA, "profile capture: %s", cudaGetErrorString(R.err != cudaSuccess ? R.err : ce));
        } else if (cudaGraphInstantiate(&gx, g, 0) != cudaSuccess) {
            rs = fail(LPP_ERR_CUDA, "profile graph instantiate failed");
        }
        if (g) cudaGraphDestroy(g);
        (void)cudaGetLastError();
    }
    for (int it = 0; it < iters + 1 && rs == LPP_OK; ++it) {  // iteration 0 is a warm-up
        rs = push_state(e, 0, pos, &sp, hist, 3, 0.5f, 0, 0);
        if (rs != LPP_OK) break;
        cudaError_t le = cudaGraphLaunch(gx, e->stream);
        cudaError_t se = cudaStreamSynchronize(e->stream);
        if (le != cudaSuccess || se != cudaSuccess) {
            rs = fail(LPP_ERR_CUDA, "profile step: %s", cudaGetErrorString(le != cudaSuccess ? le : se));
            break;
        }
        if (it == 0) continue;
        for (size_t i = 0; i + 1 < e->prof_events.size(); i += 2) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, e->prof_events[i], e->prof_events[i + 1]) != cudaSuccess) {
                rs = fail(LPP_ERR_CUDA, "cudaEventElapsedTime on graph event nodes failed");
                break;
            }
            ms[e->prof_kinds[i]] += t / iters;
            if (it == 1) launches[e->prof_kinds[i]]++;
        }
    }
    if (gx) cudaGraphExecDestroy(gx);
    for (cudaEvent_t ev : e->prof_events) cudaEventDestroy(ev);
    e->prof_events.clear();
    e->prof_kinds.clear();
    (void)cudaGetLastError();
    return rs;
}
