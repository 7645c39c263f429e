/* lpp_b200 -- C ABI of the B200 (sm_100a) batch-1 decode engine.
 *
 * This is the drop-in boundary for Lighter++'s per-token hot path.  Lighter++ has no FFI layer of
 * its own: its host code calls C++ free functions chosen at compile time by USE_CUDA.  Every entry
 * point below names the reference interface (file:line in the Lighter++ tree) it stands in for; the
 * C++ shim under lighterpp_b200/csrc/shim/ re-creates those reference symbols on top of this ABI so
 * the reference's main.cpp / loader.cpp / runtests.cpp link against it unchanged.
 *
 * Conventions: every function returns an lpp_status (0 = success) and never exits the process or
 * throws; pointers named h_* are host memory, d_* device memory; an engine belongs to one host
 * thread at a time and owns one CUDA stream on one device.
 */
#ifndef LPP_B200_H
#define LPP_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lpp_engine lpp_engine;

typedef enum {
    LPP_OK = 0,
    LPP_ERR_INVALID_ARG = 1,   /* NULL pointer, out-of-range index, unsupported shape */
    LPP_ERR_CUDA = 2,          /* a CUDA runtime call failed; see lpp_last_error() */
    LPP_ERR_NOT_READY = 3,     /* weights missing / engine not finalized */
    LPP_ERR_NCCL = 4,          /* NCCL could not be loaded or a collective failed */
    LPP_ERR_DEVICE_STATUS = 5, /* a kernel reported a bounded-wait timeout or bad index */
    LPP_ERR_TOO_LARGE = 6,     /* request exceeds a fixed capacity */
    LPP_ERR_NO_DEVICE = 7      /* no usable CUDA device */
} lpp_status;

/* Element types.  Values 0/1 match the reference's WeightPrecision (src/model.h:8-12) and GGMLType
 * F32/F16 (src/gguf.h:10-12). */
typedef enum { LPP_F32 = 0, LPP_F16 = 1 } lpp_dtype;
typedef enum { LPP_MEM_HOST = 0, LPP_MEM_DEVICE = 1 } lpp_memkind;

/* Which reference tensor an upload carries: one value per transformerWeights member
 * (src/model.h:34-53). */
typedef enum {
    LPP_T_TOK_EMB = 0,  /* token_embedding_table [V][D]                                   */
    LPP_T_RMS_ATT = 1,  /* rms_att_weight        [D]      per layer                       */
    LPP_T_WQ = 2,       /* wq                    [D][D]   per layer                       */
    LPP_T_WK = 3,       /* wk                    [KV][D]  per layer                       */
    LPP_T_WV = 4,       /* wv                    [KV][D]  per layer                       */
    LPP_T_WO = 5,       /* wo                    [D][D]   per layer                       */
    LPP_T_RMS_FFN = 6,  /* rms_ffn_weight        [D]      per layer                       */
    LPP_T_W1 = 7,       /* w1 (gate)             [F][D]   per layer                       */
    LPP_T_W2 = 8,       /* w2 (down)             [D][F]   per layer                       */
    LPP_T_W3 = 9,       /* w3 (up)               [F][D]   per layer                       */
    LPP_T_RMS_FINAL = 10, /* rms_final_weight    [D]                                      */
    LPP_T_W_CLS = 11,   /* w_cls                 [V][D]   (omit for tied embeddings)      */
    LPP_T_COUNT = 12
} lpp_tensor;

/* Engine flags (lpp_config.flags). */
#define LPP_FLAG_GEMV_LDG 0x1u   /* stream weights with 128-bit global loads instead of the bulk-copy ring */
#define LPP_FLAG_NO_PDL 0x2u     /* plain stream order between kernels (no programmatic dependent launch) */
#define LPP_FLAG_NO_GRAPH 0x4u   /* launch the step kernel by kernel instead of replaying the CUDA graph */
#define LPP_FLAG_FAST_SAMPLER 0x10u /* tree-sum sampler: ~20 us faster per token, categorical ids no longer follow the
                                      reference's sequential FP32 sums bit for bit */
#define LPP_FLAG_TP_NCCL 0x20u   /* tensor parallelism: keep the NCCL all-reduce after o_proj / down even when the peers
                                  * are mapped (lpp_tp_connect); default is the exchange fused into the GEMVs */
#define LPP_FLAG_NO_PREFILL_GEMM 0x80u /* lpp_prefill feeds the prompt token by token (the reference's way) instead of
                                        * through the batched tensor-core path */
#define LPP_FLAG_TP_LOCAL 0x40u  /* tensor parallelism without NCCL: the engine never loads or initialises NCCL and
                                  * nccl_id may be NULL; only the peer-memory exchange (lpp_tp_connect) can run */

/* Mirror of the reference Config (src/model.h:21-31) plus what a device engine needs. */
typedef struct {
    int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_base;
    int32_t weight_dtype; /* lpp_dtype of the matrices and the embedding as held on the device      */
    int32_t kv_dtype;     /* lpp_dtype of the KV cache: LPP_F16 like the reference GPU path
                             (src/model.h:108-109) or LPP_F32 like its CPU path (src/model.h:93-94)  */
    int32_t tp_rank, tp_size; /* tensor-parallel rank / degree (1 = single GPU)                     */
    int32_t device;       /* CUDA device ordinal                                                    */
    uint32_t flags;       /* LPP_FLAG_*                                                             */
    int32_t ring_kb;      /* shared-memory weight ring per CTA in KiB (0 = default)                 */
    int32_t attn_splits;  /* KV splits of the flash-decode kernel (0 = default)                     */
    int32_t wait_ms;      /* limit of a device-side wait on this GPU's own work, in milliseconds of SM
                             clocks (0 = default, about 50 ms); when it runs out the step ends with
                             LPP_ERR_DEVICE_STATUS instead of hanging                               */
    int32_t tp_wait_ms;   /* the same for a wait on a tensor-parallel peer (0 = default, seconds)   */
} lpp_config;

/* Sampling parameters of one step: forward()'s temperature / penalty arguments
 * (src/model.h:164).  top-p is not part of the device sampler, as in src/sample.cu:210-214. */
typedef struct {
    float temperature; /* 0 = argmax */
    float penalty;     /* repetition penalty, applied only when > 1 (src/model.cpp:259) */
} lpp_sample_params;

/* ---- lifetime: malloc_run_state / free_run_state (src/model.cpp:18-118) and the device half of
 *      the loaders (src/loader.cpp:73-131, 543-637) ------------------------------------------- */

/* nccl_id: 128-byte ncclUniqueId shared by all ranks when tp_size > 1 (from lpp_nccl_unique_id on
 * rank 0), NULL otherwise. */
lpp_status lpp_engine_create(const lpp_config* cfg, const void* nccl_id, lpp_engine** out);
lpp_status lpp_engine_destroy(lpp_engine* e);
lpp_status lpp_nccl_unique_id(void* out128);

/* Hand one reference-layout tensor (row-major, rows = output features; FULL, unsharded) to the
 * engine, which keeps its tensor-parallel share in its own fused layout.  layer is ignored for the
 * unstacked tensors.  Replaces the cudaMalloc+cudaMemcpy pairs of src/loader.cpp:77-130 and
 * upload_tensor_to_offset (src/loader.cpp:410-422).  src_dtype may differ from cfg.weight_dtype
 * (F16 <-> F32 conversion, exact when widening). */
lpp_status lpp_upload_tensor(lpp_engine* e, int which, int layer, const void* src, int src_dtype, int memkind);
/* Checks that every tensor arrived, ties the classifier to the embedding if w_cls was never
 * uploaded (src/loader.cpp:66, 471, 619-632), captures the step graph. */
lpp_status lpp_finalize(lpp_engine* e);

/* Tensor parallelism over peer memory (one process per GPU, tp_size <= 8).  No counterpart in the
 * reference, which has no multi-GPU code: its o_proj / down results (src/model.cpp:201, 238) are
 * complete on the one device.  Here every rank holds a slice of the heads and of the FFN columns, the
 * residual GEMV of every rank stores its partial rows straight into all ranks' receive areas over NVLink and
 * the next GEMV adds the tp_size partial vectors in rank order while it stages its input.  Each rank
 * exports an IPC handle of its receive buffer (LPP_TP_HANDLE_BYTES bytes), the caller gathers the
 * handles of all ranks in rank order over its own host channel and hands them to every engine before
 * lpp_finalize.  Without lpp_tp_connect (or with LPP_FLAG_TP_NCCL) the NCCL all-reduce is used. */
#define LPP_TP_HANDLE_BYTES 64
lpp_status lpp_tp_export(lpp_engine* e, void* handle, size_t handle_bytes);
lpp_status lpp_tp_connect(lpp_engine* e, const void* handles, size_t handle_bytes_each);

/* ---- the hot path ---------------------------------------------------------------------------- */

/* forward(token, pos, ..., temperature, topp, penalty, history, history_len) of src/model.cpp:342-384:
 * one decode step plus the fused sampler; *next_token receives the sampled id.  r is the uniform
 * draw the reference takes from rand() (src/sample.cu:211, src/model.cpp:292); pass the same value to
 * reproduce its choice.  h_history may be NULL when penalty <= 1. */
lpp_status lpp_step(lpp_engine* e, int token, int pos, const lpp_sample_params* sp, const int* h_history,
                    int history_len, float r, int* next_token);

/* The same step without the sampler's effect on the caller: runs the graph, then copies the raw
 * logits (before penalty/temperature) to h_logits[vocab_size].  Used for parity checks against
 * forward()'s logits (src/model.cpp:380). */
lpp_status lpp_step_logits(lpp_engine* e, int token, int pos, float* h_logits);

/* The generate loop of src/main.cpp:199-223 kept on the device: n steps starting from
 * (first_token, start_pos); each sampled token feeds the next step and joins a history window of
 * history_window entries (64 in src/main.cpp:158) seeded with h_history[0..history_len).  h_r holds
 * one uniform draw per step.  No host round trip happens between steps; h_out_tokens[n] is copied
 * back once at the end.  *device_ms (optional) receives the CUDA-event time of the n steps. */
lpp_status lpp_decode(lpp_engine* e, int first_token, int start_pos, int n, const lpp_sample_params* sp,
                      const int* h_history, int history_len, int history_window, const float* h_r,
                      int* h_out_tokens, float* device_ms);

/* The prompt loop of src/main.cpp:163-179 without its n calls of forward(): fills the K/V cache rows of positions
 * start_pos .. start_pos + n - 1 for the n prompt tokens and produces no logits (feed the LAST prompt token to
 * lpp_step / lpp_step_logits as usual, and only the tokens before it to this call).  With FP16 weights, an FP16
 * cache and one GPU the tokens go through the layers in blocks of 64: every matrix is streamed once per block by a
 * TMA-fed tensor-core GEMM (activations rounded to FP16 as operands, FP32 accumulation), followed by causal
 * attention inside the block; other engines (or LPP_FLAG_NO_PREFILL_GEMM) run the step graph once per token.
 * *device_ms (optional) receives the CUDA-event time. */
lpp_status lpp_prefill(lpp_engine* e, const int* h_tokens, int n, int start_pos, float* device_ms);

/* cuda_sample (src/kernels.cuh:36, src/sample.cu:210-214) on caller-supplied logits: copies
 * h_logits[vocab_size] to the device and runs the engine's sampler on them. */
lpp_status lpp_sample_logits(lpp_engine* e, const float* h_logits, const lpp_sample_params* sp,
                             const int* h_history, int history_len, float r, int* token);

/* ---- KV cache access (layout [L][KVH][seq_len][head_size], src/scatter_kv.cu:15-16) ------------ */

/* Fill positions [0, n_pos) of one layer from full-head arrays [n_kv_heads][n_pos][head_size]. */
lpp_status lpp_kv_prefill(lpp_engine* e, int layer, const void* k, const void* v, int n_pos, int src_dtype,
                          int memkind);
/* Read one cache row (this rank's kv heads only) as FP32; h_k / h_v hold head_size floats. */
lpp_status lpp_kv_read(lpp_engine* e, int layer, int kv_head, int pos, float* h_k, float* h_v);
/* Element offset, inside this engine's K (or V) cache allocation, of element `off` of kv head
 * `kv_head` (rank-local numbering) at `pos`: the reference's scatter index. */
int64_t lpp_kv_index(const lpp_engine* e, int layer, int kv_head, int pos, int off);

/* ---- introspection ---------------------------------------------------------------------------- */

const char* lpp_strerror(int status);
const char* lpp_last_error(void);           /* detail text of the calling thread's last failure */
void* lpp_engine_stream(lpp_engine* e);     /* the cudaStream_t every launch of this engine uses */
int lpp_kernels_per_step(const lpp_engine* e); /* own kernel launches in one step graph */
/* Algorithmic HBM bytes of one step at position pos on this rank: every weight byte once + norm
 * weights + one embedding row + K/V rows 0..pos + this token's K/V write. */
int64_t lpp_step_bytes(const lpp_engine* e, int pos);

/* Per-kernel-kind timing of one step at `pos`: the step is captured with a CUDA event-record node
 * before and after every kernel and replayed iters times (isolated kernel durations, no programmatic
 * overlap, no host launch latency).  kinds: 0 qkv gemv, 1 attention, 2 o_proj gemv, 3 gate|up gemv, 4 down gemv,
 * 5 lm-head gemv, 6 sampler, 7 all-reduce, 8-9 reserved.  ms[10] total device ms per step per
 * kind, launches[10] launches per step, bytes[10] algorithmic bytes per step.  The sampler runs with the
 * temperature and penalty given in *sp (NULL = temperature 0, no penalty). */
lpp_status lpp_profile_step(lpp_engine* e, int pos, int iters, const lpp_sample_params* sp, float* ms, int* launches,
                            int64_t* bytes);

/* Average duration of one launch of kernel kind `kind` (numbering above) when the step's launches of
 * that kind run back to back at `pos`, launched as the step launches them (programmatic dependent
 * launch between consecutive kernels), timed with one CUDA event pair on the engine stream around
 * the sequence and averaged over `iters` repetitions.  Each launch streams its own layer's weights.
 * *launches = launches of that kind per step.  The activations the kernels see are stale: call it
 * between steps, never inside a run. */
lpp_status lpp_profile_kind(lpp_engine* e, int pos, int kind, int iters, float* ms_per_launch, int* launches);

/* ---- standalone operators: the host wrappers of src/kernels.cuh:24-36, device pointers in/out,
 *      launched on `stream` (a cudaStream_t, NULL = default stream) ------------------------------ */

lpp_status lpp_op_convert_f32_to_f16(void* d_dst, const float* d_src, int64_t n, void* stream);
lpp_status lpp_op_gemv(float* d_out, const float* d_x, const void* d_w, int n, int d, int w_dtype, void* stream);
lpp_status lpp_op_rmsnorm(float* d_out, const float* d_x, const float* d_w, int n, void* stream);
lpp_status lpp_op_rope(float* d_q, float* d_k, int pos, int dim, int kv_dim, int head_size, float rope_base,
                       void* stream);
lpp_status lpp_op_swiglu(float* d_hb, const float* d_h1, const float* d_h3, int size, void* stream);
lpp_status lpp_op_softmax_multihead(float* d_out, const float* d_x, int n_heads, int seq_len, int att_stride,
                                    void* stream);
lpp_status lpp_op_scale_multihead(float* d_att, float scale, int n_heads, int seq_len, int att_stride,
                                  void* stream);
lpp_status lpp_op_aggregation_multihead(float* d_out, const void* d_v_f16, const float* d_att, int n_heads,
                                        int seq_len, int head_size, int gqa_factor, int att_stride, void* stream);
lpp_status lpp_op_residual_add(float* d_out, const float* d_a, const float* d_b, int n, void* stream);
lpp_status lpp_op_scatter_kv(void* d_kc_f16, void* d_vc_f16, const float* d_k, const float* d_v, int layer,
                             int pos, int n_kv_heads, int head_size, int seq_len, void* stream);
lpp_status lpp_op_multihead_gemv(float* d_out, const float* d_q, const void* d_k_cache_f16, int layer, int pos,
                                 int n_heads, int n_kv_heads, int head_size, int seq_len, void* stream);
/* Fused rope + KV scatter (the step path's form of the two calls above). */
lpp_status lpp_op_rope_scatter(float* d_q, const float* d_k, const float* d_v, void* d_kc_f16, void* d_vc_f16,
                               int layer, int pos, int dim, int n_kv_heads, int head_size, int seq_len,
                               float rope_base, void* stream);
/* cuda_sample (src/kernels.cuh:36): d_logits is modified in place like the reference kernel does (penalty,
 * temperature, probabilities).  Runs the exact-order kernel (ids equal to the reference's CPU sample() on the same
 * logits and r) whenever vocab_size <= 2048 x the GPU's SM count, the tree-sum kernel beyond that. */
lpp_status lpp_op_sample(float* d_logits, int vocab_size, float temperature, float penalty, const int* d_history,
                         int history_len, float r, int* d_sampled_token, void* stream);

/* lpp_op_sample for callers that must not allocate.  No counterpart in the reference: its
 * cuda_sample works in place with shared memory only, while this library's multi-block sampler needs
 * global scratch (step state, per-block partials, counters, the entry lists of the exact-order kernel)
 * that lpp_op_sample takes from the stream-ordered allocator on every call.  Some hosts cannot do that: a
 * serving loop whose device memory was handed out in full at start-up, code that runs while another
 * stream is being captured into a CUDA graph in global capture mode (where allocation calls are
 * refused), or a real-time path that cannot tolerate an allocator's occasional synchronisation.  Here
 * the scratch is a fixed array inside the library image (about 0.4 MiB per GPU, held from load until
 * the process exits), so this call makes no allocation of any kind.  It runs the same kernels as
 * lpp_op_sample and returns the same token.
 *
 * Limits and rules: vocab_size <= 262144 and history_len <= 4096, otherwise LPP_ERR_TOO_LARGE
 * (lpp_last_error() says which).  The first call on each device looks up the array's device address
 * and must therefore run with that device current and outside any stream capture; later calls
 * only launch kernels.  All calls on a device share the one array: two calls whose kernels can
 * overlap on the GPU (different streams without ordering) race and give undefined results, so order
 * them.  Everything that has to start clean is rewritten at the start of every call.  Arguments and
 * result are those of lpp_op_sample. */
lpp_status lpp_op_sample_static(float* d_logits, int vocab_size, float temperature, float penalty,
                                const int* d_history, int history_len, float r, int* d_sampled_token,
                                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LPP_B200_H */
