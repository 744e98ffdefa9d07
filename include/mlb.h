/*
 * mlb.h - C ABI of the B200 decode path (libmini_llm_b200.so).
 *
 * The reference (mini-llm-cuda) has no FFI: its decode path is a set of C++ free functions
 * over global pointers. Each entry point below names the reference interface it stands in
 * for. All functions return 0 (MLB_OK) on success and a negative mlb_status otherwise;
 * mlb_last_error() gives the thread-local message. The library never exits, aborts or
 * traps; every device-side wait is bounded. Buffers passed in are caller-owned HOST memory
 * unless a parameter says otherwise; objects returned are library-owned until *_free.
 * One mlb_session is driven by one host thread at a time; sessions on different GPUs may
 * be driven concurrently from different threads. There is no CPU fallback: without a CUDA
 * device every compute entry point fails with MLB_E_CUDA.
 */
#ifndef MLB_H_
#define MLB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLB_MAX_LAYERS 128

typedef enum mlb_status {
    MLB_OK = 0,
    MLB_E_INVALID = -1,      /* bad argument or inconsistent configuration            */
    MLB_E_IO = -2,           /* file missing / unreadable                             */
    MLB_E_FORMAT = -3,       /* malformed or truncated model.bin / JSON               */
    MLB_E_CUDA = -4,         /* CUDA runtime error (message holds the CUDA string)    */
    MLB_E_NOMEM = -5,        /* host or device allocation failed                      */
    MLB_E_KV_FULL = -6,      /* the paged KV pool has no free page                    */
    MLB_E_CONTEXT_FULL = -7, /* a sequence reached max_context                        */
    MLB_E_TIMEOUT = -8,      /* a bounded device-side wait ran out                    */
    MLB_E_UNSUPPORTED = -9   /* shape outside what the kernels are built for          */
} mlb_status;

typedef enum mlb_dtype {
    MLB_DT_DEFAULT = 0,      /* as the file's config says (float32 when it says nothing) */
    MLB_DT_F32 = 1,
    MLB_DT_BF16 = 2,
    MLB_DT_FP8_E4M3 = 3      /* weights only: per-output-row fp32 scale = max|row|/448 */
} mlb_dtype;

typedef enum mlb_layer_type { MLB_LAYER_ATTENTION = 0, MLB_LAYER_DELTA_NET = 1 } mlb_layer_type;

/* Runtime form of the reference's compile-time dims (network_meta.h:3-20). As an override
 * for mlb_model_load, a field < 0 (NaN for the floats) means "take it from the file". */
typedef struct mlb_config {
    int32_t dim, layers, heads, kv_heads, head_dim, ffn_dim, vocab, max_context;
    int32_t ple_dim;                 /* per-layer-embedding width, 0 = off                 */
    int32_t qk_norm, query_gating;   /* CONFIG_QK_RMS_NORM / CONFIG_QUERY_GATING           */
    int32_t dn_key_dim, dn_value_dim;/* gated delta-net per-head dims                      */
    int32_t weight_dtype, kv_dtype;  /* mlb_dtype                                          */
    int32_t layer_types_set;         /* override only: non-zero = layer_types[] is valid   */
    float rope_theta, rms_eps;
    uint8_t layer_types[MLB_MAX_LAYERS]; /* execution order (file block N-1 runs first)   */
} mlb_config;

typedef struct mlb_sampling {
    int32_t mode;            /* 0 = greedy (argmax of logits, lowest index on ties), 1 = top-k */
    int32_t top_k;           /* 1..1024 */
    float temperature;       /* > 0 */
    const uint64_t* seeds;   /* [batch] Philox keys, or NULL: key = sequence index */
} mlb_sampling;

typedef struct mlb_model mlb_model;     /* device weights of ONE GPU                     */
typedef struct mlb_session mlb_session; /* KV pages, delta-net state, stream for B seqs  */

/* One row per kernel kind launched by a decode step, filled by mlb_profile_decode. */
typedef struct mlb_kernel_stat {
    char name[48];
    int32_t launches;
    float total_ms;          /* CUDA-event time on the session's stream, summed           */
    uint64_t bytes;          /* algorithmic bytes moved, summed over the launches         */
    uint64_t flops;          /* algorithmic flops, summed                                 */
} mlb_kernel_stat;

void mlb_config_init(mlb_config* cfg);  /* fills every field with "unset" */

/* Replaces loadModel (load_model.h:6, load_model.cu:286-481) + the weight half of
 * allocateMemory (memory_allocation.cu:354-499): parses the container, uploads the
 * matrices in their file order (row-major [out][in] is the streaming layout; the
 * reference's host transpose is not needed) and rounds them to `weight_dtype`. */
int mlb_model_load(const char* path, int device, const mlb_config* override_or_null, mlb_model** out);
int mlb_model_get_config(const mlb_model* m, mlb_config* out);
/* Bytes of every tensor a decode step streams once (projections, tied embedding/LM head,
 * gains, scales), the W term of the per-step roofline. */
uint64_t mlb_model_weight_bytes(const mlb_model* m);
void mlb_model_free(mlb_model* m);

/* Host-only: parse the header of a model file (no GPU needed). */
int mlb_file_inspect(const char* path, const mlb_config* override_or_null, mlb_config* out,
                     uint64_t* n_params);

/* Replaces the activation half of allocateMemory (memory_allocation.cu:500-552): instead of
 * maxL-sized scratch per op it owns a paged KV cache (pages of kv_block positions),
 * fp32 delta-net state and one decode step's scratch. kv_pages = 0 sizes the pool for
 * batch * max_context. A session of 4 sequences or more on an FP8 model runs its steps as
 * tensor-core GEMMs on a bf16 copy of the weights that the model builds on the device the first
 * time (2 bytes per weight, shared by all its sessions); MLB_GEMM=simt in the environment keeps
 * the FP8 GEMV kernels. */
int mlb_session_new(mlb_model* m, int batch, int max_context, int kv_block, int kv_pages,
                    mlb_session** out);
int mlb_session_reset(mlb_session* s);
void mlb_session_free(mlb_session* s);

/* Replaces loadStoryContext's upload (main.cu:166) and the prompt part of the reference's
 * recompute-everything loop: ingests tokens[b*stride .. +lens[b]) for every sequence. After
 * it, position lens[b]-1 holds the last prompt token as the pending input of the next step.
 * With bf16 or FP8 weights and 64 prompt tokens or more the prompt is consumed as columns of
 * tensor-core steps, 256 tokens at a time (bf16 activations: the cache equals the token loop's
 * within the low-precision tolerance; an FP8 model gets a bf16 copy of its weights on the device
 * the first time, 2 bytes per weight); otherwise, or with MLB_PREFILL=step in the environment,
 * one token per step and sequence. MLB_PREFILL=chunk asks for the columns and fails with
 * MLB_E_UNSUPPORTED where they cannot run. */
int mlb_prefill(mlb_session* s, const int32_t* tokens, const int32_t* lens, int stride);

/* ---- several GPUs of one box ---------------------------------------------------------------------
 * The reference runs on device 0 only (memory_allocation.cu:329, no cudaSetDevice anywhere). A pool
 * serves `batch` sequences from n_devices GPUs: every device holds a full replica of the weights and the
 * KV pages / delta-net state of a contiguous block of the sequences (mlb_shard_range: the first
 * batch % n_devices devices hold one more); calls run one host thread and one stream per device and
 * return when all are done. No data crosses between the devices. A device index may repeat (two
 * shards on one GPU). Arrays are laid out as for a session of `batch` sequences. */
typedef struct mlb_pool mlb_pool;
int mlb_shard_range(int n_items, int n_shards, int shard, int* begin, int* end);      /* host only */
int mlb_pool_new(const char* model_path, const int* devices, int n_devices, int batch, int max_context,
                 const mlb_config* override_or_null, mlb_pool** out);
void mlb_pool_free(mlb_pool* p);
/* Writes device and sequence range of up to `cap` shards; returns the number of shards. */
int mlb_pool_shards(const mlb_pool* p, int* devices, int* begins, int* ends, int cap);
int mlb_pool_set_stop_token(mlb_pool* p, int token_id);
int mlb_pool_prefill(mlb_pool* p, const int32_t* tokens, const int32_t* lens, int stride);
/* out_tokens [batch][n]; with top-k sampling and no seeds the Philox key of a sequence is its index in
 * the pool, so the ids do not depend on the number of devices. */
int mlb_pool_decode_n(mlb_pool* p, const mlb_sampling* sampling, int n, int32_t* out_tokens);

/* Teacher-forced scoring forward: the full-sequence forward of runInference(L)
 * (inference.cu:376-752), whose [V x L] scores the reference's trainer consumes
 * (training_orchestrator.cu:308). logits_out [len][V] fp32 host, row t = prediction after
 * tokens[0..t] (the reference's column t of vocabScores_DEVICE, before the softmax). The tokens
 * run as columns of tensor-core steps like a long prompt, with the LM head on every column (bf16 or FP8
 * weights; activations are bf16, i.e. the logits agree with the fp32 forward within the low-precision
 * tolerance). With fp32 weights, or with MLB_SCORE=step in the environment, the tokens run through the
 * token loop instead (fp32 activations, the fp32 bound of the decode path; about 0.2 ms per token).
 * Uses sequence 0 of the session; the session is reset before and after. */
int mlb_score_tokens(mlb_session* s, const int32_t* tokens, int len, float* logits_out);

/* Replaces one iteration of the while loop of runInferenceLoop
 * (inference_orchestrator.cu:64-160): forward for the pending token of every sequence, pick
 * the next token on the device, append it. in_tokens (nullable) overrides the pending tokens
 * from the host first, as the reference's per-step upload does (:154). out_tokens receives
 * [batch] ids (-1 for a sequence that is at max_context or has drawn the stop token). */
int mlb_decode_step(mlb_session* s, const mlb_sampling* sampling, const int32_t* in_tokens,
                    int32_t* out_tokens);
/* Stop token of the session (-1, the default: none). The reference's loop ends only at maxL
 * (inference_orchestrator.cu:64); a serving loop also ends a sequence at an end-of-text id. The kernel that
 * appends a picked id compares it with this one and, on a match, takes the sequence out of all later steps
 * (the id itself is appended and returned); the other sequences of the batch go on. mlb_session_stopped
 * writes [batch] flags: 1 = the sequence has drawn the stop token since the last reset / prefill. */
int mlb_session_set_stop_token(mlb_session* s, int token_id);
int mlb_session_stopped(mlb_session* s, int32_t* out_flags);
/* n steps back to back without host round trips; out_tokens is [batch][n] (-1 behind the end of a sequence:
 * max_context reached, or the stop token drawn). */
int mlb_decode_n(mlb_session* s, const mlb_sampling* sampling, int n, int32_t* out_tokens);
/* As mlb_decode_n, timing each step with CUDA events on the session's stream; flush_l2
 * writes a buffer larger than L2 before each step, outside the per-step bracket. total_ms
 * (nullable) is first start to last end, flushes included when they are on. */
int mlb_decode_timed(mlb_session* s, const mlb_sampling* sampling, int n, int flush_l2,
                     float* step_ms, float* total_ms, int32_t* out_tokens);
/* Runs n steps kernel by kernel with events around every launch. */
int mlb_profile_decode(mlb_session* s, const mlb_sampling* sampling, int n, int flush_l2,
                       mlb_kernel_stat* stats, int max_stats, int* n_stats);

/* Parity probes, off the timed path. Logits of the LAST executed step, fp32 [batch][vocab]
 * (the reference keeps them in vocabScores_DEVICE, inference.cu:738). */
int mlb_get_logits(mlb_session* s, float* out);
/* Column L-1 of the reference's vocabScores_postSoftmax_DEVICE (inference.cu:745-749) for
 * one sequence: softmax of the last step's logits, [vocab]. */
int mlb_get_probs_col(mlb_session* s, int seq, float* out);
int mlb_session_positions(mlb_session* s, int32_t* out /* [batch] */);
/* Algorithmic bytes of the NEXT decode step at the current positions: weights once, KV read
 * + append, delta-net state read + write, embedding/PLE rows. */
int mlb_session_step_bytes(mlb_session* s, uint64_t* weights, uint64_t* kv, uint64_t* state,
                           uint64_t* rows);
/* Kernels launched per decode step by the current configuration. */
int mlb_session_launches_per_step(mlb_session* s);
/* Diagnostics of the batch-1 single-kernel step (no counterpart in the reference). When the
 * session was created with MLB_GRID_TIMERS=1 in the environment, mlb_session_grid_timers copies
 * 32 cycle counters per CTA (summed over the steps since the last call; what each one covers is
 * listed beside kGridTimerSlots in csrc/grid_params.h), clears them and returns the number of
 * CTAs; returns 0 when the session does not run that step or keeps no counters.
 * mlb_session_grid_trace copies 256 events per CTA of the last step of the shape-specialised
 * kernel: (global nanosecond timer << 8) | counter index at every point where a counter is
 * updated; 0 when no trace is kept. */
int mlb_session_grid_timers(mlb_session* s, long long* out, int cap);
int mlb_session_grid_trace(mlb_session* s, long long* out, int cap);

/* Host-only page allocator of the KV cache, exposed so that its failure paths can be
 * tested without a device. */
typedef struct mlb_kv_alloc mlb_kv_alloc;
int mlb_kv_alloc_new(int num_pages, int batch, int max_pages_per_seq, mlb_kv_alloc** out);
int mlb_kv_alloc_ensure(mlb_kv_alloc* a, int seq, int n_positions, int block);
int mlb_kv_alloc_table(const mlb_kv_alloc* a, int seq, int32_t* out, int max_entries);
int mlb_kv_alloc_free_pages(const mlb_kv_alloc* a);
void mlb_kv_alloc_release(mlb_kv_alloc* a, int seq);
void mlb_kv_alloc_free(mlb_kv_alloc* a);

/* Stand-alone split-K flash-decode attention over a paged KV cache - the kernel that replaces
 * the reference's K^T Q GEMM, mask/scale, softmax kernels and V P GEMM (inference.cu:510-579)
 * inside a decode step - on DEVICE pointers owned by the caller:
 *   kpool/vpool [page][kv_heads][16][head_dim] (kv_dtype float32 or bfloat16), page_table
 *   [batch][pt_stride] int32, positions [batch] int32 (sequence b attends to positions
 *   0..positions[b], which must already be in the cache), q [batch][heads*head_dim] fp32
 *   (normalised and rotated), gate (nullable) [batch][heads*head_dim] sigmoid gates,
 *   out [batch][heads*head_dim] fp32. `stream` is a cudaStream_t (NULL = default stream).
 * num_pages is the number of pages the pools hold. The page table is the caller's, so the kernel
 * checks it: a sequence whose position needs more than pt_stride pages is skipped, a page id
 * outside [0, num_pages) is replaced by page 0, and the call returns MLB_E_INVALID (nothing
 * outside the caller's buffers is read).
 * Allocates its split-combine scratch with cudaMalloc for the call and returns after the
 * stream has finished. */
int mlb_op_attn_decode(const void* kpool, const void* vpool, int kv_dtype, const int32_t* page_table,
                       int pt_stride, int num_pages, const int32_t* positions, const float* q,
                       const float* gate_or_null, float* out, int batch, int heads, int kv_heads, int head_dim,
                       int splits, void* stream);

/* Stand-alone batched projection on the tensor cores (tcgen05 + TMEM, TMA-fed), DEVICE pointers:
 * the kernel that replaces the reference's cublasGemmEx projections (inference.cu:401-465,
 * :581-602, :623-695, :720-743) once the batch is >= 4. W [N][K] bf16 row-major, X [batch][K]
 * bf16; K a multiple of 8. Three forms, chosen by the optional pointers:
 *   plain      out fp32 [batch][N] = X W^T
 *   residual   out fp32 [batch][N] = X W^T + resid (resid may alias out)
 *   gate/up    out bf16 [batch][N] = silu(X W^T) * (X W_up^T)
 * Returns after the stream has finished. */
int mlb_op_gemm_bf16(const void* W, const void* W_up_or_null, const void* X, const float* resid_or_null,
                     void* out, int N, int K, int batch, void* stream);

/* No counterpart in the reference. Same operator and arguments as mlb_op_attn_decode, for
 * callers that cannot allocate device memory: a server that has given all free device memory
 * to its own pool, or a token loop that must never run into the device-wide synchronisation
 * of cudaMalloc / cudaFree. The split-combine scratch lives in a fixed 4 MiB array inside the
 * library image (held by every GPU that loads the library until the process exits); the call
 * makes no cudaMalloc / cudaFree and does not wait for the stream - the result is ready when
 * `stream` reaches this point. Shapes whose scratch (about batch*heads*splits*(head_dim+2)*4
 * bytes) exceeds mlb_op_attn_decode_static_capacity() are refused with MLB_E_UNSUPPORTED.
 * The FIRST call on each device resolves the array's address (a one-time runtime query): make
 * that call with the device current and before any stream capture starts. With CUDA's lazy
 * module loading that query is also what places the array in device memory, so make it before
 * the host claims all the memory (or set CUDA_MODULE_LOADING=EAGER); MLB_E_NOMEM otherwise.
 * All calls on a device share the array, so calls whose kernels could overlap on the GPU (two
 * streams, two threads) race; keep them ordered.
 * Because the call does not wait, a page table that does not fit (see mlb_op_attn_decode) is
 * reported by mlb_op_attn_decode_static_status, which waits for `stream` and returns
 * MLB_E_INVALID if the last call on the current device met one (it allocates nothing either). */
int mlb_op_attn_decode_static(const void* kpool, const void* vpool, int kv_dtype, const int32_t* page_table,
                              int pt_stride, int num_pages, const int32_t* positions, const float* q,
                              const float* gate_or_null, float* out, int batch, int heads, int kv_heads,
                              int head_dim, int splits, void* stream);
int mlb_op_attn_decode_static_status(void* stream);
size_t mlb_op_attn_decode_static_capacity(void);

/* No counterpart in the reference. Exercises the bounded wait that every streaming kernel of the
 * library uses: a one-thread kernel waits on `device` for a shared-memory barrier that nothing
 * completes, gives up after `max_polls` polls (1..2^20, a few milliseconds at most) and records an
 * error code the way those kernels do. Returns MLB_E_TIMEOUT (the expected outcome) once the
 * kernel has ended; the CUDA context stays usable. */
int mlb_op_wait_probe(int device, uint32_t max_polls);

/* RoPE table exactly as getPreComputedRopeTheta builds it (inference.h:4,
 * inference.cu:364-374): [max_len][head_dim] interleaved (cos, sin), host float math. */
void mlb_rope_table(float* table, int max_len, int head_dim, float base);

const char* mlb_last_error(void);
const char* mlb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MLB_H_ */
