/* C ABI of libcandle_moe_sm100.so: the quantized mixture-of-experts feed-forward block of
 * candle-transformers' quantized_llama (MlpOrMoe::MoE) as CUDA launchers for sm_100a.
 *
 * Conventions (all entry points):
 *   - return 0 on success, a negative CANDLE_MOE_E_* code for an argument error found on the host
 *     before anything is enqueued, or a positive cudaError_t value; nothing aborts or throws;
 *   - every pointer named "device" is a CUDA device pointer borrowed until the enqueued work has
 *     run; the caller owns every buffer; nothing is allocated or freed inside the library unless
 *     the entry point says so;
 *   - work is enqueued on the caller's stream (a cudaStream_t passed as void*) and is
 *     asynchronous; no entry point synchronises the stream;
 *   - weights are raw GGUF blocks exactly as candle's QCudaStorage holds them (row-major
 *     [n][k / block] blocks, candle-core/src/quantized/cuda.rs:597-616); dtypes are GGML ids
 *     (GgmlDType::to_u32, candle-core/src/quantized/mod.rs:176-195);
 *   - activations are contiguous row-major f32, ids are u32, like the tensors the reference block
 *     passes between its steps.
 * Each declaration cites the reference code it replaces (paths inside the candle workspace).
 */
#ifndef CANDLE_MOE_H_
#define CANDLE_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CANDLE_MOE_API __attribute__((visibility("default")))
#else
#define CANDLE_MOE_API
#endif

#define CANDLE_MOE_MAX_EXPERTS 128
#define CANDLE_MOE_MAX_TOPK 8

/* GGML dtype ids of the supported weight formats */
#define CANDLE_GGML_Q8_0 8
#define CANDLE_GGML_Q4K 12
#define CANDLE_GGML_Q6K 14

/* error codes */
#define CANDLE_MOE_OK 0
#define CANDLE_MOE_E_NULL (-1)        /* a required pointer is NULL */
#define CANDLE_MOE_E_SHAPE (-2)       /* a dimension is zero, too large or not a block multiple */
#define CANDLE_MOE_E_DTYPE (-3)       /* weight dtype not one of Q8_0 / Q4K / Q6K */
#define CANDLE_MOE_E_WORKSPACE (-4)   /* workspace smaller than candle_moe_workspace_bytes says */
#define CANDLE_MOE_E_ALIGN (-5)       /* a pointer does not meet the documented alignment */
#define CANDLE_MOE_E_NO_DEVICE (-6)   /* no CUDA device / not an sm_100 device */
#define CANDLE_MOE_E_STATIC_SCRATCH (-7) /* the call needs more scratch than CANDLE_MOE_STATIC_SCRATCH_BYTES */
#define CANDLE_MOE_E_NCCL (-8)        /* libnccl could not be loaded or an NCCL call failed (candle_moe_ep_last_error) */
#define CANDLE_MOE_E_EP_MISMATCH (-9) /* the ranks' exchange metadata disagree; every rank returns this, nothing was exchanged */

/* size of the built-in scratch area used by candle_moe_forward_static (per GPU, held until exit) */
#define CANDLE_MOE_STATIC_SCRATCH_BYTES (16u << 20)

/* Weights of one block, as MlpOrMoe::MoE holds them
 * (candle-transformers/src/models/quantized_llama.rs:134-141; Mlp :117-122).  The pointer arrays
 * are HOST arrays of n_experts DEVICE pointers, one per `experts[i].feed_forward_w{1,2,3}`. */
typedef struct candle_moe_weights {
    int32_t d_model;          /* hidden size d; multiple of the w1/w3 block size */
    int32_t d_ff;             /* expert inner size; multiple of the w2 block size */
    int32_t n_experts;        /* <= CANDLE_MOE_MAX_EXPERTS */
    int32_t top_k;            /* n_expert_used, <= CANDLE_MOE_MAX_TOPK */
    int32_t renorm;           /* 1: divide the selected weights by their sum (quantized_llama.rs:170-178);
                                 0: keep the softmax values (qwen2_moe.rs:281-282, norm_topk_prob = false) */
    int32_t dtype_w13;        /* GGML id of w1 and w3, each [d_ff, d_model] */
    int32_t dtype_w2;         /* GGML id of w2, [d_model, d_ff] */
    int32_t d_ff_shared;      /* 0 = no shared expert (qwen2_moe.rs:315-319 when > 0) */
    int32_t dtype_shared13;
    int32_t dtype_shared2;
    const float* router;          /* device f32 [n_experts, d_model] (feed_forward_gate_inp) */
    const float* router_bias;     /* device f32 [n_experts] added to the logits, or NULL */
    const void* const* w1;        /* host array of device pointers */
    const void* const* w3;
    const void* const* w2;
    const void* shared_w1;        /* device, [d_ff_shared, d_model] */
    const void* shared_w3;
    const void* shared_w2;        /* device, [d_model, d_ff_shared] */
    const float* shared_gate;     /* device f32 [d_model] (shared_expert_gate) */
    /* Optional decode-path copies made by candle_moe_prepack (host arrays of device pointers, or
     * NULL): when all three are given, batches of up to 128 rows read these instead of the GGUF
     * blocks.  The GGUF pointers above stay required (larger batches use them). */
    const void* const* w1_prepacked;
    const void* const* w3_prepacked;
    const void* const* w2_prepacked;
    /* The same for the shared expert (device pointers or NULL; Q8_0 only: large batches then take the tensor-core GEMM). */
    const void* shared_w1_prepacked;
    const void* shared_w3_prepacked;
    const void* shared_w2_prepacked;
} candle_moe_weights_t;

/* Kernel-selection switches, for A/B checks and for re-tuning the thresholds on other shapes.  Each value starts
 * from an environment variable read once when the library is first used (CANDLE_MOE_GEMM, CANDLE_MOE_GEMM_MIN_ROWS,
 * CANDLE_MOE_STREAM_MAX_ROWS, CANDLE_MOE_FORCE_ROWS, CANDLE_MOE_MID); later changes go through candle_moe_set_tuning
 * only, so a workspace size query and the forward that follows see the same values unless the caller changes them
 * in between.  The reference has the same kind of switch as a process-wide flag
 * (candle-core/src/quantized/cuda.rs:21-25, `FORCE_DMMV` / `set_force_dmmv`).  Results stay within the documented bounds under every
 * setting; only which kernel form runs changes. */
#define CANDLE_MOE_TUNE_GEMM_ENABLED 0     /* 0: large batches stay on the streaming form (default 1) */
#define CANDLE_MOE_TUNE_GEMM_MIN_ROWS 1    /* bound on the rows of an expert above which the tensor-core GEMM runs (96) */
#define CANDLE_MOE_TUNE_STREAM_MAX_ROWS 2  /* rows per expert up to which the streaming form is used (no limit) */
#define CANDLE_MOE_TUNE_FORCE_ROWS 3       /* 1: every grouped product through the row-per-warp form (0) */
#define CANDLE_MOE_TUNE_MID_ENABLED 4      /* 0: no four-position-tile decode kernels for 17..64 rows per expert (1) */
CANDLE_MOE_API int candle_moe_set_tuning(int32_t key, int64_t value);
CANDLE_MOE_API int candle_moe_get_tuning(int32_t key, int64_t* value);

/* Library identification: returns a static string "candle_moe_sm100 <version>". */
CANDLE_MOE_API const char* candle_moe_version(void);

/* Bytes of scratch that candle_moe_forward needs for up to max_tokens rows.  Replaces the
 * per-call allocations of the reference block (dev.alloc in candle-core/src/quantized/cuda.rs:253,
 * 321 and the zeros_like/index_add copies of quantized_llama.rs:184,202). */
CANDLE_MOE_API int candle_moe_workspace_bytes(const candle_moe_weights_t* w, int64_t max_tokens, size_t* out_bytes);

/* Router: logits = x . Wg^T (+ bias), softmax over all experts, stable descending top-k (ties keep
 * the lower expert id), optional renormalisation.  Replaces quantized_llama.rs:153-179
 * (QMatMul::forward on the f32 gate, candle_nn::ops::softmax_last_dim, the host-side sort).
 *   x [T, d] f32, router [E, d] f32, bias [E] f32 or NULL
 *   topk_ids [T, k] u32 in rank order, topk_w [T, k] f32 */
CANDLE_MOE_API int candle_moe_router_topk(void* stream, const float* x, const float* router, const float* bias, int64_t T,
                           int32_t d, int32_t E, int32_t k, int32_t renorm, uint32_t* topk_ids, float* topk_w);

/* Dispatch: groups the T*k (token, expert) pairs by expert, tokens ascending inside an expert,
 * which is the order of the reference's `top_x[e]` lists (quantized_llama.rs:162-173) that feed
 * index_select (:197).
 *   expert_counts [E], expert_offsets [E + 1] (exclusive prefix sum of counts),
 *   perm_token [T*k]: token id of the row at each grouped position,
 *   pair_pos   [T*k]: grouped position of pair (t, rank) at index t*k + rank. */
CANDLE_MOE_API int candle_moe_permute(void* stream, const uint32_t* topk_ids, int64_t T, int32_t k, int32_t E,
                       uint32_t* expert_counts, uint32_t* expert_offsets, uint32_t* perm_token,
                       uint32_t* pair_pos);

/* Activation quantization, the `T::VecDotType::from_float` step of k_quants::matmul
 * (candle-core/src/quantized/k_quants.rs:1898-1902): per row, per block.
 *   for_weight_dtype Q4K / Q6K -> BlockQ8K arithmetic (k_quants.rs:1819-1856): per 256 a signed-max
 *       scale, int8 values, 16 int16 block sums
 *   for_weight_dtype Q8_0      -> BlockQ8_0 arithmetic (k_quants.rs:605-634): per 32 an f16 scale
 * Outputs are planar: qs int8 [rows, kdim]; scales f32 [rows, kdim / block] (for Q8_0 the f16-rounded
 * scale widened to f32); bsums int16 [rows, kdim / 16] (Q8K only, may be NULL for Q8_0). */
CANDLE_MOE_API int candle_moe_quantize_act(void* stream, const float* x, int64_t rows, int32_t kdim, int32_t for_weight_dtype,
                            int8_t* qs, float* scales, int16_t* bsums);

/* Weighted combine: y[t] = sum over the token's selected experts, in ascending expert id, of
 * topk_w * expert_out[pair_pos], each product rounded before it is added, starting from zero --
 * the order of broadcast_mul + index_add over the expert loop (quantized_llama.rs:185-203).
 * With a shared expert (shared_out != NULL): y[t] += shared_out[t] * sigmoid(x[t] . shared_gate)
 * afterwards (qwen2_moe.rs:315-319). */
CANDLE_MOE_API int candle_moe_combine(void* stream, const float* expert_out, const uint32_t* topk_ids, const float* topk_w,
                       const uint32_t* pair_pos, int64_t T, int32_t k, int32_t d, const float* shared_out,
                       const float* x, const float* shared_gate, float* y);

/* Grouped expert products over rows already grouped by expert (Mlp::forward,
 * quantized_llama.rs:124-131, applied to every expert's row list; QMatMul::forward ->
 * k_quants::matmul semantics, candle-core/src/quantized/mod.rs:533-556, k_quants.rs:1873-1920).
 *   gate_up: hidden[p, :] = silu(W1_e . xq[row(p)]) * (W3_e . xq[row(p)])   for p in expert e's range
 *   down   : out[p, :]    = W2_e . hq[p]
 * `row_of` maps a grouped position to the row of the quantized activations (NULL = identity).
 * Activations are the planar outputs of candle_moe_quantize_act.
 * `weights` are host arrays of E device pointers; `expert_offsets` is a device array [E + 1]. */
CANDLE_MOE_API int candle_moe_grouped_gate_up(void* stream, const void* const* w1, const void* const* w3, int32_t dtype,
                               int32_t E, int32_t d, int32_t ff, const uint32_t* expert_offsets,
                               const uint32_t* row_of, int64_t max_rows, const int8_t* xq, const float* xscales,
                               const int16_t* xbsums, float* hidden);
CANDLE_MOE_API int candle_moe_grouped_down(void* stream, const void* const* w2, int32_t dtype, int32_t E, int32_t d, int32_t ff,
                            const uint32_t* expert_offsets, int64_t max_rows, const int8_t* hq,
                            const float* hscales, const int16_t* hbsums, float* out);

/* The whole block on one GPU: MlpOrMoe::MoE::forward (quantized_llama.rs:143-210), plus the shared
 * expert of qwen2_moe.rs:261-323 when w->d_ff_shared > 0.
 *   x [T, d_model] f32 device, y [T, d_model] f32 device (overwritten), workspace device memory of at
 *   least candle_moe_workspace_bytes(w, T) bytes, 256-byte aligned.
 * No host synchronisation, no allocation: the reference's to_vec2 round trip (:158) and per-expert
 * uploads (:190-193) do not exist on this path. */
CANDLE_MOE_API int candle_moe_forward(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T, float* y,
                       void* workspace, size_t workspace_bytes);

/* The FFN half of a decoder layer around the block: y = x + MoE(RmsNorm(x)), i.e.
 * `layer.ffn_norm.forward` -> `layer.mlp_or_moe.forward` -> `x + residual`
 * (candle-transformers/src/models/quantized_llama.rs:887-891; RmsNorm arithmetic of
 * candle-nn/src/ops.rs:504-514: x / sqrt(mean(x^2) + eps) * norm_weight in f32).  The residual add
 * happens inside the combine kernel.  Workspace: candle_moe_ffn_layer_workspace_bytes(w, T) bytes
 * (the block's workspace plus the normalised rows). */
CANDLE_MOE_API int candle_moe_ffn_layer_workspace_bytes(const candle_moe_weights_t* w, int64_t T, size_t* out_bytes);
CANDLE_MOE_API int candle_moe_ffn_layer(void* stream, const candle_moe_weights_t* w, const float* norm_weight, float eps,
                                        const float* x, int64_t T, float* y, void* workspace, size_t workspace_bytes);

/* candle_moe_forward with CUDA events recorded on `stream` between its launches; synchronises the
 * stream and writes the device time of each stage in milliseconds to stage_ms[8]:
 * {router (+ fused quantization of x), dispatch, separate quantization of x, gate_up, quantization
 * of the hidden rows, down, shared expert, combine}.  For measurement only (it creates and destroys
 * events); plays the part of the tracing spans around `QMatMul::forward` in the reference
 * (candle-transformers/src/models/quantized_llama.rs:97-115). */
CANDLE_MOE_API int candle_moe_forward_timed(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T,
                                            float* y, void* workspace, size_t workspace_bytes, float* stage_ms);

/* The same block as candle_moe_forward for callers that may not allocate device memory at all.
 * (No counterpart in the reference: candle allocates its temporaries per call.)
 *
 * Who needs it: a host whose device memory is entirely owned by its own pool or arena and who
 * therefore has no buffer to hand over as `workspace` and no permission to call cudaMalloc next
 * to that pool; a decode loop with a latency budget, where an allocation could stall the device;
 * a plugin living inside a process that forbids foreign allocations.  Such a caller passes only
 * inputs and outputs; the scratch lives in a fixed array of CANDLE_MOE_STATIC_SCRATCH_BYTES that is
 * part of the library image, so every GPU that loads the library keeps that much memory until
 * the process exits.
 *
 * Rules:
 *   - a call whose scratch need (candle_moe_workspace_bytes(w, T)) exceeds
 *     CANDLE_MOE_STATIC_SCRATCH_BYTES is refused with CANDLE_MOE_E_STATIC_SCRATCH before anything is
 *     enqueued (the Mixtral-8x7B-shaped layer fits up to T = 40 rows);
 *   - the first call on each device looks the array's device address up (a host-side query, no
 *     allocation); make that first call with the device current and before starting any stream
 *     capture;
 *   - all calls on one GPU share the one array: two calls that can overlap on the GPU (different
 *     streams) race on it -- serialise them; the array keeps whatever the previous call left, and
 *     nothing in it needs clearing because every region is written before it is read in a call;
 *   - nothing is allocated or freed: no cudaMalloc, cudaFree or allocating library routine. */
CANDLE_MOE_API int candle_moe_forward_static(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T,
                                             float* y);

/* Views into the workspace of the last candle_moe_forward call with the same (w, T), for tests and
 * for expert-parallel callers: device pointers to topk_ids [T,k], topk_w [T,k], expert_counts [E],
 * perm_token [T*k].  Any output pointer may be NULL. */
CANDLE_MOE_API int candle_moe_workspace_views(const candle_moe_weights_t* w, int64_t T, void* workspace, uint32_t** topk_ids,
                               float** topk_w, uint32_t** expert_counts, uint32_t** perm_token);

/* Expert parallelism over ranks (one process per GPU): rank r owns a contiguous range of the experts and
 * every rank routes its own tokens.  The reference has no multi-device form of this block (it runs every
 * expert where the block lives, quantized_llama.rs:185-203); these calls are what an NCCL all-to-all of
 * permuted token rows needs either side of it, and they reproduce the single-device results bit for bit:
 * what travels is the quantized activation row that `VecDotType::from_float` (k_quants.rs:1898-1902) would
 * produce on the receiving side anyway.  K-quant experts only (Q4_K / Q6_K; activations Q8K).
 *
 * Sender:   candle_moe_router_topk, candle_moe_quantize_act, candle_moe_permute as on one device (the
 *           dispatch order, ascending global expert id, is also ascending destination rank), then
 *   candle_moe_ep_pack: send_rows[p] = packed row of grouped position p, candle_moe_ep_row_bytes(d) bytes:
 *           int8 values [d] | int16 block sums [d/16] | f32 block scales [d/256] | padding to 16 bytes.
 * Host:     exchange the per-expert counts, then the rows (all-to-all with those split sizes).
 * Receiver: candle_moe_ep_experts over the n_rows received rows, laid out source-major, each source's
 *           rows ordered by local expert id; recv_counts is the device array [n_src][n_local_experts] of
 *           row counts (w->n_experts is the LOCAL expert count here and w->w1/w3/w2 the local experts'
 *           matrices; router and top_k are ignored).  max_rows_per_expert is a host-side bound on the
 *           rows of any one local expert (n_rows is always valid; a tight bound picks better kernels).
 *           out_rows [n_rows, d] f32: the experts' outputs in the order the rows arrived, ready for the
 *           return all-to-all.  Workspace: candle_moe_ep_workspace_bytes(w, n_rows) bytes.
 * Sender:   candle_moe_combine over the returned rows (they are back in grouped order). */
CANDLE_MOE_API int candle_moe_ep_row_bytes(int32_t d_model, size_t* out_bytes);
CANDLE_MOE_API int candle_moe_ep_pack(void* stream, const uint32_t* perm_token, int64_t n_rows, int32_t d_model,
                                      const int8_t* xq, const float* xscales, const int16_t* xbsums, void* send_rows);
CANDLE_MOE_API int candle_moe_ep_workspace_bytes(const candle_moe_weights_t* w, int64_t max_rows_total, size_t* out_bytes);
CANDLE_MOE_API int candle_moe_ep_experts(void* stream, const candle_moe_weights_t* w, const void* recv_rows,
                                         const uint32_t* recv_counts, int32_t n_src, int64_t n_rows,
                                         int64_t max_rows_per_expert, float* out_rows, void* workspace,
                                         size_t workspace_bytes);

/* ---- Expert parallelism as ONE call per step, the collectives inside the library -------------------------------
 * The reference has no expert-parallel block; what it has is the plumbing of its multi-process example, which these
 * entry points follow: rank 0 makes an NCCL id and hands it to the others out of band, every rank builds its
 * communicator from (id, rank, world) (candle-examples/examples/llama_multiprocess/main.rs:148-173, `Id::new`,
 * `Comm::from_rank`), and the collective hides behind the op it belongs to (model.rs:30-90).
 *
 *   candle_moe_ep_unique_id      ncclGetUniqueId: CANDLE_MOE_EP_UNIQUE_ID_BYTES bytes to distribute to every rank
 *   candle_moe_ep_comm_init      ncclCommInitRank with the current device, plus a little pinned host memory
 *   candle_moe_ep_comm_from_nccl the same handle around a communicator the host already has (a cudarc `Comm`'s
 *                                ncclComm_t); the handle does not own it
 *   candle_moe_ep_comm_destroy   frees the handle (and the communicator if the handle made it)
 *
 * candle_moe_ep_forward: MlpOrMoe::MoE::forward (quantized_llama.rs:143-210) with the experts sharded: rank r owns
 * experts [r E/N, (r+1) E/N) (`local` describes them: n_experts = E/N, its router/top_k fields are ignored) and
 * routes its own T rows of x [T, d] into y [T, d] with the full router of `cfg`.  Inside: router + Q8K quantization +
 * dispatch, all-to-all of the packed quantized rows, the local experts, all-to-all of the f32 outputs back, combine;
 * both exchanges are grouped ncclSend / ncclRecv on `stream`.  Results are those of candle_moe_forward.
 * Every rank of the communicator must make the call in the same step with the same cfg (rank apart); T may differ
 * per rank (0 included) up to cfg->max_tokens.  Two forms, picked from cfg alone (candle_moe_ep_forward_form says
 * which): "slots" (form 1, small steps: fixed-capacity slots with the counts in-band, no host synchronisation and
 * no data-dependent size, so the call is a fixed sequence of launches) and "exact" (form 2, large steps: counts
 * exchanged and checked on the host first -- one stream synchronisation, plus one for the all-reduce that makes
 * every rank agree on the verdict -- then rows of exactly the needed sizes; a table that fails the check makes
 * EVERY rank return CANDLE_MOE_E_EP_MISMATCH before any row is exchanged or any expert kernel launched).
 * In the slot form a bad slot header is found on the device: that source's rows are dropped and bit 2 (value 4) of
 * candle_moe_device_status is raised.  One step at a time per communicator.  K-quant experts only. */
#define CANDLE_MOE_EP_UNIQUE_ID_BYTES 128
typedef struct candle_moe_ep_comm candle_moe_ep_comm_t;
typedef struct candle_moe_ep_config {
    int32_t rank, world;          /* must match the communicator */
    int32_t n_experts_global;     /* E, a multiple of world */
    int32_t top_k;                /* n_expert_used */
    int32_t renorm;               /* as candle_moe_weights_t.renorm */
    int32_t max_tokens;           /* bound on T of ANY rank in a step; the same on every rank (sizes the slots) */
    int32_t force_form;           /* 0: choose by size; 1: slots; 2: exact */
    int32_t inject_count_mismatch;/* tests only: 1 makes this rank announce bad metadata (exact form: a count table that fails
                                     the check; slot form: slot headers with a wrong check word) */
    int64_t max_recv_rows;        /* exact form: cap on the rows one rank may receive per step (0 = worst case,
                                     world * max_tokens * min(top_k, E / world)); sizes the workspace */
    const float* router;          /* device f32 [E, d_model], replicated on every rank */
    const float* router_bias;     /* device f32 [E] or NULL */
} candle_moe_ep_config_t;
CANDLE_MOE_API int candle_moe_ep_unique_id(void* id_out);
CANDLE_MOE_API int candle_moe_ep_comm_init(const void* unique_id, int32_t rank, int32_t world, candle_moe_ep_comm_t** comm_out);
CANDLE_MOE_API int candle_moe_ep_comm_from_nccl(void* nccl_comm, candle_moe_ep_comm_t** comm_out);
CANDLE_MOE_API int candle_moe_ep_comm_destroy(candle_moe_ep_comm_t* comm);
CANDLE_MOE_API const char* candle_moe_ep_last_error(void);  /* text of the calling thread's last CANDLE_MOE_E_NCCL / _EP_MISMATCH */
CANDLE_MOE_API int candle_moe_ep_forward_workspace_bytes(const candle_moe_ep_config_t* cfg, const candle_moe_weights_t* local,
                                                         size_t* out_bytes);
CANDLE_MOE_API int candle_moe_ep_forward_form(const candle_moe_ep_config_t* cfg, const candle_moe_weights_t* local, int32_t* form,
                                              int64_t* capacity_rows);
/* comm may be NULL when cfg->world == 1 (the exchanges are then device copies). */
CANDLE_MOE_API int candle_moe_ep_forward(void* stream, candle_moe_ep_comm_t* comm, const candle_moe_ep_config_t* cfg,
                                         const candle_moe_weights_t* local, const float* x, int64_t T, float* y,
                                         void* workspace, size_t workspace_bytes);
/* The same step with CUDA events between its phases (synchronises the stream): phase_ms[5] = {route + pack, exchange of
 * rows, local experts, exchange of results, combine}; rows_info[2] = {rows this rank received, rows of its busiest
 * expert}.  For measurement only. */
CANDLE_MOE_API int candle_moe_ep_forward_timed(void* stream, candle_moe_ep_comm_t* comm, const candle_moe_ep_config_t* cfg,
                                               const candle_moe_weights_t* local, const float* x, int64_t T, float* y,
                                               void* workspace, size_t workspace_bytes, float* phase_ms, int64_t* rows_info);

/* One quantized matrix over a batch of rows: out[rows, n] = x[rows, k] . W^T with W [n, k] in GGUF blocks
 * -- `QMatMul::forward` (candle-core/src/quantized/mod.rs:533-537 -> `QTensor::cuda_fwd` :520-530 -> `QCudaStorage::fwd`, cuda.rs:484-505)
 * for the dense projections of the model (attention wq/wk/wv/wo quantized_llama.rs:275-277,345, lm head :897).
 * The rows are quantized as `k_quants::matmul` does (k_quants.rs:1873-1920), then the product runs on the same
 * kernels as the experts' down product with one group: the tensor-core GEMM above 16 rows (Q6_K reads
 * `w_prepacked` there, the optional copy made by candle_moe_prepack) and the forms that read the GGUF layout
 * otherwise (with one group they are faster than the decode kernels over the repacked copy).  Workspace: candle_moe_qmatmul_workspace_bytes bytes, 256-byte aligned. */
CANDLE_MOE_API int candle_moe_qmatmul_workspace_bytes(int32_t dtype, int64_t rows, int32_t n, int32_t k, size_t* out_bytes);
CANDLE_MOE_API int candle_moe_qmatmul(void* stream, const void* w, const void* w_prepacked, int32_t dtype, int32_t n,
                                      int32_t k, const float* x, int64_t rows, float* out, void* workspace,
                                      size_t workspace_bytes);

/* The other pieces of a decode step's attention half, for the decode-step harness (none is part of the MoE block):
 *   candle_moe_rmsnorm: y = x / sqrt(mean(x^2) + eps) * weight per row, f32 (`candle_nn::ops::rms_norm`,
 *     candle-nn/src/ops.rs:504-514; `attention_norm` / final `norm`, quantized_llama.rs:880, 893); d a multiple of 4.
 *   candle_moe_rope_kv_append: the interleaved rotary embedding of the new token's q and k (`rope_i`,
 *     candle-nn/src/rotary_emb.rs:53-66, called from quantized_llama.rs:255-263) and the append of k and v to the
 *     f32 cache at index_pos (`KvCache::append`, candle-nn/src/kv_cache.rs:143-164, 204-226), in one pass.
 *     qkv [batch, row_stride] holds a row's q (n_head * head_dim), k and v (n_kv_head * head_dim each) side by side --
 *     the output of one product over the concatenated wq | wk | wv rows --, cos / sin [head_dim / 2] are the table rows
 *     of the position (quantized_llama.rs:410-427); q_out [batch, n_head, head_dim]; caches as below. */
CANDLE_MOE_API int candle_moe_rmsnorm(void* stream, const float* x, const float* weight, float eps, int64_t rows, int32_t d, float* y);
CANDLE_MOE_API int candle_moe_rope_kv_append(void* stream, const float* qkv, int64_t row_stride, const float* cos, const float* sin,
                                             int32_t batch, int32_t n_head, int32_t n_kv_head, int32_t head_dim, int64_t max_seq,
                                             int32_t index_pos, float* q_out, float* k_cache, float* v_cache);

/* Attention of ONE new token per sequence over an f32 KV cache: `standard_attention` of quantized_llama.rs:303-317 at
 * seq_len = 1 (q k^T / sqrt(head_dim), softmax_last_dim, times v) with `repeat_kv` folded into the indexing (query head
 * h reads kv head h / (n_head / n_kv_head)).  Outside the MoE block; it exists so that a whole decode step around the
 * block can be timed without the cache being read through generic batched matmuls.
 *   q [batch, n_head, head_dim] (after the rotary embedding), k_cache / v_cache [batch, n_kv_head, max_seq, head_dim]
 *   of which the first n_ctx positions are valid (the new token's k / v already appended), out [batch, n_head * head_dim].
 * head_dim 128 with 1, 4 or 8 query heads per kv head, or head_dim 64 with 1 or 4 (CANDLE_MOE_E_SHAPE otherwise).
 * The context is cut into chunks whose partial softmax sums are merged afterwards: f32 summation order differs from
 * a one-pass softmax, nothing else. */
CANDLE_MOE_API int candle_moe_decode_attention_workspace_bytes(int32_t batch, int32_t n_head, int32_t head_dim, int32_t n_ctx,
                                                               size_t* out_bytes);
CANDLE_MOE_API int candle_moe_decode_attention(void* stream, const float* q, const float* k_cache, const float* v_cache,
                                               int32_t batch, int32_t n_head, int32_t n_kv_head, int32_t head_dim, int64_t max_seq,
                                               int32_t n_ctx, float* out, void* workspace, size_t workspace_bytes);

/* One-time repack of a Q4_K / Q6_K matrix [n_rows, k] (n_rows a multiple of 8 -- 16 for w2 --, k a
 * multiple of 256) into the register-fragment order the decode kernels read with coalesced
 * 128-bit loads.  Q4_K grows by 2.8 % (its 12-byte packed 6-bit scales are widened to 16 bytes),
 * Q6_K keeps its size.  A Q8_0 matrix (k a multiple of 32) is repacked for the large-batch tensor-core GEMM instead:
 * per row and 256 elements a 16-byte aligned record of 256 int8 values and 8 f16 scales (the 34-byte GGUF blocks are
 * only 2-byte aligned), rows padded with zero records to a multiple of 256 elements (+6 %, more for short rows).
 * No counterpart in the reference, whose kernels read the GGUF layout
 * directly (candle-kernels/src/quantized.cu:2626-2698); optional here as well.
 *   candle_moe_prepacked_bytes: size of the destination buffer (0 bytes = shape or dtype not supported)
 *   candle_moe_prepack: src raw blocks -> dst, both device memory, 16-byte aligned */
CANDLE_MOE_API int candle_moe_prepacked_bytes(int32_t dtype, int64_t n_rows, int32_t k, size_t* out_bytes);
CANDLE_MOE_API int candle_moe_prepack(void* stream, int32_t dtype, const void* src_blocks, int64_t n_rows, int32_t k,
                                      void* dst);

/* The grouped expert products over prepacked weights (same contracts as candle_moe_grouped_gate_up /
 * candle_moe_grouped_down; at most 128 rows per expert; CANDLE_MOE_E_SHAPE when the shape is not taken). */
CANDLE_MOE_API int candle_moe_grouped_gate_up_prepacked(void* stream, const void* const* w1p, const void* const* w3p,
                                                        int32_t dtype, int32_t E, int32_t d, int32_t ff,
                                                        const uint32_t* expert_offsets, const uint32_t* row_of,
                                                        int64_t max_rows, const int8_t* xq, const float* xscales,
                                                        const int16_t* xbsums, float* hidden);
CANDLE_MOE_API int candle_moe_grouped_down_prepacked(void* stream, const void* const* w2p, int32_t dtype, int32_t E,
                                                     int32_t d, int32_t ff, const uint32_t* expert_offsets,
                                                     int64_t max_rows, const int8_t* hq, const float* hscales,
                                                     const int16_t* hbsums, float* out);

/* Health word of the device-side kernels.  Every wait inside a kernel (on a copy in flight) has an
 * iteration limit; a kernel whose wait expired raises a bit here and finishes without hanging: bit 0 (1) the
 * streaming kernels, bit 1 (2) the tensor-core GEMM; bit 2 (4) is raised by the expert-parallel slot form when a
 * received slot header fails its checks.  candle_moe_device_status synchronises the device and returns the
 * accumulated flags in *flags (0 = healthy); candle_moe_device_status_reset clears them.
 * candle_moe_selftest_bounded_wait enqueues a one-CTA kernel that waits, with the library's own wait primitive and
 * the given poll limit, on a barrier that nothing ever completes: the wait runs out, the kernel raises bit 0 and
 * returns -- the way to see the give-up path work without a stuck copy.
 * No counterpart in the reference (its kernels do not wait on asynchronous copies). */
CANDLE_MOE_API int candle_moe_device_status(int32_t* flags);
CANDLE_MOE_API int candle_moe_device_status_reset(void);
CANDLE_MOE_API int candle_moe_selftest_bounded_wait(void* stream, int32_t poll_limit);

/* Weight quantization on the device, bit-exact with QTensor::quantize -> GgmlType::from_float for
 * Q8_0 / Q4K / Q6K (k_quants.rs:605-634, 1287-1345, 1675-1744); replaces the CPU round trip of
 * QCudaStorage::quantize (candle-core/src/quantized/cuda.rs:457-478).
 *   src f32 [n_elems] device, dst raw blocks device; n_elems a multiple of the block size. */
CANDLE_MOE_API int candle_moe_quantize_weights(void* stream, int32_t dtype, const float* src, int64_t n_elems, void* dst);

/* Dequantize raw blocks to f32 (GgmlType::to_float; k_quants.rs:587-603, 1347-1374, 1747-1778). */
CANDLE_MOE_API int candle_moe_dequantize(void* stream, int32_t dtype, const void* blocks, int64_t n_elems, float* dst);

#ifdef __cplusplus
}
#endif
#endif /* CANDLE_MOE_H_ */
