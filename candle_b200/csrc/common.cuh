// Shared definitions for the sm_100a kernels of the quantized MoE feed-forward block.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/candle_moe.h"

namespace cmoe {

// GGUF block layouts (candle-core/src/quantized/k_quants.rs:81-87, 119-127, 141-149); raw bytes.
constexpr int QK_K = 256;
constexpr int QK8_0 = 32;
constexpr int Q4K_BYTES = 144;  // f16 d, f16 dmin, u8 scales[12], u8 qs[128]
constexpr int Q6K_BYTES = 210;  // u8 ql[128], u8 qh[64], i8 scales[16], f16 d
constexpr int Q8_0_BYTES = 34;  // f16 d, i8 qs[32]

__host__ __device__ inline int block_elems(int dtype) {
    return dtype == CANDLE_GGML_Q8_0 ? 32 : 256;
}
__host__ __device__ inline int block_bytes(int dtype) {
    return dtype == CANDLE_GGML_Q8_0 ? Q8_0_BYTES : (dtype == CANDLE_GGML_Q4K ? Q4K_BYTES : Q6K_BYTES);
}
inline bool dtype_supported(int dtype) {
    return dtype == CANDLE_GGML_Q8_0 || dtype == CANDLE_GGML_Q4K || dtype == CANDLE_GGML_Q6K;
}
// Activation block length used against a weight dtype (GgmlType::VecDotType): Q8K (256) for the
// k-quants, Q8_0 (32) for Q8_0.
__host__ __device__ inline int act_block(int dtype) { return dtype == CANDLE_GGML_Q8_0 ? 32 : 256; }

// Per-expert weight base pointers travel as a kernel parameter (no device-side table to allocate).
struct ExpertPtrs {
    const uint8_t* p[CANDLE_MOE_MAX_EXPERTS];
};

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

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 6-bit scale / min of sub-block j of a Q4_K block (candle-core/src/quantized/utils.rs:50-60)
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* q, int& sc, int& m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// BlockQ8K::from_float (candle-core/src/quantized/k_quants.rs:1819-1856) for one 256-element block
// by one warp, 8 consecutive elements per lane.  `max` is the signed value of the first element with
// the largest magnitude; IEEE division, roundf = round half away from zero like f32::round.
__device__ __forceinline__ void quantize_q8k_block(const float* __restrict__ xblk, int lane, int8_t* __restrict__ qs,
                                                   float* __restrict__ scale, int16_t* __restrict__ bsums) {
    const float4* src = reinterpret_cast<const float4*>(xblk) + lane * 2;
    const float4 a = src[0], b = src[1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float amax = 0.f, mx = 0.f;
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (amax < fabsf(v[i])) {
            amax = fabsf(v[i]);
            mx = v[i];
            idx = i;
        }
    }
    idx += lane * 8;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        if (oa > amax || (oa == amax && oi < idx)) {
            amax = oa;
            idx = oi;
            mx = om;
        }
    }
    int q[8];
    float d;
    if (amax == 0.f) {
        d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = 0;
    } else {
        const float iscale = __fdiv_rn(-128.0f, mx);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = (int)fminf(roundf(__fmul_rn(iscale, v[i])), 127.f);
        d = __fdiv_rn(1.0f, iscale);
    }
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += q[i];
    s += __shfl_xor_sync(0xffffffffu, s, 1);  // 16 elements = two lanes
    const uint32_t lo = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) |
                        ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t hi = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) |
                        ((uint32_t)(q[7] & 0xff) << 24);
    reinterpret_cast<uint2*>(qs)[lane] = make_uint2(lo, hi);
    if ((lane & 1) == 0) bsums[lane >> 1] = (int16_t)s;
    if (lane == 0) *scale = d;
}

// candle-core/src/op.rs:645-648 and candle-nn/src/ops.rs:59-61; IEEE division, libm-grade expf.
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (expf(-v) + 1.0f); }

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Programmatic dependent launch.  Every kernel of the block starts with pdl_trigger() (the next
// kernel in the stream may be made resident right away, hiding its launch latency) followed by
// pdl_wait() (nothing produced by earlier kernels is touched before they have completed and
// flushed).  Because every kernel waits before it exits, completion is transitive along the chain.
// Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool pdl_enabled();  // CANDLE_MOE_PDL=0 turns the launch attribute off

// Kernel-selection switches (candle_moe_set_tuning / candle_moe_get_tuning).  Each starts from its
// environment variable, read once when the library is first used; afterwards only the setter changes it.
enum TuningKey {
    TUNE_GEMM_ENABLED = CANDLE_MOE_TUNE_GEMM_ENABLED,
    TUNE_GEMM_MIN_ROWS = CANDLE_MOE_TUNE_GEMM_MIN_ROWS,
    TUNE_STREAM_MAX_ROWS = CANDLE_MOE_TUNE_STREAM_MAX_ROWS,
    TUNE_FORCE_ROWS = CANDLE_MOE_TUNE_FORCE_ROWS,
    TUNE_MID_ENABLED = CANDLE_MOE_TUNE_MID_ENABLED,
    TUNE_N_KEYS
};
int64_t tuning_get(int key);
bool tuning_set(int key, int64_t value);  // false: unknown key

template <typename... KArgs, typename... Args>
cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- launchers implemented in the other translation units (all enqueue on `st`) ----
// qs / scales / bsums non-null: also quantize every row of x the Q8K way (fused, one pass over x)
cudaError_t launch_router_topk(cudaStream_t st, const float* x, const float* router, const float* bias, int64_t T,
                               int d, int E, int k, int renorm, uint32_t* ids, float* w, int8_t* qs = nullptr,
                               float* scales = nullptr, int16_t* bsums = nullptr, uint32_t* counts = nullptr,
                               uint32_t* offsets = nullptr, uint32_t* perm_token = nullptr, uint32_t* pair_pos = nullptr);
// scratch (may be null): permute_scratch_words(T * k, E) words; with it, large batches are sorted by many CTAs
size_t permute_scratch_words(int64_t n_pairs, int E);
cudaError_t launch_permute(cudaStream_t st, const uint32_t* ids, int64_t T, int k, int E, uint32_t* counts,
                           uint32_t* offsets, uint32_t* perm_token, uint32_t* pair_pos, uint32_t* scratch = nullptr);
// offsets[0..2) = {0, rows}: one group holding every row (used for the always-on shared expert)
cudaError_t launch_single_group(cudaStream_t st, uint32_t* offsets, uint32_t rows);
// row_limit (Q8K only, may be null): device-side row count; rows at or beyond it are skipped
cudaError_t launch_quantize_act(cudaStream_t st, const float* x, int64_t rows, int kdim, int for_dtype, int8_t* qs,
                                float* scales, int16_t* bsums, const uint32_t* row_limit = nullptr,
                                uint32_t* single_group = nullptr);
cudaError_t launch_grouped_gate_up(cudaStream_t st, const ExpertPtrs& w1, const ExpertPtrs& w3, int dtype, int E,
                                   int d, int ff, const uint32_t* offsets, const uint32_t* row_of, int64_t max_rows,
                                   const int8_t* xq, const float* xs, const int16_t* xb, float* hidden);
// `max_rows` bounds the rows of any single expert.  `out` may receive up to `max_splits` partial
// results (K-splits) spaced `split_stride` floats apart; *n_splits says how many were written and
// the caller (the combine kernel) adds them in split order.
cudaError_t launch_grouped_down(cudaStream_t st, const ExpertPtrs& w2, int dtype, int E, int d, int ff,
                                const uint32_t* offsets, int64_t max_rows, const int8_t* hq, const float* hs,
                                const int16_t* hb, float* out, int64_t split_stride, int max_splits, int* n_splits);
cudaError_t launch_combine(cudaStream_t st, const float* expert_out, int n_splits, int64_t split_stride,
                           const uint32_t* ids, const float* w, const uint32_t* pair_pos, int64_t T, int k, int d,
                           const float* shared_out, int shared_splits, int64_t shared_split_stride, const float* x,
                           const float* shared_gate, float* y, const float* residual = nullptr);
cudaError_t launch_rmsnorm(cudaStream_t st, const float* x, const float* alpha, float eps, int64_t T, int d, float* y);
// streaming (TMA ring + tensor-core) form; cudaErrorNotSupported when the shape is not taken
cudaError_t launch_expert_stream(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype,
                                 int E, int K, int N, const uint32_t* offsets, const uint32_t* row_of,
                                 int64_t max_rows_per_expert, const int8_t* aq, const float* ascale,
                                 const int16_t* absum, float* out, int* n_splits_out, int64_t split_stride,
                                 int max_splits);
// prepacked-weight (register-fragment order) form for decode-sized batches
size_t prepacked_bytes(int dtype, int64_t n_rows, int k);
cudaError_t launch_prepack(cudaStream_t st, int dtype, const void* raw, int64_t n_rows, int k, void* dst);
cudaError_t launch_expert_direct(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype,
                                 int E, int K, int N, const uint32_t* offsets, const uint32_t* row_of,
                                 int64_t max_rows_per_expert, const int8_t* aq, const float* ascale,
                                 const int16_t* absum, float* out, int* n_splits_out, int64_t split_stride,
                                 int max_splits, int max_active_experts = 0, int64_t total_rows = 0);
// large-batch grouped GEMM on tcgen05 / TMEM: Q4_K in GGUF layout (repacked = false), Q6_K in the repacked
// layout (repacked = true); `scratch` of expert_gemm_scratch_bytes(P, K) bytes
size_t expert_gemm_scratch_bytes(int64_t P, int K, int parts = 1);  // parts = 2: the exact Q8_0 gate_up operand
// Q8_0 rows repacked for the GEMM: [n][ceil(k / 256)][256 int8 | 8 f16 scales]
size_t prepacked_q80_bytes(int64_t n_rows, int k);
cudaError_t launch_prepack_q80(cudaStream_t st, const void* raw, int64_t n_rows, int k, void* dst);
cudaError_t launch_expert_gemm(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype,
                               bool repacked, int E, int K, int N, const uint32_t* offsets, const uint32_t* row_of, int64_t P,
                               int64_t max_rows, const int8_t* aq, const float* ascale, const int16_t* absum, float* out,
                               void* scratch, int max_splits = 1, int* n_splits_out = nullptr, int64_t split_stride = 0);
// Q8_0 grouped products for many rows per expert (expert_q80.cu); cudaErrorNotSupported for other shapes
cudaError_t launch_expert_q80(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int E, int K, int N,
                              const uint32_t* offsets, const uint32_t* row_of, const int8_t* aq, const float* ascale, float* out);
// expert parallelism: packed quantized rows either side of the all-to-all (expert_parallel.cu)
size_t ep_row_bytes(int d);
cudaError_t launch_ep_pack(cudaStream_t st, const uint32_t* row_of, int64_t n_rows, int d, const int8_t* xq, const float* xs,
                           const int16_t* xb, void* send);
cudaError_t launch_ep_regroup(cudaStream_t st, const void* recv, const uint32_t* counts, int n_src, int E, int64_t n_rows, int d,
                              uint32_t* plan, int8_t* xq, float* xs, int16_t* xb, uint32_t* offsets, uint32_t* back_index);
// row_limit (device, may be null): rows at or beyond *row_limit are skipped (n_rows is then a capacity bound)
cudaError_t launch_ep_scatter(cudaStream_t st, const float* eo, int n_splits, int64_t split_stride, const uint32_t* back_index,
                              int64_t n_rows, int d, float* out, const uint32_t* row_limit = nullptr);
// flags raised by kernels whose bounded waits expired (0 = none); synchronises the device
cudaError_t read_stream_status(int* out);
cudaError_t stream_status_ptr(int** out);  // device address of that health word
cudaError_t reset_stream_status();
cudaError_t launch_selftest_wait(cudaStream_t st, int limit);
// attention of one new token per sequence over an f32 KV cache (decode_attention.cu); cudaErrorNotSupported for shapes not taken
size_t decode_attention_workspace_bytes(int B, int n_head, int head_dim, int n_ctx);
cudaError_t launch_decode_attention(cudaStream_t st, const float* q, const float* kc, const float* vc, int B, int n_head, int n_kv,
                                    int head_dim, int64_t max_seq, int n_ctx, float scale, float* y, float* workspace);
cudaError_t launch_rope_kv_append(cudaStream_t st, const float* qkv, int64_t row_stride, const float* cos, const float* sin, int B,
                                  int n_head, int n_kv, int D, int64_t max_seq, int pos, float* q_out, float* kc, float* vc);
cudaError_t launch_quantize_weights(cudaStream_t st, int dtype, const float* src, int64_t n, void* dst);
cudaError_t launch_dequantize(cudaStream_t st, int dtype, const void* blocks, int64_t n, float* dst);

}  // namespace cmoe
