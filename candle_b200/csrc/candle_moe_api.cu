// extern "C" entry points of libcandle_moe_sm100.so (declared in include/candle_moe.h): argument
// validation on the host, workspace carving, and the launch sequence of the whole block.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "api_internal.cuh"

using namespace cmoe;

namespace {

// Above this bound on the rows of one expert (default 96) the tensor-core GEMM takes the k-quant products (below,
// the decode kernels); the tuning key GEMM_MIN_ROWS changes it.
// A single-device forward only knows the bound T on the rows of an expert, and its experts usually hold about
// k T / E rows, i.e. a few of the decode kernels' 16-row groups.  Measured on the Mixtral-shaped layer (decode
// kernels / GEMM, microseconds per step): T = 64 308 / 419, 80 376 / 421, 96 425 / 423, 112 504 / 449, 128 507 / 450.
inline int64_t gemm_min_rows() { return tuning_get(TUNE_GEMM_MIN_ROWS); }
// When the caller knows the ACTUAL largest row count of an expert (or, in the slot form of expert parallelism, a
// bound five quarters of the expected one, so that the tile width leaves a margin), the GEMM takes over above 32 rows.
// Measured on one GPU with the experts of one rank of the Mixtral-shaped layer (decode kernels / GEMM, microseconds
// per step): one expert, 32 rows 92 / 98, 48 rows 122 / 98, 64 rows 134 / 103, 96 rows 190 / 129, 128 rows 229 / 129;
// two experts, 32 rows each 163 / 159, 40 rows 193 / 165, 64 rows 246 / 200; four experts, 32 rows 272 / 262, 40 rows
// 323 / 263.  (An earlier measurement of 248 us for two experts of ~33 rows had position tiles of 32, so that every
// expert with a row more than expected took a second, almost empty tile.)  A single-device forward only knows the
// bound T.
constexpr int64_t GEMM_MIN_ROWS_EXACT = 32;
constexpr int64_t QMM_GEMM_MIN_ROWS = 48;  // the dense product: one matrix, rows known exactly
// Decode-sized batches may split K finely (more parallel items, smaller resident activations);
// larger batches get four slots, enough for the streaming form's activation rows to fit.
inline int k_split_slots(int64_t T) { return T <= gemm_min_rows() ? MAX_K_SPLITS : 4; }

struct Workspace {
    // routing
    uint32_t* topk_ids;
    float* topk_w;
    uint32_t* counts;
    uint32_t* offsets;
    uint32_t* perm_token;
    uint32_t* pair_pos;
    uint32_t* perm_scratch;  // per-chunk tables of the many-CTA dispatch
    // quantized input rows (one per token; experts gather through perm_token)
    int8_t* xq;
    float* xs;
    int16_t* xb;
    // routed experts
    float* hidden;  // [T*k, ff]
    int8_t* hq;
    float* hs;
    int16_t* hb;
    float* eo;  // [T*k, d]
    // shared expert
    uint32_t* sh_offsets;  // [2] = {0, T}
    int8_t* sxq;
    float* sxs;
    int16_t* sxb;
    float* shidden;  // [T, ff_s]
    int8_t* shq;
    float* shs;
    int16_t* shb;
    float* so;  // [T, d]
    void* gemm;  // operand scratch of the large-batch tensor-core GEMM (null for decode-sized T)
    size_t total;
};

Workspace layout(const candle_moe_weights_t* w, int64_t T, void* base_) {
    uint8_t* base = static_cast<uint8_t*>(base_);
    Workspace ws{};
    size_t off = 0;
    const size_t Tk = (size_t)T * w->top_k, d = w->d_model, ff = w->d_ff, E = w->n_experts;
    ws.topk_ids = carve<uint32_t>(base, off, Tk);
    ws.topk_w = carve<float>(base, off, Tk);
    ws.counts = carve<uint32_t>(base, off, E);
    ws.offsets = carve<uint32_t>(base, off, E + 1);
    ws.perm_token = carve<uint32_t>(base, off, Tk);
    ws.pair_pos = carve<uint32_t>(base, off, Tk);
    ws.perm_scratch = carve<uint32_t>(base, off, permute_scratch_words((int64_t)Tk, (int)E));
    ws.xq = carve<int8_t>(base, off, (size_t)T * d);
    ws.xs = carve<float>(base, off, (size_t)T * d / act_block(w->dtype_w13));
    ws.xb = carve<int16_t>(base, off, (size_t)T * d / 16);
    ws.hidden = carve<float>(base, off, Tk * ff);
    ws.hq = carve<int8_t>(base, off, Tk * ff);
    ws.hs = carve<float>(base, off, Tk * ff / act_block(w->dtype_w2));
    ws.hb = carve<int16_t>(base, off, Tk * ff / 16);
    ws.eo = carve<float>(base, off, Tk * d * k_split_slots(T));
    if (w->d_ff_shared > 0) {
        const size_t fs = w->d_ff_shared;
        ws.sh_offsets = carve<uint32_t>(base, off, 2);
        if (act_block(w->dtype_shared13) != act_block(w->dtype_w13)) {
            ws.sxq = carve<int8_t>(base, off, (size_t)T * d);
            ws.sxs = carve<float>(base, off, (size_t)T * d / act_block(w->dtype_shared13));
            ws.sxb = carve<int16_t>(base, off, (size_t)T * d / 16);
        } else {
            ws.sxq = ws.xq;
            ws.sxs = ws.xs;
            ws.sxb = ws.xb;
        }
        ws.shidden = carve<float>(base, off, (size_t)T * fs);
        ws.shq = carve<int8_t>(base, off, (size_t)T * fs);
        ws.shs = carve<float>(base, off, (size_t)T * fs / act_block(w->dtype_shared2));
        ws.shb = carve<int16_t>(base, off, (size_t)T * fs / 16);
        ws.so = carve<float>(base, off, (size_t)T * d * k_split_slots(T));
    }
    if (T > gemm_min_rows()) {
        // large batches: fp16 activation operand of the tcgen05 GEMM (Q4_K matrices), reused by gate_up and down
        size_t g = 0;
        const auto takes = [](int dt, const void* packed) {
            return dt == CANDLE_GGML_Q4K || ((dt == CANDLE_GGML_Q6K || dt == CANDLE_GGML_Q8_0) && packed != nullptr);
        };
        if (takes(w->dtype_w13, w->w1_prepacked))
            g = std::max(g, expert_gemm_scratch_bytes((int64_t)Tk, (int)d, w->dtype_w13 == CANDLE_GGML_Q8_0 ? 2 : 1));
        if (takes(w->dtype_w2, w->w2_prepacked)) g = std::max(g, expert_gemm_scratch_bytes((int64_t)Tk, (int)ff));
        if (w->d_ff_shared > 0 && w->dtype_shared13 == CANDLE_GGML_Q8_0 && w->shared_w1_prepacked && w->shared_w3_prepacked &&
            w->shared_w2_prepacked)
            g = std::max(g, std::max(expert_gemm_scratch_bytes(T, (int)d, 2), expert_gemm_scratch_bytes(T, w->d_ff_shared)));
        if (g) {
            off = align_up(off, 1024);
            ws.gemm = base ? base + off : nullptr;
            if (!base) ws.gemm = reinterpret_cast<void*>(1);  // size query: only the extent matters
            off += g;
        }
    }
    ws.total = align_up(off, 256);
    return ws;
}

}  // namespace
int cmoe::check_weights(const candle_moe_weights_t* w) {
    if (!w) return CANDLE_MOE_E_NULL;
    if (w->d_model <= 0 || w->d_ff <= 0 || w->n_experts <= 0 || w->top_k <= 0) return CANDLE_MOE_E_SHAPE;
    if (w->n_experts > CANDLE_MOE_MAX_EXPERTS || w->top_k > CANDLE_MOE_MAX_TOPK || w->top_k > w->n_experts)
        return CANDLE_MOE_E_SHAPE;
    if (!dtype_supported(w->dtype_w13) || !dtype_supported(w->dtype_w2)) return CANDLE_MOE_E_DTYPE;
    if (w->d_model % block_elems(w->dtype_w13) || w->d_ff % block_elems(w->dtype_w2)) return CANDLE_MOE_E_SHAPE;
    if (w->d_model % 32 || w->d_ff % 32) return CANDLE_MOE_E_SHAPE;
    if (w->d_ff_shared < 0) return CANDLE_MOE_E_SHAPE;
    if (w->d_ff_shared > 0) {
        if (!dtype_supported(w->dtype_shared13) || !dtype_supported(w->dtype_shared2)) return CANDLE_MOE_E_DTYPE;
        if (w->d_model % block_elems(w->dtype_shared13) || w->d_ff_shared % block_elems(w->dtype_shared2) ||
            w->d_ff_shared % 32)
            return CANDLE_MOE_E_SHAPE;
    }
    return CANDLE_MOE_OK;
}

int cmoe::fill_ptrs(const void* const* host, int E, ExpertPtrs& out) {
    if (!host) return CANDLE_MOE_E_NULL;
    std::memset(&out, 0, sizeof(out));
    for (int e = 0; e < E; ++e) {
        if (!host[e]) return CANDLE_MOE_E_NULL;
        if (reinterpret_cast<uintptr_t>(host[e]) & 15) return CANDLE_MOE_E_ALIGN;
        out.p[e] = static_cast<const uint8_t*>(host[e]);
    }
    return CANDLE_MOE_OK;
}

namespace {
// tuning key GEMM_ENABLED = 0 keeps large batches on the streaming form (A/B checks)
inline bool gemm_enabled() { return tuning_get(TUNE_GEMM_ENABLED) != 0; }

// Optional per-stage event marks for candle_moe_forward_timed (null in normal calls).
constexpr int N_STAGES = 8;  // router, permute, quantize_x, gate_up, quantize_h, down, shared expert, combine
struct StageProbe {
    cudaEvent_t ev[N_STAGES + 1];
    bool hit[N_STAGES + 1];
};
thread_local StageProbe* g_probe = nullptr;
inline void mark(cudaStream_t st, int stage_done) {
    if (g_probe) {
        cudaEventRecord(g_probe->ev[stage_done + 1], st);
        g_probe->hit[stage_done + 1] = true;
    }
}

}  // namespace

extern "C" {

const char* candle_moe_version(void) { return "candle_moe_sm100 0.1"; }

int candle_moe_set_tuning(int32_t key, int64_t value) { return tuning_set(key, value) ? CANDLE_MOE_OK : CANDLE_MOE_E_SHAPE; }
int candle_moe_get_tuning(int32_t key, int64_t* value) {
    if (!value) return CANDLE_MOE_E_NULL;
    if (key < 0 || key >= TUNE_N_KEYS) return CANDLE_MOE_E_SHAPE;
    *value = tuning_get(key);
    return CANDLE_MOE_OK;
}

int candle_moe_workspace_bytes(const candle_moe_weights_t* w, int64_t max_tokens, size_t* out_bytes) {
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    CM_TRY(check_weights(w));
    if (max_tokens < 0 || max_tokens > (int64_t)1 << 24) return CANDLE_MOE_E_SHAPE;
    *out_bytes = layout(w, max_tokens, nullptr).total;
    return CANDLE_MOE_OK;
}

int candle_moe_router_topk(void* stream, const float* x, const float* router, const float* bias, int64_t T,
                           int32_t d, int32_t E, int32_t k, int32_t renorm, uint32_t* topk_ids, float* topk_w) {
    if (!x || !router || !topk_ids || !topk_w) return CANDLE_MOE_E_NULL;
    if (T < 0 || d <= 0 || d % 4 || E <= 0 || E > CANDLE_MOE_MAX_EXPERTS || k <= 0 || k > CANDLE_MOE_MAX_TOPK || k > E)
        return CANDLE_MOE_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(router)) & 15) return CANDLE_MOE_E_ALIGN;
    return rc(launch_router_topk((cudaStream_t)stream, x, router, bias, T, d, E, k, renorm, topk_ids, topk_w));
}

int candle_moe_permute(void* stream, const uint32_t* topk_ids, int64_t T, int32_t k, int32_t E,
                       uint32_t* expert_counts, uint32_t* expert_offsets, uint32_t* perm_token, uint32_t* pair_pos) {
    if (!topk_ids || !expert_counts || !expert_offsets || !perm_token || !pair_pos) return CANDLE_MOE_E_NULL;
    if (T < 0 || k <= 0 || k > CANDLE_MOE_MAX_TOPK || E <= 0 || E > CANDLE_MOE_MAX_EXPERTS) return CANDLE_MOE_E_SHAPE;
    return rc(launch_permute((cudaStream_t)stream, topk_ids, T, k, E, expert_counts, expert_offsets, perm_token,
                             pair_pos));
}

int candle_moe_quantize_act(void* stream, const float* x, int64_t rows, int32_t kdim, int32_t for_weight_dtype,
                            int8_t* qs, float* scales, int16_t* bsums) {
    if (!x || !qs || !scales) return CANDLE_MOE_E_NULL;
    if (!dtype_supported(for_weight_dtype)) return CANDLE_MOE_E_DTYPE;
    if (for_weight_dtype != CANDLE_GGML_Q8_0 && !bsums) return CANDLE_MOE_E_NULL;
    if (rows < 0 || kdim <= 0 || kdim % act_block(for_weight_dtype)) return CANDLE_MOE_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(qs) & 7)) return CANDLE_MOE_E_ALIGN;
    return rc(launch_quantize_act((cudaStream_t)stream, x, rows, kdim, for_weight_dtype, qs, scales, bsums));
}

int candle_moe_combine(void* stream, const float* expert_out, const uint32_t* topk_ids, const float* topk_w,
                       const uint32_t* pair_pos, int64_t T, int32_t k, int32_t d, const float* shared_out,
                       const float* x, const float* shared_gate, float* y) {
    if (!expert_out || !topk_ids || !topk_w || !pair_pos || !y) return CANDLE_MOE_E_NULL;
    if (shared_out && (!x || !shared_gate)) return CANDLE_MOE_E_NULL;
    if (T < 0 || k <= 0 || k > CANDLE_MOE_MAX_TOPK || d <= 0 || d % 4) return CANDLE_MOE_E_SHAPE;
    return rc(launch_combine((cudaStream_t)stream, expert_out, 1, 0, topk_ids, topk_w, pair_pos, T, k, d, shared_out, 1,
                             0, x, shared_gate, y));
}

int candle_moe_grouped_gate_up(void* stream, const void* const* w1, const void* const* w3, int32_t dtype,
                               int32_t E, int32_t d, int32_t ff, const uint32_t* expert_offsets,
                               const uint32_t* row_of, int64_t max_rows, const int8_t* xq, const float* xscales,
                               const int16_t* xbsums, float* hidden) {
    if (!expert_offsets || !xq || !xscales || !hidden) return CANDLE_MOE_E_NULL;
    if (!dtype_supported(dtype)) return CANDLE_MOE_E_DTYPE;
    if (dtype != CANDLE_GGML_Q8_0 && !xbsums) return CANDLE_MOE_E_NULL;
    if (E <= 0 || E > CANDLE_MOE_MAX_EXPERTS || d <= 0 || ff <= 0 || d % block_elems(dtype) || max_rows < 0)
        return CANDLE_MOE_E_SHAPE;
    ExpertPtrs p1, p3;
    CM_TRY(fill_ptrs(w1, E, p1));
    CM_TRY(fill_ptrs(w3, E, p3));
    return rc(launch_grouped_gate_up((cudaStream_t)stream, p1, p3, dtype, E, d, ff, expert_offsets, row_of, max_rows,
                                     xq, xscales, xbsums, hidden));
}

int candle_moe_grouped_down(void* stream, const void* const* w2, int32_t dtype, int32_t E, int32_t d, int32_t ff,
                            const uint32_t* expert_offsets, int64_t max_rows, const int8_t* hq, const float* hscales,
                            const int16_t* hbsums, float* out) {
    if (!expert_offsets || !hq || !hscales || !out) return CANDLE_MOE_E_NULL;
    if (!dtype_supported(dtype)) return CANDLE_MOE_E_DTYPE;
    if (dtype != CANDLE_GGML_Q8_0 && !hbsums) return CANDLE_MOE_E_NULL;
    if (E <= 0 || E > CANDLE_MOE_MAX_EXPERTS || d <= 0 || ff <= 0 || ff % block_elems(dtype) || max_rows < 0)
        return CANDLE_MOE_E_SHAPE;
    ExpertPtrs p2;
    CM_TRY(fill_ptrs(w2, E, p2));
    return rc(launch_grouped_down((cudaStream_t)stream, p2, dtype, E, d, ff, expert_offsets, max_rows, hq, hscales,
                                  hbsums, out, 0, 1, nullptr));
}

}  // extern "C"

namespace cmoe {
// The routed experts over P rows grouped by expert (device offsets [E + 1]); no expert has more than max_rows
// rows.  Picks, per product, the decode kernels over the repacked copies (max_rows <= 128), the tensor-core GEMM
// (more than that, scratch present), or the streaming / row forms.  Leaves *eo_splits partial outputs in b.eo.
int run_experts(cudaStream_t st, const candle_moe_weights_t* w, const ExpertPtrs& p1, const ExpertPtrs& p3,
                const ExpertPtrs& p2, int64_t max_rows, int64_t P, const uint32_t* offsets, const uint32_t* row_of,
                const int8_t* xq, const float* xs, const int16_t* xb, const ExpertBufs& b, int slots, int* eo_splits,
                bool marks, bool rows_exact, const uint32_t* row_limit, int64_t total_rows_hint) {
    if (total_rows_hint <= 0) total_rows_hint = P;
    const int E = w->n_experts, d = w->d_model, ff = w->d_ff;
    const bool large = b.gemm && max_rows > (rows_exact ? GEMM_MIN_ROWS_EXACT : gemm_min_rows()) && gemm_enabled();
    const bool use_prepacked = w->w1_prepacked && w->w3_prepacked && w->w2_prepacked && w->dtype_w13 != CANDLE_GGML_Q8_0 &&
                               w->dtype_w2 != CANDLE_GGML_Q8_0 && max_rows <= std::max<int64_t>(gemm_min_rows(), 64) && !large;
    bool gate_done = false, down_done = false;
    *eo_splits = 1;
    ExpertPtrs q1, q3, q2;
    if (use_prepacked) {
        CM_TRY(fill_ptrs(w->w1_prepacked, E, q1));
        CM_TRY(fill_ptrs(w->w3_prepacked, E, q3));
        CM_TRY(fill_ptrs(w->w2_prepacked, E, q2));
        const cudaError_t ce = launch_expert_direct(st, true, q1, q3, w->dtype_w13, E, d, ff, offsets, row_of, max_rows, xq,
                                                    xs, xb, b.hidden, nullptr, 0, 1, 0, total_rows_hint);
        if (ce == cudaSuccess)
            gate_done = true;
        else if (ce != cudaErrorNotSupported)
            return (int)ce;
    }
    // Position-tile width of the GEMM: from the actual largest row count when it is known, else from five quarters
    // of the average (an expert beyond the tile width simply takes a second tile)
    const int64_t tile_rows = rows_exact ? max_rows : std::min<int64_t>(max_rows, (5 * total_rows_hint + 4 * E - 1) / (4 * E));
    if (!gate_done && large) {
        // Q6_K and Q8_0 are read from the repacked copies (their GGUF blocks are only 2-byte aligned)
        const bool rp = (w->dtype_w13 == CANDLE_GGML_Q6K || w->dtype_w13 == CANDLE_GGML_Q8_0) && w->w1_prepacked && w->w3_prepacked;
        ExpertPtrs g1 = p1, g3 = p3;
        if (rp) {
            CM_TRY(fill_ptrs(w->w1_prepacked, E, g1));
            CM_TRY(fill_ptrs(w->w3_prepacked, E, g3));
        }
        const cudaError_t ce = launch_expert_gemm(st, true, g1, g3, w->dtype_w13, rp, E, d, ff, offsets, row_of, P, tile_rows, xq,
                                                  xs, xb, b.hidden, b.gemm);
        if (ce == cudaSuccess)
            gate_done = true;
        else if (ce != cudaErrorNotSupported)
            return (int)ce;
    }
    if (!gate_done)
        CM_TRY(rc(launch_grouped_gate_up(st, p1, p3, w->dtype_w13, E, d, ff, offsets, row_of, max_rows, xq, xs, xb,
                                         b.hidden)));
    if (marks) mark(st, 3);
    CM_TRY(rc(launch_quantize_act(st, b.hidden, P, ff, w->dtype_w2, b.hq, b.hs, b.hb, row_limit)));
    if (marks) mark(st, 4);
    if (use_prepacked) {
        const cudaError_t ce = launch_expert_direct(st, false, q2, q2, w->dtype_w2, E, ff, d, offsets, nullptr, max_rows, b.hq,
                                                    b.hs, b.hb, b.eo, eo_splits, P * d, slots, (int)(total_rows_hint < E ? total_rows_hint : E), total_rows_hint);
        if (ce == cudaSuccess)
            down_done = true;
        else if (ce != cudaErrorNotSupported)
            return (int)ce;
        else
            *eo_splits = 1;
    }
    if (!down_done && large) {
        const bool rp = (w->dtype_w2 == CANDLE_GGML_Q6K || w->dtype_w2 == CANDLE_GGML_Q8_0) && w->w2_prepacked;
        ExpertPtrs g2 = p2;
        if (rp) CM_TRY(fill_ptrs(w->w2_prepacked, E, g2));
        const cudaError_t ce = launch_expert_gemm(st, false, g2, g2, w->dtype_w2, rp, E, ff, d, offsets, nullptr, P, tile_rows,
                                                  b.hq, b.hs, b.hb, b.eo, b.gemm, slots, eo_splits, P * d);
        if (ce == cudaSuccess) {
            down_done = true;
        } else if (ce != cudaErrorNotSupported) {
            return (int)ce;
        }
    }
    if (!down_done)
        CM_TRY(rc(launch_grouped_down(st, p2, w->dtype_w2, E, d, ff, offsets, max_rows, b.hq, b.hs, b.hb, b.eo, P * d, slots,
                                      eo_splits)));
    return CANDLE_MOE_OK;
}

EpWorkspace ep_layout(const candle_moe_weights_t* w, int64_t P, void* base_) {
    uint8_t* base = static_cast<uint8_t*>(base_);
    EpWorkspace ws{};
    size_t off = 0;
    const size_t d = w->d_model, ff = w->d_ff, E = w->n_experts;
    ws.plan = carve<uint32_t>(base, off, 2048);
    ws.offsets = carve<uint32_t>(base, off, E + 1);
    ws.back = carve<uint32_t>(base, off, (size_t)P);
    ws.xq = carve<int8_t>(base, off, (size_t)P * d);
    ws.xs = carve<float>(base, off, (size_t)P * d / 256);
    ws.xb = carve<int16_t>(base, off, (size_t)P * d / 16);
    ws.eb.hidden = carve<float>(base, off, (size_t)P * ff);
    ws.eb.hq = carve<int8_t>(base, off, (size_t)P * ff);
    ws.eb.hs = carve<float>(base, off, (size_t)P * ff / 256);
    ws.eb.hb = carve<int16_t>(base, off, (size_t)P * ff / 16);
    ws.eo_rows = P * ep_eo_slots(P, (int)E);
    ws.eb.eo = carve<float>(base, off, (size_t)ws.eo_rows * d);
    if (P > GEMM_MIN_ROWS_EXACT) {
        const size_t g = std::max(expert_gemm_scratch_bytes(P, (int)d), expert_gemm_scratch_bytes(P, (int)ff));
        off = align_up(off, 1024);
        ws.eb.gemm = base ? base + off : reinterpret_cast<void*>(1);
        off += g;
    }
    ws.total = align_up(off, 256);
    return ws;
}
}  // namespace cmoe

extern "C" {

static int forward_impl(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T, float* y, void* workspace,
                        size_t workspace_bytes, const float* residual) {
    CM_TRY(check_weights(w));
    if (!x || !y || !w->router) return CANDLE_MOE_E_NULL;
    if (T < 0 || T > (int64_t)1 << 24) return CANDLE_MOE_E_SHAPE;
    if (T == 0) return CANDLE_MOE_OK;
    if (!workspace) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(w->router) & 15))
        return CANDLE_MOE_E_ALIGN;
    const Workspace ws = layout(w, T, workspace);
    if (workspace_bytes < ws.total) return CANDLE_MOE_E_WORKSPACE;
    const int E = w->n_experts, k = w->top_k, d = w->d_model;
    ExpertPtrs p1, p3, p2;
    CM_TRY(fill_ptrs(w->w1, E, p1));
    CM_TRY(fill_ptrs(w->w3, E, p3));
    CM_TRY(fill_ptrs(w->w2, E, p2));
    if (w->d_ff_shared > 0) {
        if (!w->shared_w1 || !w->shared_w3 || !w->shared_w2 || !w->shared_gate) return CANDLE_MOE_E_NULL;
        if (reinterpret_cast<uintptr_t>(w->shared_gate) & 15) return CANDLE_MOE_E_ALIGN;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t Tk = T * k;

    // k-quant experts: the router kernel also quantizes x (Q8K); Q8_0 experts keep the separate pass
    const bool fuse_q = w->dtype_w13 != CANDLE_GGML_Q8_0;
    if (g_probe) {
        cudaEventRecord(g_probe->ev[0], st);
        g_probe->hit[0] = true;
    }
    CM_TRY(rc(launch_router_topk(st, x, w->router, w->router_bias, T, d, E, k, w->renorm, ws.topk_ids, ws.topk_w,
                                 fuse_q ? ws.xq : nullptr, fuse_q ? ws.xs : nullptr, fuse_q ? ws.xb : nullptr,
                                 T == 1 ? ws.counts : nullptr, ws.offsets, ws.perm_token, ws.pair_pos)));
    mark(st, 0);
    // one token: the router kernel has written the dispatch itself
    if (T > 1) CM_TRY(rc(launch_permute(st, ws.topk_ids, T, k, E, ws.counts, ws.offsets, ws.perm_token, ws.pair_pos, ws.perm_scratch)));
    mark(st, 1);
    if (!fuse_q) CM_TRY(rc(launch_quantize_act(st, x, T, d, w->dtype_w13, ws.xq, ws.xs, ws.xb)));
    mark(st, 2);
    // a token selects an expert at most once: no expert sees more than T rows
    int eo_splits = 1, so_splits = 1;
    const ExpertBufs eb{ws.hidden, ws.hq, ws.hs, ws.hb, ws.eo, ws.gemm};
    CM_TRY(run_experts(st, w, p1, p3, p2, T, Tk, ws.offsets, ws.perm_token, ws.xq, ws.xs, ws.xb, eb, k_split_slots(T),
                       &eo_splits, true, false, nullptr, 0));
    mark(st, 5);

    const float* shared_out = nullptr;
    if (w->d_ff_shared > 0) {
        const int fs = w->d_ff_shared;
        CM_TRY(rc(launch_single_group(st, ws.sh_offsets, (uint32_t)T)));
        ExpertPtrs s1{}, s3{}, s2{};
        s1.p[0] = static_cast<const uint8_t*>(w->shared_w1);
        s3.p[0] = static_cast<const uint8_t*>(w->shared_w3);
        s2.p[0] = static_cast<const uint8_t*>(w->shared_w2);
        if (ws.sxq != ws.xq)
            CM_TRY(rc(launch_quantize_act(st, x, T, d, w->dtype_shared13, ws.sxq, ws.sxs, ws.sxb)));
        // large batches over repacked Q8_0 copies: the tensor-core GEMM with one group holding every row
        const bool sh_gemm = ws.gemm && T > gemm_min_rows() && gemm_enabled() && w->dtype_shared13 == CANDLE_GGML_Q8_0 &&
                             w->dtype_shared2 == CANDLE_GGML_Q8_0 && w->shared_w1_prepacked && w->shared_w3_prepacked &&
                             w->shared_w2_prepacked;
        bool sh_done = false;
        if (sh_gemm) {
            ExpertPtrs r1{}, r3{};
            r1.p[0] = static_cast<const uint8_t*>(w->shared_w1_prepacked);
            r3.p[0] = static_cast<const uint8_t*>(w->shared_w3_prepacked);
            const cudaError_t ce = launch_expert_gemm(st, true, r1, r3, CANDLE_GGML_Q8_0, true, 1, d, fs, ws.sh_offsets, nullptr, T, T,
                                                      ws.sxq, ws.sxs, ws.sxb, ws.shidden, ws.gemm);
            if (ce == cudaSuccess)
                sh_done = true;
            else if (ce != cudaErrorNotSupported)
                return (int)ce;
        }
        if (!sh_done)
            CM_TRY(rc(launch_grouped_gate_up(st, s1, s3, w->dtype_shared13, 1, d, fs, ws.sh_offsets, nullptr, T, ws.sxq,
                                             ws.sxs, ws.sxb, ws.shidden)));
        CM_TRY(rc(launch_quantize_act(st, ws.shidden, T, fs, w->dtype_shared2, ws.shq, ws.shs, ws.shb)));
        sh_done = false;
        if (sh_gemm) {
            ExpertPtrs r2{};
            r2.p[0] = static_cast<const uint8_t*>(w->shared_w2_prepacked);
            const cudaError_t ce = launch_expert_gemm(st, false, r2, r2, CANDLE_GGML_Q8_0, true, 1, fs, d, ws.sh_offsets, nullptr, T, T,
                                                      ws.shq, ws.shs, ws.shb, ws.so, ws.gemm, k_split_slots(T), &so_splits,
                                                      T * (int64_t)d);
            if (ce == cudaSuccess)
                sh_done = true;
            else if (ce != cudaErrorNotSupported)
                return (int)ce;
            else
                so_splits = 1;
        }
        if (!sh_done)
            CM_TRY(rc(launch_grouped_down(st, s2, w->dtype_shared2, 1, d, fs, ws.sh_offsets, T, ws.shq, ws.shs, ws.shb,
                                          ws.so, T * (int64_t)d, k_split_slots(T), &so_splits)));
        shared_out = ws.so;
    }
    mark(st, 6);
    CM_TRY(rc(launch_combine(st, ws.eo, eo_splits, Tk * d, ws.topk_ids, ws.topk_w, ws.pair_pos, T, k, d, shared_out,
                             so_splits, T * (int64_t)d, x, w->shared_gate, y, residual)));
    mark(st, 7);
    return CANDLE_MOE_OK;
}

int candle_moe_forward(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T, float* y,
                       void* workspace, size_t workspace_bytes) {
    return forward_impl(stream, w, x, T, y, workspace, workspace_bytes, nullptr);
}

int candle_moe_ffn_layer_workspace_bytes(const candle_moe_weights_t* w, int64_t T, size_t* out_bytes) {
    CM_TRY(check_weights(w));
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    if (T < 0 || T > (int64_t)1 << 24) return CANDLE_MOE_E_SHAPE;
    *out_bytes = layout(w, T, nullptr).total + align_up((size_t)T * w->d_model * sizeof(float), 256);
    return CANDLE_MOE_OK;
}

int candle_moe_ffn_layer(void* stream, const candle_moe_weights_t* w, const float* norm_weight, float eps, const float* x,
                         int64_t T, float* y, void* workspace, size_t workspace_bytes) {
    CM_TRY(check_weights(w));
    if (!x || !y || !norm_weight) return CANDLE_MOE_E_NULL;
    if (T < 0 || T > (int64_t)1 << 24) return CANDLE_MOE_E_SHAPE;
    if (T == 0) return CANDLE_MOE_OK;
    if (!workspace) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(norm_weight) & 15))
        return CANDLE_MOE_E_ALIGN;
    const size_t inner = layout(w, T, nullptr).total;
    const size_t need = inner + align_up((size_t)T * w->d_model * sizeof(float), 256);
    if (workspace_bytes < need) return CANDLE_MOE_E_WORKSPACE;
    float* xn = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + inner);
    CM_TRY(rc(launch_rmsnorm((cudaStream_t)stream, x, norm_weight, eps, T, w->d_model, xn)));
    return forward_impl(stream, w, xn, T, y, workspace, inner, x);
}

int candle_moe_forward_timed(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T, float* y,
                             void* workspace, size_t workspace_bytes, float* stage_ms) {
    if (!stage_ms) return CANDLE_MOE_E_NULL;
    StageProbe probe{};
    for (int i = 0; i <= N_STAGES; ++i) {
        const cudaError_t e = cudaEventCreate(&probe.ev[i]);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaEventDestroy(probe.ev[j]);
            return (int)e;
        }
    }
    g_probe = &probe;
    const int st = candle_moe_forward(stream, w, x, T, y, workspace, workspace_bytes);
    g_probe = nullptr;
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    for (int i = 0; i < N_STAGES; ++i) {
        stage_ms[i] = 0.f;
        if (st == CANDLE_MOE_OK && e == cudaSuccess && probe.hit[i] && probe.hit[i + 1])
            cudaEventElapsedTime(&stage_ms[i], probe.ev[i], probe.ev[i + 1]);
    }
    for (int i = 0; i <= N_STAGES; ++i) cudaEventDestroy(probe.ev[i]);
    return st != CANDLE_MOE_OK ? st : rc(e);
}

// ---- allocation-free variant -------------------------------------------------------------------
// Scratch for candle_moe_forward_static.  In host code `g_static_scratch` is only a handle for the
// symbol, not an address a kernel could use: the device address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the launches get.
static __device__ __align__(256) unsigned char g_static_scratch[CANDLE_MOE_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

// Device address of the built-in scratch on the current device; 0 on success.
int static_scratch_ptr(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return CANDLE_MOE_E_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255)) return CANDLE_MOE_E_ALIGN;
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return CANDLE_MOE_OK;
}
}  // namespace

int candle_moe_forward_static(void* stream, const candle_moe_weights_t* w, const float* x, int64_t T, float* y) {
    size_t need = 0;
    CM_TRY(candle_moe_workspace_bytes(w, T, &need));
    if (need > (size_t)CANDLE_MOE_STATIC_SCRATCH_BYTES) return CANDLE_MOE_E_STATIC_SCRATCH;
    void* scratch = nullptr;
    CM_TRY(static_scratch_ptr(&scratch));
    return candle_moe_forward(stream, w, x, T, y, scratch, (size_t)CANDLE_MOE_STATIC_SCRATCH_BYTES);
}

int candle_moe_workspace_views(const candle_moe_weights_t* w, int64_t T, void* workspace, uint32_t** topk_ids,
                               float** topk_w, uint32_t** expert_counts, uint32_t** perm_token) {
    CM_TRY(check_weights(w));
    if (!workspace) return CANDLE_MOE_E_NULL;
    const Workspace ws = layout(w, T, workspace);
    if (topk_ids) *topk_ids = ws.topk_ids;
    if (topk_w) *topk_w = ws.topk_w;
    if (expert_counts) *expert_counts = ws.counts;
    if (perm_token) *perm_token = ws.perm_token;
    return CANDLE_MOE_OK;
}

int candle_moe_prepacked_bytes(int32_t dtype, int64_t n_rows, int32_t k, size_t* out_bytes) {
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    if (dtype == CANDLE_GGML_Q8_0) {
        if (n_rows < 0 || k <= 0 || k % 32) return CANDLE_MOE_E_SHAPE;
        *out_bytes = prepacked_q80_bytes(n_rows, k);
        return CANDLE_MOE_OK;
    }
    if (dtype != CANDLE_GGML_Q4K && dtype != CANDLE_GGML_Q6K) return CANDLE_MOE_E_DTYPE;
    if (n_rows < 0 || k <= 0) return CANDLE_MOE_E_SHAPE;
    *out_bytes = prepacked_bytes(dtype, n_rows, k);
    return *out_bytes || n_rows == 0 ? CANDLE_MOE_OK : CANDLE_MOE_E_SHAPE;
}

int candle_moe_prepack(void* stream, int32_t dtype, const void* src_blocks, int64_t n_rows, int32_t k, void* dst) {
    if (!src_blocks || !dst) return CANDLE_MOE_E_NULL;
    if (dtype == CANDLE_GGML_Q8_0) {
        if (n_rows < 0 || k <= 0 || k % 32) return CANDLE_MOE_E_SHAPE;
        if ((reinterpret_cast<uintptr_t>(src_blocks) & 1) || (reinterpret_cast<uintptr_t>(dst) & 15)) return CANDLE_MOE_E_ALIGN;
        return rc(launch_prepack_q80((cudaStream_t)stream, src_blocks, n_rows, k, dst));
    }
    if (dtype != CANDLE_GGML_Q4K && dtype != CANDLE_GGML_Q6K) return CANDLE_MOE_E_DTYPE;
    if (n_rows < 0 || k <= 0 || k % 256 || n_rows % 8) return CANDLE_MOE_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(src_blocks) | reinterpret_cast<uintptr_t>(dst)) & 15) return CANDLE_MOE_E_ALIGN;
    if (dtype == CANDLE_GGML_Q6K && (k / 256) % 2) return CANDLE_MOE_E_SHAPE;  // rows must stay 4-byte aligned
    return rc(launch_prepack((cudaStream_t)stream, dtype, src_blocks, n_rows, k, dst));
}

int candle_moe_grouped_gate_up_prepacked(void* stream, const void* const* w1p, const void* const* w3p, int32_t dtype,
                                         int32_t E, int32_t d, int32_t ff, const uint32_t* expert_offsets,
                                         const uint32_t* row_of, int64_t max_rows, const int8_t* xq,
                                         const float* xscales, const int16_t* xbsums, float* hidden) {
    if (!expert_offsets || !xq || !xscales || !xbsums || !hidden) return CANDLE_MOE_E_NULL;
    if (dtype != CANDLE_GGML_Q4K && dtype != CANDLE_GGML_Q6K) return CANDLE_MOE_E_DTYPE;
    if (E <= 0 || E > CANDLE_MOE_MAX_EXPERTS || d <= 0 || ff <= 0 || d % 256 || max_rows < 0 || max_rows > 128)
        return CANDLE_MOE_E_SHAPE;
    ExpertPtrs p1, p3;
    CM_TRY(fill_ptrs(w1p, E, p1));
    CM_TRY(fill_ptrs(w3p, E, p3));
    const cudaError_t e = launch_expert_direct((cudaStream_t)stream, true, p1, p3, dtype, E, d, ff, expert_offsets, row_of,
                                               max_rows, xq, xscales, xbsums, hidden, nullptr, 0, 1);
    return e == cudaErrorNotSupported ? CANDLE_MOE_E_SHAPE : rc(e);
}

int candle_moe_grouped_down_prepacked(void* stream, const void* const* w2p, int32_t dtype, int32_t E, int32_t d,
                                      int32_t ff, const uint32_t* expert_offsets, int64_t max_rows, const int8_t* hq,
                                      const float* hscales, const int16_t* hbsums, float* out) {
    if (!expert_offsets || !hq || !hscales || !hbsums || !out) return CANDLE_MOE_E_NULL;
    if (dtype != CANDLE_GGML_Q4K && dtype != CANDLE_GGML_Q6K) return CANDLE_MOE_E_DTYPE;
    if (E <= 0 || E > CANDLE_MOE_MAX_EXPERTS || d <= 0 || ff <= 0 || ff % 256 || max_rows < 0 || max_rows > 128)
        return CANDLE_MOE_E_SHAPE;
    ExpertPtrs p2;
    CM_TRY(fill_ptrs(w2p, E, p2));
    const cudaError_t e = launch_expert_direct((cudaStream_t)stream, false, p2, p2, dtype, E, ff, d, expert_offsets,
                                               nullptr, max_rows, hq, hscales, hbsums, out, nullptr, 0, 1);
    return e == cudaErrorNotSupported ? CANDLE_MOE_E_SHAPE : rc(e);
}

int candle_moe_device_status(int32_t* flags) {
    if (!flags) return CANDLE_MOE_E_NULL;
    int v = 0;
    const cudaError_t e = read_stream_status(&v);
    *flags = v;
    return rc(e);
}

int candle_moe_device_status_reset(void) {
    const cudaError_t e = cudaDeviceSynchronize();
    return e != cudaSuccess ? (int)e : rc(reset_stream_status());
}

int candle_moe_selftest_bounded_wait(void* stream, int32_t poll_limit) {
    if (poll_limit < 1 || poll_limit > (1 << 20)) return CANDLE_MOE_E_SHAPE;
    return rc(launch_selftest_wait((cudaStream_t)stream, poll_limit));
}

int candle_moe_rmsnorm(void* stream, const float* x, const float* weight, float eps, int64_t rows, int32_t d, float* y) {
    if (rows < 0 || d <= 0 || d % 4) return CANDLE_MOE_E_SHAPE;
    if (rows == 0) return CANDLE_MOE_OK;
    if (!x || !weight || !y) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y)) & 15) return CANDLE_MOE_E_ALIGN;
    return rc(launch_rmsnorm((cudaStream_t)stream, x, weight, eps, rows, d, y));
}

int candle_moe_rope_kv_append(void* stream, const float* qkv, int64_t row_stride, const float* cos, const float* sin, int32_t batch,
                              int32_t n_head, int32_t n_kv_head, int32_t head_dim, int64_t max_seq, int32_t index_pos, float* q_out,
                              float* k_cache, float* v_cache) {
    if (batch < 0 || n_head <= 0 || n_kv_head <= 0 || head_dim <= 0 || head_dim % 2 || index_pos < 0 || index_pos >= max_seq ||
        row_stride < (int64_t)(n_head + 2 * n_kv_head) * head_dim)
        return CANDLE_MOE_E_SHAPE;
    if (batch == 0) return CANDLE_MOE_OK;
    if (!qkv || !cos || !sin || !q_out || !k_cache || !v_cache) return CANDLE_MOE_E_NULL;
    return rc(launch_rope_kv_append((cudaStream_t)stream, qkv, row_stride, cos, sin, batch, n_head, n_kv_head, head_dim, max_seq,
                                    index_pos, q_out, k_cache, v_cache));
}

int candle_moe_decode_attention_workspace_bytes(int32_t batch, int32_t n_head, int32_t head_dim, int32_t n_ctx, size_t* out_bytes) {
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    if (batch < 0 || n_head <= 0 || head_dim <= 0 || n_ctx < 0) return CANDLE_MOE_E_SHAPE;
    *out_bytes = decode_attention_workspace_bytes(batch, n_head, head_dim, n_ctx);
    return CANDLE_MOE_OK;
}

int candle_moe_decode_attention(void* stream, const float* q, const float* k_cache, const float* v_cache, int32_t batch,
                                int32_t n_head, int32_t n_kv_head, int32_t head_dim, int64_t max_seq, int32_t n_ctx, float* out,
                                void* workspace, size_t workspace_bytes) {
    if (batch < 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head || head_dim <= 0 || n_ctx < 0 || n_ctx > max_seq)
        return CANDLE_MOE_E_SHAPE;
    if (batch == 0 || n_ctx == 0) return CANDLE_MOE_OK;
    if (!q || !k_cache || !v_cache || !out || !workspace) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(workspace)) & 15)
        return CANDLE_MOE_E_ALIGN;
    if (workspace_bytes < decode_attention_workspace_bytes(batch, n_head, head_dim, n_ctx)) return CANDLE_MOE_E_WORKSPACE;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const cudaError_t e = launch_decode_attention((cudaStream_t)stream, q, k_cache, v_cache, batch, n_head, n_kv_head, head_dim,
                                                  max_seq, n_ctx, scale, out, static_cast<float*>(workspace));
    return e == cudaErrorNotSupported ? CANDLE_MOE_E_SHAPE : rc(e);
}

int candle_moe_quantize_weights(void* stream, int32_t dtype, const float* src, int64_t n_elems, void* dst) {
    if (!src || !dst) return CANDLE_MOE_E_NULL;
    if (!dtype_supported(dtype)) return CANDLE_MOE_E_DTYPE;
    if (n_elems < 0 || n_elems % block_elems(dtype)) return CANDLE_MOE_E_SHAPE;
    if (reinterpret_cast<uintptr_t>(src) & 15) return CANDLE_MOE_E_ALIGN;
    return rc(launch_quantize_weights((cudaStream_t)stream, dtype, src, n_elems, dst));
}

int candle_moe_dequantize(void* stream, int32_t dtype, const void* blocks, int64_t n_elems, float* dst) {
    if (!blocks || !dst) return CANDLE_MOE_E_NULL;
    if (!dtype_supported(dtype)) return CANDLE_MOE_E_DTYPE;
    if (n_elems < 0 || n_elems % block_elems(dtype)) return CANDLE_MOE_E_SHAPE;
    return rc(launch_dequantize((cudaStream_t)stream, dtype, blocks, n_elems, dst));
}

// ---------------------------------------------------------------------------------------------------------
// Expert parallelism (experts sharded over ranks; the host issues the all-to-alls between these calls)
// ---------------------------------------------------------------------------------------------------------
int candle_moe_ep_row_bytes(int32_t d_model, size_t* out_bytes) {
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    if (d_model <= 0 || d_model % 256) return CANDLE_MOE_E_SHAPE;
    *out_bytes = ep_row_bytes(d_model);
    return CANDLE_MOE_OK;
}

int candle_moe_ep_pack(void* stream, const uint32_t* perm_token, int64_t n_rows, int32_t d_model, const int8_t* xq,
                       const float* xscales, const int16_t* xbsums, void* send_rows) {
    if (n_rows < 0 || d_model <= 0 || d_model % 256) return CANDLE_MOE_E_SHAPE;
    if (n_rows == 0) return CANDLE_MOE_OK;
    if (!xq || !xscales || !xbsums || !send_rows) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(send_rows) & 15)) return CANDLE_MOE_E_ALIGN;
    return rc(launch_ep_pack((cudaStream_t)stream, perm_token, n_rows, d_model, xq, xscales, xbsums, send_rows));
}

int candle_moe_ep_workspace_bytes(const candle_moe_weights_t* w, int64_t max_rows_total, size_t* out_bytes) {
    CM_TRY(check_weights(w));
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    if (max_rows_total < 0 || max_rows_total > (int64_t)1 << 26) return CANDLE_MOE_E_SHAPE;
    if (w->dtype_w13 == CANDLE_GGML_Q8_0 || w->dtype_w2 == CANDLE_GGML_Q8_0) return CANDLE_MOE_E_DTYPE;
    *out_bytes = ep_layout(w, max_rows_total, nullptr).total;
    return CANDLE_MOE_OK;
}

int candle_moe_ep_experts(void* stream, const candle_moe_weights_t* w, const void* recv_rows, const uint32_t* recv_counts,
                          int32_t n_src, int64_t n_rows, int64_t max_rows_per_expert, float* out_rows, void* workspace,
                          size_t workspace_bytes) {
    CM_TRY(check_weights(w));
    if (w->dtype_w13 == CANDLE_GGML_Q8_0 || w->dtype_w2 == CANDLE_GGML_Q8_0) return CANDLE_MOE_E_DTYPE;
    if (n_rows < 0 || n_src <= 0 || (int64_t)n_src * w->n_experts > 1024 || max_rows_per_expert < 0 ||
        max_rows_per_expert > n_rows)
        return CANDLE_MOE_E_SHAPE;
    if (n_rows == 0) return CANDLE_MOE_OK;
    if (!recv_rows || !recv_counts || !out_rows || !workspace) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(recv_rows) & 15) ||
        (reinterpret_cast<uintptr_t>(out_rows) & 15))
        return CANDLE_MOE_E_ALIGN;
    const EpWorkspace ws = ep_layout(w, n_rows, workspace);
    if (workspace_bytes < ws.total) return CANDLE_MOE_E_WORKSPACE;
    const int E = w->n_experts, d = w->d_model;
    ExpertPtrs p1, p3, p2;
    CM_TRY(fill_ptrs(w->w1, E, p1));
    CM_TRY(fill_ptrs(w->w3, E, p3));
    CM_TRY(fill_ptrs(w->w2, E, p2));
    cudaStream_t st = (cudaStream_t)stream;
    CM_TRY(rc(launch_ep_regroup(st, recv_rows, recv_counts, n_src, E, n_rows, d, ws.plan, ws.xq, ws.xs, ws.xb, ws.offsets,
                                ws.back)));
    int eo_splits = 1;
    const int slots = ep_eo_slots(n_rows, E);
    CM_TRY(run_experts(st, w, p1, p3, p2, max_rows_per_expert, n_rows, ws.offsets, nullptr, ws.xq, ws.xs, ws.xb, ws.eb, slots,
                       &eo_splits, false, true, nullptr, 0));
    return rc(launch_ep_scatter(st, ws.eb.eo, eo_splits, n_rows * d, ws.back, n_rows, d, out_rows));
}

// ---------------------------------------------------------------------------------------------------------
// One quantized matrix over a batch of rows: QMatMul::forward for the dense projections of the model
// ---------------------------------------------------------------------------------------------------------
namespace {
struct QmmWorkspace {
    int8_t* xq;
    float* xs;
    int16_t* xb;
    uint32_t* offsets;
    float* eo;    // K-split partial outputs (null: the product writes `out` itself)
    int slots;
    void* gemm;
    size_t total;
};
// One group holds every row, so the row count is exact.  The tensor-core GEMM takes the product above 48 rows, and
// from 17 rows on when the matrix has enough 128-row tiles to fill the SMs by itself (measured at 32 rows:
// [32000, 4096] Q6_K 76 us through the GEMM against 108 us through the streaming form, [4096, 4096] Q4_K 25 against 23).
inline bool qmm_takes_gemm(int dtype, int64_t rows, int n) {
    return dtype != CANDLE_GGML_Q8_0 && (rows > QMM_GEMM_MIN_ROWS || (rows > 16 && n >= 12800));
}
QmmWorkspace qmm_layout(int dtype, int64_t rows, int n, int k, void* base_) {
    uint8_t* base = static_cast<uint8_t*>(base_);
    QmmWorkspace ws{};
    size_t off = 0;
    ws.xq = carve<int8_t>(base, off, (size_t)rows * k);
    ws.xs = carve<float>(base, off, (size_t)rows * k / act_block(dtype));
    ws.xb = carve<int16_t>(base, off, (size_t)rows * k / 16);
    ws.offsets = carve<uint32_t>(base, off, 2);
    // decode-sized batches split K to fill the device (a [4096, 4096] matrix has 256 row tiles for 148 SMs x 16 warps)
    ws.slots = rows <= 64 && n % 4 == 0 ? MAX_K_SPLITS : 1;
    if (ws.slots > 1) ws.eo = carve<float>(base, off, (size_t)rows * n * ws.slots);
    if (qmm_takes_gemm(dtype, rows, n)) {
        off = align_up(off, 1024);
        ws.gemm = base ? base + off : reinterpret_cast<void*>(1);
        off += expert_gemm_scratch_bytes(rows, k);
    }
    ws.total = align_up(off, 256);
    return ws;
}
}  // namespace

int candle_moe_qmatmul_workspace_bytes(int32_t dtype, int64_t rows, int32_t n, int32_t k, size_t* out_bytes) {
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    if (!dtype_supported(dtype)) return CANDLE_MOE_E_DTYPE;
    if (rows < 0 || rows > (int64_t)1 << 24 || n <= 0 || k <= 0 || k % block_elems(dtype)) return CANDLE_MOE_E_SHAPE;
    *out_bytes = qmm_layout(dtype, rows, n, k, nullptr).total;
    return CANDLE_MOE_OK;
}

int candle_moe_qmatmul(void* stream, const void* w, const void* w_prepacked, int32_t dtype, int32_t n, int32_t k,
                       const float* x, int64_t rows, float* out, void* workspace, size_t workspace_bytes) {
    if (!dtype_supported(dtype)) return CANDLE_MOE_E_DTYPE;
    if (rows < 0 || rows > (int64_t)1 << 24 || n <= 0 || k <= 0 || k % block_elems(dtype)) return CANDLE_MOE_E_SHAPE;
    if (rows == 0) return CANDLE_MOE_OK;
    if (!w || !x || !out || !workspace) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15))
        return CANDLE_MOE_E_ALIGN;
    const QmmWorkspace ws = qmm_layout(dtype, rows, n, k, workspace);
    if (workspace_bytes < ws.total) return CANDLE_MOE_E_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    ExpertPtrs pw{}, pp{};
    pw.p[0] = static_cast<const uint8_t*>(w);
    pp.p[0] = static_cast<const uint8_t*>(w_prepacked);
    // the quantizer also writes the offsets of the one group that holds every row
    CM_TRY(rc(launch_quantize_act(st, x, rows, k, dtype, ws.xq, ws.xs, ws.xb, nullptr, ws.offsets)));
    float* dst = ws.eo ? ws.eo : out;
    const int64_t stride = rows * (int64_t)n;
    int splits = 1;
    bool done = false;
    const bool large = ws.gemm && gemm_enabled();
    // The decode kernels over the repacked copy are not used here: with a single group their tiles are too few and
    // too short, and the streaming form over the GGUF blocks is faster (measured, [4096, 4096] Q4_K / [32000, 4096]
    // Q6_K: 1 row 10.8 / 44.5 us against 17.2 / 46.2; 8 rows 13.5 / 48.6 against 17.7 / 60.1).
    if (!done && large) {
        const bool rp = dtype == CANDLE_GGML_Q6K && w_prepacked;
        const cudaError_t ce = launch_expert_gemm(st, false, rp ? pp : pw, rp ? pp : pw, dtype, rp, 1, k, n, ws.offsets, nullptr,
                                                  rows, rows, ws.xq, ws.xs, ws.xb, dst, ws.gemm, ws.slots, &splits, stride);
        if (ce == cudaSuccess)
            done = true;
        else if (ce != cudaErrorNotSupported)
            return (int)ce;
        else
            splits = 1;
    }
    if (!done)
        CM_TRY(rc(launch_grouped_down(st, pw, dtype, 1, n, k, ws.offsets, rows, ws.xq, ws.xs, ws.xb, dst, stride, ws.slots,
                                      &splits)));
    if (ws.eo) return rc(launch_ep_scatter(st, ws.eo, splits, stride, nullptr, rows, n, out));
    return CANDLE_MOE_OK;
}

}  // extern "C"
