// Host-side pieces shared by the translation units that implement the C ABI (candle_moe_api.cu, ep_nccl.cu).
#pragma once
#include "common.cuh"

namespace cmoe {

#define CM_TRY(expr)                        \
    do {                                    \
        const int _r = (expr);              \
        if (_r != CANDLE_MOE_OK) return _r; \
    } while (0)

inline int rc(cudaError_t e) { return e == cudaSuccess ? CANDLE_MOE_OK : (int)e; }

// next 256-byte aligned piece of a workspace (base null: size query, only `off` advances)
template <class T>
T* carve(uint8_t* base, size_t& off, size_t count) {
    off = align_up(off, 256);
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
}

int check_weights(const candle_moe_weights_t* w);
int fill_ptrs(const void* const* host, int E, ExpertPtrs& out);

constexpr int MAX_K_SPLITS = 8;  // partial outputs the down product may leave for the combine kernel

struct ExpertBufs {
    float* hidden;  // [P, ff]
    int8_t* hq;
    float* hs;
    int16_t* hb;
    float* eo;      // [slots][P, d]
    void* gemm;     // scratch of the large-batch GEMM (may be null)
};

// The routed experts over P rows grouped by expert (device offsets [E + 1]).  `max_rows` picks the kernels: a bound
// on the rows of one expert, or (rows_exact) the actual / expected largest count -- every kernel is correct for any
// count, the choice only matters for speed.  `row_limit` (device, may be null): actual number of rows when P is a
// capacity bound.  Leaves *eo_splits partial outputs in b.eo.
int run_experts(cudaStream_t st, const candle_moe_weights_t* w, const ExpertPtrs& p1, const ExpertPtrs& p3,
                const ExpertPtrs& p2, int64_t max_rows, int64_t P, const uint32_t* offsets, const uint32_t* row_of,
                const int8_t* xq, const float* xs, const int16_t* xb, const ExpertBufs& b, int slots, int* eo_splits,
                bool marks, bool rows_exact, const uint32_t* row_limit, int64_t total_rows_hint);

// Scratch of the expert-parallel local phase for up to P rows
struct EpWorkspace {
    uint32_t* plan;     // [2 * 1024]
    uint32_t* offsets;  // [E + 1]
    uint32_t* back;     // [P]
    int8_t* xq;
    float* xs;
    int16_t* xb;
    ExpertBufs eb;
    int64_t eo_rows;    // rows x slots the eo region holds
    size_t total;
};
EpWorkspace ep_layout(const candle_moe_weights_t* w, int64_t P, void* base);
// K-split partial outputs the local phase may use for P rows over E local experts: eight while the rows are few
// (decode-sized steps, where splitting K is what fills the SMs), four beyond
inline int ep_eo_slots(int64_t P, int E) { return (P <= 64 * (int64_t)E || P <= 2048) ? MAX_K_SPLITS : 4; }

}  // namespace cmoe
