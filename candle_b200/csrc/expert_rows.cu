// Grouped expert products, row-per-warp form.
//
// out[p, n] = W_e[n, :] . act[row(p), :] for every grouped position p of expert e, where the weight
// row is raw GGUF blocks (Q4_K / Q6_K / Q8_0) and the activation row is the int8 quantization made
// by quantize_act.cu.  The integer block dots are exact (dp4a / integer multiply-adds); each block's
// integer result is scaled by (weight scale * activation scale) and accumulated in f32, as
// vec_dot does (candle-core/src/quantized/k_quants.rs:1205-1285, 1616-1673, 650-668 and the AVX2
// forms in avx.rs).  Only the order of the f32 additions differs from the reference.
//
// This form handles every shape the block formats allow (any k that is a block multiple, any row
// count, unaligned Q6_K / Q8_0 rows) and is the path used for shapes the tiled kernels do not
// take.  One warp owns one weight row (for gate_up: the same row of W1 and of W3) and walks the
// expert's activation rows TOK at a time, so a weight row is fetched from HBM once per expert.
#include "common.cuh"

namespace cmoe {

// Rows per expert up to which the streaming form is used.  Beyond 16 rows per expert it walks the
// expert's rows in groups of 16 and re-streams the weights for each group (mostly from L2), which
// is still far faster than the row-per-warp form; the tuning key STREAM_MAX_ROWS lowers the limit and
// FORCE_ROWS sends everything to the row-per-warp form (A/B checks in the tests).
static int64_t stream_max_rows() { return tuning_get(TUNE_STREAM_MAX_ROWS); }
static bool force_rows() { return tuning_get(TUNE_FORCE_ROWS) != 0; }

constexpr int ROWS_WARPS = 8;  // weight rows per CTA
constexpr int TOK = 4;         // activation rows per pass

struct ActView {
    const int8_t* qs;      // [rows, K]
    const float* scales;   // [rows, K / B]
    const int16_t* bsums;  // [rows, K / 16] (Q8K)
};

__device__ __forceinline__ uint32_t ld_u32_2b(const uint8_t* p) {  // 2-byte aligned 32-bit load
    const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}

// ---- Q4_K: lane owns bytes qs[4*lane .. 4*lane+4) of every block: low nibbles are 4 elements of
// sub-block 2g, high nibbles 4 elements of sub-block 2g+1, g = lane / 8.
struct Q4KRow {
    static constexpr int BYTES = Q4K_BYTES;
    static constexpr int ELEMS = 256;
    template <int NT>
    __device__ static __forceinline__ void block(const uint8_t* wb, int b, int K, const ActView& a,
                                                 const int64_t (&rows)[NT], int nt, int lane, float (&acc)[NT]) {
        const uint32_t hdr = *reinterpret_cast<const uint32_t*>(wb);
        const float d = half_bits_to_float((uint16_t)(hdr & 0xffff));
        const float dmin = half_bits_to_float((uint16_t)(hdr >> 16));
        const uint32_t s0 = *reinterpret_cast<const uint32_t*>(wb + 4);
        const uint32_t s1 = *reinterpret_cast<const uint32_t*>(wb + 8);
        const uint32_t s2 = *reinterpret_cast<const uint32_t*>(wb + 12);
        uint8_t sc8[12];
        *reinterpret_cast<uint32_t*>(sc8) = s0;
        *reinterpret_cast<uint32_t*>(sc8 + 4) = s1;
        *reinterpret_cast<uint32_t*>(sc8 + 8) = s2;
        const int g = lane >> 3;
        int sc_lo, m_lo, sc_hi, m_hi;
        q4k_scale_min(2 * g, sc8, sc_lo, m_lo);
        q4k_scale_min(2 * g + 1, sc8, sc_hi, m_hi);
        const uint32_t q = *reinterpret_cast<const uint32_t*>(wb + 16 + 4 * lane);
        const int w_lo = (int)(q & 0x0F0F0F0Fu), w_hi = (int)((q >> 4) & 0x0F0F0F0Fu);
        const int kb = K / 256;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (t < nt) {
                const int8_t* aq = a.qs + rows[t] * K + b * 256 + 64 * g + 4 * (lane & 7);
                const int a_lo = *reinterpret_cast<const int*>(aq);
                const int a_hi = *reinterpret_cast<const int*>(aq + 32);
                const int isum = sc_lo * __dp4a(w_lo, a_lo, 0) + sc_hi * __dp4a(w_hi, a_hi, 0);
                const float d8 = a.scales[rows[t] * kb + b];
                float r = (d8 * d) * (float)isum;
                if ((lane & 7) == 0) {
                    const int16_t* bs = a.bsums + (rows[t] * kb + b) * 16 + 4 * g;
                    const int msum = m_lo * ((int)bs[0] + (int)bs[1]) + m_hi * ((int)bs[2] + (int)bs[3]);
                    r = fmaf(-d8 * dmin, (float)msum, r);
                }
                acc[t] += r;
            }
        }
    }
};

// ---- Q6_K: lane owns positions l = lane of both 128-element halves: per half four elements
// (l, l+32, l+64, l+96) built from ql[l], ql[l+32], qh[l].
struct Q6KRow {
    static constexpr int BYTES = Q6K_BYTES;
    static constexpr int ELEMS = 256;
    template <int NT>
    __device__ static __forceinline__ void block(const uint8_t* wb, int b, int K, const ActView& a,
                                                 const int64_t (&rows)[NT], int nt, int lane, float (&acc)[NT]) {
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(wb + 208));
        const int8_t* sc = reinterpret_cast<const int8_t*>(wb + 192);
        int q[2][4], s[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int la = wb[64 * h + lane], lb = wb[64 * h + 32 + lane], hb = wb[128 + 32 * h + lane];
            q[h][0] = ((la & 0xF) | ((hb & 3) << 4)) - 32;
            q[h][1] = ((lb & 0xF) | (((hb >> 2) & 3) << 4)) - 32;
            q[h][2] = ((la >> 4) | (((hb >> 4) & 3) << 4)) - 32;
            q[h][3] = ((lb >> 4) | (((hb >> 6) & 3) << 4)) - 32;
            const int is = 8 * h + (lane >> 4);
#pragma unroll
            for (int c = 0; c < 4; ++c) s[h][c] = sc[is + 2 * c];
        }
        const int kb = K / 256;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (t < nt) {
                const int8_t* aq = a.qs + rows[t] * K + b * 256 + lane;
                int isum = 0;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 4; ++c) isum += s[h][c] * q[h][c] * (int)aq[128 * h + 32 * c];
                const float d8 = a.scales[rows[t] * kb + b];
                acc[t] = fmaf(d8 * d, (float)isum, acc[t]);
            }
        }
    }
};

// ---- Q8_0: lane owns whole 32-element blocks lane, lane+32, ... of the row.  `b` here counts
// groups of 32 blocks.
struct Q80Row {
    static constexpr int BYTES = Q8_0_BYTES * 32;
    static constexpr int ELEMS = 32 * 32;
    template <int NT>
    __device__ static __forceinline__ void block(const uint8_t* wb, int b, int K, const ActView& a,
                                                 const int64_t (&rows)[NT], int nt, int lane, float (&acc)[NT]) {
        const int kb = K / 32;
        const int blk = b * 32 + lane;
        if (blk >= kb) return;
        const uint8_t* w = wb + lane * Q8_0_BYTES;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(w));
        int wq[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) wq[i] = (int)ld_u32_2b(w + 2 + 4 * i);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (t < nt) {
                const int* aq = reinterpret_cast<const int*>(a.qs + rows[t] * K + blk * 32);
                int isum = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) isum = __dp4a(wq[i], aq[i], isum);
                const float da = a.scales[rows[t] * kb + blk];
                acc[t] = fmaf(d * da, (float)isum, acc[t]);
            }
        }
    }
};

template <class Fmt, bool GATE_UP>
__global__ void __launch_bounds__(ROWS_WARPS * 32)
grouped_rows_kernel(ExpertPtrs wa, ExpertPtrs wb, int K, int N, const uint32_t* __restrict__ offsets,
                    const uint32_t* __restrict__ row_of, ActView act, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.y;
    const uint32_t p0 = offsets[e], p1 = offsets[e + 1];
    if (p0 == p1) return;
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * ROWS_WARPS + (threadIdx.x >> 5);
    if (n >= N) return;
    const int n_steps = (K + Fmt::ELEMS - 1) / Fmt::ELEMS;
    const size_t row_bytes = (size_t)(K / (Fmt::ELEMS == 256 ? 256 : 32)) * (Fmt::ELEMS == 256 ? Fmt::BYTES : Q8_0_BYTES);
    const uint8_t* ra = wa.p[e] + (size_t)n * row_bytes;
    const uint8_t* rb = GATE_UP ? wb.p[e] + (size_t)n * row_bytes : nullptr;

    for (uint32_t p = p0; p < p1; p += TOK) {
        const int nt = min((uint32_t)TOK, p1 - p);
        int64_t rows[TOK];
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            const uint32_t pp = p + (t < nt ? t : 0);
            rows[t] = row_of ? (int64_t)row_of[pp] : (int64_t)pp;
        }
        float acc_a[TOK], acc_b[TOK];
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc_a[t] = acc_b[t] = 0.f;
        for (int b = 0; b < n_steps; ++b) {
            Fmt::template block<TOK>(ra + (size_t)b * Fmt::BYTES, b, K, act, rows, nt, lane, acc_a);
            if (GATE_UP) Fmt::template block<TOK>(rb + (size_t)b * Fmt::BYTES, b, K, act, rows, nt, lane, acc_b);
        }
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            const float va = warp_sum(acc_a[t]);
            const float vb = GATE_UP ? warp_sum(acc_b[t]) : 0.f;
            if (lane == 0 && t < nt) out[(int64_t)(p + t) * N + n] = GATE_UP ? silu_f(va) * vb : va;
        }
    }
}

template <bool GATE_UP>
static cudaError_t launch_rows(cudaStream_t st, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype, int E, int K,
                               int N, const uint32_t* offsets, const uint32_t* row_of, const ActView& act, float* out) {
    if (E == 0 || N == 0) return cudaSuccess;
    dim3 grid((N + ROWS_WARPS - 1) / ROWS_WARPS, E);
    dim3 block(ROWS_WARPS * 32);
    switch (dtype) {
        case CANDLE_GGML_Q4K:
            return launch_k(grouped_rows_kernel<Q4KRow, GATE_UP>, grid, block, 0, st, wa, wb, K, N, offsets, row_of, act, out);
        case CANDLE_GGML_Q6K:
            return launch_k(grouped_rows_kernel<Q6KRow, GATE_UP>, grid, block, 0, st, wa, wb, K, N, offsets, row_of, act, out);
        case CANDLE_GGML_Q8_0:
            return launch_k(grouped_rows_kernel<Q80Row, GATE_UP>, grid, block, 0, st, wa, wb, K, N, offsets, row_of, act, out);
        default:
            return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// Q8_0: above this bound on the rows of one expert the tensor-core tile kernel takes over from the row-per-warp form
constexpr int64_t Q80_TILE_MIN_ROWS = 16;

cudaError_t launch_grouped_gate_up(cudaStream_t st, const ExpertPtrs& w1, const ExpertPtrs& w3, int dtype, int E,
                                   int d, int ff, const uint32_t* offsets, const uint32_t* row_of, int64_t max_rows,
                                   const int8_t* xq, const float* xs, const int16_t* xb, float* hidden) {
    if (!force_rows() && max_rows <= stream_max_rows()) {
        const cudaError_t e = launch_expert_stream(st, true, w1, w3, dtype, E, d, ff, offsets, row_of, max_rows, xq, xs,
                                                   xb, hidden, nullptr, 0, 1);
        if (e != cudaErrorNotSupported) return e;
    }
    if (!force_rows() && dtype == CANDLE_GGML_Q8_0 && max_rows > Q80_TILE_MIN_ROWS) {
        const cudaError_t e = launch_expert_q80(st, true, w1, w3, E, d, ff, offsets, row_of, xq, xs, hidden);
        if (e != cudaErrorNotSupported) return e;
    }
    ActView a{xq, xs, xb};
    return launch_rows<true>(st, w1, w3, dtype, E, d, ff, offsets, row_of, a, hidden);
}

cudaError_t launch_grouped_down(cudaStream_t st, const ExpertPtrs& w2, int dtype, int E, int d, int ff,
                                const uint32_t* offsets, int64_t max_rows, const int8_t* hq, const float* hs,
                                const int16_t* hb, float* out, int64_t split_stride, int max_splits, int* n_splits) {
    if (n_splits) *n_splits = 1;
    if (!force_rows() && max_rows <= stream_max_rows()) {
        const cudaError_t e = launch_expert_stream(st, false, w2, w2, dtype, E, ff, d, offsets, nullptr, max_rows, hq, hs,
                                                   hb, out, n_splits, split_stride, max_splits);
        if (e != cudaErrorNotSupported) return e;
        if (n_splits) *n_splits = 1;
    }
    if (!force_rows() && dtype == CANDLE_GGML_Q8_0 && max_rows > Q80_TILE_MIN_ROWS) {
        const cudaError_t e = launch_expert_q80(st, false, w2, w2, E, ff, d, offsets, nullptr, hq, hs, out);
        if (e != cudaErrorNotSupported) return e;
    }
    ActView a{hq, hs, hb};
    return launch_rows<false>(st, w2, w2, dtype, E, ff, d, offsets, nullptr, a, out);
}

}  // namespace cmoe
