// CPU oracle for the quantized mixture-of-experts feed-forward block.
//
// THIS FILE IS TEST INFRASTRUCTURE.  It restates, in plain C++, the arithmetic of the
// reference's CPU path so that the CUDA kernels can be checked against it and so that a CPU
// baseline can be timed beside the GPU numbers.  Nothing in the shipped library links, loads or
// calls it.  Every function cites the reference location (path inside the candle workspace) whose
// behaviour it follows.
//
// Parity status: the reference is Rust and cannot be compiled where this was written, so the
// oracle is pinned piecewise against the literal known-answer values in the reference's own tests
// (candle-core/tests/quantized_tests.rs, candle-nn/tests/ops.rs, candle-core/tests/tensor_tests.rs);
// see tests/test_oracle_golden.py.  The seeded-RNG spot values of quantized_tests.rs:1050-1203
// need Rust's `rand` stream and are NOT reproduced.  The f32 router product of the reference runs
// inside the third-party `gemm` crate (0.18.2) whose summation order is not visible: the oracle
// uses candle's own 8-lane f32 dot order for it, and router parity is therefore "unpinned" at the
// last-ulp level (near-ties are reported, not hidden).
//
// Rust semantics that C++ does not share are made explicit here:
//   * `f32 as i8/u8/i32` saturates and maps NaN to 0   -> sat_cast_*()
//   * `f32::round` rounds half away from zero          -> roundf()
//   * `f16::from_f32` is IEEE round-to-nearest-even    -> _Float16 conversion (F16C)
//   * no floating-point contraction                    -> built with -ffp-contract=off
//   * `sort_by` is stable                              -> std::stable_sort
//
// Build: see oracle/Makefile (g++ -O3 -mavx2 -mfma -mf16c -ffp-contract=off -fopenmp).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#if defined(__AVX2__)
#include <immintrin.h>
#endif
#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

// GgmlDType::to_u32 ids, candle-core/src/quantized/mod.rs:176-195
enum : int { DT_Q4_0 = 2, DT_Q8_0 = 8, DT_Q4K = 12, DT_Q6K = 14, DT_Q8K = 15 };

constexpr int QK_K = 256;
constexpr int QK8_0 = 32;
constexpr int QK4_0 = 32;

// ---- block layouts, candle-core/src/quantized/k_quants.rs:45-158 (repr(C), no padding) ----
#pragma pack(push, 1)
struct BlockQ4_0 { uint16_t d; uint8_t qs[16]; };                                  // :46-51
struct BlockQ8_0 { uint16_t d; int8_t qs[32]; };                                   // :81-87
struct BlockQ4K  { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; }; // :119-127
struct BlockQ6K  { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; }; // :141-149
struct BlockQ8K  { float d; int8_t qs[256]; int16_t bsums[16]; };                  // :151-158
#pragma pack(pop)
static_assert(sizeof(BlockQ4_0) == 18, "");
static_assert(sizeof(BlockQ8_0) == 34, "");
static_assert(sizeof(BlockQ4K) == 144, "");
static_assert(sizeof(BlockQ6K) == 210, "");
static_assert(sizeof(BlockQ8K) == 292, "");

// ---- Rust cast / rounding semantics ----
inline int32_t sat_cast_i32(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 2147483648.0f) return std::numeric_limits<int32_t>::max();
    if (v <= -2147483648.0f) return std::numeric_limits<int32_t>::min();
    return (int32_t)v;
}
inline int8_t sat_cast_i8(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 127.0f) return 127;
    if (v <= -128.0f) return -128;
    return (int8_t)v;
}
inline uint8_t sat_cast_u8(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 255.0f) return 255;
    if (v <= 0.0f) return 0;
    return (uint8_t)v;
}
// utils.rs:1-3
inline int32_t nearest_int(float v) { return sat_cast_i32(roundf(v)); }

inline float f16_to_f32(uint16_t h) {
    _Float16 x;
    std::memcpy(&x, &h, 2);
    return (float)x;
}
inline uint16_t f32_to_f16(float f) {
    _Float16 x = (_Float16)f;
    uint16_t h;
    std::memcpy(&h, &x, 2);
    return h;
}

// utils.rs:50-60
inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// ------------------------------------------------------------------------------------------
// Weight quantizer helpers
// ------------------------------------------------------------------------------------------

// utils.rs:202-259  (older ggml search, nmax = 15, ntry = 5 for Q4K)
void make_qkx1_quants(int nmax, int ntry, const float* x, int n, float* out_scale, float* out_min) {
    uint8_t l[64] = {0};
    float mn = x[0], mx = x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
    }
    if (mx == mn) {
        *out_scale = 0.f;
        *out_min = 0.f;
        return;
    }
    float minv = std::fmin(mn, 0.f);
    float iscale = (float)nmax / (mx - minv);
    float scale = 1.0f / iscale;
    for (int t = 0; t < ntry; ++t) {
        float sumlx = 0.f;
        int32_t suml2 = 0;
        bool did_change = false;
        for (int i = 0; i < n; ++i) {
            int32_t li = nearest_int(iscale * (x[i] - minv));
            li = std::min(std::max(li, 0), nmax);
            uint8_t c = (uint8_t)li;
            if (c != l[i]) {
                l[i] = c;
                did_change = true;
            }
            sumlx += (x[i] - minv) * (float)li;
            suml2 += li * li;
        }
        scale = sumlx / (float)suml2;
        float sum = 0.f;
        for (int i = 0; i < n; ++i) sum += x[i] - scale * (float)l[i];
        minv = sum / (float)n;
        if (minv > 0.f) minv = 0.f;
        iscale = 1.0f / scale;
        if (!did_change) break;
    }
    *out_scale = scale;
    *out_min = -minv;
}

// utils.rs:62-199 restricted to what Q6K uses (rmse_type = 1: weights x^2, no final sweep)
float make_qx_quants_rmse1(int n, int nmax, const float* x, int8_t* ls) {
    float mx = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) {
        float ax = std::fabs(x[i]);
        if (ax > amax) {
            amax = ax;
            mx = x[i];
        }
    }
    if (amax == 0.f) {
        for (int i = 0; i < n; ++i) ls[i] = 0;
        return 0.f;
    }
    float iscale = -(float)nmax / mx;
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        int32_t l = nearest_int(iscale * x[i]);
        l = std::min(std::max(l, -nmax), nmax - 1);
        ls[i] = (int8_t)(l + nmax);
        float w = x[i] * x[i];
        float lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = sumlx / suml2;
    float best = scale * sumlx;
    for (int itry = 0; itry < 3; ++itry) {
        float is2 = 1.0f / scale;
        float slx = 0.f, sl2 = 0.f;
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            int32_t l = nearest_int(is2 * x[i]);
            l = std::min(std::max(l, -nmax), nmax - 1);
            if (l + nmax != (int32_t)ls[i]) changed = true;
            float w = x[i] * x[i];
            float lf = (float)l;
            slx += w * x[i] * lf;
            sl2 += w * lf * lf;
        }
        if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) {
            int32_t l = nearest_int(is2 * x[i]);
            ls[i] = (int8_t)(nmax + std::min(std::max(l, -nmax), nmax - 1));
        }
        sumlx = slx;
        suml2 = sl2;
        scale = sumlx / suml2;
        best = scale * sumlx;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            float w = x[i] * x[i];
            int32_t l = (int32_t)ls[i] - nmax;
            float slx = sumlx - w * x[i] * (float)l;
            if (slx > 0.f) {
                float sl2 = suml2 - w * (float)l * (float)l;
                int32_t new_l = nearest_int(x[i] * sl2 / slx);
                new_l = std::min(std::max(new_l, -nmax), nmax - 1);
                if (new_l != l) {
                    slx += w * x[i] * (float)new_l;
                    sl2 += w * (float)new_l * (float)new_l;
                    if (sl2 > 0.f && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        ls[i] = (int8_t)(nmax + new_l);
                        sumlx = slx;
                        suml2 = sl2;
                        scale = sumlx / suml2;
                        best = scale * sumlx;
                        ++n_changed;
                    }
                }
            }
        }
        if (n_changed == 0) break;
    }
    (void)best;
    return scale;
}

// ------------------------------------------------------------------------------------------
// from_float (quantizers)
// ------------------------------------------------------------------------------------------

// k_quants.rs:188-221
void quantize_q4_0(const float* xs, size_t k, BlockQ4_0* ys) {
    const size_t nb = k / QK4_0;
    for (size_t i = 0; i < nb; ++i) {
        const float* x = xs + i * QK4_0;
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < QK4_0; ++j) {
            if (amax < std::fabs(x[j])) {
                amax = std::fabs(x[j]);
                mx = x[j];
            }
        }
        float d = mx / -8.0f;
        float id = d != 0.f ? 1.0f / d : 0.f;
        ys[i].d = f32_to_f16(d);
        for (int j = 0; j < QK4_0 / 2; ++j) {
            float x0 = x[j] * id;
            float x1 = x[QK4_0 / 2 + j] * id;
            uint8_t xi0 = std::min<uint8_t>(15, sat_cast_u8(x0 + 8.5f));
            uint8_t xi1 = std::min<uint8_t>(15, sat_cast_u8(x1 + 8.5f));
            ys[i].qs[j] = (uint8_t)(xi0 | (xi1 << 4));
        }
    }
}

// k_quants.rs:605-634
void quantize_q8_0(const float* xs, size_t k, BlockQ8_0* ys) {
    const size_t nb = k / QK8_0;
    for (size_t i = 0; i < nb; ++i) {
        const float* x = xs + i * QK8_0;
        float amax = 0.f;
        for (int j = 0; j < QK8_0; ++j) amax = std::fmax(amax, std::fabs(x[j]));
        float d = amax / 127.0f;
        float id = d != 0.f ? 1.0f / d : 0.f;
        ys[i].d = f32_to_f16(d);
        for (int j = 0; j < QK8_0; ++j) ys[i].qs[j] = sat_cast_i8(roundf(x[j] * id));
    }
}

// k_quants.rs:1287-1345
void quantize_q4k(const float* xs, size_t k, BlockQ4K* ys) {
    const size_t nb = k / QK_K;
    for (size_t ib = 0; ib < nb; ++ib) {
        const float* x = xs + ib * QK_K;
        BlockQ4K& b = ys[ib];
        std::memset(&b, 0, sizeof(b));
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1_quants(15, 5, x + 32 * j, 32, &scales[j], &mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) {
            max_scale = std::fmax(scales[j], max_scale);
            max_min = std::fmax(mins[j], max_min);
        }
        float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        for (int j = 0; j < 8; ++j) {
            uint8_t ls = (uint8_t)std::min(nearest_int(inv_scale * scales[j]), 63);
            uint8_t lm = (uint8_t)std::min(nearest_int(inv_min * mins[j]), 63);
            if (j < 4) {
                b.scales[j] = ls;
                b.scales[j + 4] = lm;
            } else {
                b.scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                b.scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                b.scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        b.d = f32_to_f16(max_scale / 63.0f);
        b.dmin = f32_to_f16(max_min / 63.0f);
        uint8_t l[QK_K] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            get_scale_min_k4(j, b.scales, &sc, &m);
            float d = f16_to_f32(b.d) * (float)sc;
            if (d != 0.f) {
                float dm = f16_to_f32(b.dmin) * (float)m;
                for (int ii = 0; ii < 32; ++ii) {
                    int32_t lv = nearest_int((x[32 * j + ii] + dm) / d);
                    l[32 * j + ii] = (uint8_t)std::min(std::max(lv, 0), 15);
                }
            }
        }
        for (int j = 0; j < QK_K; j += 64)
            for (int lv = 0; lv < 32; ++lv)
                b.qs[(j / 64) * 32 + lv] = (uint8_t)(l[j + lv] | (l[j + lv + 32] << 4));
    }
}

// k_quants.rs:1675-1744
void quantize_q6k(const float* xs, size_t k, BlockQ6K* ys) {
    const size_t nb = k / QK_K;
    int8_t l[QK_K];
    float scales[16];
    for (size_t ib = 0; ib < nb; ++ib) {
        const float* x = xs + ib * QK_K;
        BlockQ6K& y = ys[ib];
        std::memset(l, 0, sizeof(l));
        float max_scale = 0.f, max_abs_scale = 0.f;
        for (int j = 0; j < 16; ++j) {
            float s = make_qx_quants_rmse1(16, 32, x + 16 * j, l + 16 * j);
            scales[j] = s;
            float a = std::fabs(s);
            if (a > max_abs_scale) {
                max_abs_scale = a;
                max_scale = s;
            }
        }
        float iscale = -128.0f / max_scale;
        y.d = f32_to_f16(1.0f / iscale);
        for (int j = 0; j < 16; ++j)
            y.scales[j] = (int8_t)std::min(nearest_int(iscale * scales[j]), 127);
        for (int j = 0; j < 16; ++j) {
            float d = f16_to_f32(y.d) * (float)y.scales[j];
            if (d == 0.f) continue;
            for (int ii = 0; ii < 16; ++ii) {
                int32_t ll = nearest_int(x[16 * j + ii] / d);
                ll = std::min(std::max(ll, -32), 31);
                l[16 * j + ii] = (int8_t)(ll + 32);
            }
        }
        for (int j = 0; j < QK_K; j += 128) {
            uint8_t* ql = y.ql + j / 2;
            uint8_t* qh = y.qh + j / 4;
            for (int i = 0; i < 32; ++i) {
                uint8_t q1 = l[j + i] & 0xF, q2 = l[j + i + 32] & 0xF;
                uint8_t q3 = l[j + i + 64] & 0xF, q4 = l[j + i + 96] & 0xF;
                ql[i] = (uint8_t)(q1 | (q3 << 4));
                ql[i + 32] = (uint8_t)(q2 | (q4 << 4));
                qh[i] = (uint8_t)((l[j + i] >> 4) | ((l[j + i + 32] >> 4) << 2) |
                                  ((l[j + i + 64] >> 4) << 4) | ((l[j + i + 96] >> 4) << 6));
            }
        }
    }
}

// k_quants.rs:1819-1856 (activation quantizer for k-quant weights).  The caller provides
// zero-initialised blocks, as `matmul` does with `VecDotType::zeros()`; an all-zero input block
// leaves `bsums` untouched, like the reference.
void quantize_q8k(const float* xs, size_t k, BlockQ8K* ys) {
    const size_t nb = k / QK_K;
    for (size_t i = 0; i < nb; ++i) {
        const float* x = xs + i * QK_K;
        BlockQ8K& y = ys[i];
        float mx = 0.f, amax = 0.f;
        for (int j = 0; j < QK_K; ++j) {
            if (amax < std::fabs(x[j])) {
                amax = std::fabs(x[j]);
                mx = x[j];
            }
        }
        if (amax == 0.f) {
            y.d = 0.f;
            std::memset(y.qs, 0, sizeof(y.qs));
        } else {
            float iscale = -128.0f / mx;
            for (int j = 0; j < QK_K; ++j) {
                float v = roundf(iscale * x[j]);
                y.qs[j] = sat_cast_i8(std::fmin(v, 127.f));
            }
            for (int j = 0; j < 16; ++j) {
                int32_t sum = 0;
                for (int ii = 0; ii < 16; ++ii) sum += y.qs[j * 16 + ii];
                y.bsums[j] = (int16_t)sum;
            }
            y.d = 1.0f / iscale;
        }
    }
}

// ------------------------------------------------------------------------------------------
// to_float (dequantizers)
// ------------------------------------------------------------------------------------------

void dequantize_q4_0(const BlockQ4_0* xs, size_t k, float* ys) {  // k_quants.rs:166-186
    for (size_t i = 0; i < k / QK4_0; ++i) {
        float d = f16_to_f32(xs[i].d);
        for (int j = 0; j < 16; ++j) {
            int x0 = (xs[i].qs[j] & 0x0F) - 8, x1 = (xs[i].qs[j] >> 4) - 8;
            ys[i * 32 + j] = (float)x0 * d;
            ys[i * 32 + j + 16] = (float)x1 * d;
        }
    }
}
void dequantize_q8_0(const BlockQ8_0* xs, size_t k, float* ys) {  // k_quants.rs:587-603
    for (size_t i = 0; i < k / QK8_0; ++i) {
        float d = f16_to_f32(xs[i].d);
        for (int j = 0; j < 32; ++j) ys[i * 32 + j] = (float)xs[i].qs[j] * d;
    }
}
void dequantize_q4k(const BlockQ4K* xs, size_t k, float* ys) {  // k_quants.rs:1347-1374
    for (size_t ib = 0; ib < k / QK_K; ++ib) {
        const BlockQ4K& b = xs[ib];
        float d = f16_to_f32(b.d), mn = f16_to_f32(b.dmin);
        float* y = ys + ib * QK_K;
        int is = 0, yi = 0;
        for (int j = 0; j < QK_K; j += 64) {
            const uint8_t* q = b.qs + j / 2;
            uint8_t sc, m;
            get_scale_min_k4(is, b.scales, &sc, &m);
            float d1 = d * (float)sc, m1 = mn * (float)m;
            get_scale_min_k4(is + 1, b.scales, &sc, &m);
            float d2 = d * (float)sc, m2 = mn * (float)m;
            for (int l = 0; l < 32; ++l) y[yi++] = d1 * (float)(q[l] & 0xF) - m1;
            for (int l = 0; l < 32; ++l) y[yi++] = d2 * (float)(q[l] >> 4) - m2;
            is += 2;
        }
    }
}
void dequantize_q6k(const BlockQ6K* xs, size_t k, float* ys) {  // k_quants.rs:1747-1778
    for (size_t ib = 0; ib < k / QK_K; ++ib) {
        const BlockQ6K& x = xs[ib];
        float d = f16_to_f32(x.d);
        for (int n = 0; n < QK_K; n += 128) {
            int idx = n / 128;
            float* y = ys + ib * QK_K + n;
            const int8_t* sc = x.scales + 8 * idx;
            const uint8_t* ql = x.ql + 64 * idx;
            const uint8_t* qh = x.qh + 32 * idx;
            for (int l = 0; l < 32; ++l) {
                int is = l / 16;
                int8_t q1 = (int8_t)(((ql[l] & 0xF) | ((qh[l] & 3) << 4))) - 32;
                int8_t q2 = (int8_t)(((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4))) - 32;
                int8_t q3 = (int8_t)(((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4))) - 32;
                int8_t q4 = (int8_t)(((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4))) - 32;
                y[l] = d * (float)sc[is] * (float)q1;
                y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                y[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
        }
    }
}
void dequantize_q8k(const BlockQ8K* xs, size_t k, float* ys) {  // k_quants.rs:1858-1870
    for (size_t i = 0; i < k / QK_K; ++i)
        for (int j = 0; j < QK_K; ++j) ys[i * QK_K + j] = xs[i].d * (float)xs[i].qs[j];
}

// ------------------------------------------------------------------------------------------
// vec_dot.  Three orderings of the same integer products:
//   ORDER_SIMD  : AVX2 intrinsics, the lane mapping of candle-core/src/quantized/avx.rs (what the
//                 reference binary computes on an x86 host built with target-cpu=native)
//   ORDER_LANES : scalar re-statement of that lane mapping (bit-identical to ORDER_SIMD;
//                 portable, used to cross-check the intrinsics)
//   ORDER_UNOPT : the reference's vec_dot_unopt summation order
// ------------------------------------------------------------------------------------------
enum : int { ORDER_SIMD = 0, ORDER_LANES = 1, ORDER_UNOPT = 2 };

// avx.rs:26-32: ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7))
inline float hsum8(const float* l) {
    float r0 = l[4] + l[0], r1 = l[5] + l[1], r2 = l[6] + l[2], r3 = l[7] + l[3];
    float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

inline void unpack_q4k_scales(const uint8_t* s, uint8_t* sc, uint8_t* mn) {
    for (int j = 0; j < 8; ++j) get_scale_min_k4(j, s, &sc[j], &mn[j]);
}

// --- Q4K x Q8K ---
float dot_q4k_q8k_lanes(size_t n, const BlockQ4K* xs, const BlockQ8K* ys) {  // avx.rs:443-525
    float acc[8] = {0}, accm[4] = {0};
    for (size_t ib = 0; ib < n / QK_K; ++ib) {
        const BlockQ4K& x = xs[ib];
        const BlockQ8K& y = ys[ib];
        float d = y.d * f16_to_f32(x.d);
        float dmin = -y.d * f16_to_f32(x.dmin);
        uint8_t sc[8], mn[8];
        unpack_q4k_scales(x.scales, sc, mn);
        for (int t = 0; t < 4; ++t) {
            int16_t s0 = (int16_t)(y.bsums[4 * t] + y.bsums[4 * t + 1]);
            int16_t s1 = (int16_t)(y.bsums[4 * t + 2] + y.bsums[4 * t + 3]);
            int32_t prod = (int32_t)mn[2 * t] * s0 + (int32_t)mn[2 * t + 1] * s1;
            accm[t] = std::fmaf(dmin, (float)prod, accm[t]);
        }
        int32_t sumi[8] = {0};
        for (int j = 0; j < 4; ++j) {
            const uint8_t* q4 = x.qs + 32 * j;
            const int8_t* q8l = y.qs + 64 * j;
            const int8_t* q8h = q8l + 32;
            for (int i = 0; i < 32; ++i) {
                int r = i >> 2;
                sumi[r] += (int32_t)sc[2 * j] * ((q4[i] & 0xF) * q8l[i]);
                sumi[r] += (int32_t)sc[2 * j + 1] * ((q4[i] >> 4) * q8h[i]);
            }
        }
        for (int r = 0; r < 8; ++r) acc[r] = std::fmaf(d, (float)sumi[r], acc[r]);
    }
    float m = (accm[0] + accm[2]) + (accm[1] + accm[3]);
    return hsum8(acc) + m;
}

float dot_q4k_q8k_unopt(size_t n, const BlockQ4K* xs, const BlockQ8K* ys) {  // k_quants.rs:1205-1285
    float sums[8] = {0};
    float sumf = 0.f;
    int8_t aux8[QK_K];
    for (size_t ib = 0; ib < n / QK_K; ++ib) {
        const BlockQ4K& x = xs[ib];
        const BlockQ8K& y = ys[ib];
        int32_t aux32[8] = {0};
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 32; ++l) {
                aux8[64 * j + l] = (int8_t)(x.qs[32 * j + l] & 0xF);
                aux8[64 * j + 32 + l] = (int8_t)(x.qs[32 * j + l] >> 4);
            }
        uint8_t sc[8], mn[8];
        unpack_q4k_scales(x.scales, sc, mn);
        int32_t sumi = 0;
        for (int j = 0; j < 16; ++j) sumi += (int32_t)y.bsums[j] * (int32_t)mn[j / 2];
        for (int j = 0; j < 8; ++j)
            for (int g = 0; g < 4; ++g)
                for (int l = 0; l < 8; ++l) {
                    int idx = 32 * j + 8 * g + l;
                    aux32[l] += (int32_t)sc[j] * (int32_t)(int16_t)(y.qs[idx] * aux8[idx]);
                }
        float d = f16_to_f32(x.d) * y.d;
        for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
        float dmin = f16_to_f32(x.dmin) * y.d;
        sumf -= dmin * (float)sumi;
    }
    float s = 0.f;
    for (int l = 0; l < 8; ++l) s += sums[l];
    return sumf + s;
}

// --- Q6K x Q8K ---
inline void unpack_q6k(const BlockQ6K& x, int8_t* a) {  // element order of to_float
    for (int h = 0; h < 2; ++h) {
        const uint8_t* ql = x.ql + 64 * h;
        const uint8_t* qh = x.qh + 32 * h;
        int8_t* o = a + 128 * h;
        for (int l = 0; l < 32; ++l) {
            o[l] = (int8_t)((int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
            o[l + 32] = (int8_t)((int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
            o[l + 64] = (int8_t)((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
            o[l + 96] = (int8_t)((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
        }
    }
}

float dot_q6k_q8k_lanes(size_t n, const BlockQ6K* xs, const BlockQ8K* ys) {  // avx.rs:131-216
    float acc[8] = {0};
    int8_t a[QK_K];
    for (size_t ib = 0; ib < n / QK_K; ++ib) {
        const BlockQ6K& x = xs[ib];
        const BlockQ8K& y = ys[ib];
        float d = y.d * f16_to_f32(x.d);
        unpack_q6k(x, a);
        int32_t sumi[8] = {0};
        for (int e = 0; e < QK_K; ++e) {
            int r = (e & 31) >> 2;
            sumi[r] += (int32_t)x.scales[e >> 4] * ((int32_t)a[e] * (int32_t)y.qs[e]);
        }
        for (int r = 0; r < 8; ++r) acc[r] = std::fmaf(d, (float)sumi[r], acc[r]);
    }
    return hsum8(acc);
}

float dot_q6k_q8k_unopt(size_t n, const BlockQ6K* xs, const BlockQ8K* ys) {  // k_quants.rs:1616-1673
    float sums[8] = {0};
    int8_t a[QK_K];
    for (size_t ib = 0; ib < n / QK_K; ++ib) {
        const BlockQ6K& x = xs[ib];
        const BlockQ8K& y = ys[ib];
        float aux32[8] = {0};
        unpack_q6k(x, a);
        for (int j = 0; j < 16; ++j) {
            float scale = (float)x.scales[j];
            for (int half = 0; half < 2; ++half)
                for (int l = 0; l < 8; ++l) {
                    int idx = 16 * j + 8 * half + l;
                    int16_t p = (int16_t)((int16_t)y.qs[idx] * (int16_t)a[idx]);
                    aux32[l] += scale * (float)p;
                }
        }
        float d = f16_to_f32(x.d) * y.d;
        for (int l = 0; l < 8; ++l) sums[l] += aux32[l] * d;
    }
    float s = 0.f;
    for (int l = 0; l < 8; ++l) s += sums[l];
    return s;
}

// --- Q8_0 x Q8_0 and Q4_0 x Q8_0 ---
float dot_q8_0_q8_0_lanes(size_t n, const BlockQ8_0* xs, const BlockQ8_0* ys) {  // avx.rs:71-87
    float acc[8] = {0};
    for (size_t ib = 0; ib < n / QK8_0; ++ib) {
        float d = f16_to_f32(xs[ib].d) * f16_to_f32(ys[ib].d);
        for (int r = 0; r < 8; ++r) {
            int32_t s = 0;
            for (int i = 4 * r; i < 4 * r + 4; ++i) s += (int32_t)xs[ib].qs[i] * (int32_t)ys[ib].qs[i];
            acc[r] = std::fmaf(d, (float)s, acc[r]);
        }
    }
    return hsum8(acc);
}
float dot_q8_0_q8_0_unopt(size_t n, const BlockQ8_0* xs, const BlockQ8_0* ys) {  // k_quants.rs:650-668
    float sumf = 0.f;
    for (size_t ib = 0; ib < n / QK8_0; ++ib) {
        int32_t s = 0;
        for (int i = 0; i < 32; ++i) s += (int32_t)xs[ib].qs[i] * (int32_t)ys[ib].qs[i];
        sumf += (float)s * f16_to_f32(xs[ib].d) * f16_to_f32(ys[ib].d);
    }
    return sumf;
}
float dot_q4_0_q8_0_lanes(size_t n, const BlockQ4_0* xs, const BlockQ8_0* ys) {  // avx.rs:51-68
    float acc[8] = {0};
    for (size_t ib = 0; ib < n / QK8_0; ++ib) {
        float d = f16_to_f32(xs[ib].d) * f16_to_f32(ys[ib].d);
        int8_t w[32];
        for (int j = 0; j < 16; ++j) {
            w[j] = (int8_t)((xs[ib].qs[j] & 0xF) - 8);
            w[j + 16] = (int8_t)((xs[ib].qs[j] >> 4) - 8);
        }
        for (int r = 0; r < 8; ++r) {
            int32_t s = 0;
            for (int i = 4 * r; i < 4 * r + 4; ++i) s += (int32_t)w[i] * (int32_t)ys[ib].qs[i];
            acc[r] = std::fmaf(d, (float)s, acc[r]);
        }
    }
    return hsum8(acc);
}
float dot_q4_0_q8_0_unopt(size_t n, const BlockQ4_0* xs, const BlockQ8_0* ys) {  // k_quants.rs:238-258
    float sumf = 0.f;
    for (size_t ib = 0; ib < n / QK8_0; ++ib) {
        int32_t s = 0;
        for (int j = 0; j < 16; ++j) {
            int v0 = (xs[ib].qs[j] & 0x0F) - 8, v1 = (xs[ib].qs[j] >> 4) - 8;
            s += v0 * ys[ib].qs[j] + v1 * ys[ib].qs[j + 16];
        }
        sumf += (float)s * f16_to_f32(xs[ib].d) * f16_to_f32(ys[ib].d);
    }
    return sumf;
}

#if defined(__AVX2__)
inline float hsum8_v(__m256 v) {
    float l[8];
    _mm256_storeu_ps(l, v);
    return hsum8(l);
}

float dot_q4k_q8k_simd(size_t n, const BlockQ4K* xs, const BlockQ8K* ys) {
    const __m256i nib = _mm256_set1_epi8(0xF);
    __m256 acc = _mm256_setzero_ps();
    float accm[4] = {0, 0, 0, 0};
    for (size_t ib = 0; ib < n / QK_K; ++ib) {
        const BlockQ4K& x = xs[ib];
        const BlockQ8K& y = ys[ib];
        const float d = y.d * f16_to_f32(x.d);
        const float dmin = -y.d * f16_to_f32(x.dmin);
        uint8_t sc[8], mn[8];
        unpack_q4k_scales(x.scales, sc, mn);
        for (int t = 0; t < 4; ++t) {
            int16_t s0 = (int16_t)(y.bsums[4 * t] + y.bsums[4 * t + 1]);
            int16_t s1 = (int16_t)(y.bsums[4 * t + 2] + y.bsums[4 * t + 3]);
            int32_t prod = (int32_t)mn[2 * t] * s0 + (int32_t)mn[2 * t + 1] * s1;
            accm[t] = std::fmaf(dmin, (float)prod, accm[t]);
        }
        __m256i sumi = _mm256_setzero_si256();
        for (int j = 0; j < 4; ++j) {
            const __m256i packed = _mm256_loadu_si256((const __m256i*)(x.qs + 32 * j));
            const __m256i lo = _mm256_and_si256(packed, nib);
            const __m256i hi = _mm256_and_si256(_mm256_srli_epi16(packed, 4), nib);
            const __m256i a_lo = _mm256_loadu_si256((const __m256i*)(y.qs + 64 * j));
            const __m256i a_hi = _mm256_loadu_si256((const __m256i*)(y.qs + 64 * j + 32));
            const __m256i p_lo = _mm256_madd_epi16(_mm256_set1_epi16(sc[2 * j]), _mm256_maddubs_epi16(lo, a_lo));
            const __m256i p_hi = _mm256_madd_epi16(_mm256_set1_epi16(sc[2 * j + 1]), _mm256_maddubs_epi16(hi, a_hi));
            sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p_lo, p_hi));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    float m = (accm[0] + accm[2]) + (accm[1] + accm[3]);
    return hsum8_v(acc) + m;
}

float dot_q6k_q8k_simd(size_t n, const BlockQ6K* xs, const BlockQ8K* ys) {
    const __m256i nib = _mm256_set1_epi8(0xF);
    const __m256i two = _mm256_set1_epi8(3);
    const __m256i off = _mm256_set1_epi8(32);
    __m256 acc = _mm256_setzero_ps();
    for (size_t ib = 0; ib < n / QK_K; ++ib) {
        const BlockQ6K& x = xs[ib];
        const BlockQ8K& y = ys[ib];
        const float d = y.d * f16_to_f32(x.d);
        __m256i sumi = _mm256_setzero_si256();
        for (int h = 0; h < 2; ++h) {
            const __m256i l0 = _mm256_loadu_si256((const __m256i*)(x.ql + 64 * h));
            const __m256i l1 = _mm256_loadu_si256((const __m256i*)(x.ql + 64 * h + 32));
            const __m256i hb = _mm256_loadu_si256((const __m256i*)(x.qh + 32 * h));
            __m256i q[4];
            q[0] = _mm256_or_si256(_mm256_and_si256(l0, nib), _mm256_slli_epi16(_mm256_and_si256(hb, two), 4));
            q[1] = _mm256_or_si256(_mm256_and_si256(l1, nib),
                                   _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 2), two), 4));
            q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), nib),
                                   _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 4), two), 4));
            q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), nib),
                                   _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 6), two), 4));
            for (int c = 0; c < 4; ++c) {
                const __m256i a8 = _mm256_loadu_si256((const __m256i*)(y.qs + 128 * h + 32 * c));
                // (q - 32) * a8 as 16-bit pair sums
                const __m256i p = _mm256_sub_epi16(_mm256_maddubs_epi16(q[c], a8), _mm256_maddubs_epi16(off, a8));
                const int si = 8 * h + 2 * c;
                const __m256i sv = _mm256_set_m128i(_mm_set1_epi16(x.scales[si + 1]), _mm_set1_epi16(x.scales[si]));
                sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(sv, p));
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum8_v(acc);
}

inline __m256 i8_pair_dot_ps(__m256i x, __m256i y) {
    const __m256i ax = _mm256_sign_epi8(x, x);
    const __m256i sy = _mm256_sign_epi8(y, x);
    const __m256i p16 = _mm256_maddubs_epi16(ax, sy);
    return _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_set1_epi16(1), p16));
}

float dot_q8_0_q8_0_simd(size_t n, const BlockQ8_0* xs, const BlockQ8_0* ys) {
    __m256 acc = _mm256_setzero_ps();
    for (size_t ib = 0; ib < n / QK8_0; ++ib) {
        const float d = f16_to_f32(xs[ib].d) * f16_to_f32(ys[ib].d);
        const __m256i bx = _mm256_loadu_si256((const __m256i*)xs[ib].qs);
        const __m256i by = _mm256_loadu_si256((const __m256i*)ys[ib].qs);
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), i8_pair_dot_ps(bx, by), acc);
    }
    return hsum8_v(acc);
}
#endif

float vec_dot(int dtype, size_t n, const void* w, const void* a, int order) {
#if !defined(__AVX2__)
    if (order == ORDER_SIMD) order = ORDER_LANES;
#endif
    switch (dtype) {
        case DT_Q4K:
#if defined(__AVX2__)
            if (order == ORDER_SIMD) return dot_q4k_q8k_simd(n, (const BlockQ4K*)w, (const BlockQ8K*)a);
#endif
            if (order == ORDER_UNOPT) return dot_q4k_q8k_unopt(n, (const BlockQ4K*)w, (const BlockQ8K*)a);
            return dot_q4k_q8k_lanes(n, (const BlockQ4K*)w, (const BlockQ8K*)a);
        case DT_Q6K:
#if defined(__AVX2__)
            if (order == ORDER_SIMD) return dot_q6k_q8k_simd(n, (const BlockQ6K*)w, (const BlockQ8K*)a);
#endif
            if (order == ORDER_UNOPT) return dot_q6k_q8k_unopt(n, (const BlockQ6K*)w, (const BlockQ8K*)a);
            return dot_q6k_q8k_lanes(n, (const BlockQ6K*)w, (const BlockQ8K*)a);
        case DT_Q8_0:
#if defined(__AVX2__)
            if (order == ORDER_SIMD) return dot_q8_0_q8_0_simd(n, (const BlockQ8_0*)w, (const BlockQ8_0*)a);
#endif
            if (order == ORDER_UNOPT) return dot_q8_0_q8_0_unopt(n, (const BlockQ8_0*)w, (const BlockQ8_0*)a);
            return dot_q8_0_q8_0_lanes(n, (const BlockQ8_0*)w, (const BlockQ8_0*)a);
        case DT_Q4_0:
            if (order == ORDER_UNOPT) return dot_q4_0_q8_0_unopt(n, (const BlockQ4_0*)w, (const BlockQ8_0*)a);
            return dot_q4_0_q8_0_lanes(n, (const BlockQ4_0*)w, (const BlockQ8_0*)a);
    }
    return std::numeric_limits<float>::quiet_NaN();
}

size_t block_bytes(int dtype) {
    switch (dtype) {
        case DT_Q4_0: return sizeof(BlockQ4_0);
        case DT_Q8_0: return sizeof(BlockQ8_0);
        case DT_Q4K: return sizeof(BlockQ4K);
        case DT_Q6K: return sizeof(BlockQ6K);
        case DT_Q8K: return sizeof(BlockQ8K);
    }
    return 0;
}
int block_elems(int dtype) {
    switch (dtype) {
        case DT_Q4_0: case DT_Q8_0: return 32;
        case DT_Q4K: case DT_Q6K: case DT_Q8K: return 256;
    }
    return 0;
}
// GgmlType::VecDotType, k_quants.rs:163,584,1189,1600
int vec_dot_dtype(int dtype) {
    switch (dtype) {
        case DT_Q4_0: case DT_Q8_0: return DT_Q8_0;
        case DT_Q4K: case DT_Q6K: return DT_Q8K;
    }
    return -1;
}

int quantize(int dtype, const float* x, size_t n, void* out) {
    switch (dtype) {
        case DT_Q4_0: quantize_q4_0(x, n, (BlockQ4_0*)out); return 0;
        case DT_Q8_0: quantize_q8_0(x, n, (BlockQ8_0*)out); return 0;
        case DT_Q4K: quantize_q4k(x, n, (BlockQ4K*)out); return 0;
        case DT_Q6K: quantize_q6k(x, n, (BlockQ6K*)out); return 0;
        case DT_Q8K: quantize_q8k(x, n, (BlockQ8K*)out); return 0;
    }
    return -1;
}

// k_quants.rs:1873-1920: quantize every lhs row to the weight type's VecDotType (serially), then
// for each row a parallel loop over the n output columns, one vec_dot each.  Rows are visited one
// after another, so the weights are streamed once per row, exactly like the reference.
int matmul(int dtype, size_t m, size_t k, size_t n, const float* lhs, const void* rhs_t, float* dst, int order) {
    const int adt = vec_dot_dtype(dtype);
    if (adt < 0) return -1;
    const int be = block_elems(dtype);
    if (k % be != 0) return -2;
    const size_t kb = k / be;
    const size_t abytes = block_bytes(adt), wbytes = block_bytes(dtype);
    std::vector<uint8_t> act(m * kb * abytes, 0);
    for (size_t r = 0; r < m; ++r) quantize(adt, lhs + r * k, k, act.data() + r * kb * abytes);
    const uint8_t* w = (const uint8_t*)rhs_t;
    for (size_t r = 0; r < m; ++r) {
        const uint8_t* arow = act.data() + r * kb * abytes;
        float* drow = dst + r * n;
#pragma omp parallel for schedule(dynamic, 128)
        for (long c = 0; c < (long)n; ++c) drow[c] = vec_dot(dtype, k, w + (size_t)c * kb * wbytes, arow, order);
    }
    return 0;
}

// candle-core/src/cpu/mod.rs:132-152 with the AVX2 `CurrentCpu` (STEP 32, EPR 8, avx.rs:53-66)
float vec_sum_f32(const float* row, size_t k) {
    const size_t np = k & ~(size_t)31;
    float lanes[4][8] = {{0}};
    for (size_t i = 0; i < np; i += 32)
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 8; ++l) lanes[j][l] += row[i + 8 * j + l];
    float x0[8];
    for (int l = 0; l < 8; ++l) x0[l] = (lanes[0][l] + lanes[1][l]) + (lanes[2][l] + lanes[3][l]);
    float t0[4];
    for (int l = 0; l < 4; ++l) t0[l] = x0[l] + x0[l + 4];
    float b = (t0[0] + t0[1]) + (t0[2] + t0[3]);
    for (size_t i = np; i < k; ++i) b += row[i];
    return b;
}

// candle-core/src/cpu/mod.rs:89-110: candle's own f32 dot (4x8 lanes mul+add, tree, tail).  Used for
// the router product; the reference routes that product through the `gemm` crate whose order is
// not visible, hence "unpinned".
float vec_dot_f32(const float* a, const float* b, size_t k) {
    const size_t np = k & ~(size_t)31;
    float lanes[4][8] = {{0}};
    for (size_t i = 0; i < np; i += 32)
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 8; ++l) lanes[j][l] = a[i + 8 * j + l] * b[i + 8 * j + l] + lanes[j][l];
    float x0[8];
    for (int l = 0; l < 8; ++l) x0[l] = (lanes[0][l] + lanes[1][l]) + (lanes[2][l] + lanes[3][l]);
    float t0[4];
    for (int l = 0; l < 4; ++l) t0[l] = x0[l] + x0[l + 4];
    float c = (t0[0] + t0[1]) + (t0[2] + t0[3]);
    for (size_t i = np; i < k; ++i) c += a[i] * b[i];
    return c;
}

// candle-nn/src/ops.rs:326-339
void softmax_row(const float* src, size_t n, float* dst) {
    float mx = src[0];
    for (size_t i = 1; i < n; ++i) mx = std::fmax(mx, src[i]);
    for (size_t i = 0; i < n; ++i) dst[i] = std::exp(src[i] - mx);
    float s = vec_sum_f32(dst, n);
    for (size_t i = 0; i < n; ++i) dst[i] /= s;
}

// Rust f32::total_cmp as a sortable key
inline int32_t total_order_key(float f) {
    int32_t b;
    std::memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

inline float silu_f(float v) { return v / (1.0f + std::exp(-v)); }          // candle-core/src/op.rs:645-648
inline float sigmoid_f(float v) { return 1.0f / (std::exp(-v) + 1.0f); }    // candle-nn/src/ops.rs:59-61

}  // namespace

// ==========================================================================================
// C interface (ctypes)
// ==========================================================================================

// RmsNorm as candle's CPU op computes it (candle-nn/src/ops.rs:504-514): the squares are summed sequentially in
// f32, m = sqrt(sum / dim + eps), and each element is x / m * alpha (division first).
ORC_API int orc_rms_norm(const float* x, const float* alpha, float eps, size_t rows, size_t d, float* out) {
    for (size_t r = 0; r < rows; ++r) {
        const float* s = x + r * d;
        float sum2 = 0.f;
        for (size_t i = 0; i < d; ++i) sum2 += s[i] * s[i];
        const float m = std::sqrt(sum2 / (float)d + eps);
        for (size_t i = 0; i < d; ++i) out[r * d + i] = s[i] / m * alpha[i];
    }
    return 0;
}

ORC_API size_t orc_block_bytes(int dtype) { return block_bytes(dtype); }
ORC_API int orc_block_elems(int dtype) { return block_elems(dtype); }
ORC_API int orc_vec_dot_dtype(int dtype) { return vec_dot_dtype(dtype); }
ORC_API int orc_has_avx2(void) {
#if defined(__AVX2__)
    return 1;
#else
    return 0;
#endif
}
ORC_API int orc_max_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// QTensor::quantize -> T::from_float.  `out` must be zero-filled by the caller for Q8K.
ORC_API int orc_quantize(int dtype, const float* x, size_t n, void* out) {
    if (block_elems(dtype) == 0 || n % block_elems(dtype) != 0) return -1;
    return quantize(dtype, x, n, out);
}
// Same, rows quantized in parallel (rows are independent; used to make large synthetic weights).
ORC_API int orc_quantize_rows(int dtype, const float* x, size_t rows, size_t k, void* out) {
    if (block_elems(dtype) == 0 || k % block_elems(dtype) != 0) return -1;
    const size_t rb = k / block_elems(dtype) * block_bytes(dtype);
#pragma omp parallel for schedule(dynamic, 16)
    for (long r = 0; r < (long)rows; ++r) quantize(dtype, x + (size_t)r * k, k, (uint8_t*)out + (size_t)r * rb);
    return 0;
}
ORC_API int orc_dequantize(int dtype, const void* blocks, size_t n, float* out) {
    switch (dtype) {
        case DT_Q4_0: dequantize_q4_0((const BlockQ4_0*)blocks, n, out); return 0;
        case DT_Q8_0: dequantize_q8_0((const BlockQ8_0*)blocks, n, out); return 0;
        case DT_Q4K: dequantize_q4k((const BlockQ4K*)blocks, n, out); return 0;
        case DT_Q6K: dequantize_q6k((const BlockQ6K*)blocks, n, out); return 0;
        case DT_Q8K: dequantize_q8k((const BlockQ8K*)blocks, n, out); return 0;
    }
    return -1;
}
ORC_API float orc_vec_dot(int dtype, size_t n, const void* w, const void* act, int order) {
    return vec_dot(dtype, n, w, act, order);
}
ORC_API int orc_matmul(int dtype, size_t m, size_t k, size_t n, const float* lhs, const void* rhs_t, float* dst,
                       int order) {
    return matmul(dtype, m, k, n, lhs, rhs_t, dst, order);
}
ORC_API void orc_softmax_last_dim(const float* x, size_t rows, size_t cols, float* out) {
    for (size_t r = 0; r < rows; ++r) softmax_row(x + r * cols, cols, out + r * cols);
}
ORC_API void orc_silu(const float* x, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = silu_f(x[i]);
}
ORC_API void orc_sigmoid(const float* x, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = sigmoid_f(x[i]);
}
// candle-core/src/cpu_backend/mod.rs:675-738, dim = 0: dst[ids[i]] += src[i] in id order
ORC_API int orc_index_add_dim0(float* dst, size_t dst_rows, size_t cols, const uint32_t* ids, size_t n_ids,
                               const float* src) {
    for (size_t i = 0; i < n_ids; ++i) {
        if (ids[i] == 0xFFFFFFFFu) continue;
        if (ids[i] >= dst_rows) return -1;
        for (size_t c = 0; c < cols; ++c) dst[(size_t)ids[i] * cols + c] += src[i * cols + c];
    }
    return 0;
}
// candle-core/tests/quantized_tests.rs:428-433
ORC_API void orc_ggml_like_vector(float offset, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = 0.1f + 2.0f * std::cos((float)i + offset);
}

// Router: logits = x . Wg^T (+ bias), softmax over all experts, stable descending top-k, optional
// renormalisation of the selected weights.  candle-transformers/src/models/quantized_llama.rs:153-179
// (renorm = 1) and qwen2_moe.rs:262-293 with norm_topk_prob = false (renorm = 0).
//   probs    [T,E]  full softmax
//   topk_ids [T,k]  expert ids in rank order
//   topk_w   [T,k]  routing weight of each selected expert
ORC_API int orc_router_topk(const float* x, const float* wg, const float* bias, size_t T, size_t d, size_t E,
                            size_t k, int renorm, float* probs, uint32_t* topk_ids, float* topk_w) {
    if (k > E) return -1;
#pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)T; ++t) {
        std::vector<float> logits(E);
        for (size_t e = 0; e < E; ++e) {
            float v = vec_dot_f32(x + (size_t)t * d, wg + e * d, d);
            if (bias) v += bias[e];
            logits[e] = v;
        }
        float* p = probs + (size_t)t * E;
        softmax_row(logits.data(), E, p);
        std::vector<uint32_t> idx(E);
        for (size_t e = 0; e < E; ++e) idx[e] = (uint32_t)e;
        std::stable_sort(idx.begin(), idx.end(),
                         [&](uint32_t i, uint32_t j) { return total_order_key(p[j]) < total_order_key(p[i]); });
        float sum = 0.f;
        for (size_t r = 0; r < k; ++r) sum += p[idx[r]];
        for (size_t r = 0; r < k; ++r) {
            topk_ids[(size_t)t * k + r] = idx[r];
            topk_w[(size_t)t * k + r] = renorm ? p[idx[r]] / sum : p[idx[r]];
        }
    }
    return 0;
}

struct OrcMoeWeights {
    int32_t d_model, d_ff, n_experts, top_k;
    int32_t renorm;          // 1: quantized_llama.rs:170-178; 0: qwen2_moe.rs norm_topk_prob=false
    int32_t dtype_w13;       // GGML id of w1 / w3
    int32_t dtype_w2;        // GGML id of w2
    int32_t d_ff_shared;     // 0 = no shared expert
    int32_t dtype_shared13, dtype_shared2;
    int32_t order;           // vec_dot summation order (ORDER_*)
    int32_t _pad;
    const float* router;     // [E, d] f32
    const float* router_bias;  // [E] or null (added to the logits before softmax)
    const void* const* w1;   // E pointers, each [ff, d] blocks
    const void* const* w3;   // E pointers, each [ff, d] blocks
    const void* const* w2;   // E pointers, each [d, ff] blocks
    const void* sw1;         // shared expert [ff_s, d]
    const void* sw3;
    const void* sw2;         // [d, ff_s]
    const float* shared_gate;  // [d] f32
};

namespace {
// quantized_llama.rs:124-131
void mlp_forward(int dt13, int dt2, size_t rows, size_t d, size_t ff, const float* x, const void* w1,
                 const void* w3, const void* w2, float* out, int order, float* hidden_out) {
    std::vector<float> a(rows * ff), b(rows * ff);
    matmul(dt13, rows, d, ff, x, w1, a.data(), order);
    matmul(dt13, rows, d, ff, x, w3, b.data(), order);
    for (size_t i = 0; i < rows * ff; ++i) a[i] = silu_f(a[i]) * b[i];
    if (hidden_out) std::memcpy(hidden_out, a.data(), rows * ff * sizeof(float));
    matmul(dt2, rows, ff, d, a.data(), w2, out, order);
}
}  // namespace

// The whole block, quantized_llama.rs:143-210 (and qwen2_moe.rs:261-323 when a shared expert is
// present).  Optional outputs (may be null):
//   topk_ids/topk_w [T,k]; expert_counts [E]; expert_rows [T*k] = concatenation over experts (in
//   index order) of each expert's token list, which is ascending by construction.
ORC_API int orc_moe_forward(const OrcMoeWeights* w, const float* x, size_t T, float* y, uint32_t* topk_ids,
                            float* topk_w, uint32_t* expert_counts, uint32_t* expert_rows) {
    const size_t d = w->d_model, ff = w->d_ff, E = w->n_experts, k = w->top_k;
    std::vector<float> probs(T * E), tw(T * k);
    std::vector<uint32_t> ids(T * k);
    int rc = orc_router_topk(x, w->router, w->router_bias, T, d, E, k, w->renorm, probs.data(), ids.data(), tw.data());
    if (rc) return rc;
    std::vector<std::vector<uint32_t>> top_x(E);
    std::vector<std::vector<float>> sel(E);
    for (size_t t = 0; t < T; ++t)
        for (size_t r = 0; r < k; ++r) {
            top_x[ids[t * k + r]].push_back((uint32_t)t);
            sel[ids[t * k + r]].push_back(tw[t * k + r]);
        }
    std::memset(y, 0, T * d * sizeof(float));
    size_t pos = 0;
    for (size_t e = 0; e < E; ++e) {
        const size_t ne = top_x[e].size();
        if (expert_counts) expert_counts[e] = (uint32_t)ne;
        if (expert_rows)
            for (size_t i = 0; i < ne; ++i) expert_rows[pos + i] = top_x[e][i];
        pos += ne;
        if (ne == 0) continue;
        std::vector<float> cur(ne * d), out(ne * d);
        for (size_t i = 0; i < ne; ++i) std::memcpy(&cur[i * d], x + (size_t)top_x[e][i] * d, d * sizeof(float));
        mlp_forward(w->dtype_w13, w->dtype_w2, ne, d, ff, cur.data(), w->w1[e], w->w3[e], w->w2[e], out.data(),
                    w->order, nullptr);
        for (size_t i = 0; i < ne; ++i) {
            const float rw = sel[e][i];
            float* dst = y + (size_t)top_x[e][i] * d;
            for (size_t c = 0; c < d; ++c) dst[c] += out[i * d + c] * rw;
        }
    }
    if (w->d_ff_shared > 0) {  // qwen2_moe.rs:315-319
        std::vector<float> so(T * d);
        mlp_forward(w->dtype_shared13, w->dtype_shared2, T, d, w->d_ff_shared, x, w->sw1, w->sw3, w->sw2, so.data(),
                    w->order, nullptr);
        for (size_t t = 0; t < T; ++t) {
            const float g = sigmoid_f(vec_dot_f32(x + t * d, w->shared_gate, d));
            for (size_t c = 0; c < d; ++c) y[t * d + c] = y[t * d + c] + so[t * d + c] * g;
        }
    }
    if (topk_ids) std::memcpy(topk_ids, ids.data(), ids.size() * sizeof(uint32_t));
    if (topk_w) std::memcpy(topk_w, tw.data(), tw.size() * sizeof(float));
    return 0;
}

// One expert (Mlp::forward), with the f32 hidden activations exposed for kernel-level checks.
ORC_API int orc_mlp_forward(int dt13, int dt2, size_t rows, size_t d, size_t ff, const float* x, const void* w1,
                            const void* w3, const void* w2, float* out, float* hidden, int order) {
    mlp_forward(dt13, dt2, rows, d, ff, x, w1, w3, w2, out, order, hidden);
    return 0;
}
