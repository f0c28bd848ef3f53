// Device-side weight quantizer and dequantizer for Q8_0 / Q4_K / Q6_K.
//
// Bit-exact with the reference's CPU `from_float` (candle-core/src/quantized/k_quants.rs:605-634,
// 1287-1345, 1675-1744 with the helpers of utils.rs:62-259), which is an older ggml search
// (make_qkx1_quants / make_qx_quants), so that tensors quantized on the device hold the same bytes
// as tensors quantized by candle on the host.  To that end this file is compiled with -fmad=false
// (the reference never contracts a*b+c), divisions are IEEE, roundf rounds half away from zero like
// f32::round, float->int conversions saturate like Rust's `as`, and f16 conversion is
// round-to-nearest-even.  The searches are serial per block; one thread handles one sub-block
// search, one warp (Q4_K: 8 lanes, Q6_K: 16 lanes active) one 256-element block.
#include "common.cuh"

namespace cmoe {

__device__ __forceinline__ int nearest_int(float v) { return (int)roundf(v); }  // cvt saturates, NaN -> 0

// utils.rs:202-259
__device__ void make_qkx1_quants(int nmax, int ntry, const float* x, float& out_scale, float& out_min) {
    uint8_t l[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) l[i] = 0;
    float mn = x[0], mx = x[0];
    for (int i = 1; i < 32; ++i) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
    }
    if (mx == mn) {
        out_scale = 0.f;
        out_min = 0.f;
        return;
    }
    float minv = fminf(mn, 0.f);
    float iscale = (float)nmax / (mx - minv);
    float scale = 1.0f / iscale;
    for (int t = 0; t < ntry; ++t) {
        float sumlx = 0.f;
        int suml2 = 0;
        bool did_change = false;
        for (int i = 0; i < 32; ++i) {
            int li = nearest_int(iscale * (x[i] - minv));
            li = min(max(li, 0), nmax);
            if ((uint8_t)li != l[i]) {
                l[i] = (uint8_t)li;
                did_change = true;
            }
            sumlx += (x[i] - minv) * (float)li;
            suml2 += li * li;
        }
        scale = sumlx / (float)suml2;
        float sum = 0.f;
        for (int i = 0; i < 32; ++i) sum += x[i] - scale * (float)l[i];
        minv = sum / 32.0f;
        if (minv > 0.f) minv = 0.f;
        iscale = 1.0f / scale;
        if (!did_change) break;
    }
    out_scale = scale;
    out_min = -minv;
}

// utils.rs:62-199 with rmse_type = 1, n = 16
__device__ float make_qx_quants_rmse1(int nmax, const float* x, int8_t* ls) {
    const int n = 16;
    float mx = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) {
        const float ax = fabsf(x[i]);
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
        int l = nearest_int(iscale * x[i]);
        l = min(max(l, -nmax), nmax - 1);
        ls[i] = (int8_t)(l + nmax);
        const float w = x[i] * x[i];
        const float lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = sumlx / suml2;
    float best = scale * sumlx;
    for (int itry = 0; itry < 3; ++itry) {
        const float is2 = 1.0f / scale;
        float slx = 0.f, sl2 = 0.f;
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(is2 * x[i]);
            l = min(max(l, -nmax), nmax - 1);
            if (l + nmax != (int)ls[i]) changed = true;
            const float w = x[i] * x[i];
            const float lf = (float)l;
            slx += w * x[i] * lf;
            sl2 += w * lf * lf;
        }
        if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) {
            const int l = nearest_int(is2 * x[i]);
            ls[i] = (int8_t)(nmax + min(max(l, -nmax), nmax - 1));
        }
        sumlx = slx;
        suml2 = sl2;
        scale = sumlx / suml2;
        best = scale * sumlx;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float w = x[i] * x[i];
            const int l = (int)ls[i] - nmax;
            float slx = sumlx - w * x[i] * (float)l;
            if (slx > 0.f) {
                float sl2 = suml2 - w * (float)l * (float)l;
                int new_l = nearest_int(x[i] * sl2 / slx);
                new_l = min(max(new_l, -nmax), nmax - 1);
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
    return scale;
}

// k_quants.rs:605-634: one thread per 32-element block
__global__ void quantize_w_q8_0_kernel(const float* __restrict__ x, int64_t n_blocks, uint8_t* __restrict__ dst) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float* xs = x + b * 32;
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(xs[j]));
    const float d = amax / 127.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    uint8_t* o = dst + b * Q8_0_BYTES;
    *reinterpret_cast<__half*>(o) = __float2half_rn(d);
    for (int j = 0; j < 32; ++j) {
        const float r = roundf(xs[j] * id);
        o[2 + j] = (uint8_t)(int8_t)(int)fmaxf(fminf(r, 127.f), -128.f);
    }
}

// k_quants.rs:1287-1345: 8 threads per block (one per 32-element sub-block), 4 blocks per warp
__global__ void __launch_bounds__(128)
quantize_w_q4k_kernel(const float* __restrict__ x, int64_t n_blocks, uint8_t* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const int j = lane & 7;
    const int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const bool live = b < n_blocks;
    float xs[32];
    float scale = 0.f, mn = 0.f;
    if (live) {
        const float4* src = reinterpret_cast<const float4*>(x + b * 256 + 32 * j);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = src[i];
            xs[4 * i] = v.x; xs[4 * i + 1] = v.y; xs[4 * i + 2] = v.z; xs[4 * i + 3] = v.w;
        }
        make_qkx1_quants(15, 5, xs, scale, mn);
    }
    // max over the 8 sub-blocks, folded with 0 (f32::max ignores NaN like fmaxf)
    float max_scale = fmaxf(scale, 0.f), max_min = fmaxf(mn, 0.f);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, o));
        max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, o));
    }
    const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
    const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
    const int ls = (uint8_t)min(nearest_int(inv_scale * scale), 63);
    const int lm = (uint8_t)min(nearest_int(inv_min * mn), 63);
    const __half dh = __float2half_rn(max_scale / 63.0f), dmh = __float2half_rn(max_min / 63.0f);
    // the sub-block is re-quantized against the 6-bit values it will be decoded with (ls, lm)
    const float d = __half2float(dh) * (float)ls;
    uint8_t L[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) L[i] = 0;
    if (live && d != 0.f) {
        const float dm = __half2float(dmh) * (float)lm;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int lv = nearest_int((xs[i] + dm) / d);
            L[i] = (uint8_t)min(max(lv, 0), 15);
        }
    }
    // pack: scales bytes need (ls, lm) of sub-blocks j and j +- 4; nibbles pair sub-block 2g with 2g+1
    const int base = lane & ~7;
    const int ls_p4 = __shfl_sync(0xffffffffu, ls, base + ((j + 4) & 7));
    const int lm_p4 = __shfl_sync(0xffffffffu, lm, base + ((j + 4) & 7));
    uint8_t* o = dst + (live ? b : 0) * Q4K_BYTES;
    if (live) {
        if (j < 4) {
            // scales[j] = ls_j | (ls_{j+4} >> 4) << 6 ; scales[j+4] = lm_j | (lm_{j+4} >> 4) << 6
            o[4 + j] = (uint8_t)(ls | ((ls_p4 >> 4) << 6));
            o[4 + j + 4] = (uint8_t)(lm | ((lm_p4 >> 4) << 6));
        } else {
            o[4 + j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
        }
        if (j == 0) {
            *reinterpret_cast<__half*>(o) = dh;
            *reinterpret_cast<__half*>(o + 2) = dmh;
        }
    }
    // nibble packing: even sub-block holds the low nibbles; fetch the partner's L through shuffles
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const uint32_t mine = (uint32_t)L[i] | ((uint32_t)L[i + 1] << 8) | ((uint32_t)L[i + 2] << 16) |
                              ((uint32_t)L[i + 3] << 24);
        const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 1);
        if (live && (j & 1) == 0)
            *reinterpret_cast<uint32_t*>(o + 16 + 32 * (j >> 1) + i) = mine | (other << 4);
    }
}

// k_quants.rs:1675-1744: 16 threads per block (one per 16-element sub-block), 2 blocks per warp
__global__ void __launch_bounds__(128)
quantize_w_q6k_kernel(const float* __restrict__ x, int64_t n_blocks, uint8_t* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const int j = lane & 15;
    const int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const bool live = b < n_blocks;
    float xs[16];
    int8_t L[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) L[i] = 0;
    float scale = 0.f;
    if (live) {
        const float4* src = reinterpret_cast<const float4*>(x + b * 256 + 16 * j);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = src[i];
            xs[4 * i] = v.x; xs[4 * i + 1] = v.y; xs[4 * i + 2] = v.z; xs[4 * i + 3] = v.w;
        }
        scale = make_qx_quants_rmse1(32, xs, L);
    }
    // the scale of largest magnitude, first one on ties (strict > while scanning j upwards)
    float best_abs = fabsf(scale), best = scale;
    int best_j = j;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, best_abs, o);
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oj = __shfl_xor_sync(0xffffffffu, best_j, o);
        if (oa > best_abs || (oa == best_abs && oj < best_j)) {
            best_abs = oa;
            best = ob;
            best_j = oj;
        }
    }
    // reference: max_abs_scale starts at 0 with strict >, so an all-zero block keeps max_scale = 0
    const float max_scale = best_abs > 0.f ? best : 0.f;
    const float iscale = -128.0f / max_scale;
    const __half dh = __float2half_rn(1.0f / iscale);
    const int sc = (int)(int8_t)min(nearest_int(iscale * scale), 127);
    const float d = __half2float(dh) * (float)sc;
    if (live && d != 0.f) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int ll = nearest_int(xs[i] / d);
            ll = min(max(ll, -32), 31);
            L[i] = (int8_t)(ll + 32);
        }
    }
    uint8_t* o = dst + (live ? b : 0) * Q6K_BYTES;
    if (live) {
        o[192 + j] = (uint8_t)(int8_t)sc;
        if (j == 0) *reinterpret_cast<__half*>(o + 208) = dh;
    }
    // pack.  Sub-block j covers elements 16j..16j+15 of the block; within a 128-element half the
    // four 32-element quarters c = 0..3 share bytes: ql[l] = q(c0)|q(c2)<<4, ql[l+32] = q(c1)|q(c3)<<4,
    // qh[l] = hi2(c0) | hi2(c1)<<2 | hi2(c2)<<4 | hi2(c3)<<6, l = 0..31.  Lane j holds quarter
    // c = (j & 7) >> 1, l-range 16*(j&1)..+16; its partners are lanes j ^ 2, j ^ 4, j ^ 6.
    const int c = (j & 7) >> 1;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        const uint32_t mine = (uint32_t)(uint8_t)L[i] | ((uint32_t)(uint8_t)L[i + 1] << 8) |
                              ((uint32_t)(uint8_t)L[i + 2] << 16) | ((uint32_t)(uint8_t)L[i + 3] << 24);
        const uint32_t x2 = __shfl_xor_sync(0xffffffffu, mine, 2);  // quarter c ^ 1
        const uint32_t x4 = __shfl_xor_sync(0xffffffffu, mine, 4);  // quarter c ^ 2
        const uint32_t x6 = __shfl_xor_sync(0xffffffffu, mine, 6);  // quarter c ^ 3
        if (!live) continue;
        const int half = j >> 3, loff = 16 * (j & 1) + i;
        if (c == 0) {
            // mine = c0, x2 = c1, x4 = c2, x6 = c3
            const uint32_t lo0 = (mine & 0x0F0F0F0Fu) | ((x4 & 0x0F0F0F0Fu) << 4);
            const uint32_t lo1 = (x2 & 0x0F0F0F0Fu) | ((x6 & 0x0F0F0F0Fu) << 4);
            const uint32_t hi = ((mine >> 4) & 0x03030303u) | (((x2 >> 4) & 0x03030303u) << 2) |
                                (((x4 >> 4) & 0x03030303u) << 4) | (((x6 >> 4) & 0x03030303u) << 6);
            uint8_t* ql = o + 64 * half + loff;
            uint8_t* qh = o + 128 + 32 * half + loff;
#pragma unroll
            for (int bb = 0; bb < 4; ++bb) {  // block base is only 2-byte aligned: byte stores
                ql[bb] = (uint8_t)(lo0 >> (8 * bb));
                ql[32 + bb] = (uint8_t)(lo1 >> (8 * bb));
                qh[bb] = (uint8_t)(hi >> (8 * bb));
            }
        }
    }
}

// GgmlType::to_float, one thread per element
__global__ void dequantize_kernel(int dtype, const uint8_t* __restrict__ blocks, int64_t n, float* __restrict__ dst) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (dtype == CANDLE_GGML_Q8_0) {
        const uint8_t* b = blocks + (i / 32) * Q8_0_BYTES;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b));
        dst[i] = (float)(int8_t)b[2 + (i & 31)] * d;
    } else if (dtype == CANDLE_GGML_Q4K) {
        const uint8_t* b = blocks + (i / 256) * Q4K_BYTES;
        const int e = (int)(i & 255), j = e >> 5, g = e >> 6, l = e & 31;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b));
        const float mn = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b + 2));
        int sc, m;
        q4k_scale_min(j, b + 4, sc, m);
        const int q = (j & 1) ? (b[16 + 32 * g + l] >> 4) : (b[16 + 32 * g + l] & 0xF);
        dst[i] = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(mn, (float)m));
    } else {
        const uint8_t* b = blocks + (i / 256) * Q6K_BYTES;
        const int e = (int)(i & 255), h = e >> 7, c = (e & 127) >> 5, l = e & 31;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b + 208));
        const int lo = b[64 * h + 32 * (c & 1) + l];
        const int hb = b[128 + 32 * h + l];
        const int q = (((c >> 1) ? (lo >> 4) : (lo & 0xF)) | (((hb >> (2 * c)) & 3) << 4)) - 32;
        const int sc = (int)(int8_t)b[192 + 8 * h + (l >> 4) + 2 * c];
        dst[i] = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    }
}

cudaError_t launch_quantize_weights(cudaStream_t st, int dtype, const float* src, int64_t n, void* dst) {
    if (n == 0) return cudaSuccess;
    uint8_t* o = static_cast<uint8_t*>(dst);
    if (dtype == CANDLE_GGML_Q8_0) {
        const int64_t nb = n / 32;
        quantize_w_q8_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(src, nb, o);
    } else if (dtype == CANDLE_GGML_Q4K) {
        const int64_t nb = n / 256;
        quantize_w_q4k_kernel<<<(unsigned)((nb * 8 + 127) / 128), 128, 0, st>>>(src, nb, o);
    } else if (dtype == CANDLE_GGML_Q6K) {
        const int64_t nb = n / 256;
        quantize_w_q6k_kernel<<<(unsigned)((nb * 16 + 127) / 128), 128, 0, st>>>(src, nb, o);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_dequantize(cudaStream_t st, int dtype, const void* blocks, int64_t n, float* dst) {
    if (n == 0) return cudaSuccess;
    dequantize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dtype, static_cast<const uint8_t*>(blocks), n, dst);
    return cudaGetLastError();
}

}  // namespace cmoe
