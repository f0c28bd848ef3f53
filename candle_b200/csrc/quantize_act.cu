// Activation quantization: the per-row `VecDotType::from_float` step that k_quants::matmul runs
// before every quantized product (candle-core/src/quantized/k_quants.rs:1898-1902).
//
// The integer values must equal the reference's exactly (the block output tolerance is tighter
// than one quantization step of these activations), so the arithmetic below is IEEE throughout:
// true division, roundf (half away from zero, like Rust's f32::round), no fast-math.
//
// Output is planar so the expert kernels read aligned int8 rows:
//   qs     int8  [rows, k]
//   scales f32   [rows, k / B]   B = 256 (Q8K) or 32 (Q8_0; the f16-rounded scale widened to f32)
//   bsums  int16 [rows, k / 16]  Q8K only
#include "common.cuh"

namespace cmoe {

// BlockQ8K::from_float: one warp per 256-element block (quantize_q8k_block in common.cuh).
__global__ void __launch_bounds__(256)
quantize_q8k_kernel(const float* __restrict__ x, int64_t n_blocks, int8_t* __restrict__ qs,
                    float* __restrict__ scales, int16_t* __restrict__ bsums, const uint32_t* __restrict__ row_limit,
                    int blocks_per_row, uint32_t* __restrict__ single_group, uint32_t group_rows) {
    pdl_trigger();
    pdl_wait();
    if (single_group && blockIdx.x == 0 && threadIdx.x < 2) single_group[threadIdx.x] = threadIdx.x ? group_rows : 0u;
    const int lane = threadIdx.x & 31;
    const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= n_blocks) return;
    // rows past the device-side count hold nothing (expert parallelism sizes its launches by a capacity bound)
    if (row_limit && blk >= (int64_t)*row_limit * blocks_per_row) return;
    quantize_q8k_block(x + blk * QK_K, lane, qs + blk * QK_K, scales + blk, bsums + blk * 16);
}

// BlockQ8_0::from_float (k_quants.rs:605-634).  One warp per 8 blocks of 32: 4 lanes per block,
// 8 elements per lane.  d = amax / 127, the values are rounded with the UNROUNDED 1/d, the stored
// scale is d rounded to f16.
__global__ void __launch_bounds__(256)
quantize_q8_0_kernel(const float* __restrict__ x, int64_t n_elems, int8_t* __restrict__ qs,
                     float* __restrict__ scales, uint32_t* __restrict__ single_group, uint32_t group_rows) {
    pdl_trigger();
    pdl_wait();
    if (single_group && blockIdx.x == 0 && threadIdx.x < 2) single_group[threadIdx.x] = threadIdx.x ? group_rows : 0u;
    const int lane = threadIdx.x & 31;
    const int64_t grp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // 256 elements
    if (grp * 256 >= n_elems) return;
    const bool live = grp * 256 + lane * 8 < n_elems;  // n_elems is a multiple of 32: whole blocks only
    const float4* src = reinterpret_cast<const float4*>(x + grp * 256) + lane * 2;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 a = live ? src[0] : z, b = live ? src[1] : z;
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = amax / 127.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    int q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float r = roundf(v[i] * id);
        q[i] = (int)fmaxf(fminf(r, 127.f), -128.f);
    }
    uint32_t lo = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) |
                  ((uint32_t)(q[3] & 0xff) << 24);
    uint32_t hi = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) |
                  ((uint32_t)(q[7] & 0xff) << 24);
    if (!live) return;
    reinterpret_cast<uint2*>(qs + grp * 256)[lane] = make_uint2(lo, hi);
    if ((lane & 3) == 0) scales[grp * 8 + (lane >> 2)] = __half2float(__float2half_rn(d));
}

// single_group (may be null): two words that receive {0, rows} -- the offsets of one group holding every row, which
// the dense product needs and would otherwise write with a launch of its own
cudaError_t launch_quantize_act(cudaStream_t st, const float* x, int64_t rows, int kdim, int for_dtype, int8_t* qs,
                                float* scales, int16_t* bsums, const uint32_t* row_limit, uint32_t* single_group) {
    const int64_t n = rows * (int64_t)kdim;
    const int64_t n256 = (n + 255) / 256;
    if (n256 == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((n256 + 7) / 8);
    if (for_dtype == CANDLE_GGML_Q8_0)
        return launch_k(quantize_q8_0_kernel, dim3(grid), dim3(256), 0, st, x, n, qs, scales, single_group, (uint32_t)rows);
    return launch_k(quantize_q8k_kernel, dim3(grid), dim3(256), 0, st, x, n256, qs, scales, bsums, row_limit, kdim / 256,
                    single_group, (uint32_t)rows);
}

}  // namespace cmoe
