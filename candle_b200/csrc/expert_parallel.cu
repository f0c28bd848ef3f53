// Expert parallelism: the data movement either side of the all-to-all of permuted token rows.
//
// The reference runs every expert on the device that holds the block (quantized_llama.rs:185-203).
// With the experts sharded over ranks (rank r owns experts [r * E/N, (r + 1) * E/N)) the grouped rows of
// a rank's tokens are already ordered by destination rank, because the dispatch orders them by expert id.
// What travels is the QUANTIZED activation row -- the int8 values, block sums and block scales that
// `VecDotType::from_float` (k_quants.rs:1898-1902) would produce on the receiving side anyway -- so the
// results are those of the single-device block bit for bit, at 29 % of the bytes of the f32 row.
//
//   pack     grouped position p of the sender -> one packed row [int8 q | int16 bsums | f32 scales | pad]
//   regroup  received rows (source-major, expert-minor) -> planar activation arrays in expert-major
//            order (what the grouped expert kernels read), expert offsets, and the way back
//   scatter  expert outputs (K-split partials summed here) -> rows in received order, ready to return
// The collectives themselves (counts, rows, results) are issued between these steps: by candle_moe_ep_forward
// (ep_nccl.cu), or by a host that drives the steps itself.
#include "common.cuh"

namespace cmoe {

size_t ep_row_bytes(int d) { return align_up((size_t)d + (size_t)d / 8 + (size_t)d / 64, 16); }

namespace {

// one warp per grouped position
__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint32_t* __restrict__ row_of, int64_t n_rows, int d, const int8_t* __restrict__ xq,
               const float* __restrict__ xs, const int16_t* __restrict__ xb, uint8_t* __restrict__ send, int row_bytes) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (p >= n_rows) return;
    const int64_t row = row_of ? (int64_t)row_of[p] : p;
    uint8_t* dst = send + p * row_bytes;
    const uint4* q = reinterpret_cast<const uint4*>(xq + row * d);
    for (int i = lane; i < d / 16; i += 32) reinterpret_cast<uint4*>(dst)[i] = q[i];
    const uint32_t* b = reinterpret_cast<const uint32_t*>(xb + row * (d / 16));
    for (int i = lane; i < d / 32; i += 32) reinterpret_cast<uint32_t*>(dst + d)[i] = b[i];
    const float* s = xs + row * (d / 256);
    for (int i = lane; i < d / 256; i += 32) reinterpret_cast<float*>(dst + d + d / 8)[i] = s[i];
}

// counts[src][e] -> in_base[src][e] (first received row of that group), out_base[src][e] (its first
// expert-major position), offsets[e]; one CTA, n_src * E <= 1024 entries
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const uint32_t* __restrict__ counts, int n_src, int E, uint32_t* __restrict__ in_base,
               uint32_t* __restrict__ out_base, uint32_t* __restrict__ offsets) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t s_cnt[1024], s_eoff[CANDLE_MOE_MAX_EXPERTS + 1];
    const int n = n_src * E;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s_cnt[i] = counts[i];
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (int e = 0; e < E; ++e) {
            s_eoff[e] = run;
            for (int s = 0; s < n_src; ++s) run += s_cnt[s * E + e];
        }
        s_eoff[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_eoff[e];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int s = i / E, e = i - s * E;
        uint32_t ib = 0, ob = s_eoff[e];
        for (int j = 0; j < i; ++j) ib += s_cnt[j];            // rows before group (s, e) in arrival order
        for (int s2 = 0; s2 < s; ++s2) ob += s_cnt[s2 * E + e];  // rows of expert e from earlier sources
        in_base[i] = ib;
        out_base[i] = ob;
    }
}

// one warp per received row: unpack into the planar arrays at its expert-major position
__global__ void __launch_bounds__(256)
ep_regroup_kernel(const uint8_t* __restrict__ recv, int64_t n_rows, int d, int row_bytes, const uint32_t* __restrict__ counts,
                  const uint32_t* __restrict__ in_base, const uint32_t* __restrict__ out_base, int n_groups,
                  int8_t* __restrict__ xq, float* __restrict__ xs, int16_t* __restrict__ xb, uint32_t* __restrict__ back_index) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    // the last group whose first row is <= row and that is not empty
    int lo = 0, hi = n_groups - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (in_base[mid] <= (uint32_t)row) lo = mid; else hi = mid - 1;
    }
    while (lo > 0 && counts[lo] == 0) --lo;  // empty groups share their successor's base
    const int64_t p = (int64_t)out_base[lo] + (row - in_base[lo]);
    const uint8_t* src = recv + row * row_bytes;
    uint4* q = reinterpret_cast<uint4*>(xq + p * d);
    for (int i = lane; i < d / 16; i += 32) q[i] = reinterpret_cast<const uint4*>(src)[i];
    uint32_t* b = reinterpret_cast<uint32_t*>(xb + p * (d / 16));
    for (int i = lane; i < d / 32; i += 32) b[i] = reinterpret_cast<const uint32_t*>(src + d)[i];
    float* s = xs + p * (d / 256);
    for (int i = lane; i < d / 256; i += 32) s[i] = reinterpret_cast<const float*>(src + d + d / 8)[i];
    if (lane == 0) back_index[p] = (uint32_t)row;
}

// out[back_index[p]] = sum over the K-split partials of expert output row p, in split order
__global__ void __launch_bounds__(256)
ep_scatter_kernel(const float* __restrict__ eo, int n_splits, int64_t split_stride, const uint32_t* __restrict__ back_index,
                  int64_t n_rows, int d, float* __restrict__ out, const uint32_t* __restrict__ row_limit) {
    pdl_trigger();
    pdl_wait();
    const int64_t p = blockIdx.x;
    if (p >= n_rows || (row_limit && p >= (int64_t)*row_limit)) return;
    const int64_t r = back_index ? (int64_t)back_index[p] : p;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        float4 a = reinterpret_cast<const float4*>(eo + p * d)[i];
        for (int s = 1; s < n_splits; ++s) {
            const float4 b = reinterpret_cast<const float4*>(eo + s * split_stride + p * d)[i];
            a.x = __fadd_rn(a.x, b.x);
            a.y = __fadd_rn(a.y, b.y);
            a.z = __fadd_rn(a.z, b.z);
            a.w = __fadd_rn(a.w, b.w);
        }
        reinterpret_cast<float4*>(out + r * d)[i] = a;
    }
}

}  // namespace

cudaError_t launch_ep_pack(cudaStream_t st, const uint32_t* row_of, int64_t n_rows, int d, const int8_t* xq, const float* xs,
                           const int16_t* xb, void* send) {
    if (n_rows == 0) return cudaSuccess;
    return launch_k(ep_pack_kernel, dim3((unsigned)((n_rows + 7) / 8)), dim3(256), 0, st, row_of, n_rows, d, xq, xs, xb,
                    static_cast<uint8_t*>(send), (int)ep_row_bytes(d));
}

// plan: uint32 scratch of 2 * n_src * E entries (in_base, out_base)
cudaError_t launch_ep_regroup(cudaStream_t st, const void* recv, const uint32_t* counts, int n_src, int E, int64_t n_rows, int d,
                              uint32_t* plan, int8_t* xq, float* xs, int16_t* xb, uint32_t* offsets, uint32_t* back_index) {
    const int n = n_src * E;
    if (n <= 0 || n > 1024) return cudaErrorInvalidValue;
    cudaError_t e = launch_k(ep_plan_kernel, dim3(1), dim3(1024), 0, st, counts, n_src, E, plan, plan + n, offsets);
    if (e != cudaSuccess || n_rows == 0) return e;
    return launch_k(ep_regroup_kernel, dim3((unsigned)((n_rows + 7) / 8)), dim3(256), 0, st, static_cast<const uint8_t*>(recv),
                    n_rows, d, (int)ep_row_bytes(d), counts, (const uint32_t*)plan, (const uint32_t*)(plan + n), n, xq, xs, xb,
                    back_index);
}

cudaError_t launch_ep_scatter(cudaStream_t st, const float* eo, int n_splits, int64_t split_stride, const uint32_t* back_index,
                              int64_t n_rows, int d, float* out, const uint32_t* row_limit) {
    if (n_rows == 0) return cudaSuccess;
    return launch_k(ep_scatter_kernel, dim3((unsigned)n_rows), dim3(256), 0, st, eo, n_splits, split_stride, back_index, n_rows,
                    d, out, row_limit);
}

}  // namespace cmoe
