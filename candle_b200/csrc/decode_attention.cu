// Attention for one new token per sequence over an f32 KV cache: the `standard_attention` of
// candle-transformers' quantized_llama (quantized_llama.rs:303-317) at seq_len = 1 --
//     att = softmax(q . K^T / sqrt(head_dim)),  y = att . V
// with `repeat_kv` (utils.rs repeat_kv: query head h reads kv head h / (n_head / n_kv_head)) folded into the
// indexing instead of materialised.  A decode step at batch 32 and a 4096-token context reads 1 GB of cache per
// layer, so the kernel is a streaming one: every (sequence, kv head) pair is cut into chunks of the context, a CTA
// reads its chunk of K once for all the query heads of the group, keeps the scores in shared memory, then reads its
// chunk of V once; a second small kernel merges the chunks' partial softmax sums (the usual split-softmax algebra:
// only the order of f32 additions differs from a one-pass softmax).  f32 throughout, like the reference.
#include "common.cuh"

namespace cmoe {

namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_MAX_GROUP = 8;    // query heads per kv head
constexpr int ATT_CHUNK = 512;      // context positions per CTA

// Sum of G per-lane values over the 32 lanes of a warp.  For G = 4 the four sums are folded as they travel (two
// exchange steps halve the values a lane carries, then three ordinary steps): 6 shuffles instead of 20; lane 8 h
// ends up with the sum of head h.  Other group sizes use the plain butterfly (every lane gets every sum).
template <int G>
__device__ __forceinline__ void warp_sum_heads(float (&acc)[G], int lane, float (&out)[G], bool& owner, int& head) {
    if constexpr (G == 4) {
        const bool hi16 = lane & 16, hi8 = lane & 8;
        const float r0 = __shfl_xor_sync(0xffffffffu, hi16 ? acc[0] : acc[2], 16);
        const float r1 = __shfl_xor_sync(0xffffffffu, hi16 ? acc[1] : acc[3], 16);
        const float k0 = (hi16 ? acc[2] : acc[0]) + r0, k1 = (hi16 ? acc[3] : acc[1]) + r1;
        const float r = __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8);
        float v = (hi8 ? k1 : k0) + r;
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        out[0] = v;
        owner = (lane & 7) == 0;
        head = (hi16 ? 2 : 0) + (hi8 ? 1 : 0);
    } else {
#pragma unroll
        for (int g = 0; g < G; ++g) out[g] = warp_sum(acc[g]);
        owner = lane == 0;
        head = -1;  // lane 0 holds all of them
    }
}

// partial[(((b * n_kv + kv) * n_chunks + c) * G + g) * (D + 2)]: chunk maximum, sum of exponentials, D weighted sums
template <int D, int G>
__global__ void __launch_bounds__(ATT_THREADS)
decode_attention_chunk_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc, int n_kv,
                              int64_t max_seq, int n_ctx, float scale, int n_chunks, float* __restrict__ partial) {
    pdl_trigger();
    pdl_wait();
    constexpr int WARPS = ATT_THREADS / 32;
    __shared__ float s_q[G][D];
    __shared__ __align__(16) float s_score[ATT_CHUNK][G];  // a position's G scores side by side: one vector load in the V pass
    __shared__ __align__(16) float s_o[WARPS / 2][G][D];
    __shared__ float s_red[G][WARPS];
    __shared__ float s_max[G], s_sum[G];
    const int c = blockIdx.x, kv = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p0 = c * ATT_CHUNK, p1 = min(n_ctx, p0 + ATT_CHUNK), np = p1 - p0;
    const int n_head = n_kv * G;
    for (int i = tid; i < G * D; i += ATT_THREADS) s_q[i / D][i % D] = q[((int64_t)b * n_head + kv * G + i / D) * D + i % D];
    __syncthreads();
    const float* kbase = kc + (((int64_t)b * n_kv + kv) * max_seq + p0) * D;
    const float* vbase = vc + (((int64_t)b * n_kv + kv) * max_seq + p0) * D;

    // ---- scores: one warp per position, a lane holds D / 32 consecutive elements of the row ----
    constexpr int PER = D / 32;
    float qr[G][PER];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < PER; ++i) qr[g][i] = s_q[g][lane * PER + i];
#pragma unroll 4
    for (int p = warp; p < np; p += WARPS) {
        float kr[PER];
        if (PER == 4) {
            const float4 v4 = reinterpret_cast<const float4*>(kbase + (int64_t)p * D)[lane];
            kr[0] = v4.x; kr[1] = v4.y; kr[2] = v4.z; kr[3] = v4.w;
        } else {
            const float2 v2 = reinterpret_cast<const float2*>(kbase + (int64_t)p * D)[lane];
            kr[0] = v2.x; kr[PER - 1] = v2.y;
        }
        float acc[G], sum[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            acc[g] = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) acc[g] = fmaf(qr[g][i], kr[i], acc[g]);
        }
        bool owner;
        int head;
        warp_sum_heads<G>(acc, lane, sum, owner, head);
        if (owner) {
            if (head >= 0) {
                s_score[p][head] = sum[0] * scale;
            } else {
#pragma unroll
                for (int g = 0; g < G; ++g) s_score[p][g] = sum[g] * scale;
            }
        }
    }
    __syncthreads();
    // ---- chunk maximum and sum of exponentials per query head ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float m = -INFINITY;
        for (int p = tid; p < np; p += ATT_THREADS) m = fmaxf(m, s_score[p][g]);
        m = warp_max(m);
        if (lane == 0) s_red[g][warp] = m;
    }
    __syncthreads();
    if (tid < G) {
        float m = -INFINITY;
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, s_red[tid][w]);
        s_max[tid] = m;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float m = s_max[g];
        float s = 0.f;
        for (int p = tid; p < np; p += ATT_THREADS) {
            const float e = expf(s_score[p][g] - m);
            s_score[p][g] = e;
            s += e;
        }
        s = warp_sum(s);
        if (lane == 0) s_red[g][warp] = s;
    }
    __syncthreads();
    if (tid < G) {
        float s = 0.f;
        for (int w = 0; w < WARPS; ++w) s += s_red[tid][w];
        s_sum[tid] = s;
    }
    // ---- weighted sum of V: D / 4 lanes cover a row with 128-bit loads, a warp takes 32 / (D / 4) positions at a time ----
    constexpr int LPP = D / 4, PPW = 32 / LPP;  // lanes per position, positions per warp and step
    const int sub = lane / LPP, l4 = lane % LPP;
    float o[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[g][i] = 0.f;
#pragma unroll 4
    for (int p = warp * PPW + sub; p < np; p += WARPS * PPW) {
        const float4 v = reinterpret_cast<const float4*>(vbase + (int64_t)p * D)[l4];
        float w[G];
        if constexpr (G == 4) {
            const float4 w4 = *reinterpret_cast<const float4*>(&s_score[p][0]);
            w[0] = w4.x; w[1] = w4.y; w[2] = w4.z; w[3] = w4.w;
        } else {
#pragma unroll
            for (int g = 0; g < G; ++g) w[g] = s_score[p][g];
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            o[g][0] = fmaf(w[g], v.x, o[g][0]);
            o[g][1] = fmaf(w[g], v.y, o[g][1]);
            o[g][2] = fmaf(w[g], v.z, o[g][2]);
            o[g][3] = fmaf(w[g], v.w, o[g][3]);
        }
    }
    if (PPW == 2) {  // the two positions a warp handles at a time meet first
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[g][i] += __shfl_xor_sync(0xffffffffu, o[g][i], 16);
    }
    // the warps meet in shared memory, halving the number of partial sums per round (a fixed order)
    for (int half = WARPS / 2; half >= 1; half >>= 1) {
        if (warp >= half && warp < 2 * half && sub == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) *reinterpret_cast<float4*>(&s_o[warp - half][g][4 * l4]) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
        }
        __syncthreads();
        if (warp < half && sub == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 t = *reinterpret_cast<const float4*>(&s_o[warp][g][4 * l4]);
                o[g][0] += t.x; o[g][1] += t.y; o[g][2] += t.z; o[g][3] += t.w;
            }
        }
        __syncthreads();
    }
    if (warp == 0 && sub == 0) {
        float* out = partial + ((((int64_t)b * n_kv + kv) * n_chunks + c) * G) * (D + 2);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            out[g * (D + 2) + 2 + 4 * l4 + 0] = o[g][0];
            out[g * (D + 2) + 2 + 4 * l4 + 1] = o[g][1];
            out[g * (D + 2) + 2 + 4 * l4 + 2] = o[g][2];
            out[g * (D + 2) + 2 + 4 * l4 + 3] = o[g][3];
            if (l4 == 0) {
                out[g * (D + 2)] = s_max[g];
                out[g * (D + 2) + 1] = s_sum[g];
            }
        }
    }
}

// y[b, head, :] = sum_c exp(m_c - M) o_c / sum_c exp(m_c - M) l_c, chunks in order
template <int D, int G>
__global__ void __launch_bounds__(D)
decode_attention_merge_kernel(const float* __restrict__ partial, int n_kv, int n_chunks, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const int head = blockIdx.x, b = blockIdx.y, dim = threadIdx.x;
    const int kv = head / G, g = head % G;
    const float* base = partial + ((((int64_t)b * n_kv + kv) * n_chunks) * G + g) * (D + 2);
    const int64_t stride = (int64_t)G * (D + 2);
    float M = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, base[c * stride]);
    float num = 0.f, den = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
        const float w = expf(base[c * stride] - M);
        den = fmaf(w, base[c * stride + 1], den);
        num = fmaf(w, base[c * stride + 2 + dim], num);
    }
    y[((int64_t)b * n_kv * G + head) * D + dim] = num / den;
}

template <int D, int G>
cudaError_t launch_att(cudaStream_t st, const float* q, const float* kc, const float* vc, int B, int n_kv, int64_t max_seq, int n_ctx,
                       float scale, float* y, float* partial) {
    const int n_chunks = (n_ctx + ATT_CHUNK - 1) / ATT_CHUNK;
    cudaError_t e = launch_k(decode_attention_chunk_kernel<D, G>, dim3(n_chunks, n_kv, B), dim3(ATT_THREADS), 0, st, q, kc, vc, n_kv,
                             max_seq, n_ctx, scale, n_chunks, partial);
    if (e != cudaSuccess) return e;
    return launch_k(decode_attention_merge_kernel<D, G>, dim3(n_kv * G, B), dim3(D), 0, st, (const float*)partial, n_kv, n_chunks, y);
}

}  // namespace

namespace {
// Interleaved rotary embedding of the new token's q and k (`rope_i`, candle-nn/src/rotary_emb.rs:53-66: pairs
// (x[2i], x[2i+1]) rotated by the angle of (position, i), product then difference / sum like the CPU loop) and the
// append of k and v to the f32 cache at that position (candle-nn/src/kv_cache.rs:143-164), in one pass.
// qkv [B, row_stride] holds q (n_head * D), k (n_kv * D), v (n_kv * D) side by side; cos / sin [D / 2] of the position.
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(const float* __restrict__ qkv, int64_t row_stride, const float* __restrict__ cos, const float* __restrict__ sin,
                      int n_head, int n_kv, int D, int64_t max_seq, int pos, float* __restrict__ q_out, float* __restrict__ kc,
                      float* __restrict__ vc) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int half = D / 2, n_q = n_head * half, n_k = n_kv * half;
    const float* row = qkv + (int64_t)b * row_stride;
    for (int i = threadIdx.x; i < n_q + 2 * n_k; i += blockDim.x) {
        if (i < n_q + n_k) {
            const bool is_q = i < n_q;
            const int j = is_q ? i : i - n_q;
            const int h = j / half, ip = j - h * half;
            const float* src = row + (is_q ? 0 : n_head * D) + h * D + 2 * ip;
            const float x0 = src[0], x1 = src[1], c = cos[ip], s = sin[ip];
            const float o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)), o1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
            float* dst = is_q ? q_out + ((int64_t)b * n_head + h) * D + 2 * ip
                              : kc + (((int64_t)b * n_kv + h) * max_seq + pos) * D + 2 * ip;
            dst[0] = o0;
            dst[1] = o1;
        } else {
            const int j = i - n_q - n_k;
            const int h = j / half, ip = j - h * half;
            const float* src = row + (n_head + n_kv) * D + h * D + 2 * ip;
            float* dst = vc + (((int64_t)b * n_kv + h) * max_seq + pos) * D + 2 * ip;
            dst[0] = src[0];
            dst[1] = src[1];
        }
    }
}
}  // namespace

cudaError_t launch_rope_kv_append(cudaStream_t st, const float* qkv, int64_t row_stride, const float* cos, const float* sin, int B,
                                  int n_head, int n_kv, int D, int64_t max_seq, int pos, float* q_out, float* kc, float* vc) {
    if (B == 0) return cudaSuccess;
    return launch_k(rope_kv_append_kernel, dim3(B), dim3(256), 0, st, qkv, row_stride, cos, sin, n_head, n_kv, D, max_seq, pos, q_out,
                    kc, vc);
}

size_t decode_attention_workspace_bytes(int B, int n_head, int head_dim, int n_ctx) {
    const size_t n_chunks = (size_t)(n_ctx + ATT_CHUNK - 1) / ATT_CHUNK;
    return (size_t)B * n_head * n_chunks * (head_dim + 2) * sizeof(float);
}

cudaError_t launch_decode_attention(cudaStream_t st, const float* q, const float* kc, const float* vc, int B, int n_head, int n_kv,
                                    int head_dim, int64_t max_seq, int n_ctx, float scale, float* y, float* workspace) {
    if (B == 0 || n_ctx == 0) return cudaSuccess;
    const int G = n_head / n_kv;
    if (head_dim == 128) {
        if (G == 4) return launch_att<128, 4>(st, q, kc, vc, B, n_kv, max_seq, n_ctx, scale, y, workspace);
        if (G == 1) return launch_att<128, 1>(st, q, kc, vc, B, n_kv, max_seq, n_ctx, scale, y, workspace);
        if (G == 8) return launch_att<128, 8>(st, q, kc, vc, B, n_kv, max_seq, n_ctx, scale, y, workspace);
    }
    if (head_dim == 64) {
        if (G == 4) return launch_att<64, 4>(st, q, kc, vc, B, n_kv, max_seq, n_ctx, scale, y, workspace);
        if (G == 1) return launch_att<64, 1>(st, q, kc, vc, B, n_kv, max_seq, n_ctx, scale, y, workspace);
    }
    return cudaErrorNotSupported;
}

}  // namespace cmoe
