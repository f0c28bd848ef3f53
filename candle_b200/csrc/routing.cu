// Router (f32 GEMV + softmax + stable top-k), dispatch (group pairs by expert) and the weighted
// combine of the quantized MoE block.  All three are small, latency- or HBM-bound kernels.
#include "common.cuh"

#include <atomic>
#include <cstdlib>

namespace cmoe {

bool pdl_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("CANDLE_MOE_PDL");
        return !(v && v[0] == '0');
    }();
    return on;
}

namespace {
struct TuningTable {
    std::atomic<int64_t> v[TUNE_N_KEYS];
    TuningTable() {
        const auto env = [](const char* name, int64_t dflt) {
            const char* s = std::getenv(name);
            return s && s[0] ? (int64_t)std::atoll(s) : dflt;
        };
        v[TUNE_GEMM_ENABLED] = env("CANDLE_MOE_GEMM", 1);
        v[TUNE_GEMM_MIN_ROWS] = env("CANDLE_MOE_GEMM_MIN_ROWS", 96);
        v[TUNE_STREAM_MAX_ROWS] = env("CANDLE_MOE_STREAM_MAX_ROWS", (int64_t)1 << 40);
        v[TUNE_FORCE_ROWS] = env("CANDLE_MOE_FORCE_ROWS", 0);
        v[TUNE_MID_ENABLED] = env("CANDLE_MOE_MID", 1);
    }
};
TuningTable& tuning_table() {
    static TuningTable t;
    return t;
}
}  // namespace
int64_t tuning_get(int key) { return key >= 0 && key < TUNE_N_KEYS ? tuning_table().v[key].load() : 0; }
bool tuning_set(int key, int64_t value) {
    if (key < 0 || key >= TUNE_N_KEYS) return false;
    tuning_table().v[key].store(value);
    return true;
}

// ------------------------------------------------------------------------------------------------
// Router (+ activation quantization).  One CTA of 1024 threads per token: for d = 4096 every thread
// issues its single 128-bit load of x and its 8 loads of the router rows at once, so the whole
// product costs about one memory latency; partial sums meet through warp shuffles and shared
// memory in a fixed order.  Warp 0 then does the softmax over all E experts and k rounds of arg-max
// with "lower expert id wins a tie", which is what a stable descending sort followed by take(k)
// yields (candle-transformers/src/models/quantized_llama.rs:162-179).  Meanwhile the other warps
// quantize the same row of x the Q8K way for the expert products (one pass over x instead of two
// kernels).  Arithmetic is plain f32 FMA (no TF32): the reference's router product is full f32.
// ------------------------------------------------------------------------------------------------
// Softmax over the E logits of one token and the top-k selection, by one warp (every lane ends up holding the
// selection); writes the token's ids and weights.
__device__ __forceinline__ void softmax_topk_warp(const float* s_logits, int lane, int E, int k, int renorm,
                                                  uint32_t* __restrict__ ids_row, float* __restrict__ w_row,
                                                  float (&sel_p)[CANDLE_MOE_MAX_TOPK], int (&sel_e)[CANDLE_MOE_MAX_TOPK]) {
    // softmax over E (candle-nn/src/ops.rs:326-339): exp(v - max) / sum, true division
    constexpr int PER = CANDLE_MOE_MAX_EXPERTS / 32;
    float p[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        p[j] = e < E ? s_logits[e] : -INFINITY;
        mx = fmaxf(mx, p[j]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        p[j] = e < E ? expf(p[j] - mx) : 0.f;
        s += p[j];
    }
    s = warp_sum(s);
#pragma unroll
    for (int j = 0; j < PER; ++j) p[j] = (lane + 32 * j) < E ? p[j] / s : 0.f;

    // Selection in the order of Rust's f32::total_cmp (the reference sorts with it, quantized_llama.rs:166), so
    // that it is total: a row holding a NaN or an infinity turns every probability into the same NaN, all keys
    // tie, and the lowest expert ids win -- the reference's stable sort gives exactly that.  Every selected id
    // is below E whatever the input holds.
    int key[PER];
    uint32_t open_mask = 0;  // bit j: expert lane + 32 j exists and has not been selected yet
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int b = (p[j] != p[j]) ? 0x7fffffff : __float_as_int(p[j]);  // all NaNs alike (they only occur together)
        key[j] = b ^ (int)(((uint32_t)(b >> 31)) >> 1);
        if (lane + 32 * j < E) open_mask |= 1u << j;
    }
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < CANDLE_MOE_MAX_TOPK; ++r) {
        if (r < k) {
            int bk = 0, be = -1;  // be < 0: no candidate in this lane
            float bv = 0.f;
#pragma unroll
            for (int j = 0; j < PER; ++j) {  // ascending expert id inside a lane: strict > keeps the lower id
                if (((open_mask >> j) & 1u) && (be < 0 || key[j] > bk)) {
                    bk = key[j];
                    bv = p[j];
                    be = lane + 32 * j;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const int ok = __shfl_xor_sync(0xffffffffu, bk, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                if (oe >= 0 && (be < 0 || ok > bk || (ok == bk && oe < be))) {
                    bk = ok;
                    be = oe;
                    bv = ov;
                }
            }
            // k <= E, so a candidate always exists; the clamp only keeps a corrupted launch inside the tables
            be = min(max(be, 0), E - 1);
            sel_p[r] = bv;
            sel_e[r] = be;
            sum += bv;  // rank order, like `sum_routing_weights += routing_weight`
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (lane + 32 * j == be) open_mask &= ~(1u << j);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < CANDLE_MOE_MAX_TOPK; ++r) {
            if (r < k) {
                ids_row[r] = (uint32_t)sel_e[r];
                w_row[r] = renorm ? sel_p[r] / sum : sel_p[r];
            }
        }
    }
}

// Few tokens: 1024 threads per token (the whole product in one round of loads).  Many tokens: 256 threads per token,
// so that eight CTAs share an SM and their load rounds overlap.  The two sizes add the partial sums in different
// orders (last-bit differences of the logits, as between any two f32 dot-product orders).
template <int ROUTER_THREADS>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_topk_kernel(const float* __restrict__ x, const float* __restrict__ wg, const float* __restrict__ bias,
                   int d, int E, int k, int renorm, uint32_t* __restrict__ ids, float* __restrict__ wout,
                   int8_t* __restrict__ qs, float* __restrict__ scales, int16_t* __restrict__ bsums,
                   uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets, uint32_t* __restrict__ perm_token,
                   uint32_t* __restrict__ pair_pos) {
    pdl_trigger();
    pdl_wait();
    constexpr int ROUTER_WARPS = ROUTER_THREADS / 32;
    __shared__ float s_logits[CANDLE_MOE_MAX_EXPERTS];
    __shared__ float s_part[ROUTER_WARPS][8];
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float4* xr = reinterpret_cast<const float4*>(x + t * (int64_t)d);
    const int d4 = d >> 2;

    for (int e0 = 0; e0 < E; e0 += 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int i = tid; i < d4; i += ROUTER_THREADS) {
            const float4 xv = xr[i];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (e0 + j < E) {
                    const float4 wv = reinterpret_cast<const float4*>(wg + (int64_t)(e0 + j) * d)[i];
                    acc[j] = fmaf(xv.x, wv.x, acc[j]);
                    acc[j] = fmaf(xv.y, wv.y, acc[j]);
                    acc[j] = fmaf(xv.z, wv.z, acc[j]);
                    acc[j] = fmaf(xv.w, wv.w, acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0) s_part[warp][j] = v;
        }
        __syncthreads();
        if (tid < 8 && e0 + tid < E) {
            float v = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < ROUTER_WARPS; ++w8) v += s_part[w8][tid];
            if (bias) v += bias[e0 + tid];
            s_logits[e0 + tid] = v;
        }
        __syncthreads();
    }
    if (warp != 0) {
        // warps 1.. quantize the row (each 256-element block by one warp)
        if (qs) {
            const int nb = d >> 8;
            for (int b = warp - 1; b < nb; b += ROUTER_WARPS - 1)
                quantize_q8k_block(x + t * (int64_t)d + b * 256, lane, qs + t * (int64_t)d + b * 256, scales + t * nb + b,
                                   bsums + (t * nb + b) * 16);
        }
        return;
    }

    float sel_p[CANDLE_MOE_MAX_TOPK];
    int sel_e[CANDLE_MOE_MAX_TOPK];
    softmax_topk_warp(s_logits, lane, E, k, renorm, ids + t * k, wout + t * k, sel_p, sel_e);
    // A single token (the step of one-sequence decoding): its k experts are distinct, so the dispatch is their
    // ascending order and needs no pass of its own.  Every lane holds the selection.
    if (counts) {
        for (int e = lane; e < E; e += 32) {
            uint32_t hit = 0, below = 0;
#pragma unroll
            for (int r = 0; r < CANDLE_MOE_MAX_TOPK; ++r) {
                if (r < k) {
                    hit += sel_e[r] == e;
                    below += sel_e[r] < e;
                }
            }
            counts[e] = hit;
            offsets[e] = below;
        }
        if (lane == 0) offsets[E] = (uint32_t)k;
#pragma unroll
        for (int r = 0; r < CANDLE_MOE_MAX_TOPK; ++r) {
            if (r < k && lane == r) {
                uint32_t pos = 0;
#pragma unroll
                for (int r2 = 0; r2 < CANDLE_MOE_MAX_TOPK; ++r2) pos += (r2 < k && sel_e[r2] < sel_e[r]);
                perm_token[pos] = 0u;
                pair_pos[r] = pos;
            }
        }
    }
}

// Many tokens and many experts (prefill of a fine-grained layer): the router product as a tiled f32 GEMM.  The
// one-token kernels spend their time in warp reductions -- one per (token, expert) -- which for 60 experts and 4096
// tokens is most of 0.15 ms.  Here a CTA takes 32 tokens x all experts: x and the router rows pass through shared
// memory in K chunks of 32 (the next chunk is fetched into registers while this one is multiplied), thread (token t,
// group g) accumulates token t against experts g, g + 8, ... in registers with no reduction at all, and the eight
// warps then do the softmax and the selection of four tokens each.  Every logit is a plain sequential f32 sum over K
// (another order than the one-token kernels': last-bit differences, as between any two f32 dot products).  No fused
// quantization: used where the activations are quantized by a pass of their own (Q8_0 experts).  Measured (60
// experts, d = 2048, 4096 tokens): 155 -> 98 us; a variant with 64-wide chunks double-buffered by cp.async took 133 us.
constexpr int RT_TOK = 32, RT_KC = 32, RT_PAD = 36, RT_EPT = CANDLE_MOE_MAX_EXPERTS / 8;
__global__ void __launch_bounds__(256)
router_topk_tiled_kernel(const float* __restrict__ x, const float* __restrict__ wg, const float* __restrict__ bias,
                         int64_t T, int d, int E, int k, int renorm, uint32_t* __restrict__ ids, float* __restrict__ wout) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float s_x[RT_TOK][RT_PAD];
    __shared__ __align__(16) float s_w[CANDLE_MOE_MAX_EXPERTS][RT_PAD];
    __shared__ float s_logits[8][CANDLE_MOE_MAX_EXPERTS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t t0 = (int64_t)blockIdx.x * RT_TOK;
    const int n_ept = (E + 7) / 8;  // experts per thread
    // loads: thread -> (row tid / 8, float4 tid % 8) of the x chunk; the router chunk takes E * 8 float4, tid, tid + 256, ...
    const float4* xsrc = reinterpret_cast<const float4*>(x + min(t0 + (tid >> 3), T - 1) * (int64_t)d) + (tid & 7);
    float acc[RT_EPT];
#pragma unroll
    for (int i = 0; i < RT_EPT; ++i) acc[i] = 0.f;
    const int n_w4 = E * 8;
    float4 px = xsrc[0], pw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int u = tid + 256 * i;
        pw[i] = u < n_w4 ? reinterpret_cast<const float4*>(wg + (int64_t)(u >> 3) * d)[u & 7] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int c = 0; c < d; c += RT_KC) {
        __syncthreads();  // the previous chunk has been consumed
        *reinterpret_cast<float4*>(&s_x[tid >> 3][4 * (tid & 7)]) = px;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int u = tid + 256 * i;
            if (u < n_w4) *reinterpret_cast<float4*>(&s_w[u >> 3][4 * (u & 7)]) = pw[i];
        }
        __syncthreads();
        if (c + RT_KC < d) {  // the next chunk travels while this one is multiplied
            px = xsrc[(c + RT_KC) >> 2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int u = tid + 256 * i;
                if (u < n_w4) pw[i] = reinterpret_cast<const float4*>(wg + (int64_t)(u >> 3) * d + c + RT_KC)[u & 7];
            }
        }
#pragma unroll
        for (int k4 = 0; k4 < RT_KC / 4; ++k4) {
            const float4 xv = *reinterpret_cast<const float4*>(&s_x[lane][4 * k4]);
#pragma unroll
            for (int i = 0; i < RT_EPT; ++i) {
                if (i < n_ept) {
                    const float4 wv = *reinterpret_cast<const float4*>(&s_w[warp + 8 * i][4 * k4]);  // one address per warp
                    acc[i] = fmaf(xv.x, wv.x, acc[i]);
                    acc[i] = fmaf(xv.y, wv.y, acc[i]);
                    acc[i] = fmaf(xv.z, wv.z, acc[i]);
                    acc[i] = fmaf(xv.w, wv.w, acc[i]);
                }
            }
        }
    }
    // four rounds of eight tokens: logits to shared memory, then warp w selects for token 8 * round + w
    for (int round = 0; round < RT_TOK / 8; ++round) {
        __syncthreads();
        if ((lane >> 3) == round) {  // this thread's token is lane: tokens 8 round .. 8 round + 7 in this round
#pragma unroll
            for (int i = 0; i < RT_EPT; ++i) {
                const int e = warp + 8 * i;
                if (i < n_ept && e < E) s_logits[lane & 7][e] = acc[i] + (bias ? bias[e] : 0.f);
            }
        }
        __syncthreads();
        const int64_t t = t0 + 8 * round + warp;
        if (t < T) {
            float sel_p[CANDLE_MOE_MAX_TOPK];
            int sel_e[CANDLE_MOE_MAX_TOPK];
            softmax_topk_warp(s_logits[warp], lane, E, k, renorm, ids + t * k, wout + t * k, sel_p, sel_e);
        }
    }
}

cudaError_t launch_router_topk(cudaStream_t st, const float* x, const float* router, const float* bias, int64_t T,
                               int d, int E, int k, int renorm, uint32_t* ids, float* w, int8_t* qs, float* scales,
                               int16_t* bsums, uint32_t* counts, uint32_t* offsets, uint32_t* perm_token, uint32_t* pair_pos) {
    if (T == 0) return cudaSuccess;
    if (counts && (T != 1 || !offsets || !perm_token || !pair_pos)) return cudaErrorInvalidValue;  // single-token dispatch only
    if (T >= 512 && E >= 16 && !qs && !counts && d % RT_KC == 0)
        return launch_k(router_topk_tiled_kernel, dim3((unsigned)((T + RT_TOK - 1) / RT_TOK)), dim3(256), 0, st, x, router, bias, T, d, E, k,
                        renorm, ids, w);
    if (T > 64)
        return launch_k(router_topk_kernel<256>, dim3((unsigned)T), dim3(256), 0, st, x, router, bias, d, E, k, renorm, ids, w, qs,
                        scales, bsums, counts, offsets, perm_token, pair_pos);
    return launch_k(router_topk_kernel<1024>, dim3((unsigned)T), dim3(1024), 0, st, x, router, bias, d, E, k, renorm, ids, w, qs,
                    scales, bsums, counts, offsets, perm_token, pair_pos);
}

// ------------------------------------------------------------------------------------------------
// Dispatch.  A counting sort of the T*k (token, rank) pairs by expert that keeps pair order inside
// an expert, so every expert's token list is ascending like the reference's `top_x[e]`.  One CTA:
// each warp owns experts warp, warp+32, ... and walks the pair list 32 at a time with a ballot, first
// to count, then (after an exclusive scan over experts) to place.
// ------------------------------------------------------------------------------------------------
constexpr int PERMUTE_THREADS = 1024;

__global__ void __launch_bounds__(PERMUTE_THREADS)
permute_kernel(const uint32_t* __restrict__ ids, int64_t n_pairs, int k, int E, uint32_t* __restrict__ counts,
               uint32_t* __restrict__ offsets, uint32_t* __restrict__ perm_token, uint32_t* __restrict__ pair_pos) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t s_count[CANDLE_MOE_MAX_EXPERTS];
    __shared__ uint32_t s_off[CANDLE_MOE_MAX_EXPERTS + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = PERMUTE_THREADS / 32;
    for (int e = warp; e < E; e += n_warps) {
        uint32_t c = 0;
        for (int64_t i0 = 0; i0 < n_pairs; i0 += 32) {
            const int64_t i = i0 + lane;
            const bool hit = i < n_pairs && ids[i] == (uint32_t)e;
            c += __popc(__ballot_sync(0xffffffffu, hit));
        }
        if (lane == 0) s_count[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (int e = 0; e < E; ++e) {
            s_off[e] = run;
            run += s_count[e];
        }
        s_off[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += PERMUTE_THREADS) counts[e] = s_count[e];
    for (int e = threadIdx.x; e <= E; e += PERMUTE_THREADS) offsets[e] = s_off[e];
    for (int e = warp; e < E; e += n_warps) {
        uint32_t base = s_off[e];
        for (int64_t i0 = 0; i0 < n_pairs; i0 += 32) {
            const int64_t i = i0 + lane;
            const bool hit = i < n_pairs && ids[i] == (uint32_t)e;
            const uint32_t m = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const uint32_t pos = base + __popc(m & ((1u << lane) - 1u));
                perm_token[pos] = (uint32_t)(i / k);
                pair_pos[i] = pos;
            }
            base += __popc(m);
        }
    }
}

// The same counting sort over many CTAs, for large batches: the pair list is cut into chunks of PERMUTE_CHUNK pairs.
//   count  every CTA counts its chunk's pairs per expert                       -> table[chunk][expert]
//   scan   one CTA: expert offsets, and table[chunk][expert] becomes the first position of that chunk's pairs of
//          that expert (earlier chunks first: the order inside an expert stays the pair order)
//   place  every CTA walks its chunk again, 32 pairs at a time per expert with a ballot, as the one-CTA kernel does
constexpr int PERMUTE_CHUNK = 512;

__global__ void __launch_bounds__(256)
permute_count_kernel(const uint32_t* __restrict__ ids, int64_t n_pairs, int E, uint32_t* __restrict__ table) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t s_hist[CANDLE_MOE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
    __syncthreads();
    const int64_t i0 = (int64_t)blockIdx.x * PERMUTE_CHUNK;
    for (int j = threadIdx.x; j < PERMUTE_CHUNK; j += blockDim.x) {
        const int64_t i = i0 + j;
        if (i < n_pairs) {
            const uint32_t e = ids[i];
            if (e < (uint32_t)E) atomicAdd(&s_hist[e], 1u);  // a count: the order of the additions does not matter
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) table[(size_t)blockIdx.x * E + e] = s_hist[e];
}

__global__ void __launch_bounds__(128)
permute_scan_kernel(uint32_t* __restrict__ table, int n_chunks, int E, uint32_t* __restrict__ counts,
                    uint32_t* __restrict__ offsets) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t s_count[CANDLE_MOE_MAX_EXPERTS], s_off[CANDLE_MOE_MAX_EXPERTS + 1];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        uint32_t c = 0;
        for (int b = 0; b < n_chunks; ++b) c += table[(size_t)b * E + e];
        s_count[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (int e = 0; e < E; ++e) {
            s_off[e] = run;
            run += s_count[e];
        }
        s_off[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        counts[e] = s_count[e];
        uint32_t run = s_off[e];
        for (int b = 0; b < n_chunks; ++b) {
            const uint32_t c = table[(size_t)b * E + e];
            table[(size_t)b * E + e] = run;
            run += c;
        }
    }
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_off[e];
}

__global__ void __launch_bounds__(PERMUTE_THREADS)
permute_place_kernel(const uint32_t* __restrict__ ids, int64_t n_pairs, int k, int E, const uint32_t* __restrict__ table,
                     uint32_t* __restrict__ perm_token, uint32_t* __restrict__ pair_pos) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = PERMUTE_THREADS / 32;
    const int64_t c0 = (int64_t)blockIdx.x * PERMUTE_CHUNK;
    const int64_t c1 = c0 + PERMUTE_CHUNK < n_pairs ? c0 + PERMUTE_CHUNK : n_pairs;
    for (int e = warp; e < E; e += n_warps) {
        uint32_t base = table[(size_t)blockIdx.x * E + e];
        for (int64_t i0 = c0; i0 < c1; i0 += 32) {
            const int64_t i = i0 + lane;
            const bool hit = i < c1 && ids[i] == (uint32_t)e;
            const uint32_t m = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const uint32_t pos = base + __popc(m & ((1u << lane) - 1u));
                perm_token[pos] = (uint32_t)(i / k);
                pair_pos[i] = pos;
            }
            base += __popc(m);
        }
    }
}

size_t permute_scratch_words(int64_t n_pairs, int E) {
    return (size_t)((n_pairs + PERMUTE_CHUNK - 1) / PERMUTE_CHUNK) * (size_t)E;
}

cudaError_t launch_permute(cudaStream_t st, const uint32_t* ids, int64_t T, int k, int E, uint32_t* counts,
                           uint32_t* offsets, uint32_t* perm_token, uint32_t* pair_pos, uint32_t* scratch) {
    const int64_t n_pairs = T * k;
    if (!scratch || n_pairs <= 4 * PERMUTE_CHUNK)
        return launch_k(permute_kernel, dim3(1), dim3(PERMUTE_THREADS), 0, st, ids, n_pairs, k, E, counts, offsets, perm_token,
                        pair_pos);
    const int n_chunks = (int)((n_pairs + PERMUTE_CHUNK - 1) / PERMUTE_CHUNK);
    cudaError_t e = launch_k(permute_count_kernel, dim3(n_chunks), dim3(256), 0, st, ids, n_pairs, E, scratch);
    if (e != cudaSuccess) return e;
    e = launch_k(permute_scan_kernel, dim3(1), dim3(128), 0, st, scratch, n_chunks, E, counts, offsets);
    if (e != cudaSuccess) return e;
    return launch_k(permute_place_kernel, dim3(n_chunks), dim3(PERMUTE_THREADS), 0, st, ids, n_pairs, k, E,
                    (const uint32_t*)scratch, perm_token, pair_pos);
}

__global__ void single_group_kernel(uint32_t* offsets, uint32_t rows) {
    pdl_trigger();
    pdl_wait();
    offsets[0] = 0u;
    offsets[1] = rows;
}
cudaError_t launch_single_group(cudaStream_t st, uint32_t* offsets, uint32_t rows) {
    return launch_k(single_group_kernel, dim3(1), dim3(1), 0, st, offsets, rows);
}

// ------------------------------------------------------------------------------------------------
// Combine.  CTAs of 256 threads over (token, 1024-column slab) with 128-bit accesses.  The k contributions are added
// in ascending expert id, each product rounded first (no FMA), starting from +0.0: the order of the
// reference's expert loop with broadcast_mul followed by index_add (quantized_llama.rs:185-203).
// Optional shared expert: y += shared_out * sigmoid(x . g) (qwen2_moe.rs:315-319).
// ------------------------------------------------------------------------------------------------
constexpr int COMBINE_THREADS = 256;

__global__ void __launch_bounds__(COMBINE_THREADS)
combine_kernel(const float* __restrict__ eo, int n_splits, int64_t split_stride, const uint32_t* __restrict__ ids,
               const float* __restrict__ w, const uint32_t* __restrict__ pair_pos, int k, int d,
               const float* __restrict__ shared_out, int shared_splits, int64_t shared_split_stride,
               const float* __restrict__ x, const float* __restrict__ gate, const float* __restrict__ residual,
               float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_red[COMBINE_THREADS / 32];
    __shared__ float s_gate;
    const int64_t t = blockIdx.x;
    // every thread sorts the token's k selections by expert id (k <= 8)
    uint32_t se[CANDLE_MOE_MAX_TOPK], sp[CANDLE_MOE_MAX_TOPK];
    float sw[CANDLE_MOE_MAX_TOPK];
#pragma unroll
    for (int r = 0; r < CANDLE_MOE_MAX_TOPK; ++r) {
        if (r < k) {
            se[r] = ids[t * k + r];
            sp[r] = pair_pos[t * k + r];
            sw[r] = w[t * k + r];
        } else {
            se[r] = 0xffffffffu;
            sp[r] = 0;
            sw[r] = 0.f;
        }
    }
#pragma unroll
    for (int a = 0; a < CANDLE_MOE_MAX_TOPK - 1; ++a)
#pragma unroll
        for (int b = 0; b < CANDLE_MOE_MAX_TOPK - 1 - a; ++b)
            if (se[b] > se[b + 1]) {
                uint32_t te = se[b]; se[b] = se[b + 1]; se[b + 1] = te;
                uint32_t tp = sp[b]; sp[b] = sp[b + 1]; sp[b + 1] = tp;
                float tw = sw[b]; sw[b] = sw[b + 1]; sw[b + 1] = tw;
            }

    float g = 0.f;
    if (shared_out) {
        float part = 0.f;
        const float4* xr = reinterpret_cast<const float4*>(x + t * (int64_t)d);
        const float4* gr = reinterpret_cast<const float4*>(gate);
        for (int i = threadIdx.x; i < (d >> 2); i += COMBINE_THREADS) {
            const float4 a = xr[i], b = gr[i];
            part = fmaf(a.x, b.x, part);
            part = fmaf(a.y, b.y, part);
            part = fmaf(a.z, b.z, part);
            part = fmaf(a.w, b.w, part);
        }
        part = warp_sum(part);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            float v = 0.f;
            for (int i = 0; i < COMBINE_THREADS / 32; ++i) v += s_red[i];
            s_gate = sigmoid_f(v);
        }
        __syncthreads();
        g = s_gate;
    }

    float4* yr = reinterpret_cast<float4*>(y + t * (int64_t)d);
    for (int i = blockIdx.y * COMBINE_THREADS + threadIdx.x; i < (d >> 2); i += COMBINE_THREADS * gridDim.y) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < CANDLE_MOE_MAX_TOPK; ++r) {
            if (r < k) {
                // an expert output may arrive as K-split partials: add them in split order first
                float4 v = reinterpret_cast<const float4*>(eo + (int64_t)sp[r] * d)[i];
                for (int s = 1; s < n_splits; ++s) {
                    const float4 u = reinterpret_cast<const float4*>(eo + s * split_stride + (int64_t)sp[r] * d)[i];
                    v.x += u.x;
                    v.y += u.y;
                    v.z += u.z;
                    v.w += u.w;
                }
                acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, sw[r]));
                acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, sw[r]));
                acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, sw[r]));
                acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, sw[r]));
            }
        }
        if (shared_out) {
            float4 s = reinterpret_cast<const float4*>(shared_out + t * (int64_t)d)[i];
            for (int q = 1; q < shared_splits; ++q) {
                const float4 u = reinterpret_cast<const float4*>(shared_out + q * shared_split_stride + t * (int64_t)d)[i];
                s.x += u.x;
                s.y += u.y;
                s.z += u.z;
                s.w += u.w;
            }
            acc.x = __fadd_rn(acc.x, __fmul_rn(s.x, g));
            acc.y = __fadd_rn(acc.y, __fmul_rn(s.y, g));
            acc.z = __fadd_rn(acc.z, __fmul_rn(s.z, g));
            acc.w = __fadd_rn(acc.w, __fmul_rn(s.w, g));
        }
        if (residual) {  // the layer's `x + residual` after the block (quantized_llama.rs:889-891)
            const float4 rr = reinterpret_cast<const float4*>(residual + t * (int64_t)d)[i];
            acc.x = __fadd_rn(acc.x, rr.x);
            acc.y = __fadd_rn(acc.y, rr.y);
            acc.z = __fadd_rn(acc.z, rr.z);
            acc.w = __fadd_rn(acc.w, rr.w);
        }
        yr[i] = acc;
    }
}

cudaError_t launch_combine(cudaStream_t st, const float* expert_out, int n_splits, int64_t split_stride,
                           const uint32_t* ids, const float* w, const uint32_t* pair_pos, int64_t T, int k, int d,
                           const float* shared_out, int shared_splits, int64_t shared_split_stride, const float* x,
                           const float* shared_gate, float* y, const float* residual) {
    if (T == 0) return cudaSuccess;
    const unsigned slabs = (unsigned)((d / 4 + COMBINE_THREADS - 1) / COMBINE_THREADS);
    return launch_k(combine_kernel, dim3((unsigned)T, slabs), dim3(COMBINE_THREADS), 0, st, expert_out, n_splits, split_stride,
                    ids, w, pair_pos, k, d, shared_out, shared_splits, shared_split_stride, x, shared_gate, residual, y);
}

// RmsNorm of the rows feeding the block (candle-nn/src/ops.rs:504-514): y = x / sqrt(mean(x^2) + eps) * alpha, f32.
// One CTA per row; the sum of squares is a fixed-order tree (the reference adds sequentially: last-bit
// differences only).
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ alpha, float eps, int d, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_part[8];
    __shared__ float s_m;
    const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)blockIdx.x * d);
    float part = 0.f;
    for (int i = threadIdx.x; i < (d >> 2); i += 256) {
        const float4 v = xr[i];
        part = fmaf(v.x, v.x, part);
        part = fmaf(v.y, v.y, part);
        part = fmaf(v.z, v.z, part);
        part = fmaf(v.w, v.w, part);
    }
    part = warp_sum(part);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; ++i) t += s_part[i];
        s_m = sqrtf(t / (float)d + eps);
    }
    __syncthreads();
    const float m = s_m;
    const float4* ar = reinterpret_cast<const float4*>(alpha);
    float4* yr = reinterpret_cast<float4*>(y + (int64_t)blockIdx.x * d);
    for (int i = threadIdx.x; i < (d >> 2); i += 256) {
        const float4 v = xr[i], a = ar[i];
        yr[i] = make_float4(__fmul_rn(__fdiv_rn(v.x, m), a.x), __fmul_rn(__fdiv_rn(v.y, m), a.y),
                            __fmul_rn(__fdiv_rn(v.z, m), a.z), __fmul_rn(__fdiv_rn(v.w, m), a.w));
    }
}

cudaError_t launch_rmsnorm(cudaStream_t st, const float* x, const float* alpha, float eps, int64_t T, int d, float* y) {
    if (T == 0) return cudaSuccess;
    return launch_k(rmsnorm_kernel, dim3((unsigned)T), dim3(256), 0, st, x, alpha, eps, d, y);
}

}  // namespace cmoe
