// Grouped expert products for large batches (prefill): tcgen05 tensor cores with TMEM accumulators.
//
// out[p, n] = W_e[n, :] . act[row(p), :] for all grouped positions p of every expert, as a grouped GEMM
// over tiles of 128 weight rows x 128 grouped positions.  The integers are the reference's
// (candle-core/src/quantized/k_quants.rs:1205-1285): activations are the int8 Q8K rows, and the weight
// operand holds sc_j * q (Q4_K: at most 63 * 15 = 945), both exact in fp16, multiplied by
// `tcgen05.mma kind::f16` with fp32 accumulation in tensor memory -- exact while a 256-element block's
// sum stays below 2^24, which it does by a wide margin for real data.  After every 256-element
// block the accumulator is drained and scaled by d_w(row, block) * d8(position, block) on the CUDA
// cores; the Q4_K min term sum_j m_j * bsum_j is one more K=16 MMA per block (mins against the int16
// block sums, both exact in fp16) into a second accumulator scaled by dmin_w * d8.
//
// One CTA per SM, persistent over tiles, warp-specialised:
//   warps 0-7   epilogue: drain TMEM (tcgen05.ld) once per block, scale, accumulate 64 columns per
//               thread in registers; at the end of a tile apply the SiLU gate and store
//   warp  8     TMA: the activation operand, [128 positions x 64 k] fp16 boxes, 128-byte swizzle
//   warp  9     one thread issues the MMAs and commits them to mbarriers
//   warps 10-17 unpack the Q4_K nibbles of [128 rows x 64 k] to fp16 (x sub-block scale, one HFMA2
//               per two elements) straight into the swizzled shared-memory operand
// A ring of 6 stages (32 KB each) decouples the three producers from the MMA thread; two TMEM
// accumulator sets (2 x 256 columns) decouple the MMA thread from the epilogue.  gate_up interleaves
// rows of W1 and W3 (tile row 2i = W1 row, 2i+1 = W3 row) so the two factors of silu(w1 x) * (w3 x)
// sit in neighbouring lanes and meet with one shuffle.
// Every mbarrier wait is bounded (see stream_common.cuh); nothing here uses cluster multicast.
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include "common.cuh"
#include "tc5_common.cuh"

namespace cmoe {

namespace {

constexpr int G_TILE_M = 128, G_TILE_N = 128, G_SLAB_K = 64;
constexpr int G_STAGES = 6;
constexpr int G_STAGE_A = G_TILE_M * G_SLAB_K * 2;  // 16 KB
constexpr int G_STAGE_B = G_TILE_N * G_SLAB_K * 2;  // 16 KB
constexpr int G_STAGE = G_STAGE_A + G_STAGE_B;
constexpr int G_EPI_WARPS = 8, G_DQ_WARPS = 8;
constexpr int G_THREADS = 32 * (G_EPI_WARPS + 2 + G_DQ_WARPS);  // 576
constexpr int G_TMEM_COLS = 512;
constexpr int G_SMEM_BYTES = G_STAGES * G_STAGE + 1024 /* alignment slack */;

// ---------------------------------------------------------------------------------------------
// Operand preparation: the int8 activation rows in grouped order as fp16 (B operand), their int16
// block sums as fp16 (B operand of the min product, 16 real + 48 zero columns per block so that it
// uses the same 128-byte-swizzled box), and the block scales transposed to [block][position].
// Inside every group of 4 k the order is (0, 2, 1, 3): the weight unpack produces that order for
// free (nibbles of bytes 0,2 and 1,3 convert pairwise), and a dot product does not care.
// Rows p >= P are zero padding so that a 128-row box never leaves the buffer.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
prep_gemm_b_kernel(const int8_t* __restrict__ aq, const float* __restrict__ ascale, const int16_t* __restrict__ absum,
                   const uint32_t* __restrict__ row_of, int P, int P_pad, int K, __half* __restrict__ bf16,
                   __half* __restrict__ bs16, float* __restrict__ d8t) {
    pdl_trigger();
    pdl_wait();
    const int kb = K >> 8;
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (p, block)
    if (unit >= (int64_t)P_pad * kb) return;
    const int p = (int)(unit / kb), blk = (int)(unit - (int64_t)p * kb);
    uint4 o = make_uint4(0, 0, 0, 0);
    uint32_t s2 = 0;
    float d8 = 0.f;
    if (p < P) {
        const int64_t row = row_of ? (int64_t)row_of[p] : (int64_t)p;
        const uint2 v = *reinterpret_cast<const uint2*>(aq + row * K + blk * 256 + lane * 8);
        const int8_t* b = reinterpret_cast<const int8_t*>(&v);
        __half2 h[4];
        h[0] = __halves2half2(__int2half_rn(b[0]), __int2half_rn(b[2]));
        h[1] = __halves2half2(__int2half_rn(b[1]), __int2half_rn(b[3]));
        h[2] = __halves2half2(__int2half_rn(b[4]), __int2half_rn(b[6]));
        h[3] = __halves2half2(__int2half_rn(b[5]), __int2half_rn(b[7]));
        o = *reinterpret_cast<uint4*>(h);
        if (lane < 8) {
            const int16_t* bs = absum + row * (K / 16) + blk * 16 + 2 * lane;
            const __half2 t = __halves2half2(__int2half_rn((int)bs[0]), __int2half_rn((int)bs[1]));
            s2 = *reinterpret_cast<const uint32_t*>(&t);
        }
        d8 = ascale[row * kb + blk];
    }
    *reinterpret_cast<uint4*>(bf16 + (int64_t)p * K + blk * 256 + lane * 8) = o;
    reinterpret_cast<uint32_t*>(bs16 + ((int64_t)p * kb + blk) * 64)[lane] = s2;  // 32 words = 64 halves
    if (lane == 0) d8t[(int64_t)blk * P_pad + p] = d8;
}

struct GemmParams {
    ExpertPtrs wa, wb;            // GGUF blocks: gate_up W1 / W3, down W2 (wb unused)
    const uint32_t* offsets;      // [E + 1]
    const float* d8t;             // [kb][P_pad]
    float* out;                   // gate_up: hidden [P, N]; down: [P, N]
    int* status;
    int E, K, N, kb, P, P_pad;
    int m_tiles;                  // tiles along the weight rows (N / 64 for gate_up, N / 128 for down)
};

// 6-bit scales / mins of a Q4_K block as bytes: sc[0] = sub-blocks 0..3, sc[1] = 4..7 (utils.rs:50-60)
__device__ __forceinline__ void q4k_unpack_scales(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t (&sc)[2], uint32_t (&mn)[2]) {
    sc[0] = s0 & 0x3f3f3f3fu;
    mn[0] = s1 & 0x3f3f3f3fu;
    sc[1] = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
    mn[1] = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
}

// two nibbles (bits 0-3 and 16-19 of x) -> half2 of (nibble * scale): 0x6400 | n is 1024 + n in fp16,
// and fma(1024 + n, sc, -1024 * sc) rounds the exact n * sc once (it is an integer <= 945: exact)
__device__ __forceinline__ uint32_t nib2_to_scaled_half2(uint32_t x, __half2 sc2, __half2 off2) {
    const uint32_t v = (x & 0x000F000Fu) | 0x64006400u;
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&v), sc2, off2);
    return *reinterpret_cast<const uint32_t*>(&r);
}

struct TileCoord {
    int e, nt, mt;
    uint32_t p0, p_end;
};

// tile id -> (expert, position tile, row tile); m-tiles are fastest so neighbouring CTAs share B
__device__ __forceinline__ bool decode_tile(long long tile, const uint32_t* offs, int E, int m_tiles, TileCoord& tc) {
    long long cum = 0;
    for (int e = 0; e < E; ++e) {
        const uint32_t cnt = offs[e + 1] - offs[e];
        const long long te = (long long)((cnt + G_TILE_N - 1) / G_TILE_N) * m_tiles;
        if (tile < cum + te) {
            const long long local = tile - cum;
            tc.e = e;
            tc.nt = (int)(local / m_tiles);
            tc.mt = (int)(local - (long long)tc.nt * m_tiles);
            tc.p0 = offs[e] + (uint32_t)tc.nt * G_TILE_N;
            tc.p_end = offs[e + 1];
            return true;
        }
        cum += te;
    }
    return false;
}

template <bool GATE_UP>
__global__ void __launch_bounds__(G_THREADS, 1)
expert_gemm_q4k_kernel(const __grid_constant__ GemmParams P, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_bs) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[G_STAGES], empty_bar[G_STAGES], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t s_offs[CANDLE_MOE_MAX_EXPERTS + 1];
    __shared__ __align__(16) float s_d8[2][G_TILE_N];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    for (int i = threadIdx.x; i <= P.E; i += G_THREADS) s_offs[i] = P.offsets[i];
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < G_STAGES; ++s) {
            mbar_init(&full_bar[s], G_DQ_WARPS + 1);  // 8 unpack warps + the TMA thread's expect_tx arrival
            mbar_init(&empty_bar[s], 1);              // one tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], G_EPI_WARPS);
        }
        fence_barrier_init();
    }
    if (warp == G_EPI_WARPS) tmem_alloc(&s_tmem_base, G_TMEM_COLS);
    tc5_fence_before_sync();
    __syncthreads();
    tc5_fence_after_sync();
    const uint32_t tmem_base = s_tmem_base;
    volatile int* abort_flag = &s_abort;
    const size_t row_bytes = (size_t)P.kb * Q4K_BYTES;
    constexpr uint32_t IDESC = umma_idesc_f16(G_TILE_M, G_TILE_N);

    if (warp < G_EPI_WARPS) {
        // ===================== epilogue =====================
        const int quarter = warp & 3, colhalf = warp >> 2;
        const int r = 32 * quarter + lane;  // tile row = TMEM lane
        const int etid = threadIdx.x;       // 0..255
        uint32_t ab = 0;
        TileCoord tc;
        for (long long tile = blockIdx.x; decode_tile(tile, s_offs, P.E, P.m_tiles, tc); tile += gridDim.x) {
            const int n = GATE_UP ? tc.mt * 64 + (r >> 1) : tc.mt * 128 + r;
            const uint8_t* wrow = ((GATE_UP && (r & 1)) ? P.wb.p[tc.e] : P.wa.p[tc.e]) + (size_t)n * row_bytes;
            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.f;
            for (int blk = 0; blk < P.kb; ++blk, ++ab) {
                const int buf = ab & 1;
                if (etid < G_TILE_N) {
                    const uint32_t p = tc.p0 + etid;
                    s_d8[buf][etid] = p < (uint32_t)P.P_pad ? P.d8t[(size_t)blk * P.P_pad + p] : 0.f;
                }
                const uint32_t hdr = *reinterpret_cast<const uint32_t*>(wrow + (size_t)blk * Q4K_BYTES);
                const float dw = half_bits_to_float((uint16_t)(hdr & 0xffff)), dmw = half_bits_to_float((uint16_t)(hdr >> 16));
                named_bar_sync(2, 32 * G_EPI_WARPS);
                mbar_wait(&tmem_full[buf], (ab >> 1) & 1, abort_flag);
                tc5_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(buf * 256 + colhalf * 64);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t vm[16], vn[16];
                    tmem_ld16(taddr + 16 * c, vm);
                    tmem_ld16(taddr + 128 + 16 * c, vn);
                    tmem_ld_wait();
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 d8 = *reinterpret_cast<const float4*>(&s_d8[buf][colhalf * 64 + 16 * c + 4 * q4]);
                        const float d8v[4] = {d8.x, d8.y, d8.z, d8.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float t = fmaf(dw, __uint_as_float(vm[4 * q4 + i]), -(dmw * __uint_as_float(vn[4 * q4 + i])));
                            acc[16 * c + 4 * q4 + i] = fmaf(d8v[i], t, acc[16 * c + 4 * q4 + i]);
                        }
                    }
                }
                tc5_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            }
            // ---- store the tile ----
            const uint32_t pc0 = tc.p0 + colhalf * 64;
            if (GATE_UP) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const float other = __shfl_xor_sync(0xffffffffu, acc[c], 1);
                    // even lane holds w1 x, odd lane w3 x of the same output row; even lanes store the first 32
                    // columns of this half, odd lanes the last 32
                    const bool mine = ((lane & 1) == 0) ? (c < 32) : (c >= 32);
                    if (mine && pc0 + c < tc.p_end) {
                        const float gv = (lane & 1) ? other : acc[c], uv = (lane & 1) ? acc[c] : other;
                        P.out[(size_t)(pc0 + c) * P.N + n] = silu_f(gv) * uv;
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (pc0 + c < tc.p_end) P.out[(size_t)(pc0 + c) * P.N + n] = acc[c];
            }
        }
    } else if (warp == G_EPI_WARPS) {
        // ===================== TMA: activation operand =====================
        if (lane == 0) {
            uint32_t it = 0;
            TileCoord tc;
            for (long long tile = blockIdx.x; decode_tile(tile, s_offs, P.E, P.m_tiles, tc); tile += gridDim.x) {
                for (int blk = 0; blk < P.kb; ++blk) {
                    for (int s = 0; s < 5; ++s, ++it) {
                        const int st = it % G_STAGES;
                        if (it >= G_STAGES) mbar_wait(&empty_bar[st], ((it / G_STAGES) & 1) ^ 1, abort_flag);
                        mbar_expect_tx(&full_bar[st], G_STAGE_B);
                        uint8_t* dst = smem + (size_t)st * G_STAGE + G_STAGE_A;
                        if (s < 4)
                            tma_load_2d(dst, &map_b, blk * 256 + s * 64, (int)tc.p0, &full_bar[st]);
                        else
                            tma_load_2d(dst, &map_bs, blk * 64, (int)tc.p0, &full_bar[st]);
                    }
                }
            }
        }
    } else if (warp == G_EPI_WARPS + 1) {
        // ===================== MMA issue =====================
        if (lane == 0) {
            uint32_t it = 0, ab = 0;
            TileCoord tc;
            for (long long tile = blockIdx.x; decode_tile(tile, s_offs, P.E, P.m_tiles, tc); tile += gridDim.x) {
                for (int blk = 0; blk < P.kb; ++blk, ++ab) {
                    const int buf = ab & 1;
                    if (ab >= 2) mbar_wait(&tmem_empty[buf], ((ab >> 1) & 1) ^ 1, abort_flag);
                    tc5_fence_after_sync();
                    const uint32_t d_main = tmem_base + (uint32_t)(buf * 256), d_min = d_main + 128;
                    for (int s = 0; s < 5; ++s, ++it) {
                        const int st = it % G_STAGES;
                        mbar_wait(&full_bar[st], (it / G_STAGES) & 1, abort_flag);
                        tc5_fence_after_sync();
                        const uint32_t a_addr = smem_u32(smem + (size_t)st * G_STAGE);
                        const uint64_t da = umma_desc_sw128(a_addr), db = umma_desc_sw128(a_addr + G_STAGE_A);
                        if (s < 4) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) umma_f16(d_main, da + 2 * k, db + 2 * k, IDESC, (s | k) != 0);
                        } else {
                            umma_f16(d_min, da, db, IDESC, false);
                        }
                        umma_commit(&empty_bar[st]);  // the stage may be refilled once these MMAs have read it
                    }
                    umma_commit(&tmem_full[buf]);
                }
            }
        }
    } else {
        // ===================== weight unpack: Q4_K nibbles -> fp16 (x sub-block scale) =====================
        const int dt = threadIdx.x - 32 * (G_EPI_WARPS + 2);  // 0..255
        const int r = dt >> 1, h = dt & 1;                    // tile row, 16-byte half of the row's 32 bytes per slab
        const uint32_t row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        const int sw = r & 7;
        uint32_t it = 0;
        TileCoord tc;
        for (long long tile = blockIdx.x; decode_tile(tile, s_offs, P.E, P.m_tiles, tc); tile += gridDim.x) {
            const int n = GATE_UP ? tc.mt * 64 + (r >> 1) : tc.mt * 128 + r;
            const uint8_t* wrow = ((GATE_UP && (r & 1)) ? P.wb.p[tc.e] : P.wa.p[tc.e]) + (size_t)n * row_bytes;
            for (int blk = 0; blk < P.kb; ++blk) {
                const uint8_t* wb = wrow + (size_t)blk * Q4K_BYTES;
                const uint4 hdr = *reinterpret_cast<const uint4*>(wb);
                uint32_t sc[2], mn[2];
                q4k_unpack_scales(hdr.y, hdr.z, hdr.w, sc, mn);
                uint4 q[4];
#pragma unroll
                for (int s = 0; s < 4; ++s) q[s] = *reinterpret_cast<const uint4*>(wb + 16 + 32 * s + 16 * h);
#pragma unroll
                for (int s = 0; s < 5; ++s, ++it) {
                    const int st = it % G_STAGES;
                    if (it >= G_STAGES) mbar_wait(&empty_bar[st], ((it / G_STAGES) & 1) ^ 1, abort_flag);
                    uint8_t* arow = smem + (size_t)st * G_STAGE + row_off;
                    if (s < 4) {
                        const int jl = 2 * s, jh = 2 * s + 1;
                        const float fl = (float)byte_u(sc[jl >> 2], jl & 3), fh = (float)byte_u(sc[jh >> 2], jh & 3);
                        const __half2 scl = __float2half2_rn(fl), offl = __float2half2_rn(-1024.f * fl);
                        const __half2 sch = __float2half2_rn(fh), offh = __float2half2_rn(-1024.f * fh);
                        const uint32_t w[4] = {q[s].x, q[s].y, q[s].z, q[s].w};
                        uint32_t lo[8], hi[8];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            lo[2 * i] = nib2_to_scaled_half2(w[i], scl, offl);            // elements (0, 2) of the 4
                            lo[2 * i + 1] = nib2_to_scaled_half2(w[i] >> 8, scl, offl);   // elements (1, 3)
                            hi[2 * i] = nib2_to_scaled_half2(w[i] >> 4, sch, offh);
                            hi[2 * i + 1] = nib2_to_scaled_half2(w[i] >> 12, sch, offh);
                        }
                        // 16-byte chunks of the 128-byte row: low nibbles -> k = 16h .. 16h+15 (chunks 2h, 2h+1),
                        // high nibbles -> k = 32 + 16h .. (chunks 4+2h, 5+2h); chunk index XOR (row & 7) = 128B swizzle
                        *reinterpret_cast<uint4*>(arow + (((2 * h) ^ sw) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        *reinterpret_cast<uint4*>(arow + (((2 * h + 1) ^ sw) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                        *reinterpret_cast<uint4*>(arow + (((4 + 2 * h) ^ sw) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(arow + (((5 + 2 * h) ^ sw) << 4)) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                    } else {
                        // min operand: k = 2j, 2j+1 both carry m_j (against the two 16-element block sums of sub-block j)
                        uint32_t mw[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const __half2 m2 = __float2half2_rn((float)byte_u(mn[h], i));
                            mw[i] = *reinterpret_cast<const uint32_t*>(&m2);
                        }
                        *reinterpret_cast<uint4*>(arow + ((h ^ sw) << 4)) = make_uint4(mw[0], mw[1], mw[2], mw[3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_bar[st]);
                }
            }
        }
    }
    tc5_fence_before_sync();
    __syncthreads();
    if (warp == G_EPI_WARPS) {
        tc5_fence_after_sync();
        tmem_dealloc(tmem_base, G_TMEM_COLS);
    }
    if (threadIdx.x == 0 && s_abort) atomicOr(P.status, 2);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link-time libcuda dependency)
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// fp16 matrix [rows, cols] row-major -> boxes of [128 rows x 64 cols], 128-byte swizzle
bool make_map_f16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {G_SLAB_K, G_TILE_N};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_gemm_sms = -1;

}  // namespace

// Scratch the GEMM needs for P grouped rows of length K (fp16 operand, block-sum operand, scales).
size_t expert_gemm_scratch_bytes(int64_t P, int K) {
    const size_t p_pad = (size_t)P + G_TILE_N, kb = (size_t)K / 256;
    return align_up(p_pad * K * 2, 256) + align_up(p_pad * kb * 64 * 2, 256) + align_up(kb * p_pad * 4, 256);
}

// cudaErrorNotSupported when the shape / dtype is not taken.
cudaError_t launch_expert_gemm(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype, int E,
                               int K, int N, const uint32_t* offsets, const uint32_t* row_of, int64_t P,
                               const int8_t* aq, const float* ascale, const int16_t* absum, float* out, void* scratch) {
    if (dtype != CANDLE_GGML_Q4K || !scratch) return cudaErrorNotSupported;
    if (K % 256 != 0 || N % (gate_up ? 64 : 128) != 0 || P <= 0 || P > (1 << 30)) return cudaErrorNotSupported;
    if (!encode_tiled_fn()) return cudaErrorNotSupported;
    if (g_gemm_sms < 0) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&g_gemm_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
    }
    const int kb = K / 256;
    const int64_t p_pad = P + G_TILE_N;
    uint8_t* base = static_cast<uint8_t*>(scratch);
    __half* bf16 = reinterpret_cast<__half*>(base);
    __half* bs16 = reinterpret_cast<__half*>(base + align_up((size_t)p_pad * K * 2, 256));
    float* d8t = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bs16) + align_up((size_t)p_pad * kb * 64 * 2, 256));

    const int64_t units = p_pad * kb;
    cudaError_t e = launch_k(prep_gemm_b_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, st, aq, ascale, absum,
                             row_of, (int)P, (int)p_pad, K, bf16, bs16, d8t);
    if (e != cudaSuccess) return e;

    CUtensorMap map_b, map_bs;
    if (!make_map_f16(&map_b, bf16, (uint64_t)p_pad, (uint64_t)K)) return cudaErrorNotSupported;
    if (!make_map_f16(&map_bs, bs16, (uint64_t)p_pad, (uint64_t)kb * 64)) return cudaErrorNotSupported;

    GemmParams G{};
    G.wa = wa;
    G.wb = wb;
    G.offsets = offsets;
    G.d8t = d8t;
    G.out = out;
    G.E = E;
    G.K = K;
    G.N = N;
    G.kb = kb;
    G.P = (int)P;
    G.P_pad = (int)p_pad;
    G.m_tiles = gate_up ? N / 64 : N / 128;
    e = stream_status_ptr(&G.status);
    if (e != cudaSuccess) return e;
    if (gate_up) {
        e = cudaFuncSetAttribute(expert_gemm_q4k_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        return launch_k(expert_gemm_q4k_kernel<true>, dim3(g_gemm_sms), dim3(G_THREADS), G_SMEM_BYTES, st, G, map_b, map_bs);
    }
    e = cudaFuncSetAttribute(expert_gemm_q4k_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return launch_k(expert_gemm_q4k_kernel<false>, dim3(g_gemm_sms), dim3(G_THREADS), G_SMEM_BYTES, st, G, map_b, map_bs);
}

}  // namespace cmoe
