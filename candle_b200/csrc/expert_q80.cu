// Grouped expert products for Q8_0 weights with many rows per expert (qwen2-moe style layers: 60 small
// experts plus a shared one, all Q8_0).
//
// The reference multiplies Q8_0 weights with Q8_0-quantized activations (k_quants.rs:636-677): per block of
// 32, an exact int8 dot product times the two f16 block scales.  One `mma.sync.m16n8k32` s8 is exactly one
// such block for 16 weight rows x 8 positions; its int32 result is scaled by d_w(row, block) * d_a(position,
// block) and added to an f32 accumulator.  (The tcgen05 GEMM of expert_gemm.cu drains its accumulator once
// per 256 elements, which fits the k-quants; scales that change every 32 elements on BOTH sides would need
// eight times as many drains or a three-product split of the operands.)
//
// CTA tile: 64 tile rows x 64 grouped positions, 8 warps (4 along the rows x 2 along the positions, each
// warp 16 rows x 32 positions).  K is walked in chunks of 128 (four blocks), double-buffered in shared
// memory: the activation rows arrive by cp.async (int8 rows and their f32 scales are planar and aligned),
// the weight blocks -- 34 bytes each, only 2-byte aligned in the GGUF layout -- are fetched by one thread per
// (row, block) with 8-byte loads and realigned in registers on their way to shared memory.
// gate_up: tile rows 0-7 of a warp are 8 rows of W1, rows 8-15 the same rows of W3, so that a lane holds the
// gate and the up value of the same output and applies silu(gate) * up itself.
#include "common.cuh"
#include "stream_common.cuh"

namespace cmoe {

namespace {

constexpr int QT_ROWS = 64, QT_POS = 64, QT_KC = 128;       // tile rows, positions, K per chunk
constexpr int QT_STRIDE = QT_KC + 16;                        // shared-memory row stride (bytes): no ldmatrix conflicts
constexpr int QT_THREADS = 256;

struct Q80Params {
    ExpertPtrs wa, wb;
    const uint32_t* offsets;  // [E + 1]
    const uint32_t* row_of;   // grouped position -> activation row (nullptr = identity)
    const int8_t* aq;         // [rows, K]
    const float* ascale;      // [rows, K / 32]
    float* out;               // [P, N]
    int E, K, N, m_tiles;
};

struct QTile {
    int e, mt;
    uint32_t p0, p_end;
};

__device__ __forceinline__ bool q80_decode_tile(long long tile, const uint32_t* offs, int E, int m_tiles, QTile& tc) {
    long long cum = 0;
    for (int e = 0; e < E; ++e) {
        const uint32_t cnt = offs[e + 1] - offs[e];
        const int n_tiles = (int)((cnt + QT_POS - 1) / QT_POS);
        const long long te = (long long)n_tiles * m_tiles;
        if (tile < cum + te) {
            const long long local = tile - cum;
            tc.e = e;
            tc.mt = (int)(local / n_tiles);
            tc.p0 = offs[e] + (uint32_t)(local - (long long)tc.mt * n_tiles) * QT_POS;
            tc.p_end = offs[e + 1];
            return true;
        }
        cum += te;
    }
    return false;
}

// 34 bytes of one Q8_0 block (f16 d, 32 int8) from an address that is only 2-byte aligned: five 8-byte loads
// of the enclosing aligned window, the tail bytes one by one where the window would leave the matrix.
struct RawBlock {
    uint2 w[5];
    int off;  // byte offset of the block inside the window: 0, 2, 4 or 6
};
__device__ __forceinline__ void q80_fetch(RawBlock& rb, const uint8_t* blk, const uint8_t* limit) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(blk) & ~(uintptr_t)7;
    rb.off = (int)(reinterpret_cast<uintptr_t>(blk) - a);
    const uint2* p = reinterpret_cast<const uint2*>(a);
#pragma unroll
    for (int i = 0; i < 4; ++i) rb.w[i] = __ldg(p + i);
    if (reinterpret_cast<const uint8_t*>(p + 5) <= limit) {
        rb.w[4] = __ldg(p + 4);
    } else {
        uint32_t lo = 0, hi = 0;
        const uint16_t* t = reinterpret_cast<const uint16_t*>(p + 4);
        const int n16 = (rb.off + 2) / 2;  // 16-bit words of the block in the last window word
        if (n16 > 0) lo |= __ldg(t);
        if (n16 > 1) lo |= (uint32_t)__ldg(t + 1) << 16;
        if (n16 > 2) hi |= __ldg(t + 2);
        if (n16 > 3) hi |= (uint32_t)__ldg(t + 3) << 16;
        rb.w[4] = make_uint2(lo, hi);
    }
}
// 32-bit word number i (0..8) of the block: i = 0 holds d in its low half and q[0..1] in its high half
// (i is a compile-time constant after unrolling, so the window stays in registers)
__device__ __forceinline__ uint32_t q80_win(const RawBlock& rb, int j) {
    return j >= 10 ? 0u : ((j & 1) ? rb.w[j >> 1].y : rb.w[j >> 1].x);
}
__device__ __forceinline__ uint32_t q80_word(const RawBlock& rb, int i) {
    const bool sh = rb.off >= 4;  // one whole 32-bit word in
    const uint32_t lo = sh ? q80_win(rb, i + 1) : q80_win(rb, i), hi = sh ? q80_win(rb, i + 2) : q80_win(rb, i + 1);
    return (rb.off & 2) ? __funnelshift_r(lo, hi, 16) : lo;
}

template <bool GATE_UP>
__global__ void __launch_bounds__(QT_THREADS, 2)
expert_q80_kernel(const __grid_constant__ Q80Params P) {
    __shared__ __align__(16) uint8_t s_a[2][QT_ROWS * QT_STRIDE];
    __shared__ __align__(16) uint8_t s_b[2][QT_POS * QT_STRIDE];
    __shared__ __align__(16) float s_as[2][QT_ROWS][4];
    __shared__ __align__(16) float s_bs[2][QT_POS][4];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp & 3, wn = warp >> 2, g = lane >> 2, t = lane & 3;
    const int kb = P.K / 32, n_chunks = P.K / QT_KC;
    const size_t row_bytes = (size_t)kb * Q8_0_BYTES;

    QTile tc;
    for (long long tile = blockIdx.x; q80_decode_tile(tile, P.offsets, P.E, P.m_tiles, tc); tile += gridDim.x) {
        // ---- this thread's loads: weight block (tile row tid / 4, block tid % 4 of the chunk) ----
        const int tr = tid >> 2, jb = tid & 3;
        const uint8_t* wbase;
        if (GATE_UP) {
            const int n = tc.mt * 32 + 8 * (tr >> 4) + (tr & 7);
            wbase = ((tr & 8) ? P.wb.p[tc.e] : P.wa.p[tc.e]) + (size_t)n * row_bytes;
        } else {
            wbase = P.wa.p[tc.e] + (size_t)(tc.mt * 64 + tr) * row_bytes;
        }
        const uint8_t* wlimit = ((GATE_UP && (tr & 8)) ? P.wb.p[tc.e] : P.wa.p[tc.e]) + (size_t)P.N * row_bytes;
        // activation rows: two 16-byte pieces of the chunk per thread (position tid / 4; pieces tid % 4 and + 4)
        const uint32_t pp = min(tc.p0 + (uint32_t)(tid >> 2), tc.p_end - 1);
        const size_t arow = P.row_of ? (size_t)P.row_of[pp] : (size_t)pp;
        const int8_t* asrc = P.aq + arow * P.K + 16 * (tid & 3);
        const float* ssrc = P.ascale + arow * kb;

        auto issue_b = [&](int c, int buf) {
            const uint32_t dst = smem_u32(&s_b[buf][(tid >> 2) * QT_STRIDE + 16 * (tid & 3)]);
            cp_async16(dst, asrc + c * QT_KC);
            cp_async16(dst + 64, asrc + c * QT_KC + 64);
            if ((tid & 3) == 0) cp_async16(smem_u32(&s_bs[buf][tid >> 2][0]), ssrc + 4 * c);
            cp_async_commit();
        };
        auto store_a = [&](const RawBlock& rb, int buf) {
            const uint32_t w0 = q80_word(rb, 0);
            s_as[buf][tr][jb] = half_bits_to_float((uint16_t)(w0 & 0xffff));
            uint32_t q[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(q80_word(rb, i), q80_word(rb, i + 1), 16);  // skip the 2 bytes of d
            uint4* dst = reinterpret_cast<uint4*>(&s_a[buf][tr * QT_STRIDE + 32 * jb]);
            dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
            dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
        };

        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

        RawBlock rb;
        __syncthreads();  // the previous tile's readers are done with both buffers
        issue_b(0, 0);
        q80_fetch(rb, wbase + (size_t)jb * Q8_0_BYTES, wlimit);
        store_a(rb, 0);
        cp_async_wait<0>();
        __syncthreads();

        for (int c = 0; c < n_chunks; ++c) {
            const int buf = c & 1;
            if (c + 1 < n_chunks) {
                issue_b(c + 1, buf ^ 1);
                q80_fetch(rb, wbase + (size_t)(4 * (c + 1) + jb) * Q8_0_BYTES, wlimit);
            }
            // ---- 16 MMAs per warp: 4 blocks x 4 position tiles ----
            const float4 sw0 = *reinterpret_cast<const float4*>(&s_as[buf][16 * wm + g][0]);
            const float4 sw1 = *reinterpret_cast<const float4*>(&s_as[buf][16 * wm + 8 + g][0]);
            const float sw0a[4] = {sw0.x, sw0.y, sw0.z, sw0.w}, sw1a[4] = {sw1.x, sw1.y, sw1.z, sw1.w};
            const uint32_t a_addr = smem_u32(&s_a[buf][(16 * wm + (lane & 7) + 8 * ((lane >> 3) & 1)) * QT_STRIDE + 16 * (lane >> 4)]);
            const uint32_t b_addr = smem_u32(&s_b[buf][(32 * wn + (lane & 7) + 8 * (lane >> 4)) * QT_STRIDE + 16 * ((lane >> 3) & 1)]);
#pragma unroll
            for (int np = 0; np < 2; ++np) {  // pairs of position tiles
                const float4 sa[4] = {*reinterpret_cast<const float4*>(&s_bs[buf][32 * wn + 16 * np + 2 * t][0]),
                                      *reinterpret_cast<const float4*>(&s_bs[buf][32 * wn + 16 * np + 2 * t + 1][0]),
                                      *reinterpret_cast<const float4*>(&s_bs[buf][32 * wn + 16 * np + 8 + 2 * t][0]),
                                      *reinterpret_cast<const float4*>(&s_bs[buf][32 * wn + 16 * np + 8 + 2 * t + 1][0])};
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    uint32_t a[4], b[4];
                    ldmatrix_x4(a, a_addr + 32 * blk);
                    ldmatrix_x4(b, b_addr + 16 * np * QT_STRIDE + 32 * blk);
                    const float w0 = sw0a[blk], w1 = sw1a[blk];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        int cfrag[4];
                        mma_s8_k32_z(cfrag, a, b[2 * h], b[2 * h + 1]);
                        const float4 s0 = sa[2 * h], s1 = sa[2 * h + 1];
                        const float d0 = blk == 0 ? s0.x : (blk == 1 ? s0.y : (blk == 2 ? s0.z : s0.w));
                        const float d1 = blk == 0 ? s1.x : (blk == 1 ? s1.y : (blk == 2 ? s1.z : s1.w));
                        float* ac = acc[2 * np + h];
                        ac[0] = fmaf((float)cfrag[0], w0 * d0, ac[0]);
                        ac[1] = fmaf((float)cfrag[1], w0 * d1, ac[1]);
                        ac[2] = fmaf((float)cfrag[2], w1 * d0, ac[2]);
                        ac[3] = fmaf((float)cfrag[3], w1 * d1, ac[3]);
                    }
                }
            }
            if (c + 1 < n_chunks) store_a(rb, buf ^ 1);
            cp_async_wait<0>();
            __syncthreads();
        }

        // ---- store ----
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const uint32_t p = tc.p0 + 32 * wn + 8 * nt + 2 * t + cc;
                if (p < tc.p_end) {
                    if (GATE_UP) {
                        P.out[(size_t)p * P.N + tc.mt * 32 + 8 * wm + g] = silu_f(acc[nt][cc]) * acc[nt][2 + cc];
                    } else {
                        float* o = P.out + (size_t)p * P.N + tc.mt * 64 + 16 * wm + g;
                        o[0] = acc[nt][cc];
                        o[8] = acc[nt][2 + cc];
                    }
                }
            }
        }
    }
}

int g_q80_sms = -1;

}  // namespace

// Q8_0 grouped products over many rows; cudaErrorNotSupported for shapes it does not take.
cudaError_t launch_expert_q80(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int E, int K, int N,
                              const uint32_t* offsets, const uint32_t* row_of, const int8_t* aq, const float* ascale, float* out) {
    if (K % QT_KC != 0 || N % (gate_up ? 32 : 64) != 0) return cudaErrorNotSupported;
    if (g_q80_sms < 0) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&g_q80_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
    }
    Q80Params P{};
    P.wa = wa;
    P.wb = wb;
    P.offsets = offsets;
    P.row_of = row_of;
    P.aq = aq;
    P.ascale = ascale;
    P.out = out;
    P.E = E;
    P.K = K;
    P.N = N;
    P.m_tiles = gate_up ? N / 32 : N / 64;
    const dim3 grid(2 * g_q80_sms);
    if (gate_up) return launch_k(expert_q80_kernel<true>, grid, dim3(QT_THREADS), 0, st, P);
    return launch_k(expert_q80_kernel<false>, grid, dim3(QT_THREADS), 0, st, P);
}

}  // namespace cmoe
