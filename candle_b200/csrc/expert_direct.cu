// Grouped expert products for decode-sized batches over PREPACKED weights.
//
// A one-time repack (candle_moe_prepack) lays every 8-row x 256-element piece of a Q4_K / Q6_K
// matrix out in the order the tensor-core fragments want it, so that in the hot loop every lane
// fetches its share of a block with a few fully coalesced 128-bit loads straight into registers:
// no K-split across warps, no cross-warp reduction, no CTA-wide barrier in the hot loop.  Each warp
// owns a 16-row MMA tile (gate_up: 8 rows of W1 and the same 8 rows of W3) over the whole K-range
// and runs a private ring of a few blocks in shared memory filled by 16-byte cp.async copies, so
// that several blocks per warp (> 100 KB per SM) are in flight while it multiplies the current one;
// the fragments come back out of the ring with conflict-free 128-bit shared loads.  The int8
// activations of the expert's rows also live in shared memory (read with ldmatrix).
//
// The arithmetic is the one of the streaming kernel (expert_stream.cu): exact integer sub-block
// dots on mma.sync s8, sub-block scales in int32, block scales in f32, i.e. the integers of the
// reference's vec_dot (candle-core/src/quantized/k_quants.rs:1205-1285, 1616-1673).
//
// Prepacked layout, per matrix [N rows, K]: [N / 8 half-tiles][K / 256 blocks][HTB bytes], where a
// half-tile block (8 rows x 256 elements) is
//   Q4_K (1184 B): quants [2][32 lanes][16 B]  lane (g = row, t): for u: {qs[32*(2u)+4t], qs[32*(2u)+16+4t],
//                                               qs[32*(2u+1)+4t], qs[32*(2u+1)+16+4t]} (4-byte words of the raw qs)
//                  d|dmin [8] u32, scales [8][8] u8, mins [8][8] u8 (the 6-bit fields widened to bytes)
//   Q6_K (1680 B): [3][32 lanes][16 B]: u = 0,1: ql words of half u {ql[64u+4t], +16, +32, +48};
//                  u = 2: qh words {qh[4t], qh[16+4t], qh[32+4t], qh[48+4t]}; scales [8][16] i8; d [8] f16
// Q4_K grows by 2.8 % (the 12-byte packed scales become 16 bytes); Q6_K keeps its size.
#include "common.cuh"
#include "stream_common.cuh"
#include "tc5_common.cuh"

namespace cmoe {

namespace {

// a * b + c in one instruction (the compiler may otherwise regroup sums of products)
__device__ __forceinline__ int imad(int a, int b, int c) {
    int d;
    asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

constexpr int Q4K_HTB = 1184;
constexpr int Q6K_HTB = 1680;
constexpr int DIRECT_WARPS = 16;
constexpr int DIRECT_THREADS = 32 * DIRECT_WARPS;

// Shared-memory side of a block product: 32-bit shared-window addresses of this lane's share of the current
// K-block, advanced by the kernel from block to block, so that every access is base + compile-time offset.
//   act_blk  int8 rows [MT][act_stride]: row (lane & 7), 16-byte chunk (lane >> 3) of the block   (ldmatrix)
//   sc_blk   f32 activation scales [block][MT]: the pair of positions 2t, 2t + 1
//   bs_blk   block sums [block][hi | lo][MT][BS_PER_BLOCK] bytes: row g, the lane's four sub-blocks
struct ActArgs {
    uint32_t act_blk, sc_blk, bs_blk;
    int act_stride8;  // bytes between position tiles (8 rows) of the int8 activations
};

// ------------------------------------------------------------------------------------------------
struct DirQ4K {
    static constexpr int HTB = Q4K_HTB;
    static constexpr int BS_PER_BLOCK = 8;
    __device__ static __forceinline__ int bs_value(const int16_t* bs16, int i) { return (int)bs16[2 * i] + (int)bs16[2 * i + 1]; }
    __device__ static __forceinline__ void bs_split(int v, uint8_t& hi, uint8_t& lo) {
        lo = (uint8_t)(v & 127);
        hi = (uint8_t)((v >> 7) & 0xff);
    }
    struct Frag {
        uint4 qa[2], qb[2];  // nibble words of rows g (half-tile A) and g + 8 (half-tile B)
        uint32_t dmA, dmB;   // f16 d | f16 dmin
        uint2 scA, scB, mA, mB;
    };
    // hta: shared-window address of the first half-tile block inside the warp's ring slot; the second follows it
    __device__ static __forceinline__ void load(Frag& F, uint32_t hta, int lane) {
        const int g = lane >> 2;
        const uint32_t bq = hta + lane * 16, bd = hta + 4 * g, bs = hta + 8 * g;
        F.qa[0] = lds128_o<0>(bq);
        F.qa[1] = lds128_o<512>(bq);
        F.qb[0] = lds128_o<HTB>(bq);
        F.qb[1] = lds128_o<HTB + 512>(bq);
        F.dmA = lds32_o<1024>(bd);
        F.dmB = lds32_o<HTB + 1024>(bd);
        F.scA = lds64_o<1056>(bs);
        F.scB = lds64_o<HTB + 1056>(bs);
        F.mA = lds64_o<1120>(bs);
        F.mB = lds64_o<HTB + 1120>(bs);
    }
    template <int NT, int NTL>
    __device__ static __forceinline__ void compute(const Frag& F, const ActArgs& A, int lane, uint64_t (&fp)[NT][2]) {
        const int g = lane >> 2, t = lane & 3;
        const float dA = half_bits_to_float((uint16_t)(F.dmA & 0xffff)), mnA = half_bits_to_float((uint16_t)(F.dmA >> 16));
        const float dB = half_bits_to_float((uint16_t)(F.dmB & 0xffff)), mnB = half_bits_to_float((uint16_t)(F.dmB >> 16));
        const uint32_t scA[2] = {F.scA.x, F.scA.y}, scB[2] = {F.scB.x, F.scB.y};
        int c[NTL][4];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) c[nt][i] = 0;
        static_for<4>([&](auto G) {
            constexpr int grp = decltype(G)::value;
            constexpr int jl = 2 * grp, jh = 2 * grp + 1;
            const uint4 wa = F.qa[grp >> 1], wb = F.qb[grp >> 1];
            // fragment order a0 (row g, k 0-15), a1 (row g+8, k 0-15), a2 (row g, k 16-31), a3 (row g+8, k 16-31)
            const uint32_t a0 = (grp & 1) ? wa.z : wa.x, a2 = (grp & 1) ? wa.w : wa.y;
            const uint32_t a1 = (grp & 1) ? wb.z : wb.x, a3 = (grp & 1) ? wb.w : wb.y;
            const uint32_t alo[4] = {a0 & 0x0f0f0f0fu, a1 & 0x0f0f0f0fu, a2 & 0x0f0f0f0fu, a3 & 0x0f0f0f0fu};
            const uint32_t ahi[4] = {(a0 >> 4) & 0x0f0f0f0fu, (a1 >> 4) & 0x0f0f0f0fu, (a2 >> 4) & 0x0f0f0f0fu,
                                     (a3 >> 4) & 0x0f0f0f0fu};
            const int sAl = byte_u(scA[jl >> 2], jl & 3), sAh = byte_u(scA[jh >> 2], jh & 3);
            const int sBl = byte_u(scB[jl >> 2], jl & 3), sBh = byte_u(scB[jh >> 2], jh & 3);
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                uint32_t b[4];
                ldmatrix_x4_o<64 * grp>(b, A.act_blk + nt * A.act_stride8);
                int p[4], q[4];
                mma_s8_k32_z(p, alo, b[0], b[1]);
                mma_s8_k32_z(q, ahi, b[2], b[3]);
                // two multiply-adds per accumulator (written as a chain: a sum of the two products first costs a third add)
                c[nt][0] = imad(sAh, q[0], imad(sAl, p[0], c[nt][0]));
                c[nt][1] = imad(sAh, q[1], imad(sAl, p[1], c[nt][1]));
                c[nt][2] = imad(sBh, q[2], imad(sBl, p[2], c[nt][2]));
                c[nt][3] = imad(sBh, q[3], imad(sBl, p[3], c[nt][3]));
            }
        });
        // min term: sum_j min_j * bsum_j as a [16 x 8] by [8 x 8] product (lanes t = 0, 1 carry the mins)
        const uint32_t am0 = t == 0 ? F.mA.x : (t == 1 ? F.mA.y : 0u);
        const uint32_t am1 = t == 0 ? F.mB.x : (t == 1 ? F.mB.y : 0u);
        static_for<NTL>([&](auto Nc) {
            constexpr int nt = decltype(Nc)::value;
            const uint32_t bh = lds32_o<nt * 8 * BS_PER_BLOCK>(A.bs_blk), bl = lds32_o<(8 * NT + nt * 8) * BS_PER_BLOCK>(A.bs_blk);
            const uint2 d8v = lds64_o<32 * nt>(A.sc_blk);
            int ch[4], cl[4];
            mma_s8_k16_z(ch, am0, am1, bh);
            mma_s8_k16_z(cl, am0, am1, bl);
            // two positions of one row at a time in packed f32x2 arithmetic: f += d8 * (d * c - dmin * m)
            const uint64_t d8p = f32x2_pack_bits(d8v.x, d8v.y);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float dw = r ? dB : dA, mw = r ? mnB : mnA;
                const uint64_t fc = f32x2_pack((float)c[nt][2 * r], (float)c[nt][2 * r + 1]);
                const uint64_t fm = f32x2_pack((float)(128 * ch[2 * r] + cl[2 * r]), (float)(128 * ch[2 * r + 1] + cl[2 * r + 1]));
                const uint64_t tq = f32x2_fma(f32x2_pack(-mw, -mw), fm, f32x2_mul(f32x2_pack(dw, dw), fc));
                fp[nt][r] = f32x2_fma(d8p, tq, fp[nt][r]);
            }
        });
    }
};

// ------------------------------------------------------------------------------------------------
struct DirQ6K {
    static constexpr int HTB = Q6K_HTB;
    static constexpr int BS_PER_BLOCK = 16;
    __device__ static __forceinline__ int bs_value(const int16_t* bs16, int i) { return (int)bs16[i]; }
    __device__ static __forceinline__ void bs_split(int v, uint8_t& hi, uint8_t& lo) {
        lo = (uint8_t)(v & 0xff);
        hi = (uint8_t)((v >> 8) & 0xff);
    }
    struct Frag {
        uint4 qlA[2], qlB[2];  // [half]: words {xo0 lr0, xo0 lr1, xo1 lr0, xo1 lr1}
        uint4 qhA, qhB;        // {h0 lr0, h0 lr1, h1 lr0, h1 lr1}
        uint4 scA, scB;        // 16 int8 scales
        uint32_t dA, dB;       // f16 d
    };
    __device__ static __forceinline__ void load(Frag& F, uint32_t hta, int lane) {
        const int g = lane >> 2;
        const uint32_t bq = hta + lane * 16, bs = hta + 16 * g, bd = hta + 2 * g;
        F.qlA[0] = lds128_o<0>(bq);
        F.qlA[1] = lds128_o<512>(bq);
        F.qhA = lds128_o<1024>(bq);
        F.qlB[0] = lds128_o<HTB>(bq);
        F.qlB[1] = lds128_o<HTB + 512>(bq);
        F.qhB = lds128_o<HTB + 1024>(bq);
        F.scA = lds128_o<1536>(bs);
        F.scB = lds128_o<HTB + 1536>(bs);
        F.dA = lds16_o<1664>(bd);
        F.dB = lds16_o<HTB + 1664>(bd);
    }
    __device__ static __forceinline__ uint32_t w4(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

    template <int NT, int NTL>
    __device__ static __forceinline__ void compute(const Frag& F, const ActArgs& A, int lane, uint64_t (&fp)[NT][2]) {
        const int g = lane >> 2, t = lane & 3;
        const float dA = half_bits_to_float((uint16_t)F.dA), dB = half_bits_to_float((uint16_t)F.dB);
        const uint32_t scA[4] = {F.scA.x, F.scA.y, F.scA.z, F.scA.w}, scB[4] = {F.scB.x, F.scB.y, F.scB.z, F.scB.w};
        int c[NTL][4];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) c[nt][i] = 0;
        static_for<2>([&](auto Hc) {
            constexpr int h = decltype(Hc)::value;
            uint32_t hqA[2][4], hqB[2][4];  // [lr][quarter]: the 2-bit highs moved to bits 4..5
#pragma unroll
            for (int lr = 0; lr < 2; ++lr) {
                const uint32_t qa = w4(F.qhA, 2 * h + lr), qb = w4(F.qhB, 2 * h + lr);
                hqA[lr][0] = (qa << 4) & 0x30303030u;
                hqA[lr][1] = (qa << 2) & 0x30303030u;
                hqA[lr][2] = qa & 0x30303030u;
                hqA[lr][3] = (qa >> 2) & 0x30303030u;
                hqB[lr][0] = (qb << 4) & 0x30303030u;
                hqB[lr][1] = (qb << 2) & 0x30303030u;
                hqB[lr][2] = qb & 0x30303030u;
                hqB[lr][3] = (qb >> 2) & 0x30303030u;
            }
            static_for<2>([&](auto Yc) {  // 64 elements = quarters 2y, 2y+1
                constexpr int y = decltype(Yc)::value;
                uint32_t aA[4], aB[4];
                int sA[4], sB[4];
#pragma unroll
                for (int xo = 0; xo < 2; ++xo) {
                    const int x = 2 * y + xo;
#pragma unroll
                    for (int lr = 0; lr < 2; ++lr) {
                        const uint32_t wla = w4(F.qlA[h], 2 * (x & 1) + lr), wlb = w4(F.qlB[h], 2 * (x & 1) + lr);
                        const uint32_t la = (x >> 1) ? (wla >> 4) : wla, lb = (x >> 1) ? (wlb >> 4) : wlb;
                        aA[2 * xo + lr] = (la & 0x0f0f0f0fu) | hqA[lr][x];
                        aB[2 * xo + lr] = (lb & 0x0f0f0f0fu) | hqB[lr][x];
                        const int j = 8 * h + 2 * x + lr;
                        sA[2 * xo + lr] = byte_s(scA[j >> 2], j & 3);
                        sB[2 * xo + lr] = byte_s(scB[j >> 2], j & 3);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) {
                    uint32_t b[4];
                    ldmatrix_x4_o<128 * h + 64 * y>(b, A.act_blk + nt * A.act_stride8);
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4) {
                        int p[4];
                        mma_s8_k16_z(p, aA[s4], aB[s4], b[s4]);
                        c[nt][0] = imad(sA[s4], p[0], c[nt][0]);
                        c[nt][1] = imad(sA[s4], p[1], c[nt][1]);
                        c[nt][2] = imad(sB[s4], p[2], c[nt][2]);
                        c[nt][3] = imad(sB[s4], p[3], c[nt][3]);
                    }
                }
            });
        });
        const uint32_t sa = scA[t], sb = scB[t];
        static_for<NTL>([&](auto Nc) {
            constexpr int nt = decltype(Nc)::value;
            const uint32_t bh = lds32_o<nt * 8 * BS_PER_BLOCK>(A.bs_blk), bl = lds32_o<(8 * NT + nt * 8) * BS_PER_BLOCK>(A.bs_blk);
            int ch[4], cl[4];
            mma_s8_k16_z(ch, sa, sb, bh);
            mma_s8u8_k16_z(cl, sa, sb, bl);
            const uint2 d8v = lds64_o<32 * nt>(A.sc_blk);
            const uint64_t d8p = f32x2_pack_bits(d8v.x, d8v.y);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float dw = r ? dB : dA;
                const int i0 = c[nt][2 * r] - 32 * (256 * ch[2 * r] + cl[2 * r]);
                const int i1 = c[nt][2 * r + 1] - 32 * (256 * ch[2 * r + 1] + cl[2 * r + 1]);
                fp[nt][r] = f32x2_fma(f32x2_mul(d8p, f32x2_pack(dw, dw)), f32x2_pack((float)i0, (float)i1), fp[nt][r]);
            }
        });
    }
};

struct DirectParams {
    ExpertPtrs wa, wb;  // prepacked matrices
    const uint32_t* offsets;
    const uint32_t* row_of;
    const int8_t* aq;
    const float* ascale;
    const int16_t* absum;
    float* out;
    int64_t out_split_stride;
    int E, K, N, kb, splits, MT;
    int blk_start[9];  // split s covers blocks [blk_start[s], blk_start[s + 1])
    int act_stride;
    uint32_t off_act, off_scale, off_bs, off_ring, off_part;
};

// DEPTH = ring slots per warp (DEPTH - 1 blocks in flight while one is multiplied)
template <class F, bool GATE_UP, int NT, int DEPTH>
// The one-position-tile Q4_K kernels are held to 96 registers (a bound of 608 threads; they are launched with 512,
// and Q6_K would spill): the
// registers a CTA leaves free let the CTAs of the next kernel on the stream become resident and run their
// prologue under programmatic dependent launch while this one drains.
__global__ void __launch_bounds__(NT == 1 && F::HTB == Q4K_HTB ? 608 : DIRECT_THREADS, 1) expert_direct_kernel(const __grid_constant__ DirectParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint32_t s_offs[CANDLE_MOE_MAX_EXPERTS + 1];
    __shared__ int s_rows[16];
    constexpr int MT = 8 * NT;
    constexpr int TILE_N = GATE_UP ? 8 : 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    pdl_trigger();
    pdl_wait();
    for (int i = tid; i <= P.E; i += DIRECT_THREADS) s_offs[i] = P.offsets[i];
    __syncthreads();

    uint8_t* act = smem + P.off_act;
    float* act_scale = reinterpret_cast<float*>(smem + P.off_scale);  // [block][MT]
    uint8_t* bs = smem + P.off_bs;                                    // [block][hi | lo][MT][BS_PER_BLOCK]
    constexpr int BSB = F::BS_PER_BLOCK;
    ActArgs A;
    A.act_stride8 = 8 * P.act_stride;
    // this lane's share of K-block 0 (see ActArgs)
    const uint32_t act_lane = smem_u32(act) + (lane & 7) * P.act_stride + 16 * (lane >> 3);
    const uint32_t sc_lane = smem_u32(act_scale) + 8 * (lane & 3);
    const uint32_t bs_lane = smem_u32(bs) + (lane >> 2) * BSB + (BSB == 8 ? 4 * (lane & 1) : 4 * (lane & 3));
    constexpr int SLOT_BYTES = 2 * F::HTB;       // both half-tile blocks of one K-block
    constexpr int VEC_PER_HT = F::HTB / 16;      // 16-byte vectors per half-tile block
    const uint32_t ring = smem_u32(smem + P.off_ring) + (uint32_t)warp * (DEPTH * SLOT_BYTES);
    const uint32_t part_base = smem_u32(smem + P.off_part);  // 512 bytes per warp (one-position-tile kernels only)

    // Cost-balanced contiguous share of the (token group, split, tile) sequence.  Cost = blocks streamed, weighted
    // by what a block costs to multiply: a group of more than eight rows takes two position tiles per block, which
    // is 11 : 8 in issued instructions against a group of up to eight.
    const int tiles = P.N / TILE_N;
    auto group_weight = [](uint32_t rows) { return (NT > 1 && rows > 8) ? 11 : 8; };
    long long ctot = 0;
    for (int i = 0; i < P.E; ++i) {
        const uint32_t cnt = s_offs[i + 1] - s_offs[i];
        ctot += (long long)tiles * P.kb * ((long long)(cnt / MT) * group_weight(MT) + (cnt % MT ? group_weight(cnt % MT) : 0));
    }
    const long long lo = ctot * blockIdx.x / gridDim.x, hi = ctot * (blockIdx.x + 1) / gridDim.x;
    if (lo >= hi) return;
    const size_t ht_stride = (size_t)P.kb * F::HTB;  // bytes of one half-tile over the whole K

    long long acc = 0;  // cost of the groups before the current one
    for (int e = 0; e < P.E && acc < hi; ++e) {
      const uint32_t cnt = s_offs[e + 1] - s_offs[e];
      for (uint32_t g0 = 0; g0 < cnt && acc < hi; g0 += MT) {
        const uint32_t rows = min((uint32_t)MT, cnt - g0);
        const int w = group_weight(rows);
        const long long gcost = (long long)tiles * P.kb * w;
        const long long g_lo = acc;
        acc += gcost;
        if (acc <= lo) continue;
        const uint32_t p_base = s_offs[e] + g0;
        const uint32_t p_end = p_base + rows;
        const int ntiles = (int)(rows + 7) / 8;
        for (int sp = 0; sp < P.splits; ++sp) {
            const int blk0 = P.blk_start[sp], nblk = P.blk_start[sp + 1] - blk0;
            const long long unit = (long long)nblk * w;  // cost of one tile over this split
            const long long ph_lo = g_lo + (long long)tiles * blk0 * w;
            const long long ph_hi = ph_lo + (long long)tiles * unit;
            const long long a = lo > ph_lo ? lo : ph_lo, b = hi < ph_hi ? hi : ph_hi;
            if (a >= b) continue;
            const int tile_lo = (int)((a - ph_lo + unit - 1) / unit), tile_hi = (int)((b - ph_lo + unit - 1) / unit);
            if (tile_lo >= tile_hi) continue;

            // ---- make the token group's int8 rows, scales and block sums resident ----
            __syncthreads();
            if (tid < MT) {
                const uint32_t pp = p_base + tid;
                s_rows[tid] = pp < p_end ? (P.row_of ? (int)P.row_of[pp] : (int)pp) : -1;
            }
            __syncthreads();
            {
                const int vec_per_row = nblk * 16;
#pragma unroll 4
                for (int idx = tid; idx < MT * vec_per_row; idx += DIRECT_THREADS) {
                    const int j = idx / vec_per_row, v = idx - j * vec_per_row;
                    const int row = s_rows[j];
                    int4 val = make_int4(0, 0, 0, 0);
                    if (row >= 0) val = *reinterpret_cast<const int4*>(P.aq + (int64_t)row * P.K + (int64_t)blk0 * 256 + 16 * v);
                    *reinterpret_cast<int4*>(act + j * P.act_stride + 16 * v) = val;
                }
                for (int idx = tid; idx < MT * nblk; idx += DIRECT_THREADS) {
                    const int j = idx / nblk, bb = idx - j * nblk;
                    const int row = s_rows[j];
                    act_scale[bb * MT + j] = row >= 0 ? P.ascale[(int64_t)row * P.kb + blk0 + bb] : 0.f;
                }
                const int per_row = nblk * F::BS_PER_BLOCK;
                for (int idx = tid; idx < MT * per_row; idx += DIRECT_THREADS) {
                    const int j = idx / per_row, bb = idx - j * per_row;
                    const int row = s_rows[j];
                    const int v = row >= 0 ? F::bs_value(P.absum + (int64_t)row * (P.K / 16) + blk0 * 16, bb) : 0;
                    uint8_t h8, l8;
                    F::bs_split(v, h8, l8);
                    const int blk = bb / BSB, i = bb - blk * BSB;
                    bs[((2 * blk) * MT + j) * BSB + i] = h8;
                    bs[((2 * blk + 1) * MT + j) * BSB + i] = l8;
                }
            }
            __syncthreads();

            // ---- every warp streams its own tiles over the K-range of this split ----
            // Whole rounds of 16 tiles go one tile per warp over all the blocks.  The tiles left over (fewer than 16)
            // are shared so that no warp of the CTA idles through a last round, and the partial sums meet in shared
            // memory, added in block order by the warp that holds a tile's first block:
            //   one position tile (a scratch of 512 bytes per warp exists): the left-over tiles' blocks, taken as one
            //     sequence, are cut into 16 equal ranges; a range touches at most two tiles;
            //   two position tiles (no room for the scratch): teams of 2, 4, 8 or 16 warps split a tile's blocks and
            //     hand their sums over through their own rings, which are free by then.
            const int n_t = tile_hi - tile_lo, n_rounds = n_t / DIRECT_WARPS, rem = n_t - n_rounds * DIRECT_WARPS;
            constexpr bool RANGES = NT == 1;
            int team = 1;
            if (!RANGES && rem > 0)
                while (2 * team * rem <= DIRECT_WARPS) team *= 2;
            const bool shared_round = rem > 0 && (RANGES || team > 1);  // uniform over the CTA
            const int my_rem = warp / team, part = warp - my_rem * team;
            const int rem_blocks = rem * nblk;  // RANGES: this warp's range [q0, q1) of the left-over block sequence
            const int q0 = RANGES ? rem_blocks * warp / DIRECT_WARPS : 0, q1 = RANGES ? rem_blocks * (warp + 1) / DIRECT_WARPS : 0;
            int n_items = n_rounds;
            if (RANGES) {
                if (q1 > q0) n_items += 1 + ((q1 - 1) / nblk > q0 / nblk);
            } else if (my_rem < rem) {
                n_items += 1;
            }
            const int g = lane >> 2, t = lane & 3;
            uint64_t fp[NT][2];  // per position tile: (row g | row g + 8) x two positions, packed f32 pairs
            auto store_tile = [&](int tile) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float f[4];
                    f32x2_unpack(fp[nt][0], f[0], f[1]);
                    f32x2_unpack(fp[nt][1], f[2], f[3]);
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const uint32_t p = p_base + nt * 8 + 2 * t + cc;
                        if (p < p_end) {
                            if (GATE_UP) {
                                P.out[(int64_t)p * P.N + tile * 8 + g] = silu_f(f[cc]) * f[2 + cc];
                            } else {
                                float* o = P.out + (int64_t)sp * P.out_split_stride + (int64_t)p * P.N + tile * 16 + g;
                                o[0] = f[cc];
                                o[8] = f[2 + cc];
                            }
                        }
                    }
                }
            };
            int own_tile = -1;    // left-over tile whose sum this warp completes after the barrier
            bool hand_over;       // this item's sum goes to the scratch for another warp to add
            for (int it = 0; it < n_items; ++it) {
                int tile = tile_lo + warp + DIRECT_WARPS * it, b0 = 0, b1 = nblk;
                hand_over = false;
                if (it >= n_rounds) {
                    if (RANGES) {
                        const int q = it == n_rounds ? q0 : (q0 / nblk + 1) * nblk;  // second item: the next tile from its start
                        const int tl = q / nblk;
                        b0 = q - tl * nblk;
                        b1 = min(nblk, b0 + (q1 - q));
                        tile = tile_lo + n_rounds * DIRECT_WARPS + tl;
                        if (b0 > 0)
                            hand_over = true;
                        else if (b1 < nblk)
                            own_tile = tile;
                    } else {
                        tile = tile_lo + n_rounds * DIRECT_WARPS + my_rem;
                        if (team > 1) {
                            b0 = nblk * part / team;
                            b1 = nblk * (part + 1) / team;
                            if (part == 0)
                                own_tile = tile;
                            else
                                hand_over = true;
                        }
                    }
                }
                const int nb = b1 - b0;
                const uint8_t* hta;
                const uint8_t* htb;
                if (GATE_UP) {
                    hta = P.wa.p[e] + (size_t)tile * ht_stride + (size_t)(blk0 + b0) * F::HTB;
                    htb = P.wb.p[e] + (size_t)tile * ht_stride + (size_t)(blk0 + b0) * F::HTB;
                } else {
                    hta = P.wa.p[e] + (size_t)(2 * tile) * ht_stride + (size_t)(blk0 + b0) * F::HTB;
                    htb = hta + ht_stride;
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) fp[nt][0] = fp[nt][1] = 0ull;
                // fill one ring slot with block j of both half-tiles (16-byte cp.async per lane).  The vector index
                // of a lane in pass i is lane + 32 i, so which half-tile a pass reads is known at compile time except
                // for the one pass that straddles the boundary: straight-line code, one predicate for the ragged end.
                auto issue = [&](int j) {
                    if (j < nb) {
                        const uint32_t slot = ring + (uint32_t)(j % DEPTH) * SLOT_BYTES + 16 * lane;
                        const uint8_t* sa = hta + (size_t)j * F::HTB + 16 * lane;
                        const uint8_t* sb = htb + (size_t)j * F::HTB + 16 * lane - 16 * VEC_PER_HT;
                        constexpr int PASSES = (2 * VEC_PER_HT + 31) / 32;
                        static_for<PASSES>([&](auto Ic) {
                            constexpr int i = decltype(Ic)::value;
                            const uint8_t* src;
                            if (32 * i + 31 < VEC_PER_HT)
                                src = sa;
                            else if (32 * i >= VEC_PER_HT)
                                src = sb;
                            else
                                src = lane + 32 * i >= VEC_PER_HT ? sb : sa;
                            if (32 * i + 31 < 2 * VEC_PER_HT || lane + 32 * i < 2 * VEC_PER_HT) cp_async16_o<512 * i>(slot, src);
                        });
                    }
                    cp_async_commit();  // one group per block, empty past the end: the count stays in step
                };
                __syncwarp();  // the previous tile's last slot reads are done in every lane
#pragma unroll
                for (int i = 0; i < DEPTH - 1; ++i) issue(i);
                for (int j = 0; j < nb; ++j) {
                    cp_async_wait<DEPTH - 2>();  // this lane's copies of block j have landed
                    __syncwarp();                // ... and everyone else's; slot (j - 1) % DEPTH is free again
                    issue(j + DEPTH - 1);
                    typename F::Frag cur;
                    const uint32_t slot = ring + (uint32_t)(j % DEPTH) * SLOT_BYTES;
                    F::load(cur, slot, lane);
                    const int bk = b0 + j;
                    A.act_blk = act_lane + bk * 256;
                    A.sc_blk = sc_lane + bk * (4 * MT);
                    A.bs_blk = bs_lane + bk * (2 * MT * BSB);
                    if (NT == 1 || ntiles == 1)
                        F::template compute<NT, 1>(cur, A, lane, fp);
                    else
                        F::template compute<NT, NT>(cur, A, lane, fp);
                }
                if (hand_over) {
                    // RANGES: a scratch of its own.  Teams: the warp's ring; this is its last item and nothing of its
                    // copies is in flight any more (the groups still pending are empty ones).
                    const uint32_t dst = RANGES ? part_base + (uint32_t)warp * 512u : ring;
                    __syncwarp();
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int r = 0; r < 2; ++r) sts64(dst + (uint32_t)(((nt * 2 + r) * 32 + lane) * 8), fp[nt][r]);
                } else if (own_tile != tile) {
                    store_tile(tile);
                }
            }
            if (shared_round) {
                __syncthreads();
                if (own_tile >= 0) {
                    const int tl = own_tile - (tile_lo + n_rounds * DIRECT_WARPS);
                    for (int w2 = warp + 1; w2 < DIRECT_WARPS; ++w2) {
                        uint32_t src;
                        if (RANGES) {
                            const int r0 = rem_blocks * w2 / DIRECT_WARPS, r1 = rem_blocks * (w2 + 1) / DIRECT_WARPS;
                            if (r0 >= (tl + 1) * nblk) break;  // the next tile begins: nothing more belongs to this one
                            if (r1 == r0) continue;
                            src = part_base + (uint32_t)w2 * 512u;
                        } else {
                            if (w2 >= warp + team) break;
                            src = ring + (uint32_t)(w2 - warp) * (DEPTH * SLOT_BYTES);
                        }
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int r = 0; r < 2; ++r)
                                fp[nt][r] = f32x2_add(fp[nt][r], lds64u(src + (uint32_t)(((nt * 2 + r) * 32 + lane) * 8)));
                    }
                    store_tile(own_tile);
                }
            }
        }
      }
    }
}

// ---- prepack kernels: one CTA per (half-tile, block) ----
__global__ void __launch_bounds__(256) prepack_q4k_kernel(const uint8_t* __restrict__ raw, int kb, uint8_t* __restrict__ dst) {
    const int ht = blockIdx.x / kb, blk = blockIdx.x - ht * kb;
    const size_t row_bytes = (size_t)kb * Q4K_BYTES;
    const uint8_t* src = raw + (size_t)ht * 8 * row_bytes + (size_t)blk * Q4K_BYTES;  // row g at + g * row_bytes
    uint8_t* out = dst + ((size_t)ht * kb + blk) * Q4K_HTB;
    const int w = threadIdx.x;  // output word 0..255 of the quant region
    {
        const int u = w >> 7, lane = (w >> 2) & 31, cw = w & 3;
        const int g = lane >> 2, t = lane & 3;
        const int grp = 2 * u + (cw >> 1), isb = cw & 1;
        const uint32_t v = *reinterpret_cast<const uint32_t*>(src + (size_t)g * row_bytes + 16 + 32 * grp + 16 * isb + 4 * t);
        reinterpret_cast<uint32_t*>(out)[w] = v;
    }
    if (w < 8) reinterpret_cast<uint32_t*>(out + 1024)[w] = *reinterpret_cast<const uint32_t*>(src + (size_t)w * row_bytes);
    if (w < 64) {
        const int g = w >> 3, j = w & 7;
        int sc, m;
        q4k_scale_min(j, src + (size_t)g * row_bytes + 4, sc, m);
        out[1056 + w] = (uint8_t)sc;
        out[1120 + w] = (uint8_t)m;
    }
}

__global__ void __launch_bounds__(384) prepack_q6k_kernel(const uint8_t* __restrict__ raw, int kb, uint8_t* __restrict__ dst) {
    const int ht = blockIdx.x / kb, blk = blockIdx.x - ht * kb;
    const size_t row_bytes = (size_t)kb * Q6K_BYTES;
    const uint8_t* src = raw + (size_t)ht * 8 * row_bytes + (size_t)blk * Q6K_BYTES;
    uint8_t* out = dst + ((size_t)ht * kb + blk) * Q6K_HTB;
    const int w = threadIdx.x;  // output word 0..383
    {
        const int u = w >> 7, lane = (w >> 2) & 31, cw = w & 3;
        const int g = lane >> 2, t = lane & 3;
        int off;
        if (u < 2)
            off = 64 * u + 32 * (cw >> 1) + 16 * (cw & 1) + 4 * t;  // ql, half u, xo = cw >> 1, lr = cw & 1
        else
            off = 128 + 32 * (cw >> 1) + 16 * (cw & 1) + 4 * t;     // qh, half cw >> 1, lr = cw & 1
        const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src + (size_t)g * row_bytes + off);
        reinterpret_cast<uint32_t*>(out)[w] = (uint32_t)s16[0] | ((uint32_t)s16[1] << 16);
    }
    if (w < 128) out[1536 + w] = src[(size_t)(w >> 4) * row_bytes + 192 + (w & 15)];
    if (w < 8) reinterpret_cast<uint16_t*>(out + 1664)[w] = *reinterpret_cast<const uint16_t*>(src + (size_t)w * row_bytes + 208);
}

int g_dir_max_smem = -1, g_dir_sms = -1;

template <class F, bool GATE_UP, int NT, int DEPTH>
cudaError_t launch_dir(cudaStream_t st, const DirectParams& P, size_t smem_bytes) {
    auto kfn = expert_direct_kernel<F, GATE_UP, NT, DEPTH>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
    if (e != cudaSuccess) return e;
    return launch_k(kfn, dim3(g_dir_sms), dim3(DIRECT_THREADS), smem_bytes, st, P);
}

}  // namespace

size_t prepacked_bytes(int dtype, int64_t n_rows, int k) {
    if (k % 256 || n_rows % 8) return 0;
    const size_t htb = dtype == CANDLE_GGML_Q4K ? Q4K_HTB : (dtype == CANDLE_GGML_Q6K ? Q6K_HTB : 0);
    return (size_t)(n_rows / 8) * (size_t)(k / 256) * htb;
}

cudaError_t launch_prepack(cudaStream_t st, int dtype, const void* raw, int64_t n_rows, int k, void* dst) {
    const int kb = k / 256;
    const unsigned grid = (unsigned)((n_rows / 8) * kb);
    if (grid == 0) return cudaSuccess;
    if (dtype == CANDLE_GGML_Q4K)
        prepack_q4k_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(raw), kb, static_cast<uint8_t*>(dst));
    else if (dtype == CANDLE_GGML_Q6K)
        prepack_q6k_kernel<<<grid, 384, 0, st>>>(static_cast<const uint8_t*>(raw), kb, static_cast<uint8_t*>(dst));
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

// Plans and launches the prepacked-weight kernel; cudaErrorNotSupported when the shape is not taken.
cudaError_t launch_expert_direct(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype,
                                 int E, int K, int N, const uint32_t* offsets, const uint32_t* row_of,
                                 int64_t max_rows_per_expert, const int8_t* aq, const float* ascale,
                                 const int16_t* absum, float* out, int* n_splits_out, int64_t split_stride,
                                 int max_splits, int max_active_experts, int64_t total_rows) {
    if (dtype != CANDLE_GGML_Q4K && dtype != CANDLE_GGML_Q6K) return cudaErrorNotSupported;
    const int tile_n = gate_up ? 8 : 16;
    if (N % tile_n != 0 || K % 256 != 0) return cudaErrorNotSupported;
    if (g_dir_max_smem < 0) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&g_dir_max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&g_dir_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
    }
    const int kb = K / 256;
    // One position tile (8 rows per group) or two (16).  An expert with more rows than a group holds is walked once
    // per group.  When the caller's bound allows more than 8 rows but the experts hold about 3 or fewer on average
    // (total_rows known), practically every expert fits one 8-row group and the one-tile kernel is the cheaper
    // choice (Mixtral-shaped layer: 145 us at 9 rows against ~200 with two tiles; from 16 rows on the two are equal
    // and beyond 20 the two-tile kernel wins).
    const bool few_rows = total_rows > 0 && total_rows <= 3 * (int64_t)E;
    const int NT = max_rows_per_expert <= 8 || few_rows ? 1 : 2;
    const int MT = 8 * NT;
    const int bs_per_block = dtype == CANDLE_GGML_Q4K ? 8 : 16;
    DirectParams P{};
    P.wa = wa;
    P.wb = wb;
    // With few active experts there are fewer 16-row tiles than warps on the GPU: split K further (the
    // down product only; partial sums meet in the combine kernel) until every warp has ~2 items.
    int min_splits = 1;
    if (!gate_up && max_active_experts > 0) {
        const long long items = (long long)max_active_experts * (N / tile_n);
        const long long want = 2LL * g_dir_sms * DIRECT_WARPS;
        min_splits = (int)((want + items - 1) / items);
        if (min_splits > max_splits) min_splits = max_splits;
        if (min_splits < 1) min_splits = 1;
    }
    for (int splits = min_splits; splits <= max_splits && splits <= kb; ++splits) {
        if (gate_up && splits > 1) break;
        const int ks_blocks = (kb + splits - 1) / splits;
        uint32_t off = 0;
        auto take = [&](uint32_t bytes) {
            off = (off + 127u) & ~127u;
            const uint32_t o = off;
            off += bytes;
            return o;
        };
        P.act_stride = ks_blocks * 256 + 16;
        P.off_act = take((uint32_t)MT * P.act_stride);
        P.off_scale = take((uint32_t)MT * ks_blocks * 4);
        P.off_bs = take((uint32_t)2 * MT * ks_blocks * bs_per_block);
        // per-warp rings of DEPTH K-blocks: 4 slots for Q4_K (2368 B each), 3 for Q6_K (3360 B each)
        const int depth = dtype == CANDLE_GGML_Q4K ? 4 : 3;
        const uint32_t slot_bytes = 2u * (dtype == CANDLE_GGML_Q4K ? Q4K_HTB : Q6K_HTB);
        P.off_ring = take((uint32_t)DIRECT_WARPS * depth * slot_bytes);
        P.off_part = NT == 1 ? take((uint32_t)DIRECT_WARPS * 512u) : 0u;
        if ((int)off > g_dir_max_smem - 1024) continue;
        P.splits = splits;
        int bs = 0;
        for (int s = 0; s < splits; ++s) {
            P.blk_start[s] = bs;
            const int rem = kb - bs, rs = splits - s;
            bs += (rem + rs - 1) / rs;
        }
        P.blk_start[splits] = kb;
        P.offsets = offsets;
        P.row_of = row_of;
        P.aq = aq;
        P.ascale = ascale;
        P.absum = absum;
        P.out = out;
        P.out_split_stride = split_stride;
        P.E = E;
        P.K = K;
        P.N = N;
        P.kb = kb;
        P.MT = MT;
        if (n_splits_out) *n_splits_out = splits;
        if (dtype == CANDLE_GGML_Q4K) {
            if (gate_up) return NT == 1 ? launch_dir<DirQ4K, true, 1, 4>(st, P, off) : launch_dir<DirQ4K, true, 2, 4>(st, P, off);
            return NT == 1 ? launch_dir<DirQ4K, false, 1, 4>(st, P, off) : launch_dir<DirQ4K, false, 2, 4>(st, P, off);
        }
        if (gate_up) return NT == 1 ? launch_dir<DirQ6K, true, 1, 3>(st, P, off) : launch_dir<DirQ6K, true, 2, 3>(st, P, off);
        return NT == 1 ? launch_dir<DirQ6K, false, 1, 3>(st, P, off) : launch_dir<DirQ6K, false, 2, 3>(st, P, off);
    }
    return cudaErrorNotSupported;
}

}  // namespace cmoe
