// Grouped expert products, streaming form for decode-sized batches (a few rows per expert).
//
// The work is HBM-bound: every active expert's weight blocks are read once and the arithmetic per
// byte is tiny.  Design:
//   * persistent CTAs (one per SM), each owning a CONTIGUOUS, cost-balanced range of work items;
//     an item is a tile of 16 weight rows of one expert over one K-range ("split"); for gate_up the
//     16 rows are 8 rows of W1 and the same 8 rows of W3, so one MMA tile yields both factors of
//     silu(w1 x) * (w3 x);
//   * warp 0 is the producer: one `cp.async.bulk` (TMA, no tensor map needed: a row chunk is
//     contiguous) per weight row per stage into a padded, bank-conflict-free shared-memory ring,
//     completion counted on an mbarrier.  Copies are >= 1.7 KB (measured: below ~2 KB the per-copy
//     cost, not HBM, limits a bulk-copy ring) and >= 70 KB are always in flight per SM;
//   * the other CW warps are consumers: each takes one 256-element block column of the stage,
//     unpacks the quants in registers straight from `ldmatrix` fragments and multiplies them with
//     the int8 activations (resident in shared memory for the expert's rows) on the tensor cores
//     with `mma.sync m16n8k32 / m16n8k16` (s8 x s8 -> s32).  Sub-block scales are applied to the
//     exact integer partial sums, the per-block f16 scales in f32 -- the same integers as the
//     reference's vec_dot (candle-core/src/quantized/k_quants.rs:1205-1285, 1616-1673), different
//     f32 order;
//   * the CW K-slices of a tile meet in shared memory in a fixed order; gate_up applies the SiLU
//     gate there and stores f32, down stores one partial per K-split which the combine kernel adds
//     in split order (deterministic, no atomics).
// Every wait on an mbarrier is bounded; on expiry the CTA raises a flag in `status`, stops waiting
// and runs its loops to the end so that no thread is left behind at a barrier.
#include "common.cuh"
#include "stream_common.cuh"

namespace cmoe {


namespace {

constexpr int TILE_ROWS = 16;         // weight rows per stage (gate_up: 8 rows of W1 followed by the same 8 rows of W3)
constexpr int RED_PAD = 17;           // floats per (warp, token) in the reduction buffer

// Everything a consumer warp needs besides the weight tile itself (32-bit shared-window addresses).
struct BlockArgs {
    uint32_t act;        // int8 rows of the token group, [MT][act_stride]
    uint32_t act_scale;  // per (token, block) scale d8 (f32), [MT][scale_stride]
    uint32_t bs_hi;      // activation block sums split into two byte planes, [MT][bs_stride]
    uint32_t bs_lo;
    int act_stride, scale_stride, bs_stride;  // act/bs in bytes, scale in floats
    int kblk_local;      // block index inside the resident K-range
};

// ---------------------------------------------------------------------------------------------
// Q4_K (144 B per 256): f16 d, f16 dmin, 12 B of 6-bit scales/mins, 128 B of nibbles.
//   value = d * sc_j * q - dmin * m_j  =>  dot = d*d8 * sum_j sc_j (q . a)_j  -  dmin*d8 * sum_j m_j * bsum_j
// The first sum: one m16n8k32 MMA per 32-element sub-block, scaled by sc_j in int32.
// The second sum is a [16 x 8] by [8 x 8] integer product per block: the 8 mins of a row are
// already packed as bytes, the block sums of the activations (|.| <= 4096) are split base 128 into
// two int8 planes, so it costs two m16n8k16 MMAs per block and token tile.
// ---------------------------------------------------------------------------------------------
struct FmtQ4K {
    static constexpr int BLOCK_BYTES = Q4K_BYTES;
    static constexpr int BS_PER_BLOCK = 8;  // one block sum per 32-element sub-block
    // shared-memory row stride for CW blocks per row: an odd multiple of 16 bytes, so the 8 rows of
    // an ldmatrix land in 8 distinct 16-byte bank groups
    __host__ __device__ static constexpr int row_stride(int cw) { return cw * Q4K_BYTES + 16; }
    __device__ static __forceinline__ int bs_value(const int16_t* bs16, int i) { return (int)bs16[2 * i] + (int)bs16[2 * i + 1]; }
    __device__ static __forceinline__ void bs_split(int v, uint8_t& hi, uint8_t& lo) {
        lo = (uint8_t)(v & 127);
        hi = (uint8_t)((v >> 7) & 0xff);
    }

    // NTL = token tiles (of 8) that hold rows
    template <int NT, int NTL, int RS>
    __device__ static __forceinline__ void block(uint32_t tile, int wblk, const BlockArgs& A, int lane, float (&f)[NT][4]) {
        const int g = lane >> 2, t = lane & 3;
        const uint32_t rowA = tile + g * RS + wblk * BLOCK_BYTES;
        const uint4 ha = lds128(rowA), hb = lds128(rowA + 8 * RS);
        const float dA = half_bits_to_float((uint16_t)(ha.x & 0xffff)), mnA = half_bits_to_float((uint16_t)(ha.x >> 16));
        const float dB = half_bits_to_float((uint16_t)(hb.x & 0xffff)), mnB = half_bits_to_float((uint16_t)(hb.x >> 16));
        uint32_t scA[2], mA[2], scB[2], mB[2];  // [0]: sub-blocks 0..3, [1]: 4..7, one byte each
        scA[0] = ha.y & 0x3f3f3f3fu;
        mA[0] = ha.z & 0x3f3f3f3fu;
        scA[1] = (ha.w & 0x0f0f0f0fu) | (((ha.y >> 6) & 0x03030303u) << 4);
        mA[1] = ((ha.w >> 4) & 0x0f0f0f0fu) | (((ha.z >> 6) & 0x03030303u) << 4);
        scB[0] = hb.y & 0x3f3f3f3fu;
        mB[0] = hb.z & 0x3f3f3f3fu;
        scB[1] = (hb.w & 0x0f0f0f0fu) | (((hb.y >> 6) & 0x03030303u) << 4);
        mB[1] = ((hb.w >> 4) & 0x0f0f0f0fu) | (((hb.z >> 6) & 0x03030303u) << 4);
        int c[NTL][4];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) c[nt][i] = 0;
        // ldmatrix lane addressing: matrices = (rows 0-7 | rows 8-15) x (bytes 0-15 | 16-31) of a 64-element group
        const uint32_t a_addr = tile + ((lane & 7) + ((lane >> 3) & 1) * 8) * RS + wblk * BLOCK_BYTES + 16 + 16 * (lane >> 4);
        const uint32_t b_addr = A.act + (lane & 7) * A.act_stride + A.kblk_local * 256 + 16 * (lane >> 3);
#pragma unroll
        for (int grp = 0; grp < 4; ++grp) {
            const int jl = 2 * grp, jh = 2 * grp + 1;  // sub-block ids of the low / high nibbles
            uint32_t a[4], alo[4], ahi[4];
            ldmatrix_x4(a, a_addr + 32 * grp);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                alo[i] = a[i] & 0x0f0f0f0fu;
                ahi[i] = (a[i] >> 4) & 0x0f0f0f0fu;
            }
            const int sAl = byte_u(scA[jl >> 2], jl & 3), sAh = byte_u(scA[jh >> 2], jh & 3);
            const int sBl = byte_u(scB[jl >> 2], jl & 3), sBh = byte_u(scB[jh >> 2], jh & 3);
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                uint32_t b[4];
                ldmatrix_x4(b, b_addr + nt * 8 * A.act_stride + 64 * grp);
                int p[4], q[4];
                mma_s8_k32_z(p, alo, b[0], b[1]);
                mma_s8_k32_z(q, ahi, b[2], b[3]);
                c[nt][0] += sAl * p[0] + sAh * q[0];
                c[nt][1] += sAl * p[1] + sAh * q[1];
                c[nt][2] += sBl * p[2] + sBh * q[2];
                c[nt][3] += sBl * p[3] + sBh * q[3];
            }
        }
        // A operand of the min product: k = sub-block id, lanes t = 0, 1 carry the 8 packed mins
        const uint32_t am0 = t == 0 ? mA[0] : (t == 1 ? mA[1] : 0u);
        const uint32_t am1 = t == 0 ? mB[0] : (t == 1 ? mB[1] : 0u);
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) {
            const uint32_t boff = (nt * 8 + g) * A.bs_stride + A.kblk_local * 8 + 4 * (t & 1);
            const uint32_t bh = lds32(A.bs_hi + boff), bl = lds32(A.bs_lo + boff);
            const float d8a = ldsf(A.act_scale + 4 * ((nt * 8 + 2 * t) * A.scale_stride + A.kblk_local));
            const float d8b = ldsf(A.act_scale + 4 * ((nt * 8 + 2 * t + 1) * A.scale_stride + A.kblk_local));
            int ch[4], cl[4];
            mma_s8_k16_z(ch, am0, am1, bh);
            mma_s8_k16_z(cl, am0, am1, bl);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float d8 = (i & 1) ? d8b : d8a;
                const float dw = (i >> 1) ? dB : dA, mw = (i >> 1) ? mnB : mnA;
                f[nt][i] = fmaf(d8 * dw, (float)c[nt][i], f[nt][i]);
                f[nt][i] = fmaf(-(d8 * mw), (float)(128 * ch[i] + cl[i]), f[nt][i]);
            }
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Q6_K (210 B per 256): 128 B low nibbles, 64 B high 2-bit pairs, 16 int8 scales, f16 d.
// A block is only 2-byte aligned inside the row, so its words are read as one 32-bit or two
// 16-bit shared loads depending on the (warp-uniform) parity of the block index.
// The quants are used unsigned (0..63); the reference's "- 32" becomes
//   - 32 * sum_j scale_j * bsum_j(token),
// itself a [16 x 16] by [16 x 8] integer product done with two more MMAs on the activation block
// sums split into a signed high byte and an unsigned low byte.
// ---------------------------------------------------------------------------------------------
struct FmtQ6K {
    static constexpr int BLOCK_BYTES = Q6K_BYTES;
    static constexpr int BS_PER_BLOCK = 16;  // one block sum per 16-element sub-block
    // stride in words must be 4 mod 8 so that rows g = 0..7 at word t = 0..3 never share a bank
    __host__ __device__ static constexpr int row_stride(int cw) {
        return ((cw * Q6K_BYTES / 4) % 8 == 4) ? cw * Q6K_BYTES : cw * Q6K_BYTES + 16;
    }
    __device__ static __forceinline__ int bs_value(const int16_t* bs16, int i) { return (int)bs16[i]; }
    __device__ static __forceinline__ void bs_split(int v, uint8_t& hi, uint8_t& lo) {
        lo = (uint8_t)(v & 0xff);
        hi = (uint8_t)((v >> 8) & 0xff);  // arithmetic shift: signed high byte
    }

    template <bool ODD>
    __device__ static __forceinline__ uint32_t ld32(uint32_t addr) {
        if (ODD) return lds16(addr) | (lds16(addr + 2) << 16);
        return lds32(addr);
    }

    template <int NT, int NTL, int RS, bool ODD>
    __device__ static __forceinline__ void block_impl(uint32_t tile, int wblk, const BlockArgs& A, int lane, float (&f)[NT][4]) {
        const int g = lane >> 2, t = lane & 3;
        const uint32_t rowA = tile + g * RS + wblk * BLOCK_BYTES;
        const uint32_t rowB = rowA + 8 * RS;
        const float dA = half_bits_to_float((uint16_t)lds16(rowA + 208));
        const float dB = half_bits_to_float((uint16_t)lds16(rowB + 208));
        uint32_t scA[4], scB[4];  // 16 int8 scales per row
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            scA[i] = ld32<ODD>(rowA + 192 + 4 * i);
            scB[i] = ld32<ODD>(rowB + 192 + 4 * i);
        }
        int c[NTL][4];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) c[nt][i] = 0;
        const uint32_t b_addr = A.act + (lane & 7) * A.act_stride + A.kblk_local * 256 + 16 * (lane >> 3);

#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // hq[lr][x]: for l-range lr (l = 16*lr + 4t .. +3), the 2-bit highs of quarter x moved to bits 4..5
            uint32_t hqA[2][4], hqB[2][4];
#pragma unroll
            for (int lr = 0; lr < 2; ++lr) {
                const uint32_t qa = ld32<ODD>(rowA + 128 + 32 * h + 16 * lr + 4 * t);
                const uint32_t qb = ld32<ODD>(rowB + 128 + 32 * h + 16 * lr + 4 * t);
                hqA[lr][0] = (qa << 4) & 0x30303030u;
                hqA[lr][1] = (qa << 2) & 0x30303030u;
                hqA[lr][2] = qa & 0x30303030u;
                hqA[lr][3] = (qa >> 2) & 0x30303030u;
                hqB[lr][0] = (qb << 4) & 0x30303030u;
                hqB[lr][1] = (qb << 2) & 0x30303030u;
                hqB[lr][2] = qb & 0x30303030u;
                hqB[lr][3] = (qb >> 2) & 0x30303030u;
            }
            // low nibbles: ql[64h + 32*(x&1) + 16*lr + 4t ..], nibble (x >> 1)
            uint32_t qlA[2][2], qlB[2][2];  // [x & 1][lr]
#pragma unroll
            for (int xo = 0; xo < 2; ++xo)
#pragma unroll
                for (int lr = 0; lr < 2; ++lr) {
                    qlA[xo][lr] = ld32<ODD>(rowA + 64 * h + 32 * xo + 16 * lr + 4 * t);
                    qlB[xo][lr] = ld32<ODD>(rowB + 64 * h + 32 * xo + 16 * lr + 4 * t);
                }
#pragma unroll
            for (int y = 0; y < 2; ++y) {  // 64 elements = quarters 2y, 2y+1 = four 16-element sub-blocks
                uint32_t aA[4], aB[4];  // [2*(x&1) + lr]
                int sA[4], sB[4];
#pragma unroll
                for (int xo = 0; xo < 2; ++xo) {
                    const int x = 2 * y + xo;  // quarter: elements 128h + 32x .. +31; low nibbles for x < 2
#pragma unroll
                    for (int lr = 0; lr < 2; ++lr) {
                        const uint32_t la = (x >> 1) ? (qlA[x & 1][lr] >> 4) : qlA[x & 1][lr];
                        const uint32_t lb = (x >> 1) ? (qlB[x & 1][lr] >> 4) : qlB[x & 1][lr];
                        aA[2 * xo + lr] = (la & 0x0f0f0f0fu) | hqA[lr][x];
                        aB[2 * xo + lr] = (lb & 0x0f0f0f0fu) | hqB[lr][x];
                        const int j = 8 * h + 2 * x + lr;  // sub-block id
                        sA[2 * xo + lr] = byte_s(scA[j >> 2], j & 3);
                        sB[2 * xo + lr] = byte_s(scB[j >> 2], j & 3);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) {
                    uint32_t b[4];  // int8 activations of the four sub-blocks
                    ldmatrix_x4(b, b_addr + nt * 8 * A.act_stride + 128 * h + 64 * y);
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4) {
                        int p[4];
                        mma_s8_k16_z(p, aA[s4], aB[s4], b[s4]);
                        c[nt][0] += sA[s4] * p[0];
                        c[nt][1] += sA[s4] * p[1];
                        c[nt][2] += sB[s4] * p[2];
                        c[nt][3] += sB[s4] * p[3];
                    }
                }
            }
        }
        // offset term: corr[row][tok] = sum_j scale[row][j] * bsum[tok][j], bsum = 256 * hi + lo
        const uint32_t sa = scA[t], sb = scB[t];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) {
            const uint32_t boff = (nt * 8 + g) * A.bs_stride + A.kblk_local * 16 + 4 * t;
            const uint32_t bh = lds32(A.bs_hi + boff), bl = lds32(A.bs_lo + boff);
            int ch[4], cl[4];
            mma_s8_k16_z(ch, sa, sb, bh);
            mma_s8u8_k16_z(cl, sa, sb, bl);
            const float d8a = ldsf(A.act_scale + 4 * ((nt * 8 + 2 * t) * A.scale_stride + A.kblk_local));
            const float d8b = ldsf(A.act_scale + 4 * ((nt * 8 + 2 * t + 1) * A.scale_stride + A.kblk_local));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int isum = c[nt][i] - 32 * (256 * ch[i] + cl[i]);
                const float dd = ((i & 1) ? d8b : d8a) * ((i >> 1) ? dB : dA);
                f[nt][i] = fmaf(dd, (float)isum, f[nt][i]);
            }
        }
    }

    template <int NT, int NTL, int RS>
    __device__ static __forceinline__ void block(uint32_t tile, int wblk, const BlockArgs& A, int lane, float (&f)[NT][4]) {
        if ((wblk & 1) || (RS & 3))
            block_impl<NT, NTL, RS, true>(tile, wblk, A, lane, f);
        else
            block_impl<NT, NTL, RS, false>(tile, wblk, A, lane, f);
    }
};

// ---------------------------------------------------------------------------------------------
// Work decomposition shared by producer and consumers (pure function of the kernel arguments and
// the expert offsets, so every warp walks the same sequence).
// ---------------------------------------------------------------------------------------------
struct StreamParams {
    ExpertPtrs wa, wb;
    const uint32_t* offsets;
    const uint32_t* row_of;
    const int8_t* aq;
    const float* ascale;
    const int16_t* absum;
    float* out;
    int* status;
    int64_t out_split_stride;  // elements between the partial outputs of consecutive K-splits
    int E, K, N, kb, n_chunks, splits, MT, stages;
    int tile_n;                // output rows per item: 16, or 8 for gate_up
    int chunk_start[5];        // split s covers chunks [chunk_start[s], chunk_start[s+1])
    int act_stride;            // bytes per token row of the resident activations
    int scale_stride;          // floats per token row of the resident activation scales
    int bs_stride;             // bytes per token row of each block-sum plane
    uint32_t off_act, off_scale, off_bs_hi, off_bs_lo, off_red, off_stage, stage_bytes;
};

struct WorkItem {
    int e, grp, split, tile;
};

struct Walker {
    const StreamParams& P;
    const uint32_t* offs;  // expert offsets (shared memory copy)
    int tiles;
    long long pos, hi;     // cost position of the next item, end of this CTA's range
    int gidx, e, grp, ng_e, split, tile;

    __device__ Walker(const StreamParams& p, const uint32_t* offsets_sm, int cta, int n_cta) : P(p), offs(offsets_sm) {
        tiles = P.N / P.tile_n;
        int gtot = 0;
        for (int i = 0; i < P.E; ++i) gtot += (int)((offs[i + 1] - offs[i] + P.MT - 1) / P.MT);
        const long long gcost = (long long)tiles * P.n_chunks;
        const long long ctot = gcost * gtot;
        const long long lo = ctot * cta / n_cta;
        hi = ctot * (cta + 1) / n_cta;
        e = grp = ng_e = 0;
        // first item whose start cost is >= lo
        gidx = (int)(lo / gcost);
        long long rem = lo % gcost;
        split = 0;
        tile = 0;
        for (int s = 0; s < P.splits; ++s) {
            const long long s_lo = (long long)tiles * P.chunk_start[s], s_hi = (long long)tiles * P.chunk_start[s + 1];
            if (rem < s_hi) {
                const int cps = P.chunk_start[s + 1] - P.chunk_start[s];
                split = s;
                tile = rem <= s_lo ? 0 : (int)((rem - s_lo + cps - 1) / cps);
                break;
            }
        }
        normalize();
        pos = item_cost_pos();
        // locate (expert, token group) of gidx
        grp = 0;
        ng_e = 0;
        int acc = 0;
        for (e = 0; e < P.E; ++e) {
            ng_e = (int)((offs[e + 1] - offs[e] + P.MT - 1) / P.MT);
            if (gidx < acc + ng_e) {
                grp = gidx - acc;
                break;
            }
            acc += ng_e;
        }
    }
    __device__ void normalize() {
        if (tile >= tiles) {
            tile = 0;
            ++split;
        }
        if (split >= P.splits) {
            split = 0;
            ++gidx;
            ++grp;
        }
    }
    __device__ long long item_cost_pos() const {
        return (long long)gidx * tiles * P.n_chunks + (long long)tiles * P.chunk_start[split] +
               (long long)tile * (P.chunk_start[split + 1] - P.chunk_start[split]);
    }
    __device__ bool valid() const { return pos < hi && e < P.E; }
    __device__ WorkItem item() const { return WorkItem{e, grp, split, tile}; }
    __device__ void next() {
        ++tile;
        const int g0 = gidx;
        normalize();
        if (gidx != g0) {
            while (e < P.E && grp >= ng_e) {  // move to the next expert that has rows
                grp = 0;
                ++e;
                ng_e = e < P.E ? (int)((offs[e + 1] - offs[e] + P.MT - 1) / P.MT) : 0;
            }
        }
        pos = item_cost_pos();
    }
};

// CW = consumer warps = 256-element blocks per stage chunk.

template <class F, bool GATE_UP, int NT, int CW>
__global__ void __launch_bounds__(32 * (1 + CW), 1) expert_stream_kernel(const __grid_constant__ StreamParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t full_bar[8], empty_bar[8];
    __shared__ uint32_t s_offs[CANDLE_MOE_MAX_EXPERTS + 1];
    __shared__ int s_abort;
    __shared__ int s_rows[16];  // activation row of each token of the resident group (-1: none)
    constexpr int MT = 8 * NT;
    constexpr int RS = F::row_stride(CW);
    constexpr int CHUNK_BYTES = CW * F::BLOCK_BYTES;
    constexpr int N_CONS = 32 * CW;
    constexpr int TILE_N = GATE_UP ? 8 : 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();

    for (int i = threadIdx.x; i <= P.E; i += blockDim.x) s_offs[i] = P.offsets[i];
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < P.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], CW);
        }
        fence_barrier_init();
    }
    __syncthreads();
    volatile int* abort_flag = &s_abort;

    Walker wk(P, s_offs, blockIdx.x, gridDim.x);
    const size_t row_bytes = (size_t)P.kb * F::BLOCK_BYTES;
    uint8_t* stage0 = smem + P.off_stage;
    const uint32_t stage_addr0 = smem_u32(stage0);

    if (warp == 0) {
        // ================= producer: lane r < 16 copies weight row r of the tile =================
        uint32_t it = 0;
        for (; wk.valid(); wk.next()) {
            const WorkItem w = wk.item();
            const bool active = lane < TILE_ROWS;
            const uint8_t* src_row = nullptr;
            if (active) {
                if (GATE_UP)
                    src_row = (lane < 8 ? P.wa.p[w.e] : P.wb.p[w.e]) + (size_t)(w.tile * TILE_N + (lane & 7)) * row_bytes;
                else
                    src_row = P.wa.p[w.e] + (size_t)(w.tile * TILE_N + lane) * row_bytes;
            }
            for (int ch = P.chunk_start[w.split]; ch < P.chunk_start[w.split + 1]; ++ch, ++it) {
                const int s = it % P.stages;
                const uint32_t ph = (it / P.stages) & 1;
                if (it >= (uint32_t)P.stages) mbar_wait(&empty_bar[s], ph ^ 1, abort_flag);
                const int blocks = min(CW, P.kb - ch * CW);
                const uint32_t bytes = (uint32_t)blocks * F::BLOCK_BYTES;
                if (lane == 0) mbar_expect_tx(&full_bar[s], bytes * TILE_ROWS);
                __syncwarp();
                if (active && !*abort_flag)
                    bulk_g2s(stage0 + (size_t)s * P.stage_bytes + lane * RS, src_row + (size_t)ch * CHUNK_BYTES, bytes,
                             &full_bar[s]);
            }
        }
        // do not leave while copies into this CTA's shared memory may still be in flight
        if (lane == 0) {
            const uint32_t n = it < (uint32_t)P.stages ? it : (uint32_t)P.stages;
            for (uint32_t j = 0; j < n; ++j) {
                const uint32_t last = it - 1 - j;
                mbar_wait(&full_bar[last % P.stages], (last / P.stages) & 1, abort_flag);
            }
        }
    } else {
        // ================= consumers =================
        const int cw = warp - 1;            // K-slice of this warp inside a chunk
        const int ctid = threadIdx.x - 32;  // 0 .. N_CONS-1
        uint8_t* act = smem + P.off_act;
        float* act_scale = reinterpret_cast<float*>(smem + P.off_scale);
        uint8_t* bs_hi = smem + P.off_bs_hi;
        uint8_t* bs_lo = smem + P.off_bs_lo;
        float* red0 = reinterpret_cast<float*>(smem + P.off_red);
        constexpr int RED_FLOATS = CW * MT * RED_PAD;
        uint32_t it = 0, n_item = 0;
        int cur_e = -1, cur_grp = -1, cur_split = -1;
        for (; wk.valid(); wk.next(), ++n_item) {
            const WorkItem w = wk.item();
            const uint32_t p_base = s_offs[w.e] + (uint32_t)w.grp * MT;
            const uint32_t p_end = min(s_offs[w.e + 1], p_base + MT);
            const int blk0 = P.chunk_start[w.split] * CW;                      // first block of this split
            const int nblk = min(P.kb, P.chunk_start[w.split + 1] * CW) - blk0;  // blocks in this split
            if (w.e != cur_e || w.grp != cur_grp || w.split != cur_split) {
                // ---- make the int8 rows, scales and block sums of this token group resident ----
                cur_e = w.e;
                cur_grp = w.grp;
                cur_split = w.split;
                consumer_sync(N_CONS);
                if (ctid < MT) {
                    const uint32_t pp = p_base + ctid;
                    s_rows[ctid] = pp < p_end ? (P.row_of ? (int)P.row_of[pp] : (int)pp) : -1;
                }
                consumer_sync(N_CONS);
                const int vec_per_row = nblk * 16;  // 16-byte vectors per token row
#pragma unroll 4
                for (int idx = ctid; idx < MT * vec_per_row; idx += N_CONS) {
                    const int j = idx / vec_per_row, v = idx - j * vec_per_row;
                    const int row = s_rows[j];
                    int4 val = make_int4(0, 0, 0, 0);
                    if (row >= 0) val = *reinterpret_cast<const int4*>(P.aq + (int64_t)row * P.K + (int64_t)blk0 * 256 + 16 * v);
                    *reinterpret_cast<int4*>(act + j * P.act_stride + 16 * v) = val;
                }
                for (int idx = ctid; idx < MT * nblk; idx += N_CONS) {
                    const int j = idx / nblk, b = idx - j * nblk;
                    const int row = s_rows[j];
                    act_scale[j * P.scale_stride + b] = row >= 0 ? P.ascale[(int64_t)row * P.kb + blk0 + b] : 0.f;
                }
                {
                    const int per_row = nblk * F::BS_PER_BLOCK;
                    for (int idx = ctid; idx < MT * per_row; idx += N_CONS) {
                        const int j = idx / per_row, b = idx - j * per_row;
                        const int row = s_rows[j];
                        const int v = row >= 0 ? F::bs_value(P.absum + (int64_t)row * (P.K / 16) + blk0 * 16, b) : 0;
                        uint8_t hi, lo;
                        F::bs_split(v, hi, lo);
                        bs_lo[j * P.bs_stride + b] = lo;
                        bs_hi[j * P.bs_stride + b] = hi;
                    }
                }
                consumer_sync(N_CONS);
            }

            BlockArgs bargs;
            bargs.act = smem_u32(act);
            bargs.act_scale = smem_u32(act_scale);
            bargs.bs_hi = smem_u32(bs_hi);
            bargs.bs_lo = smem_u32(bs_lo);
            bargs.act_stride = P.act_stride;
            bargs.scale_stride = P.scale_stride;
            bargs.bs_stride = P.bs_stride;
            const int ntiles = (int)(p_end - p_base + 7) / 8;  // token tiles that hold rows
            float f[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) f[nt][i] = 0.f;

            for (int ch = P.chunk_start[w.split]; ch < P.chunk_start[w.split + 1]; ++ch, ++it) {
                const int s = it % P.stages;
                const bool ok = mbar_wait(&full_bar[s], (it / P.stages) & 1, abort_flag);
                const int blk = ch * CW + cw;
                if (ok && blk < P.kb) {
                    bargs.kblk_local = blk - blk0;
                    const uint32_t tile_addr = stage_addr0 + (uint32_t)s * P.stage_bytes;
                    if (NT == 1 || ntiles == 1)
                        F::template block<NT, 1, RS>(tile_addr, cw, bargs, lane, f);
                    else
                        F::template block<NT, NT, RS>(tile_addr, cw, bargs, lane, f);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);
            }

            // ---- the CW K-slices of the tile meet in shared memory (two buffers, one barrier per
            // item: a buffer is rewritten only after every warp has passed the next item's barrier) ----
            float* red = red0 + (n_item & 1) * RED_FLOATS;
            {
                const int g = lane >> 2, t = lane & 3;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int tok = nt * 8 + 2 * t + (i & 1), row = g + 8 * (i >> 1);
                        red[(cw * MT + tok) * RED_PAD + row] = f[nt][i];
                    }
            }
            consumer_sync(N_CONS);
            // four threads per output: each adds a quarter of the K-slices, two shuffles finish the sum
            for (int idx = ctid; idx < MT * TILE_N * 4; idx += N_CONS) {
                const int o4 = idx >> 2, part = idx & 3;
                const int tok = o4 / TILE_N, row = o4 - tok * TILE_N;
                float va = 0.f, vb = 0.f;
#pragma unroll
                for (int sw = 0; sw < CW / 4; ++sw) {
                    const int slice = part * (CW / 4) + sw;
                    va += red[(slice * MT + tok) * RED_PAD + row];
                    if (GATE_UP) vb += red[(slice * MT + tok) * RED_PAD + row + 8];
                }
                va += __shfl_xor_sync(0xffffffffu, va, 1);
                va += __shfl_xor_sync(0xffffffffu, va, 2);
                if (GATE_UP) {
                    vb += __shfl_xor_sync(0xffffffffu, vb, 1);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 2);
                }
                if (part == 0 && p_base + tok < p_end) {
                    const int64_t o = (int64_t)(p_base + tok) * P.N + w.tile * TILE_N + row;
                    if (GATE_UP)
                        P.out[o] = silu_f(va) * vb;
                    else
                        P.out[(int64_t)w.split * P.out_split_stride + o] = va;
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_abort) atomicOr(P.status, 1);
}

int g_max_smem = -1;
int g_num_sms = -1;

cudaError_t device_limits() {
    if (g_max_smem >= 0) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    int v = 0, n = 0;
    e = cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    g_max_smem = v;
    g_num_sms = n;
    return cudaSuccess;
}

template <class F, bool GATE_UP, int NT, int CW>
cudaError_t launch_one(cudaStream_t st, const StreamParams& P, size_t smem_bytes) {
    auto kfn = expert_stream_kernel<F, GATE_UP, NT, CW>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
    if (e != cudaSuccess) return e;
    return launch_k(kfn, dim3(g_num_sms), dim3(32 * (1 + CW)), smem_bytes, st, P);
}

template <class F, int CW>
cudaError_t launch_nt(cudaStream_t st, bool gate_up, int NT, const StreamParams& P, size_t smem_bytes) {
    if (gate_up) return NT == 1 ? launch_one<F, true, 1, CW>(st, P, smem_bytes) : launch_one<F, true, 2, CW>(st, P, smem_bytes);
    return NT == 1 ? launch_one<F, false, 1, CW>(st, P, smem_bytes) : launch_one<F, false, 2, CW>(st, P, smem_bytes);
}

}  // namespace

__device__ int g_stream_status = 0;

// Plans and launches the streaming kernel; returns cudaErrorNotSupported when the shape is outside
// what the streaming form takes (the caller then uses the row-per-warp form).
cudaError_t launch_expert_stream(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype,
                                 int E, int K, int N, const uint32_t* offsets, const uint32_t* row_of,
                                 int64_t max_rows_per_expert, const int8_t* aq, const float* ascale,
                                 const int16_t* absum, float* out, int* n_splits_out, int64_t split_stride,
                                 int max_splits) {
    if (dtype != CANDLE_GGML_Q4K && dtype != CANDLE_GGML_Q6K) return cudaErrorNotSupported;
    const int tile_n = gate_up ? 8 : 16;
    if (N % tile_n != 0 || K % 256 != 0) return cudaErrorNotSupported;
    const int kb = K / 256;
    if (dtype == CANDLE_GGML_Q6K && kb % 8 != 0) return cudaErrorNotSupported;  // rows must stay 16-byte aligned
    cudaError_t e = device_limits();
    if (e != cudaSuccess) return e;
    const int NT = max_rows_per_expert <= 8 ? 1 : 2;
    const int MT = 8 * NT;
    // blocks per stage chunk = consumer warps: full 4096-element rows for Q4_K (2.3 KB copies)
    const int CW = (dtype == CANDLE_GGML_Q4K && kb >= 16) ? 16 : 8;
    const int n_chunks = (kb + CW - 1) / CW;
    const int row_stride = dtype == CANDLE_GGML_Q4K ? FmtQ4K::row_stride(CW) : FmtQ6K::row_stride(CW);
    const uint32_t stage_bytes = (uint32_t)(TILE_ROWS * row_stride);
    const int bs_per_block = dtype == CANDLE_GGML_Q4K ? FmtQ4K::BS_PER_BLOCK : FmtQ6K::BS_PER_BLOCK;

    StreamParams P{};
    P.wa = wa;
    P.wb = wb;
    for (int splits = 1; splits <= max_splits; ++splits) {
        if (splits > n_chunks) break;
        if (gate_up && splits > 1) break;  // the gate needs the full sum before silu
        const int cps = (n_chunks + splits - 1) / splits;  // chunks of the largest split
        const int ks_blocks = min(cps * CW, kb);
        uint32_t off = 0;
        auto take = [&](uint32_t bytes) {
            off = (off + 127u) & ~127u;
            const uint32_t o = off;
            off += bytes;
            return o;
        };
        P.act_stride = ks_blocks * 256 + 16;
        P.scale_stride = ks_blocks;
        P.bs_stride = ks_blocks * bs_per_block + 16;
        while ((P.bs_stride / 4) % 8 != 4) P.bs_stride += 4;  // token rows g = 0..7 land in distinct banks
        P.off_act = take((uint32_t)MT * P.act_stride);
        P.off_scale = take((uint32_t)MT * P.scale_stride * 4);
        P.off_bs_hi = take((uint32_t)MT * P.bs_stride);
        P.off_bs_lo = take((uint32_t)MT * P.bs_stride);
        P.off_red = take((uint32_t)(2 * CW * MT * RED_PAD * 4));
        off = (off + 1023u) & ~1023u;
        P.off_stage = off;
        const int avail = g_max_smem - (int)off - 2048;  // minus the static shared memory of the kernel
        int stages = avail / (int)stage_bytes;
        if (stages > 8) stages = 8;
        if (stages < 3) continue;  // try a finer K-split
        P.stages = stages;
        P.splits = splits;
        int cs = 0;
        for (int s = 0; s < splits; ++s) {
            P.chunk_start[s] = cs;
            const int rem_chunks = n_chunks - cs, rem_splits = splits - s;
            cs += (rem_chunks + rem_splits - 1) / rem_splits;
        }
        P.chunk_start[splits] = n_chunks;
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
        P.n_chunks = n_chunks;
        P.MT = MT;
        P.tile_n = tile_n;
        P.stage_bytes = stage_bytes;
        void* sp = nullptr;
        e = cudaGetSymbolAddress(&sp, g_stream_status);
        if (e != cudaSuccess) return e;
        P.status = static_cast<int*>(sp);
        const size_t smem_bytes = (size_t)off + (size_t)stages * stage_bytes;
        if (n_splits_out) *n_splits_out = splits;
        if (dtype == CANDLE_GGML_Q4K)
            return CW == 16 ? launch_nt<FmtQ4K, 16>(st, gate_up, NT, P, smem_bytes) : launch_nt<FmtQ4K, 8>(st, gate_up, NT, P, smem_bytes);
        return launch_nt<FmtQ6K, 8>(st, gate_up, NT, P, smem_bytes);
    }
    return cudaErrorNotSupported;
}

cudaError_t stream_status_ptr(int** out) {
    void* sp = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&sp, g_stream_status);
    *out = static_cast<int*>(sp);
    return e;
}

cudaError_t read_stream_status(int* out) {
    return cudaMemcpyFromSymbol(out, g_stream_status, sizeof(int));
}

cudaError_t reset_stream_status() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
}

namespace {
// Waits on a barrier that nothing completes: the bounded wait gives up after `limit` polls and the kernel returns.
__global__ void selftest_wait_kernel(int limit, int* status) {
    __shared__ uint64_t bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    mbar_wait(&bar, 0, &s_abort, limit);
    __syncthreads();
    if (threadIdx.x == 0 && s_abort) atomicOr(status, 1);
}
}  // namespace

cudaError_t launch_selftest_wait(cudaStream_t st, int limit) {
    int* status = nullptr;
    const cudaError_t e = stream_status_ptr(&status);
    if (e != cudaSuccess) return e;
    selftest_wait_kernel<<<1, 64, 0, st>>>(limit, status);
    return cudaGetLastError();
}

}  // namespace cmoe
