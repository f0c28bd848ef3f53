// Grouped expert products for large batches (prefill): tcgen05 tensor cores, operands and accumulators
// in tensor memory.
//
// out[p, n] = W_e[n, :] . act[row(p), :] for all grouped positions p of every expert, as a grouped GEMM
// over tiles of 128 weight rows x 128 grouped positions.  The integers are the reference's
// (candle-core/src/quantized/k_quants.rs:1205-1285 Q4_K, :1520-1600 Q6_K): activations are the int8
// Q8K rows, and the weight operand holds (sub-block scale) x (quant), both exact in fp16, multiplied by
// `tcgen05.mma kind::f16` with fp32 accumulation in tensor memory -- exact while a 256-element block's
// sum stays below 2^24, which it does by a wide margin for real data.  After every 256-element block
// the accumulator is drained and scaled by d_w(row, block) * d8(position, block) on the CUDA cores.
//   Q4_K: operand sc_j * q (at most 63 * 15); the min term joins the same accumulator as three tf32
//         steps per block against dmin / d (see prep_gemm_b_kernel).
//   Q6_K: sc_j * (q - 32) reaches 4096 and is not always an fp16 integer, so the int8 scale is split
//         into ceil(sc/2) + floor(sc/2) and the slab is multiplied twice (each half at most 32 * 64 =
//         2048: exact).  Reads the repacked layout of the decode kernels (16-byte aligned pieces; the
//         210-byte GGUF blocks are only 2-byte aligned).
//
// One CTA per SM, persistent over tiles, warp-specialised (20 warps, five warpgroups):
//   warps 0-7   epilogue: drain TMEM (tcgen05.ld, next load in flight) once per block, scale, keep 64
//               columns per thread in registers (128 registers per thread, taken from the last
//               warpgroup with setmaxnreg); at the end of a tile apply the SiLU gate and store
//   warps 8-15  unpack the weight nibbles of [128 rows x 64 k] to fp16 x scale with one HFMA2 per two
//               elements and store them straight into TENSOR MEMORY (tcgen05.st): the A operand never
//               touches shared memory, whose bandwidth the B operand needs
//   warp  18    TMA: the activation operand, [128 positions x 64 k] fp16 boxes, 128-byte swizzle; one
//               stage is a whole 256-wide block (four boxes + the min-term box), two stages
//   warp  19    issues the MMAs (A from TMEM, B from shared memory) and commits to mbarriers; the whole
//               warp walks the loop with warp-uniform operands, one elected lane issues
// Tensor memory: two main accumulators (2 x 128 columns: the MMAs of block b+1 overlap the drain of
// block b) and a 256-column ring of weight-operand slabs, handed over in pairs.  gate_up interleaves
// rows of W1 and W3 (tile row 2i = W1 row, 2i+1 = W3 row) so the two factors of silu(w1 x) * (w3 x)
// sit in neighbouring lanes and meet with one shuffle.
// Every mbarrier wait is bounded (see stream_common.cuh); nothing here uses cluster multicast.
#include <algorithm>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include "common.cuh"
#include "tc5_common.cuh"

namespace cmoe {

namespace {

constexpr int G_TILE_M = 128, G_SLAB_K = 64;  // the position tile (N) is a template parameter: 128, or 32 for small batches
constexpr int G_PAD_ROWS = 128;                // zero rows after the last position, so that no box leaves the buffers
constexpr int G_W_STAGES_MAX = 4;  // raw weight blocks in flight per CTA (narrow position tiles leave room for a deep ring)
constexpr int G_B_STAGES = 2;   // in shared memory, one 256-wide block each (four slabs + the min-term box for Q4_K)
constexpr int G_TILE_BYTES = G_TILE_M * G_SLAB_K * 2;  // one [128 x 64] fp16 (or [128 x 32] tf32) operand tile, 16 KB
constexpr int G_EPI_WARPS = 8, G_DQ_WARPS = 8;
// Warp roles.  The MMA and TMA warps take the highest indices: measured, their short instruction streams
// are served far better there than at the lowest ones (1.75x on the whole kernel).
constexpr int G_WARP_EPI0 = 0, G_WARP_DQ0 = G_WARP_EPI0 + G_EPI_WARPS, G_WARP_LOAD = 16, G_WARP_TMA = 18, G_WARP_MMA = 19;
constexpr int G_THREADS = 32 * 20;  // five warpgroups: 2 epilogue, 2 unpack, 1 with the TMA and MMA warps (+ 2 idle)
constexpr int G_REGS_EPI = 128, G_REGS_MISC = 32;  // budgets after the trade: 2 * 128 + 2 * 96 + 32 = 5 * 96, the launch allocation
constexpr int G_TMEM_COLS = 512;
constexpr int G_TM_MAIN = 0;    // + 128 * buffer
constexpr int G_TM_A = 256;     // weight operand ring: columns 256..511
constexpr int Q6K_HTB_BYTES = 1680;  // repacked half-tile block: 8 rows x 256 elements (expert_direct.cu)

// ---------------------------------------------------------------------------------------------
// Operand preparation: the int8 activation rows in grouped order as fp16 (B operand), the block scales
// transposed to [block][position], and the activation side of the Q4_K min term (below).
// Inside every group of 4 k the order is (0, 2, 1, 3): the weight unpack produces that order for
// free (nibbles of bytes 0,2 and 1,3 convert pairwise), and a dot product does not care.
// Rows p >= P are zero padding so that a 128-row box never leaves the buffer.
//
// Min term of Q4_K (k_quants.rs:1262-1268): block b contributes d8[p,b] * (d[r,b] * M - dmin[r,b] * sum_j m_j bsum32_j)
// = d8 * d * (M - sum_j rho_j bsum32_j) with rho_j = dmin * m_j / d, so the min term joins the SAME accumulator
// as the integer main sum M: three more K=8 steps per block, kind::tf32 (fp32 exponent range, 10-bit
// mantissa).  rho_j (fp32) is split into tf32 terms r1 + r2 (to 2^-23), the integer bsum32 (at most 32 * 127,
// 12 bits) exactly into b1 + b2; the steps are r1 b1 + r2 b1 + r1 b2.  Per (position, block) the buffer holds
// 32 floats [b1 (8) | b1 (8) | b2 (8) | 0 (8)], matched by [r1 | r2 | r1 | -] on the weight side.  The main
// sum stays an exact integer until these last three steps; what they add in error is of the order of the
// reference's own f32 rounding (2^-23 of the min term).
// ---------------------------------------------------------------------------------------------
// nearest value with a 10-bit mantissa (the 13 low bits of the fp32 container zero)
__device__ __forceinline__ float tf32_head(float v) { return __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xffffe000u); }

__global__ void __launch_bounds__(256)
prep_gemm_b_kernel(const int8_t* __restrict__ aq, const float* __restrict__ ascale, const int16_t* __restrict__ absum,
                   const uint32_t* __restrict__ row_of, int P, int P_pad, int K, __half* __restrict__ bf16,
                   float* __restrict__ bmin, float* __restrict__ d8t) {
    pdl_trigger();
    pdl_wait();
    const int kb = K >> 8;
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (p, block)
    if (unit >= (int64_t)P_pad * kb) return;
    const int p = (int)(unit / kb), blk = (int)(unit - (int64_t)p * kb);
    uint4 o = make_uint4(0, 0, 0, 0);
    float bm = 0.f, d8 = 0.f;
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
        d8 = ascale[row * kb + blk];
        if (bmin) {
            const int j = lane & 7, part = lane >> 3;  // word: part 0, 1 = b1_j; part 2 = b2_j; part 3 = 0
            const int16_t* bs = absum + row * (K / 16) + blk * 16 + 2 * j;
            const float bv = (float)((int)bs[0] + (int)bs[1]);
            const float b1 = tf32_head(bv), b2 = bv - b1;  // exact: |bv| < 4096, so b2 is -1, 0 or 1
            bm = part == 2 ? b2 : (part == 3 ? 0.f : b1);
        }
    }
    *reinterpret_cast<uint4*>(bf16 + (int64_t)p * K + blk * 256 + lane * 8) = o;
    if (bmin) bmin[((int64_t)p * kb + blk) * 32 + lane] = bm;
    if (lane == 0) d8t[(int64_t)blk * P_pad + p] = d8;
}

// Q8_0 activations (int8 values, one f32 scale per 32, candle_moe_quantize_act) as the fp16 operand d * q, rows in
// grouped order, columns padded with zeros to K_pad (a multiple of 256); the per-block scale table is all ones.
// exact = 1: 64 d q as the fp16 pair (rounded product, exact residual), a row laid out [256 of part 0 | 256 of part 1]
// per block, and 1 / 64 in the scale table.
__global__ void __launch_bounds__(256)
prep_gemm_b_q80_kernel(const int8_t* __restrict__ aq, const float* __restrict__ ascale, const uint32_t* __restrict__ row_of, int P,
                       int P_pad, int K, int K_pad, int exact, __half* __restrict__ bf16, float* __restrict__ d8t) {
    pdl_trigger();
    pdl_wait();
    const int kb = K_pad >> 8;
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (p, block of 256)
    if (unit >= (int64_t)P_pad * kb) return;
    const int p = (int)(unit / kb), blk = (int)(unit - (int64_t)p * kb);
    uint4 o = make_uint4(0, 0, 0, 0), o1 = make_uint4(0, 0, 0, 0);
    const int k0 = blk * 256 + lane * 8;
    if (p < P && k0 < K) {  // K is a multiple of 32: a lane's eight values lie inside one 32-block
        const int64_t row = row_of ? (int64_t)row_of[p] : (int64_t)p;
        const uint2 v = *reinterpret_cast<const uint2*>(aq + row * K + k0);
        const int8_t* b = reinterpret_cast<const int8_t*>(&v);
        const float df = ascale[row * (K / 32) + (k0 >> 5)];  // an f16 value widened to f32
        __half r0[8], r1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float t = __fmul_rn(__fmul_rn((float)b[i], df), exact ? 64.0f : 1.0f);  // exact in f32: 8 x 11 bits
            r0[i] = __float2half_rn(t);
            r1[i] = __float2half_rn(__fsub_rn(t, __half2float(r0[i])));
        }
        __half2 h[4] = {__halves2half2(r0[0], r0[2]), __halves2half2(r0[1], r0[3]), __halves2half2(r0[4], r0[6]), __halves2half2(r0[5], r0[7])};
        __half2 g[4] = {__halves2half2(r1[0], r1[2]), __halves2half2(r1[1], r1[3]), __halves2half2(r1[4], r1[6]), __halves2half2(r1[5], r1[7])};
        o = *reinterpret_cast<uint4*>(h);
        o1 = *reinterpret_cast<uint4*>(g);
    }
    if (exact) {
        __half* dst = bf16 + (int64_t)p * (2 * K_pad) + blk * 512 + lane * 8;
        *reinterpret_cast<uint4*>(dst) = o;
        *reinterpret_cast<uint4*>(dst + 256) = o1;
    } else {
        *reinterpret_cast<uint4*>(bf16 + (int64_t)p * K_pad + blk * 256 + lane * 8) = o;
    }
    if (lane == 0) d8t[(int64_t)blk * P_pad + p] = exact ? 1.0f / 64.0f : 1.0f;
}

// Q8_0 GGUF rows [n][K / 32 blocks of 34 bytes] -> [n][K_pad / 256][272]: 256 int8 then 8 f16 scales, zeros past K.
// One warp per (row, 256-block); a lane moves eight values with 2-byte loads (the 34-byte blocks are 2-byte aligned).
__global__ void __launch_bounds__(256)
prepack_q80_kernel(const uint8_t* __restrict__ raw, int64_t n_rows, int K, int K_pad, uint8_t* __restrict__ dst) {
    const int kb = K_pad >> 8, lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= n_rows * kb) return;
    const int64_t row = unit / kb;
    const int blk = (int)(unit - row * kb);
    uint8_t* out = dst + unit * 272;
    const int k0 = blk * 256 + lane * 8;  // this lane's eight values
    uint16_t v[4] = {0, 0, 0, 0};
    if (k0 < K) {
        const uint8_t* b = raw + (row * (K / 32) + (k0 >> 5)) * Q8_0_BYTES;
        const uint16_t* q = reinterpret_cast<const uint16_t*>(b + 2 + (k0 & 31));
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = q[i];
        if ((lane & 3) == 0) reinterpret_cast<uint16_t*>(out + 256)[lane >> 2] = *reinterpret_cast<const uint16_t*>(b);
    } else if ((lane & 3) == 0) {
        reinterpret_cast<uint16_t*>(out + 256)[lane >> 2] = 0;
    }
    reinterpret_cast<uint2*>(out)[lane] = make_uint2((uint32_t)v[0] | ((uint32_t)v[1] << 16), (uint32_t)v[2] | ((uint32_t)v[3] << 16));
}

struct GemmParams {
    ExpertPtrs wa, wb;            // gate_up: W1 / W3, down: W2 (wb unused); GGUF blocks (Q4_K) or repacked (Q6_K)
    const uint32_t* offsets;      // [E + 1]
    const float* d8t;             // [kb][P_pad]
    float* out;                   // gate_up: hidden [P, N]; down: [P, N]
    const CUtensorMap* wmaps;     // device array [E][2]: raw blocks of W1 / W3 (or W2, second unused) as byte matrices
    int* status;
    int E, K, N, kb, P, P_pad;
    int m_tiles;                  // tiles along the weight rows (N / 64 for gate_up, N / 128 for down)
    int ksplit;                   // K splits (down only): partial outputs out + ks * split_stride, summed by the caller
    long long split_stride;
    uint32_t zero;                // 0 at run time, unknown to the compiler (see the release of a weight stage in the kernel)
};

__device__ __forceinline__ __half2 h2_bits(uint32_t v) { return *reinterpret_cast<const __half2*>(&v); }
__device__ __forceinline__ uint32_t bits_h2(__half2 v) { return *reinterpret_cast<const uint32_t*>(&v); }
// (1024 + byte b of w) in both halves: 0x64xx is 1024 + xx in fp16
__device__ __forceinline__ __half2 byte_magic2(uint32_t w, int b) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0x64646464u), "r"(0x4040u | (uint32_t)b | ((uint32_t)b << 8)));
    return h2_bits(r);
}
__device__ __forceinline__ uint4 ldg128(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t w4(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// ------------------------------------------------------------------------------------------------
// Q4_K, GGUF layout (144-byte blocks: d, dmin, 12 scale bytes, 128 nibble bytes).  Thread (row, h) owns
// bytes 16h..16h+15 of each 32-byte group: low nibbles are k = 16h.. of the 64-wide slab, high
// nibbles k = 32 + 16h..; one TMEM column holds two k, so the 16 + 16 values are columns 8h.. and 16+8h..
// ------------------------------------------------------------------------------------------------
struct GemmQ4K {
    static constexpr bool HAS_MIN = true;
    static constexpr int A_COLS = 32, A_PARTS = 1, A_PAIRS = 4;  // 8 slabs of 32 columns: two blocks in flight
    static constexpr int B_PARTS = 1;
    static constexpr bool STAGE_W = true;                         // raw blocks of the tile pass through shared memory
    static constexpr int W_ROW_BYTES = Q4K_BYTES;
    static constexpr int W_MAP_ELEM = 1;     // the tensor map of the raw blocks counts bytes
    static constexpr int W_STAGES_WIDE = 1;  // staged blocks that fit beside 128-wide activation stages
    struct Row {
        const uint8_t* p;
    };
    __device__ static __forceinline__ Row row(const uint8_t* w, int n, int kb) { return Row{w + (size_t)n * kb * Q4K_BYTES}; }
    struct Pre {
        uint4 hdr, q[4];
    };
    __device__ static __forceinline__ void load(Pre& pr, const Row& r, int blk, int h) {
        const uint8_t* b = r.p + (size_t)blk * Q4K_BYTES;
        pr.hdr = ldg128(b);
#pragma unroll
        for (int s = 0; s < 4; ++s) pr.q[s] = ldg128(b + 16 + 32 * s + 16 * h);
    }
    // the same pieces from the staged copy of the block (row_addr: shared-window address of the row's 144 bytes;
    // rows are 36 words apart, so the eight lanes of a 16-byte load phase cover all 32 banks once)
    __device__ static __forceinline__ void load_staged(Pre& pr, uint32_t row_addr, int h) {
        pr.hdr = lds128_o<0>(row_addr);
        const uint32_t rb = row_addr + 16 * h;
        pr.q[0] = lds128_o<16>(rb);
        pr.q[1] = lds128_o<48>(rb);
        pr.q[2] = lds128_o<80>(rb);
        pr.q[3] = lds128_o<112>(rb);
    }
    // one word of every vector load_staged fetched: a value that exists only when all of them have arrived
    __device__ static __forceinline__ uint32_t staged_words(const Pre& pr) {
        return pr.hdr.x | pr.q[0].x | pr.q[1].x | pr.q[2].x | pr.q[3].x;
    }
    // d (low half) and dmin (high half) of the block, fp16 bits
    __device__ static __forceinline__ uint32_t hdr_of(const Pre& pr) { return pr.hdr.x; }
    struct Ctx {
        uint32_t sc[2], mn[2];  // 6-bit scales / mins as bytes: [0] = sub-blocks 0..3, [1] = 4..7 (utils.rs:50-60)
    };
    __device__ static __forceinline__ void begin(const Pre& pr, Ctx& c) {
        const uint32_t s0 = pr.hdr.y, s1 = pr.hdr.z, s2 = pr.hdr.w;
        c.sc[0] = s0 & 0x3f3f3f3fu;
        c.mn[0] = s1 & 0x3f3f3f3fu;
        c.sc[1] = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
        c.mn[1] = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
        if ((pr.hdr.x & 0x7fffu) == 0) c.sc[0] = c.sc[1] = 0;  // d = 0: the block is its min term alone (see scale_of)
    }
    // The epilogue multiplies the block's accumulator by d; a block with d = 0 (and no main sum, above) is
    // scaled by dmin instead so that its min term survives, or by 1 if both are zero.
    __device__ static __forceinline__ float scale_of(uint32_t hdr) {
        const uint32_t hb = (hdr & 0x7fffu) ? (hdr & 0xffffu) : (((hdr >> 16) & 0x7fffu) ? (hdr >> 16) : 0x3c00u);
        return half_bits_to_float((uint16_t)hb);
    }
    // slab s = sub-blocks 2s (low nibbles) and 2s+1 (high nibbles).  0x6400 | n is 1024 + n and
    // fma(1024 + n, sc, -1024 sc) rounds the exact n * sc once; 0x6400 | (n << 4) is 1024 + 16 n and
    // fma(1024 + 16 n, sc / 16, -64 sc) does the same for a nibble left in the high half of its byte.
    __device__ static __forceinline__ void emit(int s, const Pre& pr, const Ctx& c, uint32_t ta, int h) {
        const int jl = 2 * s, jh = 2 * s + 1;
        const __half2 k1024 = __float2half2_rn(1024.f);
        const __half2 scl = __hsub2(byte_magic2(c.sc[jl >> 2], jl & 3), k1024);
        const __half2 sch = __hsub2(byte_magic2(c.sc[jh >> 2], jh & 3), k1024);
        const __half2 offl = __hmul2(scl, __float2half2_rn(-1024.f));
        const __half2 sch16 = __hmul2(sch, __float2half2_rn(0.0625f)), offh = __hmul2(sch, __float2half2_rn(-64.f));
        const uint32_t w[4] = {pr.q[s].x, pr.q[s].y, pr.q[s].z, pr.q[s].w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t x = w[i], y = w[i] >> 8;  // bytes (0, 2) and (1, 3) of the four
            lo[2 * i] = bits_h2(__hfma2(h2_bits((x & 0x000F000Fu) | 0x64006400u), scl, offl));
            lo[2 * i + 1] = bits_h2(__hfma2(h2_bits((y & 0x000F000Fu) | 0x64006400u), scl, offl));
            hi[2 * i] = bits_h2(__hfma2(h2_bits((x & 0x00F000F0u) | 0x64006400u), sch16, offh));
            hi[2 * i + 1] = bits_h2(__hfma2(h2_bits((y & 0x00F000F0u) | 0x64006400u), sch16, offh));
        }
        tmem_st8(ta + 8 * h, lo);
        tmem_st8(ta + 16 + 8 * h, hi);
    }
    // weight side of the min term (see prep_gemm_b_kernel): -rho_j = -dmin m_j / d split into tf32 terms.  One
    // row is 32 floats [r1 (8) | r2 (8) | r1 (8) | unused]; thread h = 0 writes the four 16-byte chunks of r1,
    // thread h = 1 the two of r2.  2^23 + m as float bits is 0x4B000000 | m.
    __device__ static __forceinline__ void emit_min(const Pre& pr, const Ctx& c, uint8_t* arow, int h, int sw) {
        const float ratio = -__fdividef(half_bits_to_float((uint16_t)(pr.hdr.x >> 16)), scale_of(pr.hdr.x));
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float mf = __uint_as_float(0x4B000000u | byte_u(c.mn[j >> 2], j & 3)) - 8388608.f;
            const float a = __fmul_rn(ratio, mf), a1 = tf32_head(a);
            o[j] = __float_as_uint(h == 0 ? a1 : tf32_head(__fsub_rn(a, a1)));
        }
        if (h == 0) {
            *reinterpret_cast<uint4*>(arow + ((0 ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(arow + ((1 ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
            *reinterpret_cast<uint4*>(arow + ((4 ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(arow + ((5 ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        } else {
            *reinterpret_cast<uint4*>(arow + ((2 ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(arow + ((3 ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
};

// ------------------------------------------------------------------------------------------------
// Q6_K, repacked layout (expert_direct.cu: per 8 rows x 256 elements, 1680 bytes: low nibbles 2 x 512,
// high bit pairs 512, 128 scales, 8 d).  Row g's 64 nibble bytes of half n sit at 512 n + 64 g in four
// 16-byte chunks t; word cw of chunk t holds elements k0 = 16 cw + 4 t .. + 3 of the half's two slabs
// (low nibbles: even slab, high nibbles: odd slab).  Thread (row, h) takes chunks t = 2h, 2h + 1.
// The quant is placed at mantissa bits 4..9 (0x6400 | q << 4 = 1024 + 16 q); minus 1536 leaves
// 16 (q - 32), times ceil(sc/2)/16 and floor(sc/2)/16 gives the two exact operand parts.
// ------------------------------------------------------------------------------------------------
struct GemmQ6K {
    static constexpr bool HAS_MIN = false;
    static constexpr int A_COLS = 64, A_PARTS = 2, A_PAIRS = 2;  // 4 slabs of 64 columns (two operand parts each)
    static constexpr int B_PARTS = 1;
    static constexpr bool STAGE_W = false;
    static constexpr int W_ROW_BYTES = 0;
    static constexpr int W_MAP_ELEM = 1;
    static constexpr int W_STAGES_WIDE = 1;
    struct Row {
        const uint8_t* p;  // half-tile block 0 of the row's group of 8
        int g;
    };
    __device__ static __forceinline__ Row row(const uint8_t* w, int n, int kb) {
        return Row{w + (size_t)(n >> 3) * kb * Q6K_HTB_BYTES, n & 7};
    }
    struct Pre {
        uint4 ql[2][2], qh[2], sc;
        uint32_t d;  // fp16 bits
    };
    __device__ static __forceinline__ uint32_t hdr_of(const Pre& pr) { return pr.d; }
    __device__ static __forceinline__ void load_staged(Pre&, uint32_t, int) {}
    __device__ static __forceinline__ uint32_t staged_words(const Pre&) { return 0u; }
    __device__ static __forceinline__ void load(Pre& pr, const Row& r, int blk, int h) {
        const uint8_t* b = r.p + (size_t)blk * Q6K_HTB_BYTES + 64 * r.g + 32 * h;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            pr.ql[0][j] = ldg128(b + 16 * j);
            pr.ql[1][j] = ldg128(b + 512 + 16 * j);
            pr.qh[j] = ldg128(b + 1024 + 16 * j);
        }
        pr.sc = ldg128(r.p + (size_t)blk * Q6K_HTB_BYTES + 1536 + 16 * r.g);
        pr.d = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(r.p + (size_t)blk * Q6K_HTB_BYTES + 1664 + 2 * r.g));
    }
    struct Ctx {
        uint32_t xc[4], xh[4];  // per scale byte: ceil(sc/2) + 64 and floor(sc/2) + 64
    };
    __device__ static __forceinline__ void begin(const Pre& pr, Ctx& c) {
        const uint32_t w[4] = {pr.sc.x, pr.sc.y, pr.sc.z, pr.sc.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t x = w[i] ^ 0x80808080u;  // sc + 128 per byte
            c.xh[i] = (x >> 1) & 0x7f7f7f7fu;
            c.xc[i] = c.xh[i] + (x & 0x01010101u);
        }
    }
    __device__ static __forceinline__ void emit(int s, const Pre& pr, const Ctx& c, uint32_t ta, int h) {
        const int n = s >> 1, odd = s & 1;
        const __half2 k16th = __float2half2_rn(0.0625f), km68 = __float2half2_rn(-68.f), km1536 = __float2half2_rn(-1536.f);
#pragma unroll
        for (int cw = 0; cw < 4; ++cw) {
            const int idx = 4 * s + cw;
            // (1024 + x) / 16 - 68 = (x - 64) / 16: the half scale over 16; c = -1536 m, so that
            // fma(1024 + 16 q, m, c) = (q - 32) * (half scale), an integer of at most 2048: exact
            const __half2 m1 = __hfma2(byte_magic2(c.xc[idx >> 2], idx & 3), k16th, km68);
            const __half2 m2 = __hfma2(byte_magic2(c.xh[idx >> 2], idx & 3), k16th, km68);
            const __half2 c1 = __hmul2(m1, km1536), c2 = __hmul2(m2, km1536);
            const int bq = 2 * ((cw >> 1) + 2 * odd);  // bit position of this quarter's pair in the qh byte
            uint32_t o1[4], o2[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t qlw = w4(pr.ql[n][j], cw), qhw = w4(pr.qh[j], 2 * n + (cw & 1));
                const uint32_t a02 = odd ? qlw : (qlw << 4), a13 = odd ? (qlw >> 8) : (qlw >> 4);
                const uint32_t b02 = qhw << (8 - bq), b13 = qhw >> bq;
                const __half2 v02 = h2_bits(((a02 & 0x00F000F0u) | 0x64006400u) | (b02 & 0x03000300u));
                const __half2 v13 = h2_bits(((a13 & 0x00F000F0u) | 0x64006400u) | (b13 & 0x03000300u));
                o1[2 * j] = bits_h2(__hfma2(v02, m1, c1));
                o1[2 * j + 1] = bits_h2(__hfma2(v13, m1, c1));
                o2[2 * j] = bits_h2(__hfma2(v02, m2, c2));
                o2[2 * j + 1] = bits_h2(__hfma2(v13, m2, c2));
            }
            tmem_st4(ta + 8 * cw + 4 * h, o1[0], o1[1], o1[2], o1[3]);
            tmem_st4(ta + 32 + 8 * cw + 4 * h, o2[0], o2[1], o2[2], o2[3]);
        }
    }
    __device__ static __forceinline__ void emit_min(const Pre&, const Ctx&, uint8_t*, int, int) {}
    __device__ static __forceinline__ float scale_of(uint32_t hdr) { return half_bits_to_float((uint16_t)hdr); }
};

// ------------------------------------------------------------------------------------------------
// Q8_0, repacked layout (prepack_q80_kernel): per row and 256 elements a 272-byte record [256 int8 | 8 f16
// scales], rows padded with zero records to a multiple of 256 elements.  The reference multiplies per 32-element
// block (sum of int8 products) * d_w * d_a in f32 (k_quants.rs:636-668); here both scales are folded into the fp16
// operands -- weight d_w * q, activation d_a * q, each rounded once to fp16 (2^-12 relative) -- and the products
// are accumulated in f32 by the tensor core over the whole row, so no per-block scaling is left for the epilogue.
// The rounding of the operands is the one deviation from the reference's arithmetic on this path: it shows as a
// relative L2 error of a few 1e-4 on a product, inside the block's bound (1e-3), and is measured by the tests.
// Used for the down product only (see launch_expert_gemm for why gate_up cannot afford that rounding).
// Thread (row, h) owns bytes 16h..16h+15 and 32+16h..32+16h+15 of each 64-element slab, like the Q4_K thread.
// ------------------------------------------------------------------------------------------------
struct GemmQ80 {
    static constexpr bool HAS_MIN = false;
    static constexpr int A_COLS = 32, A_PARTS = 1, A_PAIRS = 4;
    static constexpr int B_PARTS = 1;
    static constexpr bool STAGE_W = true;
    static constexpr int W_ROW_BYTES = 272;
    static constexpr int W_MAP_ELEM = 4;     // the tensor map counts 4-byte elements (a box row of 272 bytes exceeds 256 bytes)
    static constexpr int W_STAGES_WIDE = 2;  // staged blocks beside 128-wide activation stages
    struct Row {
        const uint8_t* p;
    };
    __device__ static __forceinline__ Row row(const uint8_t* w, int n, int kb) { return Row{w + (size_t)n * kb * W_ROW_BYTES}; }
    struct Pre {
        uint4 sc;       // 8 f16 scales
        uint4 q[4][2];  // per slab: bytes 16h.. and 32 + 16h..
    };
    __device__ static __forceinline__ void load(Pre&, const Row&, int, int) {}
    __device__ static __forceinline__ void load_staged(Pre& pr, uint32_t row_addr, int h) {
        pr.sc = lds128_o<256>(row_addr);
        const uint32_t rb = row_addr + 16 * h;
        pr.q[0][0] = lds128_o<0>(rb);
        pr.q[0][1] = lds128_o<32>(rb);
        pr.q[1][0] = lds128_o<64>(rb);
        pr.q[1][1] = lds128_o<96>(rb);
        pr.q[2][0] = lds128_o<128>(rb);
        pr.q[2][1] = lds128_o<160>(rb);
        pr.q[3][0] = lds128_o<192>(rb);
        pr.q[3][1] = lds128_o<224>(rb);
    }
    __device__ static __forceinline__ uint32_t staged_words(const Pre& pr) {
        return pr.sc.x | pr.q[0][0].x | pr.q[0][1].x | pr.q[1][0].x | pr.q[1][1].x | pr.q[2][0].x | pr.q[2][1].x | pr.q[3][0].x | pr.q[3][1].x;
    }
    __device__ static __forceinline__ uint32_t hdr_of(const Pre&) { return 0u; }
    struct Ctx {};
    __device__ static __forceinline__ void begin(const Pre&, Ctx&) {}
    __device__ static __forceinline__ float scale_of(uint32_t) { return 1.0f; }  // the scales are inside the operands
    // 16 int8 -> 8 columns of fp16 pairs (k0, k2), (k1, k3) per word, times d: the byte plus 128 is dropped into the
    // mantissa of 1024 (0x6400 | b + 128 = 1152 + b), 1152 comes off exactly, one multiply rounds
    __device__ static __forceinline__ void cvt16(const uint4& v, __half2 d, uint32_t (&o)[8]) {
        const uint32_t w[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
        const __half2 k1152 = __float2half2_rn(1152.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t e, f;
            asm("prmt.b32 %0, %1, %2, 0x4240;" : "=r"(e) : "r"(w[i]), "r"(0x64646464u));  // bytes 0 and 2
            asm("prmt.b32 %0, %1, %2, 0x4341;" : "=r"(f) : "r"(w[i]), "r"(0x64646464u));  // bytes 1 and 3
            o[2 * i] = bits_h2(__hmul2(__hsub2(h2_bits(e), k1152), d));
            o[2 * i + 1] = bits_h2(__hmul2(__hsub2(h2_bits(f), k1152), d));
        }
    }
    __device__ static __forceinline__ void emit(int s, const Pre& pr, const Ctx&, uint32_t ta, int h) {
        const uint32_t dw = s == 0 ? pr.sc.x : (s == 1 ? pr.sc.y : (s == 2 ? pr.sc.z : pr.sc.w));  // scales of blocks 2s, 2s + 1
        const __half2 d2 = h2_bits(dw);
        uint32_t lo[8], hi[8];
        cvt16(pr.q[s][0], __low2half2(d2), lo);
        cvt16(pr.q[s][1], __high2half2(d2), hi);
        tmem_st8(ta + 8 * h, lo);
        tmem_st8(ta + 16 + 8 * h, hi);
    }
    __device__ static __forceinline__ void emit_min(const Pre&, const Ctx&, uint8_t*, int, int) {}
};

// ------------------------------------------------------------------------------------------------
// Q8_0 with EXACT operands, for the gate_up product (whose f32 result is re-quantized to int8 and therefore has to
// match the reference to f32 rounding, not to fp16 rounding).  d * q has up to 19 significant bits: it is carried as
// two fp16 numbers, the rounded product and its exact residual (one more fused multiply-add), on both sides:
//   weights      4096 d_w q  = A0 + A1      (the power of two keeps the residuals out of the fp16 subnormals;
//   activations    64 d_a q  = B0 + B1       both come off again in the epilogue's scale)
// and the tensor core accumulates A0 B0 + A1 B0 + A0 B1 in f32 (A1 B1 is below 2^-22 of a term).  Three MMAs per
// K step; the activation operand is twice as large, so its two shared-memory stages hold half a block each (see the
// kernel).
// ------------------------------------------------------------------------------------------------
struct GemmQ80X : GemmQ80 {
    static constexpr int A_COLS = 64, A_PARTS = 2, A_PAIRS = 2;
    static constexpr int B_PARTS = 2;
    static constexpr int W_STAGES_WIDE = 2;
    __device__ static __forceinline__ float scale_of(uint32_t) { return 1.0f / 4096.0f; }
    __device__ static __forceinline__ void cvt16x(const uint4& v, __half2 d, uint32_t (&p0)[8], uint32_t (&p1)[8]) {
        const uint32_t w[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
        const __half2 k1152 = __float2half2_rn(1152.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t e, f;
            asm("prmt.b32 %0, %1, %2, 0x4240;" : "=r"(e) : "r"(w[i]), "r"(0x64646464u));
            asm("prmt.b32 %0, %1, %2, 0x4341;" : "=r"(f) : "r"(w[i]), "r"(0x64646464u));
            const __half2 xe = __hsub2(h2_bits(e), k1152), xf = __hsub2(h2_bits(f), k1152);
            const __half2 re = __hmul2(xe, d), rf = __hmul2(xf, d);
            p0[2 * i] = bits_h2(re);
            p0[2 * i + 1] = bits_h2(rf);
            p1[2 * i] = bits_h2(__hfma2(xe, d, __hneg2(re)));  // exact: the residual of a 19-bit product has at most 8 bits
            p1[2 * i + 1] = bits_h2(__hfma2(xf, d, __hneg2(rf)));
        }
    }
    __device__ static __forceinline__ void emit(int s, const Pre& pr, const Ctx&, uint32_t ta, int h) {
        const uint32_t dw = s == 0 ? pr.sc.x : (s == 1 ? pr.sc.y : (s == 2 ? pr.sc.z : pr.sc.w));
        const __half2 d2 = __hmul2(h2_bits(dw), __float2half2_rn(4096.f));  // exact (a power of two)
        uint32_t a0[8], a1[8];
        cvt16x(pr.q[s][0], __low2half2(d2), a0, a1);
        tmem_st8(ta + 8 * h, a0);
        tmem_st8(ta + 32 + 8 * h, a1);
        cvt16x(pr.q[s][1], __high2half2(d2), a0, a1);
        tmem_st8(ta + 16 + 8 * h, a0);
        tmem_st8(ta + 48 + 8 * h, a1);
    }
};

// raw weight blocks staged per CTA (see the kernel): what fits beside the activation stages
template <class F, int TN>
__host__ __device__ constexpr int w_stages() {
    return !F::STAGE_W ? 1 : (TN <= 32 ? 4 : (TN <= 64 ? (F::B_PARTS == 2 ? 4 : 3) : F::W_STAGES_WIDE));
}

struct TileCoord {
    int e, nt, mt;
    int ks, kb0, kb1;  // K split: this work item covers the 256-blocks [kb0, kb1) and writes partial output ks
    uint32_t p0, p_end;
};

// tile id -> (expert, row tile, position tile); position tiles are fastest, so the CTAs that run at
// the same time share a weight tile (fetched from HBM once) and each expert's activations stay in L2
template <int TN>
__device__ __forceinline__ bool decode_tile(long long tile, const uint32_t* offs, int E, int m_tiles, int ksplit, int kb,
                                            TileCoord& tc) {
    long long cum = 0;
    for (int e = 0; e < E; ++e) {
        const uint32_t cnt = offs[e + 1] - offs[e];
        const int n_tiles = (int)((cnt + TN - 1) / TN);
        const long long te = (long long)n_tiles * m_tiles * ksplit;
        if (tile < cum + te) {
            const long long local = tile - cum;
            const int per_mt = n_tiles * ksplit;
            tc.e = e;
            tc.mt = (int)(local / per_mt);
            const int rem = (int)(local - (long long)tc.mt * per_mt);
            tc.ks = rem / n_tiles;
            tc.nt = rem - tc.ks * n_tiles;
            tc.kb0 = tc.ks * (kb / ksplit);
            tc.kb1 = tc.kb0 + kb / ksplit;
            tc.p0 = offs[e] + (uint32_t)tc.nt * TN;
            tc.p_end = offs[e + 1];
            return true;
        }
        cum += te;
    }
    return false;
}

template <class F, bool GATE_UP, int TN>
__global__ void __launch_bounds__(G_THREADS, 1)
expert_gemm_kernel(const __grid_constant__ GemmParams P, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_bs) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_a[4], empty_a[4], full_b[G_B_STAGES], empty_b[G_B_STAGES];  // A: per pair of slabs
    __shared__ uint64_t tmem_full[2], epi_done[2], full_w[G_W_STAGES_MAX], empty_w[G_W_STAGES_MAX];
    __shared__ uint32_t s_offs[CANDLE_MOE_MAX_EXPERTS + 1];
    constexpr int CH = TN / 2;            // columns (positions) per epilogue warp: two warps share a TMEM lane quarter
    constexpr int B_TILE = TN * G_SLAB_K * 2;  // one [TN x 64] fp16 activation slab
    __shared__ __align__(16) float s_d8[G_EPI_WARPS][2][CH];  // per epilogue warp: activation scales of its columns
    __shared__ float s_dw[8][G_TILE_M];  // per block (ring of 8) and tile row: the weight scale the drain multiplies by
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    // the warp index through a shuffle: the compiler then knows that it is warp-uniform and keeps role
    // dispatch, loop counters and MMA / TMA operands in uniform registers
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // One activation stage holds a whole 256-wide block (four slabs, + the min-term box for Q4_K).  With two operand
    // parts (exact Q8_0) a whole block would be twice that, so there the two stages are the two HALVES of a block
    // -- stage pr = the slabs of pair pr: [part 0: slab 2 pr, 2 pr + 1 | part 1: slab 2 pr, 2 pr + 1] -- each
    // refilled for the next block as soon as its own pair's MMAs are done; the same shared memory then takes
    // 128-wide position tiles.
    constexpr bool B_HALF = F::B_PARTS == 2;
    constexpr int G_STAGE_BYTES = (4 + (F::HAS_MIN ? 1 : 0)) * B_TILE;
    uint8_t* smem_min_a = smem + G_B_STAGES * G_STAGE_BYTES;  // Q4_K: 2 slots of the min operand (weights side)
    // staged raw blocks of the tile rows: a ring of WS blocks.  With 128-wide position tiles the activation stages
    // leave room for one block only (the L2 prefetch ahead of it has to do); narrower tiles take a deeper ring, so
    // that the copy of block b + WS - 1 is in flight while block b is unpacked.
    constexpr int WS = w_stages<F, TN>();
    constexpr int W_STAGE_BYTES = G_TILE_M * F::W_ROW_BYTES;
    uint8_t* smem_w = smem_min_a + (F::HAS_MIN ? 2 : 0) * G_TILE_BYTES;
    for (int i = threadIdx.x; i <= P.E; i += G_THREADS) s_offs[i] = P.offsets[i];
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < 4; ++s) {
            mbar_init(&full_a[s], G_DQ_WARPS);
            mbar_init(&empty_a[s], 1);
        }
        for (int s = 0; s < G_B_STAGES; ++s) {
            mbar_init(&full_b[s], 1);
            mbar_init(&empty_b[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&epi_done[b], G_EPI_WARPS);
        }
        for (int s = 0; s < G_W_STAGES_MAX; ++s) {
            mbar_init(&full_w[s], 1);
            mbar_init(&empty_w[s], G_DQ_WARPS);
        }
        fence_barrier_init();
    }
    if (warp == G_WARP_TMA) tmem_alloc(&s_tmem_base, G_TMEM_COLS);
    tc5_fence_before_sync();
    __syncthreads();
    tc5_fence_after_sync();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, s_tmem_base, 0);
    volatile int* abort_flag = &s_abort;
    constexpr uint32_t IDESC = umma_idesc_f16(G_TILE_M, TN), IDESC_TF32 = umma_idesc_tf32(G_TILE_M, TN);

    // Register budget: launched with 96 per thread; the TMA/MMA warpgroup hands 64 per thread back to the CTA's
    // pool and the two epilogue warpgroups take 32 more each, so the total stays what the launch allocated (a
    // request beyond the pool would wait forever).
    if (warp >= G_WARP_DQ0 + G_DQ_WARPS) reg_dealloc<G_REGS_MISC>();  // the whole last warpgroup (two idle warps, TMA, MMA)
    if (warp < G_WARP_DQ0) {
        reg_alloc<G_REGS_EPI>();
        // ===================== epilogue =====================
        const int quarter = warp & 3, colhalf = (warp - G_WARP_EPI0) >> 2, ew = warp - G_WARP_EPI0;
        const int r = 32 * quarter + lane;  // tile row = TMEM lane
        const uint32_t ta_lane = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(colhalf * CH);
        uint32_t ab = 0;
        long long tile = blockIdx.x;
        TileCoord tc, tcn;
        bool have = decode_tile<TN>(tile, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tc);
        if (have) {
            const float* dp = P.d8t + (size_t)tc.kb0 * P.P_pad + tc.p0 + colhalf * CH;
            for (int i = lane; i < CH; i += 32) s_d8[ew][0][i] = dp[i];
            __syncwarp();
        }
        while (have) {
            const bool have_n = decode_tile<TN>(tile + gridDim.x, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tcn);
            // the accumulators are kept as pairs of columns: one packed fused multiply-add per pair and block
            uint64_t acc2[CH / 2];
#pragma unroll
            for (int i = 0; i < CH / 2; ++i) acc2[i] = 0ull;
            for (int blk = tc.kb0; blk < tc.kb1; ++blk, ++ab) {
                const int buf = ab & 1;
                // scales of the next block (maybe of the next tile): in flight while this block is drained
                float d8_n0 = 0.f, d8_n1 = 0.f;
                const float* dp = nullptr;
                if (blk + 1 < tc.kb1)
                    dp = P.d8t + (size_t)(blk + 1) * P.P_pad + tc.p0 + colhalf * CH + lane;
                else if (have_n)
                    dp = P.d8t + (size_t)tcn.kb0 * P.P_pad + tcn.p0 + colhalf * CH + lane;
                const bool pre = dp != nullptr;
                if (pre) {
                    if (lane < CH) d8_n0 = dp[0];
                    if (CH > 32) d8_n1 = dp[32];
                }
                mbar_wait(&tmem_full[buf], (ab >> 1) & 1, abort_flag);
                tc5_fence_after_sync();
                const float dw = s_dw[ab & 7][r];  // left by the unpack warps when they produced this block
                const uint64_t dw2 = f32x2_pack(dw, dw);
                const uint32_t t_main = ta_lane + (uint32_t)(G_TM_MAIN + buf * TN);
                const uint32_t d8_addr = smem_u32(&s_d8[ew][buf][0]);
                // Four steps of 16 columns; the load of step i+1 is in flight while step i is scaled into
                // the register accumulators: acc += (d8[col] * dw[row]) * v.
                constexpr int NS = CH / 16;  // steps of 16 columns
                uint32_t stg[2][16];
                tmem_ld16(t_main, stg[0]);
                tmem_ld_wait();
                static_for<NS>([&](auto Cc) {
                    constexpr int c = decltype(Cc)::value;
                    if (c + 1 < NS) tmem_ld16(t_main + 16 * (c + 1), stg[(c + 1) & 1]);
                    static_for<4>([&](auto Qc) {
                        constexpr int q = decltype(Qc)::value;
                        const uint4 dv = lds128_o<64 * c + 16 * q>(d8_addr);  // base + constant: no address arithmetic
                        // per column pair: the two scale products in one packed multiply, the two accumulations in one
                        // packed fused multiply-add (each half is the IEEE fma of the scalar form)
                        acc2[8 * c + 2 * q] = f32x2_fma(f32x2_mul(dw2, f32x2_pack_bits(dv.x, dv.y)),
                                                        f32x2_pack_bits(stg[c & 1][4 * q], stg[c & 1][4 * q + 1]), acc2[8 * c + 2 * q]);
                        acc2[8 * c + 2 * q + 1] = f32x2_fma(f32x2_mul(dw2, f32x2_pack_bits(dv.z, dv.w)),
                                                            f32x2_pack_bits(stg[c & 1][4 * q + 2], stg[c & 1][4 * q + 3]),
                                                            acc2[8 * c + 2 * q + 1]);
                    });
                    if (c + 1 < NS) tmem_ld_wait();
                    if (c == (NS >= 2 ? NS - 2 : 0)) {  // every column of this thread has been read: the buffer may be overwritten
                        tc5_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&epi_done[buf]);
                    }
                });
                if (pre) {
                    if (lane < CH) s_d8[ew][buf ^ 1][lane] = d8_n0;
                    if (CH > 32) s_d8[ew][buf ^ 1][lane + 32] = d8_n1;
                }
                __syncwarp();
            }
            float acc[CH];
#pragma unroll
            for (int i = 0; i < CH / 2; ++i) f32x2_unpack(acc2[i], acc[2 * i], acc[2 * i + 1]);
            // ---- store the tile ----
            const int n = GATE_UP ? tc.mt * 64 + (r >> 1) : tc.mt * 128 + r;
            const uint32_t pc0 = tc.p0 + colhalf * CH;
            float* out_k = P.out + (size_t)tc.ks * P.split_stride;
            if (GATE_UP) {
                // even lane holds w1 x, odd lane w3 x of the same output row: the even lane finishes the first
                // half of this warp's columns, the odd lane the second half, one exchange per pair of columns
#pragma unroll
                for (int c = 0; c < CH / 2; ++c) {
                    const float recv = __shfl_xor_sync(0xffffffffu, (lane & 1) ? acc[c] : acc[c + CH / 2], 1);
                    const float gv = (lane & 1) ? recv : acc[c], uv = (lane & 1) ? acc[c + CH / 2] : recv;
                    const uint32_t p = pc0 + c + ((lane & 1) ? CH / 2 : 0);
                    if (p < tc.p_end) out_k[(size_t)p * P.N + n] = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
                }
            } else {
#pragma unroll
                for (int c = 0; c < CH; ++c)
                    if (pc0 + c < tc.p_end) out_k[(size_t)(pc0 + c) * P.N + n] = acc[c];
            }
            tile += gridDim.x;
            tc = tcn;
            have = have_n;
        }
    } else if (warp < G_WARP_DQ0 + G_DQ_WARPS) {
        // ===================== weight unpack -> fp16 operand in tensor memory =====================
        const int quarter = warp & 3, h = (warp - G_WARP_DQ0) >> 2;
        const int r = 32 * quarter + lane;
        const uint32_t ta_lane = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)G_TM_A;
        const uint32_t min_row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        uint32_t ita = 0, ab = 0;
        long long tile = blockIdx.x;
        TileCoord tc, tcn;
        bool have = decode_tile<TN>(tile, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tc);
        typename F::Row rowc{}, rown{};
        typename F::Pre cur, nxt;
        // staged row of tile row r: gate_up keeps the W1 rows first, then the W3 rows
        const uint32_t w_row = smem_u32(smem_w) + (GATE_UP ? (uint32_t)((r & 1) * (G_TILE_M / 2 * F::W_ROW_BYTES) + (r >> 1) * F::W_ROW_BYTES)
                                                           : (uint32_t)(r * F::W_ROW_BYTES));
        if (have && !F::STAGE_W) {
            const int n = GATE_UP ? tc.mt * 64 + (r >> 1) : tc.mt * 128 + r;
            rowc = F::row((GATE_UP && (r & 1)) ? P.wb.p[tc.e] : P.wa.p[tc.e], n, P.kb);
            F::load(cur, rowc, tc.kb0, h);
            nxt = cur;
        }
        while (have) {
            const bool have_n = decode_tile<TN>(tile + gridDim.x, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tcn);
            if (have_n && !F::STAGE_W) {
                const int nn = GATE_UP ? tcn.mt * 64 + (r >> 1) : tcn.mt * 128 + r;
                rown = F::row((GATE_UP && (r & 1)) ? P.wb.p[tcn.e] : P.wa.p[tcn.e], nn, P.kb);
            }
            for (int blk = tc.kb0; blk < tc.kb1; ++blk, ++ab) {
                if (F::STAGE_W) {
                    // this block's raw bytes were copied to shared memory by the loader warp
                    mbar_wait(&full_w[ab % WS], (ab / WS) & 1, abort_flag);
                    F::load_staged(cur, w_row + (ab % WS) * W_STAGE_BYTES, h);
                } else if (blk + 1 < tc.kb1) {
                    F::load(nxt, rowc, blk + 1, h);
                } else if (have_n) {
                    F::load(nxt, rown, tcn.kb0, h);
                }
                typename F::Ctx ctx;
                F::begin(cur, ctx);
                if (h == 0) s_dw[ab & 7][r] = F::scale_of(F::hdr_of(cur));  // read by the epilogue when it drains this block
                // Handing the stage back to the loader.  The staged words must have ARRIVED in registers first: the
                // loads are plain shared-memory loads, their results are not needed until the emits below, and an
                // arrive that merely follows them in program order was observed to overtake them -- the refill then
                // landed under loads still waiting behind the (long) wait for a free operand slot, and the first
                // rows of a tile came out with the next block's weights, rarely and only when the MMAs are the
                // bottleneck.  With a ring of two or more stages the stage is released after the emits (nothing
                // reads it later than that, whatever the order of the instructions).  With a single stage that
                // would serialise copy and unpack, so the release stays early and the barrier's ADDRESS is made to
                // depend on one word of every load of every lane (OR-reduced over the warp, masked with a kernel
                // parameter that is zero at run time): the arrive cannot be issued before those words exist.
                if (F::STAGE_W && WS == 1) {
                    const uint32_t dep = __reduce_or_sync(0xffffffffu, F::staged_words(cur)) & P.zero;
                    if (lane == 0) mbar_arrive(&empty_w[dep]);
                }
#pragma unroll
                for (int pr = 0; pr < 2; ++pr, ita += 2) {
                    // Slabs go to tensor memory in pairs; the ring holds A_PAIRS pairs (Q4_K: two blocks).  The barriers
                    // go by (block parity, pair) -- each has ONE waiting MMA warp that sees every phase, so a parity
                    // wait is never ambiguous -- while the TMEM slot is the pair index modulo the ring size: before
                    // writing it, wait for the MMAs of the block that used it last.
                    const uint32_t bidx = 2 * (ab & 1) + pr, slot = bidx % F::A_PAIRS;
                    if (ab >= F::A_PAIRS / 2) {
                        const uint32_t abp = ab - F::A_PAIRS / 2;
                        mbar_wait_relaxed(&empty_a[2 * (abp & 1) + pr], (abp >> 1) & 1, abort_flag);
                    }
                    tc5_fence_after_sync();
                    F::emit(2 * pr, cur, ctx, ta_lane + (uint32_t)(2 * slot * F::A_COLS), h);
                    F::emit(2 * pr + 1, cur, ctx, ta_lane + (uint32_t)((2 * slot + 1) * F::A_COLS), h);
                    if (F::HAS_MIN && pr == 1) {
                        // weight side of the min term, handed over with the second pair.  Its slot was last read by
                        // the min MMAs of block ab - 2, issued before the commit whose completion the wait above saw.
                        F::emit_min(cur, ctx, smem_min_a + (size_t)(ab & 1) * G_TILE_BYTES + min_row_off, h, r & 7);
                        fence_proxy_async_smem();
                    }
                    tmem_st_wait();
                    tc5_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_a[bidx]);
                }
                if (F::STAGE_W && WS > 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_w[ab % WS]);
                }
                if (!F::STAGE_W) cur = nxt;
            }
            tile += gridDim.x;
            tc = tcn;
            rowc = rown;
            have = have_n;
        }
    } else if (warp == G_WARP_LOAD) {
        // ===================== weight loader: raw blocks of the tile rows -> shared memory =====================
        // One TMA box per matrix and block: [64 or 128 rows x 144 bytes] of the byte matrix [n_rows, row_bytes]
        // (gate_up: the W1 rows, then the W3 rows; a TMA destination must be 128-byte aligned, so the halves cannot
        // be skewed against each other and neighbouring lanes, which alternate between them, share banks two by
        // two).  Two blocks ahead the same boxes are requested into L2, so the copy into the one-block-deep stage
        // finds them there.
        if (F::STAGE_W) {
            uint32_t ab = 0;
            long long tile = blockIdx.x;
            TileCoord tc, tcn;
            bool have = decode_tile<TN>(tile, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tc);
            constexpr int HALF = G_TILE_M / 2 * F::W_ROW_BYTES;  // 9216
            while (have) {
                const bool have_n = decode_tile<TN>(tile + gridDim.x, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tcn);
                const CUtensorMap* m0 = P.wmaps + 2 * tc.e;
                // the maps were written by a kernel earlier on the stream: fence each once, before its first use by
                // this warp -- the current expert's on the first tile, the next expert's one tile ahead, because the
                // prefetches reach into it (every lane fences: any may be elected)
                if (ab == 0) {
                    tensormap_fence_acquire(m0);
                    if (GATE_UP) tensormap_fence_acquire(m0 + 1);
                }
                if (have_n && tcn.e != tc.e) {
                    tensormap_fence_acquire(P.wmaps + 2 * tcn.e);
                    if (GATE_UP) tensormap_fence_acquire(P.wmaps + 2 * tcn.e + 1);
                }
                const int y0 = GATE_UP ? tc.mt * 64 : tc.mt * 128;
                for (int blk = tc.kb0; blk < tc.kb1; ++blk, ++ab) {
                    const uint32_t ws = ab % WS;
                    if (ab >= (uint32_t)WS) mbar_wait(&empty_w[ws], ((ab / WS) - 1) & 1, abort_flag);
                    if (elect_one()) {
                        uint8_t* dst = smem_w + ws * W_STAGE_BYTES;
                        mbar_expect_tx(&full_w[ws], G_TILE_M * F::W_ROW_BYTES);
                        if (GATE_UP) {
                            tma_load_2d(dst, m0, blk * (F::W_ROW_BYTES / F::W_MAP_ELEM), y0, &full_w[ws]);
                            tma_load_2d(dst + HALF, m0 + 1, blk * (F::W_ROW_BYTES / F::W_MAP_ELEM), y0, &full_w[ws]);
                        } else {
                            tma_load_2d(dst, m0, blk * (F::W_ROW_BYTES / F::W_MAP_ELEM), y0, &full_w[ws]);
                            tma_load_2d(dst + HALF, m0, blk * (F::W_ROW_BYTES / F::W_MAP_ELEM), y0 + 64, &full_w[ws]);
                        }
                        // two blocks ahead, possibly in the next tile
                        const bool same = blk + 2 < tc.kb1;
                        if (same || have_n) {
                            const CUtensorMap* mp = same ? m0 : P.wmaps + 2 * tcn.e;
                            const int yp = same ? y0 : (GATE_UP ? tcn.mt * 64 : tcn.mt * 128);
                            const int xp = (same ? blk + 2 : tcn.kb0 + blk + 2 - tc.kb1) * (F::W_ROW_BYTES / F::W_MAP_ELEM);
                            tma_prefetch_2d(mp, xp, yp);
                            tma_prefetch_2d(GATE_UP ? mp + 1 : mp, xp, GATE_UP ? yp : yp + 64);
                        }
                    }
                    __syncwarp();
                }
                tile += gridDim.x;
                tc = tcn;
                have = have_n;
            }
        }
    } else if (warp == G_WARP_TMA) {
        // ===================== TMA: activation operand =====================
        // the whole warp walks the loop (uniform control flow and addresses), one elected lane issues
        uint32_t ab = 0;
        TileCoord tc;
        for (long long tile = blockIdx.x; decode_tile<TN>(tile, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tc); tile += gridDim.x) {
            for (int blk = tc.kb0; blk < tc.kb1; ++blk, ++ab) {
                if constexpr (B_HALF) {
                    // stage pr of every block: free once the MMAs of pair pr of the block before are done
#pragma unroll
                    for (int pr = 0; pr < 2; ++pr) {
                        if (ab >= 1) mbar_wait_relaxed(&empty_b[pr], (ab - 1) & 1, abort_flag);
                        uint8_t* dst = smem + (size_t)pr * G_STAGE_BYTES;
                        if (elect_one()) {
                            mbar_expect_tx(&full_b[pr], G_STAGE_BYTES);
#pragma unroll
                            for (int j = 0; j < 4; ++j)  // a row holds [256 of part 0 | 256 of part 1] per block
                                tma_load_2d(dst + j * B_TILE, &map_b, blk * 512 + (j >> 1) * 256 + (2 * pr + (j & 1)) * 64, (int)tc.p0,
                                            &full_b[pr]);
                        }
                        __syncwarp();
                    }
                    continue;
                }
                // one stage = the whole 256-wide block: four slabs (+ the activation side of the min term), one barrier
                const int st = ab & 1;
                if (ab >= 2) mbar_wait_relaxed(&empty_b[st], ((ab >> 1) & 1) ^ 1, abort_flag);
                uint8_t* dst = smem + (size_t)st * G_STAGE_BYTES;
                if (elect_one()) {
                    mbar_expect_tx(&full_b[st], G_STAGE_BYTES);
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4)
                        tma_load_2d(dst + s4 * B_TILE, &map_b, blk * 256 + s4 * 64, (int)tc.p0, &full_b[st]);
                    if (F::HAS_MIN) tma_load_2d(dst + 4 * B_TILE, &map_bs, blk * 32, (int)tc.p0, &full_b[st]);
                }
                __syncwarp();
            }
        }
    } else if (warp == G_WARP_MMA) {
        // ===================== MMA issue =====================
        // (Splitting the blocks by parity over two issuing warps was measured: no gain.)
        uint32_t ita = 0, ab = 0;
        TileCoord tc;
        const uint32_t a_base = tmem_base + (uint32_t)G_TM_A;
        const uint64_t b_desc0 = umma_desc_sw128(smem_u32(smem));
        const uint64_t ma_desc0 = umma_desc_sw128(smem_u32(smem_min_a));
        bool rdy_a = false, rdy_b = false;
        for (long long tile = blockIdx.x; decode_tile<TN>(tile, s_offs, P.E, P.m_tiles, P.ksplit, P.kb, tc); tile += gridDim.x) {
            // The last position tile of an expert is rarely full: its MMAs run N = the rows it holds, rounded up to 16
            // (an MMA's time goes with N; the columns beyond are neither computed nor stored).
            const uint32_t n_eff = min((uint32_t)TN, (tc.p_end - tc.p0 + 15u) & ~15u);
            const uint32_t idesc = (IDESC & ~(0x3Fu << 17)) | ((n_eff >> 3) << 17);
            const uint32_t idesc_tf32 = (IDESC_TF32 & ~(0x3Fu << 17)) | ((n_eff >> 3) << 17);
            for (int blk = tc.kb0; blk < tc.kb1; ++blk, ++ab) {
                const int buf = ab & 1;  // main accumulator and B stage of this block
                // the drain of block ab - 2 has released this main accumulator
                if (ab >= 2) mbar_wait(&epi_done[buf], ((ab >> 1) & 1) ^ 1, abort_flag);
                const uint32_t d_main = tmem_base + (uint32_t)(G_TM_MAIN + buf * TN);
                const uint64_t db = b_desc0 + (uint64_t)((B_HALF ? 0 : buf) * (G_STAGE_BYTES >> 4));
#pragma unroll
                for (int pr = 0; pr < 2; ++pr, ita += 2) {
                    const uint32_t bidx = 2 * (ab & 1) + pr, slot = bidx % F::A_PAIRS;  // barrier, TMEM slot (see the unpack warps)
                    if (!rdy_a) mbar_wait(&full_a[bidx], (ab >> 1) & 1, abort_flag);
                    if constexpr (B_HALF) {
                        mbar_wait(&full_b[pr], ab & 1, abort_flag);
                    } else {
                        if (pr == 0 && !rdy_b) mbar_wait(&full_b[buf], (ab >> 1) & 1, abort_flag);
                    }
                    tc5_fence_after_sync();
                    // look at this warp's next barriers now: the answers arrive while the MMAs are issued
                    rdy_a = pr == 0 ? mbar_test(&full_a[bidx + 1], (ab >> 1) & 1)                    // second pair of this block
                                    : mbar_test(&full_a[2 * ((ab + 1) & 1)], ((ab + 1) >> 1) & 1);  // first pair of the next
                    if (!B_HALF && pr == 1) rdy_b = mbar_test(&full_b[buf ^ 1], ((ab + 1) >> 1) & 1);
                    const uint32_t a_t = a_base + (uint32_t)(2 * slot * F::A_COLS);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {  // two slabs of four K steps
                            const uint32_t a_k = a_t + (uint32_t)((k >> 2) * F::A_COLS + 8 * (k & 3));
                            // slab of this K step inside its stage: whole-block stages hold slabs 0..3, half-block
                            // stages [part 0: two slabs | part 1: two slabs] of pair pr
                            const uint64_t b_k = db + (uint64_t)((B_HALF ? pr * 4 + (k >> 2) : 2 * pr + (k >> 2)) * (B_TILE >> 4) + 2 * (k & 3));
                            umma_f16_ts(d_main, a_k, b_k, idesc, (pr | k) != 0);
                            if (F::A_PARTS == 2) umma_f16_ts(d_main, a_k + 32, b_k, idesc, true);
                            if (F::B_PARTS == 2) umma_f16_ts(d_main, a_k, b_k + (uint64_t)(2 * (B_TILE >> 4)), idesc, true);
                        }
                        if (pr == 1 && F::HAS_MIN) {
                            // the min term joins the same accumulator: three tf32 steps, last in the block
                            const uint64_t da = ma_desc0 + (uint64_t)(buf * (G_TILE_BYTES >> 4)), dm = db + (uint64_t)(4 * (B_TILE >> 4));
#pragma unroll
                            for (int k = 0; k < 3; ++k) umma_tf32(d_main, da + 2 * k, dm + 2 * k, idesc_tf32, true);
                        }
                        umma_commit(&empty_a[bidx]);  // the stages may be refilled once these MMAs have read them
                        if (B_HALF) umma_commit(&empty_b[pr]);
                        if (pr == 1) {
                            if (!B_HALF) umma_commit(&empty_b[buf]);
                            umma_commit(&tmem_full[buf]);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    }
    tc5_fence_before_sync();
    __syncthreads();
    if (warp == G_WARP_TMA) {
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

// row-major matrix [rows, cols] -> boxes of [box_rows x box_cols] (128 bytes wide), 128-byte swizzle
bool make_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// byte matrix [rows, row_bytes] -> boxes of [box_rows x box_bytes], no swizzle
bool make_map_bytes(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes, uint32_t box_rows,
                    int elem = 1) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {row_bytes / elem, rows};  // elem = 4: counted in 32-bit words (a box dimension holds at most 256 elements)
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes / elem, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_gemm_sms = -1;

// Tensor maps of the weight matrices reach device memory as kernel PARAMETERS of a small copy kernel, never
// from host memory on the stream: a copy node recorded while a stream is being captured into a CUDA graph reads
// its host source again at every replay, long after the array it pointed to has gone.
constexpr int MAPS_PER_CHUNK = 16;
struct MapChunk {
    CUtensorMap m[MAPS_PER_CHUNK];
};
__global__ void __launch_bounds__(128) write_maps_kernel(const __grid_constant__ MapChunk c, CUtensorMap* dst, int n) {
    pdl_trigger();
    pdl_wait();  // the previous user of this scratch has finished
    const uint4* src = reinterpret_cast<const uint4*>(&c);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < n * (int)(sizeof(CUtensorMap) / 16); i += blockDim.x) d[i] = src[i];
}

template <class F, bool GATE_UP, int TN>
cudaError_t launch_gemm_kernel(cudaStream_t st, const GemmParams& G, const CUtensorMap& map_b, const CUtensorMap& map_bs) {
    const int smem_bytes = G_B_STAGES * (4 + (F::HAS_MIN ? 1 : 0)) * (TN * G_SLAB_K * 2) + (F::HAS_MIN ? 2 : 0) * G_TILE_BYTES +
                           (F::STAGE_W ? w_stages<F, TN>() * G_TILE_M * F::W_ROW_BYTES : 0) + 1024 /* alignment slack */;
    auto kfn = expert_gemm_kernel<F, GATE_UP, TN>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    return launch_k(kfn, dim3(g_gemm_sms), dim3(G_THREADS), (size_t)smem_bytes, st, G, map_b, map_bs);
}

}  // namespace

size_t prepacked_q80_bytes(int64_t n_rows, int k) { return (size_t)n_rows * (size_t)((k + 255) / 256) * GemmQ80::W_ROW_BYTES; }
cudaError_t launch_prepack_q80(cudaStream_t st, const void* raw, int64_t n_rows, int k, void* dst) {
    const int k_pad = (k + 255) / 256 * 256;
    const int64_t units = n_rows * (k_pad / 256);
    if (units == 0) return cudaSuccess;
    prepack_q80_kernel<<<(unsigned)((units + 7) / 8), 256, 0, st>>>(static_cast<const uint8_t*>(raw), n_rows, k, k_pad,
                                                                 static_cast<uint8_t*>(dst));
    return cudaGetLastError();
}

// Scratch the GEMM needs for P grouped rows of length K (fp16 operand, block-sum operand, scales).
size_t expert_gemm_scratch_bytes(int64_t P, int K, int parts) {
    K = (K + 255) / 256 * 256;  // Q8_0 rows are padded to whole 256-element blocks
    const size_t p_pad = (size_t)P + G_PAD_ROWS, kb = (size_t)K / 256;
    return align_up(p_pad * K * 2 * parts, 256) + align_up(p_pad * kb * 64 * 2, 256) + align_up(kb * p_pad * 4, 256) +
           sizeof(CUtensorMap) * 2 * CANDLE_MOE_MAX_EXPERTS;
}

// Takes Q4_K weights in GGUF layout (repacked = false), Q6_K weights in the repacked layout of the decode kernels
// and Q8_0 weights in the layout of prepack_q80_kernel (repacked = true); cudaErrorNotSupported for every other
// shape / dtype / layout.
cudaError_t launch_expert_gemm(cudaStream_t st, bool gate_up, const ExpertPtrs& wa, const ExpertPtrs& wb, int dtype,
                               bool repacked, int E, int K, int N, const uint32_t* offsets, const uint32_t* row_of, int64_t P,
                               int64_t max_rows, const int8_t* aq, const float* ascale, const int16_t* absum, float* out,
                               void* scratch, int max_splits, int* n_splits_out, int64_t split_stride) {
    if (n_splits_out) *n_splits_out = 1;
    if (!scratch) return cudaErrorNotSupported;
    int tn = max_rows <= 32 ? 32 : (max_rows <= 64 ? 64 : 128);  // position tile, from the bound / hint on an expert's rows
    const bool q80 = dtype == CANDLE_GGML_Q8_0 && repacked;
    if (!((dtype == CANDLE_GGML_Q4K && !repacked) || (dtype == CANDLE_GGML_Q6K && repacked) || q80)) return cudaErrorNotSupported;
    // Q8_0: the DOWN product runs with operands that carry the block scales rounded to fp16 (a few 1e-4 relative on a
    // product), which a final product tolerates.  The gate_up product does not: its f32 hidden rows are re-quantized to
    // int8 before W2, and a relative difference of 1e-4 from the reference's hidden values already moves a few per cent
    // of those int8 values by one step (1 / 127 of the block's largest value) -- measured, that amplification puts the
    // block at 3e-3 .. 5e-3 relative L2, outside its bound.  gate_up therefore takes the exact two-part operands.
    const bool q80x = q80 && gate_up;
    const int parts = q80x ? 2 : 1;
    const int K_in = K;
    if (q80) K = (K + 255) / 256 * 256;  // the repacked rows and the fp16 operand are padded with zeros
    if (K_in % (q80 ? 32 : 256) != 0 || N % (gate_up ? 64 : 128) != 0 || P <= 0 || P > (1 << 30)) return cudaErrorNotSupported;
    if (!encode_tiled_fn()) return cudaErrorNotSupported;
    if (g_gemm_sms < 0) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&g_gemm_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
    }
    const int kb = K / 256;
    const int64_t p_pad = P + G_PAD_ROWS;
    uint8_t* base = static_cast<uint8_t*>(scratch);
    __half* bf16 = reinterpret_cast<__half*>(base);
    float* bmin = reinterpret_cast<float*>(base + align_up((size_t)p_pad * K * 2 * parts, 256));
    float* d8t = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bmin) + align_up((size_t)p_pad * kb * 32 * 4, 256));
    const bool has_min = dtype == CANDLE_GGML_Q4K;

    const int64_t units = p_pad * kb;
    cudaError_t e = q80 ? launch_k(prep_gemm_b_q80_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, st, aq, ascale, row_of,
                                   (int)P, (int)p_pad, K_in, K, q80x ? 1 : 0, bf16, d8t)
                        : launch_k(prep_gemm_b_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, st, aq, ascale, absum,
                                   row_of, (int)P, (int)p_pad, K, bf16, has_min ? bmin : (float*)nullptr, d8t);
    if (e != cudaSuccess) return e;

    CUtensorMap map_b, map_bs;
    if (!make_map_2d(&map_b, bf16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)p_pad, (uint64_t)K * parts, G_SLAB_K, tn))
        return cudaErrorNotSupported;
    if (!make_map_2d(&map_bs, bmin, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)p_pad, (uint64_t)kb * 32, 32, tn))
        return cudaErrorNotSupported;

    // byte-matrix tensor maps of the raw weight blocks (Q4_K): [n_rows, kb * 144] with boxes of 64 rows x one block,
    // written to the head of the scratch on the stream before the kernel
    CUtensorMap* wmaps_dev = reinterpret_cast<CUtensorMap*>(reinterpret_cast<uint8_t*>(d8t) + align_up((size_t)kb * p_pad * 4, 256));
    if (dtype == CANDLE_GGML_Q4K || q80) {
        const int rec = q80 ? GemmQ80::W_ROW_BYTES : Q4K_BYTES, elem = q80 ? GemmQ80::W_MAP_ELEM : 1;
        const uint64_t n_rows = (uint64_t)N, rb = (uint64_t)kb * rec;
        for (int m0 = 0; m0 < 2 * E; m0 += MAPS_PER_CHUNK) {
            MapChunk chunk;
            const int n_maps = std::min(MAPS_PER_CHUNK, 2 * E - m0);
            for (int i = 0; i < n_maps; ++i) {
                const int e2 = (m0 + i) >> 1;
                const uint8_t* wp = ((m0 + i) & 1) && gate_up ? wb.p[e2] : wa.p[e2];
                if (!make_map_bytes(&chunk.m[i], wp, n_rows, rb, rec, 64, elem)) return cudaErrorNotSupported;
            }
            for (int i = n_maps; i < MAPS_PER_CHUNK; ++i) chunk.m[i] = chunk.m[0];
            e = launch_k(write_maps_kernel, dim3(1), dim3(128), 0, st, chunk, wmaps_dev + m0, n_maps);
            if (e != cudaSuccess) return e;
        }
    }

    GemmParams G{};
    G.wmaps = wmaps_dev;
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
    // down with few tiles (few experts with rows, narrow outputs): split K so that every SM has work; the partial
    // outputs are summed by whoever consumes them (combine, or the expert-parallel scatter)
    int ksplit = 1;
    if (!gate_up && n_splits_out && max_splits > 1) {
        const int64_t rows_per = std::max<int64_t>(1, std::min<int64_t>(max_rows, P));
        const int64_t items = (int64_t)G.m_tiles * std::max<int64_t>(1, std::min<int64_t>(E, (P + rows_per - 1) / rows_per)) *
                              ((rows_per + tn - 1) / tn);
        while (ksplit * 2 <= max_splits && kb % (ksplit * 2) == 0 && items * ksplit < 2 * (int64_t)g_gemm_sms) ksplit *= 2;
        *n_splits_out = ksplit;
    }
    G.ksplit = ksplit;
    G.zero = 0;
    G.split_stride = split_stride;
    e = stream_status_ptr(&G.status);
    if (e != cudaSuccess) return e;
    if (dtype == CANDLE_GGML_Q4K) {
        if (tn == 32)
            return gate_up ? launch_gemm_kernel<GemmQ4K, true, 32>(st, G, map_b, map_bs) : launch_gemm_kernel<GemmQ4K, false, 32>(st, G, map_b, map_bs);
        if (tn == 64)
            return gate_up ? launch_gemm_kernel<GemmQ4K, true, 64>(st, G, map_b, map_bs) : launch_gemm_kernel<GemmQ4K, false, 64>(st, G, map_b, map_bs);
        return gate_up ? launch_gemm_kernel<GemmQ4K, true, 128>(st, G, map_b, map_bs) : launch_gemm_kernel<GemmQ4K, false, 128>(st, G, map_b, map_bs);
    }
    if (q80x) {
        if (tn == 32) return launch_gemm_kernel<GemmQ80X, true, 32>(st, G, map_b, map_bs);
        if (tn == 64) return launch_gemm_kernel<GemmQ80X, true, 64>(st, G, map_b, map_bs);
        return launch_gemm_kernel<GemmQ80X, true, 128>(st, G, map_b, map_bs);
    }
    if (q80) {
        if (tn == 32) return launch_gemm_kernel<GemmQ80, false, 32>(st, G, map_b, map_bs);
        if (tn == 64) return launch_gemm_kernel<GemmQ80, false, 64>(st, G, map_b, map_bs);
        return launch_gemm_kernel<GemmQ80, false, 128>(st, G, map_b, map_bs);
    }
    if (tn == 32)
        return gate_up ? launch_gemm_kernel<GemmQ6K, true, 32>(st, G, map_b, map_bs) : launch_gemm_kernel<GemmQ6K, false, 32>(st, G, map_b, map_bs);
    if (tn == 64)
        return gate_up ? launch_gemm_kernel<GemmQ6K, true, 64>(st, G, map_b, map_bs) : launch_gemm_kernel<GemmQ6K, false, 64>(st, G, map_b, map_bs);
    return gate_up ? launch_gemm_kernel<GemmQ6K, true, 128>(st, G, map_b, map_bs) : launch_gemm_kernel<GemmQ6K, false, 128>(st, G, map_b, map_bs);
}

}  // namespace cmoe
