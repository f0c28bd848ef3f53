// PTX wrappers used by the streaming expert kernels: mbarrier, bulk async copy (TMA without a
// tensor map), ldmatrix and the int8 tensor-core MMAs.  Every wait is bounded.
#pragma once
#include <utility>
#include <type_traits>

#include <stdint.h>

namespace cmoe {

constexpr int SPIN_LIMIT = 1 << 22;  // mbarrier polls before a wait gives up (tens of milliseconds)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking look at the barrier (try_wait may park the thread for a while before it answers "not yet").
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the limit is reached, or
// as soon as another thread of the CTA has raised the flag.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int limit = SPIN_LIMIT) {
    if (mbar_try_wait(bar, parity)) return true;  // the common case costs one instruction and a branch
    for (int i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (i > 128) __nanosleep(20);
    }
    *abort_flag = 1;
    return false;
}
// The same wait for warps that run ahead of their consumer (producers waiting for a free stage): they sleep
// between polls so that their polling does not take issue slots from the warps that work.  (try_wait with a
// suspend-time hint is no alternative: it is expanded into exactly such a loop.)
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    for (int i = 0; i < SPIN_LIMIT; ++i) {
        __nanosleep(100);
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16), completion counted
// in bytes on `bar`.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// ask for [src, src + bytes) to be brought into L2 (16-byte aligned address, size a multiple of 16); no completion
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// barrier among the consumer warps only (ids 1.., the producer warp never joins)
__device__ __forceinline__ void consumer_sync(int n_threads) { asm volatile("bar.sync 1, %0;" ::"r"(n_threads) : "memory"); }

// Shared-memory reads by 32-bit shared-window address: no generic-pointer arithmetic, no address
// space conversion per access.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return (uint32_t)v;
}
__device__ __forceinline__ float ldsf(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
// A loop whose index is a compile-time constant in the body (usable as a template argument there):
// static_for<N>([&](auto I) { constexpr int i = decltype(I)::value; ... });
template <class Fn, int... Is>
__device__ __forceinline__ void static_for_impl(Fn&& f, std::integer_sequence<int, Is...>) {
    (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, class Fn>
__device__ __forceinline__ void static_for(Fn&& f) {
    static_for_impl(f, std::make_integer_sequence<int, N>{});
}

// The same with a compile-time byte offset folded into the instruction (one base register serves many accesses)
template <int OFF>
__device__ __forceinline__ void ldmatrix_x4_o(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4 + %5];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32_o(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1 + %2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds16_o(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1 + %2];" : "=h"(v) : "r"(addr), "n"(OFF));
    return (uint32_t)v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64_o(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2 + %3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128_o(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4 + %5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ void cp_async16_o(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %2], 16;" ::"r"(dst), "l"(src), "n"(OFF) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint64_t v) { asm volatile("st.shared.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }
__device__ __forceinline__ uint64_t lds64u(uint32_t addr) {
    uint64_t v;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}
// 16-byte asynchronous global -> shared copy (per thread, bypassing L1) and its group fences
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// D(16x8, s32) += A(16x32, s8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_s8_k32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// D(16x8, s32) += A(16x16, s8, row) * B(16x8, s8, col)
__device__ __forceinline__ void mma_s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
// Variants that start from zero (D = A * B): the zero accumulator is an immediate, no register moves.
__device__ __forceinline__ void mma_s8_k32_z(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_s8_k16_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void mma_s8u8_k16_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// Integer partial sums leave the tensor core as floats: the accumulator starts at the bit pattern
// of 1.5 * 2^23, so `start + dot` re-read as a float is 12582912 + dot exactly (|dot| < 2^22),
// and one FADD recovers float(dot).  Scaling then runs on the FP32 pipe instead of integer
// multiplies, which are several times slower on this part.
constexpr int MAGIC_I = 0x4B400000;
constexpr float MAGIC_F = 12582912.0f;
__device__ __forceinline__ void mma_s8_k32_m(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(MAGIC_I));
}
__device__ __forceinline__ void mma_u8s8_k32_m(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(MAGIC_I));
}
__device__ __forceinline__ void mma_s8_k16_m(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(MAGIC_I));
}
__device__ __forceinline__ void mma_s8u8_k16_m(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(MAGIC_I));
}
__device__ __forceinline__ float unmagic(int v) { return __int_as_float(v) - MAGIC_F; }
// float(byte j of w) for an unsigned byte: the byte is dropped into the mantissa of 2^23
__device__ __forceinline__ float byte_to_float(uint32_t w, int j) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 | j)) - 8388608.0f;
}
// byte j of w, zero-extended / sign-extended, in one permute
__device__ __forceinline__ int byte_u(uint32_t w, int j) { return (int)__byte_perm(w, 0, 0x4440 | j); }
// (prmt with bit 3 of a selector nibble set copies the sign of the selected byte; the __byte_perm
// intrinsic ignores that bit, hence the inline PTX)
__device__ __forceinline__ int byte_s(uint32_t w, int j) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"(0x8880u | (uint32_t)(j * 0x1110) | (uint32_t)j));
    return (int)r;
}
// same with an unsigned B operand
__device__ __forceinline__ void mma_s8u8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

}  // namespace cmoe
