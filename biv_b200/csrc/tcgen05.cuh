// Inline-PTX helpers of the tcgen05 kernels: mbarriers with bounded waits, bulk
// copies, shared-memory matrix descriptors, MMA issue and commit, tensor-memory
// loads, packed f32x2 arithmetic.
#pragma once
#include <stdint.h>

namespace bivmoe {

constexpr uint32_t PF_WAIT_TRIES = 1u << 16;   // x up to 20 us each

__device__ __forceinline__ uint32_t pf_smem(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void pf_bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem(bar)), "r"(count));
}
__device__ __forceinline__ void pf_bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_smem(bar)) : "memory");
}
__device__ __forceinline__ void pf_bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pf_smem(bar)),
                 "r"(bytes)
                 : "memory");
}
// bounded wait for the phase of parity `parity`; false when it gave up
#ifndef PF_WAIT_HINT_NS
#define PF_WAIT_HINT_NS 20000
#endif
__device__ __forceinline__ bool pf_bar_wait(uint64_t* bar, uint32_t parity) {
#ifdef PF_WAIT_SPIN
    for (uint32_t i = 0; i < (PF_WAIT_TRIES << 8); i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(pf_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
#else
    for (uint32_t i = 0; i < PF_WAIT_TRIES; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(pf_smem(bar)), "r"(parity), "r"((uint32_t)PF_WAIT_HINT_NS)
            : "memory");
        if (ok) return true;
    }
    return false;
#endif
}
__device__ __forceinline__ void pf_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(pf_smem(dst)),
        "l"(src), "r"(bytes), "r"(pf_smem(bar))
        : "memory");
}
// Shared-memory matrix descriptor, K-major, no swizzle: 8 rows x 16 bytes are
// contiguous; `sbo` bytes from one 8-row group to the next, `lbo` bytes from
// one 16-byte K step to the next.
__device__ __forceinline__ uint64_t pf_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) |
           ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// The same for the 128-byte swizzle, K-major: a row is 128 contiguous bytes (64 bf16),
// 8 rows make a 1024-byte atom (1024-byte aligned), and the 16-byte piece c of row r of
// an atom sits at piece position c ^ r.  `sbo` = 1024 from one 8-row group to the next;
// a K step of 16 bf16 advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t pf_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// kind::i8 instruction descriptor: s32 accumulator, signed 8-bit A and B, both K-major
__device__ __forceinline__ uint32_t pf_idesc(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void pf_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"   // overwrite the buffer: a block dot is not accumulated
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}
// kind::f16 instruction descriptor: f32 accumulator, bf16 A and B, both K-major
__device__ __forceinline__ uint32_t pf_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// D (+)= A * B, 16 bf16 values of K per instruction
__device__ __forceinline__ void pf_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pf_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     pf_smem(bar))
                 : "memory");
}
__device__ __forceinline__ void pf_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void pf_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// 32 consecutive columns of this warp's 32 lanes of tensor memory
__device__ __forceinline__ void pf_tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void pf_tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void pf_tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// two f32 lanes per instruction (sm_100): d = a * b + c, d = a + b, d = a * b
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk(float lo, float hi) {
    return (f32x2)__float_as_uint(lo) | ((f32x2)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float lo_of(f32x2 v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_of(f32x2 v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}


}  // namespace bivmoe
