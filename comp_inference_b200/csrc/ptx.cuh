// Inline-PTX helpers shared by the staged kernels: mbarriers, bulk copies, explicit shared-memory
// loads, the rANS decode step and the bf16 packing of decoded weights.
#pragma once
#include "common.cuh"

namespace ci {

constexpr uint32_t kWaitPolls = 1u << 22;   // mbarrier polls before a wait gives up
constexpr uint32_t kLutBytes = kProbScale * 4;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// 1-D bulk copy global -> this CTA's own shared memory, 16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&x)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(b0), "r"(b1));
}

// bf16 bits of one weight from its table entry (symbol in bits 19..12) and sign+mantissa byte.
__device__ __forceinline__ uint32_t weight_bits(uint32_t entry, uint32_t man) {
    return ((entry >> 5) & 0x7F80u) | ((man & 0x80u) << 8) | (man & 0x7Fu);
}
// Two weights (rows k, k+1 of one column) as a packed bf16 pair, five instructions:
// both symbols are brought to bits 14..7 / 30..23 with one byte permute, both
// sign+mantissa bytes are doubled into their halves with another, one bit-select merges.
__device__ __forceinline__ uint32_t weight_pair(uint32_t e_lo, uint32_t e_hi, uint32_t m_lo, uint32_t m_hi) {
    const uint32_t ee = __byte_perm(e_lo >> 5, e_hi << 11, 0x7610);
    const uint32_t vv = __byte_perm(m_lo, m_hi, 0x4400);
    return (ee & 0x7F807F80u) | (vv & 0x807F807Fu);
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// One symbol with the table at shared address lut_s.
__device__ __forceinline__ uint32_t decode_fast(uint32_t &state, uint32_t lut_s) {
    const uint32_t e = lds_u32(lut_s + ((state & kProbMask) << 2));
    state = (e >> 20) * (state >> kProbBits) + (e & 0xFFFu);
    return e;
}
// The same with the table on a 16 KB boundary of the shared window: the entry's address needs no addition.
__device__ __forceinline__ uint32_t decode_aligned(uint32_t &state, uint32_t lut_s) {
    const uint32_t e = lds_u32(((state << 2) & ((kProbScale - 1) << 2)) | lut_s);
    state = (e >> 20) * (state >> kProbBits) + (e & 0xFFFu);
    return e;
}
// Renormalisation, STRIDE bytes between the rows of a stream.
//
// No lower-bound test anywhere in this family: a well-formed stream always has a byte left when its
// state is below 2^16, and the launchers guarantee enough mapped shared memory below every window
// that a malformed stream reads garbage instead of faulting.
//
// renorm_spec: exact.  The first byte is loaded by the caller before the state update is known to
// need it (its address does not depend on the new state, and some lane of the warp needs it on
// nearly every step anyway), which takes one shared-memory latency off the decode chain.  A second
// byte is needed exactly when the state before renormalisation is below 2^8, so its test and load
// do not wait for the first byte either.
template <uint32_t STRIDE>
__device__ __forceinline__ void renorm_spec(uint32_t &state, uint32_t &pos, uint32_t first) {
    asm volatile(
        "{\n\t.reg .pred p1, p2;\n\t.reg .u32 b;\n\t"
        "setp.lt.u32 p1, %0, 65536;\n\t"
        "setp.lt.u32 p2, %0, 256;\n\t"
        "@p2 ld.shared.u8 b, [%1+-%3];\n\t"
        "@p1 mad.lo.u32 %0, %0, 256, %2;\n\t"
        "@p1 sub.u32 %1, %1, %3;\n\t"
        "@p2 mad.lo.u32 %0, %0, 256, b;\n\t"
        "@p2 sub.u32 %1, %1, %3;\n\t}"
        : "+r"(state), "+r"(pos)
        : "r"(first), "n"(STRIDE));
}
// First byte only, already loaded by the caller (see renorm_spec); the caller handles a second byte.
template <uint32_t STRIDE>
__device__ __forceinline__ void renorm_first(uint32_t &state, uint32_t &pos, uint32_t first) {
    asm volatile(
        "{\n\t.reg .pred p1;\n\t"
        "setp.lt.u32 p1, %0, 65536;\n\t"
        "@p1 mad.lo.u32 %0, %0, 256, %2;\n\t"
        "@p1 sub.u32 %1, %1, %3;\n\t}"
        : "+r"(state), "+r"(pos)
        : "r"(first), "n"(STRIDE));
}
template <uint32_t STRIDE>
__device__ __forceinline__ void renorm_fast(uint32_t &state, uint32_t &pos) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .u32 b;\n\t"
        "setp.lt.u32 p, %0, 65536;\n\t"
        "@p ld.shared.u8 b, [%1];\n\t"
        "@p mad.lo.u32 %0, %0, 256, b;\n\t"
        "@p sub.u32 %1, %1, %2;\n\t}"
        : "+r"(state), "+r"(pos)
        : "n"(STRIDE));
}


__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Lane 0 polls an mbarrier phase, bounded; the verdict is broadcast to the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    if (lane_id() == 0)
        for (uint32_t it = 0; it < kWaitPolls && !ok; ++it) ok = mbar_try_wait(bar, parity);
    return __shfl_sync(kFull, ok, 0) != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

}  // namespace ci
