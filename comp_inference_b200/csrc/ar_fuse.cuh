// Device side of the all-reduce fused into the row-parallel GEMV: the warps that hold the final sums of a
// column group push them straight into every peer's exchange buffer and add the peers' values, instead of
// writing the partial output for a separate exchange kernel.  Same protocol as k_allreduce_oneshot
// (allreduce.cu): pairs of bf16 values tagged with the call's sequence number in single 8-byte peer stores,
// bounded polling of the own buffer, summation in rank order, two parities.
#pragma once
#include "common.cuh"

namespace ci {

constexpr uint32_t kFuseMaxWorld = 8;
constexpr uint32_t kFusePolls = 1u << 21;    // about a second

struct ArFuse {
    uint16_t *bufs[kFuseMaxWorld];   // every rank's exchange buffer as mapped into this process
    uint32_t *counter;               // [0] sequence number of the last finished call, [1] groups finished in this call
    uint32_t *status;                // may be null
    uint32_t rank, world, capacity;  // world == 0: no exchange
};

#ifdef __CUDACC__
__device__ __forceinline__ void fuse_st_pair(uint2 *p, uint32_t data, uint32_t tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 fuse_ld_pair(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// Sequence number of the running call (the counter is advanced by the warp that finishes the call's last group).
__device__ __forceinline__ uint32_t fuse_seq(const ArFuse &f) {
    return *reinterpret_cast<volatile uint32_t *>(f.counter) + 1;
}
// Pushes this rank's two values of elements (2 * pair, 2 * pair + 1), waits for every rank's, returns the sums.
__device__ __forceinline__ float2 fuse_exchange_pair(const ArFuse &f, uint32_t seq, uint32_t pair, float lo, float hi) {
    const uint32_t parity = seq & 1u, cap2 = f.capacity / 2;
    const uint32_t data = (uint32_t)float_to_bf16_bits(lo) | ((uint32_t)float_to_bf16_bits(hi) << 16);
    const size_t slot = ((size_t)parity * f.world + f.rank) * cap2 + pair;
    for (uint32_t q = 0; q < f.world; ++q) fuse_st_pair(reinterpret_cast<uint2 *>(f.bufs[q]) + slot, data, seq);
    const uint2 *mine = reinterpret_cast<const uint2 *>(f.bufs[f.rank]) + (size_t)parity * f.world * cap2 + pair;
    float s0 = 0.f, s1 = 0.f;
    bool timed_out = false;
    for (uint32_t q = 0; q < f.world; ++q) {
        uint2 v = fuse_ld_pair(mine + (size_t)q * cap2);
        for (uint32_t it = 0; v.y != seq && it < kFusePolls; ++it) v = fuse_ld_pair(mine + (size_t)q * cap2);
        timed_out |= v.y != seq;
        s0 += bf16_bits_to_float(v.x & 0xFFFFu);
        s1 += bf16_bits_to_float(v.x >> 16);
    }
    if (timed_out && f.status) atomicExch(f.status, 9u);
    return make_float2(s0, s1);
}
// Called by one lane once a column group's exchange is complete; the last group closes the call.
__device__ __forceinline__ void fuse_group_done(const ArFuse &f, uint32_t seq, uint32_t groups) {
    __threadfence();
    if (atomicAdd(f.counter + 1, 1u) == groups - 1) {
        f.counter[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t *>(f.counter) = seq;
    }
}
#endif

}  // namespace ci
