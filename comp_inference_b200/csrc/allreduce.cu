// One-shot all-reduce of a small bf16 activation tensor over peer memory (NVLink / NVSwitch), for the
// outputs of row-parallel linears: at 8 KB per message the exchange is pure latency, and a library
// collective spends most of it on its own launch and protocol.  The reference has no multi-GPU code;
// this replaces the NCCL all-reduce a tensor-parallel port would call.
//
// Every rank owns a buffer that all peers can write: [2 parities][world ranks][capacity / 2] words of 8
// bytes = two bf16 values + the sequence number of the call that wrote them, and one call counter per CTA
// (counted on the device, so a captured CUDA graph can be replayed).  A call with sequence number s and
// parity s % 2:
//   1. each thread stores its pairs of the input, tagged with s, into slot [parity][own rank] of EVERY rank's
//      buffer with single 8-byte stores (value and tag become visible together: no fence, no separate flag);
//   2. it polls the same pairs of all world slots of its OWN buffer until their tag equals s (bounded; on
//      expiry it sets the status word and carries on), adds them in rank order in fp32 and writes bf16.
// Two parities suffice: a rank can only get past step 2 of call s + 1 once every peer has started call
// s + 1, i.e. finished reading call s, so the slots of parity s % 2 are free again for call s + 2.  Every
// call launches the same number of CTAs and each bumps its own counter, so all counters agree and a stale
// tag is always smaller than the current one.  No multicast, no TMA, no spin without a bound.
#include "common.cuh"

namespace ci {

constexpr uint32_t kArCtas = 8;
constexpr uint32_t kArThreads = 256;
constexpr uint32_t kArMaxWorld = 8;
constexpr uint32_t kArPolls = 1u << 21;      // about a second of polling before a wait gives up

struct ArArgs {
    uint16_t *bufs[kArMaxWorld];       // every rank's buffer, as mapped into this process
    uint32_t *counters;                // this rank's per-CTA call counters (local memory)
    uint32_t *status;                  // may be null
    const uint16_t *in;
    uint16_t *out;
    uint32_t n, capacity, rank, world;
    uint32_t polls;                    // loads of one slot before a wait gives up
    uint32_t gather_cols;              // 0: sum over the ranks; else all-gather of [n / gather_cols, gather_cols] blocks
};

__device__ __forceinline__ void st_pair(uint2 *p, uint32_t data, uint32_t tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreads) k_allreduce_oneshot(const __grid_constant__ ArArgs a) {
    // activations may be the previous kernel's output (programmatic dependent launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t seq = a.counters[blockIdx.x] + 1, parity = seq & 1u;
    const uint32_t pairs = (a.n + 1) / 2, cap2 = a.capacity / 2;
    const size_t my_slot = ((size_t)parity * a.world + a.rank) * cap2;
    bool timed_out = false;
    for (uint32_t i = blockIdx.x * kArThreads + threadIdx.x; i < pairs; i += kArCtas * kArThreads) {
        const uint32_t lo = a.in[2 * i], hi = 2 * i + 1 < a.n ? a.in[2 * i + 1] : 0u;
        const uint32_t data = lo | (hi << 16);
        for (uint32_t q = 0; q < a.world; ++q) st_pair(reinterpret_cast<uint2 *>(a.bufs[q]) + my_slot + i, data, seq);
        float s0 = 0.f, s1 = 0.f;
        const uint2 *mine = reinterpret_cast<const uint2 *>(a.bufs[a.rank]) + (size_t)parity * a.world * cap2 + i;
        // all-gather: element e = (row, col) of rank q's block lands at out[row][q * gather_cols + col];
        // gather_cols is even, so a pair never straddles two rows
        const uint32_t g_row = a.gather_cols ? (2 * i) / a.gather_cols : 0u;
        const uint32_t g_col = a.gather_cols ? (2 * i) - g_row * a.gather_cols : 0u;
        for (uint32_t q = 0; q < a.world; ++q) {
            uint2 v = ld_pair(mine + (size_t)q * cap2);
            for (uint32_t it = 0; v.y != seq && it < a.polls; ++it) v = ld_pair(mine + (size_t)q * cap2);
            timed_out |= v.y != seq;
            if (a.gather_cols) {
                uint32_t *dst = reinterpret_cast<uint32_t *>(a.out + ((size_t)g_row * a.world + q) * a.gather_cols + g_col);
                *dst = v.x;
            } else {
                s0 += bf16_bits_to_float(v.x & 0xFFFFu);
                s1 += bf16_bits_to_float(v.x >> 16);
            }
        }
        if (a.gather_cols == 0) {
            a.out[2 * i] = float_to_bf16_bits(s0);
            if (2 * i + 1 < a.n) a.out[2 * i + 1] = float_to_bf16_bits(s1);
        }
    }
    if (timed_out && a.status) atomicExch(a.status, 9u);
    __syncthreads();
    if (threadIdx.x == 0) a.counters[blockIdx.x] = seq;
}

}  // namespace ci

using namespace ci;

static uint32_t g_ar_polls = kArPolls;

extern "C" {

void ci_allreduce_set_poll_limit(uint32_t polls) { g_ar_polls = polls ? polls : kArPolls; }

size_t ci_allreduce_buffer_bytes(uint32_t world, uint32_t capacity) {
    return (size_t)2 * world * (capacity / 2) * 8;             // two parities x world slots x pairs of (data, tag)
}
size_t ci_allreduce_counter_bytes(void) { return (size_t)kArCtas * sizeof(uint32_t); }

int ci_allreduce_oneshot(const uint16_t *d_in, uint16_t *d_out, uint32_t n, uint32_t capacity, void *const *peer_bufs,
                         uint32_t *d_counters, uint32_t rank, uint32_t world, uint32_t *d_status, ci_stream_t stream) {
    CI_REQUIRE(d_in && d_out && peer_bufs && d_counters, "null pointer");
    CI_REQUIRE(capacity % 8 == 0, "capacity must be a multiple of 8 elements");
    CI_REQUIRE(world >= 1 && world <= kArMaxWorld && rank < world, "world size %u / rank %u out of range", world, rank);
    CI_REQUIRE(n <= capacity, "%u elements exceed the buffer capacity %u", n, capacity);
    if (n == 0) return CI_OK;
    ArArgs a;
    for (uint32_t q = 0; q < kArMaxWorld; ++q) {
        a.bufs[q] = q < world ? reinterpret_cast<uint16_t *>(peer_bufs[q]) : nullptr;
        CI_REQUIRE(q >= world || a.bufs[q], "null peer pointer for rank %u", q);
    }
    a.counters = d_counters; a.status = d_status; a.in = d_in; a.out = d_out;
    a.n = n; a.capacity = capacity; a.rank = rank; a.world = world;
    a.polls = g_ar_polls;
    a.gather_cols = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kArCtas);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CI_CUDA(cudaLaunchKernelEx(&cfg, k_allreduce_oneshot, a));
    return CI_OK;
}

int ci_allgather_oneshot(const uint16_t *d_in, uint16_t *d_out, uint32_t rows, uint32_t cols, uint32_t capacity,
                         void *const *peer_bufs, uint32_t *d_counters, uint32_t rank, uint32_t world, uint32_t *d_status,
                         ci_stream_t stream) {
    CI_REQUIRE(d_in && d_out && peer_bufs && d_counters, "null pointer");
    CI_REQUIRE(d_in != d_out, "the all-gather cannot run in place");
    CI_REQUIRE(capacity % 8 == 0, "capacity must be a multiple of 8 elements");
    CI_REQUIRE(world >= 1 && world <= kArMaxWorld && rank < world, "world size %u / rank %u out of range", world, rank);
    CI_REQUIRE(cols % 2 == 0 && cols > 0, "the per-rank width %u must be even", cols);
    CI_REQUIRE((uint64_t)rows * cols <= capacity, "%u x %u elements exceed the buffer capacity %u", rows, cols, capacity);
    CI_REQUIRE((reinterpret_cast<uintptr_t>(d_out) & 3u) == 0, "output must be 4-byte aligned");
    if (rows == 0) return CI_OK;
    ArArgs a;
    for (uint32_t q = 0; q < kArMaxWorld; ++q) {
        a.bufs[q] = q < world ? reinterpret_cast<uint16_t *>(peer_bufs[q]) : nullptr;
        CI_REQUIRE(q >= world || a.bufs[q], "null peer pointer for rank %u", q);
    }
    a.counters = d_counters; a.status = d_status; a.in = d_in; a.out = d_out;
    a.n = rows * cols; a.capacity = capacity; a.rank = rank; a.world = world;
    a.polls = g_ar_polls;
    a.gather_cols = cols;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kArCtas);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CI_CUDA(cudaLaunchKernelEx(&cfg, k_allreduce_oneshot, a));
    return CI_OK;
}

}  // extern "C"
