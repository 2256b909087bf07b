// Fused decode + GEMM for prefill (many activation rows): y[M,N] = x[M,K] . W[K,N] with W decoded
// from its rANS streams inside the kernel and multiplied on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory).  Replaces the decompress + triton_matmul pair
// (comp_inference/triton_gemm.py:234-337) and the large-M use of fused_rans_linear_triton
// (comp_inference/linear_triton.py:229-552).
//
// The problem is computed transposed, D[n, m] = sum_k W[k, n] * x[m, k]:
//   * A operand (UMMA M = 128): 128 weight columns x 128 k rows of one tile row, written by four
//     decode warps (one 32-column unit each, two streams per lane) as bf16 straight into the
//     K-major, 128-byte-swizzled shared-memory layout the tensor core reads -- the decoded matrix
//     never exists in global memory;
//   * B operand (UMMA N = 256): 256 activation rows x 64 k, fetched by TMA (tiled tensor map over
//     x, 128-byte swizzle) into a ring of three slots by a producer warp;
//   * D: 128 x 512 fp32 in tensor memory (all 512 columns), i.e. up to 512 activation rows per CTA,
//     read back with tcgen05.ld for the epilogue.
// One thread issues the MMAs; mbarriers (full/empty per ring slot, tcgen05.commit for completion)
// connect the roles.  Grid = (N/128) x ceil(M/512) x split-K; split-K partials are fp32 and are
// summed in a fixed order (deterministic) by k_splitk_reduce, a chip-wide grid launched right behind.
//
// Every wait is bounded: on expiry the role sets the status word, raises a CTA-wide abort flag and
// falls through to the common exit, where tensor memory is released.
#include <cuda.h>

#include "linear.cuh"
#include "ptx.cuh"

namespace ci {

constexpr uint32_t kBN = 128;              // weight columns per CTA  (UMMA M)
constexpr uint32_t kBM = 256;              // activation rows per MMA  (UMMA N)
constexpr uint32_t kMChunks = 2;           // accumulators per CTA -> 512 activation rows
constexpr uint32_t kBK = 64;               // k per shared-memory sub-tile: 64 bf16 = one 128-byte row
constexpr uint32_t kTileH = 128;           // tile height this kernel is specialised for (2 sub-tiles per tile row)
constexpr uint32_t kASub = kBN * kBK * 2;  // 16 KB
constexpr uint32_t kAStage = 2 * kASub;    // 32 KB: streams "A" fill sub-tile 0, streams "B" sub-tile 1
constexpr uint32_t kAStages = 3;
constexpr uint32_t kBTile = kBM * kBK * 2; // 32 KB
constexpr uint32_t kBSlots = 2;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kDecGroups = 2;        // two groups of four decode warps work on alternate tile rows
constexpr uint32_t kDecWarps = 4 * kDecGroups;
constexpr uint32_t kTmaWarp = kDecWarps, kMmaWarp = kDecWarps + 1;
constexpr uint32_t kGemmThreads = (kDecWarps + 2) * 32;   // decode + epilogue warps, TMA producer, MMA issuer

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffA = 0;
constexpr uint32_t kOffB = kOffA + kAStages * kAStage;          // 65536
constexpr uint32_t kOffLut = kOffB + kBSlots * kBTile;          // 163840
constexpr uint32_t kOffBar = kOffLut + kLutBytes;              // + 16384
constexpr uint32_t kBarRegion = 256;
constexpr uint32_t kOffStage = kOffBar + kBarRegion;            // per-warp copy buffers follow

// barrier slots (8 bytes each) inside the barrier region
enum : uint32_t {
    kBarFullA = 0,      // [3]  4 arrivals (the decode warps of one group)
    kBarEmptyA = 3,     // [3]  1 arrival  (tcgen05.commit)
    kBarFullB = 6,      // [2]  1 arrival + bytes (TMA)
    kBarEmptyB = 8,     // [2]  1 arrival  (tcgen05.commit)
    kBarAcc = 10,       // [1]  1 arrival  (tcgen05.commit after the last MMA)
    kBarCopy = 11,      // [8][2] per decode warp, per copy stage
    kBarCount = 27,
};
constexpr uint32_t kOffTmemPtr = kBarCount * 8;                  // u32: base address from tcgen05.alloc
constexpr uint32_t kOffAbort = kOffTmemPtr + 4;                  // u32: set when a wait ran out

struct GemmArgs {
    LinArgs a;
    uint32_t win_cap;                             // bytes per copy stage (a tile's compressed byte block); 2 stages per decode warp
    uint32_t m_tiles;                             // ceil(M / 512)
    uint32_t splits, tiles_per_split;             // split-K over tile rows
    uint32_t *status;
};

// ---- tcgen05 / TMA wrappers ------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive columns of fp32 from tensor memory (lane l of the warp gets row base+l).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 2-D tiled TMA load into this CTA's shared memory; c0 is the innermost (k) coordinate in elements.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t c0, int32_t c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 bytes, eight rows
// (1024 bytes) per swizzle atom, atoms of consecutive row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
    d |= (uint64_t)1 << 16;                               // leading byte offset (not used by this layout)
    d |= (uint64_t)(1024u >> 4) << 32;                    // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                               // 128-byte swizzle
    return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kBM >> 3) << 17) | ((kBN >> 4) << 24);

// Byte offset of the 16-byte chunk (8 consecutive k) `c` of weight column `n` inside a sub-tile.
__device__ __forceinline__ uint32_t a_chunk_offset(uint32_t n, uint32_t c) {
    return (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4);
}

// ---- the kernel -----------------------------------------------------------------------------------

__global__ void __launch_bounds__(kGemmThreads, 1)
k_linear_gemm(const __grid_constant__ GemmArgs p, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ uint8_t smem_raw[];
    const LinArgs &a = p.a;
    const Geom &g = a.g;
    const uint32_t smem_s = (smem_u32(smem_raw) + 1023u) & ~1023u;      // 128-byte swizzle wants 1024-byte alignment
    uint8_t *smem = smem_raw + (smem_s - smem_u32(smem_raw));
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t bar_s = smem_s + kOffBar;
    auto bar = [&](uint32_t slot) { return bar_s + slot * 8; };
    volatile uint32_t *s_tmem = reinterpret_cast<volatile uint32_t *>(smem + kOffBar + kOffTmemPtr);
    volatile uint32_t *s_abort = reinterpret_cast<volatile uint32_t *>(smem + kOffBar + kOffAbort);

    const uint32_t nblk = blockIdx.x, mtile = blockIdx.y, split = blockIdx.z;
    const uint32_t m0 = mtile * (kBM * kMChunks);
    const uint32_t m_here = min(a.M - m0, kBM * kMChunks);
    const uint32_t chunks = (m_here + kBM - 1) / kBM;                    // accumulators in use: 1 or 2
    const uint32_t k_begin = split * p.tiles_per_split, k_end = min(k_begin + p.tiles_per_split, g.tiles_k);
    const uint32_t n_iters = k_end - k_begin;

    // ---- set-up ---------------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kAStages; ++i) { mbar_init(bar(kBarFullA + i), 4); mbar_init(bar(kBarEmptyA + i), 1); }
        for (uint32_t i = 0; i < kBSlots; ++i) { mbar_init(bar(kBarFullB + i), 1); mbar_init(bar(kBarEmptyB + i), 1); }
        mbar_init(bar(kBarAcc), 1);
        for (uint32_t i = 0; i < 2 * kDecWarps; ++i) mbar_init(bar(kBarCopy + i), 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    load_lut(reinterpret_cast<uint32_t *>(smem + kOffLut), a.lut, a.tables, a.slot_map);
    if (warp == kMmaWarp) tmem_alloc(smem_s + kOffBar + kOffTmemPtr, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    // Programmatic dependent launch: the set-up above overlapped the previous kernel's tail; activations,
    // workspace and output may be that kernel's, so wait for it here (no-ops in an ordinary launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    auto give_up = [&](uint32_t code) {
        if (lane == 0) { atomicExch(p.status, code); *s_abort = 1; }
    };

    if (warp < kDecWarps) {
        // =========================== decode warps: fill the A stages ===============================
        // Group j (warps 4j..4j+3) decodes tile rows j, j+2, ...; warp q of a group owns 32 columns.
        const uint32_t grpj = warp >> 2, q = warp & 3;
        const uint32_t grp = nblk * 4 + q;                               // this warp's 32-column group
        const bool grp_live = grp < g.groups;
        const uint32_t lut_s = smem_s + kOffLut;
        const uint32_t copy_s = smem_s + kOffStage + warp * (2 * p.win_cap);
        const uint32_t man_tile = kTileH * 32;
        const uint32_t nl = q * 32 + lane;                               // column inside the CTA's 128

        // Metadata and initial states of a unit are loaded one unit ahead (all of it is small and
        // L2/HBM resident), so a unit never starts with a dependent global load.
        struct Unit { uint32_t off, ml, stA, stB; };
        auto load_unit = [&](uint32_t tk) {
            Unit u = {0u, 0u, kRansL, kRansL};
            if (grp_live) {
                const uint32_t t0 = tk * g.tiles_n + grp;                // tile width 32: one tile per unit
                u.off = __ldg(a.tile_offsets + t0);
                u.ml = __ldg(a.tile_max_lens + t0);
                u.stA = __ldg(a.states + (size_t)t0 * 64 + lane);
                u.stB = __ldg(a.states + (size_t)t0 * 64 + 32 + lane);
            }
            return u;
        };
        auto issue = [&](const Unit &u, uint32_t cs) {                   // bulk copy of a unit's byte block
            if (lane != 0 || !grp_live) return;
            uint32_t wbytes = u.ml * 64u;
            if (wbytes > p.win_cap) { atomicExch(p.status, 2u); wbytes = 0; }
            const uint32_t b = bar(kBarCopy + warp * 2 + cs);
            fence_async_proxy();
            if (wbytes) {
                mbar_expect_tx(b, wbytes);
                bulk_load(copy_s + cs * p.win_cap, a.stream + u.off, wbytes, b);
            } else {
                mbar_arrive(b);                                          // nothing to copy: complete the phase by hand
            }
        };
        // sign+mantissa bytes of eight rows of both halves, straight from global memory (L2/L1), fetched one
        // pass ahead of their use so their latency never sits on the decode chain
        auto load_man = [&](const uint8_t *mg, uint32_t i0, uint32_t (&m)[16]) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                m[r] = __ldg(mg + (i0 + r) * 32);
                m[8 + r] = __ldg(mg + (64 + i0 + r) * 32);
            }
        };

        uint32_t copy_parity[2] = {0, 0};
        Unit cur = {0u, 0u, kRansL, kRansL}, nxt = cur, nxt2 = cur;
        if (grpj < n_iters) {
            cur = load_unit(k_begin + grpj);
            issue(cur, 0);
        }
        if (grpj + kDecGroups < n_iters) nxt = load_unit(k_begin + grpj + kDecGroups);
        uint32_t li = 0;
        for (uint32_t it = grpj; it < n_iters && !*s_abort; it += kDecGroups, ++li) {
            const uint32_t tk = k_begin + it, s = it % kAStages, cs = li & 1;
            if (it + kDecGroups < n_iters) issue(nxt, cs ^ 1);
            if (it + 2 * kDecGroups < n_iters) nxt2 = load_unit(tk + 2 * kDecGroups);
            // the stage must have been drained by the MMAs that read it kAStages iterations ago
            if (!mbar_wait_warp(bar(kBarEmptyA + s), ((it / kAStages) & 1) ^ 1)) { give_up(3); break; }
            const uint32_t a0_s = smem_s + kOffA + s * kAStage, a1_s = a0_s + kASub;
            if (!grp_live) {                                             // columns beyond N: zeros
                for (uint32_t c = 0; c < 8; ++c) {
                    sts_v4(a0_s + a_chunk_offset(nl, c), 0, 0, 0, 0);
                    sts_v4(a1_s + a_chunk_offset(nl, c), 0, 0, 0, 0);
                }
            } else {
                const uint32_t t0 = tk * g.tiles_n + grp;
                const uint8_t *mg = a.mantissa + (size_t)t0 * man_tile + lane;
                const uint32_t row0 = tk * kTileH, remain = g.K - row0;
                const uint32_t nA = min(remain, 64u), nB = remain > 64u ? min(remain - 64u, 64u) : 0;
                const bool full_tile = nB == 64;
                uint32_t m0r[16], m1r[16];
                if (full_tile) load_man(mg, 0, m0r);
                uint32_t stA = cur.stA, stB = cur.stB;
                const uint32_t ml = cur.ml;
                if (!mbar_wait_warp(bar(kBarCopy + warp * 2 + cs), copy_parity[cs])) { give_up(4); break; }
                copy_parity[cs] ^= 1;
                const uint32_t win_s = copy_s + cs * p.win_cap;
                uint32_t posA = win_s + lane + (ml - 1) * 64u, posB = posA + 32;   // an empty tile starts one row below

                // one pass = eight k rows of both halves -> one 16-byte chunk in each sub-tile
                auto pass = [&](uint32_t c, const uint32_t (&m)[16]) {
                    uint32_t pa[4], pb[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t ba = lds_u8(posA), bb = lds_u8(posB);
                        const uint32_t e0 = decode_fast(stA, lut_s);
                        const uint32_t f0 = decode_fast(stB, lut_s);
                        renorm_spec<64>(stA, posA, ba);
                        renorm_spec<64>(stB, posB, bb);
                        ba = lds_u8(posA);
                        bb = lds_u8(posB);
                        const uint32_t e1 = decode_fast(stA, lut_s);
                        const uint32_t f1 = decode_fast(stB, lut_s);
                        renorm_spec<64>(stA, posA, ba);
                        renorm_spec<64>(stB, posB, bb);
                        pa[j] = weight_pair(e0, e1, m[2 * j], m[2 * j + 1]);
                        pb[j] = weight_pair(f0, f1, m[8 + 2 * j], m[8 + 2 * j + 1]);
                    }
                    sts_v4(a0_s + a_chunk_offset(nl, c), pa[0], pa[1], pa[2], pa[3]);
                    sts_v4(a1_s + a_chunk_offset(nl, c), pb[0], pb[1], pb[2], pb[3]);
                };
                if (full_tile) {
#pragma unroll 1
                    for (uint32_t c = 0; c < 8; c += 2) {
                        load_man(mg, (c + 1) * 8, m1r);
                        pass(c, m0r);
                        if (c + 2 < 8) load_man(mg, (c + 2) * 8, m0r);
                        pass(c + 1, m1r);
                    }
                } else {                                                 // ragged last tile row: zeros beyond K
#pragma unroll 1
                    for (uint32_t c = 0; c < 8; ++c) {
                        uint32_t pa[4], pb[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t h[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                            for (int qq = 0; qq < 2; ++qq) {
                                const uint32_t i = c * 8 + 2 * j + qq;
                                if (i < nA) {
                                    const uint32_t e = decode_fast(stA, lut_s);
                                    renorm_fast<64>(stA, posA);
                                    renorm_fast<64>(stA, posA);
                                    h[qq] = weight_bits(e, __ldg(mg + i * 32));
                                }
                                if (i < nB) {
                                    const uint32_t e = decode_fast(stB, lut_s);
                                    renorm_fast<64>(stB, posB);
                                    renorm_fast<64>(stB, posB);
                                    h[2 + qq] = weight_bits(e, __ldg(mg + (64 + i) * 32));
                                }
                            }
                            pa[j] = h[0] | (h[1] << 16);
                            pb[j] = h[2] | (h[3] << 16);
                        }
                        sts_v4(a0_s + a_chunk_offset(nl, c), pa[0], pa[1], pa[2], pa[3]);
                        sts_v4(a1_s + a_chunk_offset(nl, c), pb[0], pb[1], pb[2], pb[3]);
                    }
                }
            }
            fence_async_proxy();                                         // generic writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarFullA + s));
            cur = nxt;
            nxt = nxt2;
        }
    } else if (warp == kTmaWarp) {
        // =========================== TMA producer: activation tiles ================================
        uint32_t cnt = 0;
        for (uint32_t it = 0; it < n_iters && !*s_abort; ++it) {
            const uint32_t tk = k_begin + it;
            bool ok = true;
            for (uint32_t ks = 0; ks < 2 && ok; ++ks)
                for (uint32_t mc = 0; mc < chunks && ok; ++mc, ++cnt) {
                    const uint32_t r = cnt % kBSlots;
                    if (!mbar_wait_warp(bar(kBarEmptyB + r), ((cnt / kBSlots) & 1) ^ 1)) { give_up(5); ok = false; break; }
                    if (lane == 0) {
                        mbar_expect_tx(bar(kBarFullB + r), kBTile);
                        tma_load_2d(smem_s + kOffB + r * kBTile, &x_map, (int32_t)(tk * kTileH + ks * kBK),
                                    (int32_t)(m0 + mc * kBM), bar(kBarFullB + r));
                    }
                }
            if (!ok) break;
        }
    } else {
        // =========================== MMA issuer ======================================================
        uint32_t cnt = 0;
        bool ok = true;
        for (uint32_t it = 0; it < n_iters && ok && !*s_abort; ++it) {
            const uint32_t s = it % kAStages;
            if (!mbar_wait_warp(bar(kBarFullA + s), (it / kAStages) & 1)) { give_up(6); break; }
            tc_fence_after();
            for (uint32_t ks = 0; ks < 2 && ok; ++ks)
                for (uint32_t mc = 0; mc < chunks && ok; ++mc, ++cnt) {
                    const uint32_t r = cnt % kBSlots;
                    if (!mbar_wait_warp(bar(kBarFullB + r), (cnt / kBSlots) & 1)) { give_up(7); ok = false; break; }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint64_t ad = umma_desc_sw128(smem_s + kOffA + s * kAStage + ks * kASub);
                        const uint64_t bd = umma_desc_sw128(smem_s + kOffB + r * kBTile);
#pragma unroll
                        for (uint32_t kk = 0; kk < kBK / 16; ++kk)       // 16 k per instruction = 32 bytes = +2 in the address field
                            umma_bf16(tmem_base + mc * kBM, ad + 2 * kk, bd + 2 * kk, kIdesc, (it | ks | kk) != 0);
                        umma_commit(bar(kBarEmptyB + r));                // slot free once these MMAs have read it
                    }
                    __syncwarp();
                }
            if (ok && lane == 0) umma_commit(bar(kBarEmptyA + s));
            __syncwarp();
        }
        if (lane == 0) umma_commit(bar(kBarAcc));                        // all MMAs done -> accumulators final
        __syncwarp();
    }

    // ---- epilogue: the four decode warps read the accumulators out of tensor memory ----------------
    if (warp < kDecWarps) {
        bool ok = !*s_abort;
        if (ok && !mbar_wait_warp(bar(kBarAcc), 0)) { give_up(8); ok = false; }
        if (ok) {
            tc_fence_after();
            const uint32_t q = warp & 3, half = warp >> 2;               // a warp may only touch tensor-memory lanes 32*(warp%4)..
            const uint32_t n = nblk * kBN + q * 32 + lane;               // accumulator row = weight column
            const float bias = (a.bias && n < g.N && p.splits == 1) ? load_bf16(a.bias + n) : 0.f;
            for (uint32_t mc = 0; mc < chunks; ++mc)
                for (uint32_t cc = half; cc < kBM / 32; cc += kDecGroups) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((q * 32u) << 16) + mc * kBM + cc * 32, v);
                    const uint32_t mb = m0 + mc * kBM + cc * 32;
                    if (n < g.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t m = mb + j;
                            if (m >= a.M) break;
                            const float f = __uint_as_float(v[j]);
                            if (p.splits == 1) a.y[(size_t)m * a.ldy + n] = float_to_bf16_bits(f + bias);
                            else a.partial[((size_t)split * a.M + m) * g.N + n] = f;
                        }
                    }
                }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// Split-K epilogue: y = bf16(sum over splits of the fp32 partials (+ bias)), fixed summation order
// (deterministic).  A separate grid over the whole chip: one CTA per output block would have to pull
// splits x 256 KB through a single SM.  Launched with programmatic dependent launch right behind the GEMM.
__global__ void __launch_bounds__(256) k_splitk_reduce(const float *__restrict__ partial, uint32_t splits, uint32_t M,
                                                        uint32_t N, const uint16_t *__restrict__ bias, uint16_t *y,
                                                        int64_t ldy, uint32_t vec) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t plane = (size_t)M * N;
    if (vec) {
        const uint32_t quads = N / 4;
        const size_t items = (size_t)M * quads;
        for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < items; idx += (size_t)gridDim.x * blockDim.x) {
            const uint32_t m = (uint32_t)(idx / quads), n = (uint32_t)(idx % quads) * 4;
            const float *src = partial + (size_t)m * N + n;
            float4 t[8];
#pragma unroll
            for (int sidx = 0; sidx < 8; ++sidx)                         // every split in flight before the first add
                t[sidx] = (uint32_t)sidx < splits ? __ldcg(reinterpret_cast<const float4 *>(src + sidx * plane))
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 acc = t[0];
#pragma unroll
            for (int sidx = 1; sidx < 8; ++sidx) { acc.x += t[sidx].x; acc.y += t[sidx].y; acc.z += t[sidx].z; acc.w += t[sidx].w; }
            if (bias) {
                acc.x += load_bf16(bias + n); acc.y += load_bf16(bias + n + 1);
                acc.z += load_bf16(bias + n + 2); acc.w += load_bf16(bias + n + 3);
            }
            const uint32_t lo = float_to_bf16_bits(acc.x) | ((uint32_t)float_to_bf16_bits(acc.y) << 16);
            const uint32_t hi = float_to_bf16_bits(acc.z) | ((uint32_t)float_to_bf16_bits(acc.w) << 16);
            *reinterpret_cast<uint2 *>(y + (size_t)m * ldy + n) = make_uint2(lo, hi);
        }
    } else {
        for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < plane; idx += (size_t)gridDim.x * blockDim.x) {
            const uint32_t m = (uint32_t)(idx / N), n = (uint32_t)(idx % N);
            float acc = 0.f;
            for (uint32_t sidx = 0; sidx < splits; ++sidx) acc += __ldcg(partial + sidx * plane + idx);
            if (bias) acc += load_bf16(bias + n);
            y[(size_t)m * ldy + n] = float_to_bf16_bits(acc);
        }
    }
}

// ------------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Split-K factor by a small cost model (microseconds, measured on B200 at tile height 128): a CTA needs about
// 5.6 per 128x128 tile it decodes plus 14 of set-up, pipeline fill and accumulator read-out; CTAs beyond one
// per SM run in further waves; partial sums cost one pass over splits x M x N floats at about 3.4 TB/s.
uint32_t gemm_splits(uint32_t M, uint32_t N, uint32_t tiles_k) {
    const uint32_t ctas = ((N + kBN - 1) / kBN) * ((M + kBM * kMChunks - 1) / (kBM * kMChunks));
    const uint32_t P = (uint32_t)sm_count();
    uint32_t best_s = 1;
    double best = 1e30;
    for (uint32_t s = 1; s <= 8 && s <= tiles_k; ++s) {
        const uint32_t per = (tiles_k + s - 1) / s, real_s = (tiles_k + per - 1) / per;
        if (real_s != s) continue;                                       // same partition as a smaller factor
        const uint32_t waves = (ctas * s + P - 1) / P;
        double cost = waves * (per * 5.6 + 14.0);
        if (s > 1) cost += (double)s * M * N * 4.0 / 3.4e6;
        if (cost < best) { best = cost; best_s = s; }
    }
    return best_s;
}

size_t gemm_workspace_bytes(uint32_t M, uint32_t N, uint32_t K, uint32_t th) {
    if (M <= 16 || th == 0) return 0;
    uint32_t s = gemm_splits(M, N, (K + th - 1) / th);
    return s > 1 ? (size_t)s * M * N * sizeof(float) : 0;
}

// Returns CI_OK when launched, 1 when the weight / activations do not qualify, < 0 on error.
int launch_linear_gemm(const LinArgs &a, uint32_t max_tile_len, size_t partial_capacity, uint32_t split_k,
                       cudaStream_t s) {
    const Geom &g = a.g;
    if (g.tw != 32 || g.th != kTileH || max_tile_len == 0) return 1;
    if ((reinterpret_cast<uintptr_t>(a.stream) & 15u) || (reinterpret_cast<uintptr_t>(a.mantissa) & 15u)) return 1;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || ((a.ldx * 2) & 15)) return 1;      // TMA: 16-byte base and pitch
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return 1;

    GemmArgs p;
    p.a = a;
    p.win_cap = ((max_tile_len * 64u + 15u) & ~15u) + 16u;
    int dev = 0, max_smem = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const uint32_t fixed = kOffStage + 1024;                             // + alignment slack
    const size_t smem = fixed + (size_t)kDecWarps * 2 * p.win_cap;
    if ((size_t)max_smem < smem) return 1;

    p.m_tiles = (a.M + kBM * kMChunks - 1) / (kBM * kMChunks);
    const uint32_t n_blocks = (g.N + kBN - 1) / kBN;
    uint32_t splits = split_k ? split_k : gemm_splits(a.M, g.N, g.tiles_k);
    if (splits > g.tiles_k) splits = g.tiles_k;
    if (splits > 8) splits = 8;                                       // the final reduction holds at most 8 partials
    while (splits > 1 && (size_t)splits * a.M * g.N * sizeof(float) > partial_capacity) --splits;
    p.tiles_per_split = (g.tiles_k + splits - 1) / splits;
    p.splits = (g.tiles_k + p.tiles_per_split - 1) / p.tiles_per_split;
    p.status = a.tickets + (kTicketBytes - 1);

    CUtensorMap map;
    const cuuint64_t dims[2] = {g.K, a.M};
    const cuuint64_t strides[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {kBK, kBM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(a.x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
        return CI_E_CUDA;
    }
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_linear_gemm, (size_t)max_smem)) return rc;
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_blocks, p.m_tiles, p.splits);
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cfg.attrs = pdl;
        cfg.numAttrs = 1;
        CI_CUDA(cudaLaunchKernelEx(&cfg, k_linear_gemm, p, map));
    }
    if (p.splits > 1) {
        const uint32_t vec = ((g.N & 3u) == 0 && (a.ldy & 3) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 7u) == 0) ? 1u : 0u;
        const size_t items = vec ? (size_t)a.M * (g.N / 4) : (size_t)a.M * g.N;
        size_t blocks = (items + 255) / 256;
        const size_t cap = (size_t)sm_count() * 16;
        if (blocks > cap) blocks = cap;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cfg.attrs = pdl;
        cfg.numAttrs = 1;
        CI_CUDA(cudaLaunchKernelEx(&cfg, k_splitk_reduce, (const float *)a.partial, p.splits, a.M, g.N, a.bias, a.y,
                                   a.ldy, vec));
    }
    return CI_OK;
}

}  // namespace ci
