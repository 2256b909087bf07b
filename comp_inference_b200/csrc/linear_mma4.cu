// Fused decode + linear for 32-wide tiles, register-direct tensor-core path (activation batches of
// up to 16 rows): y[M,N] = x[M,K] . W[K,N] with W decoded from its rANS streams inside the kernel.
// Replaces fused_rans_matmul_kernel_ilp2_splitk (comp_inference/linear_triton.py:317-552).
//
// Work unit: one warp decodes a pair of vertically adjacent tiles of one 32-column group = 128
// streams, four per lane.  Lane T (g = T / 4, q = T % 4) owns the four adjacent columns 4g .. 4g+3 of
// row segment q, the segments being the top / bottom halves of the upper and of the lower tile.  That
// is exactly the fragment ownership of mma.sync m16n8k16 -- the four threads that share g hold
// different k -- once the k index of the instruction is read as "segment q, rows r..r+3": four
// consecutive symbols of a stream are one packed pair of registers, the matching activations
// x[m][those rows] are one 8-byte load per activation row.  The weights are the A operand (two columns
// of the lane = mma rows g and g + 8, two mma per four rows) and activation row g the B operand; an
// instantiation for 9..16 activation rows issues a second pair of mma for row g + 8.  No shared-memory
// transpose, no ldmatrix.
//
// Measured on a B200 this kernel is bound neither by HBM (10 %) nor by one on-chip unit alone: issue
// slots are 41 % busy with about 20 integer-heavy instructions per decoded symbol on half-rate pipes,
// the shared-memory / L1 pipeline 48 %, and every mma.sync costs as much as several ordinary
// instructions.  So the data movement around the decode step is arranged to cost as few instructions,
// wavefronts and tensor instructions as possible:
//  * compressed bytes: the two tiles' byte blocks ([row][64 B] each) are copied by cp.async into one
//    window of 128-byte rows (upper tile in bytes 0..63, lower tile in 64..127).  The four streams of a
//    lane are the four bytes of one word column, so every lane reads its own bank whatever row each of
//    its cursors is on;
//  * sign+mantissa bytes never enter shared memory: one 32-bit global load per row covers the lane's
//    four columns (a warp reads four full 32-byte sectors), issued one 4-row group ahead of its use;
//    the unit's two 4 KB blocks are pulled into L2 when the unit's copies are queued;
//  * initial states arrive by bulk copy with the rest of the unit (no global load at a unit's start).
// Units are double buffered per warp; byte ranges of the next units are loaded one unit ahead by all
// lanes in parallel.
//
// Scheduling: warp-level stream-K as in linear_mma.cu (units ordered by column group then tile-row
// pair, equal contiguous runs per warp, fp32 partials + ticket, fixed summation order).
#include "linear.cuh"
#include "ptx.cuh"

namespace ci {

constexpr uint32_t kBar4Bytes = 256;         // up to 16 warps x 2 stages x 8 B
constexpr uint32_t kMma4Warps = 14;          // 448 threads x 128 registers; an instantiation for 12 warps with 158
                                             // registers executes 7 % fewer instructions but was slower (fewer warps)

struct Mma4Args {
    LinArgs a;
    uint32_t cap_rows;     // rows of a byte window (>= every tile_max_len)
    uint32_t stage_bytes;  // window + 128 initial states
    uint32_t per_warp;     // units per warp
    uint32_t total;        // units in the matrix
    uint32_t pairs_k;      // tile-row pairs = ceil(tiles_k / 2)
    uint32_t y_vec;        // outputs can be written as 16-byte rows of eight
    uint32_t *status;      // set non-zero if a wait ran out
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// The mbarrier gets one arrival when all cp.async issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Packed bf16 pair (rows k, k+1) of column c of the lane from two table entries and the two
// 4-column sign+mantissa words of those rows.
template <int C>
__device__ __forceinline__ uint32_t weight_pair4(uint32_t e_lo, uint32_t e_hi, uint32_t m_lo, uint32_t m_hi) {
    // Bits 8..23 of each entry side by side: the symbols sit at bits 4..11 / 20..27, three below their
    // place in a bf16 pair; whatever else the shift drags along is masked out by the bit-select.
    const uint32_t ee = __byte_perm(e_lo, e_hi, 0x6521) << 3;
    const uint32_t vv = __byte_perm(m_lo, m_hi, 0x4400 + 0x1111 * C);
    return (ee & 0x7F807F80u) | (vv & 0x807F807Fu);
}

__device__ __forceinline__ void prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *src) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(src));
    return v;
}

// Renormalisation of a lane's four streams.  The first byte (about one symbol in three needs it) is merged
// under a predicate; a second byte is needed only after a symbol of frequency below 16, so the whole
// warp tests for it with one vote and skips those instructions otherwise.
__device__ __forceinline__ void renorm4(uint32_t &s0, uint32_t &s1, uint32_t &s2, uint32_t &s3, uint32_t &p0, uint32_t &p1,
                                        uint32_t &p2, uint32_t &p3, uint32_t y0, uint32_t y1, uint32_t y2, uint32_t y3) {
    const uint32_t lowest = min(min(s0, s1), min(s2, s3));
    renorm_first<128>(s0, p0, y0);
    renorm_first<128>(s1, p1, y1);
    renorm_first<128>(s2, p2, y2);
    renorm_first<128>(s3, p3, y3);
    if (__any_sync(kFull, lowest < 256u)) {
        renorm_fast<128>(s0, p0);
        renorm_fast<128>(s1, p1);
        renorm_fast<128>(s2, p2);
        renorm_fast<128>(s3, p3);
    }
}

// Four symbols of each of the lane's streams -> four packed weight pairs per column -> tensor core.
// m = sign+mantissa words of the four rows, xf = the activations of those rows.
// The weights are the A operand -- columns c and c + 1 of the lane are mma rows g and g + 8, so one mma takes
// two columns -- and activation row g is the B operand (xf[0], xf[1]); with more than 8 activation rows (HI)
// a second pair of mma takes activation row g + 8 (xf[2], xf[3]).  Compared with the weights as the B
// operand (one mma per column) this halves the mma count and the accumulators for up to 8 rows and needs
// no interleaving of the activation registers.
template <bool HI>
__device__ __forceinline__ void group4(float (&acc)[4][4], uint32_t &s0, uint32_t &s1, uint32_t &s2, uint32_t &s3,
                                       uint32_t &p0, uint32_t &p1, uint32_t &p2, uint32_t &p3, uint32_t lut_s,
                                       const uint32_t (&m)[4], const uint32_t (&xf)[4]) {
    uint32_t b[4][2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {                               // two rows -> one packed pair per column
        uint32_t y0 = lds_u8(p0), y1 = lds_u8(p1), y2 = lds_u8(p2), y3 = lds_u8(p3);
        const uint32_t e0 = decode_aligned(s0, lut_s);
        const uint32_t e1 = decode_aligned(s1, lut_s);
        const uint32_t e2 = decode_aligned(s2, lut_s);
        const uint32_t e3 = decode_aligned(s3, lut_s);
        renorm4(s0, s1, s2, s3, p0, p1, p2, p3, y0, y1, y2, y3);
        y0 = lds_u8(p0);
        y1 = lds_u8(p1);
        y2 = lds_u8(p2);
        y3 = lds_u8(p3);
        const uint32_t f0 = decode_aligned(s0, lut_s);
        const uint32_t f1 = decode_aligned(s1, lut_s);
        const uint32_t f2 = decode_aligned(s2, lut_s);
        const uint32_t f3 = decode_aligned(s3, lut_s);
        renorm4(s0, s1, s2, s3, p0, p1, p2, p3, y0, y1, y2, y3);
        b[0][h] = weight_pair4<0>(e0, f0, m[2 * h], m[2 * h + 1]);
        b[1][h] = weight_pair4<1>(e1, f1, m[2 * h], m[2 * h + 1]);
        b[2][h] = weight_pair4<2>(e2, f2, m[2 * h], m[2 * h + 1]);
        b[3][h] = weight_pair4<3>(e3, f3, m[2 * h], m[2 * h + 1]);
    }
    const uint32_t w01[4] = {b[0][0], b[1][0], b[0][1], b[1][1]};
    const uint32_t w23[4] = {b[2][0], b[3][0], b[2][1], b[3][1]};
    mma_bf16(acc[0], w01, xf[0], xf[1]);
    mma_bf16(acc[1], w23, xf[0], xf[1]);
    if constexpr (HI) {
        mma_bf16(acc[2], w01, xf[2], xf[3]);
        mma_bf16(acc[3], w23, xf[2], xf[3]);
    }
}

// RAGGED: K is not a whole number of tile pairs, so the last unit of a column group lacks its lower tile or ends
// inside a tile (an instantiation of its own: the common case carries none of the bookkeeping in its registers).
// Every lane still runs the full warp-wide loop.  A lane whose segment has n_my < n_groups 4-row groups reads
// zeros instead of activations from group n_my on, and -- so that what it multiplies by those zeros stays a
// finite number -- starts its stream over whenever it has used it up (a lane without a segment decodes the top
// half of the upper tile, which always exists).  Its products are exact zeros.
__device__ __align__(16) uint16_t g_zero_activations[256];     // 64 per unit are read, 8 more are prefetched
template <bool HI, bool RAGGED>
__global__ void __launch_bounds__(kMma4Warps * 32, 1) k_linear_mma4(const __grid_constant__ Mma4Args p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const LinArgs &a = p.a;
    const Geom &g = a.g;
    const uint32_t W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t smem_s = smem_u32(smem);
    // The table sits on a 16 KB boundary of the shared window, so that an entry's address is
    // (state << 2 & 0x3FFC) | base: one shift and one three-input logic operation, no addition.
    const uint32_t lut_s = (smem_s + kLutBytes - 1) & ~(kLutBytes - 1);
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem + (lut_s - smem_s));
    const uint32_t wbase_s = lut_s + kLutBytes + kBar4Bytes + warp * 2 * p.stage_bytes;
    const uint32_t bar_base = lut_s + kLutBytes + warp * 16;
    const uint32_t seg_bytes = g.th * 16;                       // half a tile of sign+mantissa bytes
    const uint32_t st_off = p.cap_rows * 128;

    const uint32_t gq = lane >> 2, q = lane & 3;                // column quad and row segment of this lane
    const uint32_t tsel = q >> 1, hsel = q & 1;                 // upper / lower tile, top / bottom half

    const uint32_t gw = blockIdx.x * W + warp;                  // this warp's rank in the grid
    const uint32_t lo = gw * p.per_warp;
    const uint32_t hi = min(lo + p.per_warp, p.total);

    // Byte ranges of this warp's units, 32 at a time: lane j holds unit dbase + j.
    uint32_t d_off0 = 0, d_ml0 = 0, d_off1 = 0, d_ml1 = 0, dbase = lo;
    auto load_desc = [&]() {
        const uint32_t u = dbase + lane;
        if (u >= hi) return;
        const uint32_t grp = u / p.pairs_k, pk = u - grp * p.pairs_k;
        const uint32_t t0 = (2 * pk) * g.tiles_n + grp;
        d_off0 = __ldg(a.tile_offsets + t0);
        d_ml0 = __ldg(a.tile_max_lens + t0);
        d_off1 = 0;
        d_ml1 = 0;
        if (2 * pk + 1 < g.tiles_k) {
            d_off1 = __ldg(a.tile_offsets + t0 + g.tiles_n);
            d_ml1 = __ldg(a.tile_max_lens + t0 + g.tiles_n);
        }
    };

    // Starts every copy of unit u into `stage` (whole warp).
    auto issue = [&](uint32_t u, uint32_t stage, uint32_t off0, uint32_t ml0, uint32_t off1, uint32_t ml1) {
        const uint32_t grp = u / p.pairs_k, pk = u - grp * p.pairs_k;
        const uint32_t t0 = (2 * pk) * g.tiles_n + grp;
        const bool two = 2 * pk + 1 < g.tiles_k;
        const uint32_t bar = bar_base + stage * 8;
        const uint32_t dst = wbase_s + stage * p.stage_bytes;
        if (ml0 > p.cap_rows || ml1 > p.cap_rows) {             // metadata disagrees with the declared maximum
            if (lane == 0) atomicExch(p.status, 2u);
            ml0 = ml1 = 0;
        }
        if (lane == 0) {
            fence_async_proxy();
            mbar_expect_tx(bar, two ? 512u : 256u);
            bulk_load(dst + st_off, a.states + (size_t)t0 * 64, 256, bar);
            if (two) bulk_load(dst + st_off + 256, a.states + ((size_t)t0 + g.tiles_n) * 64, 256, bar);
            prefetch_l2(a.mantissa + (size_t)t0 * (2 * seg_bytes), 2 * seg_bytes);
            if (two) prefetch_l2(a.mantissa + ((size_t)t0 + g.tiles_n) * (2 * seg_bytes), 2 * seg_bytes);
        }
        // byte blocks: 16-byte pieces, piece i of a tile = (row i / 4, quarter i % 4)
        const uint8_t *s0 = a.stream + off0, *s1 = a.stream + off1;
        for (uint32_t i = lane; i < ml0 * 4; i += 32) cp_async16(dst + (i >> 2) * 128 + (i & 3) * 16, s0 + i * 16);
        for (uint32_t i = lane; i < ml1 * 4; i += 32) cp_async16(dst + (i >> 2) * 128 + 64 + (i & 3) * 16, s1 + i * 16);
        cp_async_arrive(bar);
    };

    if (lane == 0) {
        mbar_init(bar_base, 33);                                // 32 cp.async arrivals + the bulk copies' expect_tx
        mbar_init(bar_base + 8, 33);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    load_desc();
    uint32_t nx_off0 = __shfl_sync(kFull, d_off0, 0), nx_ml0 = __shfl_sync(kFull, d_ml0, 0);
    uint32_t nx_off1 = __shfl_sync(kFull, d_off1, 0), nx_ml1 = __shfl_sync(kFull, d_ml1, 0);
    if (lo < hi) issue(lo, 0, nx_off0, nx_ml0, nx_off1, nx_ml1);
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    // Everything above touches only the weight, which no kernel writes.  When this launch was allowed to
    // start before its predecessor in the stream has finished (programmatic dependent launch), wait here
    // for it -- activations, workspace and output may be its products -- and let the next launch start
    // its own preamble while this grid works.  Both are no-ops in an ordinary launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lo >= hi) return;                                       // no CTA-wide synchronisation below this line
    const bool fused_ar = a.ar.world > 1;                       // row-parallel: exchange the sums with the peers here
    const uint32_t ar_seq = fused_ar ? fuse_seq(a.ar) : 0u;

    float acc[4][4];
    auto zero_acc = [&]() {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    };

    // Writes the finished (or partial) sums of column group grp.  After a lane exchange (below) a lane
    // works on rows gq and gq + 8 of the activation batch, columns 8q .. 8q+7 of the group.
    auto flush = [&](uint32_t grp) {
        const uint32_t first_w = (grp * p.pairs_k) / p.per_warp;
        const uint32_t last_w = ((grp + 1) * p.pairs_k - 1) / p.per_warp;
        const uint32_t count = last_w - first_w + 1;
        const uint32_t n0 = grp * 32 + 8 * q;
        auto store_row = [&](uint32_t m, const float (&v)[8]) {
            if (m >= a.M) return;
            uint16_t h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float f = v[j];
                if (a.bias && n0 + j < g.N) f += load_bf16(a.bias + n0 + j);
                h[j] = float_to_bf16_bits(f);
            }
            uint16_t *dst = a.y + (size_t)m * a.ldy + n0;
            if (p.y_vec && n0 + 8 <= g.N) {
                uint4 o;
                o.x = h[0] | ((uint32_t)h[1] << 16);
                o.y = h[2] | ((uint32_t)h[3] << 16);
                o.z = h[4] | ((uint32_t)h[5] << 16);
                o.w = h[6] | ((uint32_t)h[7] << 16);
                *reinterpret_cast<uint4 *>(dst) = o;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (n0 + j < g.N) dst[j] = h[j];
            }
        };
        float v0[8], v1[8];
        {
            // The D fragments hold columns 4 gq .. 4 gq + 3 of activation rows 2q and 2q + 1 (acc[c / 2], and
            // acc[2 + c / 2] for rows 8 + 2q, 9 + 2q; element 2 (c % 2) + row parity).  Everything below works on
            // "row gq (v0) and gq + 8 (v1), columns 8q .. 8q + 7": fetch those from lanes (2q, gq / 2) and
            // (2q + 1, gq / 2).
            const uint32_t srcA = (2 * q) * 4 + (gq >> 1), srcB = srcA + 4;
            const bool odd = gq & 1;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float e0 = acc[c >> 1][2 * (c & 1)], e1 = acc[c >> 1][2 * (c & 1) + 1];
                const float a0 = __shfl_sync(kFull, e0, srcA), a1 = __shfl_sync(kFull, e1, srcA);
                const float b0 = __shfl_sync(kFull, e0, srcB), b1 = __shfl_sync(kFull, e1, srcB);
                v0[c] = odd ? a1 : a0;
                v0[4 + c] = odd ? b1 : b0;
                v1[c] = v1[4 + c] = 0.f;
                if constexpr (HI) {
                    const float h0 = acc[2 + (c >> 1)][2 * (c & 1)], h1 = acc[2 + (c >> 1)][2 * (c & 1) + 1];
                    const float c0 = __shfl_sync(kFull, h0, srcA), c1 = __shfl_sync(kFull, h1, srcA);
                    const float d0 = __shfl_sync(kFull, h0, srcB), d1 = __shfl_sync(kFull, h1, srcB);
                    v1[c] = odd ? c1 : c0;
                    v1[4 + c] = odd ? d1 : d0;
                }
            }
        }
        if (count == 1) {
            if (fused_ar) {                                     // M <= 2: rows 0 / 1 live in the lanes with gq < M
                if (gq < a.M && n0 < g.N) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (n0 + 2 * j >= g.N) break;           // N need only be even: the last quad may be short
                        const float2 r = fuse_exchange_pair(a.ar, ar_seq, (gq * g.N + n0) / 2 + j, v0[2 * j], v0[2 * j + 1]);
                        v0[2 * j] = r.x;
                        v0[2 * j + 1] = r.y;
                    }
                }
                __syncwarp();
                if (lane == 0) fuse_group_done(a.ar, ar_seq, g.groups);
            }
            store_row(gq, v0);
            store_row(gq + 8, v1);
            return;
        }
        // Slot gw + grp is unique: along the unit order both the warp rank and the group only grow.
        float *mine = a.partial + (size_t)(gw + grp) * a.M * 32 + 8 * q;
        if (gq < a.M) {
            *reinterpret_cast<float4 *>(mine + gq * 32) = make_float4(v0[0], v0[1], v0[2], v0[3]);
            *reinterpret_cast<float4 *>(mine + gq * 32 + 4) = make_float4(v0[4], v0[5], v0[6], v0[7]);
        }
        if (gq + 8 < a.M) {
            *reinterpret_cast<float4 *>(mine + (gq + 8) * 32) = make_float4(v1[0], v1[1], v1[2], v1[3]);
            *reinterpret_cast<float4 *>(mine + (gq + 8) * 32 + 4) = make_float4(v1[4], v1[5], v1[6], v1[7]);
        }
        // One acquire-release ticket instead of fence + relaxed ticket + fence: the warp barrier orders the
        // lanes' partial stores before lane 0's release, and the last arriver's acquire before the lanes' loads.
        __syncwarp();
        uint32_t last = 0;
        if (lane == 0) {
            uint32_t seen;
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(seen) : "l"(a.tickets + grp) : "memory");
            last = seen == count - 1;
        }
        last = __shfl_sync(kFull, last, 0);
        __syncwarp();                                           // lane 0's acquire is ordered before every lane's loads
        if (!last) return;
        if (a.M <= 2) {
            // One or two activation rows: lane = column, up to sixteen partials of both rows in flight at
            // once, so the reduction costs one L2 round trip.  Fixed order: partial first_w, first_w + 1, ...
            float s0 = 0.f, s1 = 0.f;
            const bool two = a.M == 2;
            for (uint32_t w0 = first_w; w0 <= last_w; w0 += 16) {
                float t0[16], t1[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const bool in = w0 + i <= last_w;
                    const float *src = a.partial + (size_t)(w0 + i + grp) * a.M * 32 + lane;
                    t0[i] = in ? __ldcg(src) : 0.f;
                    t1[i] = (in && two) ? __ldcg(src + 32) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    s0 += t0[i];
                    s1 += t1[i];
                }
            }
            const uint32_t n = grp * 32 + lane;
            if (fused_ar) {                                     // even lanes exchange (n, n + 1) of both rows
                const float o0 = __shfl_down_sync(kFull, s0, 1), o1 = __shfl_down_sync(kFull, s1, 1);
                float2 r0 = make_float2(s0, o0), r1 = make_float2(s1, o1);
                if ((lane & 1) == 0 && n < g.N) {
                    r0 = fuse_exchange_pair(a.ar, ar_seq, n / 2, s0, o0);
                    if (two) r1 = fuse_exchange_pair(a.ar, ar_seq, (g.N + n) / 2, s1, o1);
                }
                const float u0 = __shfl_up_sync(kFull, r0.y, 1), u1 = __shfl_up_sync(kFull, r1.y, 1);
                s0 = (lane & 1) ? u0 : r0.x;
                s1 = (lane & 1) ? u1 : r1.x;
                if (lane == 0) fuse_group_done(a.ar, ar_seq, g.groups);
            }
            if (n < g.N) {
                const float b = a.bias ? load_bf16(a.bias + n) : 0.f;
                a.y[n] = float_to_bf16_bits(s0 + b);
                if (two) a.y[(size_t)a.ldy + n] = float_to_bf16_bits(s1 + b);
            }
        } else {
            // Four partials in flight at a time, each two rows of eight floats per lane.
            const bool has0 = gq < a.M, has1 = gq + 8 < a.M;
#pragma unroll
            for (int j = 0; j < 8; ++j) v0[j] = v1[j] = 0.f;
            const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t w0 = first_w; w0 <= last_w; w0 += 4) {
                float4 t[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const bool in = w0 + i <= last_w;
                    const float *src = a.partial + (size_t)(w0 + i + grp) * a.M * 32 + 8 * q;
                    t[i][0] = (in && has0) ? __ldcg(reinterpret_cast<const float4 *>(src + gq * 32)) : z;
                    t[i][1] = (in && has0) ? __ldcg(reinterpret_cast<const float4 *>(src + gq * 32 + 4)) : z;
                    t[i][2] = (in && has1) ? __ldcg(reinterpret_cast<const float4 *>(src + (gq + 8) * 32)) : z;
                    t[i][3] = (in && has1) ? __ldcg(reinterpret_cast<const float4 *>(src + (gq + 8) * 32 + 4)) : z;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v0[0] += t[i][0].x; v0[1] += t[i][0].y; v0[2] += t[i][0].z; v0[3] += t[i][0].w;
                    v0[4] += t[i][1].x; v0[5] += t[i][1].y; v0[6] += t[i][1].z; v0[7] += t[i][1].w;
                    v1[0] += t[i][2].x; v1[1] += t[i][2].y; v1[2] += t[i][2].z; v1[3] += t[i][2].w;
                    v1[4] += t[i][3].x; v1[5] += t[i][3].y; v1[6] += t[i][3].z; v1[7] += t[i][3].w;
                }
            }
            store_row(gq, v0);
            store_row(gq + 8, v1);
        }
        __syncwarp();
        if (lane == 0) a.tickets[grp] = 0;                      // ready for the next call
    };

    // Activations of rows gq and gq + 8 as the A fragment: columns k .. k+3 are (a0, a2) resp. (a1, a3).
    // Rows beyond the batch read the last real row instead: their products land in output rows that are
    // never stored, so no guard (and no branch) is needed in the loop.
    const uint32_t m_last = a.M - 1;
    const uint16_t *x0 = a.x + (size_t)min(gq, m_last) * a.ldx;
    const uint16_t *x1 = a.x + (size_t)min(gq + 8, m_last) * a.ldx;

    uint32_t parity0 = 0, parity1 = 0, stage = 0;
    uint32_t cur_grp = lo / p.pairs_k;
    zero_acc();
    const uint32_t n_groups = g.half / 4;                       // 4-symbol groups per stream (even)
    const uint32_t ragged_pk = (g.K % (2 * g.th)) ? p.pairs_k - 1 : 0xFFFFFFFFu;   // the unit index with rows beyond K

    uint32_t s0, s1, s2, s3, pos0, pos1, pos2, pos3;
    // Four symbols of each of the lane's streams -> four B fragments -> four mma.  m = sign+mantissa words
    // of the four rows, xf = the activations of those rows.
    // Operands of one group straight from global memory: four 32-byte-strided words of the sign+mantissa
    // plane and two 8-byte quads of activations.
    auto fetch = [&](const uint8_t *mp, const uint16_t *xp0, const uint16_t *xp1, uint32_t (&m)[4], uint32_t (&xf)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) m[i] = ldg_stream_u32(mp + i * 32);
        const uint2 v0 = __ldg(reinterpret_cast<const uint2 *>(xp0));
        xf[0] = v0.x;
        xf[1] = v0.y;
        xf[2] = xf[3] = 0;
        if constexpr (HI) {
            const uint2 v1 = __ldg(reinterpret_cast<const uint2 *>(xp1));
            xf[2] = v1.x;
            xf[3] = v1.y;
        }
    };

    for (uint32_t t = lo; t < hi; ++t) {
        const uint32_t grp = t / p.pairs_k, pk = t - grp * p.pairs_k;
        if (grp != cur_grp) {
            flush(cur_grp);
            zero_acc();
            cur_grp = grp;
        }
        // Groups of this lane's segment that exist (n_my) and of the stream it decodes (len); see the kernel's header.
        uint32_t n_my = n_groups, len = n_groups;
        uint32_t tsel_d = tsel, hsel_d = hsel;                  // the segment whose stream and bytes this lane decodes
        if (RAGGED && pk == ragged_pk) {
            const uint32_t r0 = (2 * pk + tsel) * g.th;
            const uint32_t rows_t = r0 < g.K ? min(g.th, g.K - r0) : 0u;
            const uint32_t seg = rows_t > hsel * g.half ? min(g.half, rows_t - hsel * g.half) : 0u;
            n_my = len = seg >> 2;
            if (seg == 0) {                                     // nothing of its own: the upper tile's top half stands in
                tsel_d = hsel_d = 0;
                len = min(g.half, g.K - 2 * pk * g.th) >> 2;
            }
        }
        // (row 0 of this lane's segment, its four columns) of the sign+mantissa plane, and its activations
        const uint32_t krow = (2 * pk + tsel) * g.th + hsel * g.half;
        const uint8_t *mp = a.mantissa + ((size_t)(2 * pk + tsel_d) * g.tiles_n + grp) * (2 * seg_bytes) +
                            hsel_d * seg_bytes + gq * 4;
        const uint16_t *xp0 = x0 + krow + 0, *xp1 = x1 + krow;
        if (RAGGED && n_my == 0) xp0 = xp1 = g_zero_activations;
        uint32_t mA[4], xA[4], mB[4], xB[4];
        fetch(mp, xp0, xp1, mA, xA);                            // in flight while the copies are awaited

        const uint32_t ml = (RAGGED ? tsel_d : tsel) ? nx_ml1 : nx_ml0;
        __syncwarp();                                           // every lane is done with the other stage
        if (t + 1 < hi) {
            if (t + 1 - dbase == 32) {
                dbase = t + 1;
                load_desc();
            }
            const uint32_t j = t + 1 - dbase;
            nx_off0 = __shfl_sync(kFull, d_off0, j);
            nx_ml0 = __shfl_sync(kFull, d_ml0, j);
            nx_off1 = __shfl_sync(kFull, d_off1, j);
            nx_ml1 = __shfl_sync(kFull, d_ml1, j);
            issue(t + 1, stage ^ 1, nx_off0, nx_ml0, nx_off1, nx_ml1);
        }

        // ---- this lane's four streams --------------------------------------
        const uint32_t win_s = wbase_s + stage * p.stage_bytes;
        const uint32_t st_s = win_s + st_off + (RAGGED ? tsel_d : tsel) * 256 + ((RAGGED ? hsel_d : hsel) * 32 + gq * 4) * 4;
        pos0 = win_s + (RAGGED ? tsel_d : tsel) * 64 + (RAGGED ? hsel_d : hsel) * 32 + gq * 4;
        if (ml <= p.cap_rows) pos0 += (ml - 1) * 128;           // last byte row; an empty tile starts one row below
        const uint32_t pos_first = pos0;
        pos1 = pos0 + 1;
        pos2 = pos0 + 2;
        pos3 = pos0 + 3;

        // ---- wait for the bytes (bounded) -------------------------------------
        {
            const uint32_t bar = bar_base + stage * 8, par = stage ? parity1 : parity0;
            uint32_t ok = 0;
            if (lane == 0)
                for (uint32_t it = 0; it < kWaitPolls && !ok; ++it) ok = mbar_try_wait(bar, par);
            ok = __shfl_sync(kFull, ok, 0);
            if (stage) parity1 ^= 1; else parity0 ^= 1;
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 1u);
                stage ^= 1;
                continue;
            }
            (void)mbar_try_wait(bar, par);                      // each lane observes the completed phase itself
        }
        s0 = lds_u32(st_s);
        s1 = lds_u32(st_s + 4);
        s2 = lds_u32(st_s + 8);
        s3 = lds_u32(st_s + 12);

        uint32_t left = len;                                    // groups until this lane's stream is used up (RAGGED)
#pragma unroll 1
        for (uint32_t gi = 0; gi < n_groups; gi += 2) {         // operands are fetched one group ahead
            fetch(mp + 128, xp0 + 4, xp1 + 4, mB, xB);
            group4<HI>(acc, s0, s1, s2, s3, pos0, pos1, pos2, pos3, lut_s, mA, xA);
            mp += 256;
            xp0 += 8;
            xp1 += 8;
            if constexpr (RAGGED) {
                if (gi + 2 == n_my) xp0 = xp1 = g_zero_activations;   // rows beyond K from the next group on
            }
            if (gi + 2 < n_groups) fetch(mp, xp0, xp1, mA, xA);
            group4<HI>(acc, s0, s1, s2, s3, pos0, pos1, pos2, pos3, lut_s, mB, xB);
            if constexpr (RAGGED) {
                left -= 2;
                if (left == 0) {                                // stream used up: start it over (its products meet zeros)
                    left = len;
                    s0 = lds_u32(st_s);
                    s1 = lds_u32(st_s + 4);
                    s2 = lds_u32(st_s + 8);
                    s3 = lds_u32(st_s + 12);
                    pos0 = pos_first;
                    pos1 = pos0 + 1;
                    pos2 = pos0 + 2;
                    pos3 = pos0 + 3;
                    mp -= len * 128;                            // and its sign+mantissa rows with it
                }
            }
        }
        stage ^= 1;
    }
    flush(cur_grp);
}

// ------------------------------------------------------------------------ host

int launch_linear_mma4(const LinArgs &a, uint32_t max_tile_len, cudaStream_t s) {
    const Geom &g = a.g;
    // 16-symbol-aligned streams; K a multiple of 8 (the loop decodes and multiplies two groups of four rows per
    // pass); the last pair of tile rows may lack its lower tile and either tile may be short
    if (g.tw != 32 || g.th % 16 != 0 || g.K % 8 != 0 || a.M > 16 || max_tile_len == 0) return 1;
    if ((reinterpret_cast<uintptr_t>(a.stream) & 15u) || (reinterpret_cast<uintptr_t>(a.mantissa) & 15u) ||
        (reinterpret_cast<uintptr_t>(a.states) & 15u))
        return 1;
    if ((reinterpret_cast<uintptr_t>(a.x) & 7u) || (a.ldx & 3)) return 1;      // activations are read as 8-byte quads
    // The kernel does not bounds-test stream cursors; a malformed stream can walk at most tile_h rows of
    // 128 bytes below its window, which must still be inside the CTA's shared memory.
    if (g.th * 128u > kLutBytes) return 1;

    int dev = 0, max_smem = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    Mma4Args p;
    p.a = a;
    p.cap_rows = max_tile_len;
    p.stage_bytes = (p.cap_rows * 128u + 512u + 127u) & ~127u;
    const uint32_t fixed = 2 * kLutBytes + kBar4Bytes;         // up to one table size is lost to the table's alignment
    const uint32_t warp_bytes = 2 * p.stage_bytes;
    if ((uint32_t)max_smem < fixed + 4 * warp_bytes) return 1;
    uint32_t w_max = ((uint32_t)max_smem - fixed) / warp_bytes;
    if (w_max > kMma4Warps) w_max = kMma4Warps;

    // Units per warp must be a whole number: pick the warp count whose grid wastes the least.
    const uint32_t P = (uint32_t)sm_count();
    p.pairs_k = (g.tiles_k + 1) / 2;
    p.total = g.groups * p.pairs_k;
    // A unit here is a serial chain twice as long as in the two-streams kernel (two tiles instead of one).
    // That pays once the multiprocessors are saturated (about eight warps each); a small matrix -- a
    // tensor-parallel shard, say -- is latency bound and finishes sooner with the shorter units
    // (measured cross-over: 4096 x 2048 at tile height 128).
#ifndef CI_MMA4_MIN_UNITS
#define CI_MMA4_MIN_UNITS 6
#endif
    if (p.total < P * CI_MMA4_MIN_UNITS) return 1;
    uint32_t best_w = w_max;
    double best = -1.0;
    for (uint32_t w = 4; w <= w_max; ++w) {
        uint64_t slots = (uint64_t)P * w, per = (p.total + slots - 1) / slots;
        double eff = (double)p.total / (double)(slots * per);
        if (w < 8) eff *= w / 8.0;                              // too few warps cannot hide the decode chain
        if (eff >= best) { best = eff; best_w = w; }
    }
    const uint64_t slots = (uint64_t)P * best_w;
    p.per_warp = (uint32_t)((p.total + slots - 1) / slots);
    const uint32_t warps_needed = (p.total + p.per_warp - 1) / p.per_warp;
    const uint32_t blocks = (warps_needed + best_w - 1) / best_w;
    p.y_vec = ((reinterpret_cast<uintptr_t>(a.y) & 15u) == 0 && (a.ldy & 7) == 0) ? 1u : 0u;
    p.status = a.tickets + (kTicketBytes - 1);
    if (a.dry_run) return CI_OK;                                // qualification only

    const bool ragged = g.K % (2 * g.th) != 0;
    void (*kernel)(Mma4Args) = a.M <= 8 ? (ragged ? k_linear_mma4<false, true> : k_linear_mma4<false, false>)
                                        : (ragged ? k_linear_mma4<true, true> : k_linear_mma4<true, false>);
    static SmemLimit lim[4] = {};
    if (int rc = ensure_smem_limit(lim[(a.M > 8) * 2 + ragged], (const void *)kernel, (size_t)max_smem)) return rc;
    // Programmatic dependent launch: the grid may be scheduled while the previous kernel of the stream
    // drains; the kernel itself waits for that kernel before it reads activations or touches the workspace.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(best_w * 32);
    cfg.dynamicSmemBytes = fixed + (size_t)best_w * warp_bytes;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CI_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return CI_OK;
}

}  // namespace ci
