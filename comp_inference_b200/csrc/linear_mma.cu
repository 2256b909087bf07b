// Fused decode + linear, staged tensor-core path (activation batches of up to 16
// rows per pass): y[M,N] = x[M,K] . W[K,N] with W decoded from its rANS streams
// inside the kernel.  Replaces fused_rans_matmul_kernel_ilp2_splitk
// (comp_inference/linear_triton.py:317-552).
//
// Work unit: one warp decodes one (tile row, 32-column group) = 64 streams, two
// per lane.  All bytes a unit needs -- the tile's compressed byte block and its
// raw sign+mantissa block -- are fetched by two bulk async copies
// (cp.async.bulk, completion on an mbarrier) into a per-warp double buffer, so the
// copy of unit t+1 overlaps the decode of unit t and no load latency sits on the
// decode chain.  Decoded weights are packed to bf16 in registers, transposed
// through a 1 KB swizzled shared-memory tile and fed to mma.sync m16n8k16 with
// the activations as the A operand; the dot products never touch CUDA-core FMAs,
// so 16 activation rows cost the same as one.
//
// Scheduling: warp-level stream-K.  The units of the whole matrix, ordered by
// column group then tile row, are cut into equal contiguous runs, one per warp of
// a persistent one-CTA-per-SM grid.  A warp whose run ends inside a column group
// writes an fp32 partial; the warp that draws the last ticket of the group adds
// the partials in a fixed order (deterministic) and writes bf16.
#include "linear.cuh"
#include "ptx.cuh"

namespace ci {

constexpr uint32_t kBarBytes = 256;          // 16 warps x 2 stages x 8 B
constexpr uint32_t kWtBytes = 2048;          // two swizzled 32x16 bf16 tiles (A-half, B-half)

struct MmaArgs {
    LinArgs a;
    uint32_t win_cap;      // bytes reserved per stage for the compressed byte block
    uint32_t stage_bytes;  // win_cap + mantissa block + the unit's 64 initial states
    uint32_t warp_bytes;   // 2 stages + transpose tiles
    uint32_t per_warp;     // units per warp
    uint32_t total;        // units in the matrix
    uint32_t x_aligned;    // activations can be read as 32-bit pairs
    uint32_t red_off;      // shared-memory reduction area (16-byte aligned offset from the window base):
    uint32_t red_slots;    //   [red_slots][2][32] fp32 partials, then [red_slots] tickets; 0 = none (more than two rows)
    uint32_t *status;      // set non-zero if a wait ran out
};

// Two activations x[r][k], x[r][k+1] as one register (zero beyond M rows / K columns).
__device__ __forceinline__ uint32_t load_x_pair(const MmaArgs &p, uint32_t r, uint32_t k) {
    const LinArgs &a = p.a;
    if (r >= a.M || k >= a.g.K) return 0u;
    const uint16_t *src = a.x + (size_t)r * a.ldx + k;
    if (p.x_aligned && k + 1 < a.g.K) return __ldg(reinterpret_cast<const uint32_t *>(src));
    uint32_t lo = __ldg(src), hi = (k + 1 < a.g.K) ? (uint32_t)__ldg(src + 1) : 0u;
    return lo | (hi << 16);
}
// A operand of mma m16n8k16 for activation columns [k0, k0+16), any position (guards on M and K).
__device__ __forceinline__ void load_x_frag(const MmaArgs &p, uint32_t k0, uint32_t (&x)[4]) {
    const uint32_t r = lane_id() >> 2, c = k0 + 2 * (lane_id() & 3);
    x[0] = load_x_pair(p, r, c);
    x[1] = load_x_pair(p, r + 8, c);
    x[2] = load_x_pair(p, r, c + 8);
    x[3] = load_x_pair(p, r + 8, c + 8);
}
// Same for a block known to lie inside the matrix and 4-byte aligned activations:
// x0 / x1 point at this lane's element of rows r and r+8 (null when the row does not exist).
__device__ __forceinline__ void load_x_frag_fast(const uint16_t *x0, const uint16_t *x1, uint32_t k0, uint32_t (&x)[4]) {
    x[0] = x0 ? __ldg(reinterpret_cast<const uint32_t *>(x0 + k0)) : 0u;
    x[1] = x1 ? __ldg(reinterpret_cast<const uint32_t *>(x1 + k0)) : 0u;
    x[2] = x0 ? __ldg(reinterpret_cast<const uint32_t *>(x0 + k0 + 8)) : 0u;
    x[3] = x1 ? __ldg(reinterpret_cast<const uint32_t *>(x1 + k0 + 8)) : 0u;
}

// Swizzled [32 columns][16 k] bf16 tile: 32-byte rows, the two 16-byte halves of a row swapped
// on every second group of four rows, which makes both the 16-byte row stores and the
// ldmatrix reads bank-conflict free.
__device__ __forceinline__ uint32_t wt_offset(uint32_t n, uint32_t khalf) {
    return n * 32 + ((khalf ^ ((n >> 2) & 1u)) << 4);
}

template <uint32_t TW>
__global__ void __launch_bounds__(512, 1) k_linear_mma(const __grid_constant__ MmaArgs p) {
    constexpr uint32_t WB = 2 * TW;                             // bytes per row of a tile's byte block
    constexpr uint32_t TPG = 32 / TW;                           // tiles per 32-column group
    extern __shared__ __align__(128) uint8_t smem[];
    const LinArgs &a = p.a;
    const Geom &g = a.g;
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem);
    const uint32_t W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t smem_s = smem_u32(smem);
    const uint32_t wbase_s = smem_s + kLutBytes + kBarBytes + warp * p.warp_bytes;
    const uint32_t wt_s = wbase_s + 2 * p.stage_bytes;
    const uint32_t bar_base = smem_s + kLutBytes + warp * 16;
    const uint32_t man_tile = g.th * TW;
    const uint32_t st_off = p.win_cap + g.th * 32u;             // initial states inside a stage

    const uint32_t gw = blockIdx.x * W + warp;                  // this warp's rank in the grid
    const uint32_t lo = gw * p.per_warp;
    const uint32_t hi = min(lo + p.per_warp, p.total);

    // Byte ranges of this warp's units, 32 at a time: lane j holds unit dbase + j.  All lanes load in
    // parallel, one unit ahead of the copy that needs them, so no metadata load sits on a unit's start.
    uint32_t d_begin = 0, d_end = 0, dbase = lo;
    auto load_desc = [&]() {
        const uint32_t u = dbase + lane;
        if (u >= hi) return;
        const uint32_t grp = u / g.tiles_k, tk = u - grp * g.tiles_k;
        const uint32_t tn0 = grp * TPG;
        const uint32_t nt = min(TPG, g.tiles_n - tn0);
        const uint32_t t0 = tk * g.tiles_n + tn0, tl = t0 + nt - 1;
        d_begin = __ldg(a.tile_offsets + t0);
        d_end = __ldg(a.tile_offsets + tl) + __ldg(a.tile_max_lens + tl) * WB;
    };

    // Queues the three bulk copies of unit t (byte block, sign+mantissa block, initial states) into `stage`.
    auto issue = [&](uint32_t t, uint32_t stage, uint32_t begin, uint32_t end) {
        if (lane != 0) return;
        const uint32_t grp = t / g.tiles_k, tk = t - grp * g.tiles_k;
        const uint32_t tn0 = grp * TPG;
        const uint32_t nt = min(TPG, g.tiles_n - tn0);
        const uint32_t t0 = tk * g.tiles_n + tn0;
        uint32_t wbytes = end - begin;
        if (wbytes > p.win_cap) {                               // metadata disagrees with the declared maximum
            atomicExch(p.status, 2u);
            wbytes = 0;
        }
        const uint32_t mbytes = nt * man_tile, sbytes = nt * WB * 4;
        const uint32_t bar = bar_base + stage * 8;
        const uint32_t dst = wbase_s + stage * p.stage_bytes;
        fence_async_proxy();
        mbar_expect_tx(bar, wbytes + mbytes + sbytes);
        if (wbytes) bulk_load(dst, a.stream + begin, wbytes, bar);
        bulk_load(dst + p.win_cap, a.mantissa + (size_t)t0 * man_tile, mbytes, bar);
        bulk_load(dst + st_off, a.states + (size_t)t0 * WB, sbytes, bar);
    };

    // The first copy is started before the table is loaded so both latencies overlap.
    if (lane == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    load_desc();
    uint32_t nx_begin = __shfl_sync(kFull, d_begin, 0), nx_end = __shfl_sync(kFull, d_end, 0);
    if (lo < hi) issue(lo, 0, nx_begin, nx_end);
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    // Column groups whose units all sit in this CTA are reduced through shared memory (tickets zeroed here)
    // instead of the workspace in global memory: no L2 round trip between the last decode step and the output.
    float *s_part = reinterpret_cast<float *>(smem + p.red_off);                 // 8-byte stores: keep it aligned
    uint32_t *s_ticket = reinterpret_cast<uint32_t *>(s_part + (size_t)p.red_slots * 64);
    for (uint32_t i = threadIdx.x; i < p.red_slots; i += blockDim.x) s_ticket[i] = 0;
    const uint32_t cta_w0 = blockIdx.x * W;                     // grid rank of this CTA's first warp
    const uint32_t cta_g0 = (cta_w0 * p.per_warp) / g.tiles_k;  // first column group this CTA touches
    __syncthreads();
    // Only the weight was read so far.  Under programmatic dependent launch the activations, the workspace
    // and the output may still belong to the previous kernel of the stream: wait for it, then let the next
    // launch start its preamble (no-ops in an ordinary launch).
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

    // Writes the finished (or partial) sums of column group grp.
    auto flush = [&](uint32_t grp) {
        const uint32_t first_w = (grp * g.tiles_k) / p.per_warp;
        const uint32_t last_w = ((grp + 1) * g.tiles_k - 1) / p.per_warp;
        const uint32_t count = last_w - first_w + 1;
        const uint32_t r0 = lane >> 2, c0 = 2 * (lane & 3);
        auto store_y = [&](uint32_t m, uint32_t n, float v0, float v1) {
            if (m >= a.M) return;
            if (n < g.N) {
                if (a.bias) v0 += load_bf16(a.bias + n);
                a.y[(size_t)m * a.ldy + n] = float_to_bf16_bits(v0);
            }
            if (n + 1 < g.N) {
                if (a.bias) v1 += load_bf16(a.bias + n + 1);
                a.y[(size_t)m * a.ldy + n + 1] = float_to_bf16_bits(v1);
            }
        };
        if (count == 1) {
            if (fused_ar) {                                     // M <= 2: rows 0 / 1 live in the lanes with r0 < M
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    const uint32_t n = grp * 32 + nb * 8 + c0;
                    if (r0 < a.M && n < g.N) {
                        const float2 r = fuse_exchange_pair(a.ar, ar_seq, (r0 * g.N + n) / 2, acc[nb][0], acc[nb][1]);
                        acc[nb][0] = r.x;
                        acc[nb][1] = r.y;
                    }
                }
                __syncwarp();
                if (lane == 0) fuse_group_done(a.ar, ar_seq, g.groups);
            }
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                store_y(r0, grp * 32 + nb * 8 + c0, acc[nb][0], acc[nb][1]);
                store_y(r0 + 8, grp * 32 + nb * 8 + c0, acc[nb][2], acc[nb][3]);
            }
            return;
        }
        // All warps of this group in this CTA (and at most two activation rows): shared-memory slots and ticket.
        const bool local = p.red_slots != 0 && first_w >= cta_w0 && last_w < cta_w0 + W;
        uint32_t last = 0;
        if (local) {
            // Slot (warp + group), both relative to this CTA: unique for the same reason as below.
            float *mine = s_part + (size_t)(warp + grp - cta_g0) * 64;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb)
                if (r0 < a.M) *reinterpret_cast<float2 *>(mine + r0 * 32 + nb * 8 + c0) = make_float2(acc[nb][0], acc[nb][1]);
            __syncwarp();
            if (lane == 0) {
                uint32_t seen;
                asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;"
                             : "=r"(seen) : "r"(smem_u32(s_ticket + (grp - cta_g0))) : "memory");
                last = seen == count - 1;
            }
        } else {
            // Slot gw + grp is unique: along the unit order both the warp rank and the group only grow.
            float *mine = a.partial + (size_t)(gw + grp) * a.M * 32;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                if (r0 < a.M) *reinterpret_cast<float2 *>(mine + r0 * 32 + nb * 8 + c0) = make_float2(acc[nb][0], acc[nb][1]);
                if (r0 + 8 < a.M)
                    *reinterpret_cast<float2 *>(mine + (r0 + 8) * 32 + nb * 8 + c0) = make_float2(acc[nb][2], acc[nb][3]);
            }
            // One acquire-release ticket: the warp barrier orders the lanes' partial stores before lane 0's
            // release, and the last arriver's acquire before the lanes' loads.
            __syncwarp();
            if (lane == 0) {
                uint32_t seen;
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(seen) : "l"(a.tickets + grp) : "memory");
                last = seen == count - 1;
            }
        }
        last = __shfl_sync(kFull, last, 0);
        __syncwarp();                                           // lane 0's acquire is ordered before every lane's loads
        if (!last) return;
        if (a.M <= 2) {
            // One or two activation rows: lane = column, up to sixteen partials of both rows in flight at
            // once, so the whole reduction of a 4096-row matrix costs one L2 round trip.  Same summation
            // order everywhere (partial first_w, first_w + 1, ...), so the result does not depend on the path.
            float s0 = 0.f, s1 = 0.f;
            const bool two = a.M == 2;
            if (local) {
                for (uint32_t w = first_w; w <= last_w; ++w) {
                    const float *src = s_part + (size_t)(w - cta_w0 + grp - cta_g0) * 64 + lane;
                    s0 += src[0];
                    if (two) s1 += src[32];
                }
            } else
            for (uint32_t w0 = first_w; w0 <= last_w; w0 += 16) {
                float t0[16], t1[16];
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    const bool in = w0 + q <= last_w;
                    const float *src = a.partial + (size_t)(w0 + q + grp) * a.M * 32 + lane;
                    t0[q] = in ? __ldcg(src) : 0.f;
                    t1[q] = (in && two) ? __ldcg(src + 32) : 0.f;
                }
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    s0 += t0[q];
                    s1 += t1[q];
                }
            }
            const uint32_t n = grp * 32 + lane;
            if (fused_ar) {                                     // even lanes exchange (n, n + 1) of both rows
                const float o0 = __shfl_down_sync(kFull, s0, 1), o1 = __shfl_down_sync(kFull, s1, 1);
                float2 r0x = make_float2(s0, o0), r1x = make_float2(s1, o1);
                if ((lane & 1) == 0 && n < g.N) {
                    r0x = fuse_exchange_pair(a.ar, ar_seq, n / 2, s0, o0);
                    if (two) r1x = fuse_exchange_pair(a.ar, ar_seq, (g.N + n) / 2, s1, o1);
                }
                const float u0 = __shfl_up_sync(kFull, r0x.y, 1), u1 = __shfl_up_sync(kFull, r1x.y, 1);
                s0 = (lane & 1) ? u0 : r0x.x;
                s1 = (lane & 1) ? u1 : r1x.x;
                if (lane == 0) fuse_group_done(a.ar, ar_seq, g.groups);
            }
            if (n < g.N) {
                const float b = a.bias ? load_bf16(a.bias + n) : 0.f;
                a.y[n] = float_to_bf16_bits(s0 + b);
                if (two) a.y[(size_t)a.ldy + n] = float_to_bf16_bits(s1 + b);
            }
            __syncwarp();
            if (lane == 0 && !local) a.tickets[grp] = 0;
            return;
        }
        // All loads of a batch of four partials are issued before any of them is used: a plain running
        // sum would wait one L2 round trip per partial (16 in a row for a 4096-row matrix).
        float sum[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; ++nb)
#pragma unroll
            for (int j = 0; j < 4; ++j) sum[nb][j] = 0.f;
        const bool has0 = r0 < a.M, has1 = r0 + 8 < a.M;
        for (uint32_t w0 = first_w; w0 <= last_w; w0 += 4) {
            float2 t[4][4][2];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const bool in = w0 + q <= last_w;
                const float *src = a.partial + (size_t)(w0 + q + grp) * a.M * 32 + c0;
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    t[q][nb][0] = (in && has0) ? __ldcg(reinterpret_cast<const float2 *>(src + r0 * 32 + nb * 8))
                                               : make_float2(0.f, 0.f);
                    t[q][nb][1] = (in && has1) ? __ldcg(reinterpret_cast<const float2 *>(src + (r0 + 8) * 32 + nb * 8))
                                               : make_float2(0.f, 0.f);
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)                         // fixed order: partial w0, w0+1, ...
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    sum[nb][0] += t[q][nb][0].x;
                    sum[nb][1] += t[q][nb][0].y;
                    sum[nb][2] += t[q][nb][1].x;
                    sum[nb][3] += t[q][nb][1].y;
                }
        }
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
            store_y(r0, grp * 32 + nb * 8 + c0, sum[nb][0], sum[nb][1]);
            store_y(r0 + 8, grp * 32 + nb * 8 + c0, sum[nb][2], sum[nb][3]);
        }
        __syncwarp();
        if (lane == 0) a.tickets[grp] = 0;                      // ready for the next call
    };

    // this lane's activation rows (fragment rows r and r+8), offset to its column pair
    const uint32_t xr = lane >> 2, xc = 2 * (lane & 3);
    const uint16_t *x0 = xr < a.M ? a.x + (size_t)xr * a.ldx + xc : nullptr;
    const uint16_t *x1 = xr + 8 < a.M ? a.x + (size_t)(xr + 8) * a.ldx + xc : nullptr;
    const uint32_t mat = lane >> 3, mr = lane & 7;
    const uint32_t ld_off0 = wt_offset((mat >> 1) * 8 + mr, mat & 1);          // n-blocks 0,1
    const uint32_t ld_off1 = wt_offset((2 + (mat >> 1)) * 8 + mr, mat & 1);    // n-blocks 2,3
    const uint32_t st_off0 = wt_offset(lane, 0), st_off1 = wt_offset(lane, 1);

    uint32_t parity0 = 0, parity1 = 0, stage = 0;
    uint32_t cur_grp = lo / g.tiles_k;
    zero_acc();

    for (uint32_t t = lo; t < hi; ++t) {
        const uint32_t grp = t / g.tiles_k, tk = t - grp * g.tiles_k;
        if (grp != cur_grp) {
            flush(cur_grp);
            zero_acc();
            cur_grp = grp;
        }
        const uint32_t cur_begin = nx_begin, cur_end = nx_end;
        if (t + 1 < hi) {
            if (t + 1 - dbase == 32) {
                dbase = t + 1;
                load_desc();
            }
            nx_begin = __shfl_sync(kFull, d_begin, t + 1 - dbase);
            nx_end = __shfl_sync(kFull, d_end, t + 1 - dbase);
            issue(t + 1, stage ^ 1, nx_begin, nx_end);
        }

        // ---- this lane's two streams ---------------------------------------
        LaneTile L;
        uint32_t t0;
        if (TW == 32) {                                         // one tile per unit: its range is the unit's
            L.n = grp * 32 + lane;
            L.live = L.n < g.N;
            L.lc = lane;
            L.t = t0 = tk * g.tiles_n + grp;
            L.off = cur_begin;
            L.ml = (cur_end - cur_begin) / WB;
        } else {
            L = lane_tile(a, tk, grp);
            t0 = __shfl_sync(kFull, L.t, 0);
        }
        const uint32_t win_s = wbase_s + stage * p.stage_bytes;
        uint32_t man_s = win_s + p.win_cap + (L.t - t0) * man_tile + L.lc;      // (row 0, this column)
        const uint32_t st_s = win_s + st_off + ((L.t - t0) * WB + L.lc) * 4;
        uint32_t posA = win_s + (L.off - cur_begin) + L.lc, posB;
        if (L.live) posA += (L.ml - 1) * WB;                    // last byte row; an empty tile starts one row below
        posB = posA + TW;
        const uint32_t row0 = tk * g.th, remain = g.K - row0;
        const uint32_t nA = min(remain, g.half), nB = remain > g.half ? min(remain - g.half, g.half) : 0;
        const uint32_t manB_off = g.half * TW;

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
        }

        uint32_t stA = kRansL, stB = kRansL;
        if (L.live) {
            stA = lds_u32(st_s);
            stB = lds_u32(st_s + TW * 4);
        }

        // ---- decode 16 rows of each half at a time, multiply on the tensor cores
        const uint32_t lut_s = smem_s;
        for (uint32_t i0 = 0; i0 < nA; i0 += 16) {
            uint32_t xa[4], xb[4];
            uint32_t pa[4], pb[4];                              // four packed row pairs at a time
            const bool full = i0 + 16 <= nB;
            if (full && p.x_aligned) {
                load_x_frag_fast(x0, x1, row0 + i0, xa);
                load_x_frag_fast(x0, x1, row0 + g.half + i0, xb);
            } else {
                load_x_frag(p, row0 + i0, xa);
                load_x_frag(p, row0 + g.half + i0, xb);
            }
            __syncwarp();                                       // the previous block's ldmatrix reads are done
            if (full) {                                         // 16 rows of both halves, no bounds tests
#pragma unroll 1
                for (uint32_t hb = 0; hb < 2; ++hb) {           // eight rows per pass keeps register use bounded
                    const uint32_t mA = man_s + (i0 + 8 * hb) * TW, mB = mA + manB_off;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t ma0 = lds_u8(mA + (2 * j) * TW), ma1 = lds_u8(mA + (2 * j + 1) * TW);
                        const uint32_t mb0 = lds_u8(mB + (2 * j) * TW), mb1 = lds_u8(mB + (2 * j + 1) * TW);
                        uint32_t ba = lds_u8(posA), bb = lds_u8(posB);
                        const uint32_t e0 = decode_fast(stA, lut_s);
                        const uint32_t f0 = decode_fast(stB, lut_s);
                        renorm_spec<WB>(stA, posA, ba);
                        renorm_spec<WB>(stB, posB, bb);
                        ba = lds_u8(posA);
                        bb = lds_u8(posB);
                        const uint32_t e1 = decode_fast(stA, lut_s);
                        const uint32_t f1 = decode_fast(stB, lut_s);
                        renorm_spec<WB>(stA, posA, ba);
                        renorm_spec<WB>(stB, posB, bb);
                        pa[j] = weight_pair(e0, e1, ma0, ma1);
                        pb[j] = weight_pair(f0, f1, mb0, mb1);
                    }
                    const uint32_t so = hb ? st_off1 : st_off0;
                    sts_v4(wt_s + so, pa[0], pa[1], pa[2], pa[3]);
                    sts_v4(wt_s + 1024 + so, pb[0], pb[1], pb[2], pb[3]);
                }
            } else {                                            // ragged end: rows beyond the matrix contribute zero
#pragma unroll 1
                for (uint32_t r = 0; r < 16; ++r) {
                    const uint32_t i = i0 + r;
                    uint32_t hA = 0, hB = 0;
                    if (i < nA) {
                        const uint32_t e = decode_fast(stA, lut_s);
                        renorm_fast<WB>(stA, posA);
                        if (__any_sync(kFull, stA < kRansL)) renorm_fast<WB>(stA, posA);
                        hA = weight_bits(e, lds_u8(man_s + i * TW));
                    }
                    if (i < nB) {
                        const uint32_t e = decode_fast(stB, lut_s);
                        renorm_fast<WB>(stB, posB);
                        if (__any_sync(kFull, stB < kRansL)) renorm_fast<WB>(stB, posB);
                        hB = weight_bits(e, lds_u8(man_s + manB_off + i * TW));
                    }
                    const uint32_t o = wt_s + ((r & 8) ? st_off1 : st_off0) + (r & 7) * 2;
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(o), "h"((uint16_t)hA) : "memory");
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(o + 1024), "h"((uint16_t)hB) : "memory");
                }
            }
            __syncwarp();
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(wt_s + ld_off0, b0, b1, b2, b3);
            mma_bf16(acc[0], xa, b0, b1);
            mma_bf16(acc[1], xa, b2, b3);
            ldmatrix_x4(wt_s + ld_off1, b0, b1, b2, b3);
            mma_bf16(acc[2], xa, b0, b1);
            mma_bf16(acc[3], xa, b2, b3);
            if (i0 < nB) {
                ldmatrix_x4(wt_s + 1024 + ld_off0, b0, b1, b2, b3);
                mma_bf16(acc[0], xb, b0, b1);
                mma_bf16(acc[1], xb, b2, b3);
                ldmatrix_x4(wt_s + 1024 + ld_off1, b0, b1, b2, b3);
                mma_bf16(acc[2], xb, b0, b1);
                mma_bf16(acc[3], xb, b2, b3);
            }
        }
        stage ^= 1;
    }
    flush(cur_grp);
}

// ------------------------------------------------------------------------ host

template <uint32_t TW>
static int launch_tw(const MmaArgs &p, uint32_t blocks, uint32_t warps, size_t smem, int max_smem, cudaStream_t s) {
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_linear_mma<TW>, (size_t)max_smem)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CI_CUDA(cudaLaunchKernelEx(&cfg, k_linear_mma<TW>, p));
    return CI_OK;
}

int launch_linear_mma(const LinArgs &a, uint32_t max_tile_len, cudaStream_t s) {
    const Geom &g = a.g;
    if (!(g.tw == 8 || g.tw == 16 || g.tw == 32)) return 1;
    if ((reinterpret_cast<uintptr_t>(a.stream) & 15u) || (reinterpret_cast<uintptr_t>(a.mantissa) & 15u) ||
        (reinterpret_cast<uintptr_t>(a.states) & 15u))
        return 1;
    if (max_tile_len == 0) return 1;                            // unknown: cannot size the byte window
    if (a.M > 16 || (g.th * g.tw) % 16 != 0) return 1;
    // The kernel does not bounds-test stream cursors; a malformed stream can walk at most
    // tile_h rows below its window, which must still be inside the CTA's shared memory.
    if (g.th * g.W > kLutBytes) return 1;

    int dev = 0, max_smem = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    MmaArgs p;
    p.a = a;
    p.win_cap = ((max_tile_len * 64u + 15u) & ~15u) + 16u;
    p.stage_bytes = p.win_cap + g.th * 32u + 256u;
    p.warp_bytes = 2 * p.stage_bytes + kWtBytes;
    p.warp_bytes = (p.warp_bytes + 127u) & ~127u;
    const uint32_t fixed = kLutBytes + kBarBytes;
    if ((uint32_t)max_smem < fixed + 4 * p.warp_bytes) return 1;
    uint32_t w_max = ((uint32_t)max_smem - fixed) / p.warp_bytes;
    if (w_max > 16) w_max = 16;

    // Room for the shared-memory reduction of column groups that sit inside one CTA (one or two activation rows):
    // at most w + w * per_warp / tiles_k + 2 slots of [2][32] floats and as many tickets.
    const bool small_m = a.M <= 2;
    auto red_slots_for = [&](uint32_t w, uint64_t per) { return small_m ? (uint32_t)(w + w * per / g.tiles_k + 2) : 0u; };
    auto fits = [&](uint32_t w, uint64_t per) {
        return fixed + (size_t)w * p.warp_bytes + (size_t)red_slots_for(w, per) * 260 + 16 <= (size_t)max_smem;
    };

    // Units per warp must be a whole number: pick the warp count whose grid wastes the least; among warp counts
    // within 3 % of the best, prefer one whose CTAs hold whole column groups (their reduction then never leaves
    // the multiprocessor).
    const uint32_t P = (uint32_t)sm_count();
    p.total = g.groups * g.tiles_k;
    uint32_t best_w = 0;
    double best = -1.0;
    auto eff_of = [&](uint32_t w, uint64_t &per) {
        const uint64_t slots = (uint64_t)P * w;
        per = (p.total + slots - 1) / slots;
        double eff = (double)p.total / (double)(slots * per);
        if (w < 8) eff *= w / 8.0;                              // too few warps cannot hide the decode chain
        return eff;
    };
    for (uint32_t w = 4; w <= w_max; ++w) {
        uint64_t per;
        const double eff = eff_of(w, per);
        if (eff >= best) { best = eff; best_w = w; }
    }
    if (best_w == 0) return 1;
    bool use_red = false;                                       // the reduction area never costs a warp: it is dropped instead
    if (small_m) {
        uint64_t per;
        eff_of(best_w, per);
        use_red = fits(best_w, per);
        for (uint32_t w = w_max; w >= 4; --w) {
            const double eff = eff_of(w, per);
            if (fits(w, per) && eff >= 0.97 * best && (w * per) % g.tiles_k == 0) { best_w = w; use_red = true; break; }
        }
    }
    const uint64_t slots = (uint64_t)P * best_w;
    p.per_warp = (uint32_t)((p.total + slots - 1) / slots);
    const uint32_t warps_needed = (p.total + p.per_warp - 1) / p.per_warp;
    const uint32_t blocks = (warps_needed + best_w - 1) / best_w;
    p.x_aligned = ((reinterpret_cast<uintptr_t>(a.x) & 3u) == 0 && (a.ldx & 1) == 0) ? 1u : 0u;
    p.status = a.tickets + (kTicketBytes - 1);

    p.red_slots = use_red ? red_slots_for(best_w, p.per_warp) : 0u;
    p.red_off = (fixed + best_w * p.warp_bytes + 15u) & ~15u;
    const size_t smem = p.red_off + (size_t)p.red_slots * 260;
    if (a.dry_run) return CI_OK;                                // qualification only
    if (g.tw == 32) return launch_tw<32>(p, blocks, best_w, smem, max_smem, s);
    if (g.tw == 16) return launch_tw<16>(p, blocks, best_w, smem, max_smem, s);
    return launch_tw<8>(p, blocks, best_w, smem, max_smem, s);
}

}  // namespace ci
