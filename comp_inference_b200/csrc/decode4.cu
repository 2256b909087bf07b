// Stand-alone decoder for 32-wide tiles, four streams per lane: exponent plane (u8) or the full bf16
// weight [K,N].  Replaces rans_decompress_tiled_kernel_triton_ilp2 (comp_inference/rans_triton.py:34-119)
// and the decode + uninterleave + reconstruct chain of rans_decompress_module_weight_bf16
// (comp_inference/comp_inference.py:633-711).
//
// Work unit: one warp decodes two horizontally adjacent tiles of one tile row = 128 streams.  Lane l
// (quad = l / 2, half = l % 2) owns the four adjacent columns 4 quad .. 4 quad + 3 of the 64-column
// strip, top-half streams on even lanes and bottom-half streams on odd lanes, so
//  * the two tiles' byte blocks, copied by cp.async into one window of 128-byte rows (left tile in
//    bytes 0..63, right tile in 64..127), give every lane a word column -- a shared-memory bank -- of its
//    own: the per-symbol renormalisation byte loads never conflict, whatever row each cursor is on;
//  * the sign+mantissa bytes of a row of the lane's four columns are one 32-bit global load (a warp
//    reads four full 32-byte sectors), fetched four rows ahead of their use;
//  * a decoded row of the lane is four adjacent weights: one 8-byte store (4 bytes for the plane), and the
//    sixteen lanes of a half write 128 contiguous bytes of an output row.
// Initial states arrive by bulk copy with the unit, byte ranges of later units are loaded ahead by all
// lanes in parallel, units are double buffered per warp, and the kernel is launched with programmatic
// dependent launch (its preamble overlaps the previous kernel of the stream).
#include "decode.cuh"
#include "ptx.cuh"

namespace ci {

constexpr uint32_t kDec4Warps = 16;
constexpr uint32_t kDec4BarBytes = 256;

struct Dec4Args {
    DecArgs a;
    uint32_t cap_rows;     // rows of a byte window (>= every tile_max_len)
    uint32_t stage_bytes;  // window + 128 initial states
    uint32_t pairs_n;      // tile pairs per tile row = ceil(tiles_n / 2)
    uint32_t total;        // units
    uint32_t *status;      // may be null
};

__device__ __forceinline__ void d4_cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void d4_cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t d4_ldg_stream(const void *src) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(src));
    return v;
}

template <bool BF16>
__global__ void __launch_bounds__(kDec4Warps * 32, 1) k_decode4(const __grid_constant__ Dec4Args p, void *out) {
    extern __shared__ __align__(128) uint8_t smem[];
    const DecArgs &a = p.a;
    const Geom &g = a.g;
    const uint32_t W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t smem_s = smem_u32(smem);
    // The table sits on a 16 KB boundary of the shared window: an entry's address is then
    // (state << 2 & 0x3FFC) | base, without an addition.
    const uint32_t lut_s = (smem_s + kLutBytes - 1) & ~(kLutBytes - 1);
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem + (lut_s - smem_s));
    const uint32_t wbase_s = lut_s + kLutBytes + kDec4BarBytes + warp * 2 * p.stage_bytes;
    const uint32_t bar_base = lut_s + kLutBytes + warp * 16;
    const uint32_t st_off = p.cap_rows * 128;
    const uint32_t man_tile = g.th * 32;

    const uint32_t quad = lane >> 1, hsel = lane & 1;           // column quad of the 64-column strip, stream half
    const uint32_t tsel = quad >> 3;                            // left / right tile
    const uint32_t gw = blockIdx.x * W + warp, n_warps = gridDim.x * W;

    // Unit u = (tile row, tile pair), the pair running fastest: warps that run at the same time write
    // neighbouring pieces of the same output rows.
    auto unit_tiles = [&](uint32_t u, uint32_t &tk, uint32_t &tp, uint32_t &t0, bool &two) {
        tk = u / p.pairs_n;
        tp = u - tk * p.pairs_n;
        t0 = tk * g.tiles_n + 2 * tp;
        two = 2 * tp + 1 < g.tiles_n;
    };

    // Byte ranges of the units this warp will decode, 32 at a time: lane j holds its (dbase + j)-th unit.
    uint32_t d_off0 = 0, d_ml0 = 0, d_off1 = 0, d_ml1 = 0, dbase = 0;
    auto load_desc = [&]() {
        const uint64_t u = (uint64_t)gw + (uint64_t)(dbase + lane) * n_warps;
        d_off0 = d_ml0 = d_off1 = d_ml1 = 0;
        if (u >= p.total) return;
        uint32_t tk, tp, t0;
        bool two;
        unit_tiles((uint32_t)u, tk, tp, t0, two);
        d_off0 = __ldg(a.tile_offsets + t0);
        d_ml0 = __ldg(a.tile_max_lens + t0);
        if (two) {
            d_off1 = __ldg(a.tile_offsets + t0 + 1);
            d_ml1 = __ldg(a.tile_max_lens + t0 + 1);
        }
    };

    auto issue = [&](uint32_t u, uint32_t stage, uint32_t off0, uint32_t ml0, uint32_t off1, uint32_t ml1) {
        uint32_t tk, tp, t0;
        bool two;
        unit_tiles(u, tk, tp, t0, two);
        const uint32_t bar = bar_base + stage * 8;
        const uint32_t dst = wbase_s + stage * p.stage_bytes;
        if (ml0 > p.cap_rows || ml1 > p.cap_rows) {             // metadata disagrees with the declared maximum
            if (lane == 0 && p.status) atomicExch(p.status, 2u);
            ml0 = ml1 = 0;
        }
        if (lane == 0) {
            fence_async_proxy();
            mbar_expect_tx(bar, two ? 512u : 256u);
            bulk_load(dst + st_off, a.states + (size_t)t0 * 64, two ? 512u : 256u, bar);   // the tiles are neighbours
        }
        const uint8_t *s0 = a.stream + off0, *s1 = a.stream + off1;
        for (uint32_t i = lane; i < ml0 * 4; i += 32) d4_cp_async16(dst + (i >> 2) * 128 + (i & 3) * 16, s0 + i * 16);
        for (uint32_t i = lane; i < ml1 * 4; i += 32) d4_cp_async16(dst + (i >> 2) * 128 + 64 + (i & 3) * 16, s1 + i * 16);
        d4_cp_async_arrive(bar);
    };

    if (lane == 0) {
        mbar_init(bar_base, 33);                                // 32 cp.async arrivals + the bulk copy's expect_tx
        mbar_init(bar_base + 8, 33);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    load_desc();
    uint32_t nx_off0 = __shfl_sync(kFull, d_off0, 0), nx_ml0 = __shfl_sync(kFull, d_ml0, 0);
    uint32_t nx_off1 = __shfl_sync(kFull, d_off1, 0), nx_ml1 = __shfl_sync(kFull, d_ml1, 0);
    if (gw < p.total) issue(gw, 0, nx_off0, nx_ml0, nx_off1, nx_ml1);
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    // Only the weight was touched so far.  With programmatic dependent launch the output buffer may still
    // be in use by the previous kernel of the stream: wait for it, then let the next launch begin.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t n_groups = g.half / 4;
    uint32_t parity0 = 0, parity1 = 0, stage = 0, li = 0;
    uint32_t s0, s1, s2, s3, pos0, pos1, pos2, pos3;

    auto renorm4 = [&](uint32_t y0, uint32_t y1, uint32_t y2, uint32_t y3) {
        const uint32_t lowest = min(min(s0, s1), min(s2, s3));
        renorm_first<128>(s0, pos0, y0);
        renorm_first<128>(s1, pos1, y1);
        renorm_first<128>(s2, pos2, y2);
        renorm_first<128>(s3, pos3, y3);
        if (__any_sync(kFull, lowest < 256u)) {                 // a second byte: only after a symbol of frequency < 16
            renorm_fast<128>(s0, pos0);
            renorm_fast<128>(s1, pos1);
            renorm_fast<128>(s2, pos2);
            renorm_fast<128>(s3, pos3);
        }
    };

    for (uint32_t t = gw; t < p.total; t += n_warps, ++li) {
        uint32_t tk, tp, t0;
        bool two;
        unit_tiles(t, tk, tp, t0, two);
        const bool tile_live = tsel == 0 || two;
        const uint32_t col0 = 64 * tp + 4 * quad;               // first of this lane's four columns
        const bool store = tile_live && col0 < g.N;
        const uint32_t row = tk * g.th + hsel * g.half;         // first row of this lane's streams
        const uint8_t *mp = a.mantissa + ((size_t)t0 + tsel) * man_tile + hsel * (man_tile / 2) + (quad & 7) * 4;
        uint32_t mA[4] = {0u, 0u, 0u, 0u}, mB[4];
        if (BF16 && tile_live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) mA[i] = d4_ldg_stream(mp + i * 32);
        }
        const uint32_t ml = tsel ? nx_ml1 : nx_ml0;
        __syncwarp();                                           // every lane is done with the other stage
        if ((uint64_t)t + n_warps < p.total) {
            if (li + 1 - dbase == 32) {
                dbase = li + 1;
                load_desc();
            }
            const uint32_t j = li + 1 - dbase;
            nx_off0 = __shfl_sync(kFull, d_off0, j);
            nx_ml0 = __shfl_sync(kFull, d_ml0, j);
            nx_off1 = __shfl_sync(kFull, d_off1, j);
            nx_ml1 = __shfl_sync(kFull, d_ml1, j);
            issue(t + n_warps, stage ^ 1, nx_off0, nx_ml0, nx_off1, nx_ml1);
        }

        const uint32_t win_s = wbase_s + stage * p.stage_bytes;
        const uint32_t st_s = win_s + st_off + tsel * 256 + (hsel * 32 + (quad & 7) * 4) * 4;
        pos0 = win_s + tsel * 64 + hsel * 32 + (quad & 7) * 4;
        if (tile_live && ml <= p.cap_rows) pos0 += (ml - 1) * 128;   // last byte row; an empty tile starts one row below
        pos1 = pos0 + 1;
        pos2 = pos0 + 2;
        pos3 = pos0 + 3;

        {
            const uint32_t bar = bar_base + stage * 8, par = stage ? parity1 : parity0;
            uint32_t ok = 0;
            if (lane == 0)
                for (uint32_t it = 0; it < kWaitPolls && !ok; ++it) ok = mbar_try_wait(bar, par);
            ok = __shfl_sync(kFull, ok, 0);
            if (stage) parity1 ^= 1; else parity0 ^= 1;
            if (!ok) {
                if (lane == 0 && p.status) atomicExch(p.status, 1u);
                stage ^= 1;
                continue;
            }
            (void)mbar_try_wait(bar, par);                      // each lane observes the completed phase itself
        }
        s0 = s1 = s2 = s3 = kRansL;
        if (tile_live) {
            s0 = lds_u32(st_s);
            s1 = lds_u32(st_s + 4);
            s2 = lds_u32(st_s + 8);
            s3 = lds_u32(st_s + 12);
        }

        uint8_t *o8 = reinterpret_cast<uint8_t *>(out) + ((size_t)row * g.N + col0) * (BF16 ? 2 : 1);
        const size_t o_pitch = (size_t)g.N * (BF16 ? 2 : 1);

        // Four rows of the lane's four columns; m = their sign+mantissa words.
        auto group = [&](const uint32_t (&m)[4]) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const uint32_t y0 = lds_u8(pos0), y1 = lds_u8(pos1), y2 = lds_u8(pos2), y3 = lds_u8(pos3);
                const uint32_t e0 = decode_aligned(s0, lut_s);
                const uint32_t e1 = decode_aligned(s1, lut_s);
                const uint32_t e2 = decode_aligned(s2, lut_s);
                const uint32_t e3 = decode_aligned(s3, lut_s);
                renorm4(y0, y1, y2, y3);
                // bits 8..23 of two entries side by side: the symbols sit at bits 4..11 / 20..27
                const uint32_t a01 = __byte_perm(e0, e1, 0x6521), a23 = __byte_perm(e2, e3, 0x6521);
                if (BF16) {
                    const uint32_t w01 = ((a01 << 3) & 0x7F807F80u) | (__byte_perm(m[r], 0u, 0x1100) & 0x807F807Fu);
                    const uint32_t w23 = ((a23 << 3) & 0x7F807F80u) | (__byte_perm(m[r], 0u, 0x3322) & 0x807F807Fu);
                    if (store) *reinterpret_cast<uint2 *>(o8) = make_uint2(w01, w23);
                } else {
                    const uint32_t w = __byte_perm(a01 >> 4, a23 >> 4, 0x6420);
                    if (store) *reinterpret_cast<uint32_t *>(o8) = w;
                }
                o8 += o_pitch;
            }
        };
#pragma unroll 1
        for (uint32_t gi = 0; gi < n_groups; gi += 2) {         // sign+mantissa words are fetched one group ahead
            if (BF16 && tile_live) {
#pragma unroll
                for (int i = 0; i < 4; ++i) mB[i] = d4_ldg_stream(mp + 128 + i * 32);
            }
            group(mA);
            mp += 256;
            if (BF16 && tile_live && gi + 2 < n_groups) {
#pragma unroll
                for (int i = 0; i < 4; ++i) mA[i] = d4_ldg_stream(mp + i * 32);
            }
            group(mB);
        }
        stage ^= 1;
    }
}

// ------------------------------------------------------------------------ host

template <bool BF16>
static int launch_dec4(const Dec4Args &p, uint32_t blocks, uint32_t warps, size_t smem, int max_smem, void *out,
                       cudaStream_t s) {
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_decode4<BF16>, (size_t)max_smem)) return rc;
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
    CI_CUDA(cudaLaunchKernelEx(&cfg, k_decode4<BF16>, p, out));
    return CI_OK;
}

// Returns CI_OK when it launched, 1 when the tensor does not qualify, < 0 on error.
int launch_decode4(const DecArgs &a, uint32_t max_tile_len, bool bf16, void *out, cudaStream_t s) {
    const Geom &g = a.g;
    // whole tile rows, 16-symbol-aligned streams, rows of the output that can be written as quads
    if (g.tw != 32 || g.th % 16 != 0 || g.K % g.th != 0 || g.N % 4 != 0 || max_tile_len == 0) return 1;
    if (!a.stream_aligned || (reinterpret_cast<uintptr_t>(a.states) & 15u)) return 1;
    if (bf16 && (reinterpret_cast<uintptr_t>(a.mantissa) & 3u)) return 1;
    if (reinterpret_cast<uintptr_t>(out) & (bf16 ? 7u : 3u)) return 1;
    if (g.th * 128u > kLutBytes) return 1;                      // see the note on stream cursors in ptx.cuh
    int dev = 0, max_smem = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    Dec4Args p;
    p.a = a;
    p.cap_rows = max_tile_len;
    p.stage_bytes = (p.cap_rows * 128u + 512u + 127u) & ~127u;
    p.pairs_n = (g.tiles_n + 1) / 2;
    p.total = g.tiles_k * p.pairs_n;
    p.status = nullptr;
    const uint32_t fixed = 2 * kLutBytes + kDec4BarBytes;           // up to one table size is lost to the table's alignment
    const uint32_t warp_bytes = 2 * p.stage_bytes;
    if ((uint32_t)max_smem < fixed + 4 * warp_bytes) return 1;
    uint32_t w_max = ((uint32_t)max_smem - fixed) / warp_bytes;
    if (w_max > kDec4Warps) w_max = kDec4Warps;
    // A multiprocessor decodes at a fixed rate once it has about eight warps, so the run time follows the
    // units per multiprocessor: pick the warp count that makes (rounds per warp) x (warps) smallest.
    const uint32_t P = (uint32_t)sm_count();
    uint32_t warps = w_max;
    uint64_t best = ~0ull;
    for (uint32_t w = w_max < 8 ? w_max : 8; w <= w_max; ++w) {
        const uint64_t rounds = (p.total + (uint64_t)P * w - 1) / ((uint64_t)P * w);
        if (rounds * w <= best) { best = rounds * w; warps = w; }
    }
    uint32_t blocks = (p.total + warps - 1) / warps;
    if (blocks > P) blocks = P;
    const size_t smem = fixed + (size_t)warps * warp_bytes;
    return bf16 ? launch_dec4<true>(p, blocks, warps, smem, max_smem, out, s)
                : launch_dec4<false>(p, blocks, warps, smem, max_smem, out, s);
}

}  // namespace ci
