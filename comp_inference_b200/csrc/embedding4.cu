// Fused decode + row gather for 32-wide tiles, four streams per lane: out[i,:] = W[ids[i],:].
// Replaces fused_rans_embedding_kernel_ilp2 (comp_inference/embedding_triton.py:170-275); ids outside
// [0,K) produce a zero row (embedding_triton.py:203-210).
//
// A stream cannot be entered in the middle: to emit row r of a tile the (r mod tile_h/2) symbols above it
// in its half-tile stream are decoded and dropped.  Work unit: one warp takes (token, 128 columns) = the
// token's half (top or bottom) of four neighbouring tiles = 128 streams; lane l owns the four adjacent
// columns 4l .. 4l+3 of the strip.  The four 32-byte-wide half slices of the tiles' byte blocks are
// copied by cp.async side by side into a window of 128-byte rows, which gives every lane a word column
// (a shared-memory bank) of its own, so the renormalisation byte loads never conflict; the row's four
// weights leave as one 8-byte store.  The pipeline is three tasks deep so that no dependent global load
// (id -> tile metadata -> byte block) is ever waited for: ids are read three tasks ahead, tile offsets and
// depths two ahead, the byte blocks and initial states one ahead into the other half of a per-warp double
// buffer.
#include "embedding.cuh"
#include "ptx.cuh"

namespace ci {

constexpr uint32_t kEmb4Warps = 16;
constexpr uint32_t kEmb4BarBytes = 256;

struct Emb4Args {
    EmbArgs a;
    uint32_t cap_rows;     // rows of a byte window (>= every tile_max_len)
    uint32_t stage_bytes;
    uint32_t blocks_n;     // 128-column blocks per row = ceil(tiles_n / 4)
    uint64_t total;        // tasks
    uint32_t out_vec;      // rows of the output can be written as 8-byte quads
};

__device__ __forceinline__ void e4_cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void e4_cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// What a task needs to know about its token: tile row, half, symbols to drop; valid = id inside the table.
struct Tok {
    uint32_t tk, hsel, inner, rel;
    bool valid;
};

__global__ void __launch_bounds__(kEmb4Warps * 32, 1) k_embedding4(const __grid_constant__ Emb4Args p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const EmbArgs &a = p.a;
    const Geom &g = a.g;
    const uint32_t W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t smem_s = smem_u32(smem);
    // The table sits on a 16 KB boundary of the shared window: an entry's address is then
    // (state << 2 & 0x3FFC) | base, without an addition.
    const uint32_t lut_s = (smem_s + kLutBytes - 1) & ~(kLutBytes - 1);
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem + (lut_s - smem_s));
    const uint32_t wbase_s = lut_s + kLutBytes + kEmb4BarBytes + warp * 2 * p.stage_bytes;
    const uint32_t bar_base = lut_s + kLutBytes + warp * 16;
    const uint64_t gw = (uint64_t)blockIdx.x * W + warp, n_warps = (uint64_t)gridDim.x * W;
    const uint32_t tsel = lane >> 3, quad = lane & 7;           // tile of the block, column quad inside it

    auto parse = [&](uint64_t task, int64_t id) {
        Tok t;
        t.valid = task < p.total && id >= 0 && id < (int64_t)g.K;
        const uint32_t row = t.valid ? (uint32_t)id : 0u;
        t.tk = row / g.th;
        t.rel = row - t.tk * g.th;
        t.hsel = t.rel >= g.half ? 1u : 0u;
        t.inner = t.rel - t.hsel * g.half;
        return t;
    };
    auto load_id = [&](uint64_t task) -> int64_t { return task < p.total ? __ldg(a.ids + task / p.blocks_n) : -1; };
    // Lanes 0..3 fetch offset and depth of the block's four tiles (zero for a tile beyond the matrix).
    auto load_meta = [&](uint64_t task, const Tok &t, uint32_t &off, uint32_t &ml) {
        off = ml = 0;
        const uint32_t tn = (uint32_t)(task % p.blocks_n) * 4 + lane;
        if (t.valid && lane < 4 && tn < g.tiles_n) {
            const size_t tile = (size_t)t.tk * g.tiles_n + tn;
            off = __ldg(a.tile_offsets + tile);
            ml = __ldg(a.tile_max_lens + tile);
        }
    };
    // Copies the token's half slice (32 bytes of every row) of the four tiles into `stage`.
    auto issue = [&](const Tok &t, uint32_t off, uint32_t ml, uint32_t stage) {
        const uint32_t bar = bar_base + stage * 8, dst = wbase_s + stage * p.stage_bytes;
        if (ml > p.cap_rows) ml = 0;                            // metadata disagrees with the declared maximum
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t mlj = __shfl_sync(kFull, ml, j), offj = __shfl_sync(kFull, off, j);
            const uint8_t *src = a.stream + offj + t.hsel * 32;
            for (uint32_t i = lane; i < mlj * 2; i += 32)
                e4_cp_async16(dst + (i >> 1) * 128 + j * 32 + (i & 1) * 16, src + (size_t)(i >> 1) * 64 + (i & 1) * 16);
        }
        e4_cp_async_arrive(bar);
    };
    // This lane's four initial states of a task (one 16-byte load) and its tile's depth.
    auto load_states = [&](uint64_t task, const Tok &t) {
        uint4 s = make_uint4(kRansL, kRansL, kRansL, kRansL);
        const uint32_t tn = (uint32_t)(task % p.blocks_n) * 4 + tsel;
        if (t.valid && tn < g.tiles_n)
            s = __ldg(reinterpret_cast<const uint4 *>(a.states + ((size_t)t.tk * g.tiles_n + tn) * 64 + t.hsel * 32 + quad * 4));
        return s;
    };

    if (lane == 0) {
        mbar_init(bar_base, 32);                                // one arrival per lane when its copies have landed
        mbar_init(bar_base + 8, 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    // The ids (and the output buffer) may be products of the previous kernel of the stream: with
    // programmatic dependent launch wait for it here, after the table load that does not depend on it.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- fill the pipeline: task t = gw, t + n_warps, t + 2 n_warps; id of t + 3 n_warps -----------------
    int64_t id0 = load_id(gw), id1 = load_id(gw + n_warps), id2 = load_id(gw + 2 * n_warps);
    Tok tc = parse(gw, id0), tn1 = parse(gw + n_warps, id1), tn2 = parse(gw + 2 * n_warps, id2);
    uint32_t offC, mlC, offN, mlN, offNN = 0, mlNN = 0;
    load_meta(gw, tc, offC, mlC);
    load_meta(gw + n_warps, tn1, offN, mlN);
    int64_t id3 = load_id(gw + 3 * n_warps);
    uint4 stC = load_states(gw, tc), stN = make_uint4(kRansL, kRansL, kRansL, kRansL);
    if (gw < p.total) issue(tc, offC, mlC, 0);

    uint32_t parity0 = 0, parity1 = 0, stage = 0;
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

    for (uint64_t t = gw; t < p.total; t += n_warps) {
        const uint32_t cb = (uint32_t)(t % p.blocks_n);
        const uint64_t ti = t / p.blocks_n;
        const uint32_t tn = cb * 4 + tsel, col0 = tn * 32 + quad * 4;
        const bool tile_live = tc.valid && tn < g.tiles_n;
        const uint32_t ml = __shfl_sync(kFull, mlC, tsel);
        // sign+mantissa bytes of the wanted row of this lane's four columns: in flight during the decode
        uint32_t man = 0;
        if (tile_live)
            man = __ldg(reinterpret_cast<const uint32_t *>(a.mantissa + ((size_t)tc.tk * g.tiles_n + tn) * (g.th * 32) +
                                                           (size_t)tc.rel * 32 + quad * 4));
        __syncwarp();                                           // every lane is done with the other stage
        // next task: copies and states; the task after: metadata; the one after that: its id
        load_meta(t + 2 * n_warps, tn2, offNN, mlNN);
        const int64_t id4 = load_id(t + 4 * n_warps);
        if (t + n_warps < p.total) {
            issue(tn1, offN, mlN, stage ^ 1);
            stN = load_states(t + n_warps, tn1);
        }

        const uint32_t win_s = wbase_s + stage * p.stage_bytes;
        pos0 = win_s + tsel * 32 + quad * 4;
        if (tile_live && ml >= 1 && ml <= p.cap_rows) pos0 += (ml - 1) * 128;
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
            (void)mbar_try_wait(bar, par);                      // each lane observes the completed phase itself
            if (!ok) {                                          // give up on this task: zero row, keep the pipeline moving
                s0 = s1 = s2 = s3 = kRansL;
            } else {
                s0 = stC.x; s1 = stC.y; s2 = stC.z; s3 = stC.w;
            }
            if (ok && tc.valid) {
#pragma unroll 4
                for (uint32_t i = 0; i < tc.inner; ++i) {        // the rows above the wanted one
                    const uint32_t y0 = lds_u8(pos0), y1 = lds_u8(pos1), y2 = lds_u8(pos2), y3 = lds_u8(pos3);
                    (void)decode_aligned(s0, lut_s);
                    (void)decode_aligned(s1, lut_s);
                    (void)decode_aligned(s2, lut_s);
                    (void)decode_aligned(s3, lut_s);
                    renorm4(y0, y1, y2, y3);
                }
            }
            uint32_t w01 = 0, w23 = 0;
            if (ok && tile_live) {
                const uint32_t e0 = lds_u32(((s0 << 2) & (kProbMask << 2)) | lut_s), e1 = lds_u32(((s1 << 2) & (kProbMask << 2)) | lut_s);
                const uint32_t e2 = lds_u32(((s2 << 2) & (kProbMask << 2)) | lut_s), e3 = lds_u32(((s3 << 2) & (kProbMask << 2)) | lut_s);
                const uint32_t a01 = __byte_perm(e0, e1, 0x6521), a23 = __byte_perm(e2, e3, 0x6521);
                w01 = ((a01 << 3) & 0x7F807F80u) | (__byte_perm(man, 0u, 0x1100) & 0x807F807Fu);
                w23 = ((a23 << 3) & 0x7F807F80u) | (__byte_perm(man, 0u, 0x3322) & 0x807F807Fu);
            }
            if (col0 < g.N) {
                uint16_t *dst = a.out + ti * a.ldo + col0;
                if (p.out_vec && col0 + 4 <= g.N) {
                    *reinterpret_cast<uint2 *>(dst) = make_uint2(w01, w23);
                } else {
                    const uint32_t v[4] = {w01 & 0xFFFFu, w01 >> 16, w23 & 0xFFFFu, w23 >> 16};
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (col0 + c < g.N) dst[c] = (uint16_t)v[c];
                }
            }
        }
        // rotate the pipeline
        tc = tn1;
        tn1 = tn2;
        tn2 = parse(t + 3 * n_warps, id3);
        id3 = id4;
        offC = offN; mlC = mlN;
        offN = offNN; mlN = mlNN;
        stC = stN;
        stage ^= 1;
    }
}

// ------------------------------------------------------------------------ host

int launch_embedding4(const EmbArgs &a, uint32_t max_tile_len, cudaStream_t s) {
    const Geom &g = a.g;
    if (g.tw != 32 || g.th % 2 != 0 || max_tile_len == 0) return 1;
    if ((reinterpret_cast<uintptr_t>(a.stream) & 15u) || (reinterpret_cast<uintptr_t>(a.states) & 15u) ||
        (reinterpret_cast<uintptr_t>(a.mantissa) & 3u))
        return 1;
    if (g.th * 128u > kLutBytes) return 1;                      // see the note on stream cursors in ptx.cuh
    int dev = 0, max_smem = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    Emb4Args p;
    p.a = a;
    p.cap_rows = max_tile_len;
    p.stage_bytes = (p.cap_rows * 128u + 127u) & ~127u;
    p.blocks_n = (g.tiles_n + 3) / 4;
    p.total = a.n_ids * p.blocks_n;
    p.out_vec = ((reinterpret_cast<uintptr_t>(a.out) & 7u) == 0 && (a.ldo & 3) == 0) ? 1u : 0u;
    const uint32_t fixed = 2 * kLutBytes + kEmb4BarBytes;           // up to one table size is lost to the table's alignment
    const uint32_t warp_bytes = 2 * p.stage_bytes;
    if ((uint32_t)max_smem < fixed + 4 * warp_bytes) return 1;
    uint32_t warps = ((uint32_t)max_smem - fixed) / warp_bytes;
    if (warps > kEmb4Warps) warps = kEmb4Warps;
    uint64_t blocks = (p.total + warps - 1) / warps;
    const uint64_t P = (uint64_t)sm_count();
    if (blocks > P) blocks = P;
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_embedding4, (size_t)max_smem)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = fixed + (size_t)warps * warp_bytes;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CI_CUDA(cudaLaunchKernelEx(&cfg, k_embedding4, p));
    return CI_OK;
}

}  // namespace ci
