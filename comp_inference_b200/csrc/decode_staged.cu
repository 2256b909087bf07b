// Stand-alone decoder on the staged path: exponent plane (u8) or the full bf16 weight [K,N].
// Replaces rans_decompress_tiled_kernel_triton_ilp2 (comp_inference/rans_triton.py:34-119) and the
// decode + uninterleave + reconstruct chain of rans_decompress_module_weight_bf16
// (comp_inference/comp_inference.py:633-711).
//
// Same unit and staging as the fused linear: one warp per (tile row, 32-column group), the unit's
// compressed byte block (and, for bf16 output, its sign+mantissa block) arrive by bulk async copy
// into a per-warp double buffer while the previous unit is decoded.  Units are dealt to the warps of
// the persistent grid round-robin with the column group running fastest, so warps that run at the
// same time write neighbouring 64-byte segments of the same output rows.
#include "decode.cuh"
#include "ptx.cuh"

namespace ci {

struct StagedDecArgs {
    DecArgs a;
    uint32_t win_cap, stage_bytes, warp_bytes, total;
};

template <uint32_t TW, bool BF16>
__global__ void __launch_bounds__(512, 1) k_decode_staged(const __grid_constant__ StagedDecArgs p, void *out) {
    constexpr uint32_t WB = 2 * TW, TPG = 32 / TW;
    extern __shared__ __align__(128) uint8_t smem[];
    const DecArgs &a = p.a;
    const Geom &g = a.g;
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem);
    const uint32_t W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t smem_s = smem_u32(smem);
    const uint32_t wbase_s = smem_s + kLutBytes + 256 + warp * p.warp_bytes;
    const uint32_t bar_base = smem_s + kLutBytes + warp * 16;
    const uint32_t man_tile = g.th * TW;
    const uint32_t gw = blockIdx.x * W + warp, n_warps = gridDim.x * W;

    auto issue = [&](uint32_t t, uint32_t stage) {
        if (lane != 0) return;
        const uint32_t tk = t / g.groups, grp = t - tk * g.groups;
        const uint32_t tn0 = grp * TPG, nt = min(TPG, g.tiles_n - tn0);
        const uint32_t t0 = tk * g.tiles_n + tn0, tl = t0 + nt - 1;
        const uint32_t begin = a.tile_offsets[t0];
        uint32_t wbytes = a.tile_offsets[tl] + a.tile_max_lens[tl] * WB - begin;
        if (wbytes > p.win_cap) wbytes = 0;                      // inconsistent metadata: decode garbage, never overrun
        const uint32_t mbytes = BF16 ? nt * man_tile : 0;
        const uint32_t bar = bar_base + stage * 8, dst = wbase_s + stage * p.stage_bytes;
        fence_async_proxy();
        if (wbytes + mbytes == 0) { mbar_arrive(bar); return; }
        mbar_expect_tx(bar, wbytes + mbytes);
        if (wbytes) bulk_load(dst, a.stream + begin, wbytes, bar);
        if (mbytes) bulk_load(dst + p.win_cap, a.mantissa + (size_t)t0 * man_tile, mbytes, bar);
    };

    if (lane == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (gw < p.total) issue(gw, 0);
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    // Programmatic dependent launch: the output may still be in use by the previous kernel of the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t lut_s = smem_s;
    uint32_t parity0 = 0, parity1 = 0, stage = 0;
    for (uint32_t t = gw; t < p.total; t += n_warps) {
        if (t + n_warps < p.total) issue(t + n_warps, stage ^ 1);
        const uint32_t tk = t / g.groups, grp = t - tk * g.groups;
        // this lane's column, tile and streams
        const uint32_t n = grp * 32 + lane;
        uint32_t tn = n / TW;
        const bool live = n < g.N;
        if (tn >= g.tiles_n) tn = g.tiles_n - 1;
        const uint32_t lc = n % TW, tile = tk * g.tiles_n + tn;
        const uint32_t off = a.tile_offsets[tile], ml = a.tile_max_lens[tile];
        const uint32_t begin = __shfl_sync(kFull, off, 0), t0 = __shfl_sync(kFull, tile, 0);
        uint32_t stA = kRansL, stB = kRansL;
        if (live) {
            stA = a.states[(size_t)tile * WB + lc];
            stB = a.states[(size_t)tile * WB + TW + lc];
        }
        const uint32_t win_s = wbase_s + stage * p.stage_bytes;
        const uint32_t man_s = win_s + p.win_cap + (tile - t0) * man_tile + lc;
        uint32_t posA = win_s + (off - begin) + lc, posB;
        if (live) posA += (ml - 1) * WB;
        posB = posA + TW;
        const uint32_t row0 = tk * g.th, remain = g.K - row0;
        const uint32_t nA = min(remain, g.half), nB = remain > g.half ? min(remain - g.half, g.half) : 0;

        const bool ok = mbar_wait_warp(bar_base + stage * 8, stage ? parity1 : parity0);
        if (stage) parity1 ^= 1; else parity0 ^= 1;
        if (ok) {
            uint8_t *o8 = reinterpret_cast<uint8_t *>(out);
            uint16_t *o16 = reinterpret_cast<uint16_t *>(out);
            size_t oA = (size_t)row0 * g.N + n, oB = oA + (size_t)g.half * g.N;
            uint32_t i = 0;
            for (; i + 8 <= nB; i += 8) {                        // eight rows of both halves, no bounds tests
                const uint32_t mA = man_s + i * TW, mB = mA + g.half * TW;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    uint32_t ma = 0, mb = 0;
                    if (BF16) { ma = lds_u8(mA + r * TW); mb = lds_u8(mB + r * TW); }
                    const uint32_t ba = lds_u8(posA), bb = lds_u8(posB);
                    const uint32_t e = decode_fast(stA, lut_s);
                    const uint32_t f = decode_fast(stB, lut_s);
                    renorm_spec<WB>(stA, posA, ba);
                    renorm_spec<WB>(stB, posB, bb);
                    if (live) {
                        if (BF16) {
                            o16[oA] = (uint16_t)weight_bits(e, ma);
                            o16[oB] = (uint16_t)weight_bits(f, mb);
                        } else {
                            o8[oA] = (uint8_t)lut_sym(e);
                            o8[oB] = (uint8_t)lut_sym(f);
                        }
                    }
                    oA += g.N;
                    oB += g.N;
                }
            }
            for (; i < nA; ++i) {                                // ragged end of the last tile row
                {
                    const uint32_t e = decode_fast(stA, lut_s);
                    renorm_fast<WB>(stA, posA);
                    renorm_fast<WB>(stA, posA);
                    if (live) {
                        if (BF16) o16[oA] = (uint16_t)weight_bits(e, lds_u8(man_s + i * TW));
                        else o8[oA] = (uint8_t)lut_sym(e);
                    }
                }
                if (i < nB) {
                    const uint32_t f = decode_fast(stB, lut_s);
                    renorm_fast<WB>(stB, posB);
                    renorm_fast<WB>(stB, posB);
                    if (live) {
                        if (BF16) o16[oB] = (uint16_t)weight_bits(f, lds_u8(man_s + (g.half + i) * TW));
                        else o8[oB] = (uint8_t)lut_sym(f);
                    }
                }
                oA += g.N;
                oB += g.N;
            }
        }
        __syncwarp();
        stage ^= 1;
    }
}

template <uint32_t TW, bool BF16>
static int launch_tw(const StagedDecArgs &p, uint32_t blocks, uint32_t warps, size_t smem, int max_smem, void *out,
                     cudaStream_t s) {
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_decode_staged<TW, BF16>, (size_t)max_smem)) return rc;
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
    CI_CUDA(cudaLaunchKernelEx(&cfg, k_decode_staged<TW, BF16>, p, out));
    return CI_OK;
}

int launch_decode_staged(const DecArgs &a, uint32_t max_tile_len, bool bf16, void *out, cudaStream_t s) {
    const Geom &g = a.g;
    if (!(g.tw == 8 || g.tw == 16 || g.tw == 32) || max_tile_len == 0 || !a.stream_aligned) return 1;
    if (bf16 && (reinterpret_cast<uintptr_t>(a.mantissa) & 15u)) return 1;
    if ((g.th * g.tw) % 16 != 0 || g.th * g.W > kLutBytes) return 1;    // see the note on stream cursors in ptx.cuh
    int dev = 0, max_smem = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    StagedDecArgs p;
    p.a = a;
    p.win_cap = ((max_tile_len * 64u + 15u) & ~15u) + 16u;
    p.stage_bytes = p.win_cap + (bf16 ? g.th * 32u : 0u);
    p.warp_bytes = (2 * p.stage_bytes + 127u) & ~127u;
    const uint32_t fixed = kLutBytes + 256;
    if ((uint32_t)max_smem < fixed + 4 * p.warp_bytes) return 1;
    uint32_t warps = ((uint32_t)max_smem - fixed) / p.warp_bytes;
    if (warps > 16) warps = 16;
    p.total = g.tiles_k * g.groups;
    const uint32_t P = (uint32_t)sm_count();
    uint32_t blocks = (p.total + warps - 1) / warps;
    if (blocks > P) blocks = P;
    const size_t smem = fixed + (size_t)warps * p.warp_bytes;
    if (g.tw == 32) return bf16 ? launch_tw<32, true>(p, blocks, warps, smem, max_smem, out, s)
                                : launch_tw<32, false>(p, blocks, warps, smem, max_smem, out, s);
    if (g.tw == 16) return bf16 ? launch_tw<16, true>(p, blocks, warps, smem, max_smem, out, s)
                                : launch_tw<16, false>(p, blocks, warps, smem, max_smem, out, s);
    return bf16 ? launch_tw<8, true>(p, blocks, warps, smem, max_smem, out, s)
                : launch_tw<8, false>(p, blocks, warps, smem, max_smem, out, s);
}

}  // namespace ci
