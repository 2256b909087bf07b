// Shared declarations of the fused decode + linear kernels.
#pragma once
#include "common.cuh"
#include "ar_fuse.cuh"

namespace ci {

constexpr int kLinWarps = 8;
constexpr uint32_t kLinStage = 4096;     // per-warp compressed-byte window
constexpr uint32_t kMaxSplits = 16;
constexpr uint32_t kTicketBytes = 4096;  // number of u32 ticket counters at the head of the workspace

struct LinArgs {
    const uint8_t *stream;
    const uint32_t *states, *tables, *tile_offsets, *tile_max_lens, *lut;
    const uint8_t *slot_map, *mantissa;
    Geom g;
    uint32_t stream_aligned;
    const uint16_t *x;
    int64_t ldx;
    const uint16_t *bias;
    uint16_t *y;
    int64_t ldy;
    uint32_t M;
    uint32_t splits, tiles_per_split;
    const uint32_t *dense_sizes, *dense_offsets;   // dense layout only
    uint32_t *tickets;   // [items along the non-reduced dimension]
    float *partial;      // [splits][M][n_out]
    ArFuse ar;           // ar.world > 1: all-reduce the output over the ranks inside the kernel (M <= 2)
    uint32_t dry_run;    // launchers stop before the launch: "would this weight take the staged route?"
};

struct LaneTile {
    uint32_t n, t, lc, off, ml;
    bool live;
};

__device__ __forceinline__ LaneTile lane_tile(const LinArgs &a, uint32_t tk, uint32_t grp) {
    LaneTile L;
    L.n = grp * 32 + lane_id();
    uint32_t tn = L.n / a.g.tw;
    L.live = L.n < a.g.N;
    if (tn >= a.g.tiles_n) tn = a.g.tiles_n - 1;
    L.lc = L.n % a.g.tw;
    L.t = tk * a.g.tiles_n + tn;
    L.off = a.tile_offsets[L.t];
    L.ml = a.tile_max_lens[L.t];
    return L;
}

__device__ __forceinline__ bool stage_tile_bytes(const LinArgs &a, const LaneTile &L, uint8_t *win, uint32_t &begin) {
    begin = __shfl_sync(kFull, L.off, 0);
    uint32_t end = __shfl_sync(kFull, L.off + L.ml * a.g.W, 31);
    uint32_t bytes = end - begin;
    bool ok = a.stream_aligned && a.g.tw >= 8 && a.g.tw <= 32 && bytes <= kLinStage;
    if (!ok) return false;
    const uint4 *src = reinterpret_cast<const uint4 *>(a.stream + begin);
    uint4 *dst = reinterpret_cast<uint4 *>(win);
    for (uint32_t i = lane_id(); i < bytes / 16; i += 32) dst[i] = __ldg(src + i);
    __syncwarp();
    return true;
}

// Streams of one lane over one tile, with the byte source abstracted.
struct TileStreams {
    uint32_t stA, stB;
    bool staged;
    SmemCursor sA, sB;
    GmemCursor gA, gB;
    const uint8_t *win;
    uint32_t W;
};

__device__ __forceinline__ void open_streams(const LinArgs &a, const LaneTile &L, uint8_t *win, TileStreams &S) {
    S.stA = S.stB = kRansL;
    if (L.live) {
        S.stA = a.states[(size_t)L.t * a.g.W + L.lc];
        S.stB = a.states[(size_t)L.t * a.g.W + a.g.tw + L.lc];
    }
    S.W = a.g.W;
    S.win = win;
    uint32_t begin;
    __syncwarp();
    S.staged = stage_tile_bytes(a, L, win, begin);
    if (S.staged) {
        S.sA.low = L.off - begin + L.lc;
        S.sB.low = S.sA.low + a.g.tw;
        uint32_t top = L.live ? (L.ml - 1) * a.g.W : 0u - a.g.W;
        S.sA.pos = S.sA.low + top;
        S.sB.pos = S.sB.low + top;
    } else {
        S.gA.base = a.stream + L.off + L.lc;
        S.gB.base = S.gA.base + a.g.tw;
        S.gA.row = S.gB.row = L.live ? (int32_t)L.ml - 1 : -1;
    }
}

__device__ __forceinline__ uint32_t next_A(TileStreams &S, const uint32_t *s_lut) {
    uint32_t e = decode_symbol(S.stA, s_lut);
    if (S.staged) renorm_smem(S.stA, S.sA, S.win, S.W); else renorm_gmem(S.stA, S.gA, S.W);
    return lut_sym(e);
}
__device__ __forceinline__ uint32_t next_B(TileStreams &S, const uint32_t *s_lut) {
    uint32_t e = decode_symbol(S.stB, s_lut);
    if (S.staged) renorm_smem(S.stB, S.sB, S.win, S.W); else renorm_gmem(S.stB, S.gB, S.W);
    return lut_sym(e);
}

__device__ __forceinline__ float load_bf16(const uint16_t *p) { return __uint_as_float((uint32_t)__ldg(p) << 16); }

// Draws a ticket for `slot`; returns true in the CTA that arrived last.  All
// partial sums of this CTA must have been written before the call.
__device__ __forceinline__ bool last_arrival(uint32_t *ticket, uint32_t expected, uint32_t *s_flag) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t old = atomicAdd(ticket, 1u);
        *s_flag = (old == expected - 1u);
    }
    __syncthreads();
    bool last = *s_flag != 0;
    if (last) __threadfence();
    return last;
}


// Staged tensor-core path (linear_mma.cu).  Returns CI_OK when it launched, 1 when the
// weight does not qualify (the caller then uses the generic kernel), < 0 on error.
int launch_linear_mma(const LinArgs &a, uint32_t max_tile_len, cudaStream_t s);
// Register-direct variant for 32-wide tiles and K a multiple of the tile height (linear_mma4.cu).
int launch_linear_mma4(const LinArgs &a, uint32_t max_tile_len, cudaStream_t s);

// tcgen05 decode-GEMM for many activation rows (gemm_sm100.cu); same return convention.
// partial_capacity = bytes available behind a.partial for split-K partial sums.
int launch_linear_gemm(const LinArgs &a, uint32_t max_tile_len, size_t partial_capacity, uint32_t split_k,
                       cudaStream_t s);
size_t gemm_workspace_bytes(uint32_t M, uint32_t N, uint32_t K, uint32_t th);

}  // namespace ci
