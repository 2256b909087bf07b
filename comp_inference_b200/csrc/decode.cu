// Stand-alone decoders: exponent plane (u8) and full bf16 weight.
//
// One warp owns 32 adjacent columns of one tile row, i.e. 64 independent rANS
// streams (top-half "A" and bottom-half "B" stream per column), two per lane, so
// every lane advances two dependency chains at once.  The 4096-entry merged
// decode table lives in shared memory (one lookup per symbol instead of the
// reference's two dependent global loads, comp_inference/rans_triton.py:95-105);
// the tile's compressed bytes are pulled into a per-warp shared-memory window
// with 16-byte loads before decoding, so renormalisation never touches global
// memory.  Tiles whose byte block does not fit the window fall back to cached
// global byte loads inside the same kernel.
#include "decode.cuh"

namespace ci {

constexpr int kDecWarps = 8;           // warps per CTA
constexpr uint32_t kStageBytes = 4096; // per-warp window for compressed bytes


// Lane-level description of one 32-column task.
struct LaneTask {
    uint32_t n;        // global column
    uint32_t t;        // tile id (clamped to a valid tile for dead lanes)
    uint32_t lc;       // column inside the tile
    uint32_t off, ml;  // tile byte offset and depth
    bool live;         // column < N
};

__device__ __forceinline__ LaneTask lane_task(const DecArgs &a, uint32_t tk, uint32_t grp) {
    LaneTask L;
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

// Copies the byte range the warp's tiles occupy into its shared-memory window.
// Returns true (warp-uniform) when staged; `begin` is the range start in the stream.
__device__ __forceinline__ bool stage_bytes(const DecArgs &a, const LaneTask &L, uint8_t *win, uint32_t &begin) {
    begin = __shfl_sync(kFull, L.off, 0);
    uint32_t end = __shfl_sync(kFull, L.off + L.ml * a.g.W, 31);
    uint32_t bytes = end - begin;
    bool ok = a.stream_aligned && a.g.tw >= 8 && a.g.tw <= 32 && bytes <= kStageBytes;
    if (!ok) return false;
    const uint4 *src = reinterpret_cast<const uint4 *>(a.stream + begin);   // begin is a multiple of 2*tw >= 16
    uint4 *dst = reinterpret_cast<uint4 *>(win);
    for (uint32_t i = lane_id(); i < bytes / 16; i += 32) dst[i] = __ldg(src + i);
    __syncwarp();
    return true;
}

template <bool BF16>
__device__ __forceinline__ void emit(const DecArgs &a, const LaneTask &L, void *out, uint32_t row, uint32_t lr,
                                     uint32_t entry) {
    size_t o = (size_t)row * a.g.N + L.n;
    uint32_t sym = lut_sym(entry);
    if (BF16) {
        uint32_t m = __ldg(a.mantissa + (size_t)L.t * a.g.th * a.g.tw + (size_t)lr * a.g.tw + L.lc);
        reinterpret_cast<uint16_t *>(out)[o] = (uint16_t)assemble_bf16(sym, m);
    } else {
        reinterpret_cast<uint8_t *>(out)[o] = (uint8_t)sym;
    }
}

template <bool BF16>
__global__ void __launch_bounds__(kDecWarps * 32) k_decode_tiled(DecArgs a, void *out, uint32_t n_tasks) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem);
    uint8_t *win = smem + kProbScale * 4 + (threadIdx.x / 32) * kStageBytes;
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();

    const uint32_t warp = blockIdx.x * kDecWarps + threadIdx.x / 32, n_warps = gridDim.x * kDecWarps;
    for (uint32_t task = warp; task < n_tasks; task += n_warps) {
        uint32_t tk = task / a.g.groups, grp = task % a.g.groups;
        LaneTask L = lane_task(a, tk, grp);
        uint32_t row0 = tk * a.g.th;
        uint32_t remain = a.g.K - row0;                        // rows left from the tile's first row
        uint32_t nA = min(remain, a.g.half), nB = remain > a.g.half ? min(remain - a.g.half, a.g.half) : 0;
        uint32_t stA = kRansL, stB = kRansL;
        if (L.live) {
            stA = a.states[(size_t)L.t * a.g.W + L.lc];
            stB = a.states[(size_t)L.t * a.g.W + a.g.tw + L.lc];
        }
        uint32_t begin;
        __syncwarp();                                           // previous task's window reads are done
        if (stage_bytes(a, L, win, begin)) {
            SmemCursor cA, cB;
            cA.low = L.off - begin + L.lc;
            cB.low = cA.low + a.g.tw;
            cA.pos = cA.low + (L.ml - 1) * a.g.W;
            cB.pos = cB.low + (L.ml - 1) * a.g.W;
            if (!L.live) { cA.pos = cA.low - a.g.W; cB.pos = cB.low - a.g.W; }
            for (uint32_t i = 0; i < nA; ++i) {
                uint32_t eA = decode_symbol(stA, s_lut);
                renorm_smem(stA, cA, win, a.g.W);
                if (L.live) emit<BF16>(a, L, out, row0 + i, i, eA);
                if (i < nB) {
                    uint32_t eB = decode_symbol(stB, s_lut);
                    renorm_smem(stB, cB, win, a.g.W);
                    if (L.live) emit<BF16>(a, L, out, row0 + a.g.half + i, a.g.half + i, eB);
                }
            }
        } else {
            GmemCursor cA, cB;
            cA.base = a.stream + L.off + L.lc;
            cB.base = cA.base + a.g.tw;
            cA.row = cB.row = L.live ? (int32_t)L.ml - 1 : -1;
            for (uint32_t i = 0; i < nA; ++i) {
                uint32_t eA = decode_symbol(stA, s_lut);
                renorm_gmem(stA, cA, a.g.W);
                if (L.live) emit<BF16>(a, L, out, row0 + i, i, eA);
                if (i < nB) {
                    uint32_t eB = decode_symbol(stB, s_lut);
                    renorm_gmem(stB, cB, a.g.W);
                    if (L.live) emit<BF16>(a, L, out, row0 + a.g.half + i, a.g.half + i, eB);
                }
            }
        }
    }
}

// Dense layout: one stream per (tile, column), bytes contiguous per stream and
// read backwards from its last byte (comp_inference/linear_triton.py:1099-1170).
struct DenseArgs {
    const uint8_t *stream;
    const uint32_t *states, *sizes, *offsets, *tables, *lut;
    const uint8_t *slot_map, *mantissa;
    Geom g;
};

template <bool BF16>
__global__ void __launch_bounds__(256) k_decode_dense(DenseArgs a, void *out) {
    __shared__ uint32_t s_lut[kProbScale];
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    uint32_t slot = blockIdx.x * blockDim.x + threadIdx.x, tk = blockIdx.y;
    uint32_t padded = a.g.tiles_n * a.g.tw;
    bool live = slot < a.g.N;
    uint32_t tn = min(slot, padded - 1) / a.g.tw, lc = slot % a.g.tw;
    size_t t = (size_t)tk * a.g.tiles_n + tn, sid = t * a.g.tw + lc;
    uint32_t state = kRansL;
    GmemCursor c;
    c.base = a.stream;
    c.row = -1;
    if (live) {
        state = a.states[sid];
        c.base = a.stream + a.offsets[sid];
        c.row = (int32_t)a.sizes[sid] - 1;
    }
    uint32_t row0 = tk * a.g.th, rows = min(a.g.th, a.g.K - row0);
    for (uint32_t i = 0; i < rows; ++i) {
        uint32_t e = decode_symbol(state, s_lut);
        renorm_gmem(state, c, 1);
        if (live) {
            size_t o = (size_t)(row0 + i) * a.g.N + slot;
            uint32_t sym = lut_sym(e);
            if (BF16) {
                uint32_t m = __ldg(a.mantissa + t * a.g.th * a.g.tw + (size_t)i * a.g.tw + lc);
                reinterpret_cast<uint16_t *>(out)[o] = (uint16_t)assemble_bf16(sym, m);
            } else {
                reinterpret_cast<uint8_t *>(out)[o] = (uint8_t)sym;
            }
        }
    }
}

// Legacy flat layout.  seg_rows == 0: stream g yields flat indices g, g + num_streams, ...
// (src/cuda/rans_kernels.cuh:626-708).  seg_rows > 0: stream g yields rows [seg * seg_rows, +seg_rows) of
// column g % cols, seg = g / cols, of a row-major [rows, cols] plane with rows * cols = output_len
// (comp_inference/rans_triton.py:171-233, the order the reference's legacy encoder writes,
// src/cuda/rans_kernels.cuh:393-509).
__global__ void __launch_bounds__(256) k_decode_legacy(const uint8_t *__restrict__ stream,
                                                       const uint32_t *__restrict__ states,
                                                       const uint32_t *__restrict__ sizes, uint32_t num_streams,
                                                       uint64_t output_len, const uint32_t *__restrict__ tables,
                                                       const uint8_t *__restrict__ slot_map,
                                                       uint8_t *__restrict__ out, uint32_t cols, uint32_t seg_rows) {
    __shared__ uint32_t s_lut[kProbScale];
    load_lut(s_lut, nullptr, tables, slot_map);
    __syncthreads();
    uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    bool live = gid < num_streams;
    uint32_t state = kRansL;
    GmemCursor c;
    c.base = stream;
    c.row = -1;
    if (live) { state = states[gid]; c.base = stream + gid; c.row = (int32_t)sizes[gid] - 1; }
    if (seg_rows != 0) {
        const uint64_t col = gid % cols, row0 = (uint64_t)(gid / cols) * seg_rows, rows = output_len / cols;
        const uint64_t n = (live && row0 < rows) ? (rows - row0 < seg_rows ? rows - row0 : seg_rows) : 0;
        // every lane walks the warp's longest run: renorm_gmem votes warp-wide
        const uint64_t n_warp = __reduce_max_sync(kFull, (uint32_t)n);
        for (uint64_t i = 0; i < n_warp; ++i) {
            uint32_t e = decode_symbol(state, s_lut);
            if (i >= n) c.row = -1;
            renorm_gmem(state, c, num_streams);
            if (i < n) out[(row0 + i) * cols + col] = (uint8_t)lut_sym(e);
        }
        return;
    }
    uint64_t per_stream = (output_len + num_streams - 1) / num_streams;
    for (uint64_t i = 0; i < per_stream; ++i) {
        uint32_t e = decode_symbol(state, s_lut);
        renorm_gmem(state, c, num_streams);
        uint64_t o = (uint64_t)gid + i * num_streams;
        if (live && o < output_len) out[o] = (uint8_t)lut_sym(e);
    }
}

static DecArgs make_args(const ci_tiled_weight *w) {
    DecArgs a;
    a.stream = w->stream; a.states = w->states; a.tables = w->tables; a.tile_offsets = w->tile_offsets;
    a.tile_max_lens = w->tile_max_lens; a.lut = w->lut; a.slot_map = w->slot_map; a.mantissa = w->mantissa;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    a.stream_aligned = (reinterpret_cast<uintptr_t>(w->stream) & 15u) == 0;
    return a;
}

template <bool BF16>
static int decode_tiled(const ci_tiled_weight *w, void *d_out, cudaStream_t s) {
    int rc = check_weight(w, BF16);
    if (rc) return rc;
    CI_REQUIRE(d_out != nullptr, "null output");
    DecArgs a = make_args(w);
    rc = launch_decode4(a, w->max_tile_len, BF16, d_out, s);         // 32-wide tiles, whole tile rows
    if (rc <= 0) return rc;
    rc = launch_decode_staged(a, w->max_tile_len, BF16, d_out, s);   // other staged shapes
    if (rc <= 0) return rc;
    uint32_t n_tasks = a.g.tiles_k * a.g.groups;
    size_t smem = kProbScale * 4 + (size_t)kDecWarps * kStageBytes;
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_decode_tiled<BF16>, smem)) return rc;
    uint32_t blocks = (n_tasks + kDecWarps - 1) / kDecWarps;
    uint32_t cap = (uint32_t)sm_count() * 4;
    if (blocks > cap) blocks = cap;
    k_decode_tiled<BF16><<<blocks, kDecWarps * 32, smem, s>>>(a, d_out, n_tasks);
    CI_LAUNCH_CHECK(k_decode_tiled);
    return CI_OK;
}

template <bool BF16>
static int decode_dense(const ci_dense_weight *w, void *d_out, cudaStream_t s) {
    CI_REQUIRE(w && d_out, "null pointer");
    int rc = check_tile(w->K, w->N, w->tile_h, w->tile_w);
    if (rc) return rc;
    CI_REQUIRE(w->states && w->stream_sizes && w->stream_offsets, "null metadata pointer");
    CI_REQUIRE(w->lut || (w->tables && w->slot_map), "neither a prepared table nor tables + slot_map given");
    CI_REQUIRE(!BF16 || w->mantissa, "mantissa plane required");
    DenseArgs a;
    a.stream = w->stream; a.states = w->states; a.sizes = w->stream_sizes; a.offsets = w->stream_offsets;
    a.tables = w->tables; a.lut = w->lut; a.slot_map = w->slot_map; a.mantissa = w->mantissa;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    dim3 grid((a.g.tiles_n * a.g.tw + 255) / 256, a.g.tiles_k);
    k_decode_dense<BF16><<<grid, 256, 0, s>>>(a, d_out);
    CI_LAUNCH_CHECK(k_decode_dense);
    return CI_OK;
}

}  // namespace ci

using namespace ci;

extern "C" {

int ci_decode_plane(const ci_tiled_weight *w, uint8_t *d_out, ci_stream_t stream) {
    return decode_tiled<false>(w, d_out, (cudaStream_t)stream);
}
int ci_decode_bf16(const ci_tiled_weight *w, uint16_t *d_out, ci_stream_t stream) {
    return decode_tiled<true>(w, d_out, (cudaStream_t)stream);
}
int ci_decode_plane_dense(const ci_dense_weight *w, uint8_t *d_out, ci_stream_t stream) {
    return decode_dense<false>(w, d_out, (cudaStream_t)stream);
}
int ci_decode_bf16_dense(const ci_dense_weight *w, uint16_t *d_out, ci_stream_t stream) {
    return decode_dense<true>(w, d_out, (cudaStream_t)stream);
}

int ci_decode_legacy(const uint8_t *d_stream, uint64_t stream_len, const uint32_t *d_states, const uint32_t *d_sizes,
                     uint32_t num_streams, uint64_t output_len, const uint32_t *d_tables, const uint8_t *d_slot_map,
                     uint8_t *d_out, ci_stream_t stream) {
    (void)stream_len;
    CI_REQUIRE(d_states && d_sizes && d_tables && d_slot_map && d_out, "null pointer");
    CI_REQUIRE(num_streams > 0, "no streams");
    k_decode_legacy<<<(num_streams + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        d_stream, d_states, d_sizes, num_streams, output_len, d_tables, d_slot_map, d_out, 1, 0);
    CI_LAUNCH_CHECK(k_decode_legacy);
    return CI_OK;
}

int ci_decode_legacy_segments(const uint8_t *d_stream, uint64_t stream_len, const uint32_t *d_states,
                              const uint32_t *d_sizes, uint32_t num_streams, uint32_t rows, uint32_t cols,
                              uint32_t seg_rows, const uint32_t *d_tables, const uint8_t *d_slot_map, uint8_t *d_out,
                              ci_stream_t stream) {
    (void)stream_len;
    CI_REQUIRE(d_states && d_sizes && d_tables && d_slot_map && d_out, "null pointer");
    CI_REQUIRE(rows > 0 && cols > 0 && seg_rows > 0, "empty plane or zero segment height");
    CI_REQUIRE((uint64_t)num_streams == (uint64_t)((rows + seg_rows - 1) / seg_rows) * cols,
               "%u streams, ceil(%u / %u) * %u expected", num_streams, rows, seg_rows, cols);
    k_decode_legacy<<<(num_streams + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        d_stream, d_states, d_sizes, num_streams, (uint64_t)rows * cols, d_tables, d_slot_map, d_out, cols, seg_rows);
    CI_LAUNCH_CHECK(k_decode_legacy);
    return CI_OK;
}

}  // extern "C"
