// Fused decode + row gather: out[i,:] = W[ids[i],:].
//
// Replaces fused_rans_embedding_kernel_ilp2 (comp_inference/embedding_triton.py:170-275).
// A stream cannot be entered in the middle, so the warp that owns (token, 32
// columns) opens the row's half-tile streams and discards the symbols of the rows
// above it.  Only the bytes those skipped rows consume are touched, straight from
// L2/global memory; ids outside [0,K) produce a zero row (embedding_triton.py:203-210).
#include "embedding.cuh"

namespace ci {

constexpr int kEmbWarps = 8;

__global__ void __launch_bounds__(kEmbWarps * 32) k_embedding(EmbArgs a) {
    __shared__ uint32_t s_lut[kProbScale];
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    const uint64_t n_tasks = a.n_ids * a.g.groups;
    const uint64_t warp = (uint64_t)blockIdx.x * kEmbWarps + threadIdx.x / 32, n_warps = (uint64_t)gridDim.x * kEmbWarps;
    for (uint64_t task = warp; task < n_tasks; task += n_warps) {
        const uint64_t tok_i = task / a.g.groups;
        const uint32_t grp = (uint32_t)(task % a.g.groups);
        const uint32_t n = grp * 32 + lane_id();
        const bool live = n < a.g.N;
        const int64_t tok = a.ids[tok_i];
        uint16_t *dst = a.out + tok_i * a.ldo + n;
        if (tok < 0 || tok >= (int64_t)a.g.K) {                 // warp-uniform
            if (live) *dst = 0;
            continue;
        }
        const uint32_t tk = (uint32_t)(tok / a.g.th), rel = (uint32_t)(tok % a.g.th);
        const bool bottom = rel >= a.g.half;
        const uint32_t inner = rel % a.g.half;                  // symbols to discard
        uint32_t tn = n / a.g.tw;
        if (tn >= a.g.tiles_n) tn = a.g.tiles_n - 1;
        const uint32_t lc = n % a.g.tw, j = lc + (bottom ? a.g.tw : 0);
        const size_t t = (size_t)tk * a.g.tiles_n + tn;
        uint32_t state = kRansL;
        GmemCursor c;
        c.base = a.stream + a.tile_offsets[t] + j;
        c.row = -1;
        if (live) { state = a.states[t * a.g.W + j]; c.row = (int32_t)a.tile_max_lens[t] - 1; }
        for (uint32_t s = 0; s < inner; ++s) {
            decode_symbol(state, s_lut);
            renorm_gmem(state, c, a.g.W);
        }
        uint32_t sym = lut_sym(s_lut[state & kProbMask]);
        if (live) {
            uint32_t m = __ldg(a.mantissa + t * a.g.th * a.g.tw + (size_t)rel * a.g.tw + lc);
            *dst = (uint16_t)assemble_bf16(sym, m);
        }
    }
}

// Dense layout (comp_inference/embedding_triton.py:333-428): one stream per tile
// column over the full tile height, so `rel` symbols are discarded.
struct EmbDenseArgs {
    const uint8_t *stream;
    const uint32_t *states, *sizes, *offsets, *tables, *lut;
    const uint8_t *slot_map, *mantissa;
    Geom g;
    const int64_t *ids;
    uint64_t n_ids;
    uint16_t *out;
    int64_t ldo;
};

__global__ void __launch_bounds__(kEmbWarps * 32) k_embedding_dense(EmbDenseArgs a) {
    __shared__ uint32_t s_lut[kProbScale];
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    const uint64_t n_tasks = a.n_ids * a.g.groups;
    const uint64_t warp = (uint64_t)blockIdx.x * kEmbWarps + threadIdx.x / 32, n_warps = (uint64_t)gridDim.x * kEmbWarps;
    for (uint64_t task = warp; task < n_tasks; task += n_warps) {
        const uint64_t tok_i = task / a.g.groups;
        const uint32_t grp = (uint32_t)(task % a.g.groups);
        const uint32_t n = grp * 32 + lane_id();
        const bool live = n < a.g.N;
        const int64_t tok = a.ids[tok_i];
        uint16_t *dst = a.out + tok_i * a.ldo + n;
        if (tok < 0 || tok >= (int64_t)a.g.K) {
            if (live) *dst = 0;
            continue;
        }
        const uint32_t tk = (uint32_t)(tok / a.g.th), rel = (uint32_t)(tok % a.g.th);
        uint32_t tn = n / a.g.tw;
        if (tn >= a.g.tiles_n) tn = a.g.tiles_n - 1;
        const uint32_t lc = n % a.g.tw;
        const size_t t = (size_t)tk * a.g.tiles_n + tn, sid = t * a.g.tw + lc;
        uint32_t state = kRansL;
        GmemCursor c;
        c.base = a.stream;
        c.row = -1;
        if (live) { state = a.states[sid]; c.base = a.stream + a.offsets[sid]; c.row = (int32_t)a.sizes[sid] - 1; }
        for (uint32_t s = 0; s < rel; ++s) {
            decode_symbol(state, s_lut);
            renorm_gmem(state, c, 1);
        }
        uint32_t sym = lut_sym(s_lut[state & kProbMask]);
        if (live) {
            uint32_t m = __ldg(a.mantissa + t * a.g.th * a.g.tw + (size_t)rel * a.g.tw + lc);
            *dst = (uint16_t)assemble_bf16(sym, m);
        }
    }
}

}  // namespace ci

using namespace ci;

extern "C" {

int ci_embedding(const ci_tiled_weight *w, const int64_t *d_ids, uint64_t n_ids, uint16_t *d_out, int64_t ldo,
                 ci_stream_t stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (n_ids == 0) return CI_OK;
    CI_REQUIRE(d_ids && d_out, "null pointer");
    CI_REQUIRE(ldo >= (int64_t)w->N, "output row stride smaller than the row length");
    EmbArgs a;
    a.stream = w->stream; a.states = w->states; a.tables = w->tables; a.tile_offsets = w->tile_offsets;
    a.tile_max_lens = w->tile_max_lens; a.lut = w->lut; a.slot_map = w->slot_map; a.mantissa = w->mantissa;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    a.ids = d_ids; a.n_ids = n_ids; a.out = d_out; a.ldo = ldo;
    rc = launch_embedding4(a, w->max_tile_len, (cudaStream_t)stream);  // 32-wide tiles: four streams per lane
    if (rc <= 0) return rc;
    uint64_t tasks = n_ids * a.g.groups, blocks = (tasks + kEmbWarps - 1) / kEmbWarps, cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    k_embedding<<<(uint32_t)blocks, kEmbWarps * 32, 0, (cudaStream_t)stream>>>(a);
    CI_LAUNCH_CHECK(k_embedding);
    return CI_OK;
}

int ci_embedding_dense(const ci_dense_weight *w, const int64_t *d_ids, uint64_t n_ids, uint16_t *d_out, int64_t ldo,
                       ci_stream_t stream) {
    CI_REQUIRE(w != nullptr, "null weight descriptor");
    int rc = check_tile(w->K, w->N, w->tile_h, w->tile_w);
    if (rc) return rc;
    if (n_ids == 0) return CI_OK;
    CI_REQUIRE(d_ids && d_out && w->states && w->stream_sizes && w->stream_offsets && w->mantissa, "null pointer");
    CI_REQUIRE(w->lut || (w->tables && w->slot_map), "neither a prepared table nor tables + slot_map given");
    CI_REQUIRE(ldo >= (int64_t)w->N, "output row stride smaller than the row length");
    EmbDenseArgs a;
    a.stream = w->stream; a.states = w->states; a.sizes = w->stream_sizes; a.offsets = w->stream_offsets;
    a.tables = w->tables; a.lut = w->lut; a.slot_map = w->slot_map; a.mantissa = w->mantissa;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    a.ids = d_ids; a.n_ids = n_ids; a.out = d_out; a.ldo = ldo;
    uint64_t tasks = n_ids * a.g.groups, blocks = (tasks + kEmbWarps - 1) / kEmbWarps, cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    k_embedding_dense<<<(uint32_t)blocks, kEmbWarps * 32, 0, (cudaStream_t)stream>>>(a);
    CI_LAUNCH_CHECK(k_embedding_dense);
    return CI_OK;
}

}  // extern "C"
