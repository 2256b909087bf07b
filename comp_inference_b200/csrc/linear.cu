// Fused decode + linear for small activation batches (decode-time GEMV, M <= 16
// per pass): the weight is decoded tile by tile into registers and multiplied
// at once; the dense matrix never exists in global memory.
//
//  * k_linear            y[M,N] = x[M,K] . W[K,N]         (replaces linear_triton.py:317-552)
//  * k_linear_transposed y[M,V] = x[M,H] . W[V,H]^T       (replaces transposed_linear_triton.py:187-358)
//
// Work split.  A 32-column group of one tile row is one warp task (64 streams, two
// per lane).  A CTA of 8 warps walks a contiguous run of K tiles of one column
// group (split-K over CTAs), keeps fp32 accumulators in registers, reduces the 8
// warps through shared memory and either stores the result directly or writes an
// fp32 partial; the CTA that draws the last ticket of a column group sums the
// partials in a fixed order, so results are deterministic (the reference writes
// bf16 partials and sums them with a second kernel, linear_triton.py:302-314).
#include "linear.cuh"

namespace ci {

// CTA-level tail shared by the tiled and dense kernels: sums the 8 warps' register
// accumulators through shared memory, then stores bf16 (+bias) or goes through the
// ticketed split-K reduction.
template <int MT>
__device__ __forceinline__ void reduce_and_store(const LinArgs &a, float (&acc)[MT], uint32_t grp, uint32_t split,
                                                 float *s_red, uint32_t *s_flag) {
    const uint32_t warp = threadIdx.x / 32, lane = lane_id();
    __syncthreads();                                            // every warp is done with its byte window
#pragma unroll
    for (int m = 0; m < MT; ++m) s_red[(warp * MT + m) * 32 + lane] = acc[m];
    __syncthreads();
    const uint32_t n = grp * 32 + lane;
    for (uint32_t m = warp; m < a.M; m += kLinWarps) {          // warp w finishes rows w, w+8, ...
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kLinWarps; ++w) v += s_red[(w * MT + m) * 32 + lane];
        if (a.splits == 1) {
            if (n < a.g.N) {
                if (a.bias) v += load_bf16(a.bias + n);
                a.y[(size_t)m * a.ldy + n] = float_to_bf16_bits(v);
            }
        } else if (n < a.g.N) {
            a.partial[((size_t)split * a.M + m) * a.g.N + n] = v;
        }
    }
    if (a.splits > 1) {
        if (last_arrival(a.tickets + grp, a.splits, s_flag)) {
            for (uint32_t m = warp; m < a.M; m += kLinWarps) {
                if (n < a.g.N) {
                    float v = 0.f;
                    for (uint32_t s = 0; s < a.splits; ++s) v += __ldcg(a.partial + ((size_t)s * a.M + m) * a.g.N + n);
                    if (a.bias) v += load_bf16(a.bias + n);
                    a.y[(size_t)m * a.ldy + n] = float_to_bf16_bits(v);
                }
            }
            if (threadIdx.x == 0) a.tickets[grp] = 0;           // leave the workspace ready for the next call
        }
    }
    __syncthreads();                                            // s_red and the windows may be reused
}

// ------------------------------------------------------------------ y = x . W
template <int MT>
__global__ void __launch_bounds__(kLinWarps * 32) k_linear(LinArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem);
    uint8_t *s_win_all = smem + kProbScale * 4;
    const uint32_t warp = threadIdx.x / 32, lane = lane_id();
    uint8_t *win = s_win_all + warp * kLinStage;
    float *s_red = reinterpret_cast<float *>(s_win_all);       // reused after decoding: [warps][MT][32]
    __shared__ uint32_t s_flag;

    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();

    const uint32_t items = a.g.groups * a.splits;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t grp = item % a.g.groups, split = item / a.g.groups;
        const uint32_t k_begin = split * a.tiles_per_split, k_end = min(k_begin + a.tiles_per_split, a.g.tiles_k);
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;

        for (uint32_t tk = k_begin + warp; tk < k_end; tk += kLinWarps) {
            LaneTile L = lane_tile(a, tk, grp);
            TileStreams S;
            open_streams(a, L, win, S);
            const uint32_t row0 = tk * a.g.th, remain = a.g.K - row0;
            const uint32_t nA = min(remain, a.g.half), nB = remain > a.g.half ? min(remain - a.g.half, a.g.half) : 0;
            const uint8_t *man = a.mantissa + (size_t)L.t * a.g.th * a.g.tw + L.lc;
            const uint16_t *xa = a.x + row0, *xb = a.x + row0 + a.g.half;
            for (uint32_t i = 0; i < nA; ++i) {
                uint32_t symA = next_A(S, s_lut);
                float wA = bf16_bits_to_float(assemble_bf16(symA, __ldg(man + (size_t)i * a.g.tw)));
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < (int)a.M) acc[m] = fmaf(load_bf16(xa + (size_t)m * a.ldx + i), wA, acc[m]);
                if (i < nB) {
                    uint32_t symB = next_B(S, s_lut);
                    float wB = bf16_bits_to_float(assemble_bf16(symB, __ldg(man + (size_t)(a.g.half + i) * a.g.tw)));
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        if (m < (int)a.M) acc[m] = fmaf(load_bf16(xb + (size_t)m * a.ldx + i), wB, acc[m]);
                }
            }
        }

        reduce_and_store<MT>(a, acc, grp, split, s_red, &s_flag);
    }
}

// Dense layout (comp_inference/linear_triton.py:1044-1186): one stream per tile
// column over the whole tile height, bytes contiguous per stream.
template <int MT>
__global__ void __launch_bounds__(kLinWarps * 32) k_linear_dense(LinArgs a) {
    __shared__ uint32_t s_lut[kProbScale];
    __shared__ float s_red[kLinWarps * MT * 32];
    __shared__ uint32_t s_flag;
    const uint32_t warp = threadIdx.x / 32;
    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();
    const uint32_t items = a.g.groups * a.splits;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t grp = item % a.g.groups, split = item / a.g.groups;
        const uint32_t k_begin = split * a.tiles_per_split, k_end = min(k_begin + a.tiles_per_split, a.g.tiles_k);
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;
        for (uint32_t tk = k_begin + warp; tk < k_end; tk += kLinWarps) {
            const uint32_t n = grp * 32 + lane_id();
            const bool live = n < a.g.N;
            uint32_t tn = n / a.g.tw;
            if (tn >= a.g.tiles_n) tn = a.g.tiles_n - 1;
            const uint32_t lc = n % a.g.tw;
            const size_t t = (size_t)tk * a.g.tiles_n + tn, sid = t * a.g.tw + lc;
            uint32_t state = kRansL;
            GmemCursor c;
            c.base = a.stream;
            c.row = -1;
            if (live) { state = a.states[sid]; c.base = a.stream + a.dense_offsets[sid]; c.row = (int32_t)a.dense_sizes[sid] - 1; }
            const uint32_t row0 = tk * a.g.th, rows = min(a.g.th, a.g.K - row0);
            const uint8_t *man = a.mantissa + t * a.g.th * a.g.tw + lc;
            for (uint32_t i = 0; i < rows; ++i) {
                uint32_t e = decode_symbol(state, s_lut);
                renorm_gmem(state, c, 1);
                float wv = bf16_bits_to_float(assemble_bf16(lut_sym(e), __ldg(man + (size_t)i * a.g.tw)));
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < (int)a.M) acc[m] = fmaf(load_bf16(a.x + (size_t)m * a.ldx + row0 + i), wv, acc[m]);
            }
        }
        reduce_and_store<MT>(a, acc, grp, split, s_red, &s_flag);
    }
}

// ------------------------------------------------------- y = x . W^T (LM head)
// W is stored [K = V rows, N = H columns]; a lane owns hidden column h and walks
// vocabulary rows, so every decoded row needs a sum over lanes.  32 rows are
// collected per lane and reduced with a 31-shuffle transpose, after which lane r
// holds the sum for row r.  Per-warp row accumulators live in shared memory.
template <int MT>
__global__ void __launch_bounds__(kLinWarps * 32) k_linear_transposed(LinArgs a, uint32_t groups_per_split) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem);
    uint8_t *s_win_all = smem + kProbScale * 4;
    const uint32_t warp = threadIdx.x / 32, lane = lane_id();
    uint8_t *win = s_win_all + warp * kLinStage;
    float *s_acc_all = reinterpret_cast<float *>(s_win_all + kLinWarps * kLinStage);   // [warps][th][MT]
    float *s_acc = s_acc_all + (size_t)warp * a.g.th * MT;
    __shared__ uint32_t s_flag;

    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();

    const uint32_t items = a.g.tiles_k * a.splits;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t tk = item % a.g.tiles_k, split = item / a.g.tiles_k;
        const uint32_t g_begin = split * groups_per_split, g_end = min(g_begin + groups_per_split, a.g.groups);
        const uint32_t row0 = tk * a.g.th, remain = a.g.K - row0;
        const uint32_t nA = min(remain, a.g.half), nB = remain > a.g.half ? min(remain - a.g.half, a.g.half) : 0;
        for (uint32_t i = lane; i < a.g.th * MT; i += 32) s_acc[i] = 0.f;
        __syncwarp();

        for (uint32_t grp = g_begin + warp; grp < g_end; grp += kLinWarps) {
            LaneTile L = lane_tile(a, tk, grp);
            TileStreams S;
            open_streams(a, L, win, S);
            const uint8_t *man = a.mantissa + (size_t)L.t * a.g.th * a.g.tw + L.lc;
            float xv[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                xv[m] = (L.live && m < (int)a.M) ? load_bf16(a.x + (size_t)m * a.ldx + L.n) : 0.f;
            for (uint32_t c0 = 0; c0 < nA; c0 += 32) {          // 32-row chunks of both halves
                float wA[32], wB[32];                           // this lane's column, 32 rows of each half
#pragma unroll
                for (int r = 0; r < 32; ++r) {
                    wA[r] = 0.f;
                    wB[r] = 0.f;
                    uint32_t i = c0 + r;
                    if (i < nA) {
                        uint32_t symA = next_A(S, s_lut);
                        wA[r] = bf16_bits_to_float(assemble_bf16(symA, __ldg(man + (size_t)i * a.g.tw)));
                    }
                    if (i < nB) {
                        uint32_t symB = next_B(S, s_lut);
                        wB[r] = bf16_bits_to_float(assemble_bf16(symB, __ldg(man + (size_t)(a.g.half + i) * a.g.tw)));
                    }
                }
                const uint32_t i = c0 + lane;                   // after the transpose lane r holds row c0 + r
#pragma unroll
                for (int m = 0; m < MT; ++m) {
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        float p[32];
#pragma unroll
                        for (int r = 0; r < 32; ++r) p[r] = (hb ? wB[r] : wA[r]) * xv[m];
#pragma unroll
                        for (int s = 16; s >= 1; s >>= 1) {
#pragma unroll
                            for (int j = 0; j < s; ++j) {
                                bool up = (lane & s) != 0;
                                float send = up ? p[j] : p[j + s], keep = up ? p[j + s] : p[j];
                                p[j] = keep + __shfl_xor_sync(kFull, send, s);
                            }
                        }
                        if (hb == 0) { if (i < nA) s_acc[(size_t)i * MT + m] += p[0]; }
                        else         { if (i < nB) s_acc[(size_t)(a.g.half + i) * MT + m] += p[0]; }
                    }
                }
                __syncwarp();
            }
        }

        // ---- CTA reduction over warps, then split reduction ------------------
        __syncthreads();
        const uint32_t rows = min(a.g.th, remain);
        for (uint32_t idx = threadIdx.x; idx < rows * a.M; idx += blockDim.x) {
            uint32_t r = idx / a.M, m = idx % a.M;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kLinWarps; ++w) v += s_acc_all[((size_t)w * a.g.th + r) * MT + m];
            uint32_t vrow = row0 + r;
            if (a.splits == 1) {
                if (a.bias) v += load_bf16(a.bias + vrow);
                a.y[(size_t)m * a.ldy + vrow] = float_to_bf16_bits(v);
            } else {
                a.partial[((size_t)split * a.M + m) * a.g.K + vrow] = v;
            }
        }
        if (a.splits > 1) {
            if (last_arrival(a.tickets + tk, a.splits, &s_flag)) {
                for (uint32_t idx = threadIdx.x; idx < rows * a.M; idx += blockDim.x) {
                    uint32_t r = idx / a.M, m = idx % a.M, vrow = row0 + r;
                    float v = 0.f;
                    for (uint32_t s = 0; s < a.splits; ++s) v += __ldcg(a.partial + ((size_t)s * a.M + m) * a.g.K + vrow);
                    if (a.bias) v += load_bf16(a.bias + vrow);
                    a.y[(size_t)m * a.ldy + vrow] = float_to_bf16_bits(v);
                }
                if (threadIdx.x == 0) a.tickets[tk] = 0;
            }
        }
        __syncthreads();
    }
}

// Dense-layout LM head (comp_inference/transposed_linear_triton.py:660-810): W stored [K = V rows, N = H
// columns], one stream per tile column over the whole tile height.  Same scheme as k_linear_transposed:
// a lane walks the vocabulary rows of its hidden column, 32 rows at a time are summed over the lanes
// with the shuffle transpose, per-warp row accumulators live in shared memory.
template <int MT>
__global__ void __launch_bounds__(kLinWarps * 32) k_linear_transposed_dense(LinArgs a, uint32_t groups_per_split) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(smem);
    const uint32_t warp = threadIdx.x / 32, lane = lane_id();
    float *s_acc_all = reinterpret_cast<float *>(smem + kProbScale * 4);                  // [warps][th][MT]
    float *s_acc = s_acc_all + (size_t)warp * a.g.th * MT;
    __shared__ uint32_t s_flag;

    load_lut(s_lut, a.lut, a.tables, a.slot_map);
    __syncthreads();

    const uint32_t items = a.g.tiles_k * a.splits;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t tk = item % a.g.tiles_k, split = item / a.g.tiles_k;
        const uint32_t g_begin = split * groups_per_split, g_end = min(g_begin + groups_per_split, a.g.groups);
        const uint32_t row0 = tk * a.g.th, rows = min(a.g.th, a.g.K - row0);
        for (uint32_t i = lane; i < a.g.th * MT; i += 32) s_acc[i] = 0.f;
        __syncwarp();

        for (uint32_t grp = g_begin + warp; grp < g_end; grp += kLinWarps) {
            const uint32_t n = grp * 32 + lane;
            const bool live = n < a.g.N;
            uint32_t tn = n / a.g.tw;
            if (tn >= a.g.tiles_n) tn = a.g.tiles_n - 1;
            const uint32_t lc = n % a.g.tw;
            const size_t t = (size_t)tk * a.g.tiles_n + tn, sid = t * a.g.tw + lc;
            uint32_t state = kRansL;
            GmemCursor c;
            c.base = a.stream;
            c.row = -1;
            if (live) { state = a.states[sid]; c.base = a.stream + a.dense_offsets[sid]; c.row = (int32_t)a.dense_sizes[sid] - 1; }
            const uint8_t *man = a.mantissa + t * a.g.th * a.g.tw + lc;
            float xv[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) xv[m] = (live && m < (int)a.M) ? load_bf16(a.x + (size_t)m * a.ldx + n) : 0.f;
            for (uint32_t c0 = 0; c0 < rows; c0 += 32) {
                float wv[32];
#pragma unroll
                for (int r = 0; r < 32; ++r) {
                    wv[r] = 0.f;
                    if (c0 + r < rows) {
                        uint32_t e = decode_symbol(state, s_lut);
                        renorm_gmem(state, c, 1);
                        wv[r] = bf16_bits_to_float(assemble_bf16(lut_sym(e), __ldg(man + (size_t)(c0 + r) * a.g.tw)));
                    }
                }
                const uint32_t i = c0 + lane;                   // after the transpose lane r holds row c0 + r
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float p[32];
#pragma unroll
                    for (int r = 0; r < 32; ++r) p[r] = wv[r] * xv[m];
#pragma unroll
                    for (int s = 16; s >= 1; s >>= 1) {
#pragma unroll
                        for (int j = 0; j < s; ++j) {
                            bool up = (lane & s) != 0;
                            float send = up ? p[j] : p[j + s], keep = up ? p[j + s] : p[j];
                            p[j] = keep + __shfl_xor_sync(kFull, send, s);
                        }
                    }
                    if (i < rows) s_acc[(size_t)i * MT + m] += p[0];
                }
                __syncwarp();
            }
        }

        __syncthreads();
        for (uint32_t idx = threadIdx.x; idx < rows * a.M; idx += blockDim.x) {
            uint32_t r = idx / a.M, m = idx % a.M;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kLinWarps; ++w) v += s_acc_all[((size_t)w * a.g.th + r) * MT + m];
            uint32_t vrow = row0 + r;
            if (a.splits == 1) {
                if (a.bias) v += load_bf16(a.bias + vrow);
                a.y[(size_t)m * a.ldy + vrow] = float_to_bf16_bits(v);
            } else {
                a.partial[((size_t)split * a.M + m) * a.g.K + vrow] = v;
            }
        }
        if (a.splits > 1) {
            if (last_arrival(a.tickets + tk, a.splits, &s_flag)) {
                for (uint32_t idx = threadIdx.x; idx < rows * a.M; idx += blockDim.x) {
                    uint32_t r = idx / a.M, m = idx % a.M, vrow = row0 + r;
                    float v = 0.f;
                    for (uint32_t s = 0; s < a.splits; ++s) v += __ldcg(a.partial + ((size_t)s * a.M + m) * a.g.K + vrow);
                    if (a.bias) v += load_bf16(a.bias + vrow);
                    a.y[(size_t)m * a.ldy + vrow] = float_to_bf16_bits(v);
                }
                if (threadIdx.x == 0) a.tickets[tk] = 0;
            }
        }
        __syncthreads();
    }
}

// -------------------------------------------------------------------- host ---

static LinArgs base_args(const ci_tiled_weight *w) {
    LinArgs a;
    memset(&a, 0, sizeof a);
    a.stream = w->stream; a.states = w->states; a.tables = w->tables; a.tile_offsets = w->tile_offsets;
    a.tile_max_lens = w->tile_max_lens; a.lut = w->lut; a.slot_map = w->slot_map; a.mantissa = w->mantissa;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    a.stream_aligned = (reinterpret_cast<uintptr_t>(w->stream) & 15u) == 0;
    return a;
}

// Tickets + the larger of: split-K partials of the generic kernels, stream-K partials of the
// staged kernel (one [M][32] fp32 slot per warp of the grid plus one per column group).
static size_t workspace_bytes(uint32_t M, uint32_t n_out) {
    uint32_t mt = M < 16 ? M : 16;
    size_t split = (size_t)kMaxSplits * mt * n_out * sizeof(float);
    size_t slots = (size_t)sm_count() * 16 + (n_out + 31) / 32 + 2;
    size_t streamk = slots * mt * 32 * sizeof(float);
    return (size_t)kTicketBytes * 4 + (split > streamk ? split : streamk);
}

template <int MT>
static int launch_linear(LinArgs a, cudaStream_t s) {
    size_t smem = kProbScale * 4 + (size_t)kLinWarps * kLinStage;
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_linear<MT>, smem)) return rc;
    uint32_t items = a.g.groups * a.splits, cap = (uint32_t)sm_count() * 4;
    k_linear<MT><<<items < cap ? items : cap, kLinWarps * 32, smem, s>>>(a);
    CI_LAUNCH_CHECK(k_linear);
    return CI_OK;
}

template <int MT>
static int launch_transposed(LinArgs a, uint32_t groups_per_split, cudaStream_t s) {
    size_t smem = kProbScale * 4 + (size_t)kLinWarps * kLinStage + (size_t)kLinWarps * a.g.th * MT * sizeof(float);
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_linear_transposed<MT>, smem)) return rc;
    uint32_t items = a.g.tiles_k * a.splits, cap = (uint32_t)sm_count() * 3;
    k_linear_transposed<MT><<<items < cap ? items : cap, kLinWarps * 32, smem, s>>>(a, groups_per_split);
    CI_LAUNCH_CHECK(k_linear_transposed);
    return CI_OK;
}

template <int MT>
static int launch_transposed_dense(LinArgs a, uint32_t groups_per_split, cudaStream_t s) {
    size_t smem = kProbScale * 4 + (size_t)kLinWarps * a.g.th * MT * sizeof(float);
    static SmemLimit lim = {};
    if (int rc = ensure_smem_limit(lim, (const void *)k_linear_transposed_dense<MT>, smem)) return rc;
    uint32_t items = a.g.tiles_k * a.splits, cap = (uint32_t)sm_count() * 3;
    k_linear_transposed_dense<MT><<<items < cap ? items : cap, kLinWarps * 32, smem, s>>>(a, groups_per_split);
    CI_LAUNCH_CHECK(k_linear_transposed_dense);
    return CI_OK;
}

template <int MT>
static int launch_dense(LinArgs a, cudaStream_t s) {
    uint32_t items = a.g.groups * a.splits, cap = (uint32_t)sm_count() * 4;
    k_linear_dense<MT><<<items < cap ? items : cap, kLinWarps * 32, 0, s>>>(a);
    CI_LAUNCH_CHECK(k_linear_dense);
    return CI_OK;
}

// Split-K factor: enough CTAs for about one resident wave, at least one K tile per
// warp where possible; a caller-given factor is honoured up to kMaxSplits.
static void choose_splits(LinArgs &a, uint32_t split_k) {
    uint32_t splits = split_k;
    if (splits == 0) {
        uint32_t target = (uint32_t)sm_count() * 4;
        splits = (target + a.g.groups - 1) / a.g.groups;
        uint32_t by_tiles = (a.g.tiles_k + kLinWarps - 1) / kLinWarps;
        if (splits > by_tiles) splits = by_tiles;
    }
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits > a.g.tiles_k) splits = a.g.tiles_k;
    if (splits < 1) splits = 1;
    a.tiles_per_split = (a.g.tiles_k + splits - 1) / splits;
    a.splits = (a.g.tiles_k + a.tiles_per_split - 1) / a.tiles_per_split;
}

}  // namespace ci

using namespace ci;

extern "C" {

size_t ci_linear_workspace_bytes(uint32_t M, uint32_t n_out, uint32_t K, uint32_t tile_h) {
    size_t small = workspace_bytes(M, n_out);
    size_t big = (size_t)kTicketBytes * 4 + gemm_workspace_bytes(M, n_out, K, tile_h);    // prefill path, split-K partials
    return small > big ? small : big;
}

static int linear_impl(const ci_tiled_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M, const uint16_t *d_bias,
                       uint16_t *d_y, int64_t ldy, void *d_ws, size_t ws_bytes, uint32_t split_k, const ArFuse *ar,
                       ci_stream_t stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    CI_REQUIRE(d_x && d_y, "null activation / output pointer");
    if (M == 0) return CI_OK;
    CI_REQUIRE(ldx >= (int64_t)w->K && ldy >= (int64_t)w->N, "row strides smaller than the row length");
    LinArgs a = base_args(w);
    CI_REQUIRE(a.g.groups < kTicketBytes, "too many column groups for the ticket area");
    choose_splits(a, split_k);
    const bool have_ws = d_ws != nullptr && ws_bytes >= workspace_bytes(M, w->N);
    if (a.splits > 1 && !have_ws) {
        CI_REQUIRE(d_ws != nullptr, "split-K needs a workspace");
        set_error("workspace of %zu bytes, %zu needed", ws_bytes, workspace_bytes(M, w->N));
        return CI_E_WORKSPACE;
    }
    a.tickets = reinterpret_cast<uint32_t *>(d_ws);
    a.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d_ws) + kTicketBytes * 4);
    a.bias = d_bias; a.ldx = ldx; a.ldy = ldy;
    cudaStream_t s = (cudaStream_t)stream;
    if (ar != nullptr) {
        // output all-reduced inside the kernel: only the staged GEMV kernels do that, for one or two rows
        CI_REQUIRE(M <= 2 && split_k == 0 && have_ws, "the fused exchange takes at most two activation rows and needs a workspace");
        CI_REQUIRE(w->N % 2 == 0 && (uint64_t)M * w->N <= ar->capacity, "output does not fit the exchange buffer");
        CI_REQUIRE(ldy == (int64_t)w->N, "the fused exchange writes a dense [M, N] output");
        a.ar = *ar;
        a.x = d_x; a.y = d_y; a.M = M;
        rc = launch_linear_mma4(a, w->max_tile_len, s);
        if (rc == 1) rc = launch_linear_mma(a, w->max_tile_len, s);
        if (rc == 1) {
            set_error("this weight does not qualify for the staged kernels the fused exchange lives in");
            return CI_E_INVALID;
        }
        return rc;
    }
    if (M > 16 && d_ws != nullptr && ws_bytes > (size_t)kTicketBytes * 4) {
        // prefill: tcgen05 decode-GEMM over all rows at once (split_k: 0 = library's choice)
        a.x = d_x; a.y = d_y; a.M = M;
        rc = launch_linear_gemm(a, w->max_tile_len, ws_bytes - (size_t)kTicketBytes * 4, split_k, s);
        if (rc == CI_OK) return CI_OK;
        if (rc < 0) return rc;
    }
    for (uint32_t m0 = 0; m0 < M; m0 += 16) {                   // otherwise: 16 activation rows per pass
        uint32_t mc = M - m0 < 16 ? M - m0 : 16;
        a.x = d_x + (size_t)m0 * ldx;
        a.y = d_y + (size_t)m0 * ldy;
        a.M = mc;
        // staged tensor-core kernel when the weight qualifies (tile width <= 32, known maximum tile
        // depth, aligned buffers, a workspace); split_k != 0 asks for the generic split-K kernel
        if (split_k == 0 && have_ws) {
            rc = launch_linear_mma4(a, w->max_tile_len, s);     // 32-wide tiles, whole tile rows
            if (rc == CI_OK) continue;
            if (rc < 0) return rc;
            rc = launch_linear_mma(a, w->max_tile_len, s);
            if (rc == CI_OK) continue;
            if (rc < 0) return rc;
        }
        if (mc == 1) rc = launch_linear<1>(a, s);
        else if (mc == 2) rc = launch_linear<2>(a, s);
        else if (mc <= 4) rc = launch_linear<4>(a, s);
        else if (mc <= 8) rc = launch_linear<8>(a, s);
        else rc = launch_linear<16>(a, s);
        if (rc) return rc;
    }
    return CI_OK;
}

int ci_linear(const ci_tiled_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M, const uint16_t *d_bias,
              uint16_t *d_y, int64_t ldy, void *d_ws, size_t ws_bytes, uint32_t split_k, ci_stream_t stream) {
    return linear_impl(w, d_x, ldx, M, d_bias, d_y, ldy, d_ws, ws_bytes, split_k, nullptr, stream);
}

int ci_linear_route(const ci_tiled_weight *w, uint32_t M) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M == 0) return 0;
    if (M > 16) return 3;                                       // tcgen05 decode-GEMM (given a workspace)
    LinArgs a = base_args(w);
    a.M = M;
    a.ldx = w->K;
    a.ldy = w->N;
    a.dry_run = 1;
    rc = launch_linear_mma4(a, w->max_tile_len, nullptr);
    if (rc == CI_OK) return 2;
    if (rc < 0) return rc;
    rc = launch_linear_mma(a, w->max_tile_len, nullptr);
    if (rc == CI_OK) return 1;
    return rc < 0 ? rc : 0;
}

size_t ci_linear_allreduce_counter_bytes(void) { return 2 * sizeof(uint32_t); }

int ci_linear_allreduce_qualifies(const ci_tiled_weight *w, uint32_t M) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M == 0 || M > 2 || w->N % 2) return 0;
    LinArgs a = base_args(w);
    if (a.g.groups >= kTicketBytes) return 0;
    a.M = M;
    a.ldx = w->K;
    a.ldy = w->N;
    a.dry_run = 1;
    rc = launch_linear_mma4(a, w->max_tile_len, nullptr);
    if (rc == 1) rc = launch_linear_mma(a, w->max_tile_len, nullptr);
    return rc == CI_OK ? 1 : (rc == 1 ? 0 : rc);
}

int ci_linear_allreduce(const ci_tiled_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M, const uint16_t *d_bias,
                        uint16_t *d_y, void *d_ws, size_t ws_bytes, void *const *peer_bufs, uint32_t capacity,
                        uint32_t *d_counter, uint32_t rank, uint32_t world, uint32_t *d_status, ci_stream_t stream) {
    CI_REQUIRE(w != nullptr && peer_bufs && d_counter, "null pointer");
    CI_REQUIRE(world >= 2 && world <= kFuseMaxWorld && rank < world, "world size %u / rank %u out of range", world, rank);
    CI_REQUIRE(capacity % 8 == 0, "capacity must be a multiple of 8 elements");
    ArFuse ar;
    memset(&ar, 0, sizeof ar);
    for (uint32_t q = 0; q < world; ++q) {
        CI_REQUIRE(peer_bufs[q] != nullptr, "null peer pointer for rank %u", q);
        ar.bufs[q] = reinterpret_cast<uint16_t *>(peer_bufs[q]);
    }
    ar.counter = d_counter; ar.status = d_status; ar.rank = rank; ar.world = world; ar.capacity = capacity;
    return linear_impl(w, d_x, ldx, M, d_bias, d_y, (int64_t)w->N, d_ws, ws_bytes, 0, &ar, stream);
}

int ci_linear_transposed(const ci_tiled_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M,
                         const uint16_t *d_bias, uint16_t *d_y, int64_t ldy, void *d_ws, size_t ws_bytes,
                         ci_stream_t stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    CI_REQUIRE(d_x && d_y, "null activation / output pointer");
    if (M == 0) return CI_OK;
    CI_REQUIRE(ldx >= (int64_t)w->N && ldy >= (int64_t)w->K, "row strides smaller than the row length");
    LinArgs a = base_args(w);
    CI_REQUIRE(a.g.tiles_k <= kTicketBytes, "too many row tiles for the ticket area");
    // rows per pass limited by the per-warp shared-memory accumulators: tile_h * MT floats <= 4 KB
    uint32_t mt_cap = a.g.th <= 256 ? 4 : (a.g.th <= 512 ? 2 : 1);
    CI_REQUIRE(a.g.th <= 1024, "tile height %u above 1024 is not supported by the transposed linear", a.g.th);
    uint32_t target = (uint32_t)sm_count() * 6;
    uint32_t splits = (target + a.g.tiles_k - 1) / a.g.tiles_k;
    uint32_t by_groups = (a.g.groups + kLinWarps - 1) / kLinWarps;
    if (splits > by_groups) splits = by_groups;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 1) splits = 1;
    uint32_t gps = (a.g.groups + splits - 1) / splits;
    a.splits = (a.g.groups + gps - 1) / gps;
    if (a.splits > 1) {
        CI_REQUIRE(d_ws != nullptr, "split reduction needs a workspace");
        if (ws_bytes < workspace_bytes(M, w->K)) {
            set_error("workspace of %zu bytes, %zu needed", ws_bytes, workspace_bytes(M, w->K));
            return CI_E_WORKSPACE;
        }
    }
    a.tickets = reinterpret_cast<uint32_t *>(d_ws);
    a.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d_ws) + kTicketBytes * 4);
    a.bias = d_bias; a.ldx = ldx; a.ldy = ldy;
    cudaStream_t s = (cudaStream_t)stream;
    for (uint32_t m0 = 0; m0 < M; m0 += mt_cap) {
        uint32_t mc = M - m0 < mt_cap ? M - m0 : mt_cap;
        a.x = d_x + (size_t)m0 * ldx;
        a.y = d_y + (size_t)m0 * ldy;
        a.M = mc;
        if (mc == 1) rc = launch_transposed<1>(a, gps, s);
        else if (mc == 2) rc = launch_transposed<2>(a, gps, s);
        else rc = launch_transposed<4>(a, gps, s);
        if (rc) return rc;
    }
    return CI_OK;
}

int ci_linear_transposed_dense(const ci_dense_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M,
                               const uint16_t *d_bias, uint16_t *d_y, int64_t ldy, void *d_ws, size_t ws_bytes,
                               ci_stream_t stream) {
    CI_REQUIRE(w != nullptr, "null weight descriptor");
    int rc = check_tile(w->K, w->N, w->tile_h, w->tile_w);
    if (rc) return rc;
    CI_REQUIRE(w->states && w->stream_sizes && w->stream_offsets && w->mantissa, "null pointer in weight descriptor");
    CI_REQUIRE(w->lut || (w->tables && w->slot_map), "neither a prepared table nor tables + slot_map given");
    CI_REQUIRE(d_x && d_y, "null activation / output pointer");
    if (M == 0) return CI_OK;
    CI_REQUIRE(ldx >= (int64_t)w->N && ldy >= (int64_t)w->K, "row strides smaller than the row length");
    LinArgs a;
    memset(&a, 0, sizeof a);
    a.stream = w->stream; a.states = w->states; a.tables = w->tables; a.lut = w->lut; a.slot_map = w->slot_map;
    a.mantissa = w->mantissa; a.dense_sizes = w->stream_sizes; a.dense_offsets = w->stream_offsets;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    CI_REQUIRE(a.g.tiles_k <= kTicketBytes, "too many row tiles for the ticket area");
    CI_REQUIRE(a.g.th <= 1024, "tile height %u above 1024 is not supported by the transposed linear", a.g.th);
    uint32_t mt_cap = a.g.th <= 256 ? 4 : (a.g.th <= 512 ? 2 : 1);
    uint32_t target = (uint32_t)sm_count() * 6;
    uint32_t splits = (target + a.g.tiles_k - 1) / a.g.tiles_k;
    uint32_t by_groups = (a.g.groups + kLinWarps - 1) / kLinWarps;
    if (splits > by_groups) splits = by_groups;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 1) splits = 1;
    uint32_t gps = (a.g.groups + splits - 1) / splits;
    a.splits = (a.g.groups + gps - 1) / gps;
    if (a.splits > 1) {
        CI_REQUIRE(d_ws != nullptr, "split reduction needs a workspace");
        if (ws_bytes < workspace_bytes(M, w->K)) {
            set_error("workspace of %zu bytes, %zu needed", ws_bytes, workspace_bytes(M, w->K));
            return CI_E_WORKSPACE;
        }
    }
    a.tickets = reinterpret_cast<uint32_t *>(d_ws);
    a.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d_ws) + kTicketBytes * 4);
    a.bias = d_bias; a.ldx = ldx; a.ldy = ldy;
    cudaStream_t s = (cudaStream_t)stream;
    for (uint32_t m0 = 0; m0 < M; m0 += mt_cap) {
        uint32_t mc = M - m0 < mt_cap ? M - m0 : mt_cap;
        a.x = d_x + (size_t)m0 * ldx;
        a.y = d_y + (size_t)m0 * ldy;
        a.M = mc;
        if (mc == 1) rc = launch_transposed_dense<1>(a, gps, s);
        else if (mc == 2) rc = launch_transposed_dense<2>(a, gps, s);
        else rc = launch_transposed_dense<4>(a, gps, s);
        if (rc) return rc;
    }
    return CI_OK;
}

int ci_linear_dense(const ci_dense_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M, const uint16_t *d_bias,
                    uint16_t *d_y, int64_t ldy, void *d_ws, size_t ws_bytes, uint32_t split_k, ci_stream_t stream) {
    CI_REQUIRE(w != nullptr, "null weight descriptor");
    int rc = check_tile(w->K, w->N, w->tile_h, w->tile_w);
    if (rc) return rc;
    CI_REQUIRE(w->states && w->stream_sizes && w->stream_offsets && w->mantissa, "null pointer in weight descriptor");
    CI_REQUIRE(w->lut || (w->tables && w->slot_map), "neither a prepared table nor tables + slot_map given");
    CI_REQUIRE(d_x && d_y, "null activation / output pointer");
    if (M == 0) return CI_OK;
    CI_REQUIRE(ldx >= (int64_t)w->K && ldy >= (int64_t)w->N, "row strides smaller than the row length");
    LinArgs a;
    memset(&a, 0, sizeof a);
    a.stream = w->stream; a.states = w->states; a.tables = w->tables; a.lut = w->lut; a.slot_map = w->slot_map;
    a.mantissa = w->mantissa; a.dense_sizes = w->stream_sizes; a.dense_offsets = w->stream_offsets;
    a.g = make_geom(w->K, w->N, w->tile_h, w->tile_w);
    CI_REQUIRE(a.g.groups <= kTicketBytes, "too many column groups for the ticket area");
    choose_splits(a, split_k);
    if (a.splits > 1) {
        CI_REQUIRE(d_ws != nullptr, "split-K needs a workspace");
        if (ws_bytes < workspace_bytes(M, w->N)) {
            set_error("workspace of %zu bytes, %zu needed", ws_bytes, workspace_bytes(M, w->N));
            return CI_E_WORKSPACE;
        }
    }
    a.tickets = reinterpret_cast<uint32_t *>(d_ws);
    a.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d_ws) + kTicketBytes * 4);
    a.bias = d_bias; a.ldx = ldx; a.ldy = ldy;
    cudaStream_t s = (cudaStream_t)stream;
    for (uint32_t m0 = 0; m0 < M; m0 += 16) {
        uint32_t mc = M - m0 < 16 ? M - m0 : 16;
        a.x = d_x + (size_t)m0 * ldx;
        a.y = d_y + (size_t)m0 * ldy;
        a.M = mc;
        if (mc == 1) rc = launch_dense<1>(a, s);
        else if (mc == 2) rc = launch_dense<2>(a, s);
        else if (mc <= 4) rc = launch_dense<4>(a, s);
        else if (mc <= 8) rc = launch_dense<8>(a, s);
        else rc = launch_dense<16>(a, s);
        if (rc) return rc;
    }
    return CI_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Fused linear for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc (or any allocating routine) on the path that
// runs the model: a serving process whose device memory was carved up front between tenants and
// whose allocator is then closed, a plug-in sandbox that only receives input and output buffers, a
// runtime that must not touch the allocator once it is streaming tokens.  ci_linear needs
// scratch memory (the stream-K / split-K ticket counters and fp32 partial sums) that such a caller
// has no way to provide.  This variant keeps that scratch inside the library, in the fixed array
// below, so the caller passes nothing but the weight, the activations and the output.
//
// The price: the array has a fixed size (kStaticScratchBytes, 16 MiB), every GPU whose context loads
// this library holds it until the process exits, and all calls on a device share it.
static __device__ __align__(256) unsigned char ci_static_scratch[16u << 20];

namespace ci {
constexpr size_t kStaticScratchBytes = 16u << 20;
constexpr uint32_t kStaticMaxRows = 16;
// In host code the array's name is only a stand-in; the device address is asked for once per device,
// with that device current, and remembered.
static void *g_static_scratch_ptr[64] = {nullptr};

static int static_scratch(void **out) {
    int dev = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void *p = nullptr;
        CI_CUDA(cudaGetSymbolAddress(&p, ci_static_scratch));
        CI_REQUIRE(p != nullptr, "no device address for the built-in scratch array");
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return CI_OK;
}
}  // namespace ci

extern "C" {

size_t ci_linear_static_max_bytes(void) { return ci::kStaticScratchBytes; }

int ci_linear_static(const ci_tiled_weight *w, const uint16_t *d_x, int64_t ldx, uint32_t M, const uint16_t *d_bias,
                     uint16_t *d_y, int64_t ldy, ci_stream_t stream) {
    CI_REQUIRE(w != nullptr, "null weight descriptor");
    if (M > ci::kStaticMaxRows) {
        ci::set_error("ci_linear_static takes at most %u activation rows per call, got %u", ci::kStaticMaxRows, M);
        return CI_E_WORKSPACE;
    }
    const size_t need = ci_linear_workspace_bytes(M, w->N, w->K, w->tile_h);
    if (need > ci::kStaticScratchBytes) {
        ci::set_error("ci_linear_static: %u x %u outputs need %zu bytes of scratch, the built-in array holds %zu; "
                      "use ci_linear with a caller-provided workspace", M, w->N, need, ci::kStaticScratchBytes);
        return CI_E_WORKSPACE;
    }
    void *scratch = nullptr;
    int rc = ci::static_scratch(&scratch);          // first call on a device: looks the address up
    if (rc) return rc;
    // The array keeps whatever the last call left.  Only the ticket counters have to start at zero (a
    // call that ended normally leaves them so; this also covers one that did not); partial sums are
    // always written before they are read.  The last word of the ticket area is the kernels' status
    // word: it is left alone, so that a fault reported by one call can still be read after the next
    // (ci_linear_static_status).
    CI_CUDA(cudaMemsetAsync(scratch, 0, (size_t)(ci::kTicketBytes - 1) * 4, (cudaStream_t)stream));
    return ci_linear(w, d_x, ldx, M, d_bias, d_y, ldy, scratch, ci::kStaticScratchBytes, 0, stream);
}

int ci_linear_static_status(uint32_t *code, int clear, ci_stream_t stream) {
    void *scratch = nullptr;
    int rc = ci::static_scratch(&scratch);
    if (rc) return rc;
    return ci_status(ci_workspace_status_word(scratch), code, clear, stream);
}

}  // extern "C"
