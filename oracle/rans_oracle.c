/*
 * CPU oracle for the compressed-weight path of comp_inference.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * with (tests, the smoke test, and the CPU legs of the benchmark).  No product
 * code path may call into it.
 *
 * It restates, in plain C, what the reference computes on the GPU / in Python.
 * Every function cites the reference file and lines it follows (paths are
 * relative to the reference project root).  The reference ships no CPU codec:
 * src/cpp/ holds two headers only, so this restatement *is* the CPU baseline.
 *
 * Parity pinning: the byte layout produced here is decoded bit-exactly by the
 * reference's own Triton decoder and embedding kernel run under the Triton
 * interpreter (tests/golden/make_golden.py generated the committed fixtures).
 *
 * Format recap (rans.cuh:23-52, rans_host.cuh:22-24): 8-bit symbols, 32-bit
 * state, byte-wise renormalisation, 12-bit probability scale, lower bound
 * L = 1<<16, so a normalised state lies in [2^16, 2^24).
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#define PROB_BITS 12u
#define PROB_SCALE 4096u
#define RANS_L (1u << 16)

typedef struct {
    uint32_t K, N, th, tw;          /* matrix [K,N], tile height / width      */
    uint32_t tiles_k, tiles_n;      /* ceil(K/th), ceil(N/tw)                 */
} geom_t;

static geom_t make_geom(uint32_t K, uint32_t N, uint32_t th, uint32_t tw) {
    geom_t g; g.K = K; g.N = N; g.th = th; g.tw = tw;
    g.tiles_k = (K + th - 1) / th; g.tiles_n = (N + tw - 1) / tw;
    return g;
}

/* ---------------------------------------------------------------- threads */

typedef void (*range_fn)(void *ctx, uint64_t begin, uint64_t end);
typedef struct { range_fn fn; void *ctx; uint64_t begin, end; } job_t;
static void *job_main(void *p) { job_t *j = (job_t *)p; j->fn(j->ctx, j->begin, j->end); return NULL; }

/* Runs fn over [0,count) split into contiguous ranges, one per thread. */
static void parallel_for(uint64_t count, int nthreads, range_fn fn, void *ctx) {
    if (nthreads < 1) nthreads = 1;
    if ((uint64_t)nthreads > count) nthreads = count ? (int)count : 1;
    if (nthreads == 1) { fn(ctx, 0, count); return; }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * nthreads);
    job_t *jobs = (job_t *)malloc(sizeof(job_t) * nthreads);
    for (int i = 0; i < nthreads; ++i) {
        jobs[i].fn = fn; jobs[i].ctx = ctx;
        jobs[i].begin = count * (uint64_t)i / nthreads;
        jobs[i].end = count * (uint64_t)(i + 1) / nthreads;
        pthread_create(&th[i], NULL, job_main, &jobs[i]);
    }
    for (int i = 0; i < nthreads; ++i) pthread_join(th[i], NULL);
    free(th); free(jobs);
}

/* ------------------------------------------------------ bf16 split / merge */

/* comp_inference/comp_inference.py:10-32 (extract_exp_and_mantissa):
 * exponent = (raw >> 7) & 0xFF ; mantissa byte = (sign << 7) | (raw & 0x7F). */
void orc_split_bf16(const uint16_t *raw, uint64_t n, uint8_t *exp, uint8_t *man) {
    for (uint64_t i = 0; i < n; ++i) {
        uint32_t r = raw[i];
        exp[i] = (uint8_t)((r >> 7) & 0xFF);
        man[i] = (uint8_t)((((r >> 15) & 1u) << 7) | (r & 0x7F));
    }
}

/* comp_inference/comp_inference.py:156-180 (reconstruct_from_exp_and_mantissa)
 * and comp_inference/rans_triton.py:12-28 (_assemble_bf16). */
static inline uint16_t merge_one(uint8_t e, uint8_t m) {
    return (uint16_t)((((uint32_t)m & 0x80u) << 8) | ((uint32_t)e << 7) | ((uint32_t)m & 0x7Fu));
}
void orc_merge_bf16(const uint8_t *exp, const uint8_t *man, uint64_t n, uint16_t *raw) {
    for (uint64_t i = 0; i < n; ++i) raw[i] = merge_one(exp[i], man[i]);
}

/* ------------------------------------------------------------ frequency LUT */

/* comp_inference/comp_inference.py:183-239 (get_rans_lut).  numpy computes
 * floor(counts / counts.sum() * 4096) in float64; the same two IEEE operations
 * are done here in the same order.  Zero frequencies become 1; a positive
 * deficit goes to the first arg-max; a surplus is removed one unit at a time
 * from the (first) arg-max, re-evaluated after every unit. */
int orc_rans_lut(const uint8_t *data, uint64_t n, uint16_t *freqs_out, uint16_t *cdf_out) {
    uint64_t counts[256]; memset(counts, 0, sizeof counts);
    for (uint64_t i = 0; i < n; ++i) counts[data[i]]++;
    int64_t f[256]; int64_t sum = 0;
    double total = (double)n;
    for (int s = 0; s < 256; ++s) {
        double v = floor(((double)counts[s] / total) * 4096.0);
        f[s] = (int64_t)v;
        if (f[s] == 0) f[s] = 1;
        sum += f[s];
    }
    int64_t diff = 4096 - sum;
    if (diff > 0) {
        int best = 0; for (int s = 1; s < 256; ++s) if (f[s] > f[best]) best = s;
        f[best] += diff;
    } else {
        while (diff < 0) {
            int best = 0; for (int s = 1; s < 256; ++s) if (f[s] > f[best]) best = s;
            f[best] -= 1;
            if (f[best] < 1) return -1;
            diff += 1;
        }
    }
    uint32_t run = 0;
    for (int s = 0; s < 256; ++s) { cdf_out[s] = (uint16_t)run; freqs_out[s] = (uint16_t)f[s]; run += (uint32_t)f[s]; }
    return run == 4096 ? 0 : -2;
}

/* src/cuda/rans_host.cuh:476-488 (packed sym-info + slot map) with the packed
 * entry of src/cuda/rans.cuh:10-13 read as a little-endian u32: freq | cdf<<16
 * (that is what src/cuda/rans_ops.cu:392-394 downloads as `tables`). */
void orc_build_tables(const uint16_t *freqs, const uint16_t *cdf, uint32_t *tables, uint8_t *slot_map) {
    memset(slot_map, 0, PROB_SCALE);
    for (int s = 0; s < 256; ++s) {
        tables[s] = (uint32_t)freqs[s] | ((uint32_t)cdf[s] << 16);
        for (uint32_t j = 0; j < freqs[s]; ++j) {
            uint32_t slot = (uint32_t)cdf[s] + j;
            if (slot < PROB_SCALE) slot_map[slot] = (uint8_t)s;
        }
    }
}

/* ------------------------------------------------------- mantissa re-tiling */

/* comp_inference/comp_inference.py:35-64 (interleave_mantissas): zero-pad to
 * tile multiples, [K,N] -> [tiles_k][tiles_n][th][tw], flattened. */
void orc_interleave_mantissa(const uint8_t *man, uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint8_t *out) {
    geom_t g = make_geom(K, N, th, tw);
    uint64_t total = (uint64_t)g.tiles_k * g.tiles_n * th * tw;
    memset(out, 0, total);
    for (uint32_t r = 0; r < K; ++r)
        for (uint32_t c = 0; c < N; ++c) {
            uint64_t t = (uint64_t)(r / th) * g.tiles_n + (c / tw);
            out[t * th * tw + (uint64_t)(r % th) * tw + (c % tw)] = man[(uint64_t)r * N + c];
        }
}

/* comp_inference/comp_inference.py:67-93 (uninterleave_mantissas); a buffer
 * shorter than the full grid is treated as zero-padded at the end. */
void orc_uninterleave_mantissa(const uint8_t *tiled, uint64_t tiled_len, uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint8_t *man) {
    geom_t g = make_geom(K, N, th, tw);
    for (uint32_t r = 0; r < K; ++r)
        for (uint32_t c = 0; c < N; ++c) {
            uint64_t t = (uint64_t)(r / th) * g.tiles_n + (c / tw);
            uint64_t idx = t * th * tw + (uint64_t)(r % th) * tw + (c % tw);
            man[(uint64_t)r * N + c] = idx < tiled_len ? tiled[idx] : 0;
        }
}

/* ------------------------------------------------------------------ encoder */

/* One rANS stream: rows [row_hi-1 .. row_lo] of one column, last row first, as
 * in the loops of src/cuda/rans_kernels.cuh:128-152 / :155-178 / :45-69.
 * Rows at or beyond K are skipped, not encoded (:129-131).  Bytes are appended
 * to `bytes` in emission order; returns the byte count, writes the final state. */
static uint32_t encode_stream(const uint8_t *plane, uint32_t K, uint32_t N, uint32_t col,
                              uint32_t row_lo, uint32_t row_hi,
                              const uint16_t *freqs, const uint16_t *cdf,
                              uint8_t *bytes, uint32_t *state_out) {
    uint32_t state = RANS_L, n = 0;
    const uint32_t x_max_base = ((RANS_L >> PROB_BITS) << 8);     /* 4096 */
    for (int64_t r = (int64_t)row_hi - 1; r >= (int64_t)row_lo; --r) {
        if ((uint64_t)r >= K) continue;
        uint8_t sym = plane[(uint64_t)r * N + col];
        uint32_t freq = freqs[sym], start = cdf[sym];
        uint32_t x_max = x_max_base * freq;
        while (state >= x_max) { if (bytes) bytes[n] = (uint8_t)(state & 0xFF); n++; state >>= 8; }
        state = ((state / freq) << PROB_BITS) + (state % freq) + start;
    }
    *state_out = state;
    return n;
}

typedef struct {
    const uint8_t *plane; geom_t g; const uint16_t *freqs, *cdf;
    uint32_t *states, *sizes, *tile_max_lens;
    const uint64_t *tile_offsets64; uint8_t *stream;   /* pass 2 only */
    int dense;                                       /* 0 = ILP2 tiles, 1 = one stream per column */
    const uint32_t *stream_offsets;                  /* dense pass 2 */
} enc_ctx;

/* Pass 1 over tiles: sizes, final states, per-tile longest stream.
 * Stream ids: src/cuda/rans_kernels.cuh:106-111 (tile*2*tw + c for the top
 * half "A", + tw for the bottom half "B") or :32-34 for the dense layout.
 * Columns beyond N get state L and size 0 (the reference leaves them unset,
 * :99-100; its decoders mask those lanes, rans_triton.py:57-67). */
static void enc_pass1(void *vctx, uint64_t t0, uint64_t t1) {
    enc_ctx *c = (enc_ctx *)vctx; geom_t g = c->g;
    for (uint64_t t = t0; t < t1; ++t) {
        uint32_t tk = (uint32_t)(t / g.tiles_n), tn = (uint32_t)(t % g.tiles_n);
        uint32_t row0 = tk * g.th, half = g.th / 2, maxlen = 0;
        for (uint32_t lc = 0; lc < g.tw; ++lc) {
            uint32_t col = tn * g.tw + lc;
            if (c->dense) {
                uint64_t sid = t * g.tw + lc;
                if (col >= g.N) { c->states[sid] = RANS_L; c->sizes[sid] = 0; continue; }
                c->sizes[sid] = encode_stream(c->plane, g.K, g.N, col, row0, row0 + g.th, c->freqs, c->cdf, NULL, &c->states[sid]);
            } else {
                uint64_t sa = t * 2 * g.tw + lc, sb = sa + g.tw;
                if (col >= g.N) { c->states[sa] = c->states[sb] = RANS_L; c->sizes[sa] = c->sizes[sb] = 0; continue; }
                c->sizes[sb] = encode_stream(c->plane, g.K, g.N, col, row0 + half, row0 + g.th, c->freqs, c->cdf, NULL, &c->states[sb]);
                c->sizes[sa] = encode_stream(c->plane, g.K, g.N, col, row0, row0 + half, c->freqs, c->cdf, NULL, &c->states[sa]);
                if (c->sizes[sa] > maxlen) maxlen = c->sizes[sa];
                if (c->sizes[sb] > maxlen) maxlen = c->sizes[sb];
            }
        }
        if (!c->dense) c->tile_max_lens[t] = maxlen;
    }
}

/* Pass 2: write bytes at their final place.
 * ILP2 tiles (src/cuda/rans_ops.cu:328-370): the tile is a row-major
 * [max_len][2*tw] byte matrix, column j = stream j of the tile, each stream
 * bottom-aligned (zero rows above its first emitted byte, last emitted byte on
 * the last row).  Dense layout (src/cuda/rans_ops.cu:165-176): streams
 * concatenated in id order, bytes in emission order. */
static void enc_pass2(void *vctx, uint64_t t0, uint64_t t1) {
    enc_ctx *c = (enc_ctx *)vctx; geom_t g = c->g;
    uint8_t *tmp = (uint8_t *)malloc((size_t)g.th * 2 + 16);
    for (uint64_t t = t0; t < t1; ++t) {
        uint32_t tk = (uint32_t)(t / g.tiles_n), tn = (uint32_t)(t % g.tiles_n);
        uint32_t row0 = tk * g.th, half = g.th / 2;
        for (uint32_t lc = 0; lc < g.tw; ++lc) {
            uint32_t col = tn * g.tw + lc, st;
            if (col >= g.N) continue;
            if (c->dense) {
                uint64_t sid = t * g.tw + lc;
                uint32_t n = encode_stream(c->plane, g.K, g.N, col, row0, row0 + g.th, c->freqs, c->cdf, tmp, &st);
                memcpy(c->stream + c->stream_offsets[sid], tmp, n);
            } else {
                uint32_t maxlen = c->tile_max_lens[t], W = 2 * g.tw;
                uint8_t *base = c->stream + c->tile_offsets64[t];
                for (int h = 0; h < 2; ++h) {
                    uint32_t lo = h ? row0 + half : row0, hi = h ? row0 + g.th : row0 + half;
                    uint32_t n = encode_stream(c->plane, g.K, g.N, col, lo, hi, c->freqs, c->cdf, tmp, &st);
                    uint32_t j = h ? g.tw + lc : lc, pad = maxlen - n;
                    for (uint32_t b = 0; b < n; ++b) base[(uint64_t)(pad + b) * W + j] = tmp[b];
                }
            }
        }
    }
    free(tmp);
}

/* Shrinks tile sizes that exceed the matrix, by halving, as
 * src/cuda/rans_ops.cu:219-223 does.  (The reference applies this after its
 * kernel already ran with the unshrunk sizes, which leaves an undecodable
 * result; here the shrunk sizes are the ones encoded with.) */
void orc_effective_tile(uint32_t K, uint32_t N, uint32_t *th, uint32_t *tw) {
    while (*th > K && *th > 1) *th /= 2;
    while (*tw > N && *tw > 1) *tw /= 2;
}

/* ILP2 tiled encoder = RansManager::compress_tiled
 * (src/python_bindings.cpp:302-347 -> src/cuda/rans_ops.cu:205-410).
 * states/sizes: [tiles*2*tw]; tile_offsets/tile_max_lens: [tiles].
 * *stream_out is malloc'ed (release with orc_free).  Returns 0 on success. */
int orc_encode_tiled(const uint8_t *plane, uint32_t K, uint32_t N,
                     const uint16_t *freqs, const uint16_t *cdf, uint32_t th, uint32_t tw,
                     uint32_t *states, uint32_t *sizes, uint32_t *tile_offsets, uint32_t *tile_max_lens,
                     uint8_t **stream_out, uint64_t *stream_len, int nthreads) {
    if (th % 16 != 0 || tw == 0) return -1;              /* src/cuda/rans_host.cuh:440-445 */
    geom_t g = make_geom(K, N, th, tw);
    uint64_t T = (uint64_t)g.tiles_k * g.tiles_n;
    enc_ctx c; memset(&c, 0, sizeof c);
    c.plane = plane; c.g = g; c.freqs = freqs; c.cdf = cdf;
    c.states = states; c.sizes = sizes; c.tile_max_lens = tile_max_lens; c.dense = 0;
    parallel_for(T, nthreads, enc_pass1, &c);
    uint64_t *off64 = (uint64_t *)malloc(sizeof(uint64_t) * (T ? T : 1));
    uint64_t run = 0;
    for (uint64_t t = 0; t < T; ++t) { off64[t] = run; tile_offsets[t] = (uint32_t)run; run += (uint64_t)tile_max_lens[t] * 2 * tw; }
    if (run > 0xFFFFFFFFull) { free(off64); return -3; }  /* offsets are u32 in the format */
    uint8_t *stream = (uint8_t *)calloc(run ? run : 1, 1);
    c.tile_offsets64 = off64; c.stream = stream;
    parallel_for(T, nthreads, enc_pass2, &c);
    free(off64);
    *stream_out = stream; *stream_len = run;
    return 0;
}

/* Dense ("uncoalesced") encoder = RansManager::compress_tiled_uncoalesced
 * (src/python_bindings.cpp:349-397 -> src/cuda/rans_ops.cu:74-203). */
int orc_encode_dense(const uint8_t *plane, uint32_t K, uint32_t N,
                     const uint16_t *freqs, const uint16_t *cdf, uint32_t th, uint32_t tw,
                     uint32_t *states, uint32_t *sizes, uint32_t *stream_offsets,
                     uint8_t **stream_out, uint64_t *stream_len, int nthreads) {
    if (th % 16 != 0 || tw == 0) return -1;
    geom_t g = make_geom(K, N, th, tw);
    uint64_t T = (uint64_t)g.tiles_k * g.tiles_n, S = T * tw;
    enc_ctx c; memset(&c, 0, sizeof c);
    c.plane = plane; c.g = g; c.freqs = freqs; c.cdf = cdf;
    c.states = states; c.sizes = sizes; c.dense = 1;
    parallel_for(T, nthreads, enc_pass1, &c);
    uint64_t run = 0;
    for (uint64_t s = 0; s < S; ++s) { stream_offsets[s] = (uint32_t)run; run += sizes[s]; }
    if (run > 0xFFFFFFFFull) return -3;
    uint8_t *stream = (uint8_t *)calloc(run ? run : 1, 1);
    c.stream_offsets = stream_offsets; c.stream = stream;
    parallel_for(T, nthreads, enc_pass2, &c);
    *stream_out = stream; *stream_len = run;
    return 0;
}

void orc_free(void *p) { free(p); }

/* ------------------------------------------------------------------ decoder */

typedef struct { uint32_t state; int64_t row; const uint8_t *base; uint32_t stride; } dec_t;

/* One decode step of one stream: comp_inference/rans_triton.py:92-119
 * (slot -> symbol -> packed {freq,cdf} -> state update -> at most two byte
 * reads, each only while state < L and bytes remain above the cursor). */
static inline uint8_t dec_step(dec_t *d, const uint32_t *tables, const uint8_t *slot_map) {
    uint32_t slot = d->state & (PROB_SCALE - 1);
    uint8_t sym = slot_map[slot];
    uint32_t pk = tables[sym];
    d->state = (pk & 0xFFFF) * (d->state >> PROB_BITS) + (slot - (pk >> 16));
    for (int k = 0; k < 2; ++k)
        if (d->state < RANS_L && d->row >= 0) {
            d->state = (d->state << 8) | d->base[(uint64_t)d->row * d->stride];
            d->row--;
        }
    return sym;
}

typedef struct {
    const uint8_t *stream; const uint32_t *states, *tables; const uint8_t *slot_map;
    const uint32_t *tile_offsets, *tile_max_lens; geom_t g;
    uint8_t *plane;            /* exponent plane out, or NULL                 */
    const uint8_t *mantissa;   /* tiled mantissa, for bf16 / linear           */
    uint16_t *bf16;            /* bf16 [K,N] out, or NULL                     */
    float *wf32;               /* fp32 [K,N] out, or NULL                     */
} dec_ctx;

static inline float bf16_to_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

/* Tiled ILP2 decode: comp_inference/rans_triton.py:34-119.  Both streams of a
 * column start on the tile's last byte row and walk upwards. */
static void dec_tiles(void *vctx, uint64_t t0, uint64_t t1) {
    dec_ctx *c = (dec_ctx *)vctx; geom_t g = c->g;
    uint32_t half = g.th / 2, W = 2 * g.tw;
    for (uint64_t t = t0; t < t1; ++t) {
        uint32_t tk = (uint32_t)(t / g.tiles_n), tn = (uint32_t)(t % g.tiles_n);
        const uint8_t *tb = c->stream + c->tile_offsets[t];
        int64_t depth = c->tile_max_lens[t];
        for (uint32_t lc = 0; lc < g.tw; ++lc) {
            uint32_t col = tn * g.tw + lc;
            if (col >= g.N) continue;
            dec_t A = { c->states[t * W + lc], depth - 1, tb + lc, W };
            dec_t B = { c->states[t * W + g.tw + lc], depth - 1, tb + g.tw + lc, W };
            for (uint32_t i = 0; i < half; ++i) {
                for (int h = 0; h < 2; ++h) {
                    uint32_t lr = i + (h ? half : 0);
                    uint64_t row = (uint64_t)tk * g.th + lr;
                    if (row >= g.K) continue;
                    uint8_t e = dec_step(h ? &B : &A, c->tables, c->slot_map);
                    uint64_t o = row * g.N + col;
                    if (c->plane) c->plane[o] = e;
                    if (c->bf16 || c->wf32) {
                        uint8_t m = c->mantissa[t * g.th * g.tw + (uint64_t)lr * g.tw + lc];
                        uint16_t b = merge_one(e, m);
                        if (c->bf16) c->bf16[o] = b;
                        if (c->wf32) c->wf32[o] = bf16_to_f32(b);
                    }
                }
            }
        }
    }
}

static void fill_dec(dec_ctx *c, const uint8_t *stream, const uint32_t *states, const uint32_t *tables,
                     const uint8_t *slot_map, const uint32_t *tile_offsets, const uint32_t *tile_max_lens,
                     uint32_t K, uint32_t N, uint32_t th, uint32_t tw) {
    memset(c, 0, sizeof *c);
    c->stream = stream; c->states = states; c->tables = tables; c->slot_map = slot_map;
    c->tile_offsets = tile_offsets; c->tile_max_lens = tile_max_lens; c->g = make_geom(K, N, th, tw);
}

/* rans_decomp_triton_tiled (comp_inference/rans_triton.py:122-168): exponent plane u8 [K,N]. */
void orc_decode_plane(const uint8_t *stream, const uint32_t *states, const uint32_t *tables, const uint8_t *slot_map,
                      const uint32_t *tile_offsets, const uint32_t *tile_max_lens,
                      uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint8_t *plane, int nthreads) {
    dec_ctx c; fill_dec(&c, stream, states, tables, slot_map, tile_offsets, tile_max_lens, K, N, th, tw);
    c.plane = plane;
    parallel_for((uint64_t)c.g.tiles_k * c.g.tiles_n, nthreads, dec_tiles, &c);
}

/* rans_decompress_module_weight_bf16 (comp_inference/comp_inference.py:573-713)
 * = tiled decode + mantissa un-tiling + bit merge, with the module's own tile
 * size (the reference hard-codes 1024x32 at :642-643,:694-696). Output bf16 bits [K,N]. */
void orc_decode_bf16(const uint8_t *stream, const uint32_t *states, const uint32_t *tables, const uint8_t *slot_map,
                     const uint32_t *tile_offsets, const uint32_t *tile_max_lens, const uint8_t *mantissa,
                     uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint16_t *out, int nthreads) {
    dec_ctx c; fill_dec(&c, stream, states, tables, slot_map, tile_offsets, tile_max_lens, K, N, th, tw);
    c.mantissa = mantissa; c.bf16 = out;
    parallel_for((uint64_t)c.g.tiles_k * c.g.tiles_n, nthreads, dec_tiles, &c);
}

/* Dense-layout decode of the exponent plane: per-stream offset/size, bytes read
 * from the stream's last byte backwards (comp_inference/linear_triton.py:1044-1186
 * uses stream_offset + size - 1 as the start cursor, stride 1). */
typedef struct { const uint8_t *stream; const uint32_t *states, *sizes, *offsets, *tables; const uint8_t *slot_map; geom_t g; uint8_t *plane; } dd_ctx;
static void dec_dense_tiles(void *vctx, uint64_t t0, uint64_t t1) {
    dd_ctx *c = (dd_ctx *)vctx; geom_t g = c->g;
    for (uint64_t t = t0; t < t1; ++t) {
        uint32_t tk = (uint32_t)(t / g.tiles_n), tn = (uint32_t)(t % g.tiles_n);
        for (uint32_t lc = 0; lc < g.tw; ++lc) {
            uint32_t col = tn * g.tw + lc; uint64_t sid = t * g.tw + lc;
            if (col >= g.N) continue;
            dec_t d = { c->states[sid], (int64_t)c->sizes[sid] - 1, c->stream + c->offsets[sid], 1 };
            for (uint32_t i = 0; i < g.th; ++i) {
                uint64_t row = (uint64_t)tk * g.th + i;
                if (row >= g.K) break;
                c->plane[row * g.N + col] = dec_step(&d, c->tables, c->slot_map);
            }
        }
    }
}
void orc_decode_plane_dense(const uint8_t *stream, const uint32_t *states, const uint32_t *sizes, const uint32_t *offsets,
                            const uint32_t *tables, const uint8_t *slot_map,
                            uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint8_t *plane, int nthreads) {
    dd_ctx c = { stream, states, sizes, offsets, tables, slot_map, make_geom(K, N, th, tw), plane };
    parallel_for((uint64_t)c.g.tiles_k * c.g.tiles_n, nthreads, dec_dense_tiles, &c);
}

/* -------------------------------------------------------------- embedding */

/* fused_rans_embedding_triton (comp_inference/embedding_triton.py:170-330):
 * out[i,:] = W[ids[i],:]; the kernel picks stream A or B of the row's tile,
 * fast-forwards (row % th) % (th/2) symbols and emits one; ids outside [0,K)
 * give a zero row (:203-210). */
typedef struct { dec_ctx d; const int64_t *ids; uint16_t *out; } emb_ctx;
static void emb_rows(void *vctx, uint64_t i0, uint64_t i1) {
    emb_ctx *e = (emb_ctx *)vctx; dec_ctx *c = &e->d; geom_t g = c->g;
    uint32_t half = g.th / 2, W = 2 * g.tw;
    for (uint64_t i = i0; i < i1; ++i) {
        int64_t tok = e->ids[i];
        uint16_t *o = e->out + i * g.N;
        if (tok < 0 || tok >= (int64_t)g.K) { memset(o, 0, (size_t)g.N * 2); continue; }
        uint32_t tk = (uint32_t)(tok / g.th), rel = (uint32_t)(tok % g.th);
        uint32_t bottom = rel >= half, inner = rel % half;
        for (uint32_t col = 0; col < g.N; ++col) {
            uint32_t tn = col / g.tw, lc = col % g.tw;
            uint64_t t = (uint64_t)tk * g.tiles_n + tn;
            uint32_t j = bottom ? g.tw + lc : lc;
            dec_t d = { c->states[t * W + j], (int64_t)c->tile_max_lens[t] - 1, c->stream + c->tile_offsets[t] + j, W };
            uint8_t sym = 0;
            for (uint32_t s = 0; s <= inner; ++s) sym = dec_step(&d, c->tables, c->slot_map);
            uint8_t m = c->mantissa[t * g.th * g.tw + (uint64_t)rel * g.tw + lc];
            o[col] = merge_one(sym, m);
        }
    }
}
void orc_embedding(const int64_t *ids, uint64_t n_ids,
                   const uint8_t *stream, const uint32_t *states, const uint32_t *tables, const uint8_t *slot_map,
                   const uint32_t *tile_offsets, const uint32_t *tile_max_lens, const uint8_t *mantissa,
                   uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint16_t *out, int nthreads) {
    emb_ctx e; fill_dec(&e.d, stream, states, tables, slot_map, tile_offsets, tile_max_lens, K, N, th, tw);
    e.d.mantissa = mantissa; e.ids = ids; e.out = out;
    parallel_for(n_ids, nthreads, emb_rows, &e);
}

/* ------------------------------------------------------------------ linear */

/* The stated check for the fused linears is decompress-then-matmul with fp32
 * accumulation (tests/test_mat_mul.py:186-238 compares the fused kernel of
 * comp_inference/linear_triton.py:229-552 with torch.matmul on the
 * reconstructed weight).  y[m,n] = sum_k x[m,k] * W[k,n], x and W bf16, sum in
 * fp32 (double accumulator, rounded once, so the oracle itself adds no error). */
typedef struct { const float *w; const uint16_t *x; uint32_t M, K, N; float *y; int transposed; } mm_ctx;
static void mm_cols(void *vctx, uint64_t n0, uint64_t n1) {
    mm_ctx *c = (mm_ctx *)vctx;
    double *acc = (double *)malloc(sizeof(double) * (n1 - n0 ? n1 - n0 : 1));
    for (uint32_t m = 0; m < c->M; ++m) {
        if (!c->transposed) {
            for (uint64_t n = n0; n < n1; ++n) acc[n - n0] = 0.0;
            for (uint32_t k = 0; k < c->K; ++k) {
                double xv = bf16_to_f32(c->x[(uint64_t)m * c->K + k]);
                const float *wr = c->w + (uint64_t)k * c->N;
                for (uint64_t n = n0; n < n1; ++n) acc[n - n0] += xv * wr[n];
            }
            for (uint64_t n = n0; n < n1; ++n) c->y[(uint64_t)m * c->N + n] = (float)acc[n - n0];
        } else {
            /* weight stored [V=K rows, H=N cols]; y[m,v] = sum_h x[m,h] W[v,h]
             * (comp_inference/transposed_linear_triton.py:187-435); here n0..n1 ranges over v. */
            for (uint64_t v = n0; v < n1; ++v) {
                double a = 0.0; const float *wr = c->w + v * c->N;
                for (uint32_t h = 0; h < c->N; ++h) a += (double)bf16_to_f32(c->x[(uint64_t)m * c->N + h]) * wr[h];
                c->y[(uint64_t)m * c->K + v] = (float)a;
            }
        }
    }
    free(acc);
}

/* transposed = 0: x [M,K] -> y [M,N].  transposed = 1: x [M,N] -> y [M,K]. */
int orc_linear(const uint16_t *x, uint32_t M,
               const uint8_t *stream, const uint32_t *states, const uint32_t *tables, const uint8_t *slot_map,
               const uint32_t *tile_offsets, const uint32_t *tile_max_lens, const uint8_t *mantissa,
               uint32_t K, uint32_t N, uint32_t th, uint32_t tw, int transposed, float *y, int nthreads) {
    float *w = (float *)malloc(sizeof(float) * (size_t)K * N);
    if (!w) return -1;
    dec_ctx c; fill_dec(&c, stream, states, tables, slot_map, tile_offsets, tile_max_lens, K, N, th, tw);
    c.mantissa = mantissa; c.wf32 = w;
    parallel_for((uint64_t)c.g.tiles_k * c.g.tiles_n, nthreads, dec_tiles, &c);
    mm_ctx m = { w, x, M, K, N, y, transposed };
    parallel_for(transposed ? K : N, nthreads, mm_cols, &m);
    free(w);
    return 0;
}
