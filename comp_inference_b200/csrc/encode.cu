// GPU rANS encoder writing the packed stream layouts directly.
//
// Replaces the reference's one-warp-per-block encoder kernels
// (src/cuda/rans_kernels.cuh:76-188 ILP2, :7-74 dense), their strided scratch
// buffer and the single-threaded host re-interleave (src/cuda/rans_ops.cu:328-370,
// :165-176).  Two passes over the symbols: pass 1 only counts bytes and produces
// the final states, a scan turns the per-tile (per-stream) byte counts into
// offsets, pass 2 re-encodes and stores every byte at its final address.  The
// symbol plane (1 byte per weight) is read twice from L2/HBM; no scratch sized
// by the payload exists and nothing is repacked on the host.
#include "common.cuh"

namespace ci {

struct EncArgs {
    const uint8_t *plane;
    uint32_t K, N, th, tw, tiles_n, half;
};

// Encodes rows [row_hi-1 .. row_lo] of column `col`, last row first
// (src/cuda/rans_kernels.cuh:128-152).  Rows >= K are skipped (:129-131).
// When dst != nullptr byte b is stored at dst + b * dst_stride.
__device__ __forceinline__ uint32_t encode_run(const EncArgs &a, const uint32_t *s_info, uint32_t col, uint32_t row_lo,
                                               uint32_t row_hi, uint32_t &state_out, uint8_t *dst,
                                               uint32_t dst_stride) {
    uint32_t state = kRansL, n = 0;
    if (row_hi > a.K) row_hi = a.K;
    for (int64_t r = (int64_t)row_hi - 1; r >= (int64_t)row_lo; --r) {
        uint32_t sym = a.plane[(size_t)r * a.N + col];
        uint32_t info = s_info[sym];
        uint32_t freq = info & 0xFFFFu, start = info >> 16;
        uint32_t x_max = freq << 12;                          // ((L >> 12) << 8) * freq
        while (state >= x_max) {
            if (dst) dst[(size_t)n * dst_stride] = (uint8_t)(state & 0xFFu);
            ++n;
            state >>= 8;
        }
        uint32_t q = state / freq;
        state = (q << kProbBits) + (state - q * freq) + start;
    }
    state_out = state;
    return n;
}

__device__ __forceinline__ void load_sym_info(uint32_t *s_info, const uint32_t *info) {
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) s_info[i] = info[i];
    __syncthreads();
}

// grid (ceil(tiles_n*tw / block), tiles_k); one thread per (tile row, column slot).
template <bool DENSE, bool WRITE>
__global__ void k_encode(EncArgs a, const uint32_t *__restrict__ info, uint32_t *__restrict__ states,
                         uint32_t *__restrict__ sizes, const uint32_t *__restrict__ in_sizes,
                         const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ max_lens,
                         uint8_t *__restrict__ stream) {
    __shared__ uint32_t s_info[256];
    load_sym_info(s_info, info);
    uint32_t slot = blockIdx.x * blockDim.x + threadIdx.x;    // column slot inside the padded tile row
    if (slot >= a.tiles_n * a.tw) return;
    uint32_t tk = blockIdx.y, tn = slot / a.tw, lc = slot % a.tw;
    uint32_t col = slot;                                        // tn * tw + lc
    size_t t = (size_t)tk * a.tiles_n + tn;
    uint32_t row0 = tk * a.th;
    bool live = col < a.N;
    if (DENSE) {
        size_t sid = t * a.tw + lc;
        uint32_t st = kRansL, n = 0;
        if (live) n = encode_run(a, s_info, col, row0, row0 + a.th, st, WRITE ? stream + offsets[sid] : nullptr, 1);
        if (!WRITE) { states[sid] = st; sizes[sid] = n; }
    } else {
        size_t sa = t * 2 * a.tw + lc, sb = sa + a.tw;
        uint32_t stA = kRansL, stB = kRansL, nA = 0, nB = 0;
        if (live) {
            uint8_t *dA = nullptr, *dB = nullptr;
            uint32_t W = 2 * a.tw;
            if (WRITE) {
                // bottom-aligned columns of the [max_len][2*tw] tile matrix (src/cuda/rans_ops.cu:348-368)
                uint32_t ml = max_lens[t];
                uint8_t *base = stream + offsets[t];
                dA = base + (size_t)(ml - in_sizes[sa]) * W + lc;
                dB = base + (size_t)(ml - in_sizes[sb]) * W + a.tw + lc;
            }
            nB = encode_run(a, s_info, col, row0 + a.half, row0 + a.th, stB, dB, W);
            nA = encode_run(a, s_info, col, row0, row0 + a.half, stA, dA, W);
        }
        if (!WRITE) { states[sa] = stA; sizes[sa] = nA; states[sb] = stB; sizes[sb] = nB; }
    }
}

// One thread per tile: longest stream of the tile (src/cuda/rans_ops.cu:338-345).
__global__ void k_tile_max_len(const uint32_t *__restrict__ sizes, uint32_t W, uint64_t tiles,
                               uint32_t *__restrict__ max_lens) {
    uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tiles) return;
    uint32_t m = 0;
    for (uint32_t j = 0; j < W; ++j) m = max(m, sizes[t * W + j]);
    max_lens[t] = m;
}

// Exclusive scan of in[i] * mult over n items by a single 1024-thread block;
// offsets are 32-bit in the format, the 64-bit total is reported for the overflow check.
__global__ void k_scan_offsets(const uint32_t *__restrict__ in, uint32_t mult, uint64_t n,
                               uint32_t *__restrict__ offsets, unsigned long long *__restrict__ total) {
    __shared__ unsigned long long s_part[1024];
    const uint32_t T = blockDim.x, tid = threadIdx.x;
    uint64_t chunk = (n + T - 1) / T, b = (uint64_t)tid * chunk, e = b + chunk;
    if (b > n) b = n;
    if (e > n) e = n;
    unsigned long long sum = 0;
    for (uint64_t i = b; i < e; ++i) sum += (unsigned long long)in[i] * mult;
    s_part[tid] = sum;
    __syncthreads();
    for (uint32_t d = 1; d < T; d <<= 1) {                    // Hillis-Steele inclusive scan
        unsigned long long v = tid >= d ? s_part[tid - d] : 0;
        __syncthreads();
        s_part[tid] += v;
        __syncthreads();
    }
    unsigned long long run = s_part[tid] - sum;
    for (uint64_t i = b; i < e; ++i) { offsets[i] = (uint32_t)run; run += (unsigned long long)in[i] * mult; }
    if (tid == T - 1) *total = s_part[tid];
}

static int upload_sym_info(const uint16_t *freqs, const uint16_t *cdf, uint32_t **d_info, cudaStream_t s) {
    CI_REQUIRE(freqs && cdf, "null frequency tables");
    uint32_t h[256], sum = 0;
    for (int i = 0; i < 256; ++i) {
        CI_REQUIRE(freqs[i] >= 1, "symbol %d has zero frequency; every symbol needs at least 1", i);
        h[i] = (uint32_t)freqs[i] | ((uint32_t)cdf[i] << 16);
        sum += freqs[i];
    }
    CI_REQUIRE(sum == kProbScale, "frequencies sum to %u, expected 4096", sum);
    CI_CUDA(cudaMallocAsync((void **)d_info, sizeof h, s));
    // pageable source: the copy is staged before the call returns, so the stack buffer may go away
    CI_CUDA(cudaMemcpyAsync(*d_info, h, sizeof h, cudaMemcpyHostToDevice, s));
    return CI_OK;
}

template <bool DENSE>
static int encode_sizes(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                        uint32_t th, uint32_t tw, uint32_t *d_states, uint32_t *d_sizes, uint32_t *d_offsets,
                        uint32_t *d_max_lens, uint64_t *stream_len, cudaStream_t s) {
    CI_REQUIRE(d_plane && d_states && d_sizes && d_offsets && stream_len, "null pointer");
    CI_REQUIRE(DENSE || d_max_lens, "null pointer");
    int rc = check_tile(K, N, th, tw);
    if (rc) return rc;
    Geom g = make_geom(K, N, th, tw);
    uint32_t *d_info = nullptr;
    rc = upload_sym_info(freqs, cdf, &d_info, s);
    if (rc) return rc;
    unsigned long long *d_total = nullptr;
    CI_CUDA(cudaMallocAsync((void **)&d_total, sizeof(unsigned long long), s));
    EncArgs a{d_plane, K, N, th, tw, g.tiles_n, g.half};
    const uint32_t block = 128, slots = g.tiles_n * tw;
    dim3 grid((slots + block - 1) / block, g.tiles_k);
    k_encode<DENSE, false><<<grid, block, 0, s>>>(a, d_info, d_states, d_sizes, nullptr, nullptr, nullptr, nullptr);
    CI_LAUNCH_CHECK(k_encode);
    uint64_t tiles = (uint64_t)g.tiles_k * g.tiles_n;
    if (DENSE) {
        k_scan_offsets<<<1, 1024, 0, s>>>(d_sizes, 1, tiles * tw, d_offsets, d_total);
    } else {
        k_tile_max_len<<<(uint32_t)((tiles + 127) / 128), 128, 0, s>>>(d_sizes, g.W, tiles, d_max_lens);
        CI_LAUNCH_CHECK(k_tile_max_len);
        k_scan_offsets<<<1, 1024, 0, s>>>(d_max_lens, g.W, tiles, d_offsets, d_total);
    }
    CI_LAUNCH_CHECK(k_scan_offsets);
    unsigned long long total = 0;
    CI_CUDA(cudaMemcpyAsync(&total, d_total, sizeof total, cudaMemcpyDeviceToHost, s));
    CI_CUDA(cudaFreeAsync(d_info, s));
    CI_CUDA(cudaFreeAsync(d_total, s));
    CI_CUDA(cudaStreamSynchronize(s));
    *stream_len = total;
    if (total > 0xFFFFFFFFull) {
        set_error("compressed stream of %llu bytes exceeds the format's 32-bit offsets", total);
        return CI_E_OVERFLOW;
    }
    return CI_OK;
}

template <bool DENSE>
static int encode_write(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                        uint32_t th, uint32_t tw, const uint32_t *d_sizes, const uint32_t *d_offsets,
                        const uint32_t *d_max_lens, uint8_t *d_stream, uint64_t stream_len, cudaStream_t s) {
    CI_REQUIRE(d_plane && d_offsets, "null pointer");
    CI_REQUIRE(DENSE || (d_sizes && d_max_lens), "null pointer");
    CI_REQUIRE(d_stream || stream_len == 0, "null stream buffer");
    int rc = check_tile(K, N, th, tw);
    if (rc) return rc;
    if (stream_len == 0) return CI_OK;
    Geom g = make_geom(K, N, th, tw);
    uint32_t *d_info = nullptr;
    rc = upload_sym_info(freqs, cdf, &d_info, s);
    if (rc) return rc;
    CI_CUDA(cudaMemsetAsync(d_stream, 0, stream_len, s));      // zero prefix above short streams
    EncArgs a{d_plane, K, N, th, tw, g.tiles_n, g.half};
    const uint32_t block = 128, slots = g.tiles_n * tw;
    dim3 grid((slots + block - 1) / block, g.tiles_k);
    k_encode<DENSE, true><<<grid, block, 0, s>>>(a, d_info, nullptr, nullptr, d_sizes, d_offsets, d_max_lens, d_stream);
    CI_LAUNCH_CHECK(k_encode);
    CI_CUDA(cudaFreeAsync(d_info, s));
    return CI_OK;
}

// Legacy flat layout, the inverse of k_decode_legacy: stream g holds the symbols at flat indices g,
// g + num_streams, ... encoded last first; byte b of a stream is stored at stream + g + b * num_streams, so
// the decoder, which starts at byte sizes[g] - 1, meets them in reverse order of emission.
// stream == nullptr: count only.
// seg_rows > 0 selects the reference encoder's own assignment instead (src/cuda/rans_kernels.cuh:393-509):
// stream g codes rows [seg * seg_rows, + seg_rows) of column g % cols, seg = g / cols.
__global__ void __launch_bounds__(128) k_encode_legacy(const uint8_t *__restrict__ data, uint64_t n, uint32_t num_streams,
                                                       const uint32_t *__restrict__ info, uint32_t *__restrict__ states,
                                                       uint32_t *__restrict__ sizes, uint8_t *__restrict__ stream,
                                                       uint32_t cols, uint32_t seg_rows) {
    __shared__ uint32_t s_info[256];
    load_sym_info(s_info, info);
    const uint32_t g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= num_streams) return;
    const uint64_t per_stream = seg_rows ? seg_rows : (n + num_streams - 1) / num_streams;
    const uint64_t seg_base = seg_rows ? (uint64_t)(g / cols) * seg_rows * cols + g % cols : g;
    const uint64_t step = seg_rows ? cols : num_streams;
    uint32_t state = kRansL, cnt = 0;
    for (uint64_t i = per_stream; i-- > 0;) {
        const uint64_t o = seg_base + i * step;
        if (o >= n) continue;
        const uint32_t inf = s_info[data[o]];
        const uint32_t freq = inf & 0xFFFFu, start = inf >> 16;
        const uint32_t x_max = freq << 12;
        while (state >= x_max) {
            if (stream) stream[(size_t)g + (size_t)cnt * num_streams] = (uint8_t)(state & 0xFFu);
            ++cnt;
            state >>= 8;
        }
        const uint32_t q = state / freq;
        state = (q << kProbBits) + (state - q * freq) + start;
    }
    if (states) states[g] = state;
    if (sizes) sizes[g] = cnt;
}

}  // namespace ci

using namespace ci;

extern "C" {

static int legacy_sizes(const uint8_t *d_data, uint64_t n, uint32_t num_streams, const uint16_t *freqs,
                        const uint16_t *cdf, uint32_t *d_states, uint32_t *d_sizes, uint32_t cols, uint32_t seg_rows,
                        ci_stream_t stream) {
    CI_REQUIRE(d_data && d_states && d_sizes && freqs && cdf, "null pointer");
    CI_REQUIRE(num_streams > 0 && n > 0, "empty input");
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t *d_info = nullptr;
    int rc = upload_sym_info(freqs, cdf, &d_info, s);
    if (rc) return rc;
    k_encode_legacy<<<(num_streams + 127) / 128, 128, 0, s>>>(d_data, n, num_streams, d_info, d_states, d_sizes, nullptr, cols, seg_rows);
    CI_LAUNCH_CHECK(k_encode_legacy);
    CI_CUDA(cudaFreeAsync(d_info, s));
    return CI_OK;
}

static int legacy_write(const uint8_t *d_data, uint64_t n, uint32_t num_streams, const uint16_t *freqs,
                        const uint16_t *cdf, uint8_t *d_stream, uint64_t stream_len, uint32_t cols, uint32_t seg_rows,
                        ci_stream_t stream) {
    CI_REQUIRE(d_data && freqs && cdf, "null pointer");
    CI_REQUIRE(d_stream || stream_len == 0, "null stream buffer");
    CI_REQUIRE(num_streams > 0 && n > 0, "empty input");
    if (stream_len == 0) return CI_OK;
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t *d_info = nullptr;
    int rc = upload_sym_info(freqs, cdf, &d_info, s);
    if (rc) return rc;
    CI_CUDA(cudaMemsetAsync(d_stream, 0, stream_len, s));
    k_encode_legacy<<<(num_streams + 127) / 128, 128, 0, s>>>(d_data, n, num_streams, d_info, nullptr, nullptr, d_stream, cols, seg_rows);
    CI_LAUNCH_CHECK(k_encode_legacy);
    CI_CUDA(cudaFreeAsync(d_info, s));
    return CI_OK;
}

int ci_encode_legacy_sizes(const uint8_t *d_data, uint64_t n, uint32_t num_streams, const uint16_t *freqs,
                           const uint16_t *cdf, uint32_t *d_states, uint32_t *d_sizes, ci_stream_t stream) {
    return legacy_sizes(d_data, n, num_streams, freqs, cdf, d_states, d_sizes, 1, 0, stream);
}
int ci_encode_legacy_write(const uint8_t *d_data, uint64_t n, uint32_t num_streams, const uint16_t *freqs,
                           const uint16_t *cdf, uint8_t *d_stream, uint64_t stream_len, ci_stream_t stream) {
    return legacy_write(d_data, n, num_streams, freqs, cdf, d_stream, stream_len, 1, 0, stream);
}
int ci_encode_legacy_segments_sizes(const uint8_t *d_data, uint32_t rows, uint32_t cols, uint32_t seg_rows,
                                    const uint16_t *freqs, const uint16_t *cdf, uint32_t *d_states, uint32_t *d_sizes,
                                    ci_stream_t stream) {
    CI_REQUIRE(rows > 0 && cols > 0 && seg_rows > 0, "empty plane or zero segment height");
    return legacy_sizes(d_data, (uint64_t)rows * cols, ((rows + seg_rows - 1) / seg_rows) * cols, freqs, cdf, d_states,
                        d_sizes, cols, seg_rows, stream);
}
int ci_encode_legacy_segments_write(const uint8_t *d_data, uint32_t rows, uint32_t cols, uint32_t seg_rows,
                                    const uint16_t *freqs, const uint16_t *cdf, uint8_t *d_stream, uint64_t stream_len,
                                    ci_stream_t stream) {
    CI_REQUIRE(rows > 0 && cols > 0 && seg_rows > 0, "empty plane or zero segment height");
    return legacy_write(d_data, (uint64_t)rows * cols, ((rows + seg_rows - 1) / seg_rows) * cols, freqs, cdf, d_stream,
                        stream_len, cols, seg_rows, stream);
}

int ci_encode_tiled_sizes(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t th, uint32_t tw, uint32_t *d_states, uint32_t *d_sizes, uint32_t *d_tile_offsets,
                          uint32_t *d_tile_max_lens, uint64_t *stream_len, ci_stream_t stream) {
    return encode_sizes<false>(d_plane, K, N, freqs, cdf, th, tw, d_states, d_sizes, d_tile_offsets, d_tile_max_lens,
                               stream_len, (cudaStream_t)stream);
}

int ci_encode_tiled_write(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t th, uint32_t tw, const uint32_t *d_sizes, const uint32_t *d_tile_offsets,
                          const uint32_t *d_tile_max_lens, uint8_t *d_stream, uint64_t stream_len, ci_stream_t stream) {
    return encode_write<false>(d_plane, K, N, freqs, cdf, th, tw, d_sizes, d_tile_offsets, d_tile_max_lens, d_stream,
                               stream_len, (cudaStream_t)stream);
}

int ci_encode_dense_sizes(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t th, uint32_t tw, uint32_t *d_states, uint32_t *d_sizes, uint32_t *d_stream_offsets,
                          uint64_t *stream_len, ci_stream_t stream) {
    return encode_sizes<true>(d_plane, K, N, freqs, cdf, th, tw, d_states, d_sizes, d_stream_offsets, nullptr,
                              stream_len, (cudaStream_t)stream);
}

int ci_encode_dense_write(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t th, uint32_t tw, const uint32_t *d_stream_offsets, uint8_t *d_stream,
                          uint64_t stream_len, ci_stream_t stream) {
    return encode_write<true>(d_plane, K, N, freqs, cdf, th, tw, nullptr, d_stream_offsets, nullptr, d_stream,
                              stream_len, (cudaStream_t)stream);
}

}  // extern "C"
