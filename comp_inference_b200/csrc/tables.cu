// Error plumbing, table construction, bf16 split / mantissa tiling / histogram.
#include <math.h>
#include <stdarg.h>

#include "common.cuh"

namespace ci {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return CI_E_CUDA;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int ensure_smem_limit(SmemLimit &st, const void *kernel, size_t bytes) {
    int dev = 0;
    CI_CUDA(cudaGetDevice(&dev));
    CI_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (st.granted[dev] < bytes) {
        CI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        st.granted[dev] = bytes;
    }
    return CI_OK;
}

int check_tile(uint32_t K, uint32_t N, uint32_t th, uint32_t tw) {
    CI_REQUIRE(K > 0 && N > 0, "empty matrix %u x %u", K, N);
    // src/cuda/rans_host.cuh:440-445: the tile height must be a multiple of 16
    CI_REQUIRE(th >= 16 && th % 16 == 0, "tile height %u is not a positive multiple of 16", th);
    CI_REQUIRE(tw >= 1 && tw <= 128 && (tw & (tw - 1)) == 0, "tile width %u is not a power of two in [1,128]", tw);
    return CI_OK;
}

int check_weight(const ci_tiled_weight *w, bool need_mantissa) {
    CI_REQUIRE(w != nullptr, "null weight descriptor");
    int rc = check_tile(w->K, w->N, w->tile_h, w->tile_w);
    if (rc) return rc;
    CI_REQUIRE(w->states && w->tile_offsets && w->tile_max_lens, "null metadata pointer");
    CI_REQUIRE(w->stream || w->stream_len == 0, "null stream with non-zero length");
    CI_REQUIRE(w->lut || (w->tables && w->slot_map), "neither a prepared table nor tables + slot_map given");
    CI_REQUIRE(!need_mantissa || w->mantissa, "mantissa plane required");
    CI_REQUIRE(w->lut == nullptr || (reinterpret_cast<uintptr_t>(w->lut) & 15u) == 0, "prepared table must be 16-byte aligned");
    return CI_OK;
}

// ---------------------------------------------------------------- kernels ---

__global__ void k_prepare_lut(const uint32_t *__restrict__ tables, const uint8_t *__restrict__ slot_map,
                              uint32_t *__restrict__ lut) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kProbScale) {
        uint32_t sym = slot_map[i];
        lut[i] = make_lut_entry(i, sym, tables[sym]);
    }
}

// One thread per element of the row-major [K,N] matrix.
__global__ void k_split_bf16(const uint16_t *__restrict__ w, uint32_t K, uint32_t N, uint32_t th, uint32_t tw,
                             uint32_t tiles_n, uint8_t *__restrict__ exp_plane, uint8_t *__restrict__ man_tiled,
                             unsigned long long *__restrict__ hist, unsigned long long *__restrict__ man_hist) {
    __shared__ uint32_t s_hist[256], s_mhist[256];
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) { s_hist[i] = 0; s_mhist[i] = 0; }
    __syncthreads();
    const uint64_t total = (uint64_t)K * N;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t raw = w[idx];
        uint32_t e = (raw >> 7) & 0xFFu;                       // comp_inference.py:27
        uint32_t m = ((raw >> 15) << 7) | (raw & 0x7Fu);       // comp_inference.py:26,28,31
        if (exp_plane) exp_plane[idx] = (uint8_t)e;
        if (man_tiled) {
            if (th == 0) {
                man_tiled[idx] = (uint8_t)m;                    // plain [K,N] plane
            } else {
                uint32_t r = (uint32_t)(idx / N), c = (uint32_t)(idx - (uint64_t)r * N);
                uint64_t t = (uint64_t)(r / th) * tiles_n + c / tw;
                man_tiled[t * th * tw + (uint64_t)(r % th) * tw + (c % tw)] = (uint8_t)m;
            }
        }
        if (hist) atomicAdd(&s_hist[e], 1u);
        if (man_hist) atomicAdd(&s_mhist[m], 1u);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) {
        if (hist && s_hist[i]) atomicAdd(&hist[i], (unsigned long long)s_hist[i]);
        if (man_hist && s_mhist[i]) atomicAdd(&man_hist[i], (unsigned long long)s_mhist[i]);
    }
}

__global__ void k_histogram_u8(const uint8_t *__restrict__ data, uint64_t n, unsigned long long *__restrict__ hist) {
    __shared__ uint32_t s_hist[256];
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (uint64_t)gridDim.x * blockDim.x)
        atomicAdd(&s_hist[data[idx]], 1u);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x)
        if (s_hist[i]) atomicAdd(&hist[i], (unsigned long long)s_hist[i]);
}

__global__ void k_untile_mantissa(const uint8_t *__restrict__ tiled, uint32_t K, uint32_t N, uint32_t th, uint32_t tw,
                                  uint32_t tiles_n, uint8_t *__restrict__ plane) {
    const uint64_t total = (uint64_t)K * N;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t r = (uint32_t)(idx / N), c = (uint32_t)(idx - (uint64_t)r * N);
        uint64_t t = (uint64_t)(r / th) * tiles_n + c / tw;
        plane[idx] = tiled[t * th * tw + (uint64_t)(r % th) * tw + (c % tw)];
    }
}

}  // namespace ci

using namespace ci;

extern "C" {

int ci_abi_version(void) { return CI_ABI_VERSION; }

const char *ci_last_error(void) { return g_err; }

int ci_device_info(int *sms, int *max_smem) {
    int dev = 0;
    CI_CUDA(cudaGetDevice(&dev));
    if (sms) CI_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    if (max_smem) CI_CUDA(cudaDeviceGetAttribute(max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    return CI_OK;
}

int ci_build_tables(const uint16_t *freqs, const uint16_t *cdf, uint32_t *tables, uint8_t *slot_map) {
    CI_REQUIRE(freqs && cdf && tables && slot_map, "null pointer");
    uint32_t sum = 0;
    for (int s = 0; s < 256; ++s) sum += freqs[s];
    CI_REQUIRE(sum == kProbScale, "frequencies sum to %u, expected 4096", sum);
    memset(slot_map, 0, kProbScale);
    for (int s = 0; s < 256; ++s) {
        tables[s] = (uint32_t)freqs[s] | ((uint32_t)cdf[s] << 16);
        CI_REQUIRE((uint32_t)cdf[s] + freqs[s] <= kProbScale, "symbol %d: cdf + freq exceeds 4096", s);
        for (uint32_t j = 0; j < freqs[s]; ++j) slot_map[cdf[s] + j] = (uint8_t)s;
    }
    return CI_OK;
}

int ci_normalize_freqs(const uint64_t *hist, uint16_t *freqs, uint16_t *cdf) {
    CI_REQUIRE(hist && freqs && cdf, "null pointer");
    uint64_t total = 0;
    for (int s = 0; s < 256; ++s) total += hist[s];
    CI_REQUIRE(total > 0, "empty histogram");
    // comp_inference/comp_inference.py:197-198: floor(counts / counts.sum() * 4096) in float64, zeros -> 1
    long long f[256], sum = 0;
    const double tot = (double)total;
    for (int s = 0; s < 256; ++s) {
        double v = floor(((double)hist[s] / tot) * 4096.0);
        f[s] = (long long)v;
        if (f[s] == 0) f[s] = 1;
        sum += f[s];
    }
    long long diff = 4096 - sum;
    auto argmax = [&]() { int b = 0; for (int s = 1; s < 256; ++s) if (f[s] > f[b]) b = s; return b; };
    if (diff > 0) {
        f[argmax()] += diff;                                   // :204-206
    } else {
        while (diff < 0) {                                     // :215-227, one unit at a time
            int b = argmax();
            f[b] -= 1;
            CI_REQUIRE(f[b] >= 1, "frequency of symbol %d dropped to zero", b);
            diff += 1;
        }
    }
    uint32_t run = 0;
    for (int s = 0; s < 256; ++s) { cdf[s] = (uint16_t)run; freqs[s] = (uint16_t)f[s]; run += (uint32_t)f[s]; }
    CI_REQUIRE(run == kProbScale, "normalised frequencies sum to %u", run);
    return CI_OK;
}

int ci_prepare_lut(const uint32_t *d_tables, const uint8_t *d_slot_map, uint32_t *d_lut, ci_stream_t stream) {
    CI_REQUIRE(d_tables && d_slot_map && d_lut, "null pointer");
    k_prepare_lut<<<kProbScale / 256, 256, 0, (cudaStream_t)stream>>>(d_tables, d_slot_map, d_lut);
    CI_LAUNCH_CHECK(k_prepare_lut);
    return CI_OK;
}

int ci_split_bf16(const uint16_t *d_w, uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint8_t *d_exp,
                  uint8_t *d_man_tiled, uint64_t *d_hist, uint64_t *d_man_hist, ci_stream_t stream) {
    CI_REQUIRE(d_w != nullptr, "null input");
    CI_REQUIRE(K > 0 && N > 0, "empty matrix %u x %u", K, N);
    Geom g;
    memset(&g, 0, sizeof g);
    if (th != 0) {
        int rc = check_tile(K, N, th, tw);
        if (rc) return rc;
        g = make_geom(K, N, th, tw);
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (d_man_tiled && th != 0) CI_CUDA(cudaMemsetAsync(d_man_tiled, 0, (size_t)g.tiles_k * g.tiles_n * th * tw, s));
    if (d_hist) CI_CUDA(cudaMemsetAsync(d_hist, 0, 256 * sizeof(uint64_t), s));
    if (d_man_hist) CI_CUDA(cudaMemsetAsync(d_man_hist, 0, 256 * sizeof(uint64_t), s));
    uint64_t total = (uint64_t)K * N;
    uint32_t blocks = (uint32_t)((total + 255) / 256);
    uint32_t cap = (uint32_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    k_split_bf16<<<blocks, 256, 0, s>>>(d_w, K, N, th, tw, g.tiles_n, d_exp, d_man_tiled,
                                        reinterpret_cast<unsigned long long *>(d_hist),
                                        reinterpret_cast<unsigned long long *>(d_man_hist));
    CI_LAUNCH_CHECK(k_split_bf16);
    return CI_OK;
}

int ci_histogram_u8(const uint8_t *d_data, uint64_t n, uint64_t *d_hist, ci_stream_t stream) {
    CI_REQUIRE(d_hist && (d_data || n == 0), "null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    CI_CUDA(cudaMemsetAsync(d_hist, 0, 256 * sizeof(uint64_t), s));
    if (n == 0) return CI_OK;
    uint64_t blocks = (n + 255) / 256, cap = (uint64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    k_histogram_u8<<<(uint32_t)blocks, 256, 0, s>>>(d_data, n, reinterpret_cast<unsigned long long *>(d_hist));
    CI_LAUNCH_CHECK(k_histogram_u8);
    return CI_OK;
}

int ci_untile_mantissa(const uint8_t *d_tiled, uint32_t K, uint32_t N, uint32_t th, uint32_t tw, uint8_t *d_plane,
                       ci_stream_t stream) {
    CI_REQUIRE(d_tiled && d_plane, "null pointer");
    int rc = check_tile(K, N, th, tw);
    if (rc) return rc;
    Geom g = make_geom(K, N, th, tw);
    uint64_t total = (uint64_t)K * N;
    uint32_t blocks = (uint32_t)((total + 255) / 256);
    uint32_t cap = (uint32_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    k_untile_mantissa<<<blocks, 256, 0, (cudaStream_t)stream>>>(d_tiled, K, N, th, tw, g.tiles_n, d_plane);
    CI_LAUNCH_CHECK(k_untile_mantissa);
    return CI_OK;
}

}  // extern "C"
