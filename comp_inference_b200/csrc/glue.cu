// The weightless steps between the fused decode-linears of a Llama-style decode step, one kernel each:
// residual add + RMSNorm, rotary embedding + KV-cache write, single-query attention over the cache,
// SiLU(gate) * up.  In eager PyTorch these are some thirty small launches per layer; at batch 1 on a
// tensor-parallel rank, where each compressed GEMV takes 10 microseconds, they would dominate the token
// time.  The reference leaves them to Hugging Face's modules (it has no decode loop of its own:
// tests/test_rans_pytorch_runtime.py:89-118 calls model.generate).
//
// All tensors are bf16 bits; arithmetic is fp32 with one rounding at the end.  Every kernel starts with
// griddepcontrol.wait so that it can be launched programmatically behind the kernel that produces its input.
#include "common.cuh"

namespace ci {

__device__ __forceinline__ float bf(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }

__device__ __forceinline__ float block_sum(float v, float *s_red) {
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = lane < nw ? s_red[lane] : 0.f;
    for (int o = 16; o >= 1; o >>= 1) t += __shfl_xor_sync(kFull, t, o);
    return t;
}
__device__ __forceinline__ float block_max(float v, float *s_red) {
    for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = lane < nw ? s_red[lane] : -INFINITY;
    for (int o = 16; o >= 1; o >>= 1) t = fmaxf(t, __shfl_xor_sync(kFull, t, o));
    return t;
}

// h = x (+ res);  res_out = h (bf16);  y = bf16(bf16(h * rsqrt(mean(h^2) + eps)) * w)   -- the rounding
// points of LlamaRMSNorm (normalised value to bf16, then the weight product to bf16).  VEC: every row pointer is
// 8-byte aligned and cols % 4 == 0, so a thread moves four values per load / store.
template <bool VEC>
__global__ void __launch_bounds__(1024) k_add_rmsnorm(const uint16_t *__restrict__ x, int64_t ldx,
                                                     const uint16_t *__restrict__ res, int64_t ldr,
                                                     const uint16_t *__restrict__ w, float eps, uint32_t cols,
                                                     uint16_t *__restrict__ y, int64_t ldy, uint16_t *__restrict__ res_out,
                                                     int64_t ldo) {
    __shared__ float s_red[32];
    extern __shared__ float s_h[];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t row = blockIdx.x;
    const uint16_t *xr = x + (size_t)row * ldx, *rr = res ? res + (size_t)row * ldr : nullptr;
    float ss = 0.f;
    if (VEC) {
        for (uint32_t c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
            const uint2 xv = __ldg(reinterpret_cast<const uint2 *>(xr + c));
            float h[4] = {__uint_as_float(xv.x << 16), __uint_as_float(xv.x & 0xFFFF0000u), __uint_as_float(xv.y << 16),
                          __uint_as_float(xv.y & 0xFFFF0000u)};
            if (rr) {
                const uint2 rv = __ldg(reinterpret_cast<const uint2 *>(rr + c));
                const float r[4] = {__uint_as_float(rv.x << 16), __uint_as_float(rv.x & 0xFFFF0000u),
                                    __uint_as_float(rv.y << 16), __uint_as_float(rv.y & 0xFFFF0000u)};
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = bf(float_to_bf16_bits(h[j] + r[j]));   // the residual stream itself is bf16
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) { s_h[c + j] = h[j]; ss += h[j] * h[j]; }
        }
    } else {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
            float h = bf(xr[c]);
            if (rr) h = bf(float_to_bf16_bits(h + bf(rr[c])));
            s_h[c] = h;
            ss += h * h;
        }
    }
    const float inv = rsqrtf(block_sum(ss, s_red) / (float)cols + eps);
    if (VEC) {
        for (uint32_t c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
            const uint2 wv = __ldg(reinterpret_cast<const uint2 *>(w + c));
            const float wf[4] = {__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xFFFF0000u), __uint_as_float(wv.y << 16),
                                 __uint_as_float(wv.y & 0xFFFF0000u)};
            uint16_t hb[4], yb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float h = s_h[c + j];
                hb[j] = float_to_bf16_bits(h);
                yb[j] = float_to_bf16_bits(bf(float_to_bf16_bits(h * inv)) * wf[j]);
            }
            if (res_out)
                *reinterpret_cast<uint2 *>(res_out + (size_t)row * ldo + c) =
                    make_uint2(hb[0] | ((uint32_t)hb[1] << 16), hb[2] | ((uint32_t)hb[3] << 16));
            *reinterpret_cast<uint2 *>(y + (size_t)row * ldy + c) =
                make_uint2(yb[0] | ((uint32_t)yb[1] << 16), yb[2] | ((uint32_t)yb[3] << 16));
        }
    } else {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float h = s_h[c];
            if (res_out) res_out[(size_t)row * ldo + c] = float_to_bf16_bits(h);
            const float n = bf(float_to_bf16_bits(h * inv));
            y[(size_t)row * ldy + c] = float_to_bf16_bits(n * bf(w[c]));
        }
    }
}

// Rotary embedding of one new position (the same for every row of the batch) applied to q and k, and the
// KV-cache write: q_out[b][h][:] = rot(q), k_cache[b][h][pos][:] = rot(k), v_cache[b][h][pos][:] = v.
// rot(t)[i] = t[i] cos[i] - t[i + d/2] sin[i] for i < d/2, t[i] cos[i] + t[i - d/2] sin[i] above
// (the rotate_half convention of Hugging Face's Llama).  grid = (heads_q + 2 heads_kv, batch), block = d / 2.
__global__ void k_rope_kv(const uint16_t *__restrict__ q, int64_t ldq, const uint16_t *__restrict__ k, int64_t ldk,
                          const uint16_t *__restrict__ v, int64_t ldv, const uint16_t *__restrict__ cos_t,
                          const uint16_t *__restrict__ sin_t, const int64_t *__restrict__ pos_p, uint32_t n_q, uint32_t n_kv,
                          uint32_t d, uint32_t T, uint16_t *__restrict__ q_out, uint16_t *__restrict__ k_cache,
                          uint16_t *__restrict__ v_cache) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t h = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = d / 2;
    int64_t pos = *pos_p;
    if (pos < 0) pos = 0;
    if (pos >= (int64_t)T) pos = T - 1;
    if (h < n_q + n_kv) {
        const bool is_q = h < n_q;
        const uint32_t hh = is_q ? h : h - n_q;
        const uint16_t *src = (is_q ? q + (size_t)b * ldq : k + (size_t)b * ldk) + (size_t)hh * d;
        uint16_t *dst = is_q ? q_out + ((size_t)b * n_q + hh) * d : k_cache + (((size_t)b * n_kv + hh) * T + pos) * d;
        const float lo = bf(src[i]), hi = bf(src[i + half]);
        const float c0 = bf(cos_t[pos * d + i]), s0 = bf(sin_t[pos * d + i]);
        const float c1 = bf(cos_t[pos * d + i + half]), s1 = bf(sin_t[pos * d + i + half]);
        dst[i] = float_to_bf16_bits(lo * c0 - hi * s0);
        dst[i + half] = float_to_bf16_bits(hi * c1 + lo * s1);
    } else {
        const uint32_t hh = h - n_q - n_kv;
        const uint16_t *src = v + (size_t)b * ldv + (size_t)hh * d;
        uint16_t *dst = v_cache + (((size_t)b * n_kv + hh) * T + pos) * d;
        dst[i] = src[i];
        dst[i + half] = src[i + half];
    }
}

// One query per (batch row, head) against cache positions 0 .. pos: softmax(q . K^T / sqrt(d)) . V.
// grid = (heads_q, batch, splits), block = 256 threads; head dimension d in {64, 128, 256}.
// The cache rows come from L2 / HBM and a decode step has few (batch x heads) queries, so the positions of one
// query are cut into `splits` ranges, one CTA each; a CTA keeps several 16-byte loads per lane in flight
// (d / 8 lanes cover one cache row), leaves (max, sum, unnormalised output) of its range in the workspace and
// draws a ticket; the CTA that draws the last ticket of a query merges the ranges and writes bf16.
constexpr uint32_t kAttnThreads = 256;
constexpr uint32_t kAttnMaxSplits = 8;
constexpr uint32_t kAttnTickets = 4096;      // ticket counters at the head of the workspace: a fixed area, so that calls
                                             // of different batch sizes can share one workspace (partials never overlap it)

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xFFFF0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xFFFF0000u);
}

__global__ void __launch_bounds__(kAttnThreads) k_decode_attention(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k_cache,
                                                                   const uint16_t *__restrict__ v_cache,
                                                                   const int64_t *__restrict__ pos_p, uint32_t n_q,
                                                                   uint32_t n_kv, uint32_t d, uint32_t T, float scale,
                                                                   uint32_t *tickets, float *partial, uint16_t *__restrict__ out,
                                                                   int64_t ldo) {
    extern __shared__ float s_mem[];                            // [chunk cap] scores, [d] query, [256 * 8] partial outputs
    __shared__ float s_red[32];
    __shared__ uint32_t s_last;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t splits = gridDim.z, sp = blockIdx.z;
    const uint32_t cap = (T + splits - 1) / splits;
    float *s_score = s_mem, *s_q = s_mem + cap, *s_part = s_q + d;
    const uint32_t h = blockIdx.x, b = blockIdx.y, kvh = h / (n_q / n_kv);
    int64_t pos = *pos_p;
    if (pos < 0) pos = 0;
    if (pos >= (int64_t)T) pos = T - 1;
    const uint32_t n_pos = (uint32_t)pos + 1;
    const uint32_t chunk = (n_pos + splits - 1) / splits;       // <= cap
    const uint32_t p0 = min(sp * chunk, n_pos), n = min(p0 + chunk, n_pos) - p0;
    const uint16_t *qr = q + ((size_t)b * n_q + h) * d;
    const uint16_t *kb = k_cache + (((size_t)b * n_kv + kvh) * T + p0) * d;
    const uint16_t *vb = v_cache + (((size_t)b * n_kv + kvh) * T + p0) * d;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) s_q[i] = bf(qr[i]) * scale;
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t lpr = d / 8;                                 // lanes per cache row: 8, 16 or 32
    const uint32_t sub = lane % lpr, rsel = lane / lpr, rpw = 32 / lpr;
    float qv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) qv[j] = s_q[sub * 8 + j];
    float mx = -INFINITY;
    // scores: a warp takes rpw rows per load and four loads per round
    for (uint32_t base = warp * rpw; base < n; base += 4 * nw * rpw) {
        uint4 kv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t t = base + u * nw * rpw + rsel;
            kv[u] = __ldg(reinterpret_cast<const uint4 *>(kb + (size_t)min(t, n - 1) * d) + sub);   // clamped; dropped below
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float f[8], a = 0.f;
            unpack8(kv[u], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) a += qv[j] * f[j];
            for (uint32_t o = lpr >> 1; o >= 1; o >>= 1) a += __shfl_xor_sync(kFull, a, o);
            const uint32_t t = base + u * nw * rpw + rsel;
            if (t < n) {
                if (sub == 0) s_score[t] = a;
                mx = fmaxf(mx, a);
            }
        }
    }
    mx = block_max(mx, s_red);
    float sum = 0.f;
    for (uint32_t t = threadIdx.x; t < n; t += blockDim.x) {
        const float e = __expf(s_score[t] - mx);
        s_score[t] = e;
        sum += e;
    }
    sum = block_sum(sum, s_red);                                // (its barriers also publish s_score)
    // values: lpr threads form a group (eight output dimensions each), group pg takes rows pg, pg + groups, ...
    const uint32_t groups = blockDim.x / lpr, pg = threadIdx.x / lpr, dg = threadIdx.x % lpr;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t base = pg; base < n; base += 4 * groups) {
        uint4 vv[4];
        float p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t t = base + u * groups;
            vv[u] = __ldg(reinterpret_cast<const uint4 *>(vb + (size_t)min(t, n - 1) * d) + dg);
            p[u] = t < n ? s_score[t] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float f[8];
            unpack8(vv[u], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += p[u] * f[j];
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s_part[pg * d + dg * 8 + j] = acc[j];
    __syncthreads();
    float o = 0.f;                                              // thread c < d owns output dimension c
    if (threadIdx.x < d)
        for (uint32_t gI = 0; gI < groups; ++gI) o += s_part[gI * d + threadIdx.x];
    uint16_t *dst = out + (size_t)b * ldo + (size_t)h * d;
    if (splits == 1) {
        if (threadIdx.x < d) dst[threadIdx.x] = float_to_bf16_bits(o / sum);
        return;
    }
    // several ranges: leave (max, sum, output) of this one in the workspace; the last arriver merges
    const uint32_t query = b * n_q + h;
    float *mine = partial + ((size_t)query * splits + sp) * (d + 2);
    if (threadIdx.x < d) mine[2 + threadIdx.x] = o;
    if (threadIdx.x == 0) { mine[0] = mx; mine[1] = sum; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t seen = atomicAdd(tickets + query, 1u);
        s_last = seen == splits - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x < d) {
        const float *all = partial + (size_t)query * splits * (d + 2);
        float M = -INFINITY;
        for (uint32_t s = 0; s < splits; ++s) M = fmaxf(M, __ldcg(all + s * (d + 2)));
        float L = 0.f, O = 0.f;
        for (uint32_t s = 0; s < splits; ++s) {                 // fixed order; an empty range has sum 0 and max -inf
            const float w = __expf(__ldcg(all + s * (d + 2)) - M);
            L += w * __ldcg(all + s * (d + 2) + 1);
            O += w * __ldcg(all + s * (d + 2) + 2 + threadIdx.x);
        }
        dst[threadIdx.x] = float_to_bf16_bits(O / L);
    }
    if (threadIdx.x == 0) tickets[query] = 0;                   // ready for the next call
}

// out = silu(gate) * up, element-wise over [rows, cols]; the product of the two bf16 values as PyTorch forms it
// (silu rounded to bf16, then the product).
__global__ void __launch_bounds__(256) k_silu_mul(const uint16_t *__restrict__ gate, int64_t ldg, const uint16_t *__restrict__ up,
                                                  int64_t ldu, uint32_t rows, uint32_t cols, uint16_t *__restrict__ out,
                                                  int64_t ldo) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint64_t total = (uint64_t)rows * cols;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(idx / cols), c = (uint32_t)(idx % cols);
        const float g = bf(gate[(size_t)r * ldg + c]);
        const float s = bf(float_to_bf16_bits(g / (1.f + __expf(-g))));
        out[(size_t)r * ldo + c] = float_to_bf16_bits(s * bf(up[(size_t)r * ldu + c]));
    }
}

template <typename... Args>
static int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CI_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
    return CI_OK;
}

}  // namespace ci

using namespace ci;

extern "C" {

int ci_add_rmsnorm(const uint16_t *d_x, int64_t ldx, const uint16_t *d_res, int64_t ldr, const uint16_t *d_weight, float eps,
                   uint32_t rows, uint32_t cols, uint16_t *d_y, int64_t ldy, uint16_t *d_res_out, int64_t ldo,
                   ci_stream_t stream) {
    CI_REQUIRE(d_x && d_weight && d_y, "null pointer");
    CI_REQUIRE(cols > 0 && cols <= 12288, "row length %u outside (0, 12288]", cols);
    if (rows == 0) return CI_OK;
    auto al8 = [](const void *p, int64_t ld) { return p == nullptr || ((reinterpret_cast<uintptr_t>(p) & 7u) == 0 && ld % 4 == 0); };
    const bool vec = cols % 4 == 0 && al8(d_x, ldx) && al8(d_res, ldr) && al8(d_weight, 0) && al8(d_y, ldy) && al8(d_res_out, ldo);
    // few rows (decode steps): the row is short and latency-bound, so spread it over many threads
    const uint32_t per = vec ? 4u : 1u;
    uint32_t threads = (cols / per + 31u) & ~31u;
    if (threads > 1024) threads = 1024;
    if (threads < 128) threads = 128;
    if (vec)
        return launch_pdl(k_add_rmsnorm<true>, dim3(rows), dim3(threads), (size_t)cols * sizeof(float), (cudaStream_t)stream,
                          d_x, ldx, d_res, ldr, d_weight, eps, cols, d_y, ldy, d_res_out, ldo);
    return launch_pdl(k_add_rmsnorm<false>, dim3(rows), dim3(threads), (size_t)cols * sizeof(float), (cudaStream_t)stream, d_x, ldx,
                      d_res, ldr, d_weight, eps, cols, d_y, ldy, d_res_out, ldo);
}

int ci_rope_kv(const uint16_t *d_q, int64_t ldq, const uint16_t *d_k, int64_t ldk, const uint16_t *d_v, int64_t ldv,
               const uint16_t *d_cos, const uint16_t *d_sin, const int64_t *d_pos, uint32_t batch, uint32_t n_q,
               uint32_t n_kv, uint32_t head_dim, uint32_t T, uint16_t *d_q_out, uint16_t *d_k_cache, uint16_t *d_v_cache,
               ci_stream_t stream) {
    CI_REQUIRE(d_q && d_k && d_v && d_cos && d_sin && d_pos && d_q_out && d_k_cache && d_v_cache, "null pointer");
    CI_REQUIRE(head_dim >= 2 && head_dim % 2 == 0 && head_dim <= 2048, "head dimension %u not supported", head_dim);
    CI_REQUIRE(n_q > 0 && n_kv > 0 && T > 0, "empty geometry");
    if (batch == 0) return CI_OK;
    return launch_pdl(k_rope_kv, dim3(n_q + 2 * n_kv, batch), dim3(head_dim / 2), 0, (cudaStream_t)stream, d_q, ldq, d_k, ldk,
                      d_v, ldv, d_cos, d_sin, d_pos, n_q, n_kv, head_dim, T, d_q_out, d_k_cache, d_v_cache);
}

static uint32_t attention_splits(uint32_t batch, uint32_t n_q, uint32_t T) {
    const uint32_t queries = batch * n_q, want = 2 * (uint32_t)sm_count();
    uint32_t s = (want + queries - 1) / queries;                // about two CTAs per multiprocessor
    const uint32_t by_len = (T + 63) / 64;                      // at least 64 positions per range
    if (s > by_len) s = by_len;
    if (s > kAttnMaxSplits) s = kAttnMaxSplits;
    return s < 1 ? 1 : s;
}

size_t ci_decode_attention_workspace_bytes(uint32_t batch, uint32_t n_q, uint32_t head_dim, uint32_t T) {
    const size_t queries = (size_t)batch * n_q;
    return (size_t)kAttnTickets * sizeof(uint32_t) + queries * attention_splits(batch, n_q, T) * (head_dim + 2) * sizeof(float);
}

int ci_decode_attention(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, const int64_t *d_pos,
                        uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t T, float scale,
                        void *d_workspace, size_t workspace_bytes, uint16_t *d_out, int64_t ldo, ci_stream_t stream) {
    CI_REQUIRE(d_q && d_k_cache && d_v_cache && d_pos && d_out, "null pointer");
    CI_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "head dimension %u must be 64, 128 or 256", head_dim);
    CI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "%u query heads over %u key/value heads", n_q, n_kv);
    CI_REQUIRE(T > 0 && T <= 32768, "cache length %u outside (0, 32768]", T);
    CI_REQUIRE(((reinterpret_cast<uintptr_t>(d_k_cache) | reinterpret_cast<uintptr_t>(d_v_cache)) & 15u) == 0,
               "KV caches must be 16-byte aligned");
    if (batch == 0) return CI_OK;
    uint32_t splits = attention_splits(batch, n_q, T);
    CI_REQUIRE((size_t)batch * n_q <= kAttnTickets, "%u x %u queries exceed the %u the workspace has tickets for", batch, n_q,
               kAttnTickets);
    if (splits > 1) {
        CI_REQUIRE(d_workspace != nullptr && (reinterpret_cast<uintptr_t>(d_workspace) & 15u) == 0, "attention needs an aligned workspace");
        if (workspace_bytes < ci_decode_attention_workspace_bytes(batch, n_q, head_dim, T)) {
            set_error("attention workspace of %zu bytes, %zu needed", workspace_bytes,
                      ci_decode_attention_workspace_bytes(batch, n_q, head_dim, T));
            return CI_E_WORKSPACE;
        }
    }
    uint32_t *tickets = reinterpret_cast<uint32_t *>(d_workspace);
    float *partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d_workspace) + (size_t)kAttnTickets * sizeof(uint32_t));
    const uint32_t cap = (T + splits - 1) / splits;
    const size_t smem = (size_t)(cap + head_dim + kAttnThreads * 8) * sizeof(float);
    static SmemLimit lim = {};
    if (smem > 48 * 1024)
        if (int rc = ensure_smem_limit(lim, (const void *)k_decode_attention, smem)) return rc;
    return launch_pdl(k_decode_attention, dim3(n_q, batch, splits), dim3(kAttnThreads), smem, (cudaStream_t)stream, d_q,
                      d_k_cache, d_v_cache, d_pos, n_q, n_kv, head_dim, T, scale, tickets, partial, d_out, ldo);
}

int ci_silu_mul(const uint16_t *d_gate, int64_t ldg, const uint16_t *d_up, int64_t ldu, uint32_t rows, uint32_t cols,
                uint16_t *d_out, int64_t ldo, ci_stream_t stream) {
    CI_REQUIRE(d_gate && d_up && d_out, "null pointer");
    if (rows == 0 || cols == 0) return CI_OK;
    uint64_t blocks = ((uint64_t)rows * cols + 255) / 256, cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    return launch_pdl(k_silu_mul, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, d_gate, ldg, d_up, ldu, rows,
                      cols, d_out, ldo);
}

}  // extern "C"
