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
// points of LlamaRMSNorm (normalised value to bf16, then the weight product to bf16).
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
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        float h = bf(xr[c]);
        if (rr) h = bf(float_to_bf16_bits(h + bf(rr[c])));      // the residual stream itself is bf16
        s_h[c] = h;
        ss += h * h;
    }
    const float inv = rsqrtf(block_sum(ss, s_red) / (float)cols + eps);
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float h = s_h[c];
        if (res_out) res_out[(size_t)row * ldo + c] = float_to_bf16_bits(h);
        const float n = bf(float_to_bf16_bits(h * inv));
        y[(size_t)row * ldy + c] = float_to_bf16_bits(n * bf(w[c]));
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
// grid = (heads_q, batch), block = 512 threads; head dimension d <= 256, a multiple of 64.
// The cache rows come from L2 / HBM, so what matters is how many loads are in flight: the score pass keeps
// four positions (eight 4-byte loads) per lane in the air, the value pass eight positions per thread.
constexpr uint32_t kAttnThreads = 512;

__global__ void __launch_bounds__(kAttnThreads) k_decode_attention(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k_cache,
                                                                   const uint16_t *__restrict__ v_cache,
                                                                   const int64_t *__restrict__ pos_p, uint32_t n_q,
                                                                   uint32_t n_kv, uint32_t d, uint32_t T, float scale,
                                                                   uint16_t *__restrict__ out, int64_t ldo) {
    extern __shared__ float s_mem[];                            // [T] scores, [d] query, [groups][d] partial outputs
    __shared__ float s_red[32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    float *s_score = s_mem, *s_q = s_mem + T, *s_part = s_q + d;
    const uint32_t h = blockIdx.x, b = blockIdx.y, kvh = h / (n_q / n_kv);
    int64_t pos = *pos_p;
    if (pos < 0) pos = 0;
    if (pos >= (int64_t)T) pos = T - 1;
    const uint32_t n_pos = (uint32_t)pos + 1;
    const uint16_t *qr = q + ((size_t)b * n_q + h) * d;
    const uint16_t *kb = k_cache + ((size_t)b * n_kv + kvh) * T * d;
    const uint16_t *vb = v_cache + ((size_t)b * n_kv + kvh) * T * d;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) s_q[i] = bf(qr[i]) * scale;
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    float mx = -INFINITY;
    // scores: a warp takes four positions per round (t, t + nw, t + 2 nw, t + 3 nw), lanes across the head dimension
    for (uint32_t t0 = warp; t0 < n_pos; t0 += 4 * nw) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t i = lane * 2; i < d; i += 64) {
            uint32_t two[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t t = min(t0 + u * nw, n_pos - 1);      // clamped: the result of a repeated row is dropped below
                two[u] = __ldg(reinterpret_cast<const uint32_t *>(kb + (size_t)t * d + i));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                acc[u] += s_q[i] * __uint_as_float(two[u] << 16) + s_q[i + 1] * __uint_as_float(two[u] & 0xFFFF0000u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float a = acc[u];
            for (int o = 16; o >= 1; o >>= 1) a += __shfl_xor_sync(kFull, a, o);
            const uint32_t t = t0 + u * nw;
            if (t < n_pos) {
                if (lane == 0) s_score[t] = a;
                mx = fmaxf(mx, a);
            }
        }
    }
    mx = block_max(mx, s_red);
    float sum = 0.f;
    for (uint32_t t = threadIdx.x; t < n_pos; t += blockDim.x) {
        const float e = __expf(s_score[t] - mx);
        s_score[t] = e;
        sum += e;
    }
    sum = block_sum(sum, s_red);                                // (its barriers also publish s_score)
    const float inv = 1.f / sum;
    // values: d / 2 threads form a group (a thread per pair of output dimensions), group g takes positions
    // g, g + groups, ...; eight positions per round
    const uint32_t per_group = d / 2, groups = blockDim.x / per_group;
    const uint32_t grp = threadIdx.x / per_group, i = (threadIdx.x % per_group) * 2;
    float a0 = 0.f, a1 = 0.f;
    if (grp < groups) {
        for (uint32_t t0 = grp; t0 < n_pos; t0 += 8 * groups) {
            uint32_t two[8];
            float p[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t t = t0 + u * groups;
                const bool in = t < n_pos;
                two[u] = __ldg(reinterpret_cast<const uint32_t *>(vb + (size_t)(in ? t : t0) * d + i));
                p[u] = in ? s_score[t] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                a0 += p[u] * __uint_as_float(two[u] << 16);
                a1 += p[u] * __uint_as_float(two[u] & 0xFFFF0000u);
            }
        }
        s_part[grp * d + i] = a0;
        s_part[grp * d + i + 1] = a1;
    }
    __syncthreads();
    for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) {
        float v = 0.f;
        for (uint32_t gI = 0; gI < groups; ++gI) v += s_part[gI * d + c];
        out[(size_t)b * ldo + (size_t)h * d + c] = float_to_bf16_bits(v * inv);
    }
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
    // few rows (decode steps): the row is short and latency-bound, so spread it over many threads
    const uint32_t threads = cols >= 4096 ? 1024u : (cols >= 1024 ? 512u : 256u);
    return launch_pdl(k_add_rmsnorm, dim3(rows), dim3(threads), (size_t)cols * sizeof(float), (cudaStream_t)stream, d_x, ldx,
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

int ci_decode_attention(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, const int64_t *d_pos,
                        uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t T, float scale,
                        uint16_t *d_out, int64_t ldo, ci_stream_t stream) {
    CI_REQUIRE(d_q && d_k_cache && d_v_cache && d_pos && d_out, "null pointer");
    CI_REQUIRE(head_dim % 64 == 0 && head_dim <= 256, "head dimension %u must be a multiple of 64, at most 256", head_dim);
    CI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "%u query heads over %u key/value heads", n_q, n_kv);
    CI_REQUIRE(T > 0 && T <= 8192, "cache length %u outside (0, 8192]", T);
    if (batch == 0) return CI_OK;
    const uint32_t groups = kAttnThreads / (head_dim / 2);
    return launch_pdl(k_decode_attention, dim3(n_q, batch), dim3(kAttnThreads),
                      (size_t)(T + head_dim + groups * head_dim) * sizeof(float), (cudaStream_t)stream, d_q, d_k_cache, d_v_cache, d_pos, n_q, n_kv, head_dim, T, scale, d_out, ldo);
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
