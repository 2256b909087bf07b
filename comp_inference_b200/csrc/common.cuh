// Shared host/device helpers of the compressed-weight kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/comp_inference_b200.h"

namespace ci {

// rANS parameters of the format: src/cuda/rans.cuh:23-52, src/cuda/rans_host.cuh:22-24
// (8-bit symbols, 32-bit state, byte renormalisation, 12-bit scale, L = 2^16).
constexpr uint32_t kProbBits = 12;
constexpr uint32_t kProbScale = 1u << kProbBits;
constexpr uint32_t kProbMask = kProbScale - 1;
constexpr uint32_t kRansL = 1u << 16;

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xFFFFFFFFu;

// ---- error plumbing -------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define CI_CUDA(call)                                                   \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return ::ci::cuda_fail(e__, #call);     \
    } while (0)

#define CI_REQUIRE(cond, ...)                                           \
    do {                                                                \
        if (!(cond)) { ::ci::set_error(__VA_ARGS__); return CI_E_INVALID; } \
    } while (0)

#define CI_LAUNCH_CHECK(name) CI_CUDA(cudaGetLastError())

int sm_count();

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a device's context, not to the process: a
// launcher keeps one SmemLimit per kernel and raises the limit once on every device it runs on.
struct SmemLimit {
    size_t granted[64];
};
int ensure_smem_limit(SmemLimit &st, const void *kernel, size_t bytes);

// ---- geometry ---------------------------------------------------------------
struct Geom {
    uint32_t K, N, th, tw;
    uint32_t tiles_k, tiles_n;
    uint32_t half;   // th / 2 : symbols per stream in a full tile
    uint32_t W;      // 2 * tw : streams per tile = bytes per tile row
    uint32_t groups; // 32-column groups per tile row = ceil(tiles_n * tw / 32)
};

inline Geom make_geom(uint32_t K, uint32_t N, uint32_t th, uint32_t tw) {
    Geom g;
    g.K = K; g.N = N; g.th = th; g.tw = tw;
    g.tiles_k = (K + th - 1) / th;
    g.tiles_n = (N + tw - 1) / tw;
    g.half = th / 2;
    g.W = 2 * tw;
    g.groups = (g.tiles_n * tw + 31) / 32;
    return g;
}

int check_tile(uint32_t K, uint32_t N, uint32_t th, uint32_t tw);
int check_weight(const ci_tiled_weight *w, bool need_mantissa);

#ifdef __CUDACC__

// ---- decode table -----------------------------------------------------------
// entry[slot] = bias | sym << 12 | freq << 20 with bias = slot - cdf[sym]: the two operands of the
// state update come out with one instruction each (freq = e >> 20, bias = e & 0xFFF).
// A frequency of 4096 (single-symbol alphabet) wraps to 0 in its 12-bit field;
// the state then stops being meaningful but every slot still maps to that one
// symbol and such a plane has no stream bytes, so decoding stays exact.
__device__ __forceinline__ uint32_t make_lut_entry(uint32_t slot, uint32_t sym, uint32_t packed) {
    uint32_t freq = packed & 0xFFFFu, cdf = packed >> 16;
    return ((slot - cdf) & 0xFFFu) | (sym << 12) | ((freq & 0xFFFu) << 20);
}

// Fills a 4096-entry shared-memory table, either by copying a prepared one or by
// merging tables + slot_map (two dependent loads per slot, L2 resident).
__device__ __forceinline__ void load_lut(uint32_t *s_lut, const uint32_t *lut, const uint32_t *tables,
                                         const uint8_t *slot_map) {
    if (lut != nullptr) {
        const uint4 *src = reinterpret_cast<const uint4 *>(lut);
        uint4 *dst = reinterpret_cast<uint4 *>(s_lut);
        for (uint32_t i = threadIdx.x; i < kProbScale / 4; i += blockDim.x) dst[i] = __ldg(src + i);
    } else {
        for (uint32_t i = threadIdx.x; i < kProbScale; i += blockDim.x) {
            uint32_t sym = __ldg(slot_map + i);
            s_lut[i] = make_lut_entry(i, sym, __ldg(tables + sym));
        }
    }
}

__device__ __forceinline__ uint32_t lut_sym(uint32_t e) { return (e >> 12) & 0xFFu; }

// One symbol: comp_inference/rans_triton.py:92-105 with the two lookups merged.
// Returns the table entry; the symbol is lut_sym(entry).
__device__ __forceinline__ uint32_t decode_symbol(uint32_t &state, const uint32_t *s_lut) {
    uint32_t e = s_lut[state & kProbMask];
    state = (e >> 20) * (state >> kProbBits) + (e & 0xFFFu);
    return e;
}

// bf16 bits from exponent symbol and sign+mantissa byte
// (comp_inference/rans_triton.py:12-28).
__device__ __forceinline__ uint32_t assemble_bf16(uint32_t sym, uint32_t man) {
    return ((man & 0x80u) << 8) | (sym << 7) | (man & 0x7Fu);
}
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits) { return __uint_as_float(bits << 16); }

__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
    // round to nearest even, NaN kept quiet
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// A stream cursor over bytes that live at `base + row * stride`, consumed from
// the last row towards row 0 (comp_inference/rans_triton.py:107-119).
// Shared-memory flavour: 32-bit offsets into a byte array.
struct SmemCursor {
    uint32_t pos;   // offset of the next byte to read
    uint32_t low;   // offset of row 0 of this stream; nothing below it may be read
};

template <int STRIDE_DYNAMIC = 1>
__device__ __forceinline__ void renorm_smem(uint32_t &state, SmemCursor &c, const uint8_t *s_bytes, uint32_t stride) {
    // first byte: common (about one symbol in three at 2.6 bit/symbol)
    if (state < kRansL && (int32_t)(c.pos - c.low) >= 0) {
        state = (state << 8) | s_bytes[c.pos];
        c.pos -= stride;
    }
    // second byte: only after very improbable symbols; skip the probe warp-wide when nobody needs it
    if (__any_sync(kFull, state < kRansL)) {
        if (state < kRansL && (int32_t)(c.pos - c.low) >= 0) {
            state = (state << 8) | s_bytes[c.pos];
            c.pos -= stride;
        }
    }
}

// Global-memory flavour (tiles too large to stage, or unaligned streams).
struct GmemCursor {
    const uint8_t *base;  // address of row 0 of this stream
    int32_t row;          // next row to read; < 0 when exhausted
};

__device__ __forceinline__ void renorm_gmem(uint32_t &state, GmemCursor &c, uint32_t stride) {
    if (state < kRansL && c.row >= 0) {
        state = (state << 8) | __ldg(c.base + (size_t)c.row * stride);
        c.row--;
    }
    if (__any_sync(kFull, state < kRansL)) {
        if (state < kRansL && c.row >= 0) {
            state = (state << 8) | __ldg(c.base + (size_t)c.row * stride);
            c.row--;
        }
    }
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

#endif  // __CUDACC__

}  // namespace ci
