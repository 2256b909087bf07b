// Shared declarations of the stand-alone decoders.
#pragma once
#include "common.cuh"

namespace ci {

struct DecArgs {
    const uint8_t *stream;
    const uint32_t *states, *tables, *tile_offsets, *tile_max_lens, *lut;
    const uint8_t *slot_map, *mantissa;
    Geom g;
    uint32_t stream_aligned;   // stream pointer is 16-byte aligned
};

// Staged decoder (decode_staged.cu): CI_OK when launched, 1 when the tensor does not qualify
// (the caller then uses the generic kernel), < 0 on error.
// Four-streams-per-lane decoder for 32-wide tiles (decode4.cu); same return convention.
int launch_decode4(const DecArgs &a, uint32_t max_tile_len, bool bf16, void *out, cudaStream_t s);
int launch_decode_staged(const DecArgs &a, uint32_t max_tile_len, bool bf16, void *out, cudaStream_t s);

}  // namespace ci
