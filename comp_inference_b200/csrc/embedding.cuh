// Shared declarations of the fused decode + row gather kernels.
#pragma once
#include "common.cuh"

namespace ci {

struct EmbArgs {
    const uint8_t *stream;
    const uint32_t *states, *tables, *tile_offsets, *tile_max_lens, *lut;
    const uint8_t *slot_map, *mantissa;
    Geom g;
    const int64_t *ids;
    uint64_t n_ids;
    uint16_t *out;
    int64_t ldo;
};

// Four-streams-per-lane gather for 32-wide tiles (embedding4.cu): CI_OK when launched, 1 when the
// table does not qualify (the caller then uses the generic kernel), < 0 on error.
int launch_embedding4(const EmbArgs &a, uint32_t max_tile_len, cudaStream_t s);

}  // namespace ci
