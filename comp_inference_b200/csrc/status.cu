// Status words and metadata validation: the ways an error found on the device, or a malformed
// package found before anything runs, gets back to the caller through the C ABI.
//
// The staged kernels never trap and never spin without a bound; when a wait runs out or the tile
// metadata contradicts the descriptor they record a code in a status word and carry on with
// garbage.  The reference loses such information altogether (its encoder's overflow flag is passed
// by value and never reaches the host, src/cuda/rans_kernels.cuh:145); here it is read back with
// ci_status and reported as CI_E_DEVICE.
#include "linear.cuh"

using namespace ci;

extern "C" {

uint32_t *ci_workspace_status_word(void *d_workspace) {
    return d_workspace ? reinterpret_cast<uint32_t *>(d_workspace) + (kTicketBytes - 1) : nullptr;
}

int ci_status(uint32_t *d_status_word, uint32_t *code, int clear, ci_stream_t stream) {
    CI_REQUIRE(d_status_word != nullptr, "null status word");
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t v = 0;
    CI_CUDA(cudaMemcpyAsync(&v, d_status_word, sizeof v, cudaMemcpyDeviceToHost, s));
    CI_CUDA(cudaStreamSynchronize(s));
    if (code) *code = v;
    if (v == 0) return CI_OK;
    if (clear) CI_CUDA(cudaMemsetAsync(d_status_word, 0, sizeof v, s));
    const char *what = v == 1   ? "a bounded wait for a copy into shared memory ran out"
                       : v == 2 ? "tile_max_lens holds an entry above the descriptor's max_tile_len"
                       : v == 9 ? "a bounded wait for a peer rank ran out"
                                : "a kernel reported a pipeline error";
    set_error("device status %u: %s; the outputs of the affected calls are not valid", v, what);
    return CI_E_DEVICE;
}

int ci_validate_tiled_metadata(const uint32_t *tile_offsets, const uint32_t *tile_max_lens, const uint32_t *tables,
                               const uint8_t *slot_map, uint64_t stream_len, uint64_t n_states, uint64_t mantissa_len,
                               uint32_t K, uint32_t N, uint32_t tile_h, uint32_t tile_w, uint32_t max_tile_len) {
    CI_REQUIRE(tile_offsets && tile_max_lens, "null metadata pointer");
    int rc = check_tile(K, N, tile_h, tile_w);
    if (rc) return rc;
    const Geom g = make_geom(K, N, tile_h, tile_w);
    const uint64_t tiles = (uint64_t)g.tiles_k * g.tiles_n;
    CI_REQUIRE(n_states == tiles * g.W, "%llu initial states, %llu expected (tiles x 2 x tile width)",
               (unsigned long long)n_states, (unsigned long long)(tiles * g.W));
    CI_REQUIRE(mantissa_len == 0 || mantissa_len >= tiles * tile_h * tile_w, "sign+mantissa plane of %llu bytes, %llu expected",
               (unsigned long long)mantissa_len, (unsigned long long)(tiles * tile_h * tile_w));
    uint64_t floor_off = 0;
    for (uint64_t t = 0; t < tiles; ++t) {
        const uint64_t off = tile_offsets[t], len = tile_max_lens[t], bytes = len * g.W;
        // a symbol emits at most two bytes (state < 2^24, renormalisation threshold >= 2^12), a stream codes
        // tile_h / 2 symbols: no byte block is deeper than tile_h rows
        CI_REQUIRE(len <= tile_h, "tile %llu: tile_max_lens = %llu exceeds what %u rows can emit",
                   (unsigned long long)t, (unsigned long long)len, tile_h);
        CI_REQUIRE(max_tile_len == 0 || len <= max_tile_len, "tile %llu: tile_max_lens = %llu above the declared maximum %u",
                   (unsigned long long)t, (unsigned long long)len, max_tile_len);
        CI_REQUIRE(off >= floor_off, "tile %llu: offset %llu overlaps the previous tile's bytes (which end at %llu)",
                   (unsigned long long)t, (unsigned long long)off, (unsigned long long)floor_off);
        CI_REQUIRE(off + bytes <= stream_len, "tile %llu: bytes [%llu, %llu) run past the stream's %llu bytes",
                   (unsigned long long)t, (unsigned long long)off, (unsigned long long)(off + bytes),
                   (unsigned long long)stream_len);
        floor_off = off + bytes;
    }
    if (tables != nullptr) {
        uint32_t run = 0;
        for (uint32_t s = 0; s < 256; ++s) {
            const uint32_t freq = tables[s] & 0xFFFFu, cdf = tables[s] >> 16;
            CI_REQUIRE(cdf == run, "tables[%u]: cumulative %u, %u expected", s, cdf, run);
            CI_REQUIRE(run + freq <= kProbScale, "tables: frequencies exceed %u at symbol %u", kProbScale, s);
            if (slot_map != nullptr)
                for (uint32_t j = 0; j < freq; ++j)
                    CI_REQUIRE(slot_map[run + j] == s, "slot_map[%u] = %u, %u expected", run + j, slot_map[run + j], s);
            run += freq;
        }
        CI_REQUIRE(run == kProbScale, "tables: frequencies sum to %u, %u expected", run, kProbScale);
    }
    return CI_OK;
}

}  // extern "C"
