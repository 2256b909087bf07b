/*
 * comp_inference_b200 -- C ABI of the compressed-weight hot path (sm_100a).
 *
 * This is the boundary a binding of the reference project would attach to in
 * place of its own extension module (src/python_bindings.cpp) and of the Triton
 * kernels its Python ops launch.  Plain pointers and sizes only; every pointer
 * named "d_*" or living inside ci_tiled_weight is DEVICE memory, everything
 * else is host memory.  All launches go to the cudaStream_t passed as
 * `stream` (void* here so the header needs no CUDA include) and do not
 * synchronise unless stated.
 *
 * Return value: 0 on success, a negative CI_E_* code otherwise; the message of
 * the last failure on the calling thread is returned by ci_last_error().
 * There is no CPU fallback anywhere behind this header.
 *
 * File:line citations name the reference interface an entry point replaces
 * (paths relative to the reference project root).
 */
#ifndef COMP_INFERENCE_B200_H
#define COMP_INFERENCE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CI_ABI_VERSION 1

#define CI_OK 0
#define CI_E_INVALID (-1)   /* bad argument (shape, tile size, null pointer, alignment) */
#define CI_E_CUDA (-2)      /* a CUDA runtime call failed; ci_last_error() has its text   */
#define CI_E_OVERFLOW (-3)  /* compressed stream would exceed the format's 32-bit offsets */
#define CI_E_WORKSPACE (-4) /* caller-provided workspace too small                         */
#define CI_E_DEVICE (-5)    /* a kernel reported an error through its status word         */

typedef void *ci_stream_t; /* cudaStream_t */

/*
 * One compressed tensor W[K,N] in the reference's "coalesced ILP2" layout
 * (produced by RansManager.compress_tiled, src/python_bindings.cpp:302-347;
 * stored as rans_exp_* / rans_man_raw by comp_inference/rans_saving.py:383-475;
 * held by RansLinear / RansLMHead / RansEmbedding,
 * comp_inference/pytorch_runtime.py:414-425).
 *
 * Tile t = tk*ceil(N/tile_w) + tn covers rows [tk*tile_h, +tile_h) and columns
 * [tn*tile_w, +tile_w).  It owns 2*tile_w streams: t*2*tile_w + c codes the top
 * half rows of column c, + tile_w the bottom half.  Its bytes start at
 * tile_offsets[t] and form a row-major [tile_max_lens[t]][2*tile_w] matrix, one
 * column per stream, each stream bottom-aligned.  mantissa is the raw
 * sign+mantissa plane re-tiled to [tk][tn][tile_h][tile_w].
 */
typedef struct ci_tiled_weight {
    const uint8_t *stream;         /* rans_exp_stream          [stream_len]            */
    const uint32_t *states;        /* rans_exp_states          [tiles * 2 * tile_w]    */
    const uint32_t *tables;        /* rans_exp_tables          [256]  freq | cdf << 16 */
    const uint8_t *slot_map;       /* rans_exp_slot_map        [4096]                  */
    const uint32_t *tile_offsets;  /* rans_exp_tile_offsets    [tiles]                 */
    const uint32_t *tile_max_lens; /* rans_exp_tile_max_lens   [tiles]                 */
    const uint8_t *mantissa;       /* rans_man_raw             [tiles * tile_h * tile_w]; may be NULL for ci_decode_plane */
    const uint32_t *lut;           /* optional: [4096] from ci_prepare_lut, or NULL (kernels then build it themselves) */
    uint64_t stream_len;           /* bytes in stream                                   */
    uint32_t K, N;                 /* logical matrix                                    */
    uint32_t tile_h, tile_w;       /* tile_h % 16 == 0; tile_w a power of two <= 128   */
    uint32_t max_tile_len;         /* max over tile_max_lens if known, else 0           */
    uint32_t reserved;
} ci_tiled_weight;

/* Same tensor in the dense ("uncoalesced") layout: one stream per tile column,
 * streams concatenated (RansManager.compress_tiled_uncoalesced,
 * src/python_bindings.cpp:349-397; rans_exp_stream_offsets in rans_saving.py). */
typedef struct ci_dense_weight {
    const uint8_t *stream;
    const uint32_t *states;         /* [tiles * tile_w] */
    const uint32_t *stream_sizes;   /* [tiles * tile_w] */
    const uint32_t *stream_offsets; /* [tiles * tile_w] */
    const uint32_t *tables;
    const uint8_t *slot_map;
    const uint8_t *mantissa;
    const uint32_t *lut;
    uint64_t stream_len;
    uint32_t K, N, tile_h, tile_w;
} ci_dense_weight;

int ci_abi_version(void);
const char *ci_last_error(void);

/* ---- errors found on the device, malformed metadata ---------------------- */

/* The staged kernels never trap and never wait without a bound.  When a wait runs out, or a tile's
 * entry in tile_max_lens contradicts the descriptor's max_tile_len, they write a code into a status
 * word and finish with invalid output: 1 = a copy into shared memory did not arrive, 2 = metadata
 * mismatch, 9 = a peer rank did not answer (the tensor-parallel exchanges), other values = a pipeline
 * stage of the prefill GEMM gave up.  For ci_linear / ci_linear_transposed / ci_linear_dense the word
 * lives inside the workspace, at the address ci_workspace_status_word() returns (host arithmetic, no
 * CUDA call); the exchanges take a d_status argument of their own.
 *
 * ci_status copies a status word to the host on `stream` and WAITS for the stream.  0: the word was
 * zero.  CI_E_DEVICE: it was not; *code (may be NULL) receives it, ci_last_error() says what it means,
 * and with clear != 0 the word is reset so that later calls start clean.  This is the path the
 * reference lacks: its encoder's overflow flag is a by-value kernel argument that never reaches the
 * host (src/cuda/rans_kernels.cuh:145, src/cuda/rans_host.cuh:505-541). */
uint32_t *ci_workspace_status_word(void *d_workspace);
int ci_status(uint32_t *d_status_word, uint32_t *code, int clear, ci_stream_t stream);

/* Host.  Consistency of a tiled weight's metadata, given as HOST copies, before any kernel touches
 * it: tile count against the shape, every tile's byte block [offset, offset + max_len * 2 * tile_w)
 * inside the stream and not overlapping its predecessor, max_len <= tile_h (a symbol emits at most two
 * bytes) and <= max_tile_len when that is non-zero, n_states = tiles * 2 * tile_w, mantissa_len (0 =
 * not given) >= tiles * tile_h * tile_w, and -- when tables / slot_map are given -- frequencies that
 * sum to 4096 with matching cumulative values and slot map.  CI_E_INVALID names the first offender.
 * The reference loads whatever the file holds (comp_inference/pytorch_runtime.py:631-637). */
int ci_validate_tiled_metadata(const uint32_t *tile_offsets, const uint32_t *tile_max_lens, const uint32_t *tables,
                               const uint8_t *slot_map, uint64_t stream_len, uint64_t n_states, uint64_t mantissa_len,
                               uint32_t K, uint32_t N, uint32_t tile_h, uint32_t tile_w, uint32_t max_tile_len);

/* Device properties the host side sizes launches with (SM count etc.); fills
 * sm_count / max dynamic shared memory per block of the current device. */
int ci_device_info(int *sm_count, int *max_smem_per_block);

/* ---- tables ------------------------------------------------------------ */

/* Host.  Packed {freq,cdf} table and slot->symbol map from 12-bit frequencies.
 * Replaces the table packing of src/cuda/rans_host.cuh:476-488. */
int ci_build_tables(const uint16_t *freqs, const uint16_t *cdf, uint32_t *tables, uint8_t *slot_map);

/* Device.  Merges tables + slot_map into the 4096-entry decode table the
 * kernels keep in shared memory: entry[slot] = bias | sym << 12 | freq << 20,
 * bias = slot - cdf[sym].  (The reference's decoders do two dependent global
 * lookups per symbol instead: comp_inference/rans_triton.py:95-105.) */
int ci_prepare_lut(const uint32_t *d_tables, const uint8_t *d_slot_map, uint32_t *d_lut, ci_stream_t stream);

/* ---- bf16 split / merge, histogram ------------------------------------- */

/* Device.  bf16 bits [K,N] -> exponent plane u8 [K,N], sign+mantissa bytes
 * re-tiled to [tk][tn][tile_h][tile_w] (zero padded; tile_h = 0 keeps the plain
 * [K,N] order), and 256-bin histograms of both byte planes (u64[256] each,
 * zeroed by the call).  Replaces extract_exp_and_mantissa + interleave_mantissas
 * + the bincount of get_rans_lut (comp_inference/comp_inference.py:10-32, 35-64,
 * 190-191).  Any output may be NULL. */
int ci_split_bf16(const uint16_t *d_w, uint32_t K, uint32_t N, uint32_t tile_h, uint32_t tile_w,
                  uint8_t *d_exp_plane, uint8_t *d_mantissa_tiled, uint64_t *d_exp_hist256,
                  uint64_t *d_man_hist256, ci_stream_t stream);

/* Device.  256-bin histogram of a byte array (the np.bincount of get_rans_lut,
 * comp_inference/comp_inference.py:190-191); d_hist256 is zeroed by the call. */
int ci_histogram_u8(const uint8_t *d_data, uint64_t n, uint64_t *d_hist256, ci_stream_t stream);

/* Host.  12-bit frequency table from a 256-bin histogram with exactly the
 * rounding and fix-up rules of get_rans_lut (comp_inference/comp_inference.py:193-239). */
int ci_normalize_freqs(const uint64_t *hist256, uint16_t *freqs, uint16_t *cdf);

/* Device.  Inverse re-tiling of the mantissa plane (uninterleave_mantissas,
 * comp_inference/comp_inference.py:67-93). */
int ci_untile_mantissa(const uint8_t *d_tiled, uint32_t K, uint32_t N, uint32_t tile_h, uint32_t tile_w,
                       uint8_t *d_plane, ci_stream_t stream);

/* ---- encoder ------------------------------------------------------------ */

/* GPU encoder, ILP2 tiled layout, in two steps so that the caller owns every
 * allocation.  Replaces RansManager::compress_tiled_ilp2 (src/cuda/rans_ops.cu:205-410:
 * kernel src/cuda/rans_kernels.cuh:76-188 plus the single-threaded host repack
 * :328-370); the bytes are written straight into their final, packed place.
 *
 * Step 1 fills d_states, d_sizes [tiles*2*tile_w], d_tile_max_lens and
 * d_tile_offsets [tiles], returns the stream length in *stream_len and
 * SYNCHRONISES the stream (the caller needs the number to allocate).
 * Step 2 writes d_stream[stream_len] (the call zero-fills it first).
 * freqs / cdf are host arrays of 256.  tile_h % 16 == 0 is required
 * (src/cuda/rans_host.cuh:440-445). */
int ci_encode_tiled_sizes(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t tile_h, uint32_t tile_w, uint32_t *d_states, uint32_t *d_sizes,
                          uint32_t *d_tile_offsets, uint32_t *d_tile_max_lens, uint64_t *stream_len,
                          ci_stream_t stream);
int ci_encode_tiled_write(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t tile_h, uint32_t tile_w, const uint32_t *d_sizes, const uint32_t *d_tile_offsets,
                          const uint32_t *d_tile_max_lens, uint8_t *d_stream, uint64_t stream_len, ci_stream_t stream);

/* Dense layout encoder (RansManager::compress_tiled_uncoalesced,
 * src/cuda/rans_ops.cu:74-203; kernel src/cuda/rans_kernels.cuh:7-74). */
int ci_encode_dense_sizes(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t tile_h, uint32_t tile_w, uint32_t *d_states, uint32_t *d_sizes,
                          uint32_t *d_stream_offsets, uint64_t *stream_len, ci_stream_t stream);
int ci_encode_dense_write(const uint8_t *d_plane, uint32_t K, uint32_t N, const uint16_t *freqs, const uint16_t *cdf,
                          uint32_t tile_h, uint32_t tile_w, const uint32_t *d_stream_offsets, uint8_t *d_stream,
                          uint64_t stream_len, ci_stream_t stream);

/* ---- decoders ----------------------------------------------------------- */

/* Exponent plane u8 [K,N].  Replaces rans_decomp_triton_tiled
 * (comp_inference/rans_triton.py:34-168). */
int ci_decode_plane(const ci_tiled_weight *w, uint8_t *d_out, ci_stream_t stream);

/* Full weight, bf16 bits [K,N] row-major.  Replaces the three passes of
 * rans_decompress_module_weight_bf16 (comp_inference/comp_inference.py:573-713:
 * tiled decode, uninterleave_mantissas, reconstruct_from_exp_and_mantissa). */
int ci_decode_bf16(const ci_tiled_weight *w, uint16_t *d_out, ci_stream_t stream);

/* Dense-layout counterparts. */
int ci_decode_plane_dense(const ci_dense_weight *w, uint8_t *d_out, ci_stream_t stream);
int ci_decode_bf16_dense(const ci_dense_weight *w, uint16_t *d_out, ci_stream_t stream);

/* ---- fused consumers ---------------------------------------------------- */

/* Bytes of workspace ci_linear / ci_linear_transposed need for M activation
 * rows and n_out output features (0 is a valid answer). */
size_t ci_linear_workspace_bytes(uint32_t M, uint32_t n_out, uint32_t K, uint32_t tile_h);

/* y[M,N] = x[M,K] . W[K,N] (+ bias[N]), W decoded on the fly and never written
 * to global memory.  x, bias, y are bf16 bits; x rows are x_row_stride elements
 * apart, y rows y_row_stride.  Accumulation is fp32.  Replaces
 * fused_rans_linear_triton (comp_inference/linear_triton.py:229-552) and, for
 * large M, the decompress + triton_matmul pair (comp_inference/triton_gemm.py:324-337).
 * d_workspace must hold ci_linear_workspace_bytes() bytes and must have been
 * zero-filled once when allocated; each call leaves it zeroed again.
 * split_k = 0 lets the library choose. */
int ci_linear(const ci_tiled_weight *w, const uint16_t *d_x, int64_t x_row_stride, uint32_t M, const uint16_t *d_bias,
              uint16_t *d_y, int64_t y_row_stride, void *d_workspace, size_t workspace_bytes, uint32_t split_k,
              ci_stream_t stream);

/* Which kernel ci_linear (split_k = 0, aligned buffers, a workspace) runs for this weight and M rows:
 * 0 = generic split-K kernel, 1 = staged two-streams-per-lane kernel (k_linear_mma), 2 = register-direct
 * four-streams-per-lane kernel (k_linear_mma4), 3 = tcgen05 decode-GEMM (k_linear_gemm).  Launches nothing;
 * benchmarks label their roofline with it. */
int ci_linear_route(const ci_tiled_weight *w, uint32_t M);

/* ci_linear for callers that cannot allocate device memory (no counterpart in the reference).
 *
 * Meant for hosts that are forbidden to call cudaMalloc or any allocating routine while the model
 * runs -- a server whose device memory was handed out in advance and whose allocator is closed, a
 * plug-in that is only given input and output buffers.  The ticket counters and fp32 partial sums
 * that ci_linear takes as d_workspace live in a fixed 16 MiB array inside the library instead
 * (ci_linear_static_max_bytes()); every GPU that loads the library holds that array until exit.
 * The call itself allocates nothing and frees nothing.
 *
 * Limits: M <= 16 activation rows, and ci_linear_workspace_bytes(M, N, K, tile_h) must fit in the
 * array (true for N up to about 16000 at M = 16); otherwise CI_E_WORKSPACE with the sizes in
 * ci_last_error().  The first call on a device looks up the array's device address (with that
 * device current); make that first call outside any stream capture.  All calls on a device share
 * the array: two calls that overlap on the GPU (different streams, no ordering) race on it. */
size_t ci_linear_static_max_bytes(void);
int ci_linear_static(const ci_tiled_weight *w, const uint16_t *d_x, int64_t x_row_stride, uint32_t M,
                     const uint16_t *d_bias, uint16_t *d_y, int64_t y_row_stride, ci_stream_t stream);
/* ci_status for the built-in array of ci_linear_static (the caller has no pointer to it).  The status
 * word is not touched by the per-call clearing of the ticket counters, so a code written by one call
 * is still there after the next.  Allocates nothing; waits for `stream`.  No counterpart in the reference. */
int ci_linear_static_status(uint32_t *code, int clear, ci_stream_t stream);

/* y[M,V] = x[M,H] . W[V,H]^T for a weight stored as [K=V, N=H] (LM head / tied
 * embedding).  Replaces fused_rans_linear_transposed_triton
 * (comp_inference/transposed_linear_triton.py:187-435). */
int ci_linear_transposed(const ci_tiled_weight *w, const uint16_t *d_x, int64_t x_row_stride, uint32_t M,
                         const uint16_t *d_bias, uint16_t *d_y, int64_t y_row_stride, void *d_workspace,
                         size_t workspace_bytes, ci_stream_t stream);

/* out[i,:] = W[ids[i],:] as bf16 bits; ids outside [0,K) give a zero row.
 * Replaces fused_rans_embedding_triton (comp_inference/embedding_triton.py:170-330). */
int ci_embedding(const ci_tiled_weight *w, const int64_t *d_ids, uint64_t n_ids, uint16_t *d_out,
                 int64_t out_row_stride, ci_stream_t stream);

/* Dense-layout fused linear and embedding (comp_inference/linear_triton.py:1044-1265,
 * comp_inference/embedding_triton.py:333-483). */
int ci_linear_dense(const ci_dense_weight *w, const uint16_t *d_x, int64_t x_row_stride, uint32_t M,
                    const uint16_t *d_bias, uint16_t *d_y, int64_t y_row_stride, void *d_workspace,
                    size_t workspace_bytes, uint32_t split_k, ci_stream_t stream);
int ci_embedding_dense(const ci_dense_weight *w, const int64_t *d_ids, uint64_t n_ids, uint16_t *d_out,
                       int64_t out_row_stride, ci_stream_t stream);
/* Dense-layout LM head: y[M,V] = x[M,H] . W[V,H]^T for W stored [K=V, N=H], one stream per tile column.
 * Replaces fused_rans_linear_transposed_triton_uncoalesced
 * (comp_inference/transposed_linear_triton.py:660-883). */
int ci_linear_transposed_dense(const ci_dense_weight *w, const uint16_t *d_x, int64_t x_row_stride, uint32_t M,
                               const uint16_t *d_bias, uint16_t *d_y, int64_t y_row_stride, void *d_workspace,
                               size_t workspace_bytes, ci_stream_t stream);

/* ---- legacy flat layout -------------------------------------------------- */

/* Decoder of the non-tiled legacy layout: stream g yields the symbols at flat
 * indices g, g+num_streams, ...; its bytes sit at stride num_streams and are read
 * from index sizes[g]-1 downwards.  Replaces ccore.decompress
 * (src/python_bindings.cpp:61-78 -> src/cuda/rans_kernels.cuh:626-708). */
int ci_decode_legacy(const uint8_t *d_stream, uint64_t stream_len, const uint32_t *d_states, const uint32_t *d_sizes,
                     uint32_t num_streams, uint64_t output_len, const uint32_t *d_tables, const uint8_t *d_slot_map,
                     uint8_t *d_out, ci_stream_t stream);

/* Encoder of the same layout, two steps like the tiled encoder: _sizes writes the final state and byte count
 * of every stream (the caller takes the maximum count, allocates max * num_streams bytes), _write stores byte b
 * of stream g at d_stream[g + b * num_streams] (zero above a short stream).  num_streams as the reference chooses
 * it: ceil(rows / min_block_size) * columns.  Replaces RansManager.compress
 * (src/python_bindings.cpp:225-299 -> src/cuda/rans_ops.cu:17-72); the reference's own legacy encoder assigns
 * symbols to streams by (row segment, column), which its decoder above does not invert, so this follows the
 * decoder. */
int ci_encode_legacy_sizes(const uint8_t *d_data, uint64_t n, uint32_t num_streams, const uint16_t *freqs,
                           const uint16_t *cdf, uint32_t *d_states, uint32_t *d_sizes, ci_stream_t stream);
int ci_encode_legacy_write(const uint8_t *d_data, uint64_t n, uint32_t num_streams, const uint16_t *freqs,
                           const uint16_t *cdf, uint8_t *d_stream, uint64_t stream_len, ci_stream_t stream);

/* The same flat byte arrangement with the symbol-to-stream assignment of the reference's legacy ENCODER
 * (src/cuda/rans_kernels.cuh:393-509) and of its Triton decoder rans_decomp_triton
 * (comp_inference/rans_triton.py:171-271): the plane is a row-major [rows, cols] matrix, stream
 * g = seg * cols + col codes rows [seg * seg_rows, + seg_rows) of column col (the reference fixes
 * seg_rows = 512); num_streams = ceil(rows / seg_rows) * cols. */
int ci_decode_legacy_segments(const uint8_t *d_stream, uint64_t stream_len, const uint32_t *d_states,
                              const uint32_t *d_sizes, uint32_t num_streams, uint32_t rows, uint32_t cols,
                              uint32_t seg_rows, const uint32_t *d_tables, const uint8_t *d_slot_map, uint8_t *d_out,
                              ci_stream_t stream);
int ci_encode_legacy_segments_sizes(const uint8_t *d_data, uint32_t rows, uint32_t cols, uint32_t seg_rows,
                                    const uint16_t *freqs, const uint16_t *cdf, uint32_t *d_states, uint32_t *d_sizes,
                                    ci_stream_t stream);
int ci_encode_legacy_segments_write(const uint8_t *d_data, uint32_t rows, uint32_t cols, uint32_t seg_rows,
                                    const uint16_t *freqs, const uint16_t *cdf, uint8_t *d_stream, uint64_t stream_len,
                                    ci_stream_t stream);

/* ---- between the linears of a decode step ----------------------------------------- */

/* The weightless steps of a Llama-style decode step, one launch each instead of the thirty-odd element-wise
 * launches of eager PyTorch; bf16 bits in and out, fp32 arithmetic.  No counterpart in the reference, which has
 * no decode loop of its own (tests/test_rans_pytorch_runtime.py:89-118 calls Hugging Face's generate).
 *
 * ci_add_rmsnorm: h = x (+ res, if given); res_out = h (if given); y = rmsnorm(h) * weight, row by row,
 *   with LlamaRMSNorm's rounding points.  cols <= 12288.
 * ci_rope_kv: rotary embedding (rotate-half convention) of position *d_pos on q [batch, n_q * d] and
 *   k [batch, n_kv * d] (row strides ldq / ldk / ldv), from bf16 cos / sin tables [T, d]; writes
 *   q_out [batch, n_q, d], k_cache[b][h][*d_pos][:] and v_cache[b][h][*d_pos][:] (caches [batch, n_kv, T, d]).
 * ci_decode_attention: out[b][h*d ...] = softmax(scale * q[b][h] . K[b][h / (n_q / n_kv)][0 .. *d_pos]^T) . V
 *   (d = 64, 128 or 256; T <= 32768).  The positions of a query are cut into ranges, one CTA each; d_workspace
 *   (ci_decode_attention_workspace_bytes, 16-byte aligned, zeroed once; calls leave its ticket area zeroed) holds the
 *   ranges' partial results.  Calls that overlap on the GPU must not share a workspace.
 * ci_silu_mul: out = silu(gate) * up over [rows, cols] with row strides. */
int ci_add_rmsnorm(const uint16_t *d_x, int64_t ldx, const uint16_t *d_res, int64_t ldr, const uint16_t *d_weight, float eps,
                   uint32_t rows, uint32_t cols, uint16_t *d_y, int64_t ldy, uint16_t *d_res_out, int64_t ldo,
                   ci_stream_t stream);
int ci_rope_kv(const uint16_t *d_q, int64_t ldq, const uint16_t *d_k, int64_t ldk, const uint16_t *d_v, int64_t ldv,
               const uint16_t *d_cos, const uint16_t *d_sin, const int64_t *d_pos, uint32_t batch, uint32_t n_q,
               uint32_t n_kv, uint32_t head_dim, uint32_t T, uint16_t *d_q_out, uint16_t *d_k_cache, uint16_t *d_v_cache,
               ci_stream_t stream);
size_t ci_decode_attention_workspace_bytes(uint32_t batch, uint32_t n_q, uint32_t head_dim, uint32_t T);
int ci_decode_attention(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, const int64_t *d_pos,
                        uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t T, float scale,
                        void *d_workspace, size_t workspace_bytes, uint16_t *d_out, int64_t ldo, ci_stream_t stream);
int ci_silu_mul(const uint16_t *d_gate, int64_t ldg, const uint16_t *d_up, int64_t ldu, uint32_t rows, uint32_t cols,
                uint16_t *d_out, int64_t ldo, ci_stream_t stream);

/* ---- tensor-parallel exchange ---------------------------------------------- */

/* One-shot all-reduce (sum) of a small bf16 tensor over peer memory, for the outputs of row-parallel linears.
 * No counterpart in the reference (it has no multi-GPU code); a tensor-parallel port of it would call an NCCL
 * all-reduce here.  Every rank owns a buffer of ci_allreduce_buffer_bytes(world, capacity) bytes that all peers
 * can write (CUDA IPC / symmetric memory), zeroed once, plus ci_allreduce_counter_bytes() of zeroed local memory.
 * peer_bufs is a host array of `world` device pointers: rank q's buffer as mapped into this process (entry `rank`
 * is the local one).  capacity (elements) must be a multiple of 8.  Every rank must make the same sequence of
 * calls; a rank that waits longer than a few seconds for a peer sets *d_status to 9 and returns garbage instead
 * of hanging.  d_in == d_out is allowed. */
size_t ci_allreduce_buffer_bytes(uint32_t world, uint32_t capacity);
size_t ci_allreduce_counter_bytes(void);
int ci_allreduce_oneshot(const uint16_t *d_in, uint16_t *d_out, uint32_t n, uint32_t capacity, void *const *peer_bufs,
                         uint32_t *d_counters, uint32_t rank, uint32_t world, uint32_t *d_status, ci_stream_t stream);
/* One-shot all-gather with the same buffers, protocol and bounds: every rank contributes a bf16 block
 * [rows, cols] (cols even, rows * cols <= capacity) and receives d_out[rows, world * cols] with rank q's block in
 * columns [q * cols, (q + 1) * cols) -- the logits of a vocabulary-parallel LM head.  Give it a buffer and
 * counters of its own (do not share them with an all-reduce: the call sequences are counted per buffer).
 * d_in and d_out must differ.  No counterpart in the reference; a port would call an NCCL all-gather. */
int ci_allgather_oneshot(const uint16_t *d_in, uint16_t *d_out, uint32_t rows, uint32_t cols, uint32_t capacity,
                         void *const *peer_bufs, uint32_t *d_counters, uint32_t rank, uint32_t world, uint32_t *d_status,
                         ci_stream_t stream);
/* How often ci_allreduce_oneshot re-reads a slot before it gives up on a peer (process-wide; 0 restores
 * the default of about a second).  For tests of the give-up path and for hosts with their own watchdog. */
void ci_allreduce_set_poll_limit(uint32_t polls);

/* Row-parallel fused decode-linear with the all-reduce inside the kernel: y[M, N] = sum over ranks of
 * x_rank[M, K_rank] . W_rank[K_rank, N] (+ bias, added once after the sum).  The warps that hold a column group's
 * final sums push them into every peer's exchange buffer and add the peers' (same tagged 8-byte protocol and
 * buffer size as ci_allreduce_oneshot; use a buffer of its own), so no partial output is written and no second
 * kernel runs.  M <= 2, N even, M * N <= capacity, dense output rows; d_counter: ci_linear_allreduce_counter_bytes()
 * of zeroed local memory.  Returns CI_E_INVALID when the weight does not qualify for the staged GEMV kernels
 * (the caller then runs ci_linear followed by ci_allreduce_oneshot).  No counterpart in the reference. */
size_t ci_linear_allreduce_counter_bytes(void);
/* 1 if ci_linear_allreduce would take this weight for M rows, 0 if it would answer CI_E_INVALID, < 0 on a
 * malformed descriptor.  Launches nothing.  Shards differ in their deepest tile, so the answer can differ
 * between ranks: a tensor-parallel group takes the minimum over its ranks once, at set-up, and all ranks
 * then use the same route for that layer. */
int ci_linear_allreduce_qualifies(const ci_tiled_weight *w, uint32_t M);
int ci_linear_allreduce(const ci_tiled_weight *w, const uint16_t *d_x, int64_t x_row_stride, uint32_t M,
                        const uint16_t *d_bias, uint16_t *d_y, void *d_workspace, size_t workspace_bytes,
                        void *const *peer_bufs, uint32_t capacity, uint32_t *d_counter, uint32_t rank, uint32_t world,
                        uint32_t *d_status, ci_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* COMP_INFERENCE_B200_H */
