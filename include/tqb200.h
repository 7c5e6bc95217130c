/*
 * tqb200.h -- C ABI of the B200 TurboQuant engine (libtqb200.so).
 *
 * Plain pointers and sizes only.  Every pointer named "device" must be valid on the
 * CUDA device that is current when the call is made; launches are asynchronous on the
 * given stream unless stated otherwise.  Functions returning `int` return a tqb_status;
 * the `void` symbols of section 1 keep the reference's own signatures so that a Rust
 * `extern "C"` block written for the reference links unchanged.
 *
 * Citations are file:line inside the reference crate turboquant-rs 0.3.1.
 */
#ifndef TQB200_H
#define TQB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t / CUstream, passed as an opaque pointer (src/cache/cuda/ffi.rs:7). */
typedef void *tqb_stream_t;

/* Status codes.  1..5 mirror TurboQuantError (src/error.rs:4-29). */
typedef enum tqb_status {
    TQB_OK = 0,
    TQB_ERR_INVALID_DIMENSION = 1,   /* InvalidDimension: dim not a power of two / not a multiple of 32 */
    TQB_ERR_UNSUPPORTED_BITS = 2,    /* UnsupportedBits */
    TQB_ERR_DIMENSION_MISMATCH = 3,  /* DimensionMismatch */
    TQB_ERR_LAYER_OUT_OF_RANGE = 4,  /* LayerOutOfRange */
    TQB_ERR_RANGE_OUT_OF_BOUNDS = 5, /* RangeOutOfBounds */
    TQB_ERR_NULL_POINTER = 6,
    TQB_ERR_INVALID_ARGUMENT = 7,
    TQB_ERR_MISALIGNED = 8,
    TQB_ERR_UNSUPPORTED = 9,         /* valid for the reference, outside what this build covers */
    TQB_ERR_CUDA = 10,               /* a CUDA call failed; see tqb_last_cuda_error() */
    TQB_ERR_OUT_OF_MEMORY = 11,
    TQB_ERR_TOO_LARGE = 12,          /* exceeds a fixed capacity of the called entry point */
    TQB_ERR_PEER_TIMEOUT = 13        /* a bounded device-side wait for another rank's data ran out */
} tqb_status;

const char *tqb_status_string(int status);
/* cudaError_t of the last failing CUDA call made by this library on the calling thread. */
int tqb_last_cuda_error(void);
/* Library version, for the loader's sanity check. */
int tqb_version(void);

/* Element types accepted for K, V, Q and outputs. */
typedef enum tqb_dtype { TQB_F32 = 0, TQB_F16 = 1, TQB_BF16 = 2 } tqb_dtype;
/* QuantNormMode (src/cache/config.rs:21-31). */
typedef enum tqb_norm_mode { TQB_MAXNORM = 0, TQB_L2NORM = 1 } tqb_norm_mode;
/* outlier_blocks = usize::MAX in the reference (src/cache/config.rs:49-50). */
#define TQB_ALL_BLOCKS (-1)

/* =====================================================================================
 * 1. The reference's own FFI (src/cache/cuda/ffi.rs:10-79), same names and arguments.
 *    Defined in the reference at tq_dequant_kernel.cu:104, tq_quant_kernel.cu:416,441,
 *    tq_attention_kernel.cu:337.  All pointers are device pointers.  `void`, no error
 *    report, early return on zero counts -- exactly the reference's convention; the
 *    tqb_* twins in section 2 do the same work and return a status.
 * ===================================================================================== */
void tq_dequant_batch(const uint8_t *packed_indices, const uint16_t *scales, const float *codebook,
                      const float *sign_pattern, float *output, int32_t num_blocks, int32_t block_size,
                      int32_t bits, int32_t bytes_per_block, tqb_stream_t stream);

void tq_quant_maxnorm_batch(const float *rotated_input, const float *boundaries, uint8_t *packed_out,
                            uint16_t *scales_out, int32_t num_blocks, int32_t block_size, int32_t bits,
                            int32_t num_boundaries, int32_t bytes_per_block, float outer_centroid,
                            float scale_sign, tqb_stream_t stream);

void tq_pack_indices(const uint8_t *indices, uint8_t *packed_out, int32_t num_vectors, int32_t block_size,
                     int32_t bits, int32_t bytes_per_block, tqb_stream_t stream);

void tq_fused_attention(const float *q, const uint8_t *k_indices, const uint16_t *k_scales,
                        const uint8_t *v_indices, const uint16_t *v_scales, const float *codebook,
                        const float *sign_pattern, float *output, float *partial_out, float *partial_max,
                        float *partial_sum, const uint8_t *qjl_signs, const uint16_t *qjl_residual_norms,
                        const float *rq, int32_t qjl_enabled, int32_t num_attention_heads,
                        int32_t num_kv_heads, int32_t head_dim, int32_t kv_len, int32_t kv_stride,
                        int32_t packed_dim, int32_t num_qblocks, int32_t bits, float softmax_scale,
                        int32_t num_partitions, tqb_stream_t stream);

/* =====================================================================================
 * 2. Status-returning twins of section 1 (same arguments, validated before any launch).
 * ===================================================================================== */
int tqb_dequant_batch(const uint8_t *packed_indices, const uint16_t *scales, const float *codebook,
                      const float *sign_pattern, float *output, int32_t num_blocks, int32_t block_size,
                      int32_t bits, int32_t bytes_per_block, tqb_stream_t stream);
int tqb_quant_maxnorm_batch(const float *rotated_input, const float *boundaries, uint8_t *packed_out,
                            uint16_t *scales_out, int32_t num_blocks, int32_t block_size, int32_t bits,
                            int32_t num_boundaries, int32_t bytes_per_block, float outer_centroid,
                            float scale_sign, tqb_stream_t stream);
int tqb_pack_indices(const uint8_t *indices, uint8_t *packed_out, int32_t num_vectors, int32_t block_size,
                     int32_t bits, int32_t bytes_per_block, tqb_stream_t stream);
int tqb_fused_attention(const float *q, const uint8_t *k_indices, const uint16_t *k_scales,
                        const uint8_t *v_indices, const uint16_t *v_scales, const float *codebook,
                        const float *sign_pattern, float *output, float *partial_out, float *partial_max,
                        float *partial_sum, const uint8_t *qjl_signs, const uint16_t *qjl_residual_norms,
                        const float *rq, int32_t qjl_enabled, int32_t num_attention_heads,
                        int32_t num_kv_heads, int32_t head_dim, int32_t kv_len, int32_t kv_stride,
                        int32_t packed_dim, int32_t num_qblocks, int32_t bits, float softmax_scale,
                        int32_t num_partitions, tqb_stream_t stream);

/* =====================================================================================
 * 3. Whole-vector format of the core crate, batched over n vectors resident on the device.
 *    Storage is the flat layout of PackedImport (src/attention.rs:147-166):
 *      packed  [n, tqb_packed_bytes(bits, dim)]  u8   bit stream of src/packed/mod.rs:242-309
 *      scales  [n]                               u16  IEEE f16 bits of the L2 norm
 *      signs   [n, dim/8]                        u8   QJL sign bits, LSB first
 *      rnorms  [n]                               u16  f16 bits of the residual norm
 * ===================================================================================== */

/* TurboQuantConfig (src/packed/mod.rs:93-139): bits in {2,3,4}, dim a power of two.
 * This build carries the reference's twelve static codebooks (src/codebook/tables.rs),
 * i.e. dim in {32, 64, 128, 256}; other powers of two return TQB_ERR_UNSUPPORTED. */
typedef struct tqb_config {
    int32_t bits;
    int32_t dim;
    uint64_t rotation_seed;
} tqb_config;

int tqb_config_validate(const tqb_config *cfg);
/* Bytes of the packed index stream for `count` codes (src/packed/indices.rs). */
size_t tqb_packed_bytes(int32_t bits, size_t count);
/* get_codebook (src/codebook/mod.rs:118-122): copies 2^bits centroids and 2^bits-1
 * boundaries (f64) to host arrays. */
int tqb_get_codebook(int32_t bits, int32_t dim, double *centroids, double *boundaries);
/* generate_sign_pattern (src/rotation.rs:60-70), host output. */
int tqb_generate_sign_pattern(int32_t dim, uint64_t seed, float *out);

/* quantize_vec over a batch (src/quantize.rs:142-157).  x: device [n, dim] f32. */
int tqb_quantize_batch(const tqb_config *cfg, const float *x, int64_t n, uint8_t *packed, uint16_t *scales,
                       tqb_stream_t stream);
/* dequantize_vec over a batch (src/quantize.rs:207-239).  out: device [n, dim] f32. */
int tqb_dequantize_batch(const tqb_config *cfg, const uint8_t *packed, const uint16_t *scales, int64_t n,
                         float *out, tqb_stream_t stream);
/* dequantize_rotated (src/quantize.rs:306-316): no inverse rotation. */
int tqb_dequantize_rotated_batch(const tqb_config *cfg, const uint8_t *packed, const uint16_t *scales,
                                 int64_t n, float *out, tqb_stream_t stream);

/* The hash Rademacher matrix of src/qjl.rs:143-171 as a bit matrix: host output
 * [dim, dim/32] u32, bit c%32 of word [row, c/32] set when the entry is -1/sqrt(dim).
 * The QJL kernels read it from a device copy that the caller owns. */
int tqb_qjl_rademacher_bits(int32_t dim, uint64_t qjl_seed, uint32_t *host_out);

/* quantize_with_qjl over a batch (src/qjl.rs:355-377): cfg->bits is the TOTAL width
 * (3 or 4); the polar stage uses bits-1.  rbits: device bit matrix (see above). */
int tqb_qjl_quantize_batch(const tqb_config *cfg, const uint32_t *rbits, const float *x, int64_t n,
                           uint8_t *packed, uint16_t *scales, uint8_t *signs, uint16_t *rnorms,
                           tqb_stream_t stream);
/* precompute_query_projections (src/qjl.rs:488-492) for nq queries: rq [nq, dim]. */
int tqb_qjl_query_projections(int32_t dim, const uint32_t *rbits, const float *q, int64_t nq, float *rq,
                              tqb_stream_t stream);
/* QuantizedKVCache::attention_scores (src/attention.rs:319-353): raw, unscaled,
 * un-softmaxed scores [n] for one query.  cfg->bits is the total width. */
int tqb_qjl_attention_scores(const tqb_config *cfg, const float *q, const float *rq, const uint8_t *packed,
                             const uint16_t *scales, const uint8_t *signs, const uint16_t *rnorms, int64_t n,
                             float *scores, tqb_stream_t stream);
/* QuantizedKVCache::weighted_values (src/attention.rs:371-408): out [dim] = sum_i w[i] *
 * dequantize(polar part of value i).  scratch: device, tqb_weighted_values_scratch_bytes(). */
size_t tqb_weighted_values_scratch_bytes(int32_t dim);
int tqb_weighted_values(const tqb_config *cfg, const float *w, const uint8_t *packed, const uint16_t *scales,
                        int64_t n, float *out, void *scratch, size_t scratch_bytes, tqb_stream_t stream);

/* =====================================================================================
 * 4. Block-32 format of the cache module ("PQ" / "PQO" / "TQ" caches).
 *      indices [rows, head_dim*bits/8] u8, scales [rows, head_dim/32] u16 (f16 bits; a
 *      negative scale marks a block coded with the outlier codebook,
 *      src/cache/storage.rs:122-125, src/cache/quantize_tensor.rs:68-70).
 * ===================================================================================== */

/* CacheConfig (src/cache/config.rs:52-66) plus the two seeds (config.rs:15,18) and a
 * batch count (the reference is batch 1; equal-length sequences fold into heads). */
typedef struct tqb_cache_config {
    int32_t bits;           /* 3 or 4 */
    int32_t head_dim;       /* multiple of 32 */
    int32_t num_kv_heads;
    int32_t num_layers;
    int32_t norm_mode;      /* tqb_norm_mode */
    int32_t outlier_blocks; /* TQB_ALL_BLOCKS = PQO, 0 = PQ/TQ */
    int32_t batch;          /* >= 1 */
    int32_t reserved;
    uint64_t rotation_seed; /* unused for block size 32 (fixed pattern), kept for parity */
    uint64_t qjl_seed;
} tqb_cache_config;

/* build_codebooks (src/cache/precomputed/codebooks.rs:18-88): host output of the
 * codebook with 2^cb_bits entries for the norm mode; returns the entry count or <0. */
int tqb_block_codebook(int32_t cb_bits, int32_t norm_mode, float *centroids, float *boundaries);
/* The fixed 32-entry sign pattern (src/cache/precomputed/rotation.rs:16-20), host output. */
void tqb_block_sign_pattern(float *out32);

/* polar_quantize (src/cache/quantize_tensor.rs:40-79) with the rotation fused in
 * (replaces the sgemm at src/cache/cuda/quantize.rs:111-113 + tq_quant_maxnorm_batch).
 * x: device [n, head_dim] of x_dtype, rows x_row_stride elements apart (0 = dense).
 * Row i is written to output row  (i / rows_per_group) * out_group_stride + out_row_offset
 * + i % rows_per_group  -- with rows_per_group = new tokens, out_group_stride = capacity
 * and out_row_offset = old length this is CompressedStorage::append
 * (src/cache/storage.rs:145-172) without a staging copy.  rows_per_group = 0 means
 * dense output (row i -> i). */
int tqb_block_quantize(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks,
                       const void *x, int32_t x_dtype, int64_t n, int64_t x_row_stride, uint8_t *indices,
                       uint16_t *scales, int64_t rows_per_group, int64_t out_group_stride,
                       int64_t out_row_offset, tqb_stream_t stream);

/* The same for the K and V tensors of one append in ONE launch (the reference quantizes them one
 * after the other, quantize_kv_pair in src/cache/common.rs:102-111); both tensors share shape, dtype, stride and
 * row mapping. */
int tqb_block_quantize_pair(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks,
                            const void *k, const void *v, int32_t x_dtype, int64_t n, int64_t x_row_stride,
                            uint8_t *k_indices, uint16_t *k_scales, uint8_t *v_indices, uint16_t *v_scales,
                            int64_t rows_per_group, int64_t out_group_stride, int64_t out_row_offset,
                            tqb_stream_t stream);

/* polar_dequantize (src/cache/quantize_tensor.rs:179-220).  Input row mapping as above
 * (rows_per_group = 0: dense); out: device [n, head_dim] of out_dtype, dense. */
int tqb_block_dequantize(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks,
                         const uint8_t *indices, const uint16_t *scales, int64_t n, int64_t rows_per_group,
                         int64_t in_group_stride, int64_t in_row_offset, void *out, int32_t out_dtype,
                         tqb_stream_t stream);

/* Fused decode attention over the packed cache (tq_attention_kernel.cu:63-392,
 * src/cache/cuda/attention.rs:41-174), one query token per head.
 *   q, out      [num_q_heads, head_dim]   (batch folded into heads: query head h reads KV
 *                                          head h / (num_q_heads / num_kv_heads))
 *   k/v_indices [num_kv_heads, kv_stride, head_dim*bits/8], k/v_scales [.., head_dim/32]
 *   scratch     device, >= tqb_decode_scratch_bytes(...); holds the split-K partials.
 * With lse_out != NULL the per-head (max, sum) pair is written to lse_out[num_q_heads][2]
 * and `out` receives the UN-normalised output (f32 only): the shard-local result that a
 * sequence-parallel caller gathers and merges with tqb_lse_combine(). */
typedef struct tqb_decode_params {
    const void *q;
    const uint8_t *k_indices;
    const uint16_t *k_scales;
    const uint8_t *v_indices;
    const uint16_t *v_scales;
    void *out;
    float *lse_out;
    void *scratch;
    size_t scratch_bytes;
    const uint8_t *qjl_signs;     /* [num_kv_heads, kv_stride, head_dim/8] or NULL */
    const uint16_t *qjl_norms;    /* [num_kv_heads, kv_stride] or NULL */
    const float *rq;              /* [num_q_heads, head_dim] or NULL */
    int32_t qjl_enabled;
    int32_t q_dtype;
    int32_t out_dtype;
    int32_t bits;
    int32_t head_dim;
    int32_t norm_mode;
    int32_t outlier_blocks;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t kv_len;
    int32_t kv_stride;
    int32_t num_partitions;       /* 0 = let the library choose */
    float softmax_scale;
    int32_t flags;                /* TQB_DECODE_* bits */
    /* Optional fused append (src/cache/pqo.rs:106-174 quantizes the new token, stores it, then attends):
     * device [num_kv_heads, head_dim] of q_dtype each, or both NULL.  The vectors are quantized and written
     * to row kv_len - 1 of every KV head (kv_len counts the new token; the cache arrays are written
     * although declared const) before attention reads them - inside the attention kernel for the
     * tensor-core shapes, by one extra launch otherwise. */
    const void *append_k;
    const void *append_v;
} tqb_decode_params;

/* flags: stop after the split-K pass and leave the per-partition (max, sum, out) partials in
 * `scratch`; `out` is not written.  Scratch layout: merge tickets (1 + G u32 per query head, rounded up to
 * 256 bytes; G = 0 for P <= 16, else ceil(P / 8): the partition groups of the two-level merge), then
 * [num_q_heads, P, head_dim] f32, then [num_q_heads, P] max, then sum, then the group partials. */
#define TQB_DECODE_PARTIALS_ONLY 1
/* flags: always take the general (SIMT, any shape) kernel; used to cross-check the tensor-core kernels. */
#define TQB_DECODE_FORCE_GENERAL 2
/* flags: the caller vouches that the ticket area at the start of `scratch` is zero (zero-filled once when
 * the buffer was allocated; every completed call leaves it zero), so the library skips clearing it. */
#define TQB_DECODE_TICKETS_ZERO 4
/* flags: stage the packed tiles with the tensor copy engine (TMA: 2-D tiled maps with the 64-byte swizzle for
 * the index arrays, 1-D maps for the scale rows, one 64-token tile per CTA and stage) instead of per-warp
 * cp.async rings.  Same bits; measured 5 to 13 % slower on B200, so it is opt-in.  Falls back to cp.async by itself
 * when kv_stride is odd or a cache array is not 16-byte aligned. */
#define TQB_DECODE_TMA 8

/* flags (tqb_chunk_attention only): fold the chunk into decode launches (one per query token, see below) instead of
 * running the chunk kernel; the cross-check of that kernel. */
#define TQB_DECODE_FOLD_CHUNK 16

/* flags: this launch may START before the previous kernel on the stream has finished (programmatic dependent launch),
 * when that kernel is one of the library's tensor-core decode launches: its streaming pass then overlaps the
 * predecessor's tail and split-K merge, and waits for the predecessor's completion only before it writes the scratch,
 * the tickets and the outputs.  The caller vouches that nothing this launch READS - q, append_k / append_v, rq, the
 * cache arrays - is written by the immediately preceding kernel on the stream, except rows appended by that kernel
 * (those are stored and fenced before a successor may start).  Honoured together with TQB_DECODE_TICKETS_ZERO on the
 * head_dim-128 tensor-core path; ignored elsewhere (the launch is then ordered like any other). */
#define TQB_DECODE_OVERLAP 32

/* Diagnostic: how many bounded waits on a staged tile ran out on the current device since the library was
 * loaded (synchronises the device).  Always 0 in a healthy run; -1 on a CUDA error.  A non-zero count invalidates
 * the outputs of the TQB_DECODE_TMA calls since the last check.  No reference counterpart. */
long long tqb_decode_stage_timeouts(void);

/* Partitions the library would use for this shape, and the scratch it then needs. */
int32_t tqb_decode_num_partitions(int32_t num_kv_heads, int32_t kv_len);
/* The same for launches made with TQB_DECODE_OVERLAP: fewer, longer partitions (several launches are resident at
 * once, so one launch need not fill the GPU by itself). */
int32_t tqb_decode_num_partitions_overlapped(int32_t num_kv_heads, int32_t kv_len);
size_t tqb_decode_scratch_bytes(int32_t num_q_heads, int32_t head_dim, int32_t num_partitions);
int tqb_decode_attention(const tqb_decode_params *p, tqb_stream_t stream);

/* Causal attention of a chunk of q_len query tokens over the packed cache (the chunk's own K/V rows already
 * stored, e.g. by tqb_block_quantize_pair or tqb_pqo_cache_prefill).  No counterpart kernel in the reference:
 * its prefill dequantizes the whole cache and hands it to the engine's attention (src/cache/pqo.rs:184-200,
 * src/cache/common.rs:16-62).
 * head_dim 128, GQA group 1 / 2 / 4 / 8, PQO4 or a 3-bit format of the tensor-core kernels, no QJL: a dedicated kernel
 * on the tcgen05 tensor cores (128 query rows per CTA, every K / V tile unpacked once per CTA; scratch unused).  It
 * rounds the rotated query, the keys, the probabilities and the values to f16 once each: outputs within 1e-3 of the
 * CPU attention over the same bytes (the folded path: 1e-4).
 * Everything else, or TQB_DECODE_FOLD_CHUNK: the chunk is folded into the decode kernels, one grid head per query
 * token.  tqb_chunk_umma_timeouts() counts bounded waits of the dedicated kernel that ran out (always 0 in a healthy
 * run; a non-zero count invalidates the outputs since the last check; synchronises the device).
 *   q, out   [q_len, num_q_heads, head_dim] (token-major); query token i attends to the first
 *            kv_len - q_len + i + 1 tokens, so p->kv_len counts the chunk and must be >= q_len.
 *   scratch  >= tqb_decode_scratch_bytes(num_q_heads * q_len, head_dim, P), with P = p->num_partitions or
 *            tqb_decode_num_partitions(num_kv_heads * q_len, kv_len) when that is 0 (used by the folded path).
 *   lse_out  [q_len, num_q_heads][2] when given; append_k / append_v must be NULL; rq (QJL) is
 *            [q_len, num_q_heads, head_dim].  All other fields as for tqb_decode_attention. */
int tqb_chunk_attention(const tqb_decode_params *p, int32_t q_len, tqb_stream_t stream);
long long tqb_chunk_umma_timeouts(void);

/* tqb_decode_attention for callers that cannot allocate device memory.  No counterpart in the
 * reference (there the caller always allocates the partial buffers, src/cache/cuda/attention.rs:65-77).
 * Meant for hosts that have given all free device memory to their own pool at start-up, or that must
 * not take the device-wide synchronisation of cudaMalloc / cudaFree in their serving loop: the split-K
 * partials go into a fixed 8 MiB array inside the library image (held by every GPU that loads the
 * library, until exit), and the call performs no allocation of any kind.
 *   - p->scratch and p->scratch_bytes are ignored; inputs and outputs are still the caller's.
 *     TQB_DECODE_PARTIALS_ONLY is refused (TQB_ERR_INVALID_ARGUMENT): the partials would be left in an array
 *     the caller cannot address.
 *   - Shapes whose partials need more than tqb_decode_static_scratch_capacity() bytes
 *     (tqb_decode_scratch_bytes(num_q_heads, head_dim, partitions)) are refused with TQB_ERR_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress with
 *     that device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Every call
 *     clears the merge tickets at its start on the stream (TQB_DECODE_TICKETS_ZERO is ignored) and the
 *     kernels overwrite every partial slot they later read, so the caller clears nothing; but two calls
 *     that overlap on the GPU (different streams, no ordering) race on the array.  Order them on one
 *     stream or with events. */
size_t tqb_decode_static_scratch_capacity(void);
int tqb_decode_attention_static(const tqb_decode_params *p, tqb_stream_t stream);

/* Log-sum-exp merge of `num_shards` shard-local results (the algebra of
 * tq_fused_attention_reduce, tq_attention_kernel.cu:299-332, one level up):
 *   partial_out [num_shards, num_q_heads, head_dim] f32 un-normalised,
 *   partial_lse [num_shards, num_q_heads, 2] f32 (max, sum);  out [num_q_heads, head_dim]. */
int tqb_lse_combine(const float *partial_out, const float *partial_lse, int32_t num_shards,
                    int32_t num_q_heads, int32_t head_dim, void *out, int32_t out_dtype, tqb_stream_t stream);
/* The same for shards packed one record per shard, [num_q_heads * head_dim floats of out | num_q_heads * 2 floats
 * of (max, sum)]: the layout a single all-gather of one flat buffer per rank produces. */
int tqb_lse_combine_packed(const float *gathered, int32_t num_shards, int32_t num_q_heads, int32_t head_dim,
                           void *out, int32_t out_dtype, tqb_stream_t stream);

/* =====================================================================================
 * 5. Host-side cache objects (own their device memory; calls are ordered on `stream`).
 * ===================================================================================== */

/* PqoCache (src/cache/pqo.rs:21-236) over CompressedStorage (src/cache/storage.rs:24-203).
 * k, v: [batch, num_kv_heads, new_tokens, head_dim]; q: [batch, num_q_heads, 1, head_dim];
 * `host_buffers` != 0 means k, v, q and the outputs are HOST pointers (pinned or pageable)
 * and the copies are part of the call. */
typedef struct tqb_pqo_cache tqb_pqo_cache;
int tqb_pqo_cache_create(const tqb_cache_config *cfg, tqb_pqo_cache **out);
void tqb_pqo_cache_destroy(tqb_pqo_cache *c);
/* prefill (pqo.rs:184-200): quantize and append.  When the layer already held tokens and
 * k_out/v_out are non-NULL they receive the full dequantized cache
 * [batch, num_kv_heads, seq_len, head_dim]; on the first call the reference returns the
 * original tensors, so nothing is written. */
int tqb_pqo_cache_prefill(tqb_pqo_cache *c, int32_t layer, const void *k, const void *v, int32_t dtype,
                          int32_t new_tokens, void *k_out, void *v_out, int32_t host_buffers,
                          tqb_stream_t stream);
/* decode (pqo.rs:202-222): append one token per sequence, then fused attention;
 * out: [batch, num_q_heads, 1, head_dim] of `dtype` (DecodeOutput::Fused). */
int tqb_pqo_cache_decode(tqb_pqo_cache *c, int32_t layer, const void *k, const void *v, const void *q,
                         int32_t dtype, int32_t num_q_heads, float softmax_scale, void *out,
                         int32_t host_buffers, tqb_stream_t stream);
/* With host_buffers != 0, tqb_pqo_cache_decode takes host pointers.  Pinned, device-mapped buffers (cudaHostAlloc or
 * cudaHostRegister under unified addressing) are read and written by the attention kernel itself over PCIe - no
 * staging copy, nothing between two launches, so they overlap like device-resident ones (tqb_pqo_cache_set_overlap).
 * Other host memory is staged: inputs go up on an internal copy stream into one of two slots, the result comes down
 * on a second one, so that copies overlap the kernels of neighbouring calls.  Either way the caller's k / v / q are
 * in use and `out` is incomplete until tqb_pqo_cache_host_sync() returns (it blocks the calling thread on the
 * outstanding work of this cache). */
int tqb_pqo_cache_host_sync(tqb_pqo_cache *c);
/* Prefill with attention inside the cache: quantize and append the chunk (as tqb_pqo_cache_prefill), then causal
 * attention of its new_tokens queries over everything stored (tqb_chunk_attention).  The reference's prefill
 * (pqo.rs:184-200) returns the dequantized cache for the engine's own attention instead.  Device buffers:
 * k, v [batch, num_kv_heads, new_tokens, head_dim]; q, out [new_tokens, batch * num_q_heads, head_dim]. */
int tqb_pqo_cache_prefill_attend(tqb_pqo_cache *c, int32_t layer, const void *k, const void *v, const void *q,
                                 int32_t dtype, int32_t new_tokens, int32_t num_q_heads, float softmax_scale,
                                 void *out, tqb_stream_t stream);

/* dequantize_full (pqo.rs:176-180): [batch, num_kv_heads, seq_len, head_dim] of `dtype`. */
int tqb_pqo_cache_dequantize_full(tqb_pqo_cache *c, int32_t layer, void *k_out, void *v_out, int32_t dtype,
                                  int32_t host_buffers, tqb_stream_t stream);
int64_t tqb_pqo_cache_seq_len(const tqb_pqo_cache *c, int32_t layer);
int64_t tqb_pqo_cache_capacity(const tqb_pqo_cache *c, int32_t layer);
int tqb_pqo_cache_reset(tqb_pqo_cache *c);
/* enabled != 0: the decode launches of this cache (tqb_pqo_cache_decode with device buffers, tqb_pqo_cache_attend_partial,
 * tqb_pqo_cache_attend_push) are made with TQB_DECODE_OVERLAP whenever the layer differs from the layer of the
 * cache's previous decode launch, so that the launches of successive layers overlap head to tail.  The caller vouches
 * that q / new_k / new_v of a call are not written by the immediately preceding kernel on the stream (in a model
 * they come from a projection kernel in between, which orders them).  Off by default.  No reference counterpart. */
int tqb_pqo_cache_set_overlap(tqb_pqo_cache *c, int32_t enabled);
size_t tqb_pqo_cache_memory_usage(const tqb_pqo_cache *c);
/* Device pointers of one layer's storage (k_indices, k_scales, v_indices, v_scales). */
int tqb_pqo_cache_layer_ptrs(const tqb_pqo_cache *c, int32_t layer, const uint8_t **k_indices,
                             const uint16_t **k_scales, const uint8_t **v_indices, const uint16_t **v_scales);
/* Dense copy of one layer's stored rows without the capacity padding (the block-32 counterpart of
 * export_packed_range, src/attention.rs:663-693, which the reference offers for the whole-vector cache only):
 * k/v_indices [batch * num_kv_heads, seq_len, head_dim*bits/8], k/v_scales [.., seq_len, head_dim/32].
 * host_buffers != 0: the destinations are host memory and the call returns when they are filled. */
int tqb_pqo_cache_export_layer(const tqb_pqo_cache *c, int32_t layer, uint8_t *k_indices, uint16_t *k_scales,
                               uint8_t *v_indices, uint16_t *v_scales, int32_t host_buffers, tqb_stream_t stream);
/* Sequence-parallel decode: shard-local un-normalised output + (max, sum), no append. */
int tqb_pqo_cache_attend_partial(tqb_pqo_cache *c, int32_t layer, const void *q, int32_t dtype,
                                 int32_t num_q_heads, float softmax_scale, float *out_unnorm, float *lse_out,
                                 tqb_stream_t stream);

/* Sequence-parallel decode with the exchange fused into the attention kernel (no counterpart in the reference,
 * which is single-GPU; the merge algebra is that of tq_fused_attention_reduce, tq_attention_kernel.cu:299-332).
 * One sequence is split along the tokens over `world` <= 8 ranks of one NVLink domain, one process per GPU.  Every
 * rank owns a receive buffer; its 64-byte CUDA IPC handle is exchanged by the host (any channel) and opened by the
 * peers.  Per layer, tqb_pqo_cache_attend_push runs the shard-local attention: the CTA that finishes a KV head stores
 * the head group's (un-normalised output, max, sum) record into every rank's buffer with plain global stores and
 * releases a flag; tqb_peer_exchange_combine then acquires the flags of all ranks - each wait bounded by wait_cycles
 * GPU clock cycles - and merges the records in local memory into out [num_q_heads, 128].  All ranks must make the
 * same sequence of calls.  A wait that runs out is counted, zeros are written, the kernel returns and the context
 * stays usable: tqb_peer_exchange_check reports TQB_ERR_PEER_TIMEOUT (it synchronises the device).  head_dim 128,
 * the formats of the tensor-core kernels, every rank's shard non-empty. */
typedef struct tqb_peer_exchange tqb_peer_exchange;
int tqb_peer_exchange_create(int32_t world, int32_t rank, int32_t num_q_heads, int32_t head_dim, tqb_peer_exchange **out);
void tqb_peer_exchange_destroy(tqb_peer_exchange *x);
int tqb_peer_exchange_handle(const tqb_peer_exchange *x, void *handle64);
/* handles: world x 64 bytes in rank order (this rank's own entry is ignored). */
int tqb_peer_exchange_connect(tqb_peer_exchange *x, const void *handles);
/* The same for ranks that live in ONE process (an IPC handle cannot be opened by the process that made it):
 * `all` = the world's exchange objects in rank order. */
int tqb_peer_exchange_connect_local(tqb_peer_exchange *x, tqb_peer_exchange *const *all);
int tqb_pqo_cache_attend_push(tqb_pqo_cache *c, int32_t layer, const void *q, int32_t dtype, int32_t num_q_heads,
                              float softmax_scale, tqb_peer_exchange *x, tqb_stream_t stream);
int tqb_peer_exchange_combine(tqb_peer_exchange *x, int32_t num_kv_heads, void *out, int32_t out_dtype,
                              int64_t wait_cycles, tqb_stream_t stream);
long long tqb_peer_exchange_timeouts(const tqb_peer_exchange *x);
int tqb_peer_exchange_check(const tqb_peer_exchange *x);

/* compute_qjl_signs_and_norms (src/cache/tq.rs:380-411) as a kernel: residual = original - dequantized
 * for n vectors of `dim` (32, 64, 128 or 256), its L2 norm as f16 bits and the dim-wide sign sketch,
 * written at storage rows (same row mapping as tqb_block_quantize).  rbits: device bit matrix of
 * tqb_qjl_rademacher_bits.  original: device [n, dim] of `dtype`; dequantized: device [n, dim] f32. */
int tqb_residual_sketch(int32_t dim, const uint32_t *rbits, const void *original, int32_t dtype,
                        const float *dequantized, int64_t n, uint8_t *signs, uint16_t *norms,
                        int64_t rows_per_group, int64_t out_group_stride, int64_t out_row_offset,
                        tqb_stream_t stream);
/* compute_logit_bias (src/cache/tq.rs:185-253): bias[h, i, t] = (sum_d rq[h, i, d] * sign_td) * norm_t *
 * sqrt(pi/2) / sqrt(head_dim).  rq: device [num_q_heads, q_len, head_dim] f32 (tqb_qjl_query_projections);
 * signs [num_kv_heads, kv_stride, head_dim/8]; norms [num_kv_heads, kv_stride];
 * bias: device [num_q_heads, q_len, kv_len] of bias_dtype. */
int tqb_qjl_logit_bias(int32_t head_dim, const float *rq, const uint8_t *signs, const uint16_t *norms, void *bias,
                       int32_t bias_dtype, int32_t num_q_heads, int32_t num_kv_heads, int32_t q_len,
                       int32_t kv_len, int32_t kv_stride, tqb_stream_t stream);

/* TqCache (src/cache/tq.rs:21-412): polar codes (outlier_blocks = 0: the bits-1 codebook stored at
 * `bits` width) plus a QJL sign sketch of the key residual.  All pointers are DEVICE pointers.
 * k, v: [batch, num_kv_heads, new_tokens, head_dim]; q: [batch, num_q_heads, q_len, head_dim];
 * logit_bias: [batch, num_q_heads, q_len, seq_len] of `dtype` (DequantResult::logit_bias). */
typedef struct tqb_tq_cache tqb_tq_cache;
int tqb_tq_cache_create(const tqb_cache_config *cfg, tqb_tq_cache **out);
void tqb_tq_cache_destroy(tqb_tq_cache *c);
/* prefill (tq.rs:263-288): k_out/v_out receive the full dequantized cache when the layer already held tokens. */
int tqb_tq_cache_prefill(tqb_tq_cache *c, int32_t layer, const void *k, const void *v, const void *q, int32_t dtype,
                         int32_t new_tokens, int32_t num_q_heads, int32_t q_len, void *k_out, void *v_out,
                         void *logit_bias, tqb_stream_t stream);
/* decode (tq.rs:290-311): DecodeOutput::Dequantized { k, v, logit_bias } over all seq_len tokens. */
int tqb_tq_cache_decode(tqb_tq_cache *c, int32_t layer, const void *k, const void *v, const void *q, int32_t dtype,
                        int32_t num_q_heads, void *k_out, void *v_out, void *logit_bias, tqb_stream_t stream);
/* Fused alternative that the reference's kernel offers but never calls (tq_attention_kernel.cu:197-231):
 * append, then attention with the QJL correction added inside the kernel; out [batch, num_q_heads, 1, head_dim]. */
int tqb_tq_cache_decode_fused(tqb_tq_cache *c, int32_t layer, const void *k, const void *v, const void *q,
                              int32_t dtype, int32_t num_q_heads, float softmax_scale, void *out,
                              tqb_stream_t stream);
int64_t tqb_tq_cache_seq_len(const tqb_tq_cache *c, int32_t layer);
int tqb_tq_cache_reset(tqb_tq_cache *c);
size_t tqb_tq_cache_memory_usage(const tqb_tq_cache *c);
int tqb_tq_cache_qjl_ptrs(const tqb_tq_cache *c, int32_t layer, const uint8_t **signs, const uint16_t **norms,
                          int64_t *capacity);

/* QuantizedKVCache (src/attention.rs:45-694): whole-vector polar + QJL blocks for keys
 * and values, one growable device array set per layer.  Vectors are HOST pointers unless
 * the name says otherwise; these calls synchronise the stream before returning. */
typedef struct tqb_kv_cache tqb_kv_cache;
int tqb_kv_cache_create(const tqb_config *cfg, int32_t num_layers, uint64_t qjl_seed, tqb_kv_cache **out);
void tqb_kv_cache_destroy(tqb_kv_cache *c);
/* push / push_batch (attention.rs:238-305): keys, values host [n, vec_dim] f32; vec_dim
 * must equal the configured dim (DimensionMismatch otherwise). */
int tqb_kv_cache_push_batch(tqb_kv_cache *c, int32_t layer, const float *keys, const float *values, int64_t n,
                            int64_t vec_dim, tqb_stream_t stream);
/* attention_scores (attention.rs:319-353): scores host [entry_count]. */
int tqb_kv_cache_attention_scores(tqb_kv_cache *c, int32_t layer, const float *query, int64_t query_len,
                                  float *scores, tqb_stream_t stream);
/* weighted_values (attention.rs:371-408): weights host [num_weights], out host [dim]. */
int tqb_kv_cache_weighted_values(tqb_kv_cache *c, int32_t layer, const float *weights, int64_t num_weights,
                                 float *out, tqb_stream_t stream);
/* dequantize_{keys,values}_range (attention.rs:589-611): out host [end-start, dim]. */
int tqb_kv_cache_dequantize_range(tqb_kv_cache *c, int32_t layer, int64_t start, int64_t end, int32_t is_keys,
                                  float *out, tqb_stream_t stream);
/* export_packed_range / import_packed_range (attention.rs:663-693) in PackedImport's
 * field layout; signs and rnorms may be NULL on export. */
int tqb_kv_cache_export_packed_range(tqb_kv_cache *c, int32_t layer, int64_t start, int64_t end,
                                     int32_t is_keys, uint8_t *packed_bytes, uint16_t *scales,
                                     uint8_t *qjl_signs, uint16_t *residual_norms, tqb_stream_t stream);
int tqb_kv_cache_import_packed_range(tqb_kv_cache *c, int32_t layer, int32_t polar_bits,
                                     const uint8_t *packed_bytes, const uint16_t *scales,
                                     const uint8_t *qjl_signs_flat, const uint16_t *residual_norms,
                                     int64_t count, int64_t bytes_per_block, int64_t signs_per_block,
                                     int32_t is_keys, tqb_stream_t stream);
int64_t tqb_kv_cache_entry_count(const tqb_kv_cache *c, int32_t layer);
int32_t tqb_kv_cache_num_layers(const tqb_kv_cache *c);
size_t tqb_kv_cache_memory_usage(const tqb_kv_cache *c);          /* attention.rs:414-428 */
size_t tqb_kv_cache_fp16_equivalent_memory(const tqb_kv_cache *c); /* attention.rs:437-440 */

#ifdef __cplusplus
}
#endif
#endif /* TQB200_H */
