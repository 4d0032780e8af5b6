/*
 * tinytitan_cuda.h -- C ABI of the B200 (sm_100a) attention / Gated-DeltaNet
 * library that stands behind TinyTitan's attention operator entry points.
 *
 * The header is strict C99 so that a SwiftPM C target can import it the way
 * the reference imports its own C kernels (Package.swift:105-124). Every entry
 * point names the reference interface it replaces (file:line inside the
 * TinyTitan source tree).
 *
 * Conventions
 *   - Device buffers are plain pointers; "MTLBuffer + byte offset" of the
 *     reference becomes pointer arithmetic done by the caller.
 *   - `tt_stream` is a cudaStream_t. Every op ENQUEUES on that stream and
 *     returns (the reference's encode-into-a-command-buffer semantics);
 *     ordering is stream order.
 *   - Every function returns an int status (TT_OK == 0); creators return NULL
 *     and set *out_err. Nothing traps, throws or writes to stdout/stderr.
 *   - A context belongs to one device and is not re-entrant: two threads must
 *     not enqueue through the same context at once (the reference's operators
 *     are not re-entrant either, Attention.swift:173-192).
 *   - There is no CPU fallback: without a usable CUDA device the ops fail with
 *     TT_ERR_CUDA.
 */
#ifndef TINYTITAN_CUDA_H
#define TINYTITAN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tt_context tt_context;
typedef struct tt_kv_cache tt_kv_cache;
typedef struct tt_gdn_state tt_gdn_state;
typedef void *tt_stream;

enum tt_status {
    TT_OK = 0,
    TT_ERR_INVALID_ARG = 1,       /* the reference's precondition failures */
    TT_ERR_UNSUPPORTED_SHAPE = 2, /* refused outright, never silently skipped */
    TT_ERR_OOM = 3,               /* ModelError.residentBufferWrapFailed */
    TT_ERR_CUDA = 4,
    TT_ERR_TIMEOUT = 5,
    TT_ERR_BUSY = 6
};

enum tt_dtype { TT_F16 = 0, TT_BF16 = 1 };

/* ---------------------------------------------------------------- context */

typedef struct tt_context_options {
    size_t workspace_bytes; /* split-KV partials, scan records; 0 selects 256 MiB */
    uint32_t max_sessions;  /* rows of one batched call; 0 selects 1024 */
    uint32_t reserved;
} tt_context_options;

/* Replaces MetalContext + the per-operator scratch the Swift classes own
 * (sources/TinyTitan/Kernels/Attention/Attention.swift:140-156): all device
 * scratch is allocated here, never on the decode path.
 *
 * A context serves ONE stream at a time. Its scratch (the tables and split partials of the
 * current call, the status word) belongs to the operation that was enqueued last: TT_ERR_BUSY
 * only rejects host calls that overlap in time, and it is released when the enqueue returns,
 * while the kernels may still be running. Two operations through one context on different
 * streams with no ordering between them would overwrite each other's scratch; use one context
 * per stream (contexts are independent and cheap next to a KV cache), or order the streams
 * with events. The reference's Attention has the same rule for its shared partial scratch
 * (Attention.swift:173-192: one encode in flight per instance). */
tt_context *tt_context_create(int device, const tt_context_options *options, int *out_err);
void tt_context_destroy(tt_context *ctx);
/* Text of the last failure seen through this context (never NULL). */
const char *tt_last_error_string(const tt_context *ctx);
const char *tt_status_string(int status);
/* Asynchronous device-side status word (bounded waits that ran out, unsupported
 * work reached on the device). 0 when clean. Synchronises the stream. */
int tt_ctx_poll_status(tt_context *ctx, tt_stream stream, uint32_t *out_flags);
int tt_stream_synchronize(tt_context *ctx, tt_stream stream);
/* Number of kernels this context has launched since creation (diagnostic). */
uint64_t tt_ctx_launch_count(const tt_context *ctx);
/* Per-kernel device timing, the counterpart of the reference's per-command-buffer
 * GPU timestamps (EngineRunner.kernelGPUTimingSummary, EngineRunner.swift:58-66;
 * TINYTITAN_KERNEL_SPLIT in RealForwardRunner+DecodeGEMV.swift:29-50). While
 * enabled, every launch of the selected kernel classes is bracketed by a pair of
 * events on its own stream (up to 256 launches are kept). `enabled` is 0 (off) or a
 * mask of TT_PROFILE_*; 1 selects the split-KV pass-1 kernel.
 * tt_ctx_profile_collect waits for the recorded events, writes the durations in
 * milliseconds in launch order, returns how many there were in *out_count and
 * clears the record. */
#define TT_PROFILE_DECODE_PARTIAL 1
#define TT_PROFILE_GDN_STEP 2
#define TT_PROFILE_EXCHANGE 4 /* the merge + peer exchange kernel of tt_attn_decode_exchange */
int tt_ctx_profile_enable(tt_context *ctx, int enabled);
int tt_ctx_profile_collect(tt_context *ctx, float *out_ms, uint32_t capacity, uint32_t *out_count);

/* ------------------------------------------------- decode attention (SDPA) */

/* KVView's format fields (KVCacheManager.swift:20-43). bits 16 = fp16 rows; 8 / 4 =
 * affine-quantised rows [packed codes | fp16 scale per 64-element group | fp16 bias per
 * group] (KVCacheManager+Validation.swift:30-41), decoded as code*scale+bias
 * (attn_load_kv, attention.metal:89-117). Quantised rows need head_dim 128 or 256,
 * group_size 64, fp16 queries and 16-byte aligned strides; a keep mask, a sliding window and
 * a ring work as with fp16 rows. */
typedef struct tt_kv_format {
    uint32_t bits;
    uint32_t stride_bytes; /* bytes per token row; 0 means n_kv_heads*head_dim*2 */
    uint32_t value_bytes;
    uint32_t group_size;
} tt_kv_format;

/* One query row against one session's cache. Replaces Attention.encodeFull and
 * Attention.encodeSWA -> encodeSplit (Attention.swift:233-470) and the kernels
 * attention_decode_partial / attention_decode_combine
 * (sources/TinyTitanCore/Metal/Attention/attention.metal:162-269, :395-437).
 * q,out: [n_q_heads, head_dim] fp16. k,v: logical position 0 of the session's
 * rows, row p at p*stride (or (p % ring_capacity)*stride). Keys attended are
 * [kv_start, seq_len); keep_mask[p]==0 drops key p. An empty range writes
 * zeros. SWA callers pass kv_start = seq_len > window ? seq_len - window : 0. */
int tt_attn_decode(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                   const void *v, void *out, uint32_t head_dim, uint32_t n_q_heads,
                   uint32_t n_kv_heads, uint32_t seq_len, uint32_t kv_start, float scale,
                   const tt_kv_format *kv_format, const uint8_t *keep_mask,
                   uint32_t ring_capacity);

/* Attention over a compact selection with row indirection: key s of sel_count lives at
 * physical row sel_rows[s] of the K / V buffers (device array). Replaces
 * Attention.encodeFull(windowSelection:) -> attention_decode_window_partial
 * (attention.metal:612-870), the read side of the host-KV window. */
int tt_attn_decode_window(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                          const void *v, void *out, uint32_t head_dim, uint32_t n_q_heads,
                          uint32_t n_kv_heads, uint32_t sel_count, float scale,
                          const tt_kv_format *kv_format, const uint32_t *sel_rows);

/* One session of a batched / few-token decode step. Row r of `q_rows` sits at
 * base position seq_len - q_rows + r and attends keys
 * [kv_start, seq_len - (q_rows - 1 - r)), which is the decode-order verify rule
 * of RealForwardRunner+VerifyDecodeOrderAttention.swift:84-105. */
typedef struct tt_attn_session {
    const void *q;   /* [q_rows] rows, q_row_stride elements apart */
    void *out;       /* [q_rows] rows, out_row_stride elements apart */
    const void *k;   /* position 0 of this session's K rows */
    const void *v;
    uint32_t seq_len; /* keys visible to the LAST row (cursor + q_rows) */
    uint32_t q_rows;  /* 1 for plain decode; up to 64/(Hq/Hkv) per kernel pass */
    uint32_t kv_start;
    uint32_t reserved;
} tt_attn_session;

typedef struct tt_attn_batch_params {
    uint32_t head_dim, n_q_heads, n_kv_heads;
    uint32_t kv_token_stride_elements; /* >= n_kv_heads*head_dim */
    uint32_t q_row_stride_elements;    /* >= n_q_heads*head_dim */
    uint32_t out_row_stride_elements;
    float scale;
    uint32_t io_dtype; /* tt_dtype of q, k, v, out */
} tt_attn_batch_params;

/* Replaces the per-row loop of RealForwardRunner+BatchAttention.swift:165-218
 * (N serial encodeFull calls) with one launch pair over all sessions; work is
 * split by KV bytes, not by session. `sessions` is host memory and may be
 * reused as soon as the call returns. */
int tt_attn_decode_batched(tt_context *ctx, tt_stream stream, const tt_attn_session *sessions,
                           uint32_t n_sessions, const tt_attn_batch_params *params);

/* Split-KV halves exposed for a KV range that lives on several GPUs: pass 1
 * leaves ONE unnormalised (m, d, o) triple per q head for keys
 * [kv_start, seq_len) of this device (the chunk-partial format of
 * attention.metal:146-159), pass 2 merges n_parts such triples
 * (attention.metal:395-437). m,d: [n_parts][n_q_heads] fp32; o:
 * [n_parts][n_q_heads][head_dim] fp32. */
int tt_attn_decode_partial(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                           const void *v, uint32_t head_dim, uint32_t n_q_heads,
                           uint32_t n_kv_heads, uint32_t seq_len, uint32_t kv_start, float scale,
                           uint32_t kv_token_stride_elements, uint32_t io_dtype, float *m_out,
                           float *d_out, float *o_out);
int tt_attn_combine(tt_context *ctx, tt_stream stream, const float *m, const float *d,
                    const float *o, uint32_t n_parts, uint32_t n_q_heads, uint32_t head_dim,
                    void *out, uint32_t io_dtype);

/* The same merge when the n_parts triples live on `world` GPUs of one node, one per GPU (one
 * process per GPU): exchange and merge in ONE kernel over peer memory instead of a collective
 * followed by tt_attn_combine. The reference has no multi-device code; the triple is its
 * chunk-partial format (attention.metal:146-159) and the result equals tt_attn_combine over the
 * world triples (attention.metal:395-437).
 *
 * Every rank owns an exchange buffer (tt_peer_buffer_create) that the other ranks map
 * (tt_peer_buffer_open) with the 64-byte handle the owner hands out through any host channel.
 * tt_attn_exchange_combine stores this rank's triple into slot `rank` of every rank's buffer
 * (plain 16-byte stores over NVLink in which every 8 bytes are one value and `epoch`, so a word
 * validates itself and no flag or fence follows the data), polls -- with a limit,
 * TT_DEV_WAIT_TIMEOUT in the status word when it runs out -- until every word of every rank's
 * slot in its own buffer carries this epoch, and merges. `epoch` must be
 * the same on all ranks for one step and grow by exactly 1 per step, starting at 1 (slots are
 * double-buffered on its parity: a rank can be at most one step ahead of another).
 * peer_buffers[r] is rank r's buffer as mapped by THIS process (its own for r == rank).
 * world <= 16; head_dim a multiple of 4. */
size_t tt_attn_exchange_bytes(uint32_t world, uint32_t n_q_heads, uint32_t head_dim);
/* No counterpart in the reference. How many polls (about 0.25 us each) the exchange kernels of
 * this context wait for the other ranks' words before they give up, set TT_DEV_WAIT_TIMEOUT in
 * the status word and leave the output untouched; 0 restores the default (about one second).
 * A short limit lets a host that already knows a peer is gone (a heartbeat, a store) get its
 * stream back quickly; the status is read with tt_ctx_poll_status (TT_ERR_TIMEOUT). */
int tt_ctx_set_exchange_poll_limit(tt_context *ctx, uint32_t polls);
int tt_peer_buffer_create(tt_context *ctx, size_t bytes, void **out_ptr, unsigned char out_handle[64]);
int tt_peer_buffer_open(tt_context *ctx, const unsigned char handle[64], void **out_ptr);
int tt_peer_buffer_close(tt_context *ctx, void *ptr);
int tt_peer_buffer_destroy(tt_context *ctx, void *ptr);
int tt_attn_exchange_combine(tt_context *ctx, tt_stream stream, const float *m, const float *d,
                             const float *o, void *const *peer_buffers, uint32_t rank, uint32_t world,
                             uint32_t n_q_heads, uint32_t head_dim, uint32_t epoch, void *out,
                             uint32_t io_dtype);

/* One decode step of a session whose KV rows are split over `world` GPUs, in two launches: the
 * split-KV pass over this GPU's rows [kv_start, seq_len) (as tt_attn_decode_partial), then ONE
 * kernel that merges this GPU's split partials, exchanges the result over peer memory and merges
 * across GPUs (as tt_attn_exchange_combine, same buffers, same epoch rule); x->out receives the
 * [n_q_heads][head_dim] output row on every rank. */
typedef struct tt_attn_exchange {
    void *const *peer_buffers; /* [world], as mapped by this process */
    uint32_t rank;
    uint32_t world;
    uint32_t epoch;
    uint32_t reserved;
    void *out;
} tt_attn_exchange;
int tt_attn_decode_exchange(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                            const void *v, uint32_t head_dim, uint32_t n_q_heads,
                            uint32_t n_kv_heads, uint32_t seq_len, uint32_t kv_start, float scale,
                            uint32_t kv_token_stride_elements, uint32_t io_dtype,
                            const tt_attn_exchange *x);

/* No counterpart in the reference. One query row against one session's fp16 cache
 * ([kv_start, seq_len), tight K/V rows), computed exactly like tt_attn_decode, for
 * callers that must not allocate device memory -- code running where cudaMalloc is off
 * limits (inside another component's latency-critical or capture-restricted section, or
 * after the host has handed out its whole memory budget). It needs no context and calls no
 * allocator: the split-KV scratch is a fixed 8 MiB array inside the library image, present
 * on every GPU that loads the library until the process exits. The session is passed to the
 * kernels by value and nothing is copied from host memory. Limits: at most
 * TT_NOALLOC_MAX_KEYS keys in [kv_start, seq_len) (a longer range is refused with
 * TT_ERR_UNSUPPORTED_SHAPE before anything is launched; below it the split is coarsened
 * until the partial triples fit the array); head_dim 64, 128 or 256; n_q_heads <= 96;
 * buffers 16-byte aligned. The first call on a device looks the array's device address up;
 * make that call outside stream capture. All calls on a device share the array: calls that
 * overlap on the GPU race, so keep them ordered (one stream, or events). Runs on the
 * current device. A bounded wait that runs out inside a kernel cannot be reported through
 * the return value of an asynchronous call: read it with tt_attn_decode_noalloc_status. */
#define TT_NOALLOC_MAX_KEYS (1u << 22)
int tt_attn_decode_noalloc(tt_stream stream, const void *q, const void *k, const void *v, void *out,
                           uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads,
                           uint32_t seq_len, uint32_t kv_start, float scale);
/* No counterpart in the reference. Waits for `stream`, then stores the device status word of
 * the allocation-free entry point on the current device in *out_flags: 0, or bit 0 when a
 * bounded wait in the last call's kernels gave up (that call's output is then not valid).
 * Allocates nothing either. */
int tt_attn_decode_noalloc_status(tt_stream stream, uint32_t *out_flags);

/* Split geometry of the reference, kept for callers and tests that pin it
 * (Attention.splitGeometry, Attention.swift:196-227). This library's own split
 * is chosen per call from the byte count; any partition of the key range is
 * legal because the result is defined by the merge. */
typedef struct tt_split_geometry {
    uint32_t effective_length, num_chunks, chunk_length, partial_threadgroups;
    uint32_t use_swa_grouped_partial;
} tt_split_geometry;
void tt_attn_reference_split_geometry(uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t seq_len,
                                      uint32_t kv_start, int prefer_gqa_swa,
                                      tt_split_geometry *out);

/* The split this library would use (host-only arithmetic, no device needed):
 * keys per work item and number of work items for a batch with the given
 * per-session key counts. */
int tt_attn_plan_splits(const uint32_t *keys_per_session, const uint32_t *q_rows_per_session,
                        uint32_t n_sessions, uint32_t head_dim, uint32_t n_q_heads,
                        uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes,
                        uint32_t *out_keys_per_item, uint32_t *out_n_items);

/* The split plan of the tensor-core verify pass (17..128 packed rows per KV head, head_dim 256), as
 * pure arithmetic: one work item per (session, kv head, part); the parts of a session have one
 * common length, a multiple of the 128-key tile, chosen for the whole batch by simulating the
 * in-order dispatch of the items over sm_count SMs. out_parts / out_part_len: [n_sessions].
 * TT_ERR_OOM when no plan fits workspace_bytes (0 = no limit). */
int tt_attn_plan_verify_splits(const uint32_t *keys_per_session, const uint32_t *q_rows_per_session,
                               uint32_t n_sessions, uint32_t head_dim, uint32_t n_q_heads,
                               uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes,
                               uint32_t *out_parts, uint32_t *out_part_len, uint32_t *out_n_items);

/* Replaces kv_cache_quantize_affine
 * (sources/TinyTitanCore/Metal/Quant/kv_cache_quantize.metal:4-72): fp16 rows
 * [tokens][source_stride_elements] -> packed rows of destination_stride_bytes with the
 * codes in the first values_bytes bytes, then one fp16 scale and one fp16 bias per group. */
int tt_kv_quantize_affine(tt_context *ctx, tt_stream stream, const void *source, void *destination,
                          uint32_t source_stride_elements, uint32_t destination_stride_bytes,
                          uint32_t values_bytes, uint32_t element_count, uint32_t bits,
                          uint32_t group_size, uint32_t tokens);

/* The elementwise step before full-attention SDPA in the gated-attention layer, one launch for
 * the reference's five (RealForwardRunner.encodeGatedFullPostProjection,
 * sources/TinyTitan/Runtime/Inference/RealForwardRunner+DecodeFullAttention.swift:123-185):
 * split per-head [query ; gate] (split_q_gate_fp16, Primitives/utility.metal:142-160), per-head
 * RMS norm of q and of the just-written K rows with bf16 weights (rmsnorm_bf16w_perhead,
 * Primitives/rmsnorm.metal:101-128), NeoX partial RoPE over the first rotary_dim elements
 * (rope_neox_subdim, Primitives/rope.metal:80-108). q_packed fp16 [rows][H][2D]; q_out, gate_out
 * fp16 [rows][H][D]; K row r ([Hkv][D], in place) at k_rows + r*k_row_stride_elements; row r is at
 * position `position + r`. */
int tt_attn_pre(tt_context *ctx, tt_stream stream, const void *q_packed, void *q_out, void *gate_out,
                void *k_rows, const void *q_norm_weight, const void *k_norm_weight, uint32_t head_dim,
                uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t rotary_dim, float theta, float eps,
                uint32_t position, uint32_t rows, uint32_t k_row_stride_elements);
/* out[i] *= sigmoid(gate[i]) (sigmoid_gate_mul_fp16, Primitives/utility.metal:48-58), the
 * full-attention output gate (RealForwardRunner+DecodeFullAttention.swift:84-88). */
int tt_attn_gate_mul(tt_context *ctx, tt_stream stream, void *out, const void *gate, uint32_t count);

/* ------------------------------------------------------- prefill attention */

/* Field for field the reference's PrefillAttentionParams
 * (sources/TinyTitan/Kernels/Attention/PrefillAttention.swift:5-21; MSL mirror
 * sources/TinyTitanCore/Metal/Prefill/prefill.metal:754-770). */
typedef struct tt_prefill_params {
    uint32_t start_position;
    uint32_t query_count;
    uint32_t head_dim;
    uint32_t n_q_heads;
    uint32_t n_kv_heads;
    uint32_t kv_valid_count;
    uint32_t sliding_window; /* 0 = none */
    uint32_t kv_token_stride_elements;
    uint32_t q_token_stride_elements;
    uint32_t o_token_stride_elements;
    float scale;
    uint32_t kv_bits; /* 16, or 8 / 4 (quantised rows run on the generic kernel) */
    uint32_t kv_token_stride_bytes;
    uint32_t kv_value_bytes;
    uint32_t kv_group_size;
} tt_prefill_params;

/* Replaces PrefillAttention.encodeCausal (PrefillAttention.swift:165-258) and
 * the kernels attention_prefill_causal_q8 / _tiled (prefill.metal:1056-1313).
 * Query t is at absolute position start_position + t and sees keys
 * [first, min(kv_valid_count, start_position + t + 1)). Shapes whose strides
 * and base pointers are 16-byte aligned with head_dim 256 run on the
 * tcgen05/TMA kernel; everything else runs on a generic CUDA kernel. */
int tt_attn_prefill_causal(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                           const void *v, void *out, const tt_prefill_params *params,
                           uint32_t kv_ring_capacity, uint32_t io_dtype);
/* Which kernel the call above would take: 0 generic, 1 tcgen05. */
int tt_attn_prefill_path(const void *q, const void *k, const void *v, const void *out,
                         const tt_prefill_params *params, uint32_t kv_ring_capacity);
/* PrefillAttention.encodeCausal with a per-query key selection (its keepMask / keepIndices /
 * keepCounts / keepRows arguments, PrefillAttention.swift:165-258; kernel
 * attention_prefill_causal_qsa_tiled, prefill.metal:898-1054). What is bound selects the form, as
 * in the reference: keep_indices + keep_counts = a compact list of logical keys per query row
 * (keep_indices[t * keep_index_stride + i], i < keep_counts[t]; entries outside the row's visible
 * range [first, last) are dropped); with keep_rows as well, keep_rows[...] names the cache row
 * that holds each listed key (host-KV window, tt_kv_window_prepare_prefill); otherwise keep_mask
 * is one byte per key, keep_mask[t * keep_stride + key] != 0 keeps it. All NULL = the dense call.
 * A row whose keys are all dropped is written as zeros. Selections run on the generic kernel. */
int tt_attn_prefill_causal_selected(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                                    const void *v, void *out, const tt_prefill_params *params,
                                    uint32_t kv_ring_capacity, uint32_t io_dtype,
                                    const uint8_t *keep_mask, uint32_t keep_stride,
                                    const uint32_t *keep_indices, uint32_t keep_index_stride,
                                    const uint32_t *keep_counts, const uint32_t *keep_rows);

/* ----------------------------------------- sparse-attention block indexer */

/* QSAIndexer's device work (sources/TinyTitan/Kernels/Attention/QSAIndexer.swift,
 * QSAIndexer+Scratch.swift; kernels sources/TinyTitanCore/Metal/Attention/qsa.metal:1-226).
 * The caller owns the caches, as the Swift class does: raw indexer keys fp16 [cells][head_dim]
 * (before norm and rotation), pooled blocks fp16 [cells / ratio + 1][head_dim], scores fp32.
 *
 * tt_qsa_pool_blocks: blocks first_block .. first_block + block_count - 1 become the mean of
 * their raw members present below n_kv (a ragged last block divides by its own count), then --
 * when key_norm_weight (bf16 [head_dim]) is given -- the RMS norm and the NeoX rotation over
 * the whole row at position block * ratio, the three launches of encodePoolPrefill
 * (QSAIndexer.swift:196-238) / encodeAppendKey (QSAIndexer+Scratch.swift:92-122) in one.
 * head_dim a multiple of 64, at most 512. */
int tt_qsa_pool_blocks(tt_context *ctx, tt_stream stream, const void *raw_keys, void *pooled,
                       uint32_t head_dim, uint32_t first_block, uint32_t block_count,
                       uint32_t ratio, uint32_t n_kv, const void *key_norm_weight, float eps,
                       float theta);
/* The indexer query after its projection: per-head RMS norm (bf16 weight) and NeoX rotation of
 * the whole head, in place over fp16 [rows][heads][head_dim]; row r is at position + r
 * (encodeScores / encodeScoresPrefill, QSAIndexer.swift:259-274, :322-337). */
int tt_qsa_query_norm_rope(tt_context *ctx, tt_stream stream, void *query, uint32_t head_dim,
                           uint32_t heads, uint32_t rows, uint32_t position,
                           const void *query_norm_weight, float eps, float theta);
/* qsa_block_scores / qsa_block_scores_rows (qsa.metal:67-126): scores[t * score_stride + b] =
 * sum over heads of max(0, query[t][h] . pooled[b]) for b < blocks, t < rows. */
int tt_qsa_block_scores(tt_context *ctx, tt_stream stream, const void *query, const void *pooled,
                        float *scores, uint32_t head_dim, uint32_t heads, uint32_t blocks,
                        uint32_t rows, uint32_t score_stride);
/* The key selection of `rows` query rows, row r seeing keys [0, start_position + r + 1)
 * (selectKeys / selectKeysCompact, QSAIndexer+Scratch.swift:178-251; selectKeysPrefill,
 * QSAIndexer.swift:391-498; qsa_select_decode, qsa.metal:128-226). A row with at most `width`
 * (= budget + ratio - 1) visible keys keeps them all. Otherwise the ragged tail of its own block
 * is kept, then complete blocks by score descending (ties to the lower block index) while the
 * cell budget lasts, the last admitted block cut to the cells that remain. Outputs, each
 * optional: keep[r * keep_stride + key] bytes (cells past the row's position are cleared up to
 * keep_stride); indices[r * index_stride + i] the kept keys in ascending order, at most
 * index_stride of them, with counts[r]. One decode step is rows = 1, start_position = visible - 1. */
int tt_qsa_select_keys(tt_context *ctx, tt_stream stream, const float *scores,
                       uint32_t score_stride, uint32_t start_position, uint32_t rows,
                       uint32_t ratio, uint32_t width, uint8_t *keep, uint32_t keep_stride,
                       uint32_t *indices, uint32_t index_stride, uint32_t *counts);

/* ------------------------------------------------------ Gated DeltaNet ops */

enum tt_gdn_flags {
    TT_GDN_A_LOG_PREEXP = 1, /* `a_log` already holds -exp(A_log) (GGUF ssm_a) */
    TT_GDN_V_TILED = 2,      /* key head = h % Hk instead of h / (Hv/Hk) */
    TT_GDN_GATES_F32 = 4     /* a,b hold per-token alpha,beta as fp32 (the
                                tinytitan_delta_rule_chunk calling form) */
};

/* LinearAttentionConfig's geometry
 * (sources/TinyTitanCore/Format/ModelTypes+Configs.swift:147-188) and the two
 * storage conventions of GDNStorageConvention.swift:7-25. */
typedef struct tt_gdn_shape {
    uint32_t n_k_heads, n_v_heads, key_dim, value_dim;
    uint32_t flags;
    float readout_scale; /* y = (S q) * readout_scale; 1.0 on the GPU path */
} tt_gdn_shape;

/* `rows` tokens applied one after another with the state carried; rows == 1 is
 * GDN.encodeDeltaStepDecode -> gdn_delta_step_decode
 * (sources/TinyTitan/Kernels/GDN/GDN.swift:318-347,
 * sources/TinyTitanCore/Metal/GDN/gdn.metal:529-585); rows > 1 is
 * GDN.encodeDeltaStepPrefill -> gdn_delta_step_prefill (GDN.swift:351-396,
 * gdn.metal:590-669), exact sequential arithmetic.
 * conv_out: fp16 [rows][row_stride] = [q: Hk*Dk | k: Hk*Dk | v: Hv*Dv | ...];
 * a,b: fp16 [rows][Hv]; a_log, dt_bias: bf16 [Hv]; state: fp32 [Hv][Dv][Dk]
 * updated in place; y: fp16 [rows][Hv*Dv]; checkpoint_state (nullable)
 * receives the state after row 0. */
int tt_gdn_step(tt_context *ctx, tt_stream stream, const void *conv_out, const void *a,
                const void *b, const void *a_log, const void *dt_bias, float *state, void *y,
                const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride,
                float *checkpoint_state);

typedef struct tt_gdn_session {
    const void *conv_out;
    const void *a;
    const void *b;
    float *state;
    void *y;
    float *checkpoint_state; /* nullable */
} tt_gdn_session;

/* The same step over many independent sessions in one launch (the per-row
 * loops of RealForwardRunner+VerifyDecodeOrderAttention.swift:166-189 and
 * RealForwardRunner+BatchAttention.swift). */
int tt_gdn_step_batched(tt_context *ctx, tt_stream stream, const tt_gdn_session *sessions,
                        uint32_t n_sessions, const void *a_log, const void *dt_bias,
                        const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride);

/* Chunk-parallel prefill scan: the same recurrence evaluated `chunk` tokens at
 * a time (the algorithm of tinytitan_delta_rule_chunk,
 * sources/TinyTitanKernelsC/gdn_chunk.c:72-195, on tensor cores). Same
 * arguments as tt_gdn_step; agrees with it to rounding, not bit for bit.
 * chunk must be 64. */
int tt_gdn_scan_chunked(tt_context *ctx, tt_stream stream, const void *conv_out, const void *a,
                        const void *b, const void *a_log, const void *dt_bias, float *state,
                        void *y, const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride,
                        uint32_t chunk);

/* The elementwise kernels around the delta rule (first "next" row of the scope).
 * conv_mix: causal depthwise conv + SiLU over [tail rows | rows of qkv]; tail fp16
 * [taps-1][channels], qkv fp16 [rows][channels], conv_weight bf16 [channels][taps],
 * out fp16 [rows][channels]. update_tail != 0 is GDN.encodeConvDecode ->
 * gdn_conv_mix_decode (rows must be 1; the tail is shifted in place), 0 is
 * GDN.encodeConvPrefill -> gdn_conv_mix_prefill with the tail read-only
 * (sources/TinyTitan/Kernels/GDN/GDN.swift:185-236,
 * sources/TinyTitanCore/Metal/GDN/gdn.metal:330-393). */
int tt_gdn_conv_mix(tt_context *ctx, tt_stream stream, void *tail, const void *qkv,
                    const void *conv_weight, void *out, uint32_t channels, uint32_t taps,
                    uint32_t rows, int update_tail);
/* GDN.encodeConvTailUpdate -> gdn_conv_tail_update (GDN.swift:238-262, gdn.metal:396-447):
 * tail := last taps-1 raw rows of [old tail | rows of qkv]. */
/* The decode prologue of a GDN layer for a batch of sessions in one launch: what
 * GDN.encodeConvDecode followed by GDN.encodeQKNorm (GDN.swift:185-229, :399-427) does with two
 * launches per session. For every session: conv_out := SiLU(conv([tail | qkv])), the tail shifted
 * in place, then the q and k heads of conv_out RMS-normed with the folded scales. Bit-identical to
 * tt_gdn_conv_mix(update_tail = 1) + tt_gdn_qk_norm. key_dim <= 256; the value width must be a
 * multiple of key_dim. */
typedef struct tt_gdn_pre_session {
    void *tail;       /* fp16 [(taps-1)][channels], updated in place */
    const void *qkv;  /* fp16 [channels], the new raw row */
    void *conv_out;   /* fp16 [channels] */
} tt_gdn_pre_session;
int tt_gdn_decode_pre(tt_context *ctx, tt_stream stream, const tt_gdn_pre_session *sessions,
                      uint32_t n_sessions, const void *conv_weight, uint32_t n_k_heads,
                      uint32_t key_dim, uint32_t channels, uint32_t taps);
int tt_gdn_conv_tail_update(tt_context *ctx, tt_stream stream, void *tail, const void *qkv,
                            uint32_t channels, uint32_t taps, uint32_t rows);
/* The prefill prologue of a GDN layer over a chunk of rows in one launch: what
 * GDN.encodeConvPrefill, GDN.encodeConvTailCheckpoint, GDN.encodeConvTailUpdate and GDN.encodeQKNorm
 * (GDN.swift:206-313) do with four. conv_out := SiLU(conv([tail | rows of qkv])) with the q and k
 * heads RMS-normed with the folded scales; checkpoint_tail (nullable) := the tail as it stands after
 * row 0 alone; with update_tail != 0 the tail becomes the last taps-1 raw rows of [old tail | rows].
 * Bit-identical to the four separate calls. key_dim 32, 64, 128 or 256; channels a multiple of
 * key_dim; taps <= 8; buffers aligned to key_dim / 16 bytes. */
int tt_gdn_prefill_pre(tt_context *ctx, tt_stream stream, void *tail, const void *qkv,
                       const void *conv_weight, void *conv_out, void *checkpoint_tail,
                       uint32_t n_k_heads, uint32_t key_dim, uint32_t channels, uint32_t taps,
                       uint32_t rows, int update_tail);
/* GDN.encodeConvTailCheckpoint -> gdn_conv_tail_checkpoint (GDN.swift:264-286,
 * gdn.metal:449-464): the tail as it stands after qkv row 0 alone. */
int tt_gdn_conv_tail_checkpoint(tt_context *ctx, tt_stream stream, const void *tail, const void *qkv,
                                void *checkpoint, uint32_t channels, uint32_t taps);
/* GDN.encodeQKNorm -> gdn_qk_norm (GDN.swift:288-313, gdn.metal:472-521): per key head,
 * in place on the q and k slices of conv_out rows: x * rsqrt(mean(x^2) + 1e-6) * (q: 1/Dk,
 * k: 1/sqrt(Dk)). */
int tt_gdn_qk_norm(tt_context *ctx, tt_stream stream, void *conv_out, uint32_t n_k_heads,
                   uint32_t key_dim, uint32_t row_stride, uint32_t rows);
/* GDN.encodeGatedNorm -> gdn_gated_norm (GDN.swift:399-427, gdn.metal:678-727):
 * out = rmsnorm(y per value head) * weight * gate(z), gate = SiLU or sigmoid
 * (LinearAttentionConfig.OutputGate). y,z,out fp16 [rows][Hv*Dv], weight bf16 [Dv]. */
int tt_gdn_gated_norm(tt_context *ctx, tt_stream stream, const void *y, const void *z,
                      const void *weight, void *out, uint32_t n_v_heads, uint32_t value_dim,
                      uint32_t rows, int sigmoid_gate);

/* ------------------------------------------------------------- allocators */

/* Where the managers get memory. NULL selects CUDA device memory on the
 * current device; a host implementation lets the bookkeeping be tested without
 * a GPU. copy/zero return 0 on success. */
typedef struct tt_allocator {
    void *user;
    void *(*alloc)(void *user, size_t bytes);
    void (*release)(void *user, void *ptr);
    int (*copy)(void *user, void *dst, const void *src, size_t bytes);
    int (*zero)(void *user, void *dst, size_t bytes);
    /* managed memory <-> host memory, used by the snapshot calls only; may be NULL, in
     * which case snapshots are refused with TT_ERR_UNSUPPORTED_SHAPE */
    int (*download)(void *user, void *host_dst, const void *src, size_t bytes);
    int (*upload)(void *user, void *dst, const void *host_src, size_t bytes);
} tt_allocator;

/* The part of ArchConfig the managers read. layer_kind[i]: 0 sliding-window,
 * 1 full attention, 2 linear (ArchConfig.fullAttentionLayerMask). */
typedef struct tt_arch {
    uint32_t n_layers;
    const uint8_t *layer_kind;
    uint32_t n_kv_heads, head_dim;           /* sliding-window layers */
    uint32_t n_full_kv_heads, full_head_dim; /* full-attention layers */
    uint32_t sliding_window;
    uint32_t gdn_k_heads, gdn_v_heads, gdn_key_dim, gdn_value_dim, gdn_conv_kernel;
} tt_arch;

typedef struct tt_kv_view {
    void *buffer;              /* the layer's K (or V) allocation */
    size_t offset;             /* byte offset of logical position 0 of the slot */
    uint32_t stride;           /* bytes per token */
    uint32_t valid_token_count;
    uint32_t precision_bits;
    uint32_t value_bytes;
    uint32_t group_size;
    uint32_t ring_capacity;    /* 0 unless a ring-backed sliding-window layer */
} tt_kv_view;

/* KVCacheManager.rowLayout (KVCacheManager+Validation.swift:30-41): bytes per
 * token row and bytes of packed values for `elements` values at 16/8/4 bits. */
void tt_kv_row_layout(uint32_t elements, uint32_t precision_bits, uint32_t *out_stride,
                      uint32_t *out_value_bytes);

/* KVCacheManager.init (sources/TinyTitan/Runtime/KVCache/KVCacheManager.swift:
 * 161-333): per non-linear layer one K and one V allocation of
 * slots*capacity*stride bytes; capacity starts at min(max_context, 8192). */
tt_kv_cache *tt_kv_cache_create(const tt_arch *arch, uint32_t max_context, uint32_t slots,
                                uint32_t precision_bits, int fp16_ring_enabled,
                                uint32_t max_prefill_chunk_tokens, const tt_allocator *allocator,
                                int *out_err);
void tt_kv_cache_destroy(tt_kv_cache *cache);
/* reserve(tokens:slot:) (KVCacheManager+Storage.swift:92-139): doubling growth
 * that keeps min(capacity, position[s]) rows of every slot. Views and slot
 * pointers fetched earlier are invalid afterwards. */
int tt_kv_cache_reserve(tt_kv_cache *cache, uint32_t tokens, uint32_t slot);
/* The reference's managers are touched by the CPU between command buffers (unified memory); here
 * their row copies (reserve) are device work. Unbound, they are synchronous calls on the legacy
 * default stream, which non-blocking streams do not wait for. After _bind_stream they are enqueued
 * on `stream`, in order with the kernels launched there; reserve then synchronises that stream
 * before it releases the old buffers. Only for managers on the built-in CUDA allocator
 * (TT_ERR_UNSUPPORTED_SHAPE otherwise). */
int tt_kv_cache_bind_stream(tt_kv_cache *cache, tt_stream stream);
/* kSlot / vSlot (:161-211): where the projection writes position `position`. */
int tt_kv_cache_k_slot(tt_kv_cache *cache, uint32_t layer, uint32_t position, uint32_t slot,
                       void **out_ptr);
int tt_kv_cache_v_slot(tt_kv_cache *cache, uint32_t layer, uint32_t position, uint32_t slot,
                       void **out_ptr);
/* kSlot / vSlot for a whole decode batch: row i of k_rows / v_rows (device memory,
 * src_stride_bytes apart, the K and V projections' outputs) is written to slot slots[i] at
 * position positions[i] of `layer`, one launch for up to 256 rows (the reference's projection
 * kernels write through kSlot / vSlot one session at a time). Cursors are not moved: advance
 * stays the caller's call, as in the reference. slots / positions are host arrays. */
int tt_kv_cache_write_rows(tt_kv_cache *cache, tt_stream stream, uint32_t layer, const uint32_t *slots,
                           const uint32_t *positions, uint32_t n, const void *k_rows,
                           const void *v_rows, uint32_t src_stride_bytes);
/* keyView / valueView (KVCacheManager+Views.swift:11-72). */
int tt_kv_cache_key_view(tt_kv_cache *cache, uint32_t layer, uint32_t slot,
                         uint32_t valid_token_count, tt_kv_view *out_view);
int tt_kv_cache_value_view(tt_kv_cache *cache, uint32_t layer, uint32_t slot,
                           uint32_t valid_token_count, tt_kv_view *out_view);
/* advance / rewind / reset / reset(slot:) (KVCacheManager+Storage.swift:272-337):
 * cursors only; rows are never cleared. */
int tt_kv_cache_advance(tt_kv_cache *cache, uint32_t slot, uint32_t count);
int tt_kv_cache_rewind(tt_kv_cache *cache, uint32_t slot, uint32_t new_position);
int tt_kv_cache_reset(tt_kv_cache *cache);
int tt_kv_cache_reset_slot(tt_kv_cache *cache, uint32_t slot);
uint32_t tt_kv_cache_position(const tt_kv_cache *cache, uint32_t slot);
uint32_t tt_kv_cache_capacity(const tt_kv_cache *cache, uint32_t layer);
uint32_t tt_kv_cache_stride(const tt_kv_cache *cache, uint32_t layer);
uint32_t tt_kv_cache_layer_kind(const tt_kv_cache *cache, uint32_t layer);
size_t tt_kv_cache_buffer_length(const tt_kv_cache *cache, uint32_t layer);
/* worstCaseBytes: every non-linear layer at max_context, K and V, all slots. */
size_t tt_kv_cache_worst_case_bytes(const tt_arch *arch, uint32_t max_context,
                                    uint32_t precision_bits, uint32_t slots);

/* Inference-state snapshot of slot 0, the segment layout of
 * KVCacheManager+Snapshot.swift:12-121: for every non-linear layer in order, the first
 * min(position, capacity) rows of K, then of V. _bytes gives the payload size at a position;
 * _export writes slot 0's prefix at its current cursor to host memory; _restore grows the
 * stores to `position` first (the lengths depend on capacity), resets every cursor, copies the
 * segments in and sets slot 0's cursor. A payload of the wrong size is TT_ERR_INVALID_ARG
 * (InferenceStateSnapshotError.invalidLayout). */
size_t tt_kv_cache_snapshot_bytes(const tt_kv_cache *cache, uint32_t position);
int tt_kv_cache_snapshot_export(tt_kv_cache *cache, void *host_dst, size_t capacity, size_t *out_bytes);
int tt_kv_cache_snapshot_restore(tt_kv_cache *cache, uint32_t position, const void *host_src, size_t bytes);

/* Host-KV streaming tier (KVCacheManager+HostStreaming.swift:33-364,
 * KVCacheManager+HostStreamingPrefill.swift:12-436): for `n_layers` streamed (full-attention)
 * layers the authoritative K/V rows live in a host arena [slots][max_context][stride]; device
 * memory holds only a window of min(window_tokens, max_context) rows per (layer, slot), filled
 * on demand with clock-hand eviction and write-back of dirty rows. Attention reads the window
 * through (logical key, window row) lists: tt_attn_decode_window takes the rows of a decode step,
 * tt_attn_prefill_causal_selected (keep_rows) those of a prefill chunk. `allocator` supplies the
 * window and staging memory and the arena<->window copies (NULL = CUDA device memory, synchronous
 * copies on the legacy default stream; the bookkeeping runs between steps, like the reference's,
 * which touches its shared buffers from the CPU between command buffers).
 *   _write_slot      kSlot / vSlot of a streamed layer: where the projection writes a position
 *                    (a window row, made dirty and pinned for the step; inside an active prefill
 *                    staging range, the staging row)
 *   _prepare_decode  prepareDecodeWindow: `indices` (host, ascending logical keys; NULL = all keys
 *                    0..count-1) made resident; out_indices / out_rows (host, count entries).
 *                    TT_ERR_OOM when the selection does not fit the window
 *   _begin_prefill   beginPrefillWrite: staging rows for a chunk, [token_count][stride]
 *   _prepare_prefill preparePrefillWindow: the union of the chunk's per-row selections
 *                    (sel_indices[t * sel_index_stride + i], i < sel_counts[t]; NULL = dense) made
 *                    resident, staged rows copied into the window, per-row lists written with
 *                    out_index_stride entries per row
 *   _commit          commitStreamedRows (called with advance): rows reach the arena
 *   _reset_slot      resetStreamedWindow
 *   _host_row        one arena row (hostRowBytes); _counters: evictions, rows copied in, bytes */
typedef struct tt_kv_window tt_kv_window;
tt_kv_window *tt_kv_window_create(uint32_t n_layers, uint32_t stride_bytes, uint32_t max_context,
                                  uint32_t slots, uint32_t window_tokens,
                                  const tt_allocator *allocator, int *out_err);
void tt_kv_window_destroy(tt_kv_window *window);
size_t tt_kv_window_bytes(const tt_kv_window *window);
size_t tt_kv_window_host_arena_bytes(const tt_kv_window *window);
uint32_t tt_kv_window_tokens(const tt_kv_window *window);
uint32_t tt_kv_window_prefill_chunk_tokens(const tt_kv_window *window, uint32_t configured,
                                           uint32_t selection_width);
int tt_kv_window_base(tt_kv_window *window, uint32_t layer, uint32_t slot, void **out_k, void **out_v);
int tt_kv_window_write_slot(tt_kv_window *window, uint32_t layer, uint32_t position, uint32_t slot,
                            void **out_k, void **out_v);
int tt_kv_window_row_of(tt_kv_window *window, uint32_t layer, uint32_t slot, uint32_t position,
                        int64_t *out_row);
int tt_kv_window_prepare_decode(tt_kv_window *window, uint32_t layer, uint32_t slot, uint32_t position,
                                const uint32_t *indices, uint32_t count, uint32_t *out_indices,
                                uint32_t *out_rows);
int tt_kv_window_begin_prefill(tt_kv_window *window, uint32_t layer, uint32_t slot,
                               uint32_t start_position, uint32_t token_count, void **out_stage_k,
                               void **out_stage_v);
int tt_kv_window_prepare_prefill(tt_kv_window *window, uint32_t layer, uint32_t slot,
                                 uint32_t start_position, uint32_t token_count,
                                 const uint32_t *sel_indices, uint32_t sel_index_stride,
                                 const uint32_t *sel_counts, uint32_t *out_indices,
                                 uint32_t *out_rows, uint32_t *out_counts, uint32_t out_index_stride);
int tt_kv_window_commit(tt_kv_window *window, uint32_t slot, uint32_t position, uint32_t count);
int tt_kv_window_reset_slot(tt_kv_window *window, uint32_t slot);
int tt_kv_window_host_row(tt_kv_window *window, uint32_t layer, uint32_t slot, uint32_t position,
                          int key, void *dst);
void tt_kv_window_counters(const tt_kv_window *window, uint64_t *out_evictions,
                           uint64_t *out_row_copies, uint64_t *out_copy_bytes);

/* GDNStateManager (sources/TinyTitan/Runtime/KVCache/GDNStateManager.swift:
 * 18-354): per linear layer a zero-initialised fp32 state buffer of
 * slots*Hv*Dv*Dk*4 bytes and an fp16 conv-tail buffer of
 * slots*(K-1)*qkvDim*2 bytes, optional checkpoint twins. */
tt_gdn_state *tt_gdn_state_create(const tt_arch *arch, uint32_t slots,
                                  int enable_speculative_checkpoint,
                                  const tt_allocator *allocator, int *out_err);
void tt_gdn_state_destroy(tt_gdn_state *state);
int tt_gdn_state_state_slot(tt_gdn_state *state, uint32_t layer, uint32_t slot, void **out_ptr);
int tt_gdn_state_conv_tail_slot(tt_gdn_state *state, uint32_t layer, uint32_t slot,
                                void **out_ptr);
int tt_gdn_state_speculative_state_slot(tt_gdn_state *state, uint32_t layer, uint32_t slot,
                                        void **out_ptr);
/* reset() / reset(slot:) (:207-226) zero-fill; like the KV manager's copies they run on the legacy
 * default stream until _bind_stream names the stream they are enqueued on. */
int tt_gdn_state_reset(tt_gdn_state *state);
int tt_gdn_state_reset_slot(tt_gdn_state *state, uint32_t slot);
int tt_gdn_state_bind_stream(tt_gdn_state *state, tt_stream stream);
/* encodeSpeculativeRestore(commandBuffer:) (:265-292): checkpoint twins -> live buffers of slot 0,
 * enqueued on `stream` (the stream of the verify pass that wrote the checkpoint), so it is ordered
 * with that pass exactly as the reference's blit is ordered inside its command buffer. */
int tt_gdn_state_speculative_restore(tt_gdn_state *state, tt_stream stream);
size_t tt_gdn_state_bytes_per_layer(const tt_gdn_state *state);
size_t tt_gdn_state_conv_tail_bytes_per_layer(const tt_gdn_state *state);
int tt_gdn_state_is_linear(const tt_gdn_state *state, uint32_t layer);
size_t tt_gdn_state_worst_case_bytes(const tt_arch *arch, uint32_t slots);
/* Snapshot segments of slot 0 (GDNStateManager.swift:228-344): for every linear layer in
 * order, the fp32 state then the fp16 conv tail. _restore zeroes everything first. */
size_t tt_gdn_state_snapshot_bytes(const tt_gdn_state *state);
int tt_gdn_state_snapshot_export(tt_gdn_state *state, void *host_dst, size_t capacity, size_t *out_bytes);
int tt_gdn_state_snapshot_restore(tt_gdn_state *state, const void *host_src, size_t bytes);

#ifdef __cplusplus
}
#endif

#endif /* TINYTITAN_CUDA_H */
