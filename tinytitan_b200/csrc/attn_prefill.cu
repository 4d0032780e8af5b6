// Causal prefill attention: dispatch + the generic CUDA kernel.
//
// Replaces PrefillAttention.encodeCausal
// (sources/TinyTitan/Kernels/Attention/PrefillAttention.swift:165-258) and the kernels
// attention_prefill_causal_tiled / _q8 (sources/TinyTitanCore/Metal/Prefill/prefill.metal:
// 1056-1313). The generic kernel takes any head_dim <= 512 and any element strides / 2-byte
// aligned base pointers (the reference's tests use padded strides and odd buffer offsets); the
// tcgen05 kernel in attn_prefill_tc.cu takes the aligned head_dim-256 case.
#include "tt_common.h"

int tt_launch_prefill_tc(tt_context *ctx, cudaStream_t stream, const void *q, const void *k, const void *v,
                         void *out, const tt_prefill_params *p, uint32_t io_dtype);

namespace {

constexpr int kGenericWarps = 4;
constexpr int kMaxHeadDim = 512;

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Element `flat` of a cache row: fp16/bf16 rows directly, affine-quantised rows as
// code * scale[group] + bias[group] with the scales and biases stored after the packed codes
// (attn_load_kv, sources/TinyTitanCore/Metal/Attention/attention.metal:89-117;
// prefill.metal:772-797).
template <typename T>
__device__ __forceinline__ float load_kv(const T *cache, uint32_t row, uint32_t flat, const tt_prefill_params &p) {
    if (p.kv_bits == 16) return to_f32<T>(cache[(size_t)row * p.kv_token_stride_elements + flat]);
    const unsigned char *r = reinterpret_cast<const unsigned char *>(cache) + (size_t)row * p.kv_token_stride_bytes;
    uint32_t code;
    if (p.kv_bits == 8) {
        code = r[flat];
    } else {
        const unsigned char packed = r[flat >> 1];
        code = (flat & 1u) ? (packed >> 4) : (packed & 0x0fu);
    }
    const uint32_t elems = p.n_kv_heads * p.head_dim;
    const uint32_t groups = (elems + p.kv_group_size - 1) / p.kv_group_size;
    const __half *scales = reinterpret_cast<const __half *>(r + p.kv_value_bytes);
    const uint32_t g = flat / p.kv_group_size;
    return (float)code * __half2float(scales[g]) + __half2float(scales[groups + g]);
}

// A per-query key selection (the `useKeep` modes of attention_prefill_causal_qsa_tiled,
// sources/TinyTitanCore/Metal/Prefill/prefill.metal:914-1054): 0 every visible key; 1 a byte mask
// keep[t * keep_stride + key]; 2 a compact list indices[t * index_stride + i], i < counts[t], of logical
// keys (entries outside the row's visible range are dropped); 3 the same list with rows[...] giving the
// cache row that holds each key (host-KV window).
struct PrefillSelection {
    uint32_t mode;
    const uint8_t *keep;
    uint32_t keep_stride;
    const uint32_t *indices;
    const uint32_t *counts;
    uint32_t index_stride;
    const uint32_t *rows;
};

// One warp per (query row, q head). Keys are taken 32 at a time: lane j scores key j (a full
// head_dim dot product against the query held in shared memory), the tile's softmax update is
// done with warp reductions, then every lane accumulates its own output dimensions over the
// 32 probabilities (broadcast by shuffle).
template <typename T>
__global__ void __launch_bounds__(kGenericWarps * 32)
attn_prefill_generic_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                            T *__restrict__ out, tt_prefill_params p, uint32_t ring, PrefillSelection sel) {
    __shared__ float q_s[kGenericWarps][kMaxHeadDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair = blockIdx.x * kGenericWarps + warp;
    if (pair >= p.query_count * p.n_q_heads) return;
    const uint32_t t = pair / p.n_q_heads, h = pair % p.n_q_heads;
    const uint32_t hd = p.head_dim;
    const uint32_t kvh = h / (p.n_q_heads / p.n_kv_heads);
    const uint32_t abs_q = p.start_position + t;
    uint32_t first = 0;
    if (p.sliding_window != 0 && abs_q + 1 > p.sliding_window) first = abs_q + 1 - p.sliding_window;
    const uint32_t last = min(p.kv_valid_count, abs_q + 1);

    const T *qr = q + (size_t)t * p.q_token_stride_elements + (size_t)h * hd;
    for (uint32_t d = lane; d < hd; d += 32) q_s[warp][d] = to_f32<T>(qr[d]) * p.scale;
    __syncwarp();

    constexpr int kPerLane = kMaxHeadDim / 32;
    float acc[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    // steps of the row: visible keys, or the entries of its compact list
    const bool compact = sel.mode >= 2;
    const uint32_t steps = compact ? sel.counts[t] : (last > first ? last - first : 0u);
    for (uint32_t step0 = 0; step0 < steps; step0 += 32) {
        const uint32_t step = step0 + lane;
        float s = -INFINITY;
        uint32_t phys = 0;
        if (step < steps) {
            uint32_t key;
            bool valid;
            if (compact) {
                key = sel.indices[(size_t)t * sel.index_stride + step];
                valid = key >= first && key < last;
                phys = sel.mode == 3 ? sel.rows[(size_t)t * sel.index_stride + step] : (ring ? key % ring : key);
            } else {
                key = first + step;
                valid = sel.mode == 0 || sel.keep[(size_t)t * sel.keep_stride + key] != 0;
                phys = ring ? key % ring : key;
            }
            if (valid) {
                float dot = 0.f;
                if (p.kv_bits == 16) {
                    const T *kr = k + (size_t)phys * p.kv_token_stride_elements + (size_t)kvh * hd;
                    for (uint32_t d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], to_f32<T>(kr[d]), dot);
                } else {
                    for (uint32_t d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], load_kv<T>(k, phys, kvh * hd + d, p), dot);
                }
                s = dot;
            }
        }
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run, mx);
        if (m_new == -INFINITY) continue;              // every key so far was dropped: nothing to carry (prefill.metal:1013-1020)
        const float alpha = __expf(m_run - m_new);     // exp(-inf) == 0 on the first contributing tile
        const float pe = (s != -INFINITY) ? __expf(s - m_new) : 0.f;
        float ps = pe;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l_run = l_run * alpha + ps;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) acc[i] *= alpha;
        const uint32_t n = min(32u, steps - step0);
        for (uint32_t j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pe, j);
            const uint32_t pr = __shfl_sync(0xffffffffu, phys, j);
            if (pj == 0.f) continue;                   // dropped keys are never read
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                const uint32_t d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, load_kv<T>(v, pr, kvh * hd + d, p), acc[i]);
            }
        }
    }
    T *orow = out + (size_t)t * p.o_token_stride_elements + (size_t)h * hd;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;   // row_sum == 0 -> 0 (prefill.metal:1154-1157)
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < hd) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

int validate_prefill(tt_context *ctx, const void *q, const void *k, const void *v, const void *out,
                     const tt_prefill_params *p, uint32_t io_dtype) {
    // PrefillAttention.validate (PrefillAttention.swift:334-363)
    if (p == nullptr || q == nullptr || k == nullptr || v == nullptr || out == nullptr)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "prefill attention needs non-null buffers and params");
    if (p->head_dim == 0) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "headDim must be positive");
    if (p->query_count == 0) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "queryCount must be positive");
    if (p->n_q_heads == 0 || p->n_kv_heads == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "numQHeads and numKVHeads must be positive");
    if (p->n_q_heads % p->n_kv_heads != 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "numQHeads must be divisible by numKVHeads");
    if (p->q_token_stride_elements < p->n_q_heads * p->head_dim)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "q token stride is too small");
    if (p->o_token_stride_elements < p->n_q_heads * p->head_dim)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "output token stride is too small");
    if (p->kv_bits != 16) {
        if (p->kv_bits != 4 && p->kv_bits != 8)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "KV bits must be 4, 8, or 16");
        if (p->kv_token_stride_bytes == 0)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "quantized KV token stride must be positive");
        const uint32_t elems = p->n_kv_heads * p->head_dim;
        if (p->kv_group_size == 0 || p->kv_value_bytes < (elems * p->kv_bits + 7) / 8 ||
            p->kv_token_stride_bytes < p->kv_value_bytes + (elems + p->kv_group_size - 1) / p->kv_group_size * 4)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "quantized KV row layout is too small for its values and groups");
    } else if (p->kv_token_stride_elements < p->n_kv_heads * p->head_dim) {
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "KV token stride is too small");
    }
    if ((uint64_t)p->start_position + p->query_count > p->kv_valid_count)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "kvValidCount must include all in-flight query rows");
    if (p->head_dim > (uint32_t)kMaxHeadDim)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "head_dim %u exceeds %d", p->head_dim, kMaxHeadDim);
    if (io_dtype != TT_F16 && io_dtype != TT_BF16)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "io_dtype must be TT_F16 or TT_BF16");
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 1)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "buffers must be 2-byte aligned");
    return TT_OK;
}

}  // namespace

TT_API int tt_attn_prefill_path(const void *q, const void *k, const void *v, const void *out,
                                const tt_prefill_params *p, uint32_t kv_ring_capacity) {
    if (p == nullptr) return 0;
    const bool aligned = ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) == 0) &&
                         (p->q_token_stride_elements % 8 == 0) && (p->kv_token_stride_elements % 8 == 0) &&
                         (p->o_token_stride_elements % 8 == 0);
    // the tensor-core kernel takes row maxima before scaling, which needs a positive scale
    return (aligned && p->head_dim == 256 && kv_ring_capacity == 0 && p->kv_bits == 16 && p->scale > 0.f) ? 1 : 0;
}

static int launch_generic(tt_context *ctx, cudaStream_t stream, const void *q, const void *k, const void *v, void *out,
                          const tt_prefill_params *params, uint32_t kv_ring_capacity, uint32_t io_dtype,
                          const PrefillSelection &sel) {
    const uint32_t pairs = params->query_count * params->n_q_heads;
    const uint32_t blocks = (pairs + kGenericWarps - 1) / kGenericWarps;
    if (io_dtype == TT_F16)
        attn_prefill_generic_kernel<__half><<<blocks, kGenericWarps * 32, 0, stream>>>(
            (const __half *)q, (const __half *)k, (const __half *)v, (__half *)out, *params, kv_ring_capacity, sel);
    else
        attn_prefill_generic_kernel<__nv_bfloat16><<<blocks, kGenericWarps * 32, 0, stream>>>(
            (const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v, (__nv_bfloat16 *)out,
            *params, kv_ring_capacity, sel);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_prefill_generic launch");
    ctx->launches++;
    return TT_OK;
}

TT_API int tt_attn_prefill_causal(tt_context *ctx, tt_stream stream, const void *q, const void *k, const void *v,
                                  void *out, const tt_prefill_params *params, uint32_t kv_ring_capacity,
                                  uint32_t io_dtype) {
    TT_ENTER(ctx);
    int rc = validate_prefill(ctx, q, k, v, out, params, io_dtype);
    if (rc != TT_OK) return rc;
    if (tt_attn_prefill_path(q, k, v, out, params, kv_ring_capacity) == 1 && getenv("TT_PREFILL_FORCE_GENERIC") == nullptr)
        return tt_launch_prefill_tc(ctx, (cudaStream_t)stream, q, k, v, out, params, io_dtype);
    PrefillSelection none = {0, nullptr, 0, nullptr, nullptr, 0, nullptr};
    return launch_generic(ctx, (cudaStream_t)stream, q, k, v, out, params, kv_ring_capacity, io_dtype, none);
}

TT_API int tt_attn_prefill_causal_selected(tt_context *ctx, tt_stream stream, const void *q, const void *k, const void *v,
                                           void *out, const tt_prefill_params *params, uint32_t kv_ring_capacity,
                                           uint32_t io_dtype, const uint8_t *keep_mask, uint32_t keep_stride,
                                           const uint32_t *keep_indices, uint32_t keep_index_stride,
                                           const uint32_t *keep_counts, const uint32_t *keep_rows) {
    TT_ENTER(ctx);
    int rc = validate_prefill(ctx, q, k, v, out, params, io_dtype);
    if (rc != TT_OK) return rc;
    // the mode follows from what was bound, as in PrefillAttention.encodeCausal (PrefillAttention.swift:214-226)
    PrefillSelection sel = {0, keep_mask, keep_stride, keep_indices, keep_counts, keep_index_stride, keep_rows};
    const bool compacted = keep_indices != nullptr && keep_counts != nullptr;
    if (compacted) sel.mode = keep_rows != nullptr ? 3u : 2u;
    else if (keep_mask != nullptr) sel.mode = 1u;
    else if (keep_indices != nullptr || keep_counts != nullptr || keep_rows != nullptr)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "a compact selection needs both its index list and its counts");
    if (sel.mode == 1 && keep_stride < params->kv_valid_count && keep_stride < params->start_position + params->query_count)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "keep mask stride does not cover the visible keys");
    if (sel.mode >= 2 && keep_index_stride == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "compact selection with a zero index stride");
    if (sel.mode == 0) {
        if (tt_attn_prefill_path(q, k, v, out, params, kv_ring_capacity) == 1 && getenv("TT_PREFILL_FORCE_GENERIC") == nullptr)
            return tt_launch_prefill_tc(ctx, (cudaStream_t)stream, q, k, v, out, params, io_dtype);
    }
    return launch_generic(ctx, (cudaStream_t)stream, q, k, v, out, params, kv_ring_capacity, io_dtype, sel);
}
