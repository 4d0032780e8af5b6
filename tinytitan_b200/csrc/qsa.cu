// Qwen Sparse Attention's block indexer: pooled-key cache, block scores and the key selection.
//
// Replaces the kernels of sources/TinyTitanCore/Metal/Attention/qsa.metal:1-226 and the host-side
// selection of sources/TinyTitan/Kernels/Attention/QSAIndexer.swift:391-498 (selectKeysPrefill) and
// QSAIndexer+Scratch.swift:178-251 (selectKeysCompact / selectKeys):
//
//   qsa_pool_kernel     qsa_pool_block / qsa_pool_blocks (:14-65) fused with the per-block RMS norm and
//                       the NeoX rotation the reference launches right after them
//                       (QSAIndexer.encodePoolPrefill, QSAIndexer.swift:196-238; rmsnorm_bf16w_perhead,
//                       Primitives/rmsnorm.metal:101-128; rope_neox_subdim_strided, Primitives/rope.metal:
//                       116-141). The fp16 stores between the three reference kernels are kept as
//                       roundings in registers, so the cache holds the same values.
//   qsa_query_kernel    the indexer query's per-head norm and rotation (QSAIndexer.swift:259-274, :322-337)
//   qsa_scores_kernel   qsa_block_scores / qsa_block_scores_rows (:67-126): sum over heads of
//                       max(0, q[h] . pooled[b]), rectified per head BEFORE the sum
//   qsa_select_kernel   qsa_select_decode (:128-226) for every query row of a chunk: radix select of the
//                       block at rank B over the 64-bit key (orderable score, inverted index), whole
//                       blocks above it, a partial block at it, the ragged tail always; the mask AND the
//                       ascending compact index list with its count leave the same kernel, so neither the
//                       scores nor the mask travel to the host (the reference compacts on the CPU).
#include "tt_common.h"

namespace {

constexpr int kMaxIndexerDim = 512;

__device__ __forceinline__ float round_half(float x) { return __half2float(__float2half_rn(x)); }

// RMS norm with a bf16 weight, then the NeoX rotation of the whole row at `position`; one warp per
// row, `x` holds this lane's elements lane, lane + 32, ... (fp16-representable values). Both
// reference kernels store fp16, so the value is rounded after the norm and after the rotation.
template <int PER_LANE>
__device__ __forceinline__ void warp_norm_rope(float (&x)[PER_LANE], uint32_t dim, const __nv_bfloat16 *weight, float eps,
                                               float theta, float position, int lane) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) ss = fmaf(x[i], x[i], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)dim + eps);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < dim) x[i] = round_half(x[i] * inv * __bfloat162float(weight[d]));
    }
    // pair (p, dim/2 + p): element d < dim/2 is the lower member, d >= dim/2 the upper one. The partner
    // sits in lane (d +- dim/2) % 32 at slot (d +- dim/2) / 32; dim/2 is a multiple of 32 when dim is a
    // multiple of 64, so the partner is in the SAME lane, dim/64 slots away.
    const uint32_t half_dim = dim / 2;
    const int shift = half_dim / 32;
#pragma unroll
    for (int i = 0; i < PER_LANE / 2; ++i) {
        if (i >= shift) break;
        const uint32_t pair = lane + 32 * i;
        const float exponent = -(float)(2u * pair) / (float)dim;
        const float angle = position * powf(theta, exponent);
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float x0 = x[i], x1 = x[i + shift];
        x[i] = round_half(x0 * cs - x1 * sn);
        x[i + shift] = round_half(x0 * sn + x1 * cs);
    }
}

// grid = ceil(block_count / 4), block = 128: one warp per pooled block.
template <int PER_LANE>
__global__ void __launch_bounds__(128)
qsa_pool_kernel(const __half *__restrict__ raw, __half *__restrict__ pooled, uint32_t dim, uint32_t first_block,
                uint32_t block_count, uint32_t ratio, uint32_t n_kv, const __nv_bfloat16 *__restrict__ weight, float eps,
                float theta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t local = blockIdx.x * 4 + warp;
    if (local >= block_count) return;
    const uint32_t block = first_block + local;
    const uint32_t first = block * ratio;
    if (first >= n_kv) return;
    const uint32_t count = min(ratio, n_kv - first);       // the tail block is the mean of the members present
    float x[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t d = lane + 32 * i;
        float acc = 0.f;
        if (d < dim)
            for (uint32_t m = 0; m < count; ++m) acc += __half2float(raw[(size_t)(first + m) * dim + d]);
        x[i] = d < dim ? round_half(acc / (float)count) : 0.f;
    }
    if (weight != nullptr) warp_norm_rope<PER_LANE>(x, dim, weight, eps, theta, (float)(block * ratio), lane);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < dim) pooled[(size_t)block * dim + d] = __float2half_rn(x[i]);
    }
}

// In place over [rows][heads][dim]: one warp per (row, head); row r sits at position + r.
template <int PER_LANE>
__global__ void __launch_bounds__(128)
qsa_query_kernel(__half *__restrict__ query, uint32_t dim, uint32_t heads, uint32_t rows, uint32_t position,
                 const __nv_bfloat16 *__restrict__ weight, float eps, float theta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t idx = blockIdx.x * 4 + warp;
    if (idx >= rows * heads) return;
    __half *row = query + (size_t)idx * dim;
    float x[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t d = lane + 32 * i;
        x[i] = d < dim ? __half2float(row[d]) : 0.f;
    }
    warp_norm_rope<PER_LANE>(x, dim, weight, eps, theta, (float)(position + idx / heads), lane);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < dim) row[d] = __float2half_rn(x[i]);
    }
}

// grid = (ceil(blocks / 128), rows), block = 128: the row's query heads sit in shared memory as fp32;
// thread j scores pooled block j against all of them, one 16-byte load of the pooled row at a time.
__global__ void __launch_bounds__(128)
qsa_scores_kernel(const __half *__restrict__ query, const __half *__restrict__ pooled, float *__restrict__ scores,
                  uint32_t dim, uint32_t heads, uint32_t blocks, uint32_t score_stride) {
    extern __shared__ float q_s[];   // [heads][dim]
    const uint32_t t = blockIdx.y;
    const __half *q = query + (size_t)t * heads * dim;
    for (uint32_t i = threadIdx.x; i < heads * dim; i += blockDim.x) q_s[i] = __half2float(q[i]);
    __syncthreads();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const uint4 *row = reinterpret_cast<const uint4 *>(pooled + (size_t)b * dim);
    float total = 0.f;
    for (uint32_t h = 0; h < heads; ++h) {
        const float *qh = q_s + h * dim;
        float dot = 0.f;
        for (uint32_t c = 0; c < dim / 8; ++c) {
            const uint4 u = row[c];
            const __half2 *p = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(p[e]);
                dot = fmaf(qh[c * 8 + 2 * e], f.x, dot);
                dot = fmaf(qh[c * 8 + 2 * e + 1], f.y, dot);
            }
        }
        total += fmaxf(dot, 0.f);     // rectified per head, before the sum over heads
    }
    scores[(size_t)t * score_stride + b] = total;
}

__device__ __forceinline__ uint32_t qsa_orderable(float s) {
    if (s == 0.0f) s = 0.0f;          // -0.0 ties +0.0
    const uint32_t f = __float_as_uint(s);
    return (f & 0x80000000u) ? ~f : (f | 0x80000000u);
}
__device__ __forceinline__ unsigned long long qsa_key(const float *scores, uint32_t i) {
    return ((unsigned long long)qsa_orderable(scores[i]) << 32) | (unsigned long long)(0xFFFFFFFFu - i);
}

// grid = rows, block = 256. Row r sees keys [0, start + r + 1).
constexpr int kSelectThreads = 256;
__global__ void __launch_bounds__(kSelectThreads)
qsa_select_kernel(const float *__restrict__ scores_all, uint32_t score_stride, uint32_t start_position, uint32_t ratio,
                  uint32_t width, uint8_t *__restrict__ keep_all, uint32_t keep_stride, uint32_t *__restrict__ indices_all,
                  uint32_t index_stride, uint32_t *__restrict__ counts) {
    __shared__ uint32_t hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ uint32_t rank_s;
    __shared__ uint32_t scan_s[kSelectThreads];
    __shared__ uint32_t running_s;
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const uint32_t visible = start_position + row + 1;
    const float *scores = scores_all + (size_t)row * score_stride;
    uint8_t *keep = keep_all ? keep_all + (size_t)row * keep_stride : nullptr;
    uint32_t *indices = indices_all ? indices_all + (size_t)row * index_stride : nullptr;

    // cells past the row's own position are never selected
    if (keep)
        for (uint32_t c = visible + tid; c < keep_stride; c += kSelectThreads) keep[c] = 0;

    if (visible <= width) {           // inside the dense window every visible key is kept
        for (uint32_t c = tid; c < visible; c += kSelectThreads) {
            if (keep && c < keep_stride) keep[c] = 1;
            if (indices && c < index_stride) indices[c] = c;
        }
        if (tid == 0 && counts) counts[row] = min(visible, indices ? index_stride : visible);
        return;
    }
    const uint32_t complete = (visible / ratio) * ratio;
    const uint32_t tail = visible - complete;
    const uint32_t blocks = complete / ratio;
    // how many cells every complete block contributes: ratio above the rank-B key, `partial` at it
    uint32_t whole_blocks, partial;
    bool take_all = false, take_none = false;
    if (width <= tail) {
        take_none = true; whole_blocks = 0; partial = 0;
    } else {
        const uint32_t remaining = width - tail;
        whole_blocks = remaining / ratio;
        partial = remaining - whole_blocks * ratio;
        if (whole_blocks >= blocks) take_all = true;
    }
    unsigned long long key_b = 0;
    if (!take_all && !take_none) {
        // radix select, eight 8-bit passes from the top digit: the key of the block at rank B (descending)
        if (tid == 0) { prefix_s = 0ull; rank_s = whole_blocks; }
        __syncthreads();
        for (int pass = 7; pass >= 0; --pass) {
            const uint32_t shift = (uint32_t)pass * 8u;
            hist[tid] = 0;            // 256 threads, 256 bins
            __syncthreads();
            const unsigned long long prefix = prefix_s;
            const unsigned long long mask = (pass == 7) ? 0ull : (~0ull << (shift + 8u));
            for (uint32_t i = tid; i < blocks; i += kSelectThreads) {
                const unsigned long long k = qsa_key(scores, i);
                if ((k & mask) == prefix) atomicAdd(&hist[(uint32_t)((k >> shift) & 0xFFull)], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                uint32_t r = rank_s, digit = 0;
                for (int b = 255; b >= 0; --b) {
                    const uint32_t n = hist[b];
                    if (r < n) { digit = (uint32_t)b; break; }
                    r -= n;
                }
                rank_s = r;
                prefix_s = prefix | ((unsigned long long)digit << shift);
            }
            __syncthreads();
        }
        key_b = prefix_s;
    }
    // mask and ascending compaction, 256 blocks per round: an exclusive scan of the per-block counts
    if (tid == 0) running_s = 0;
    __syncthreads();
    for (uint32_t base = 0; base < blocks; base += kSelectThreads) {
        const uint32_t i = base + tid;
        uint32_t take = 0;
        if (i < blocks) {
            if (take_all) take = ratio;
            else if (!take_none) {
                const unsigned long long k = qsa_key(scores, i);
                take = k > key_b ? ratio : (k == key_b ? partial : 0u);
            }
            if (keep)
                for (uint32_t c = 0; c < ratio; ++c)
                    if (i * ratio + c < keep_stride) keep[i * ratio + c] = c < take ? 1 : 0;
        }
        scan_s[tid] = take;
        __syncthreads();
        for (uint32_t off = 1; off < kSelectThreads; off <<= 1) {      // inclusive Hillis-Steele scan
            const uint32_t v = tid >= off ? scan_s[tid - off] : 0u;
            __syncthreads();
            scan_s[tid] += v;
            __syncthreads();
        }
        const uint32_t before = running_s + scan_s[tid] - take;
        if (indices)
            for (uint32_t c = 0; c < take; ++c)
                if (before + c < index_stride) indices[before + c] = i * ratio + c;
        __syncthreads();
        if (tid == kSelectThreads - 1) running_s += scan_s[tid];
        __syncthreads();
    }
    // the ragged tail of the query's own block, always kept, highest indices of the row
    const uint32_t kept_blocks = running_s;
    for (uint32_t c = tid; c < tail; c += kSelectThreads) {
        if (keep && complete + c < keep_stride) keep[complete + c] = 1;
        if (indices && kept_blocks + c < index_stride) indices[kept_blocks + c] = complete + c;
    }
    if (tid == 0 && counts) counts[row] = indices ? min(kept_blocks + tail, index_stride) : kept_blocks + tail;
}

}  // namespace

TT_API int tt_qsa_pool_blocks(tt_context *ctx, tt_stream stream, const void *raw_keys, void *pooled, uint32_t head_dim,
                              uint32_t first_block, uint32_t block_count, uint32_t ratio, uint32_t n_kv,
                              const void *key_norm_weight, float eps, float theta) {
    TT_ENTER(ctx);
    if (raw_keys == nullptr || pooled == nullptr || ratio == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa pool: null buffer or zero compress ratio");
    if (head_dim == 0 || head_dim > (uint32_t)kMaxIndexerDim || head_dim % 64 != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "qsa: indexer head_dim must be a multiple of 64 up to %d", kMaxIndexerDim);
    if (block_count == 0) return TT_OK;
    const uint32_t grid = (block_count + 3) / 4;
    const __half *raw = static_cast<const __half *>(raw_keys);
    const __nv_bfloat16 *w = static_cast<const __nv_bfloat16 *>(key_norm_weight);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim <= 128)
        qsa_pool_kernel<4><<<grid, 128, 0, s>>>(raw, static_cast<__half *>(pooled), head_dim, first_block, block_count, ratio, n_kv, w, eps, theta);
    else if (head_dim <= 256)
        qsa_pool_kernel<8><<<grid, 128, 0, s>>>(raw, static_cast<__half *>(pooled), head_dim, first_block, block_count, ratio, n_kv, w, eps, theta);
    else
        qsa_pool_kernel<16><<<grid, 128, 0, s>>>(raw, static_cast<__half *>(pooled), head_dim, first_block, block_count, ratio, n_kv, w, eps, theta);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "qsa_pool launch");
    ctx->launches++;
    return TT_OK;
}

TT_API int tt_qsa_query_norm_rope(tt_context *ctx, tt_stream stream, void *query, uint32_t head_dim, uint32_t heads,
                                  uint32_t rows, uint32_t position, const void *query_norm_weight, float eps, float theta) {
    TT_ENTER(ctx);
    if (query == nullptr || query_norm_weight == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa query: null buffer");
    if (head_dim == 0 || head_dim > (uint32_t)kMaxIndexerDim || head_dim % 64 != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "qsa: indexer head_dim must be a multiple of 64 up to %d", kMaxIndexerDim);
    if (rows == 0 || heads == 0) return TT_OK;
    const uint32_t grid = (rows * heads + 3) / 4;
    const __nv_bfloat16 *w = static_cast<const __nv_bfloat16 *>(query_norm_weight);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim <= 128) qsa_query_kernel<4><<<grid, 128, 0, s>>>(static_cast<__half *>(query), head_dim, heads, rows, position, w, eps, theta);
    else if (head_dim <= 256) qsa_query_kernel<8><<<grid, 128, 0, s>>>(static_cast<__half *>(query), head_dim, heads, rows, position, w, eps, theta);
    else qsa_query_kernel<16><<<grid, 128, 0, s>>>(static_cast<__half *>(query), head_dim, heads, rows, position, w, eps, theta);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "qsa_query launch");
    ctx->launches++;
    return TT_OK;
}

TT_API int tt_qsa_block_scores(tt_context *ctx, tt_stream stream, const void *query, const void *pooled, float *scores,
                               uint32_t head_dim, uint32_t heads, uint32_t blocks, uint32_t rows, uint32_t score_stride) {
    TT_ENTER(ctx);
    if (query == nullptr || pooled == nullptr || scores == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa scores: null buffer");
    if (head_dim == 0 || head_dim % 8 != 0 || ((uintptr_t)pooled & 15))
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "qsa scores: head_dim must be a multiple of 8 and the pooled cache 16-byte aligned");
    if (score_stride < blocks) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa scores: score stride below the block count");
    const size_t smem = (size_t)heads * head_dim * sizeof(float);
    if (smem > 48 * 1024) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "qsa scores: heads * head_dim exceeds 12288");
    if (rows == 0 || blocks == 0 || heads == 0) return TT_OK;
    if (rows > 65535) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "qsa scores: at most 65535 query rows per call");
    const dim3 grid((blocks + 127) / 128, rows);
    qsa_scores_kernel<<<grid, 128, smem, (cudaStream_t)stream>>>(static_cast<const __half *>(query), static_cast<const __half *>(pooled),
                                                                  scores, head_dim, heads, blocks, score_stride);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "qsa_scores launch");
    ctx->launches++;
    return TT_OK;
}

TT_API int tt_qsa_select_keys(tt_context *ctx, tt_stream stream, const float *scores, uint32_t score_stride,
                              uint32_t start_position, uint32_t rows, uint32_t ratio, uint32_t width, uint8_t *keep,
                              uint32_t keep_stride, uint32_t *indices, uint32_t index_stride, uint32_t *counts) {
    TT_ENTER(ctx);
    if (scores == nullptr || ratio == 0 || width == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa select: null scores, zero ratio or zero width");
    if (keep == nullptr && indices == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa select: no output requested");
    if (indices != nullptr && counts == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa select: an index list needs its counts");
    if (rows == 0) return TT_OK;
    if ((uint64_t)start_position + rows > 0xFFFFFFFFull) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qsa select: position overflow");
    qsa_select_kernel<<<rows, kSelectThreads, 0, (cudaStream_t)stream>>>(scores, score_stride, start_position, ratio, width, keep,
                                                                         keep_stride, indices, index_stride, counts);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "qsa_select launch");
    ctx->launches++;
    return TT_OK;
}
