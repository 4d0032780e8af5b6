// The elementwise steps either side of full-attention SDPA in the Qwen gated-attention layer:
// split [query ; gate], per-head RMS norm of q and k with bf16 weights, NeoX partial RoPE, and the
// sigmoid output gate.
//
// Replaces the kernel chain of RealForwardRunner.encodeGatedFullPostProjection
// (sources/TinyTitan/Runtime/Inference/RealForwardRunner+DecodeFullAttention.swift:123-185):
// split_q_gate_fp16 (sources/TinyTitanCore/Metal/Primitives/utility.metal:142-160),
// rmsnorm_bf16w_perhead (Primitives/rmsnorm.metal:101-128), rope_neox_subdim
// (Primitives/rope.metal:32-49, :80-108) -- five launches in the reference, one here -- and
// sigmoid_gate_mul_fp16 (utility.metal:48-58). The reference's rounding points are kept (the
// normed value is rounded to fp16 before it is rotated), so the fused kernel gives what the chain
// of separate kernels gives.
#include "tt_common.h"

namespace {

struct PreParams {
    const __half *q_packed;   // [rows][H][2*D]  per head [query(D) ; gate(D)]
    __half *q_out;            // [rows][H][D]
    __half *gate_out;         // [rows][H][D]
    __half *k_rows;           // row r at k_rows + r * k_row_stride: [Hkv][D], normed + rotated in place
    const __nv_bfloat16 *q_norm_w, *k_norm_w;   // [D]
    uint32_t head_dim, n_q_heads, n_kv_heads, rotary_dim, rows, position0, k_row_stride;
    float theta, eps;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int kMaxPerLane = 16;   // head_dim <= 512

// one warp per (row, q head or k head)
__global__ void __launch_bounds__(128) attn_pre_kernel(PreParams p) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t heads = p.n_q_heads + p.n_kv_heads;
    const uint32_t row = warp / heads, hidx = warp % heads;
    if (row >= p.rows) return;
    const bool is_q = hidx < p.n_q_heads;
    const uint32_t D = p.head_dim;
    const __half *src;
    __half *dst;
    const __nv_bfloat16 *w;
    if (is_q) {
        src = p.q_packed + ((size_t)row * p.n_q_heads + hidx) * 2 * D;
        dst = p.q_out + ((size_t)row * p.n_q_heads + hidx) * D;
        w = p.q_norm_w;
        __half *g = p.gate_out + ((size_t)row * p.n_q_heads + hidx) * D;
        for (uint32_t i = lane; i < D; i += 32) g[i] = src[D + i];
    } else {
        dst = p.k_rows + (size_t)row * p.k_row_stride + (size_t)(hidx - p.n_q_heads) * D;
        src = dst;
        w = p.k_norm_w;
    }
    float x[kMaxPerLane];
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const uint32_t i = lane + 32 * j;
        x[j] = i < D ? __half2float(src[i]) : 0.f;
        acc = fmaf(x[j], x[j], acc);
    }
    acc = warp_sum(acc);
    const float inv = rsqrtf(acc / (float)D + p.eps);
    // normed value, rounded to fp16 exactly where the separate norm kernel stores it
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const uint32_t i = lane + 32 * j;
        if (i < D) dst[i] = __float2half_rn(x[j] * inv * __bfloat162float(w[i]));
    }
    __syncwarp();
    // NeoX pairing (i, rotary/2 + i) inside the first rotary_dim elements, frequency divisor
    // rotary_dim; elements >= rotary_dim pass through (rope_neox_subdim). The row was just written
    // by this warp, so the pairs are re-read from L1.
    const uint32_t half_rot = p.rotary_dim / 2;
    const float pos = (float)(p.position0 + row);
    for (uint32_t pair = lane; pair < half_rot; pair += 32) {
        const float exponent = -(float)(2u * pair) / (float)p.rotary_dim;
        const float angle = pos * powf(p.theta, exponent);
        const float c = cosf(angle), sn = sinf(angle);
        const float x0 = __half2float(dst[pair]), x1 = __half2float(dst[half_rot + pair]);
        dst[pair] = __float2half_rn(x0 * c - x1 * sn);
        dst[half_rot + pair] = __float2half_rn(x0 * sn + x1 * c);
    }
}

__global__ void sigmoid_gate_mul_kernel(__half *out, const __half *gate, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float g = __half2float(gate[i]);
    out[i] = __float2half_rn(__half2float(out[i]) / (1.f + expf(-g)));
}

}  // namespace

TT_API int tt_attn_pre(tt_context *ctx, tt_stream stream, const void *q_packed, void *q_out, void *gate_out, void *k_rows,
                       const void *q_norm_weight, const void *k_norm_weight, uint32_t head_dim, uint32_t n_q_heads,
                       uint32_t n_kv_heads, uint32_t rotary_dim, float theta, float eps, uint32_t position,
                       uint32_t rows, uint32_t k_row_stride_elements) {
    TT_ENTER(ctx);
    if (q_packed == nullptr || q_out == nullptr || gate_out == nullptr || k_rows == nullptr || q_norm_weight == nullptr ||
        k_norm_weight == nullptr || head_dim == 0 || n_q_heads == 0 || n_kv_heads == 0 || rows == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "attention pre-step needs non-null buffers and positive sizes");
    if (head_dim > 32 * kMaxPerLane) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "head_dim must be <= 512");
    if (rotary_dim > head_dim || (rotary_dim & 1))
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "rotary_dim must be even and <= head_dim");
    if (k_row_stride_elements < n_kv_heads * head_dim)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "K row stride is smaller than n_kv_heads*head_dim");
    PreParams p;
    p.q_packed = (const __half *)q_packed; p.q_out = (__half *)q_out; p.gate_out = (__half *)gate_out;
    p.k_rows = (__half *)k_rows; p.q_norm_w = (const __nv_bfloat16 *)q_norm_weight;
    p.k_norm_w = (const __nv_bfloat16 *)k_norm_weight; p.head_dim = head_dim; p.n_q_heads = n_q_heads;
    p.n_kv_heads = n_kv_heads; p.rotary_dim = rotary_dim; p.rows = rows; p.position0 = position;
    p.k_row_stride = k_row_stride_elements; p.theta = theta; p.eps = eps;
    const uint64_t warps = (uint64_t)rows * (n_q_heads + n_kv_heads);
    attn_pre_kernel<<<(uint32_t)((warps + 3) / 4), 128, 0, (cudaStream_t)stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_pre launch");
    ctx->launches++;
    return TT_OK;
}

TT_API int tt_attn_gate_mul(tt_context *ctx, tt_stream stream, void *out, const void *gate, uint32_t count) {
    TT_ENTER(ctx);
    if (out == nullptr || gate == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "gate multiply needs non-null buffers");
    if (count == 0) return TT_OK;
    sigmoid_gate_mul_kernel<<<(count + 255) / 256, 256, 0, (cudaStream_t)stream>>>((__half *)out, (const __half *)gate, count);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "sigmoid_gate_mul launch");
    ctx->launches++;
    return TT_OK;
}
