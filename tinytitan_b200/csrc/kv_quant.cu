// Affine quantisation of K/V rows into the cache's packed row format.
//
// Replaces kv_cache_quantize_affine (sources/TinyTitanCore/Metal/Quant/kv_cache_quantize.metal:4-72).
// A destination row is [packed codes | fp16 scale per group | fp16 bias per group]
// (KVCacheManager.rowLayout, KVCacheManager+Validation.swift:30-41). One CTA of `group_size`
// threads per (group, token): bias = min, scale = (max - min) / levels, code =
// round(clamp((x - bias) / scale, 0, levels)) computed with the fp32 scale and bias; the stored
// scale and bias are their fp16 roundings, exactly as the reference does.
#include "tt_common.h"

namespace {

__global__ void kv_quantize_affine_kernel(const __half *__restrict__ source, unsigned char *__restrict__ destination,
                                          uint32_t source_stride, uint32_t destination_stride, uint32_t values_bytes,
                                          uint32_t element_count, uint32_t bits, uint32_t group_size) {
    __shared__ float mins[32], maxs[32];
    __shared__ float s_scale, s_bias;
    const uint32_t lid = threadIdx.x, lane = lid & 31, warp = lid >> 5;
    const uint32_t group = blockIdx.x, token = blockIdx.y;
    const uint32_t flat = group * group_size + lid;
    const bool active = flat < element_count;
    const float value = active ? __half2float(source[(size_t)token * source_stride + flat]) : 0.f;
    float lo = active ? value : INFINITY, hi = active ? value : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) { mins[warp] = lo; maxs[warp] = hi; }
    __syncthreads();
    const float levels = bits == 4u ? 15.f : 255.f;
    if (lid == 0) {
        const uint32_t warps = (blockDim.x + 31) / 32;
        float mn = mins[0], mx = maxs[0];
        for (uint32_t w = 1; w < warps; ++w) { mn = fminf(mn, mins[w]); mx = fmaxf(mx, maxs[w]); }
        s_bias = mn;
        s_scale = mx > mn ? (mx - mn) / levels : 0.f;
        unsigned char *row = destination + (size_t)token * destination_stride;
        const uint32_t groups = (element_count + group_size - 1) / group_size;
        __half *scales = reinterpret_cast<__half *>(row + values_bytes);
        scales[group] = __float2half_rn(s_scale);
        scales[groups + group] = __float2half_rn(s_bias);
    }
    __syncthreads();
    const float scale = s_scale, bias = s_bias;
    unsigned char *row = destination + (size_t)token * destination_stride;
    const float q = scale > 0.f ? roundf(fminf(fmaxf((value - bias) / scale, 0.f), levels)) : 0.f;
    if (bits == 8u) {
        if (active) row[flat] = (unsigned char)q;
    } else {
        // two codes per byte: the even element in the low nibble
        const float other = __shfl_down_sync(0xffffffffu, q, 1);
        if ((lid & 1u) == 0u && active) {
            const unsigned char low = (unsigned char)q;
            const unsigned char high = (flat + 1u < element_count) ? (unsigned char)other : 0;
            row[flat / 2u] = low | (unsigned char)(high << 4);
        }
    }
}

}  // namespace

TT_API int tt_kv_quantize_affine(tt_context *ctx, tt_stream stream, const void *source, void *destination,
                                 uint32_t source_stride_elements, uint32_t destination_stride_bytes,
                                 uint32_t values_bytes, uint32_t element_count, uint32_t bits, uint32_t group_size,
                                 uint32_t tokens) {
    TT_ENTER(ctx);
    if (source == nullptr || destination == nullptr || element_count == 0 || tokens == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "quantise needs non-null buffers and positive sizes");
    if (bits != 8 && bits != 4) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "KV bits must be 4 or 8");
    if (group_size == 0 || group_size % 32 != 0 || group_size > 1024)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "group size must be a multiple of 32 up to 1024");
    const uint32_t groups = (element_count + group_size - 1) / group_size;
    if (source_stride_elements < element_count || values_bytes < (element_count * bits + 7) / 8 ||
        destination_stride_bytes < values_bytes + groups * 4 || (values_bytes & 1) || (destination_stride_bytes & 1))
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "row strides too small for the quantised layout");
    kv_quantize_affine_kernel<<<dim3(groups, tokens), group_size, 0, (cudaStream_t)stream>>>(
        (const __half *)source, (unsigned char *)destination, source_stride_elements, destination_stride_bytes,
        values_bytes, element_count, bits, group_size);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "kv_quantize_affine launch");
    ctx->launches++;
    return TT_OK;
}
