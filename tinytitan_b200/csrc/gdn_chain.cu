// The elementwise kernels around the delta rule in a Gated-DeltaNet layer: causal depthwise
// conv + SiLU (decode and prefill), conv-tail update / checkpoint, per-head q/k RMS norm with the
// folded delta-rule scales, and the gated output norm.
//
// Replaces gdn_conv_mix_decode / gdn_conv_mix_prefill / gdn_conv_tail_update /
// gdn_conv_tail_checkpoint / gdn_qk_norm / gdn_gated_norm
// (sources/TinyTitanCore/Metal/GDN/gdn.metal:330-521, :678-727) and their wrappers
// GDN.encodeConvDecode / encodeConvPrefill / encodeConvTailUpdate / encodeConvTailCheckpoint /
// encodeQKNorm / encodeGatedNorm (sources/TinyTitan/Kernels/GDN/GDN.swift:185-313, :399-427).
// All of them are small and HBM/launch bound; each reads its inputs once with 16-bit vector
// loads where alignment allows and keeps the reference's fp32 arithmetic and fp16 rounding points.
#include "tt_common.h"

namespace {

constexpr float kRmsEps = 1e-6f;   // kGdnRmsEps (gdn.metal:35)

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }

// conv over [tail rows | chunk rows], one thread per (channel, row). update_tail != 0 is the
// decode form: rows must be 1 and the tail is shifted in place by the same thread afterwards
// (each thread owns its channel column).
__global__ void gdn_conv_mix_kernel(__half *tail, const __half *qkv, const __nv_bfloat16 *conv_w, __half *out,
                                    uint32_t channels, uint32_t taps, uint32_t rows, int update_tail) {
    const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t t = blockIdx.y;
    if (ch >= channels || t >= rows) return;
    const int history = (int)taps - 1;
    float acc;
    if (update_tail) {
        // decode arithmetic order of gdn_conv_mix_decode: current row first, then the tail rows
        acc = __half2float(qkv[ch]) * __bfloat162float(conv_w[(size_t)ch * taps + (taps - 1)]);
        for (int j = 0; j < history; ++j)
            acc = fmaf(__half2float(tail[(size_t)j * channels + ch]), __bfloat162float(conv_w[(size_t)ch * taps + j]), acc);
    } else {
        acc = 0.f;
        for (int j = 0; j < (int)taps; ++j) {
            const int src = (int)t + j - history;
            const float value = src >= 0 ? __half2float(qkv[(size_t)src * channels + ch])
                                         : __half2float(tail[(size_t)(history + src) * channels + ch]);
            acc = fmaf(value, __bfloat162float(conv_w[(size_t)ch * taps + j]), acc);
        }
    }
    out[(size_t)t * channels + ch] = __float2half_rn(silu(acc));
    if (update_tail) {
        for (int j = 0; j + 1 < history; ++j) tail[(size_t)j * channels + ch] = tail[(size_t)(j + 1) * channels + ch];
        if (history > 0) tail[(size_t)(history - 1) * channels + ch] = qkv[ch];
    }
}

// tail := last K-1 raw rows of [old tail | chunk]; one thread per channel does the ordered shift
// (the reference splits this over threads only when rows >= K-1; per-channel is always safe).
__global__ void gdn_conv_tail_update_kernel(__half *tail, const __half *qkv, uint32_t channels, uint32_t taps,
                                            uint32_t rows) {
    const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= channels) return;
    const int history = (int)taps - 1;
    for (int row = 0; row < history; ++row) {
        const int src = (int)rows + row - history;
        const __half value = src >= 0 ? qkv[(size_t)src * channels + ch] : tail[(size_t)(history + src) * channels + ch];
        tail[(size_t)row * channels + ch] = value;   // src row index (history+src) > row: read-before-write is safe
    }
}

// checkpoint := last K-1 rows of [tail | qkv row 0]
__global__ void gdn_conv_tail_checkpoint_kernel(const __half *tail, const __half *qkv, __half *checkpoint,
                                                uint32_t channels, uint32_t taps) {
    const uint32_t history = taps - 1;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= history * channels) return;
    const uint32_t row = idx / channels, ch = idx - row * channels;
    checkpoint[idx] = (row + 1 < history) ? tail[(size_t)(row + 1) * channels + ch] : qkv[ch];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// one warp per (q-or-k head, row): x * rsqrt(mean(x^2) + eps) * (q: 1/Dk, k: 1/sqrt(Dk)), in place
__global__ void gdn_qk_norm_kernel(__half *conv_out, uint32_t hk, uint32_t dk, uint32_t row_stride, uint32_t rows) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t head_index = warp % (2 * hk), row = warp / (2 * hk);
    if (row >= rows) return;
    const bool is_q = head_index < hk;
    const uint32_t head = is_q ? head_index : head_index - hk;
    __half *x = conv_out + (size_t)row * row_stride + (is_q ? 0u : hk * dk) + (size_t)head * dk;
    float sumsq = 0.f;
    for (uint32_t i = lane; i < dk; i += 32) { const float v = __half2float(x[i]); sumsq = fmaf(v, v, sumsq); }
    sumsq = warp_sum(sumsq);
    const float inv_rms = rsqrtf(sumsq / (float)dk + kRmsEps);
    const float scale = is_q ? 1.f / (float)dk : rsqrtf((float)dk);
    for (uint32_t i = lane; i < dk; i += 32) x[i] = __float2half_rn(__half2float(x[i]) * inv_rms * scale);
}

// one warp per (value head, row): rmsnorm(y) * weight * gate(z)
__global__ void gdn_gated_norm_kernel(const __half *y, const __half *z, const __nv_bfloat16 *weight, __half *out,
                                      uint32_t hv, uint32_t dv, uint32_t rows, int sigmoid_gate) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t head = warp % hv, row = warp / hv;
    if (row >= rows) return;
    const size_t base = (size_t)row * hv * dv + (size_t)head * dv;
    float sumsq = 0.f;
    for (uint32_t i = lane; i < dv; i += 32) { const float v = __half2float(y[base + i]); sumsq = fmaf(v, v, sumsq); }
    sumsq = warp_sum(sumsq);
    const float inv_rms = rsqrtf(sumsq / (float)dv + kRmsEps);
    for (uint32_t i = lane; i < dv; i += 32) {
        const float normed = __half2float(y[base + i]) * inv_rms * __bfloat162float(weight[i]);
        const float zz = __half2float(z[base + i]);
        const float gate = sigmoid_gate ? 1.f / (1.f + expf(-zz)) : silu(zz);
        out[base + i] = __float2half_rn(normed * gate);
    }
}

// The decode-step prologue of a Gated-DeltaNet layer in ONE launch for a whole batch of sessions:
// causal conv + SiLU of the new qkv row with the in-place tail shift (gdn_conv_mix_decode), and the
// q/k head norm with the folded scales (gdn_qk_norm). One warp per (session, Dk-wide channel group):
// the q and k groups are heads and get the norm, the v groups only the conv. The conv output is
// rounded to fp16 before the norm reads it, exactly as the separate kernels store and re-load it,
// so the result is bit-identical to tt_gdn_conv_mix(update_tail = 1) followed by tt_gdn_qk_norm.
constexpr uint32_t kPreSessions = 64;
struct GdnPreTable {
    struct Entry { __half *tail; const __half *qkv; __half *conv_out; } s[kPreSessions];
};
__global__ void __launch_bounds__(128)
gdn_decode_pre_kernel(const __grid_constant__ GdnPreTable table, const __nv_bfloat16 *__restrict__ conv_w, uint32_t channels,
                      uint32_t taps, uint32_t hk, uint32_t dk, uint32_t n_sessions) {
    const uint32_t groups = (channels + dk - 1) / dk;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t z = warp / groups, grp = warp % groups;
    if (z >= n_sessions) return;
    __half *tail = table.s[z].tail;
    const __half *qkv = table.s[z].qkv;
    __half *out = table.s[z].conv_out;
    const int history = (int)taps - 1;
    const bool is_head = grp < 2 * hk;                   // q heads, then k heads, then the value channels
    float sumsq = 0.f;
    constexpr int kMaxPerLane = 8;                       // dk <= 256
    float vals[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const uint32_t ch = grp * dk + lane + 32 * i;
        vals[i] = 0.f;
        if (lane + 32 * i >= dk || ch >= channels) continue;
        // decode arithmetic order of gdn_conv_mix_decode: current row first, then the tail rows
        float acc = __half2float(qkv[ch]) * __bfloat162float(conv_w[(size_t)ch * taps + (taps - 1)]);
        for (int j = 0; j < history; ++j)
            acc = fmaf(__half2float(tail[(size_t)j * channels + ch]), __bfloat162float(conv_w[(size_t)ch * taps + j]), acc);
        const __half rounded = __float2half_rn(silu(acc));
        for (int j = 0; j + 1 < history; ++j) tail[(size_t)j * channels + ch] = tail[(size_t)(j + 1) * channels + ch];
        if (history > 0) tail[(size_t)(history - 1) * channels + ch] = qkv[ch];
        if (!is_head) { out[ch] = rounded; continue; }
        vals[i] = __half2float(rounded);
        sumsq = fmaf(vals[i], vals[i], sumsq);
    }
    if (!is_head) return;
    // summation order of gdn_qk_norm_kernel: lane-strided partial sums, then the xor tree
    sumsq = warp_sum(sumsq);
    const float inv_rms = rsqrtf(sumsq / (float)dk + kRmsEps);
    const float scale = grp < hk ? 1.f / (float)dk : rsqrtf((float)dk);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const uint32_t ch = grp * dk + lane + 32 * i;
        if (lane + 32 * i < dk && ch < channels) out[ch] = __float2half_rn(vals[i] * inv_rms * scale);
    }
}

int finish(tt_context *ctx, const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, what);
    ctx->launches++;
    return TT_OK;
}

}  // namespace

TT_API int tt_gdn_conv_mix(tt_context *ctx, tt_stream stream, void *tail, const void *qkv, const void *conv_weight,
                           void *out, uint32_t channels, uint32_t taps, uint32_t rows, int update_tail) {
    TT_ENTER(ctx);
    if (tail == nullptr || qkv == nullptr || conv_weight == nullptr || out == nullptr || channels == 0 || taps == 0 || rows == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "conv mix needs non-null buffers and positive sizes");
    if (update_tail && rows != 1)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "the in-place tail shift is the one-row (decode) form");
    const dim3 grid((channels + 255) / 256, rows);
    gdn_conv_mix_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__half *)tail, (const __half *)qkv,
                                                               (const __nv_bfloat16 *)conv_weight, (__half *)out,
                                                               channels, taps, rows, update_tail);
    return finish(ctx, "gdn_conv_mix launch");
}

TT_API int tt_gdn_decode_pre(tt_context *ctx, tt_stream stream, const tt_gdn_pre_session *sessions, uint32_t n_sessions,
                             const void *conv_weight, uint32_t n_k_heads, uint32_t key_dim, uint32_t channels, uint32_t taps) {
    TT_ENTER(ctx);
    if (sessions == nullptr || conv_weight == nullptr || n_k_heads == 0 || key_dim == 0 || channels == 0 || taps == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "decode prologue needs non-null buffers and positive sizes");
    if (key_dim > 256 || channels < 2 * n_k_heads * key_dim || (channels - 2 * n_k_heads * key_dim) % key_dim != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE,
                            "decode prologue: key_dim <= 256 and a value width that is a multiple of key_dim");
    const uint32_t groups = channels / key_dim;
    for (uint32_t base = 0; base < n_sessions; base += kPreSessions) {
        const uint32_t n = n_sessions - base < kPreSessions ? n_sessions - base : kPreSessions;
        static thread_local GdnPreTable table;
        for (uint32_t i = 0; i < n; ++i) {
            const tt_gdn_pre_session &s = sessions[base + i];
            if (s.tail == nullptr || s.qkv == nullptr || s.conv_out == nullptr)
                return tt_set_error(ctx, TT_ERR_INVALID_ARG, "session %u has a null buffer", base + i);
            table.s[i].tail = (__half *)s.tail; table.s[i].qkv = (const __half *)s.qkv; table.s[i].conv_out = (__half *)s.conv_out;
        }
        const uint32_t warps = n * groups;
        cudaError_t e = tt_launch_pdl(gdn_decode_pre_kernel, dim3((warps + 3) / 4), dim3(128), 0, (cudaStream_t)stream, table,
                                      (const __nv_bfloat16 *)conv_weight, channels, taps, n_k_heads, key_dim, n);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_decode_pre launch");
        ctx->launches++;
    }
    return TT_OK;
}

TT_API int tt_gdn_conv_tail_update(tt_context *ctx, tt_stream stream, void *tail, const void *qkv, uint32_t channels,
                                   uint32_t taps, uint32_t rows) {
    TT_ENTER(ctx);
    if (tail == nullptr || qkv == nullptr || channels == 0 || taps == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "tail update needs non-null buffers and positive sizes");
    if (taps == 1 || rows == 0) return TT_OK;
    gdn_conv_tail_update_kernel<<<(channels + 255) / 256, 256, 0, (cudaStream_t)stream>>>((__half *)tail, (const __half *)qkv,
                                                                                         channels, taps, rows);
    return finish(ctx, "gdn_conv_tail_update launch");
}

TT_API int tt_gdn_conv_tail_checkpoint(tt_context *ctx, tt_stream stream, const void *tail, const void *qkv,
                                       void *checkpoint, uint32_t channels, uint32_t taps) {
    TT_ENTER(ctx);
    if (tail == nullptr || qkv == nullptr || checkpoint == nullptr || channels == 0 || taps == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "tail checkpoint needs non-null buffers and positive sizes");
    if (taps == 1) return TT_OK;
    const uint32_t total = (taps - 1) * channels;
    gdn_conv_tail_checkpoint_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        (const __half *)tail, (const __half *)qkv, (__half *)checkpoint, channels, taps);
    return finish(ctx, "gdn_conv_tail_checkpoint launch");
}

TT_API int tt_gdn_qk_norm(tt_context *ctx, tt_stream stream, void *conv_out, uint32_t n_k_heads, uint32_t key_dim,
                          uint32_t row_stride, uint32_t rows) {
    TT_ENTER(ctx);
    if (conv_out == nullptr || n_k_heads == 0 || key_dim == 0 || rows == 0 || row_stride < 2 * n_k_heads * key_dim)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "qk norm needs a buffer, positive sizes and row_stride >= 2*Hk*Dk");
    const uint64_t warps = (uint64_t)2 * n_k_heads * rows;
    gdn_qk_norm_kernel<<<(uint32_t)((warps + 3) / 4), 128, 0, (cudaStream_t)stream>>>((__half *)conv_out, n_k_heads, key_dim,
                                                                                     row_stride, rows);
    return finish(ctx, "gdn_qk_norm launch");
}

TT_API int tt_gdn_gated_norm(tt_context *ctx, tt_stream stream, const void *y, const void *z, const void *weight,
                             void *out, uint32_t n_v_heads, uint32_t value_dim, uint32_t rows, int sigmoid_gate) {
    TT_ENTER(ctx);
    if (y == nullptr || z == nullptr || weight == nullptr || out == nullptr || n_v_heads == 0 || value_dim == 0 || rows == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "gated norm needs non-null buffers and positive sizes");
    const uint64_t warps = (uint64_t)n_v_heads * rows;
    gdn_gated_norm_kernel<<<(uint32_t)((warps + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
        (const __half *)y, (const __half *)z, (const __nv_bfloat16 *)weight, (__half *)out, n_v_heads, value_dim, rows,
        sigmoid_gate);
    return finish(ctx, "gdn_gated_norm launch");
}
