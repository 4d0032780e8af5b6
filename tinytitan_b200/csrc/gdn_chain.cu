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

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int kMaxTaps = 8;
constexpr int kConvRowBlock = 16;      // rows a warp walks with its sliding window
constexpr int kConvWarps = 4;

// Element i of lane `lane` inside a group of `width` channels that a warp owns: contiguous chunks of
// width/32 channels per lane when the width is a multiple of 32 (vector loads), else lane-strided.
// The q/k norm sums a lane's elements in this order and then over the lanes with the xor tree, in
// every kernel that computes it, so fused and separate launches agree bit for bit.
__device__ __forceinline__ uint32_t lane_elem(uint32_t width, uint32_t lane, uint32_t i) {
    return (width & 31u) == 0 ? lane * (width >> 5) + i : lane + 32u * i;
}

template <int CPL>
__device__ __forceinline__ void load_halves(const __half *p, float (&v)[CPL]) {
    if constexpr (CPL == 1) {
        v[0] = __half2float(p[0]);
    } else if constexpr (CPL == 2) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(p));
        v[0] = f.x; v[1] = f.y;
    } else {
        static_assert(CPL == 4 || CPL == 8, "lane chunk");
        uint32_t w[CPL / 2];
        if constexpr (CPL == 4) { const uint2 r = *reinterpret_cast<const uint2 *>(p); w[0] = r.x; w[1] = r.y; }
        else { const uint4 r = *reinterpret_cast<const uint4 *>(p); w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w; }
#pragma unroll
        for (int i = 0; i < CPL / 2; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
}
template <int CPL>
__device__ __forceinline__ void store_halves(__half *p, const __half (&h)[CPL]) {
    if constexpr (CPL == 1) p[0] = h[0];
    else if constexpr (CPL == 2) *reinterpret_cast<__half2 *>(p) = __halves2half2(h[0], h[1]);
    else if constexpr (CPL == 4) *reinterpret_cast<uint2 *>(p) = *reinterpret_cast<const uint2 *>(h);
    else *reinterpret_cast<uint4 *>(p) = *reinterpret_cast<const uint4 *>(h);
}

struct ConvParams {
    __half *tail;                 // [taps-1][channels]
    const __half *qkv;            // [rows][channels]
    const __nv_bfloat16 *conv_w;  // [channels][taps]
    __half *out;                  // [rows][channels]
    __half *checkpoint;           // nullable: the tail as it stands after row 0 alone
    uint32_t channels, taps, rows;
    uint32_t norm_heads;          // 2 * Hk when the q/k norm is fused (the groups below that index are heads), else 0
    uint32_t group;               // channels per warp: Dk when the norm is fused, else 32 * CPL
    int decode_order;             // the one-row decode form: current row first, then the tail rows
    int update_tail;              // tail := last taps-1 raw rows of [old tail | rows]
};

// Causal depthwise conv + SiLU over [tail | rows] with a sliding window in registers: a warp owns
// `group` channels (CPL contiguous ones per lane, one vector load per row) and walks kConvRowBlock
// rows, so every input element is loaded once instead of once per tap; the q/k head norm
// (gdn_qk_norm) is applied on the way out when the group is a head, and the warp of the first row
// block, the only one that reads the tail, also writes the checkpoint and the new tail when asked
// to. grid = (channel groups, row blocks / kConvWarps), block = kConvWarps warps.
template <int CPL>
__global__ void __launch_bounds__(kConvWarps * 32) gdn_conv_rows_kernel(ConvParams p) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t grp = blockIdx.x;
    const uint32_t block = blockIdx.y * kConvWarps + warp;
    const uint32_t r0 = block * kConvRowBlock;
    if (r0 >= p.rows) return;
    const uint32_t ch0 = grp * p.group + lane * CPL;
    if (lane * CPL >= p.group || ch0 >= p.channels) return;       // a partial last group (never a head)
    const int taps = (int)p.taps, history = taps - 1;
    const bool is_head = grp < p.norm_heads;

    // taps 0..history-1 weigh the window rows, the last one the current row
    float w[CPL][kMaxTaps - 1], w_last[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
#pragma unroll
        for (int j = 0; j < kMaxTaps - 1; ++j)
            w[c][j] = j < history ? __bfloat162float(p.conv_w[(size_t)(ch0 + c) * taps + j]) : 0.f;
        w_last[c] = __bfloat162float(p.conv_w[(size_t)(ch0 + c) * taps + history]);
    }

    // window[j] = raw row (r - history + j) of this lane's channels, j < history; rows before the chunk come from the tail
    float win[kMaxTaps - 1][CPL];
#pragma unroll
    for (int j = 0; j < kMaxTaps - 1; ++j) {
        if (j < history) {
            const int src = (int)r0 - history + j;
            const __half *row = src >= 0 ? p.qkv + (size_t)src * p.channels : p.tail + (size_t)(history + src) * p.channels;
            load_halves<CPL>(row + ch0, win[j]);
        }
    }
    const uint32_t r1 = min(p.rows, r0 + kConvRowBlock);
    const float norm_scale = grp < p.norm_heads / 2 ? 1.f / (float)p.group : rsqrtf((float)p.group);
    for (uint32_t r = r0; r < r1; ++r) {
        float x[CPL];
        load_halves<CPL>(p.qkv + (size_t)r * p.channels + ch0, x);
        __half rounded[CPL];
        float sumsq = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            float acc;
            if (p.decode_order) {
                acc = x[c] * w_last[c];
#pragma unroll
                for (int j = 0; j < kMaxTaps - 1; ++j)
                    if (j < history) acc = fmaf(win[j][c], w[c][j], acc);
            } else {
                acc = 0.f;
#pragma unroll
                for (int j = 0; j < kMaxTaps - 1; ++j)
                    if (j < history) acc = fmaf(win[j][c], w[c][j], acc);
                acc = fmaf(x[c], w_last[c], acc);
            }
            rounded[c] = __float2half_rn(silu(acc));
            const float v = __half2float(rounded[c]);
            sumsq = fmaf(v, v, sumsq);
        }
        if (is_head) {
            // the conv output is rounded to fp16 before the norm reads it, as the separate kernels store and re-load it
            sumsq = warp_sum(sumsq);
            const float inv_rms = rsqrtf(sumsq / (float)p.group + kRmsEps);
#pragma unroll
            for (int c = 0; c < CPL; ++c) rounded[c] = __float2half_rn(__half2float(rounded[c]) * inv_rms * norm_scale);
        }
        store_halves<CPL>(p.out + (size_t)r * p.channels + ch0, rounded);
        if (r == 0 && p.checkpoint != nullptr) {
            // the last taps-1 rows of [tail | row 0]
#pragma unroll
            for (int j = 0; j < kMaxTaps - 1; ++j) {
                if (j < history) {
                    __half h[CPL];
#pragma unroll
                    for (int c = 0; c < CPL; ++c)
                        h[c] = __float2half_rn(j + 1 < history ? win[j + 1 < kMaxTaps - 1 ? j + 1 : j][c] : x[c]);
                    store_halves<CPL>(p.checkpoint + (size_t)j * p.channels + ch0, h);
                }
            }
        }
        // slide the window: slot j takes slot j + 1, the last slot in use takes the current row (slots beyond
        // the history are never read)
#pragma unroll
        for (int j = 0; j < kMaxTaps - 1; ++j) {
#pragma unroll
            for (int c = 0; c < CPL; ++c)
                win[j][c] = j + 1 < history ? win[j + 1 < kMaxTaps - 1 ? j + 1 : j][c] : x[c];
        }
    }
    if (p.update_tail && block == 0) {
        // new tail = the last taps-1 raw rows of [old tail | rows]; this warp has read the old tail (nobody
        // else does), so writing it now races with nothing
        for (int j = 0; j < history; ++j) {
            const int src = (int)p.rows - history + j;        // row of the chunk, negative: row of the old tail
            float v[CPL];
            if (src >= (int)r0 - history && src < (int)r1) {
                // inside this warp's window (the whole chunk when it is one row block)
#pragma unroll
                for (int c = 0; c < CPL; ++c) v[c] = 0.f;
                const int k = src - ((int)r1 - history);       // window slot after the walk above
#pragma unroll
                for (int jj = 0; jj < kMaxTaps - 1; ++jj)
                    if (jj == k) {
#pragma unroll
                        for (int c = 0; c < CPL; ++c) v[c] = win[jj][c];
                    }
            } else {
                load_halves<CPL>(p.qkv + (size_t)src * p.channels + ch0, v);   // src >= r1 > 0: a later row of the chunk
            }
            __half h[CPL];
#pragma unroll
            for (int c = 0; c < CPL; ++c) h[c] = __float2half_rn(v[c]);
            store_halves<CPL>(p.tail + (size_t)j * p.channels + ch0, h);
        }
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

// one warp per (q-or-k head, row): x * rsqrt(mean(x^2) + eps) * (q: 1/Dk, k: 1/sqrt(Dk)), in place
__global__ void gdn_qk_norm_kernel(__half *conv_out, uint32_t hk, uint32_t dk, uint32_t row_stride, uint32_t rows) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t head_index = warp % (2 * hk), row = warp / (2 * hk);
    if (row >= rows) return;
    const bool is_q = head_index < hk;
    const uint32_t head = is_q ? head_index : head_index - hk;
    __half *x = conv_out + (size_t)row * row_stride + (is_q ? 0u : hk * dk) + (size_t)head * dk;
    const uint32_t per_lane = (dk + 31) / 32;
    float sumsq = 0.f;
    for (uint32_t k = 0; k < per_lane; ++k) {
        const uint32_t i = lane_elem(dk, lane, k);
        if (i < dk) { const float v = __half2float(x[i]); sumsq = fmaf(v, v, sumsq); }
    }
    sumsq = warp_sum(sumsq);
    const float inv_rms = rsqrtf(sumsq / (float)dk + kRmsEps);
    const float scale = is_q ? 1.f / (float)dk : rsqrtf((float)dk);
    for (uint32_t k = 0; k < per_lane; ++k) {
        const uint32_t i = lane_elem(dk, lane, k);
        if (i < dk) x[i] = __float2half_rn(__half2float(x[i]) * inv_rms * scale);
    }
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
        const uint32_t e = lane_elem(dk, lane, i), ch = grp * dk + e;
        vals[i] = 0.f;
        if ((uint32_t)i >= (dk + 31) / 32 || e >= dk || ch >= channels) continue;
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
    // summation order of gdn_qk_norm_kernel: a lane's elements in lane_elem order, then the xor tree
    sumsq = warp_sum(sumsq);
    const float inv_rms = rsqrtf(sumsq / (float)dk + kRmsEps);
    const float scale = grp < hk ? 1.f / (float)dk : rsqrtf((float)dk);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const uint32_t e = lane_elem(dk, lane, i), ch = grp * dk + e;
        if ((uint32_t)i < (dk + 31) / 32 && e < dk && ch < channels) out[ch] = __float2half_rn(vals[i] * inv_rms * scale);
    }
}

int finish(tt_context *ctx, const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, what);
    ctx->launches++;
    return TT_OK;
}

}  // namespace

// Launches gdn_conv_rows_kernel with the widest lane chunk the shapes and addresses allow.
static int launch_conv_rows(tt_context *ctx, cudaStream_t stream, ConvParams p, uint32_t key_dim) {
    if (p.taps > (uint32_t)kMaxTaps)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "conv kernel sizes up to %d are supported, got %u", kMaxTaps, p.taps);
    uint32_t cpl;
    if (p.norm_heads != 0) {
        cpl = key_dim / 32;                       // one head per warp
        p.group = key_dim;
    } else {
        cpl = 8;
        while (cpl > 1 && p.channels % cpl != 0) cpl /= 2;
        p.group = 32 * cpl;
    }
    const uintptr_t addrs = (uintptr_t)p.tail | (uintptr_t)p.qkv | (uintptr_t)p.out | (uintptr_t)p.checkpoint;
    if ((addrs & (2 * cpl - 1)) != 0 || p.channels % cpl != 0) {
        if (p.norm_heads != 0)
            return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "fused q/k norm: buffers must be aligned to %u bytes", 2 * cpl);
        cpl = 1; p.group = 32;
    }
    const uint32_t blocks = (p.rows + kConvRowBlock - 1) / kConvRowBlock;
    const dim3 grid((p.channels + p.group - 1) / p.group, (blocks + kConvWarps - 1) / kConvWarps);
    cudaError_t e;
    switch (cpl) {
        case 8: e = tt_launch_pdl(gdn_conv_rows_kernel<8>, grid, dim3(kConvWarps * 32), 0, stream, p); break;
        case 4: e = tt_launch_pdl(gdn_conv_rows_kernel<4>, grid, dim3(kConvWarps * 32), 0, stream, p); break;
        case 2: e = tt_launch_pdl(gdn_conv_rows_kernel<2>, grid, dim3(kConvWarps * 32), 0, stream, p); break;
        default: e = tt_launch_pdl(gdn_conv_rows_kernel<1>, grid, dim3(kConvWarps * 32), 0, stream, p); break;
    }
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_conv_rows launch");
    return finish(ctx, "gdn_conv_rows launch");
}

TT_API int tt_gdn_conv_mix(tt_context *ctx, tt_stream stream, void *tail, const void *qkv, const void *conv_weight,
                           void *out, uint32_t channels, uint32_t taps, uint32_t rows, int update_tail) {
    TT_ENTER(ctx);
    if (tail == nullptr || qkv == nullptr || conv_weight == nullptr || out == nullptr || channels == 0 || taps == 0 || rows == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "conv mix needs non-null buffers and positive sizes");
    if (update_tail && rows != 1)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "the in-place tail shift is the one-row (decode) form");
    ConvParams p = {};
    p.tail = (__half *)tail; p.qkv = (const __half *)qkv; p.conv_w = (const __nv_bfloat16 *)conv_weight; p.out = (__half *)out;
    p.channels = channels; p.taps = taps; p.rows = rows;
    p.decode_order = update_tail ? 1 : 0; p.update_tail = update_tail ? 1 : 0;
    return launch_conv_rows(ctx, (cudaStream_t)stream, p, 0);
}

TT_API int tt_gdn_prefill_pre(tt_context *ctx, tt_stream stream, void *tail, const void *qkv, const void *conv_weight,
                              void *conv_out, void *checkpoint_tail, uint32_t n_k_heads, uint32_t key_dim, uint32_t channels,
                              uint32_t taps, uint32_t rows, int update_tail) {
    TT_ENTER(ctx);
    if (tail == nullptr || qkv == nullptr || conv_weight == nullptr || conv_out == nullptr || channels == 0 || taps == 0 ||
        rows == 0 || n_k_heads == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "prefill prologue needs non-null buffers and positive sizes");
    if ((key_dim != 32 && key_dim != 64 && key_dim != 128 && key_dim != 256) || channels < 2 * n_k_heads * key_dim ||
        channels % key_dim != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE,
                            "prefill prologue: key_dim 32, 64, 128 or 256 and a channel count that is a multiple of it");
    ConvParams p = {};
    p.tail = (__half *)tail; p.qkv = (const __half *)qkv; p.conv_w = (const __nv_bfloat16 *)conv_weight;
    p.out = (__half *)conv_out; p.checkpoint = (__half *)checkpoint_tail;
    p.channels = channels; p.taps = taps; p.rows = rows;
    p.norm_heads = 2 * n_k_heads; p.decode_order = 0; p.update_tail = update_tail ? 1 : 0;
    return launch_conv_rows(ctx, (cudaStream_t)stream, p, key_dim);
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
