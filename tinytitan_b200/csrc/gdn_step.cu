// Gated delta rule, token-ordered: decode step (rows == 1) and the exact sequential
// multi-row form (verify rows / sequential prefill), batched over independent sessions.
//
// Replaces gdn_delta_step_decode and gdn_delta_step_prefill
// (sources/TinyTitanCore/Metal/GDN/gdn.metal:529-669) and their host wrappers
// GDN.encodeDeltaStepDecode / encodeDeltaStepPrefill
// (sources/TinyTitan/Kernels/GDN/GDN.swift:318-396).
//
// HBM-bound design: the fp32 state [Hv][Dv][Dk] is read once and written once per call
// whatever the number of rows. A CTA owns 32 state rows of one (session, head); each of its 4
// warps holds 8 rows in registers (a lane owns Dk/32 consecutive floats of each row), so the
// eight 16-byte loads of a lane are in flight together. Per token the two dot products of the
// eight rows (S.k and S.q) are reduced together with a 9-shuffle transposing butterfly; the state
// never leaves registers between tokens, and the next token's inputs are fetched while the
// current one is applied.
#include "tt_common.h"

namespace {

constexpr int kRowsPerWarp = 8;
constexpr int kWarps = 4;
constexpr int kRowsPerCta = kRowsPerWarp * kWarps;

struct GdnParams {
    const tt_gdn_session *sessions;
    const __nv_bfloat16 *a_log;
    const __nv_bfloat16 *dt_bias;
    uint32_t hk, hv, dk, dv, rows, row_stride, flags;
    float readout_scale;
};

// Sums of 8 per-lane values over the warp in 9 shuffles instead of 40: at each of the first three
// butterfly steps a lane hands the half of its values the partner keeps and adds the half it keeps,
// then the single remaining value is summed over the last four lanes. Lane L ends with the total
// of value index 4*bit4(L) + 2*bit3(L) + bit2(L), i.e. index r is held by lanes 4r..4r+3.
__device__ __forceinline__ float warp_sum8(const float (&v)[8], int lane) {
    float a[4], b[2];
    bool up = (lane & 16) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = up ? v[i] : v[i + 4], keep = up ? v[i + 4] : v[i];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    up = (lane & 8) != 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = up ? a[i] : a[i + 2], keep = up ? a[i + 2] : a[i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    up = (lane & 4) != 0;
    const float send = up ? b[0] : b[1], keep = up ? b[1] : b[0];
    float c = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

template <int NPL>
__device__ __forceinline__ void load_vec(float (&dst)[NPL], const float *src) {
    if constexpr (NPL == 4) {
        const float4 t = *reinterpret_cast<const float4 *>(src);
        dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
    } else if constexpr (NPL == 2) {
        const float2 t = *reinterpret_cast<const float2 *>(src);
        dst[0] = t.x; dst[1] = t.y;
    } else {
        dst[0] = *src;
    }
}

template <int NPL>
__device__ __forceinline__ void store_vec(float *dst, const float (&src)[NPL]) {
    if constexpr (NPL == 4) {
        *reinterpret_cast<float4 *>(dst) = make_float4(src[0], src[1], src[2], src[3]);
    } else if constexpr (NPL == 2) {
        *reinterpret_cast<float2 *>(dst) = make_float2(src[0], src[1]);
    } else {
        *dst = src[0];
    }
}

template <int NPL>
__device__ __forceinline__ void load_half_vec(float (&dst)[NPL], const __half *src) {
    if constexpr (NPL == 4) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(src);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
        dst[0] = lo.x; dst[1] = lo.y; dst[2] = hi.x; dst[3] = hi.y;
    } else if constexpr (NPL == 2) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(src));
        dst[0] = t.x; dst[1] = t.y;
    } else {
        dst[0] = __half2float(*src);
    }
}

// grid = (dv blocks, Hv, sessions), block = 128.
template <int NPL>
__global__ void __launch_bounds__(kWarps * 32) gdn_step_kernel(GdnParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t h = blockIdx.y;
    const tt_gdn_session ses = p.sessions[blockIdx.z];
    const uint32_t dv0 = blockIdx.x * kRowsPerCta + warp * kRowsPerWarp;
    const uint32_t hk = (p.flags & TT_GDN_V_TILED) ? h % p.hk : h / (p.hv / p.hk);
    const uint32_t col = lane * NPL;

    float *state = ses.state + ((size_t)h * p.dv) * p.dk;
    float s[kRowsPerWarp][NPL];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        if (dv0 + r < p.dv) {
            load_vec<NPL>(s[r], state + (size_t)(dv0 + r) * p.dk + col);
        } else {
#pragma unroll
            for (int i = 0; i < NPL; ++i) s[r][i] = 0.f;
        }
    }

    const float a_param = __bfloat162float(p.a_log[h]);
    const float dtb = __bfloat162float(p.dt_bias[h]);
    const bool rows_valid = dv0 < p.dv;   // value_dim is a multiple of 8: a warp's 8 rows are all in or all out

    // One token's inputs; the next token's are fetched while the current one is being applied,
    // so the multi-row form does not pay a global-load latency per token.
    struct Tok { float q[NPL], k[NPL], v[kRowsPerWarp], g, beta; };
    auto load_tok = [&](uint32_t t, Tok &tok) {
        const __half *row = reinterpret_cast<const __half *>(ses.conv_out) + (size_t)t * p.row_stride;
        load_half_vec<NPL>(tok.q, row + (size_t)hk * p.dk + col);
        load_half_vec<NPL>(tok.k, row + (size_t)p.hk * p.dk + (size_t)hk * p.dk + col);
        const __half *vrow = row + (size_t)2 * p.hk * p.dk + (size_t)h * p.dv;
        if (rows_valid) {
            const uint2 lo = *reinterpret_cast<const uint2 *>(vrow + dv0);
            const uint2 hi = *reinterpret_cast<const uint2 *>(vrow + dv0 + 4);
            const float2 v0 = __half22float2(*reinterpret_cast<const __half2 *>(&lo.x));
            const float2 v1 = __half22float2(*reinterpret_cast<const __half2 *>(&lo.y));
            const float2 v2 = __half22float2(*reinterpret_cast<const __half2 *>(&hi.x));
            const float2 v3 = __half22float2(*reinterpret_cast<const __half2 *>(&hi.y));
            tok.v[0] = v0.x; tok.v[1] = v0.y; tok.v[2] = v1.x; tok.v[3] = v1.y;
            tok.v[4] = v2.x; tok.v[5] = v2.y; tok.v[6] = v3.x; tok.v[7] = v3.y;
        } else {
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) tok.v[r] = 0.f;
        }
        if (p.flags & TT_GDN_GATES_F32) {
            tok.g = reinterpret_cast<const float *>(ses.a)[(size_t)t * p.hv + h];
            tok.beta = reinterpret_cast<const float *>(ses.b)[(size_t)t * p.hv + h];
        } else {
            const float av = __half2float(reinterpret_cast<const __half *>(ses.a)[(size_t)t * p.hv + h]);
            const float bv = __half2float(reinterpret_cast<const __half *>(ses.b)[(size_t)t * p.hv + h]);
            const float x = av + dtb;
            const float sp = x > 20.f ? x : logf(1.f + expf(x));
            tok.g = (p.flags & TT_GDN_A_LOG_PREEXP) ? expf(a_param * sp) : expf(-expf(a_param) * sp);
            tok.beta = 1.f / (1.f + expf(-bv));
        }
    };

    Tok cur;
    load_tok(0, cur);
    for (uint32_t t = 0; t < p.rows; ++t) {
        Tok nxt = cur;
        if (t + 1 < p.rows) load_tok(t + 1, nxt);
        float q[NPL], k[NPL];
#pragma unroll
        for (int i = 0; i < NPL; ++i) { q[i] = cur.q[i]; k[i] = cur.k[i]; }
        const float g = cur.g, beta = cur.beta;

        float kv[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                s[r][i] *= g;
                acc = fmaf(s[r][i], k[i], acc);
            }
            kv[r] = acc;
        }
        {   // all eight S.k sums, then every lane fetches the eight totals (row r sits in lane 4r)
            const float mine = warp_sum8(kv, lane);
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) kv[r] = __shfl_sync(0xffffffffu, mine, r << 2);
        }

        float out[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const float vv = cur.v[r];
            const float delta = (vv - kv[r]) * beta;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                s[r][i] = fmaf(k[i], delta, s[r][i]);
                acc = fmaf(s[r][i], q[i], acc);
            }
            out[r] = acc;
        }
        // S.q sums: lane 4r holds row r's readout and stores it
        const float mine = warp_sum8(out, lane);
        if ((lane & 3) == 0 && rows_valid) {
            __half *y = reinterpret_cast<__half *>(ses.y) + (size_t)t * p.hv * p.dv + (size_t)h * p.dv;
            y[dv0 + (lane >> 2)] = __float2half_rn(mine * p.readout_scale);
        }

        if (t == 0 && ses.checkpoint_state != nullptr) {
            float *ck = ses.checkpoint_state + ((size_t)h * p.dv) * p.dk;
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r)
                if (dv0 + r < p.dv) store_vec<NPL>(ck + (size_t)(dv0 + r) * p.dk + col, s[r]);
        }
        cur = nxt;
    }

#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
        if (dv0 + r < p.dv) store_vec<NPL>(state + (size_t)(dv0 + r) * p.dk + col, s[r]);
}

int validate_shape(tt_context *ctx, const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride) {
    if (shape == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "shape must not be null");
    if (shape->n_k_heads == 0 || shape->n_v_heads == 0 || shape->n_v_heads % shape->n_k_heads != 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_v_heads must be a positive multiple of n_k_heads");
    if (shape->key_dim != 32 && shape->key_dim != 64 && shape->key_dim != 128)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "key_dim must be 32, 64 or 128, got %u", shape->key_dim);
    if (shape->value_dim == 0 || shape->value_dim % 8 != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "value_dim must be a multiple of 8");
    if (rows == 0) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "rows must be positive");
    const uint32_t tight = 2 * shape->n_k_heads * shape->key_dim + shape->n_v_heads * shape->value_dim;
    if (row_stride < tight)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "row_stride %u is smaller than the qkv width %u", row_stride, tight);
    if (row_stride % 4 != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "row_stride must be a multiple of 4 elements");
    return TT_OK;
}

int launch_step(tt_context *ctx, cudaStream_t stream, const tt_gdn_session *h_sessions, uint32_t n,
                const void *a_log, const void *dt_bias, const tt_gdn_shape *shape, uint32_t rows,
                uint32_t row_stride) {
    int rc = validate_shape(ctx, shape, rows, row_stride);
    if (rc != TT_OK) return rc;
    if (n == 0) return TT_OK;
    if (n > ctx->max_sessions)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_sessions %u exceeds the context's max_sessions %u", n,
                            ctx->max_sessions);
    const bool f32_gates = (shape->flags & TT_GDN_GATES_F32) != 0;
    if (!f32_gates && (a_log == nullptr || dt_bias == nullptr))
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "a_log and dt_bias must not be null");
    for (uint32_t i = 0; i < n; ++i) {
        const tt_gdn_session &s = h_sessions[i];
        if (!s.conv_out || !s.a || !s.b || !s.state || !s.y)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "session %u has a null buffer", i);
        if (((uintptr_t)s.conv_out & 7) || ((uintptr_t)s.state & 15) || ((uintptr_t)s.checkpoint_state & 15))
            return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "session %u: misaligned buffer", i);
    }
    cudaError_t e = cudaMemcpyAsync(ctx->gdn_sessions, h_sessions, sizeof(tt_gdn_session) * n,
                                    cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "copy gdn session table");
    GdnParams p;
    p.sessions = reinterpret_cast<const tt_gdn_session *>(ctx->gdn_sessions);
    // with fp32 gates the decay parameters are unused; point them at the session table so the
    // two scalar loads stay in bounds
    p.a_log = reinterpret_cast<const __nv_bfloat16 *>(f32_gates && !a_log ? ctx->gdn_sessions : a_log);
    p.dt_bias = reinterpret_cast<const __nv_bfloat16 *>(f32_gates && !dt_bias ? ctx->gdn_sessions : dt_bias);
    p.hk = shape->n_k_heads; p.hv = shape->n_v_heads; p.dk = shape->key_dim; p.dv = shape->value_dim;
    p.rows = rows; p.row_stride = row_stride; p.flags = shape->flags; p.readout_scale = shape->readout_scale;
    const dim3 grid((shape->value_dim + kRowsPerCta - 1) / kRowsPerCta, shape->n_v_heads, n);
    switch (shape->key_dim) {
        case 128: gdn_step_kernel<4><<<grid, kWarps * 32, 0, stream>>>(p); break;
        case 64: gdn_step_kernel<2><<<grid, kWarps * 32, 0, stream>>>(p); break;
        default: gdn_step_kernel<1><<<grid, kWarps * 32, 0, stream>>>(p); break;
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_step launch");
    ctx->launches++;
    return TT_OK;
}

}  // namespace

TT_API int tt_gdn_step(tt_context *ctx, tt_stream stream, const void *conv_out, const void *a, const void *b,
                       const void *a_log, const void *dt_bias, float *state, void *y, const tt_gdn_shape *shape,
                       uint32_t rows, uint32_t row_stride, float *checkpoint_state) {
    TT_ENTER(ctx);
    tt_gdn_session s;
    s.conv_out = conv_out; s.a = a; s.b = b; s.state = state; s.y = y; s.checkpoint_state = checkpoint_state;
    return launch_step(ctx, (cudaStream_t)stream, &s, 1, a_log, dt_bias, shape, rows, row_stride);
}

TT_API int tt_gdn_step_batched(tt_context *ctx, tt_stream stream, const tt_gdn_session *sessions,
                               uint32_t n_sessions, const void *a_log, const void *dt_bias,
                               const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride) {
    TT_ENTER(ctx);
    if (sessions == nullptr && n_sessions != 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "sessions must not be null");
    return launch_step(ctx, (cudaStream_t)stream, sessions, n_sessions, a_log, dt_bias, shape, rows, row_stride);
}
