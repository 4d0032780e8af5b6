// Gated delta rule, token-ordered: decode step (rows == 1) and the exact sequential
// multi-row form (verify rows / sequential prefill), batched over independent sessions.
//
// Replaces gdn_delta_step_decode and gdn_delta_step_prefill
// (sources/TinyTitanCore/Metal/GDN/gdn.metal:529-669) and their host wrappers
// GDN.encodeDeltaStepDecode / encodeDeltaStepPrefill
// (sources/TinyTitan/Kernels/GDN/GDN.swift:318-396).
//
// HBM-bound design: the fp32 state [Hv][Dv][Dk] is read once and written once per call
// whatever the number of rows. A warp owns 8 state rows at a time in registers: 8 lanes share two
// rows, so the two dot products of a token (S.k and S.q) are 3 shuffles each, and the state never
// leaves registers between tokens. The kernel is persistent: each warp walks a list of 8-row
// items, the rows arrive through a per-warp ring of bulk copies (three items ahead), and the next
// token's inputs are fetched while the current one is applied.
#include "tt_sm100.h"

#include <algorithm>
#include <type_traits>

namespace {

constexpr int kRowsPerWarp = 8;
constexpr int kWarps = 4;
constexpr uint32_t kSlots = 2;        // state items in flight per warp
constexpr uint32_t kTokDepth = 8;     // (item, token) pairs whose inputs are requested ahead
constexpr uint32_t kSmemSessions = 64, kSmemHeads = 128;   // tables staged in shared memory up to these sizes
constexpr int kCtasPerSm = 4;

struct GdnParams {
    const tt_gdn_session *sessions;
    const __nv_bfloat16 *a_log;
    const __nv_bfloat16 *dt_bias;
    uint32_t hk, hv, dk, dv, rows, row_stride, flags;
    uint32_t shift_blocks, shift_heads;   // log2 of dv/8 and of hv when both are powers of two, else 0xff
    float readout_scale;
};

// The two dot products a lane takes part in (its rows A and B) summed over the 8 lanes that share
// the rows, in 3 shuffles: the lanes first swap the half they do not keep, then butterfly over the
// remaining four. Lanes 0-3 of the group end with row A's total, lanes 4-7 with row B's.
__device__ __forceinline__ float group_sum2(float a, float b, bool upper) {
    const float send = upper ? a : b, keep = upper ? b : a;
    float c = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

__device__ __forceinline__ float4 ld_f4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st_f4(float *p, const float4 &v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ float4 half4_to_float4(const uint2 &raw) {
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void scale4(float4 &s, float2 gg) {
    const float2 lo = mul2(make_float2(s.x, s.y), gg), hi = mul2(make_float2(s.z, s.w), gg);
    s = make_float4(lo.x, lo.y, hi.x, hi.y);
}
// s += k * d (d broadcast in both halves of dd)
__device__ __forceinline__ void axpy4(float4 &s, const float4 &k, float2 dd) {
    const float2 lo = fma2(make_float2(k.x, k.y), dd, make_float2(s.x, s.y));
    const float2 hi = fma2(make_float2(k.z, k.w), dd, make_float2(s.z, s.w));
    s = make_float4(lo.x, lo.y, hi.x, hi.y);
}
// two partial sums per dot product (even and odd elements); the caller adds them
__device__ __forceinline__ float2 dot4(const float4 &s, const float4 &k, float2 acc) {
    acc = fma2(make_float2(s.x, s.y), make_float2(k.x, k.y), acc);
    return fma2(make_float2(s.z, s.w), make_float2(k.z, k.w), acc);
}

// exp(x) in about 8 instructions, ~2 ulp: the product x*log2(e) is carried as hi + lo so that
// the only error left is that of ex2.approx (2^-22 relative); libm's expf costs three times as
// much and this kernel is bound by instruction issue once several tokens share a state read.
__device__ __forceinline__ float exp_2ulp(float x) {
    constexpr float kL2eHi = 1.4426950408889634f, kL2eLo = 1.92596299112661746e-8f;
    const float hi = x * kL2eHi;
    float lo = fmaf(x, kL2eHi, -hi);
    lo = fmaf(x, kL2eLo, lo);
    const float r = fast_exp2(hi);
    return fmaf(r, lo * 0.6931471805599453f, r);
}
// softplus(x) = log(1 + exp(x)), evaluated like the reference (gdn.metal:134-157: the sum is
// formed in fp32 first), with lg2.approx (2^-22 absolute in log2 units on (0.5, 2), relative beyond).
__device__ __forceinline__ float softplus_fast(float x) {
    if (x > 20.f) return x;
    return __log2f(1.f + exp_2ulp(x)) * 0.6931471805599453f;
}

__device__ __forceinline__ void cp_async8(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Persistent, warp-granular pipeline. A work item is 8 consecutive state rows of one (session,
// head): 8*Dk*4 contiguous bytes. Warp w of CTA c takes items (iter*gridDim.x + c)*4 + w, so the four
// warps of a CTA stream adjacent pieces. Every warp owns two rings in shared memory:
//   * state ring, kSlots items: lane 0 fills a slot with one bulk copy (completion on the slot's
//     mbarrier); a slot is free again as soon as its rows sit in registers, so kSlots items are in
//     flight while one more is applied;
//   * token ring, kTokDepth (item, token) pairs ahead: each pair's q, k and v pieces arrive by
//     8-byte cp.async, its two gate scalars as the aligned 4-byte words that contain them (a
//     register destination would make every later read of that register wait for the load).
// Token inputs are requested kTokDepth tokens before they are used because under a saturated
// memory system one token of arithmetic (a few hundred cycles) hides nothing of a load.
// The warps never synchronise with each other after the tables below are staged.
//
// Register layout: the 8 lanes of group g = lane/8 share rows 2g and 2g+1; lane l of the group owns
// the 16-byte column chunks l, l+8, l+16, ... of both rows (Dk/8 floats per row), so a row's dot
// product is 3 shuffles away and shared-memory / global accesses of a group are 128 contiguous bytes.
//
// grid = min(ceil(items / 4), kCtasPerSm * SMs), block = 128.
// Up to kSmemSessions sessions travel in the kernel parameters (n != 0), so a batched step uploads
// no table; larger batches read the table the host copied to device memory.
struct GdnSessionTable {
    tt_gdn_session s[kSmemSessions];
    uint32_t n;
};

template <int DK>
__global__ void __launch_bounds__(kWarps * 32, kCtasPerSm)
gdn_step_kernel(GdnParams p, uint32_t n_sessions, uint32_t n_items, uint32_t *__restrict__ status,
                const __grid_constant__ GdnSessionTable ptab) {
    constexpr int C = DK / 32;                       // 16-byte chunks per lane per row
    constexpr uint32_t kItemFloats = kRowsPerWarp * DK;
    constexpr uint32_t kItemBytes = kItemFloats * 4;
    constexpr uint32_t kTokHalves = 2 * DK + kRowsPerWarp + 4;   // q | k | v of the 8 rows | a word | b word
    constexpr uint32_t kWarpBytes = kSlots * kItemBytes + kTokDepth * kTokHalves * 2;
    extern __shared__ __align__(128) unsigned char gdn_smem[];
    __shared__ uint64_t bars_all[kWarps][kSlots];
    __shared__ tt_gdn_session ses_tab[kSmemSessions];
    __shared__ float2 head_tab[kSmemHeads];          // (decay coefficient, dt_bias) per value head

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int l = lane & 7;
    const bool upper = (lane & 4) != 0;
    const uint32_t row_a = (lane >> 3) * 2;          // this lane's rows inside the item: row_a, row_a + 1
    float *ring = reinterpret_cast<float *>(gdn_smem + (size_t)warp * kWarpBytes);
    __half *tok_ring = reinterpret_cast<__half *>(gdn_smem + (size_t)warp * kWarpBytes + kSlots * kItemBytes);
    uint64_t *bars = bars_all[warp];
    const uint32_t blocks_per_head = p.dv / kRowsPerWarp;
    const uint32_t stride = gridDim.x * kWarps;
    const uint32_t first = blockIdx.x * kWarps + warp;
    const bool f32_gates = (p.flags & TT_GDN_GATES_F32) != 0;
    const uint32_t gate_bytes = f32_gates ? 4 : 2;

    // session table and per-head decay parameters: staged once so that the item loop never waits
    // on a dependent global load for a pointer
    const bool tab_in_smem = n_sessions <= kSmemSessions;
    const bool heads_in_smem = !f32_gates && p.hv <= kSmemHeads;
    auto head_params = [&](uint32_t h) {
        float a = __bfloat162float(p.a_log[h]);
        if (!(p.flags & TT_GDN_A_LOG_PREEXP)) a = -expf(a);
        return make_float2(a, __bfloat162float(p.dt_bias[h]));
    };
    const tt_gdn_session *src_tab = ptab.n != 0 ? ptab.s : p.sessions;
    const tt_gdn_session *tab = src_tab;      // switched to the staged copy once it is complete

    // item -> (session, head, first row)
    struct Where { uint32_t z, h, dv0; };
    auto where = [&](uint32_t item) {
        Where w;
        if (p.shift_blocks != 0xffu) {      // both divisors are powers of two (the usual shapes)
            const uint32_t hb = item >> p.shift_blocks;
            w.dv0 = (item & (blocks_per_head - 1)) * kRowsPerWarp;
            w.z = hb >> p.shift_heads;
            w.h = hb & (p.hv - 1);
        } else {
            const uint32_t hb = item / blocks_per_head;
            w.dv0 = (item - hb * blocks_per_head) * kRowsPerWarp;
            w.z = hb / p.hv;
            w.h = hb - w.z * p.hv;
        }
        return w;
    };
    auto issue = [&](uint32_t item, uint32_t slot) {      // lane 0 only
        const Where w = where(item);
        const float *src = tab[w.z].state + ((size_t)w.h * p.dv + w.dv0) * DK;
        mbar_expect_tx(&bars[slot], kItemBytes);
        bulk_copy_g2s(ring + slot * kItemFloats, src, kItemBytes, &bars[slot]);
    };

    // the first state copies leave before anything else; the tables are staged while they fly
    pdl_launch_dependents();
    if (lane == 0) {
        for (uint32_t s = 0; s < kSlots; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    pdl_wait();     // the kernel before this one in the stream (it may have written state or inputs) is complete
    if (lane == 0) {
        for (uint32_t s = 0; s < kSlots; ++s)
            if (first + s * stride < n_items) issue(first + s * stride, s);
    }
    if (tab_in_smem)
        for (uint32_t i = threadIdx.x; i < n_sessions; i += blockDim.x) ses_tab[i] = src_tab[i];
    if (heads_in_smem)
        for (uint32_t h = threadIdx.x; h < p.hv; h += blockDim.x) head_tab[h] = head_params(h);
    __syncthreads();
    if (tab_in_smem) tab = ses_tab;

    // ---- token prefetch cursor: walks the (item, token) pairs kTokDepth ahead of the consumer
    struct Cursor {
        uint32_t item, t;
        const __half *q;       // q piece base of token 0: conv_out + hk*DK
        const __half *v;       // v base of token 0 for this item's rows
        const char *a, *b;     // gate scalars of token 0 for this item's head
    } pf;
    auto cursor_set = [&](uint32_t item) {
        pf.item = item; pf.t = 0;
        if (item >= n_items) return;
        const Where w = where(item);
        const uint32_t hk = (p.flags & TT_GDN_V_TILED) ? w.h % p.hk : w.h / (p.hv / p.hk);
        const tt_gdn_session &ses = tab[w.z];
        const __half *conv = reinterpret_cast<const __half *>(ses.conv_out);
        pf.q = conv + (size_t)hk * DK;
        pf.v = conv + (size_t)2 * p.hk * DK + (size_t)w.h * p.dv + w.dv0;
        pf.a = reinterpret_cast<const char *>(ses.a) + (size_t)w.h * gate_bytes;
        pf.b = reinterpret_cast<const char *>(ses.b) + (size_t)w.h * gate_bytes;
    };
    auto prefetch = [&](uint32_t pair) {
        if (pf.item < n_items) {
            __half *entry = tok_ring + (pair % kTokDepth) * kTokHalves;
            const size_t row = (size_t)pf.t * p.row_stride;
            const __half *qk = pf.q + row;
#pragma unroll
            for (int piece = lane; piece < DK / 2; piece += 32) {
                // pieces [0, DK/4) are q, [DK/4, DK/2) are k (which sits hk_count*DK after q)
                const __half *src = qk + 4 * piece + (4 * piece < DK ? 0 : (size_t)p.hk * DK - DK);
                cp_async8(entry + 4 * piece, src);
            }
            if (lane < 2) cp_async8(entry + 2 * DK + 4 * lane, pf.v + row + 4 * lane);
            if (lane == 2 || lane == 3) {
                // the aligned word holding the scalar: it shares the scalar's page, so the two
                // neighbouring bytes of a 16-bit gate are always readable
                const char *g = (lane == 2 ? pf.a : pf.b) + (size_t)pf.t * p.hv * gate_bytes;
                cp_async4(entry + 2 * DK + kRowsPerWarp + 2 * (lane - 2),
                          reinterpret_cast<const char *>(reinterpret_cast<uintptr_t>(g) & ~(uintptr_t)3));
            }
            if (++pf.t == p.rows) cursor_set(pf.item + stride);
        }
        cp_async_commit();   // one group per pair, empty or not, so the wait below counts pairs
    };

    cursor_set(first);
    for (uint32_t j = 0; j < kTokDepth; ++j) prefetch(j);

    bool timed_out = false;
    uint32_t iter = 0, pair = 0;
    for (uint32_t item = first; item < n_items; item += stride, ++iter) {
        const uint32_t slot = iter % kSlots;
        const Where w = where(item);
        const tt_gdn_session ses = tab[w.z];
        float2 hp = make_float2(0.f, 0.f);
        if (!f32_gates) hp = heads_in_smem ? head_tab[w.h] : head_params(w.h);
        if (!warp_all(mbar_wait(&bars[slot], (iter / kSlots) & 1))) { timed_out = true; break; }

        float4 sa[C], sb[C];
        {
            const float *src = ring + slot * kItemFloats + row_a * DK + 4 * l;
#pragma unroll
            for (int j = 0; j < C; ++j) { sa[j] = ld_f4(src + 32 * j); sb[j] = ld_f4(src + DK + 32 * j); }
        }
        __syncwarp();   // every lane holds its part of the slot: it may be refilled
        const uint32_t refill = item + kSlots * stride;
        if (lane == 0 && refill < n_items) issue(refill, slot);

        const size_t lane_off = ((size_t)w.h * p.dv + w.dv0 + row_a) * DK + 4 * l;

        // Gates of a short multi-row item (2..4 tokens, the verify step): lane t evaluates token t's pair once
        // and the warp reads it back with two shuffles per token, instead of every lane evaluating the two
        // exponentials and the logarithm of every token. The item's tokens were all requested at least
        // kTokDepth - 4 tokens ago.
        const bool lane_gates = !f32_gates && p.rows > 1 && p.rows <= 4;
        float g_lane = 1.f, beta_lane = 0.f;
        auto gate_pair = [&](const __half *entry, uint32_t t, float &g, float &beta) {
            const uint2 gw = *reinterpret_cast<const uint2 *>(entry + 2 * DK + kRowsPerWarp);
            const size_t gi = ((size_t)t * p.hv + w.h) * 2;
            const uint32_t sh_a = ((reinterpret_cast<uintptr_t>(ses.a) + gi) & 2) * 8;
            const uint32_t sh_b = ((reinterpret_cast<uintptr_t>(ses.b) + gi) & 2) * 8;
            const float raw_a = __half2float(__ushort_as_half((unsigned short)(gw.x >> sh_a)));
            const float raw_b = __half2float(__ushort_as_half((unsigned short)(gw.y >> sh_b)));
            g = exp_2ulp(hp.x * softplus_fast(raw_a + hp.y));
            beta = __frcp_rn(1.f + exp_2ulp(-raw_b));
        };
        if (lane_gates) {
            cp_async_wait<kTokDepth - 4>();
            __syncwarp();
            const uint32_t t = (uint32_t)lane < p.rows ? lane : 0;
            gate_pair(tok_ring + ((pair + t) % kTokDepth) * kTokHalves, t, g_lane, beta_lane);
        }

        // one token applied to the 8 rows in registers
        auto apply_token = [&](const __half *entry, uint32_t t, float g, float beta) {
            const float2 vv = __half22float2(*reinterpret_cast<const __half2 *>(entry + 2 * DK + row_a));
            const __half *qs = entry + 4 * l, *ks = entry + DK + 4 * l;

            // decay, then S.k for both rows
            float4 k4[C];
            float2 ka2 = make_float2(0.f, 0.f), kb2 = make_float2(0.f, 0.f);
            const float2 gg = make_float2(g, g);
#pragma unroll
            for (int j = 0; j < C; ++j) {
                k4[j] = half4_to_float4(*reinterpret_cast<const uint2 *>(ks + 32 * j));
                scale4(sa[j], gg);
                scale4(sb[j], gg);
                ka2 = dot4(sa[j], k4[j], ka2);
                kb2 = dot4(sb[j], k4[j], kb2);
            }
            const float mine = group_sum2(ka2.x + ka2.y, kb2.x + kb2.y, upper);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 4);
            const float da = (vv.x - (upper ? other : mine)) * beta;
            const float db = (vv.y - (upper ? mine : other)) * beta;

            // rank-one update, then the readout S.q
            float2 ya2 = make_float2(0.f, 0.f), yb2 = make_float2(0.f, 0.f);
            const float2 dda = make_float2(da, da), ddb = make_float2(db, db);
#pragma unroll
            for (int j = 0; j < C; ++j) {
                const float4 q4 = half4_to_float4(*reinterpret_cast<const uint2 *>(qs + 32 * j));
                axpy4(sa[j], k4[j], dda);
                axpy4(sb[j], k4[j], ddb);
                ya2 = dot4(sa[j], q4, ya2);
                yb2 = dot4(sb[j], q4, yb2);
            }
            const float y_mine = group_sum2(ya2.x + ya2.y, yb2.x + yb2.y, upper);
            if ((lane & 3) == 0) {     // lane 0 of the group holds row A's readout, lane 4 row B's
                __half *y = reinterpret_cast<__half *>(ses.y) + (size_t)t * p.hv * p.dv + (size_t)w.h * p.dv;
                y[w.dv0 + row_a + (upper ? 1 : 0)] = __float2half_rn(y_mine * p.readout_scale);
            }
            if (t == 0 && ses.checkpoint_state != nullptr) {
                float *ck = ses.checkpoint_state + lane_off;
#pragma unroll
                for (int j = 0; j < C; ++j) { st_f4(ck + 32 * j, sa[j]); st_f4(ck + DK + 32 * j, sb[j]); }
            }
        };

        if (lane_gates) {
            // all tokens of the item in one unrolled block: the loads and conversions of a token's q and k
            // are independent of the state, so the compiler moves them under the shuffle reductions of the
            // token before (with one token per loop trip every warp sat through each reduction idle)
            auto block = [&](auto n_const) {
                constexpr uint32_t N = decltype(n_const)::value;
#pragma unroll
                for (uint32_t t = 0; t < N; ++t) {
                    const float g = __shfl_sync(0xffffffffu, g_lane, t), beta = __shfl_sync(0xffffffffu, beta_lane, t);
                    apply_token(tok_ring + ((pair + t) % kTokDepth) * kTokHalves, t, g, beta);
                }
                __syncwarp();                   // every lane has read the entries: they may be refilled
#pragma unroll
                for (uint32_t t = 0; t < N; ++t) prefetch(pair + kTokDepth + t);
                pair += N;
            };
            if (p.rows == 4) block(std::integral_constant<uint32_t, 4>{});
            else if (p.rows == 3) block(std::integral_constant<uint32_t, 3>{});
            else block(std::integral_constant<uint32_t, 2>{});
        } else {
            for (uint32_t t = 0; t < p.rows; ++t, ++pair) {
                cp_async_wait<kTokDepth - 1>();   // this lane's pieces of `pair` have landed ...
                __syncwarp();                     // ... and so have everyone else's
                const __half *entry = tok_ring + (pair % kTokDepth) * kTokHalves;
                float g, beta;
                if (f32_gates) {
                    const uint2 gw = *reinterpret_cast<const uint2 *>(entry + 2 * DK + kRowsPerWarp);
                    g = __uint_as_float(gw.x); beta = __uint_as_float(gw.y);
                } else {
                    gate_pair(entry, t, g, beta);
                }
                apply_token(entry, t, g, beta);
                __syncwarp();                       // every lane has read the entry: it may be refilled
                prefetch(pair + kTokDepth);
            }
        }

        float *dst = ses.state + lane_off;
#pragma unroll
        for (int j = 0; j < C; ++j) { st_f4(dst + 32 * j, sa[j]); st_f4(dst + DK + 32 * j, sb[j]); }
    }

    cp_async_wait<0>();
    if (timed_out) {
        // leave the state of the unprocessed items untouched; give the copies still in flight a
        // bounded chance to land before the shared memory is released
        if (lane == 0) {
            atomicOr(status, TT_DEV_WAIT_TIMEOUT);
            for (uint32_t k = 0; k < kSlots; ++k) {
                const uint32_t it = iter + k;
                if (first + (size_t)it * stride < n_items) mbar_wait(&bars[it % kSlots], (it / kSlots) & 1, 1u << 16);
            }
        }
        __syncwarp();
    }
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
    cudaError_t e = cudaSuccess;
    static thread_local GdnSessionTable ptab;
    ptab.n = 0;
    if (n <= kSmemSessions) {
        memcpy(ptab.s, h_sessions, sizeof(tt_gdn_session) * n);
        ptab.n = n;
    } else {
        e = cudaMemcpyAsync(ctx->gdn_sessions, h_sessions, sizeof(tt_gdn_session) * n, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "copy gdn session table");
    }
    GdnParams p;
    p.sessions = reinterpret_cast<const tt_gdn_session *>(ctx->gdn_sessions);
    // with fp32 gates the decay parameters are unused; point them at the session table so the
    // two scalar loads stay in bounds
    p.a_log = reinterpret_cast<const __nv_bfloat16 *>(f32_gates && !a_log ? ctx->gdn_sessions : a_log);
    p.dt_bias = reinterpret_cast<const __nv_bfloat16 *>(f32_gates && !dt_bias ? ctx->gdn_sessions : dt_bias);
    p.hk = shape->n_k_heads; p.hv = shape->n_v_heads; p.dk = shape->key_dim; p.dv = shape->value_dim;
    p.rows = rows; p.row_stride = row_stride; p.flags = shape->flags; p.readout_scale = shape->readout_scale;
    {
        const uint32_t nb = shape->value_dim / kRowsPerWarp, nh = shape->n_v_heads;
        const bool pow2 = (nb & (nb - 1)) == 0 && (nh & (nh - 1)) == 0;
        p.shift_blocks = pow2 ? (uint32_t)__builtin_ctz(nb) : 0xffu;
        p.shift_heads = pow2 ? (uint32_t)__builtin_ctz(nh) : 0xffu;
    }
    const uint32_t n_items = n * shape->n_v_heads * (shape->value_dim / kRowsPerWarp);
    const uint32_t grid = std::min((n_items + kWarps - 1) / kWarps, (uint32_t)(kCtasPerSm * ctx->sm_count));
    const size_t smem = (size_t)kWarps * (kSlots * kRowsPerWarp * shape->key_dim * sizeof(float) +
                                          kTokDepth * (2 * shape->key_dim + kRowsPerWarp + 4) * sizeof(__half));
    TTLaunchTimer timer(ctx, stream, TT_PROFILE_GDN_STEP);
    auto launch = [&](auto kernel) {
        cudaError_t le = tt_set_smem_once(kernel, (int)smem);
        if (le != cudaSuccess) return le;
        return tt_launch_pdl(kernel, dim3(grid), dim3(kWarps * 32), smem, stream, p, n, n_items, ctx->status, ptab);
    };
    switch (shape->key_dim) {
        case 128: e = launch(gdn_step_kernel<128>); break;
        case 64: e = launch(gdn_step_kernel<64>); break;
        default: e = launch(gdn_step_kernel<32>); break;
    }
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_step shared memory attribute");
    e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_step launch");
    timer.stop();
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
