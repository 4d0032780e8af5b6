// Chunk-parallel Gated-DeltaNet prefill scan (chunk = 64 tokens, Dk = Dv = 128).
//
// The recurrence of gdn_delta_step_prefill (sources/TinyTitanCore/Metal/GDN/gdn.metal:590-669)
// evaluated chunk by chunk, following the algebra of tinytitan_delta_rule_chunk
// (sources/TinyTitanKernelsC/gdn_chunk.c:72-195, benchmark/gdn_chunked_scan.py:70-97):
//
//   S_t = a_t S_{t-1} + c_t k_t^T,  c_t = b_t (v_t - a_t S_{t-1} k_t),  o_t = S_t q_t
//
// With A_t = prod_{i<=t} a_i inside a chunk and S_0 the state entering it, the corrections of
// the whole chunk solve (I + L) C = diag(b) (V - diag(A) K S_0^T), L[t,s] = b_t (A_t/A_s)(k_t.k_s)
// for s < t. Writing T = (I + L)^-1:
//
//   C = U - W S_0^T           U = T diag(b) V,  W = T diag(b A) K       (state independent)
//   O = diag(A) Q S_0^T + M C     M[t,s] = (A_t/A_s)(q_t.k_s), s <= t   (state independent)
//   S_C = A_C S_0 + (diag(A_C/A_s) C)^T K
//
// Decay ratios are exp(logA_t - logA_s) of cumulative log-decays (never A_t / A_s, cf.
// gdn_chunk.c:141-147). Two kernels per segment of chunks:
//   gdn_scan_prepare_kernel   one CTA per (chunk, value head), fully parallel: tiles by TMA, Gram
//                             matrices on mma.sync, T by forward substitution in fp32, U (fp32), W, M
//                             (fp16); U and W leave through TMA tensor stores
//   gdn_scan_state_tc_kernel  one CTA per (32 state rows, value head), chunks in order, on tcgen05:
//                             the fp32 state lives transposed in tensor memory for the whole segment
//   gdn_scan_state_kernel     the same recurrence on mma.sync (state in accumulator registers), kept
//                             as the A/B partner selected by TT_GDN_SCAN_FORCE_MMA_SYNC=1
// The rows of S (value dimension) are independent of one another, which is what lets the state
// be split over CTAs with no communication.
#include "tt_sm100.h"

#include <cstdlib>

namespace {

constexpr int kC = 64;          // tokens per chunk
constexpr int kD = 128;         // Dk == Dv
constexpr int kPitch = kD + 8;  // fp16 row pitch of [*][128] tiles (272 B: ldmatrix conflict-free)
constexpr int kDvb = 32;        // state rows per CTA of the state kernel
constexpr int kStateThreads = 256;   // 8 warps: (token tile / column group) x (half of the state rows)

// Per (chunk, value head) record in the workspace.
struct ChunkRecord {
    float u[kC][kD];        // U, fp32 (enters C by a plain subtraction, so it keeps full precision)
    __half w[kC][kD];       // W
    __half m[kC][kC];       // M (lower triangle incl. diagonal, zeros above)
    float decay_a[kC];      // A_t
    float decay_w[kC];      // A_C / A_t
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// ldmatrix addressing helpers for a row-major fp16 tile with `pitch` elements per row.
// A operand (16 rows x 16 k) at (row0, k0); B operand for two n-tiles from a [n][k] tile
// (k contiguous) at (n0, k0); transposed variants read [k][n] tiles (n contiguous).
__device__ __forceinline__ uint32_t addr_b(uint32_t base, int pitch, int n0, int k0, int lane) {
    return base + ((n0 + (lane & 7) + ((lane >> 4) << 3)) * pitch + k0 + ((lane >> 3) & 1) * 8) * 2;
}
__device__ __forceinline__ uint32_t addr_bt(uint32_t base, int pitch, int k0, int n0, int lane) {
    return base + ((k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + n0 + (lane >> 4) * 8) * 2;
}
// A operand (16 m x 16 k) read from a [k][m] tile (m contiguous) with .trans:
// matrices: (k 0-7, m 0-7) -> a0, (k 0-7, m 8-15) -> a1, (k 8-15, m 0-7) -> a2, (k 8-15, m 8-15) -> a3
__device__ __forceinline__ uint32_t addr_at(uint32_t base, int pitch, int k0, int m0, int lane) {
    return base + ((k0 + (lane & 7) + (lane >> 4) * 8) * pitch + m0 + ((lane >> 3) & 1) * 8) * 2;
}

// Operand tiles that arrive by TMA use the 128-byte swizzle: a [64 tokens][128] fp16 tile is two boxes
// of [64][64] (8 KB each), the 16-byte piece c of row r sitting at (c ^ (r & 7)) << 4 within the row.
// Address of the 16-byte piece holding column `col` (a multiple of 8) of row `row` in a swizzled tile.
__device__ __forceinline__ uint32_t sw_piece(uint32_t base, int row, int col) {
    return base + ((col >> 6) << 13) + (row << 7) + ((((col >> 3) & 7) ^ (row & 7)) << 4);
}
// ldmatrix row addresses on swizzled tiles, lane roles as in addr_a / addr_b / addr_bt
__device__ __forceinline__ uint32_t sw_a(uint32_t base, int row0, int k0, int lane) {
    return sw_piece(base, row0 + (lane & 15), k0 + (lane >> 4) * 8);
}
__device__ __forceinline__ uint32_t sw_b(uint32_t base, int n0, int k0, int lane) {
    return sw_piece(base, n0 + (lane & 7) + ((lane >> 4) << 3), k0 + ((lane >> 3) & 1) * 8);
}
// A operand (16 m x 16 k) read with .trans from a swizzled [k][m] tile (m contiguous), lane roles as in addr_at
__device__ __forceinline__ uint32_t sw_at(uint32_t base, int k0, int m0, int lane) {
    return sw_piece(base, k0 + (lane & 7) + (lane >> 4) * 8, m0 + ((lane >> 3) & 1) * 8);
}
__device__ __forceinline__ uint32_t sw_bt(uint32_t base, int k0, int n0, int lane) {
    return sw_piece(base, k0 + (lane & 7) + ((lane >> 3) & 1) * 8, n0 + (lane >> 4) * 8);
}

// Records seen as 2-D tensors: a record is 226 rows of 256 bytes (W), 452 rows of 128 bytes (M) or
// 113 rows of 512 bytes (U), so one map per field covers the whole workspace.
static_assert(sizeof(ChunkRecord) % 512 == 0, "record rows");
constexpr uint32_t kRecRowsW = sizeof(ChunkRecord) / 256, kRecRowsM = sizeof(ChunkRecord) / 128,
                   kRecRowsU = sizeof(ChunkRecord) / 512;

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, const void *src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(smem_u32(src))
                 : "memory");
}
// Ends the group of stores issued so far and waits until their sources have been read (the writes
// themselves are complete by the end of the grid).
__device__ __forceinline__ void bulk_commit_and_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

struct ScanParams {
    const __half *conv_out;
    const void *a;
    const void *b;
    const __nv_bfloat16 *a_log;
    const __nv_bfloat16 *dt_bias;
    float *state;
    __half *y;
    ChunkRecord *records;     // [chunks in segment][Hv]
    uint32_t hk, hv, rows, row_stride, flags;
    uint32_t token0;          // first token of the segment
    uint32_t n_chunks;        // chunks in the segment
    float readout_scale;
    uint32_t *status;         // device status word of the context
};

// ---------------------------------------------------------------------------------------
// Phase 1: state-independent quantities of one chunk of one value head.
// grid = (chunks in segment, Hv), block = 256.
// ---------------------------------------------------------------------------------------
struct PrepSmem {
    __half k[2][kC][64];            // swizzled boxes, filled by TMA
    __half v[2][kC][64];
    __half q[2][kC][64];            // after the Gram phase: T diag(b) as fp16 hi (box 0) and lo (box 1)
    float l[kC][kC + 4];            // strictly lower triangle of L; after the solve: T diag(b A), hi and lo
    float log_a[kC];                // cumulative log decay (inclusive)
    float beta[kC];
    uint64_t full;                  // completes when the three tiles have landed
};
static_assert(sizeof(float) * kC * (kC + 4) >= 2 * kC * 64 * sizeof(__half), "T diag(b A) reuses L");
static_assert(3 * (sizeof(PrepSmem) + 1024) <= 228 * 1024, "three CTAs of the prepare kernel per SM");

__global__ void __launch_bounds__(256, 3)
gdn_scan_prepare_kernel(ScanParams p, const __grid_constant__ CUtensorMap conv_map,
                        const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap u_map) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    PrepSmem &s = *reinterpret_cast<PrepSmem *>(smem_raw);
    if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need the alignment the attribute asks for
        if (threadIdx.x == 0) atomicOr(p.status, TT_DEV_BAD_ITEM);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t chunk = blockIdx.x, h = blockIdx.y;
    const uint32_t hk = (p.flags & TT_GDN_V_TILED) ? h % p.hk : h / (p.hv / p.hk);
    const uint32_t t0 = p.token0 + chunk * kC;
    const uint32_t n_tok = min((uint32_t)kC, p.rows - t0);
    ChunkRecord &rec = p.records[(size_t)chunk * p.hv + h];

    // ---- K, Q, V tiles by TMA (tokens past the end of the sequence read as zero rows) ----
    if (tid == 0) {
        mbar_init(&s.full, 1);
        mbar_fence_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        const int xq = (int)(hk * kD), xk = (int)((p.hk + hk) * kD), xv = (int)((2 * p.hk + h) * kD);
        mbar_expect_tx(&s.full, 3 * kC * kD * 2);
        tma_load_2d(&s.k[0][0][0], &conv_map, xk, (int)t0, &s.full);
        tma_load_2d(&s.k[1][0][0], &conv_map, xk + 64, (int)t0, &s.full);
        tma_load_2d(&s.q[0][0][0], &conv_map, xq, (int)t0, &s.full);
        tma_load_2d(&s.q[1][0][0], &conv_map, xq + 64, (int)t0, &s.full);
        tma_load_2d(&s.v[0][0][0], &conv_map, xv, (int)t0, &s.full);
        tma_load_2d(&s.v[1][0][0], &conv_map, xv + 64, (int)t0, &s.full);
    }

    // ---- per-token gates: log decay and beta (padding tokens: decay 1, beta 0) ----
    if (tid < kC) {
        float la = 0.f, be = 0.f;
        if ((uint32_t)tid < n_tok) {
            const size_t gi = (size_t)(t0 + tid) * p.hv + h;
            if (p.flags & TT_GDN_GATES_F32) {
                la = logf(fmaxf(reinterpret_cast<const float *>(p.a)[gi], 1e-37f));
                be = reinterpret_cast<const float *>(p.b)[gi];
            } else {
                const float x = __half2float(reinterpret_cast<const __half *>(p.a)[gi]) + __bfloat162float(p.dt_bias[h]);
                const float sp = x > 20.f ? x : logf(1.f + expf(x));
                const float al = __bfloat162float(p.a_log[h]);
                la = (p.flags & TT_GDN_A_LOG_PREEXP) ? al * sp : -expf(al) * sp;
                be = 1.f / (1.f + expf(-__half2float(reinterpret_cast<const __half *>(p.b)[gi])));
            }
        }
        s.log_a[tid] = la;
        s.beta[tid] = be;
    }
    __syncthreads();
    if (tid == 0) {   // inclusive running sum of 64 values
        float run = 0.f;
        for (int t = 0; t < kC; ++t) { run += s.log_a[t]; s.log_a[t] = run; }
    }
    {
        const bool landed = mbar_wait(&s.full, 0);   // thread 0 initialised the barrier two __syncthreads ago
        if (__syncthreads_or(!landed)) {
            if (tid == 0) atomicOr(p.status, TT_DEV_WAIT_TIMEOUT);
            return;
        }
    }
    if (tid < kC) {
        rec.decay_a[tid] = expf(s.log_a[tid]);
        rec.decay_w[tid] = expf(s.log_a[kC - 1] - s.log_a[tid]);
    }

    // ---- Gram matrices: warp w -> rows 16*(w&3), columns 32*(w>>2) of K K^T and Q K^T ----
    {
        const int r0 = 16 * (warp & 3), c0 = 32 * (warp >> 2);
        float gk[4][4], gq[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) { gk[n][j] = 0.f; gq[n][j] = 0.f; }
        const uint32_t kb = smem_u32(&s.k[0][0][0]), qb = smem_u32(&s.q[0][0][0]);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
            uint32_t ak[4], aq[4], b0[4], b1[4];
            ldsm_x4(ak, sw_a(kb, r0, ks * 16, lane));
            ldsm_x4(aq, sw_a(qb, r0, ks * 16, lane));
            ldsm_x4(b0, sw_b(kb, c0, ks * 16, lane));
            ldsm_x4(b1, sw_b(kb, c0 + 16, ks * 16, lane));
            mma16816(gk[0], ak, b0[0], b0[1]); mma16816(gk[1], ak, b0[2], b0[3]);
            mma16816(gk[2], ak, b1[0], b1[1]); mma16816(gk[3], ak, b1[2], b1[3]);
            mma16816(gq[0], aq, b0[0], b0[1]); mma16816(gq[1], aq, b0[2], b0[3]);
            mma16816(gq[2], aq, b1[0], b1[1]); mma16816(gq[3], aq, b1[2], b1[3]);
        }
        // L[t][s] = b_t (A_t/A_s)(k_t.k_s) for s < t ;  M[t][s] = (A_t/A_s)(q_t.k_s) for s <= t
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int t = r0 + (lane >> 2) + hh * 8;
                const int sx = c0 + n * 8 + (lane & 3) * 2;      // this thread holds columns sx, sx + 1
                const float la_t = s.log_a[t], be_t = s.beta[t];
                const float2 la_s = *reinterpret_cast<const float2 *>(&s.log_a[sx]);
                const float r0v = sx <= t ? __expf(la_t - la_s.x) : 0.f;
                const float r1v = sx + 1 <= t ? __expf(la_t - la_s.y) : 0.f;
                *reinterpret_cast<float2 *>(&s.l[t][sx]) =
                    make_float2(sx < t ? be_t * r0v * gk[n][2 * hh] : 0.f, sx + 1 < t ? be_t * r1v * gk[n][2 * hh + 1] : 0.f);
                *reinterpret_cast<uint32_t *>(&rec.m[t][sx]) = pack_h2(r0v * gq[n][2 * hh], r1v * gq[n][2 * hh + 1]);
            }
    }
    __syncthreads();

    // ---- T = (I + L)^-1 by forward substitution: thread j owns column j in registers ----
    float x[kC];
    if (tid < kC) {
#pragma unroll
        for (int t = 0; t < kC; ++t) {
            float acc = (t == tid) ? 1.f : 0.f, acc1 = 0.f;   // two chains: a dependent FMA costs 4 cycles
#pragma unroll
            for (int s4 = 0; s4 < t; s4 += 4) {      // row t of L, four columns per (broadcast) load
                const float4 lv = *reinterpret_cast<const float4 *>(&s.l[t][s4]);
                acc = fmaf(-lv.x, x[s4], acc);                       // x[sx] == 0 for sx < j
                if (s4 + 1 < t) acc1 = fmaf(-lv.y, x[s4 + 1], acc1);
                if (s4 + 2 < t) acc = fmaf(-lv.z, x[s4 + 2], acc);
                if (s4 + 3 < t) acc1 = fmaf(-lv.w, x[s4 + 3], acc1);
            }
            x[t] = acc + acc1;
        }
    }
    __syncthreads();   // every column is solved: L (and, since the Gram phase, Q) may be overwritten
    // The T operands are stored TRANSPOSED ([s][t], swizzled boxes, hi then lo): the thread that owns
    // column j of T then writes one 128-byte row per box as eight 16-byte stores instead of 64 scattered
    // 2-byte ones, and the products below read their A fragments with ldmatrix.trans.
    __half *tb = &s.q[0][0][0], *ta = reinterpret_cast<__half *>(&s.l[0][0]);
    if (tid < kC) {
        // column j of T diag(b) and T diag(b A), split into fp16 hi + lo
        const float bj = s.beta[tid], baj = s.beta[tid] * expf(s.log_a[tid]);
        unsigned char *rb = reinterpret_cast<unsigned char *>(tb) + tid * 128;
        unsigned char *ra = reinterpret_cast<unsigned char *>(ta) + tid * 128;
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) {
            uint32_t hb[4], ha[4], lb[4], la[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float vb0 = x[8 * pc + 2 * e] * bj, vb1 = x[8 * pc + 2 * e + 1] * bj;
                const float va0 = x[8 * pc + 2 * e] * baj, va1 = x[8 * pc + 2 * e + 1] * baj;
                hb[e] = pack_h2(vb0, vb1);
                ha[e] = pack_h2(va0, va1);
                const float2 qb = __half22float2(*reinterpret_cast<const __half2 *>(&hb[e]));
                const float2 qa = __half22float2(*reinterpret_cast<const __half2 *>(&ha[e]));
                lb[e] = pack_h2(vb0 - qb.x, vb1 - qb.y);     // what the fp16 rounding left over
                la[e] = pack_h2(va0 - qa.x, va1 - qa.y);
            }
            const uint32_t off = (pc ^ (tid & 7)) << 4;
            *reinterpret_cast<uint4 *>(rb + off) = make_uint4(hb[0], hb[1], hb[2], hb[3]);
            *reinterpret_cast<uint4 *>(rb + kC * 128 + off) = make_uint4(lb[0], lb[1], lb[2], lb[3]);
            *reinterpret_cast<uint4 *>(ra + off) = make_uint4(ha[0], ha[1], ha[2], ha[3]);
            *reinterpret_cast<uint4 *>(ra + kC * 128 + off) = make_uint4(la[0], la[1], la[2], la[3]);
        }
    }
    __syncthreads();

    // ---- U = (T diag b) V and W = (T diag(b A)) K : warp w -> rows 16*(w&3), columns 64*(w>>2) ----
    {
        const int r0 = 16 * (warp & 3), c0 = 64 * (warp >> 2);
        float u[8][4], w[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) { u[n][j] = 0.f; w[n][j] = 0.f; }
        const uint32_t vb = smem_u32(&s.v[0][0][0]), kb = smem_u32(&s.k[0][0][0]);
        const uint32_t tbh = smem_u32(tb), tbl = tbh + kC * 64 * 2, tah = smem_u32(ta), tal = tah + kC * 64 * 2;
#pragma unroll
        for (int ks = 0; ks < kC / 16; ++ks) {
            uint32_t abh[4], abl[4], aah[4], aal[4];
            ldsm_x4_t(abh, sw_at(tbh, ks * 16, r0, lane));
            ldsm_x4_t(abl, sw_at(tbl, ks * 16, r0, lane));
            ldsm_x4_t(aah, sw_at(tah, ks * 16, r0, lane));
            ldsm_x4_t(aal, sw_at(tal, ks * 16, r0, lane));
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bv[4], bk[4];
                ldsm_x4_t(bv, sw_bt(vb, ks * 16, c0 + np * 16, lane));
                ldsm_x4_t(bk, sw_bt(kb, ks * 16, c0 + np * 16, lane));
                mma16816(u[2 * np], abh, bv[0], bv[1]); mma16816(u[2 * np + 1], abh, bv[2], bv[3]);
                mma16816(u[2 * np], abl, bv[0], bv[1]); mma16816(u[2 * np + 1], abl, bv[2], bv[3]);
                mma16816(w[2 * np], aah, bk[0], bk[1]); mma16816(w[2 * np + 1], aah, bk[2], bk[3]);
                mma16816(w[2 * np], aal, bk[0], bk[1]); mma16816(w[2 * np + 1], aal, bk[2], bk[3]);
            }
        }
        // U and W leave through shared memory as the swizzled boxes the state kernel will load (U: four
        // boxes of [64][32 floats] over the K and V tiles, W: two of [64][64 halves] over the T operands)
        // and six TMA tensor stores: whole lines instead of 8- and 4-byte fragment stores from every lane.
        __syncthreads();   // every warp is done with K, V and the T operands
        unsigned char *ust = reinterpret_cast<unsigned char *>(&s.k[0][0][0]);
        unsigned char *wst = reinterpret_cast<unsigned char *>(&s.q[0][0][0]);
        static_assert(sizeof(s.k) + sizeof(s.v) == sizeof(float) * kC * kD && sizeof(s.q) == sizeof(__half) * kC * kD,
                      "staging areas");
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int col = c0 + n * 8 + (lane & 3) * 2;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int r = r0 + (lane >> 2) + hh * 8;
                *reinterpret_cast<float2 *>(ust + (col >> 5) * (kC * 128) + r * 128 + ((((col & 31) >> 2) ^ (r & 7)) << 4) +
                                            (col & 3) * 4) = make_float2(u[n][2 * hh], u[n][2 * hh + 1]);
                *reinterpret_cast<uint32_t *>(wst + (col >> 6) * (kC * 128) + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4) +
                                              (col & 7) * 2) = pack_h2(w[n][2 * hh], w[n][2 * hh + 1]);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            const uint32_t rec_index = chunk * p.hv + h;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                tma_store_2d(&u_map, 32 * q4, (int)(rec_index * kRecRowsU), ust + q4 * (kC * 128));
            tma_store_2d(&w_map, 0, (int)(rec_index * kRecRowsW), wst);
            tma_store_2d(&w_map, 64, (int)(rec_index * kRecRowsW), wst + kC * 128);
            bulk_commit_and_wait_read();
        }
    }
}

// ---------------------------------------------------------------------------------------
// Phase 2: the chunks of a segment in order, for 32 state rows of one value head.
// grid = (Dv / 32, Hv), block = 256 (8 warps). Warp w = (tt = w % 4, sh = w / 4) owns token rows
// 16tt..16tt+15 x state rows 16sh..16sh+15 of the per-chunk products, and state rows 16sh..16sh+15 x
// columns 32tt..32tt+31 as accumulators (four warps alone left the SM's MMA issue mostly idle: one CTA
// per SM, 6 % of the warp slots).
// ---------------------------------------------------------------------------------------
// Two swizzled boxes per [64][128] fp16 tile; U is one box of [64][32] fp32.
struct StateStage {
    __half q[2][kC][64];
    __half k[2][kC][64];
    __half w[2][kC][64];
    __half m[kC][64];
    float u[kC][kDvb];
    float decay_a[kC];
    float decay_w[kC];
    unsigned char pad[512];        // keeps every stage (and so every tile) 1024-byte aligned
};
constexpr int kStages = 3;
constexpr uint32_t kStageTxBytes = 3 * 2 * kC * 64 * 2 + kC * 64 * 2 + kC * kDvb * 4 + 2 * kC * 4;
static_assert(sizeof(StateStage) % 1024 == 0, "stage tiles must stay 1024-byte aligned");
struct StateSmem {
    StateStage stage[kStages];
    __half s16[kDvb][kPitch];      // the state slice as an fp16 MMA operand
    __half c16[kC][kDvb + 8];      // corrections C (tokens x state rows)
    __half cw16[kC][kDvb + 8];     // diag(A_C/A_t) C, the operand of the state update
    uint64_t full[kStages];        // one mbarrier per stage, completed by the copies' byte count
};
static_assert(sizeof(StateSmem) <= 227 * 1024, "state kernel shared memory");

// One thread issues the ten copies of a chunk; they complete on the stage's mbarrier.
__device__ __forceinline__ void state_issue_chunk(StateStage &st, uint64_t *bar, const ScanParams &p,
                                                  const CUtensorMap *conv_map, const CUtensorMap *w_map,
                                                  const CUtensorMap *m_map, const CUtensorMap *u_map,
                                                  uint32_t chunk, uint32_t h, uint32_t hk, uint32_t dv0) {
    const int t0 = (int)(p.token0 + chunk * kC);      // rows past the sequence read as zeros
    const uint32_t rec = chunk * p.hv + h;
    const int xq = (int)(hk * kD), xk = (int)((p.hk + hk) * kD);
    mbar_expect_tx(bar, kStageTxBytes);
    tma_load_2d(&st.w[0][0][0], w_map, 0, (int)(rec * kRecRowsW), bar);
    tma_load_2d(&st.w[1][0][0], w_map, 64, (int)(rec * kRecRowsW), bar);
    tma_load_2d(&st.q[0][0][0], conv_map, xq, t0, bar);
    tma_load_2d(&st.q[1][0][0], conv_map, xq + 64, t0, bar);
    tma_load_2d(&st.u[0][0], u_map, (int)dv0, (int)(rec * kRecRowsU), bar);
    bulk_copy_g2s(&st.decay_a[0], &p.records[rec].decay_a[0], 2 * kC * 4, bar);
    tma_load_2d(&st.m[0][0], m_map, 0, (int)(rec * kRecRowsM), bar);
    tma_load_2d(&st.k[0][0][0], conv_map, xk, t0, bar);
    tma_load_2d(&st.k[1][0][0], conv_map, xk + 64, t0, bar);
}

__global__ void __launch_bounds__(kStateThreads)
gdn_scan_state_kernel(ScanParams p, const __grid_constant__ CUtensorMap conv_map,
                      const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap m_map,
                      const __grid_constant__ CUtensorMap u_map) {
    extern __shared__ __align__(1024) unsigned char state_smem_raw[];
    StateSmem &s = *reinterpret_cast<StateSmem *>(state_smem_raw);
    if ((smem_u32(state_smem_raw) & 1023u) != 0) {   // the swizzled tiles need the alignment the attribute asks for
        if (threadIdx.x == 0) atomicOr(p.status, TT_DEV_BAD_ITEM);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tt = warp & 3;     // token tile of the per-chunk products, column group of the state update
    const int sh = warp >> 2;    // which 16 of the CTA's 32 state rows
    const uint32_t h = blockIdx.y, dv0 = blockIdx.x * kDvb;
    const uint32_t hk = (p.flags & TT_GDN_V_TILED) ? h % p.hk : h / (p.hv / p.hk);
    float *state = p.state + ((size_t)h * kD + dv0) * kD;
    const int g = lane >> 2, q2 = (lane & 3) * 2;

    // state rows sh*16 + g (+8), columns tt*32 + nt*8 + q2 (+1) -> accumulator fragments
    float sacc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const int col = tt * 32 + nt * 8 + q2;
        const float2 lo = *reinterpret_cast<const float2 *>(state + (size_t)(sh * 16 + g) * kD + col);
        const float2 hi = *reinterpret_cast<const float2 *>(state + (size_t)(sh * 16 + g + 8) * kD + col);
        sacc[nt][0] = lo.x; sacc[nt][1] = lo.y; sacc[nt][2] = hi.x; sacc[nt][3] = hi.y;
    }

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) mbar_init(&s.full[i], 1);
        mbar_fence_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (uint32_t c = 0; c < (uint32_t)(kStages - 1) && c < p.n_chunks; ++c)
            state_issue_chunk(s.stage[c], &s.full[c], p, &conv_map, &w_map, &m_map, &u_map, c, h, hk, dv0);
    }
    __syncthreads();

    for (uint32_t c = 0; c < p.n_chunks; ++c) {
        const uint32_t slot = c % kStages;
        StateStage &st = s.stage[slot];
        // publish the current state as an fp16 operand
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int col = tt * 32 + nt * 8 + q2;
            *reinterpret_cast<uint32_t *>(&s.s16[sh * 16 + g][col]) = pack_h2(sacc[nt][0], sacc[nt][1]);
            *reinterpret_cast<uint32_t *>(&s.s16[sh * 16 + g + 8][col]) = pack_h2(sacc[nt][2], sacc[nt][3]);
        }
        const bool landed = mbar_wait(&s.full[slot], (c / kStages) & 1);
        // (1) stage c and s16 are complete; everyone is done with chunk c-1
        if (__syncthreads_or(!landed)) {
            if (tid == 0) atomicOr(p.status, TT_DEV_WAIT_TIMEOUT);
            return;
        }
        // only now may chunk c-1's stage be refilled: its M C and state update read it
        if (tid == 0 && c + kStages - 1 < p.n_chunks) {
            const uint32_t nxt = (c + kStages - 1) % kStages;
            state_issue_chunk(s.stage[nxt], &s.full[nxt], p, &conv_map, &w_map, &m_map, &u_map, c + kStages - 1, h,
                              hk, dv0);
        }

        // ---- P = W S^T and R = Q S^T for this warp's 16 tokens x 16 state rows ----
        const int r0 = tt * 16;
        float pw[2][4], rq[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) { pw[n][j] = 0.f; rq[n][j] = 0.f; }
        const uint32_t wb = smem_u32(&st.w[0][0][0]), qb = smem_u32(&st.q[0][0][0]), sb = smem_u32(&s.s16[0][0]);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
            uint32_t aw[4], aq[4], bs[4];
            ldsm_x4(aw, sw_a(wb, r0, ks * 16, lane));
            ldsm_x4(aq, sw_a(qb, r0, ks * 16, lane));
            ldsm_x4(bs, addr_b(sb, kPitch, sh * 16, ks * 16, lane));
            mma16816(pw[0], aw, bs[0], bs[1]); mma16816(pw[1], aw, bs[2], bs[3]);
            mma16816(rq[0], aq, bs[0], bs[1]); mma16816(rq[1], aq, bs[2], bs[3]);
        }
        // C = U - P (fp32), stored as fp16 twice: plain (for M C) and scaled by A_C/A_t (for the state)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int t = r0 + g + hh * 8;
                const int col = sh * 16 + n * 8 + q2;
                const float2 u = *reinterpret_cast<const float2 *>(
                    reinterpret_cast<const unsigned char *>(&st.u[t][0]) + ((((col >> 2) ^ (t & 7)) << 4) | ((col & 3) << 2)));
                const float c0v = u.x - pw[n][2 * hh], c1v = u.y - pw[n][2 * hh + 1];
                const float wgt = st.decay_w[t];
                *reinterpret_cast<uint32_t *>(&s.c16[t][col]) = pack_h2(c0v, c1v);
                *reinterpret_cast<uint32_t *>(&s.cw16[t][col]) = pack_h2(c0v * wgt, c1v * wgt);
            }
        __syncthreads();   // (2) C of all 64 tokens and 32 state rows is visible

        // ---- O = diag(A) R + M C ; write y ----
        {
            float o[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float a = st.decay_a[r0 + g + hh * 8];
                    o[n][2 * hh] = rq[n][2 * hh] * a; o[n][2 * hh + 1] = rq[n][2 * hh + 1] * a;
                }
            const uint32_t mb = smem_u32(&st.m[0][0]), cb = smem_u32(&s.c16[0][0]);
#pragma unroll
            for (int ks = 0; ks < kC / 16; ++ks) {
                uint32_t am[4], bc[4];
                ldsm_x4(am, sw_a(mb, r0, ks * 16, lane));
                ldsm_x4_t(bc, addr_bt(cb, kDvb + 8, ks * 16, sh * 16, lane));
                mma16816(o[0], am, bc[0], bc[1]); mma16816(o[1], am, bc[2], bc[3]);
            }
            const uint32_t t0 = p.token0 + c * kC;
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const uint32_t t = t0 + r0 + g + hh * 8;
                    if (t < p.rows) {
                        __half *dst = p.y + (size_t)t * p.hv * kD + (size_t)h * kD + dv0 + sh * 16 + n * 8 + q2;
                        *reinterpret_cast<uint32_t *>(dst) =
                            pack_h2(o[n][2 * hh] * p.readout_scale, o[n][2 * hh + 1] * p.readout_scale);
                    }
                }
        }

        // ---- S = A_C S + (diag(A_C/A_t) C)^T K : this warp's 16 rows x 32 columns ----
        {
            const float a_c = st.decay_a[kC - 1];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) sacc[nt][j] *= a_c;
            const uint32_t cwb = smem_u32(&s.cw16[0][0]), kb = smem_u32(&st.k[0][0][0]);
#pragma unroll
            for (int ks = 0; ks < kC / 16; ++ks) {
                uint32_t ac[4], b0[4], b1[4];
                ldsm_x4_t(ac, addr_at(cwb, kDvb + 8, ks * 16, sh * 16, lane));
                ldsm_x4_t(b0, sw_bt(kb, ks * 16, tt * 32, lane));
                ldsm_x4_t(b1, sw_bt(kb, ks * 16, tt * 32 + 16, lane));
                mma16816(sacc[0], ac, b0[0], b0[1]); mma16816(sacc[1], ac, b0[2], b0[3]);
                mma16816(sacc[2], ac, b1[0], b1[1]); mma16816(sacc[3], ac, b1[2], b1[3]);
            }
        }
        // the next iteration's barrier (1) orders these reads of stage c / c16 / cw16 against
        // their next writes; s16 is rewritten before it, but only after barrier (2) of this chunk
    }

#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const int col = tt * 32 + nt * 8 + q2;
        *reinterpret_cast<float2 *>(state + (size_t)(sh * 16 + g) * kD + col) = make_float2(sacc[nt][0], sacc[nt][1]);
        *reinterpret_cast<float2 *>(state + (size_t)(sh * 16 + g + 8) * kD + col) = make_float2(sacc[nt][2], sacc[nt][3]);
    }
}

// ---------------------------------------------------------------------------------------
// Phase 2 on tcgen05. One CTA per (32 state rows, value head); chunks in order. The state slice is
// kept TRANSPOSED in tensor memory as an fp32 accumulator (lane = state column, TMEM column = state
// row) for the whole segment. Per chunk, three chains of MMAs (M = 128, N = 32):
//   D1 = [Q; W] S_0^T          A: 128 token rows (Q rows 0-63, W rows 64-127) x 128, K-major
//                              B: S_0^T as fp16 [128 columns][32 rows], N-major, rewritten every chunk
//   D3 = a_C S_0^T + K^T Cw    A: K [64 tokens][128] read M-major; B: Cw [64 tokens][32 rows], N-major;
//                              a_C S_0^T is put there beforehand by the threads that publish S_0
//   D2 = M C                   A: M [64][64] K-major (rows 64-127 of the operand are whatever follows
//                              it in shared memory; those accumulator lanes are never read)
//                              B: C [64 tokens][32 rows], N-major
// The N-major B operands are what a thread that owns one TMEM lane can write as whole 16-byte pieces
// (its 32 values are 32 consecutive n). The recurrence is one dependent chain per chunk,
//   publish S_0 -> D1 -> C = U - P -> D3 -> publish ...,
// so everything else is kept off it: D2 is issued after D3, the next operands are requested after
// D1 is under way, U is in registers before P arrives.
// Warps 0-3 own the TMEM lanes (warp w lanes 32w..32w+31): all four publish S_0 and rescale the
// accumulator; warps 0-1 (lanes = R rows) combine R and D2 into y, warps 2-3 (lanes = P rows) form
// C = U - P. Warp 4, one lane, loads the operands by TMA and issues the MMAs. Every wait is bounded.
// ---------------------------------------------------------------------------------------
struct TcStage {
    __half qw[2][2 * kC][64];      // per 64-column box: Q rows, then W rows
    __half k[2][kC][64];
    __half m[kC][64];
    float u[kC][kDvb];             // directly after m (see D2 above)
    float decay_a[kC];
    float decay_w[kC];
    unsigned char pad[512];
};
static_assert(sizeof(TcStage) % 1024 == 0, "stage tiles must stay 1024-byte aligned");
constexpr int kTcStages = 3;
constexpr int kTcThreads = 160;
constexpr uint32_t kTcCols = 128, kColPR = 0, kColO = 32, kColS = 64;
struct TcSmem {
    TcStage stage[kTcStages];
    __half s16[kD][64];            // S_0^T: row = state column, halves 0-31 = state rows (32-63 unused)
    __half ccw[kC][64];            // row = token: halves 0-31 = C, 32-63 = diag(A_C/A_t) C
    uint64_t full[kTcStages];      // operands of a chunk have landed
    uint64_t s16_ready;            // 128 arrivals: S_0 published
    uint64_t pr_done;              // D1 complete
    uint64_t c_ready;              // 128 arrivals: accumulator rescaled (all), C and Cw written (warps 2-3)
    uint64_t o_done;               // D2 complete
    uint64_t s_done;               // D3 complete
    uint32_t tmem_base;
};
static_assert(sizeof(TcSmem) + 1024 <= 227 * 1024, "tcgen05 state kernel shared memory");

__device__ __forceinline__ void tc_issue_chunk(TcStage &st, uint64_t *bar, const ScanParams &p,
                                               const CUtensorMap *conv_map, const CUtensorMap *w_map,
                                               const CUtensorMap *m_map, const CUtensorMap *u_map, uint32_t chunk,
                                               uint32_t h, uint32_t hk, uint32_t dv0) {
    const int t0 = (int)(p.token0 + chunk * kC);      // rows past the sequence read as zeros
    const uint32_t rec = chunk * p.hv + h;
    const int xq = (int)(hk * kD), xk = (int)((p.hk + hk) * kD);
    mbar_expect_tx(bar, kStageTxBytes);
    tma_load_2d(&st.qw[0][0][0], conv_map, xq, t0, bar);
    tma_load_2d(&st.qw[1][0][0], conv_map, xq + 64, t0, bar);
    tma_load_2d(&st.qw[0][kC][0], w_map, 0, (int)(rec * kRecRowsW), bar);
    tma_load_2d(&st.qw[1][kC][0], w_map, 64, (int)(rec * kRecRowsW), bar);
    bulk_copy_g2s(&st.decay_a[0], &p.records[rec].decay_a[0], 2 * kC * 4, bar);
    tma_load_2d(&st.u[0][0], u_map, (int)dv0, (int)(rec * kRecRowsU), bar);
    tma_load_2d(&st.m[0][0], m_map, 0, (int)(rec * kRecRowsM), bar);
    tma_load_2d(&st.k[0][0][0], conv_map, xk, t0, bar);
    tma_load_2d(&st.k[1][0][0], conv_map, xk + 64, t0, bar);
}

__global__ void __launch_bounds__(kTcThreads)
gdn_scan_state_tc_kernel(ScanParams p, const __grid_constant__ CUtensorMap conv_map,
                         const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap m_map,
                         const __grid_constant__ CUtensorMap u_map, uint32_t idesc_kn, uint32_t idesc_mn) {
    extern __shared__ __align__(1024) unsigned char tc_smem_raw[];
    TcSmem &s = *reinterpret_cast<TcSmem *>(tc_smem_raw);
    if ((smem_u32(tc_smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicOr(p.status, TT_DEV_BAD_ITEM);
        return;
    }
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t h = blockIdx.y, dv0 = blockIdx.x * kDvb;
    const uint32_t hk = (p.flags & TT_GDN_V_TILED) ? h % p.hk : h / (p.hv / p.hk);
    float *state = p.state + ((size_t)h * kD + dv0) * kD;

    if (tid == 4 * 32) {
        for (int i = 0; i < kTcStages; ++i) mbar_init(&s.full[i], 1);
        mbar_init(&s.s16_ready, 128);
        mbar_init(&s.pr_done, 1);
        mbar_init(&s.c_ready, 128);
        mbar_init(&s.o_done, 1);
        mbar_init(&s.s_done, 1);
        mbar_fence_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (uint32_t c = 0; c < 2 && c < p.n_chunks; ++c)
            tc_issue_chunk(s.stage[c], &s.full[c], p, &conv_map, &w_map, &m_map, &u_map, c, h, hk, dv0);
    }
    if (warp == 4) {
        __syncwarp();
        tmem_alloc(&s.tmem_base, kTcCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    bool ok = true;

    if (warp == 4) {
        if (lane == 0) {
            const uint32_t s16_a = smem_u32(&s.s16[0][0]), ccw_a = smem_u32(&s.ccw[0][0]);
            for (uint32_t c = 0; c < p.n_chunks && ok; ++c) {
                const uint32_t slot = c % kTcStages;
                TcStage &st = s.stage[slot];
                const uint32_t qw_a = smem_u32(&st.qw[0][0][0]), m_a = smem_u32(&st.m[0][0]),
                               k_a = smem_u32(&st.k[0][0][0]);
                ok = mbar_wait(&s.full[slot], (c / kTcStages) & 1) && mbar_wait(&s.s16_ready, c & 1);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kD / 16; ++ks) {
                    const uint64_t ad = make_desc(qw_a + (ks >> 2) * (2 * kC * 128) + (ks & 3) * 32, 16, 1024);
                    const uint64_t bd = make_desc(s16_a + ks * 2048, kD * 128, 1024);
                    mma_ss(tmem + kColPR, ad, bd, idesc_kn, ks > 0 ? 1u : 0u);
                }
                mma_commit(&s.pr_done);
                // every consumer is past chunk c-1 (it published S_0 of chunk c): that stage may take chunk c+2
                if (c + 2 < p.n_chunks) {
                    const uint32_t nxt = (c + 2) % kTcStages;
                    tc_issue_chunk(s.stage[nxt], &s.full[nxt], p, &conv_map, &w_map, &m_map, &u_map, c + 2, h, hk, dv0);
                }
                ok = mbar_wait(&s.c_ready, c & 1);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kC / 16; ++kk) {
                    // K as the M-major operand: 64-column groups 8 KB apart (LBO), 8-token groups 1 KB apart (SBO)
                    const uint64_t ad = make_desc(k_a + kk * 2048, kC * 128, 1024);
                    const uint64_t bd = make_desc(ccw_a + kk * 2048 + 64, kC * 128, 1024);   // the Cw half of each row
                    mma_ss(tmem + kColS, ad, bd, idesc_mn, 1u);
                }
                mma_commit(&s.s_done);
#pragma unroll
                for (int ks = 0; ks < kC / 16; ++ks) {
                    const uint64_t ad = make_desc(m_a + ks * 32, 16, 1024);
                    const uint64_t bd = make_desc(ccw_a + ks * 2048, kC * 128, 1024);
                    mma_ss(tmem + kColO, ad, bd, idesc_kn, ks > 0 ? 1u : 0u);
                }
                mma_commit(&s.o_done);
            }
        }
    } else {
        const uint32_t i = warp * 32 + lane;                 // TMEM lane: state column, or operand row of D1 / D2
        const uint32_t lane_addr = (warp * 32) << 16;
        uint32_t sv[32];
#pragma unroll
        for (int r = 0; r < 32; ++r) sv[r] = __float_as_uint(state[(size_t)r * kD + i]);
        unsigned char *s16_row = reinterpret_cast<unsigned char *>(&s.s16[i][0]);
        const uint32_t t = i & 63;                           // token of this lane in D1 / D2
        unsigned char *ccw_row = reinterpret_cast<unsigned char *>(&s.ccw[t][0]);
        for (uint32_t c = 0; c < p.n_chunks; ++c) {
            const uint32_t slot = c % kTcStages;
            TcStage &st = s.stage[slot];
            if (c > 0) {
                ok = warp_all(mbar_wait(&s.s_done, (c - 1) & 1));
                if (!ok) break;
                tc_fence_after();
                tmem_ld32(tmem + lane_addr + kColS, sv);
                tmem_wait_ld();
            }
            // S_0^T row i: state rows 8j..8j+7 are the 16-byte piece j
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_h2(__uint_as_float(sv[8 * j]), __uint_as_float(sv[8 * j + 1]));
                v.y = pack_h2(__uint_as_float(sv[8 * j + 2]), __uint_as_float(sv[8 * j + 3]));
                v.z = pack_h2(__uint_as_float(sv[8 * j + 4]), __uint_as_float(sv[8 * j + 5]));
                v.w = pack_h2(__uint_as_float(sv[8 * j + 6]), __uint_as_float(sv[8 * j + 7]));
                *reinterpret_cast<uint4 *>(s16_row + ((j ^ (i & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&s.s16_ready);

            // off the chain: the accumulator becomes a_C S_0^T before D3 adds to it
            ok = warp_all(mbar_wait(&s.full[slot], (c / kTcStages) & 1));
            if (!ok) break;
            const float a_c = st.decay_a[kC - 1];
#pragma unroll
            for (int r = 0; r < 32; ++r) sv[r] = __float_as_uint(__uint_as_float(sv[r]) * a_c);
            tmem_st32(tmem + lane_addr + kColS, sv);
            tmem_wait_st();
            tc_fence_before();
            float uu[32];
            float wgt = 0.f, a_t = 0.f;
            if (warp >= 2) {
                wgt = st.decay_w[t];
                const unsigned char *urow = reinterpret_cast<const unsigned char *>(&st.u[t][0]);
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                    const float4 u4 = *reinterpret_cast<const float4 *>(urow + ((q4 ^ (t & 7)) << 4));
                    uu[4 * q4] = u4.x; uu[4 * q4 + 1] = u4.y; uu[4 * q4 + 2] = u4.z; uu[4 * q4 + 3] = u4.w;
                }
            } else {
                a_t = st.decay_a[t];
                mbar_arrive(&s.c_ready);
            }

            ok = warp_all(mbar_wait(&s.pr_done, c & 1));
            if (!ok) break;
            tc_fence_after();
            uint32_t pv[32];
            tmem_ld32(tmem + lane_addr + kColPR, pv);
            tmem_wait_ld();
            if (warp >= 2) {
                // P rows: C = U - P for token t; pieces 0-3 of the row are C, pieces 4-7 are Cw
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float cv[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) cv[e] = uu[8 * j + e] - __uint_as_float(pv[8 * j + e]);
                    uint4 v, w;
                    v.x = pack_h2(cv[0], cv[1]); v.y = pack_h2(cv[2], cv[3]);
                    v.z = pack_h2(cv[4], cv[5]); v.w = pack_h2(cv[6], cv[7]);
                    w.x = pack_h2(cv[0] * wgt, cv[1] * wgt); w.y = pack_h2(cv[2] * wgt, cv[3] * wgt);
                    w.z = pack_h2(cv[4] * wgt, cv[5] * wgt); w.w = pack_h2(cv[6] * wgt, cv[7] * wgt);
                    *reinterpret_cast<uint4 *>(ccw_row + ((j ^ (t & 7)) << 4)) = v;
                    *reinterpret_cast<uint4 *>(ccw_row + (((j + 4) ^ (t & 7)) << 4)) = w;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                mbar_arrive(&s.c_ready);
            } else {
                // R rows: y_t = readout_scale (A_t R_t + (M C)_t)
                ok = warp_all(mbar_wait(&s.o_done, c & 1));
                if (!ok) break;
                tc_fence_after();
                uint32_t ov[32];
                tmem_ld32(tmem + lane_addr + kColO, ov);
                tmem_wait_ld();
                const uint32_t tok = p.token0 + c * kC + t;
                if (tok < p.rows) {
                    uint4 *dst = reinterpret_cast<uint4 *>(p.y + (size_t)tok * p.hv * kD + (size_t)h * kD + dv0);
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        uint32_t w4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int r = q8 * 8 + e * 2;
                            const float o0 = fmaf(__uint_as_float(pv[r]), a_t, __uint_as_float(ov[r]));
                            const float o1 = fmaf(__uint_as_float(pv[r + 1]), a_t, __uint_as_float(ov[r + 1]));
                            w4[e] = pack_h2(o0 * p.readout_scale, o1 * p.readout_scale);
                        }
                        dst[q8] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                    }
                }
            }
        }
        if (ok) {
            ok = warp_all(mbar_wait(&s.s_done, (p.n_chunks - 1) & 1));
            if (ok) {
                tc_fence_after();
                tmem_ld32(tmem + lane_addr + kColS, sv);
                tmem_wait_ld();
#pragma unroll
                for (int r = 0; r < 32; ++r) state[(size_t)r * kD + i] = __uint_as_float(sv[r]);
            }
        }
    }

    if (!ok) atomicOr(p.status, TT_DEV_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kTcCols);
    }
}

}  // namespace

TT_API int tt_gdn_scan_chunked(tt_context *ctx, tt_stream stream, const void *conv_out, const void *a,
                               const void *b, const void *a_log, const void *dt_bias, float *state, void *y,
                               const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride, uint32_t chunk) {
    TT_ENTER(ctx);
    if (shape == nullptr || conv_out == nullptr || a == nullptr || b == nullptr || state == nullptr || y == nullptr)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "chunked scan needs non-null buffers and shape");
    const bool f32_gates = (shape->flags & TT_GDN_GATES_F32) != 0;
    if (!f32_gates && (a_log == nullptr || dt_bias == nullptr))
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "a_log and dt_bias must not be null");
    if (shape->n_k_heads == 0 || shape->n_v_heads == 0 || shape->n_v_heads % shape->n_k_heads != 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_v_heads must be a positive multiple of n_k_heads");
    if (rows == 0) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "rows must be positive");
    if (chunk != (uint32_t)kC)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "chunk must be %d, got %u", kC, chunk);
    if (shape->key_dim != (uint32_t)kD || shape->value_dim != (uint32_t)kD)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE,
                            "the chunked scan is built for key_dim == value_dim == %d (use tt_gdn_step otherwise)", kD);
    const uint32_t tight = 2 * shape->n_k_heads * kD + shape->n_v_heads * kD;
    if (row_stride < tight) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "row_stride %u is smaller than the qkv width %u", row_stride, tight);
    if (row_stride % 8 != 0 || ((uintptr_t)conv_out & 15) || ((uintptr_t)state & 15) || ((uintptr_t)y & 3))
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "chunked scan needs 16-byte aligned rows and state");
    const size_t per_chunk = sizeof(ChunkRecord) * shape->n_v_heads;
    const uint32_t seg_chunks = (uint32_t)(ctx->workspace_bytes / per_chunk);
    if (seg_chunks == 0) return tt_set_error(ctx, TT_ERR_OOM, "context workspace too small for one chunk of the scan");

    static bool attrs_set = false;
    if (!attrs_set) {
        cudaError_t e = cudaFuncSetAttribute(gdn_scan_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)sizeof(PrepSmem));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gdn_scan_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)sizeof(StateSmem));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gdn_scan_state_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)sizeof(TcSmem));
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn scan smem attribute");
        attrs_set = true;
    }
    CUtensorMap conv_map, w_map, m_map, u_map;
    {
        ChunkRecord *rec0 = reinterpret_cast<ChunkRecord *>(ctx->partials);
        const uint64_t n_rec = (uint64_t)seg_chunks * shape->n_v_heads;
        const bool ok =
            tt_make_tensor_map_2d(&conv_map, conv_out, TT_F16, tight, rows, row_stride, kC) &&
            tt_make_tensor_map_2d(&w_map, &rec0->w[0][0], TT_F16, kD, (n_rec - 1) * kRecRowsW + kC, kD, kC) &&
            tt_make_tensor_map_2d(&m_map, &rec0->m[0][0], TT_F16, kC, (n_rec - 1) * kRecRowsM + kC, kC, kC) &&
            tt_make_tensor_map_2d_f32(&u_map, &rec0->u[0][0], kD, (n_rec - 1) * kRecRowsU + kC, kD * 4, kC);
        if (!ok) return tt_set_error(ctx, TT_ERR_CUDA, "cuTensorMapEncodeTiled failed for the scan operands");
    }
    ScanParams p;
    p.conv_out = reinterpret_cast<const __half *>(conv_out); p.a = a; p.b = b;
    p.a_log = reinterpret_cast<const __nv_bfloat16 *>(a_log); p.dt_bias = reinterpret_cast<const __nv_bfloat16 *>(dt_bias);
    p.state = state; p.y = reinterpret_cast<__half *>(y);
    p.records = reinterpret_cast<ChunkRecord *>(ctx->partials);
    p.hk = shape->n_k_heads; p.hv = shape->n_v_heads; p.rows = rows; p.row_stride = row_stride; p.flags = shape->flags;
    p.readout_scale = shape->readout_scale;
    p.status = ctx->status;
    // TT_GDN_SCAN_FORCE_MMA_SYNC=1 keeps the state recurrence on the mma.sync kernel (an A/B switch for tests)
    const char *force = getenv("TT_GDN_SCAN_FORCE_MMA_SYNC");
    const bool use_mma_sync = force != nullptr && force[0] == '1';
    if (!use_mma_sync && ((uintptr_t)y & 15))
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "chunked scan needs a 16-byte aligned output");
    const uint32_t idesc_kn = tt_make_idesc_f16(TT_F16, kDvb, true, false);   // A K-major, B N-major
    const uint32_t idesc_mn = tt_make_idesc_f16(TT_F16, kDvb, true, true);    // A M-major, B N-major
    const uint32_t total_chunks = (rows + kC - 1) / kC;
    for (uint32_t c0 = 0; c0 < total_chunks; c0 += seg_chunks) {
        p.token0 = c0 * kC;
        p.n_chunks = total_chunks - c0 < seg_chunks ? total_chunks - c0 : seg_chunks;
        gdn_scan_prepare_kernel<<<dim3(p.n_chunks, p.hv), 256, sizeof(PrepSmem), (cudaStream_t)stream>>>(
            p, conv_map, w_map, u_map);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_scan_prepare launch");
        if (use_mma_sync)
            gdn_scan_state_kernel<<<dim3(kD / kDvb, p.hv), kStateThreads, sizeof(StateSmem), (cudaStream_t)stream>>>(
                p, conv_map, w_map, m_map, u_map);
        else
            gdn_scan_state_tc_kernel<<<dim3(kD / kDvb, p.hv), kTcThreads, sizeof(TcSmem), (cudaStream_t)stream>>>(
                p, conv_map, w_map, m_map, u_map, idesc_kn, idesc_mn);
        e = cudaGetLastError();
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "gdn_scan_state launch");
        ctx->launches += 2;
    }
    return TT_OK;
}
