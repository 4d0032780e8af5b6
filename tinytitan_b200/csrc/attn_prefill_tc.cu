// Causal prefill attention on the sm_100a tensor cores (tcgen05 + TMEM + TMA), head_dim 256.
//
// One CTA owns 128 consecutive query rows of one q head and walks the keys in tiles of 128.
// Eleven warps: warp 0 holds the two TMA producers (lane 0: K, lane 1: V), warp 1 issues the
// Q.K^T MMAs and owns the TMEM allocation, warp 6 issues the P.V MMAs, warps 2-5 and 7-10 are two
// softmax warpgroups (two threads per query row: group A takes keys 0..63 of every tile, group B
// keys 64..127):
//
//   S       = Q . K_j^T        TS MMA  M128 N128 K16 x16   A = Q in TMEM columns 384..511 (stored there
//                                                          once by the softmax threads), D = columns 256..383
//   P_j     = exp2(S - m)      tcgen05.ld -> registers -> shared memory (K-major A operand, 128-byte swizzle)
//   O      += P_j . V_j        SS MMA  M128 N256 K16 x8    D = TMEM columns 0..255
//
// How it got here (config 3, bf16, 0.571 ms -> 0.441 ms):
//  * An M128 K16 tcgen05.mma costs about the same for every N up to 128 (measured: the tile time is
//    the same for N = 16 ... 128 and falls steeply with the NUMBER of instructions), so Q.K^T is
//    issued 128 keys wide: 24 instructions per 128 keys instead of 40.
//  * With tiles that wide one softmax warpgroup became the limit, hence two; the two warps of a TMEM
//    lane quarter exchange their row maxima through shared memory once per tile (an mbarrier with a
//    bounded wait, one arrive per warp) and then take identical decisions.
//  * The score tile is released as soon as both groups hold it in registers (s_read), and P goes
//    through shared memory instead of being aliased over S, so Q.K^T of tile j+1 overlaps the softmax
//    of tile j with ONE score tile; the TMEM columns this frees hold Q, which takes the 4 KB of Q
//    per instruction off the shared-memory port.
//  * Two issuing threads, so that neither product waits behind the other's barrier.
//
// Shared memory (all 227 KB): K streams as [128 keys][128 head-dim] chunks (32 KB, two [128][64]
// sub-tiles) through a 4-slot ring, each released as soon as its eight MMAs have retired; one V tile
// (64 KB) is fetched and released in two 64-key halves; P is 32 KB (two [128 rows][64 keys]
// sub-tiles).
//
// The running maximum is only raised when it moved by more than 2^8 ("lazy rescale"); O and the
// row sum then share one stale reference maximum, which cancels in O / l. The row sum is taken on
// the ROUNDED weights the MMA consumes. Every mbarrier wait is bounded: when a wait runs out the
// role sets TT_DEV_WAIT_TIMEOUT in the status word and falls through to the common exit, where
// TMEM is released.
//
// Arithmetic semantics: sources/TinyTitanCore/Metal/Prefill/prefill.metal:1056-1158 (visible
// keys [first, min(kvValid, start+t+1)), fp32 accumulation, row_sum == 0 -> 0).
#include "tt_sm100.h"

#include <cstdlib>
#include <type_traits>

namespace {

constexpr int kHD = 256;
constexpr int kBM = 128;              // query rows per CTA
constexpr int kBN = 128;              // keys per tile
constexpr int kBox = 64;              // keys per TMA box
constexpr int kThreads = 352;             // 11 warps: producers, Q.K^T issuer, softmax A (2-5), P.V issuer, softmax B (7-10)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

constexpr int kKVTile = kBN * kHD * 2;         // 65536: 4 sub-tiles [128 keys][64]
constexpr int kKVSub = kBN * 64 * 2;           // 16384
constexpr int kBoxBytes = kBox * 64 * 2;       // 8192: one TMA box, half a sub-tile
constexpr int kKSlots = 4;
constexpr int kKChunk = kKVTile / 2;           // 32768: [128 keys][128 head-dim] = 2 sub-tiles
constexpr int kPBytes = kBM * kBN * 2;           // 32768: 2 sub-tiles [128 rows][64 keys], K-major A operand
constexpr int kPSub = kBM * 64 * 2;              // 16384
constexpr int kSmemBytes = kKSlots * kKChunk + kKVTile + kPBytes + 2304 /*barriers, exchange*/;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS = 256, kColQ = 384;   // Q: 128 columns of 16-bit pairs

struct Barriers {
    uint64_t q_ready;                 // the 256 softmax threads have stored their halves of the Q rows into TMEM
    uint64_t k_full[kKSlots], k_empty[kKSlots];   // per K chunk slot
    uint64_t v_full[2], v_empty[2];   // per 64-key half of the V tile
    uint64_t s_full;
    uint64_t s_read;                  // both softmax warpgroups hold the tile's scores in registers: the score
                                      // tile may take Q.K^T of the next tile
    uint64_t p_ready;                 // P of the tile is in shared memory
    uint64_t p_free;                  // P.V of the tile retired: P may be overwritten
    uint64_t o_ready;
    uint64_t pair[4];                 // the two softmax warps of a TMEM lane quarter (count 2, bounded waits)
    uint32_t tmem_base;
    uint32_t pad;
    float xchg[2][2][kBM];            // [buffer][key half][row]: per-tile row maxima, at the end the row sums
};
static_assert(sizeof(Barriers) <= 2304, "the barrier block must fit its share of shared memory");

struct PrefillTcParams {
    uint32_t start_position, query_count, n_q_heads, n_kv_heads, kv_valid_count, sliding_window;
    uint32_t o_token_stride;   // elements
    uint32_t q_token_stride;   // elements
    uint32_t n_q_tiles;
    float scale_log2;
    uint32_t idesc_qk, idesc_pv;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const T *__restrict__ q, const __grid_constant__ CUtensorMap k_map,
                       const __grid_constant__ CUtensorMap v_map, T *__restrict__ out, PrefillTcParams p,
                       uint32_t *__restrict__ status) {
    // every byte of the 227 KB is spoken for, so there is no slack to align the tiles by hand: the
    // dynamic window of a kernel without static shared memory starts 1024-byte aligned, and a launch
    // where it does not is refused rather than run with broken swizzles
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = smem_raw;
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicOr(status, TT_DEV_BAD_ITEM);
        return;
    }
    unsigned char *k_s = smem;
    unsigned char *v_s = smem + kKSlots * kKChunk;
    unsigned char *p_s = v_s + kKVTile;
    Barriers *bars = reinterpret_cast<Barriers *>(p_s + kPBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // heavy (late) query tiles first; the heads of one KV group are adjacent so they share K/V in L2
    const uint32_t head = blockIdx.x % p.n_q_heads;
    const uint32_t q_tile = p.n_q_tiles - 1 - blockIdx.x / p.n_q_heads;
    const uint32_t kv_head = head / (p.n_q_heads / p.n_kv_heads);
    const uint32_t row0 = q_tile * kBM;                              // first query row of the tile
    const uint32_t rows_here = min((uint32_t)kBM, p.query_count - row0);
    const uint32_t abs_lo = p.start_position + row0;                 // absolute position of row 0
    const uint32_t abs_hi = abs_lo + rows_here - 1;                  // ... of the last valid row
    uint32_t key_lo = 0;
    if (p.sliding_window != 0 && abs_lo + 1 > p.sliding_window) key_lo = abs_lo + 1 - p.sliding_window;
    const uint32_t key_hi = min(p.kv_valid_count, abs_hi + 1);       // exclusive
    const uint32_t tile_lo = key_lo / kBN;
    const uint32_t n_tiles = (key_hi + kBN - 1) / kBN - tile_lo;     // >= 1

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_ready, 256);
        mbar_init(&bars->s_full, 1);
        mbar_init(&bars->s_read, 256);
        for (int s = 0; s < kKSlots; ++s) { mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->v_full[s], 1);
            mbar_init(&bars->v_empty[s], 1);
        }
        mbar_init(&bars->p_ready, 256);
        mbar_init(&bars->p_free, 1);
        mbar_init(&bars->o_ready, 1);
        for (int s = 0; s < 4; ++s) mbar_init(&bars->pair[s], 2);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    bool failed = false;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producers
        // lane 0: Q, then the K tiles; lane 1: the V tiles in halves (independent progress).
        // A box is [64 keys][64 elements]; sub-tile `sub` of a tile holds keys 0..127 of 64 head-dim columns.
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kc = 0; ok && kc < 2 * n_tiles; ++kc) {      // chunk kc = tile kc/2, head-dim half kc%2
                const uint32_t slot = kc % kKSlots;
                if (kc >= (uint32_t)kKSlots) ok = mbar_wait(&bars->k_empty[slot], ((kc / kKSlots) - 1) & 1);
                if (!ok) break;
                mbar_expect_tx(&bars->k_full[slot], kKChunk);
                for (int sub = 0; sub < 2; ++sub)
                    for (int half = 0; half < 2; ++half)
                        tma_load_2d(k_s + slot * kKChunk + sub * kKVSub + half * kBoxBytes, &k_map,
                                    (int)(kv_head * kHD + (kc & 1) * 128 + sub * 64),
                                    (int)((tile_lo + (kc >> 1)) * kBN + half * kBox), &bars->k_full[slot]);
            }
            failed = !ok;
        } else if (lane == 1) {
            bool ok = true;
            for (uint32_t j = 0; ok && j < n_tiles; ++j)
                for (int half = 0; ok && half < 2; ++half) {
                    if (j >= 1) ok = mbar_wait(&bars->v_empty[half], (j - 1) & 1);
                    if (!ok) break;
                    mbar_expect_tx(&bars->v_full[half], kKVTile / 2);
                    for (int sub = 0; sub < 4; ++sub)
                        tma_load_2d(v_s + sub * kKVSub + half * kBoxBytes, &v_map, (int)(kv_head * kHD + sub * 64),
                                    (int)((tile_lo + j) * kBN + half * kBox), &bars->v_full[half]);
                }
            failed = !ok;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ Q.K^T issuer
        if (lane == 0) {
            const uint32_t k_addr = smem_u32(k_s);
            bool ok = mbar_wait(&bars->q_ready, 0);
            for (uint32_t j = 0; ok && j < n_tiles; ++j) {
                if (j >= 1) ok = mbar_wait(&bars->s_read, (j - 1) & 1);
                for (uint32_t half = 0; ok && half < 2; ++half) {
                    const uint32_t kc = 2 * j + half, slot = kc % kKSlots;
                    ok = mbar_wait(&bars->k_full[slot], (kc / kKSlots) & 1);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        // A = Q from TMEM (8 columns per 16-wide step), B = the K chunk
                        const uint64_t bd = make_desc(k_addr + slot * kKChunk + (ks >> 2) * kKVSub + (ks & 3) * 32, 16, 1024);
                        mma_ts(tmem + kColS, tmem + kColQ + (half * 8 + ks) * 8, bd, p.idesc_qk, (half > 0 || ks > 0) ? 1u : 0u);
                    }
                    mma_commit(&bars->k_empty[slot]);
                }
                if (!ok) break;
                mma_commit(&bars->s_full);
            }
            failed = !ok;
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------------ P.V issuer
        if (lane == 0) {
            const uint32_t v_addr = smem_u32(v_s), p_addr = smem_u32(p_s);
            bool ok = true;
            for (uint32_t j = 0; ok && j < n_tiles; ++j) {
                ok = mbar_wait(&bars->p_ready, j & 1);
                for (int half = 0; ok && half < 2; ++half) {
                    ok = mbar_wait(&bars->v_full[half], j & 1);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        // P: K-major A operand from shared memory, sub-tile `half` = keys 64*half.., 16 keys
                        // (32 B) per step. V: MN-major B operand, 64-wide head-dim atoms kKVSub apart (LBO),
                        // 8-key groups 1024 B apart (SBO), 16 keys (2048 B) per step.
                        const int kk = half * 4 + k4;
                        const uint64_t ad = make_desc(p_addr + half * kPSub + k4 * 32, 16, 1024);
                        const uint64_t bd = make_desc(v_addr + kk * 2048, kKVSub, 1024);
                        mma_ss(tmem + kColO, ad, bd, p.idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&bars->v_empty[half]);
                }
                if (!ok) break;
                mma_commit(&bars->p_free);
                mma_commit(&bars->o_ready);
            }
            failed = !ok;
        }
    } else {
        // ------------------------------------------------------------------ softmax: two threads per row
        // Warpgroup A (warps 2-5) takes keys 0..63 of every tile, warpgroup B (warps 7-10) keys 64..127;
        // the two warps of a TMEM lane quarter exchange their row maxima through shared memory once per
        // tile (bounded mbarrier, one arrive per warp) and then take identical decisions.
        const uint32_t quarter = warp & 3;                       // TMEM lane quarter this warp may touch
        const uint32_t wg = warp >= 7 ? 1u : 0u;                 // key half of the tile
        const uint32_t row = quarter * 32 + lane;                // row inside the tile
        const uint32_t lane_addr = (quarter * 32) << 16;
        const bool row_valid = row < rows_here;
        const uint32_t abs_q = abs_lo + row;
        uint32_t first = 0;
        if (p.sliding_window != 0 && abs_q + 1 > p.sliding_window) first = abs_q + 1 - p.sliding_window;
        const uint32_t last = min(p.kv_valid_count, abs_q + 1);  // exclusive
        uint32_t pair_phase = 0;
        auto pair_sync = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->pair[quarter]);
            const bool got = warp_all(mbar_wait(&bars->pair[quarter], pair_phase & 1));
            pair_phase ^= 1;
            return got;
        };

        // this thread's half of its query row -> TMEM lane `row`, columns kColQ + 64*wg.. (two 16-bit
        // elements per column)
        {
            const T *qrow = q + (size_t)(row0 + row) * p.q_token_stride + (size_t)head * kHD + wg * (kHD / 2);
#pragma unroll 1
            for (int c0 = 0; c0 < kHD / 4; c0 += 32) {
                uint32_t w[32];
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    uint4 x = make_uint4(0u, 0u, 0u, 0u);
                    if (row_valid) x = *reinterpret_cast<const uint4 *>(qrow + 2 * (c0 + c));
                    w[c] = x.x; w[c + 1] = x.y; w[c + 2] = x.z; w[c + 3] = x.w;
                }
                tmem_st32(tmem + lane_addr + kColQ + wg * (kHD / 4) + c0, w);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars->q_ready);
        }
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (uint32_t j = 0; j < n_tiles; ++j) {
            const int st = j & 1;
            ok = warp_all(mbar_wait(&bars->s_full, j & 1));
            if (!ok) break;
            tc_fence_after();
            const uint32_t s_addr = tmem + lane_addr + kColS;
            uint32_t raw[2][32];
            tmem_ld32(s_addr + wg * 64, raw[0]);
            tmem_ld32(s_addr + wg * 64 + 32, raw[1]);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&bars->s_read);        // this half of the score tile is in registers

            const uint32_t key0 = (tile_lo + j) * kBN + wg * 64;   // first key of this thread's half
            const bool need_mask = (key0 + 64 > abs_lo + 1) || (key0 < first) || (key0 + 64 > p.kv_valid_count);
            // masked keys become -inf before the scale (which is positive, so they stay -inf and the row
            // maximum can be taken on the unscaled scores, in four independent chains)
            if (need_mask) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const uint32_t key = key0 + h * 32 + c;
                        if (key < first || key >= last) raw[h][c] = 0xff800000u;
                    }
            }
            float mx4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(__uint_as_float(raw[0][u]), __uint_as_float(raw[1][u]));
#pragma unroll
            for (int c = 4; c < 32; ++c)
                mx4[c & 3] = fmaxf(mx4[c & 3], fmaxf(__uint_as_float(raw[0][c]), __uint_as_float(raw[1][c])));
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            bars->xchg[st][wg][row] = mx;
            ok = pair_sync();
            if (!ok) break;
            mx = fmaxf(mx, bars->xchg[st][wg ^ 1][row]);
            float m_new = fmaxf(m_ref, mx);
            // lazy rescale: keep the stale reference while it is within 2^8 of the true maximum
            const bool raise = (m_new - m_ref > kRescaleThreshold) || (m_ref == -INFINITY && m_new != -INFINITY);
            if (j == 0) {
                m_ref = m_new;
            } else if (__any_sync(0xffffffffu, raise)) {
                // O holds sum over tiles < j; it may only be touched once P.V of tile j-1 retired.
                // Both warps of the quarter see the same rows, hence the same votes: A rescales head-dim
                // columns 0..127, B columns 128..255.
                ok = warp_all(mbar_wait(&bars->o_ready, (j - 1) & 1));
                if (!ok) break;
                tc_fence_after();
                const float factor = raise ? fast_exp2(m_ref - m_new) : 1.f;   // exp2(-inf) == 0: O was all zero
                if (raise) { l_run *= factor; m_ref = m_new; }
#pragma unroll 1
                for (int c0 = 0; c0 < kHD / 2; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem + lane_addr + kColO + wg * (kHD / 2) + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                    tmem_st32(tmem + lane_addr + kColO + wg * (kHD / 2) + c0, o);
                }
                tmem_wait_st();
            }
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                // one FMA per exponent argument: raw * scale - m
                const float p0 = fast_exp2(fmaf(__uint_as_float(raw[c >> 4][(2 * c) & 31]), p.scale_log2, neg_m));
                const float p1 = fast_exp2(fmaf(__uint_as_float(raw[c >> 4][(2 * c + 1) & 31]), p.scale_log2, neg_m));
                pk[c] = pack2<T>(p0, p1);       // P takes V's type: A and B of one tcgen05.mma must share a format
                rs4[c & 3] += sum2<T>(pk[c]);   // the row sum uses the ROUNDED weights the MMA will see, so
                                                // O / l stays an exact convex combination of V rows (summing
                                                // before the rounding fails the 2e-3 bar on peaked rows, fp16 too)
            }
            l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            // P row of this query, keys 64*wg..: 128 bytes in sub-tile wg, 16-byte chunk c at (c ^ (row & 7));
            // stored once P.V of the previous tile has retired
            if (j >= 1) {
                ok = warp_all(mbar_wait(&bars->p_free, (j - 1) & 1));
                if (!ok) break;
            }
            unsigned char *prow = p_s + wg * kPSub + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4 *>(prow + ((c ^ (row & 7)) << 4)) =
                    make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();                 // orders a rescale of O (above) before the P.V it precedes
            mbar_arrive(&bars->p_ready);
        }
        if (ok) ok = mbar_wait(&bars->o_ready, (n_tiles - 1) & 1);
        ok = warp_all(ok);
        if (ok) ok = pair_sync();   // the partner is done reading the last tile's maxima
        if (ok) {                   // total row sum = the two halves
            bars->xchg[0][wg][row] = l_run;
            ok = pair_sync();
        }
        if (ok) {
            tc_fence_after();
            const float l_tot = l_run + bars->xchg[0][wg ^ 1][row];
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            T *orow = out + (size_t)(row0 + row) * p.o_token_stride + (size_t)head * kHD + wg * (kHD / 2);
#pragma unroll 1
            for (int c0 = 0; c0 < kHD / 2; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem + lane_addr + kColO + wg * (kHD / 2) + c0, o);
                tmem_wait_ld();
                if (row_valid) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        w.x = pack2<T>(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        w.y = pack2<T>(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        w.z = pack2<T>(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        w.w = pack2<T>(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        *reinterpret_cast<uint4 *>(orow + c0 + c) = w;
                    }
                }
            }
        }
        failed = !ok;
    }

    if (failed) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

}  // namespace

// 2-D map over [rows][width] 16-bit elements, rows `stride_elems` apart, box [box_rows][64].
bool tt_make_tensor_map_2d(CUtensorMap *map, const void *base, uint32_t io_dtype, uint64_t width, uint64_t rows,
              uint64_t stride_elems, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {width, rows};
    const cuuint64_t strides[1] = {stride_elems * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = io_dtype == TT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D map over 4-byte floats: [rows][width], rows `stride_bytes` apart, box [box_rows][32 floats].
bool tt_make_tensor_map_2d_f32(CUtensorMap *map, const void *base, uint64_t width, uint64_t rows,
                               uint64_t stride_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {width, rows};
    const cuuint64_t strides[1] = {stride_bytes};
    const cuuint32_t box[2] = {32, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int tt_launch_prefill_tc(tt_context *ctx, cudaStream_t stream, const void *q, const void *k, const void *v,
                         void *out, const tt_prefill_params *p, uint32_t io_dtype) {
    CUtensorMap k_map, v_map;
    const bool ok = tt_make_tensor_map_2d(&k_map, k, io_dtype, (uint64_t)p->n_kv_heads * kHD, p->kv_valid_count,
                             p->kv_token_stride_elements, kBox) &&
                    tt_make_tensor_map_2d(&v_map, v, io_dtype, (uint64_t)p->n_kv_heads * kHD, p->kv_valid_count,
                             p->kv_token_stride_elements, kBox);
    if (!ok) return tt_set_error(ctx, TT_ERR_CUDA, "cuTensorMapEncodeTiled failed for the prefill operands");
    PrefillTcParams kp;
    kp.start_position = p->start_position; kp.query_count = p->query_count; kp.n_q_heads = p->n_q_heads;
    kp.n_kv_heads = p->n_kv_heads; kp.kv_valid_count = p->kv_valid_count; kp.sliding_window = p->sliding_window;
    kp.o_token_stride = p->o_token_stride_elements;
    kp.q_token_stride = p->q_token_stride_elements;
    kp.n_q_tiles = (p->query_count + kBM - 1) / kBM;
    kp.scale_log2 = p->scale * kLog2e;
    kp.idesc_qk = tt_make_idesc_f16(io_dtype, kBN, false);
    kp.idesc_pv = tt_make_idesc_f16(io_dtype, kHD, true);
    const uint32_t grid = kp.n_q_tiles * p->n_q_heads;
    cudaError_t e;
    if (io_dtype == TT_F16) {
        auto kernel = attn_prefill_tc_kernel<__half>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "prefill smem attribute");
        kernel<<<grid, kThreads, kSmemBytes, stream>>>(reinterpret_cast<const __half *>(q), k_map, v_map, reinterpret_cast<__half *>(out), kp, ctx->status);
    } else {
        auto kernel = attn_prefill_tc_kernel<__nv_bfloat16>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "prefill smem attribute");
        kernel<<<grid, kThreads, kSmemBytes, stream>>>(reinterpret_cast<const __nv_bfloat16 *>(q), k_map, v_map, reinterpret_cast<__nv_bfloat16 *>(out), kp, ctx->status);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_prefill_tc launch");
    ctx->launches++;
    return TT_OK;
}
