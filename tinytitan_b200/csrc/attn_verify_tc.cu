// Few-token ("verify") decode attention on the sm_100a tensor cores, head_dim 256.
//
// With W draft rows and G query heads per KV head, W*G packed query rows (17..64) share every K/V
// row of a KV head. The mma.sync decode kernel serves 16 packed rows per pass and re-reads the key
// range for the rest; here one CTA computes all of them against each K/V row it streams, in the
// transposed form so that the 128-wide MMA dimension is filled by KEYS, not by padded query rows:
//
//   S^T[j%2] = K_j . Q^T          SS MMA  M128 (keys) N64 (rows) K16 x16    TMEM cols   0..127
//   P^T_j    = exp2(S^T - m)      tcgen05.ld -> registers -> shared memory (B operand, N-major)
//   O^T     += V_j^T . P^T_j      SS MMA  M128 (head-dim half) N64 K16 x8, twice   cols 128..255
//   l^T     += 1 . P^T_j          SS MMA  against ones: the row sums of the ROUNDED weights,
//                                 replicated over the lanes                         cols 256..319
//
// K streams as [128 keys][64 head-dim] chunks (one TMA box, 16 KB) through a 4-slot ring and is
// released chunk by chunk as its four MMAs retire; V streams as [128 keys][128 head-dim] blocks
// (two boxes, 32 KB) through a 3-slot ring, so the loads of the next tile's V are in flight while
// this tile's is consumed. Lanes 0 and 1 of warp 0 are the K and V producers, warp 1 issues the
// MMAs and owns TMEM, warps 2-5 (one thread per key of the tile) run the softmax. The per-row
// reference maximum lives in shared memory and is only raised when a score exceeds it by more than
// 2^8; the raise (rare after the first tile) rescales O^T and l^T in TMEM. Each CTA writes one
// unnormalised (m, l, o) partial per packed row, in the layout the split-KV combine kernel merges.
//
// Semantics: attention.metal:162-269 (partial pass over a key range, row r of a W-row group
// masked at seq_len - (W-1-r)); every mbarrier wait is bounded.
#include "tt_sm100.h"

#include <type_traits>

namespace {

constexpr int kHD = 256;
constexpr int kBK = 128;                   // keys per tile
constexpr int kRows = 64;                  // packed query rows (MMA N)
constexpr int kThreads = 192;
constexpr int kKSlots = 4, kVSlots = 3;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRaiseThreshold = 8.0f;

constexpr int kChunkBytes = kBK * 64 * 2;      // [128 keys][64 head-dim], 128-byte rows: 16384
constexpr int kVBlockBytes = 2 * kChunkBytes;  // [128 keys][128 head-dim]
constexpr int kQBytes = kRows * kHD * 2;       // 4 sub-tiles [64][64]
constexpr int kQSub = kRows * 64 * 2;          // 8192
constexpr int kPBytes = kBK * kRows * 2;       // [128 keys][64 rows], 128-byte rows
constexpr int kOnesBytes = 1024;               // one 8-row group of 1.0; every group of the operand aliases it
constexpr int kOffV = kKSlots * kChunkBytes;
constexpr int kOffQ = kOffV + kVSlots * kVBlockBytes;
constexpr int kOffP = kOffQ + kQBytes;
constexpr int kOffOnes = kOffP + kPBytes;
constexpr int kOffMisc = kOffOnes + kOnesBytes;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 128, kColL = 256;

struct Misc {
    uint64_t k_full[kKSlots], k_empty[kKSlots];
    uint64_t v_full[kVSlots], v_empty[kVSlots];
    uint64_t s_full[2];
    uint64_t p_ready, p_free;
    uint64_t o_ready;
    uint64_t sync;              // softmax warps' own barrier (count 4: one arrive per warp)
    uint32_t tmem_base;
    uint32_t pad;
    uint32_t raise_tile[2];     // [tile parity]: 1 + the last tile for which some key asked for higher maxima
    float mref[kRows];          // log2-domain reference maximum per packed row
    float factor[kRows];
    float tile_max[4][kRows];
    float lsum[kRows];
    uint32_t limit[kRows];      // first masked key per packed row
    uint32_t prow[kRows];       // partial row index per packed row
};
constexpr int kSmemBytes = kOffMisc + (int)sizeof(Misc) + 1024 /*align*/;

struct VerifyParams {
    const TTDecodeItem *items;
    const TTDecodeSession *sessions;
    const CUtensorMap *maps;     // [2 * session]: K map (box 128 x 64), V map (box 128 x 64)
    float *part_o, *part_m, *part_l;
    uint32_t n_q_heads, n_kv_heads, q_row_stride;
    uint32_t out_row_stride;     // elements
    uint32_t direct;             // every session is one part: write the normalised rows, no partials
    float scale_log2;
    uint32_t idesc_qk, idesc_pv, idesc_l;
};

// Barrier among the four softmax warps with a bounded wait (a named barrier could not give up if a
// warp left after a time-out): one arrive per warp, every lane waits. `phase` flips per use.
__device__ __forceinline__ bool softmax_sync(uint64_t *bar, uint32_t &phase, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    const bool ok = warp_all(mbar_wait(bar, phase & 1));
    phase ^= 1;
    return ok;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Column maxima over the warp: every lane holds one value for each of 64 columns; afterwards lane L
// holds the warp-wide maxima of columns 2L and 2L+1. Each butterfly step hands the partner the half
// of the columns it keeps, so the whole reduction is 62 shuffles instead of 320.
__device__ __forceinline__ void warp_colmax64(const uint32_t (&v)[2][32], int lane, float &m0, float &m1) {
    float a[32], b[16], c[8], d[4];
    bool up = (lane & 16) != 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float lo = __uint_as_float(v[0][i]), hi = __uint_as_float(v[1][i]);
        a[i] = fmaxf(up ? hi : lo, __shfl_xor_sync(0xffffffffu, up ? lo : hi, 16));
    }
    up = (lane & 8) != 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) b[i] = fmaxf(up ? a[i + 16] : a[i], __shfl_xor_sync(0xffffffffu, up ? a[i] : a[i + 16], 8));
    up = (lane & 4) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = fmaxf(up ? b[i + 8] : b[i], __shfl_xor_sync(0xffffffffu, up ? b[i] : b[i + 8], 4));
    up = (lane & 2) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = fmaxf(up ? c[i + 4] : c[i], __shfl_xor_sync(0xffffffffu, up ? c[i] : c[i + 4], 2));
    up = (lane & 1) != 0;
    m0 = fmaxf(up ? d[2] : d[0], __shfl_xor_sync(0xffffffffu, up ? d[0] : d[2], 1));
    m1 = fmaxf(up ? d[3] : d[1], __shfl_xor_sync(0xffffffffu, up ? d[1] : d[3], 1));
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) attn_verify_tc_kernel(VerifyParams p, uint32_t *__restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *k_ring = smem;
    unsigned char *v_ring = smem + kOffV;
    unsigned char *q_s = smem + kOffQ;
    unsigned char *p_s = smem + kOffP;
    unsigned char *ones_s = smem + kOffOnes;
    Misc *ms = reinterpret_cast<Misc *>(smem + kOffMisc);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TTDecodeItem item = p.items[blockIdx.x];
    const TTDecodeSession ses = p.sessions[item.session];
    const uint32_t group = p.n_q_heads / p.n_kv_heads;
    const uint32_t n_rows = ses.q_rows * group;                    // packed rows in use (<= 64)
    const uint32_t n_tiles = (item.key_end - item.key_begin + kBK - 1) / kBK;
    const uint32_t rows_total = ses.q_rows * p.n_q_heads;

    // K chunk kc = 4*tile + (64-wide head-dim slice); V block vb = 2*tile + head-dim half
    const CUtensorMap *k_map = p.maps + 2 * item.session, *v_map = k_map + 1;
    const uint32_t n_kchunks = 4 * n_tiles, n_vblocks = 2 * n_tiles;
    auto load_k = [&](uint32_t kc) {
        const uint32_t slot = kc % kKSlots;
        mbar_expect_tx(&ms->k_full[slot], kChunkBytes);
        tma_load_2d(k_ring + slot * kChunkBytes, k_map, (int)(item.kv_head * kHD + (kc & 3) * 64),
                    (int)(item.key_begin + (kc >> 2) * kBK), &ms->k_full[slot]);
    };
    auto load_v = [&](uint32_t vb) {
        const uint32_t slot = vb % kVSlots;
        mbar_expect_tx(&ms->v_full[slot], kVBlockBytes);
        const int x = (int)(item.kv_head * kHD + (vb & 1) * 128), y = (int)(item.key_begin + (vb >> 1) * kBK);
        tma_load_2d(v_ring + slot * kVBlockBytes, v_map, x, y, &ms->v_full[slot]);
        tma_load_2d(v_ring + slot * kVBlockBytes + kChunkBytes, v_map, x + 64, y, &ms->v_full[slot]);
    };
    // The first ring fills leave before the CTA-wide sync so that they overlap the staging of Q (the
    // thread that initialises the barriers is the one that uses them first).
    if (threadIdx.x == 0) {
        for (int s = 0; s < kKSlots; ++s) { mbar_init(&ms->k_full[s], 1); mbar_init(&ms->k_empty[s], 1); }
        for (int s = 0; s < kVSlots; ++s) { mbar_init(&ms->v_full[s], 1); mbar_init(&ms->v_empty[s], 1); }
        mbar_init(&ms->s_full[0], 1); mbar_init(&ms->s_full[1], 1);
        mbar_init(&ms->p_ready, 128);
        mbar_init(&ms->p_free, 1);
        mbar_init(&ms->o_ready, 1);
        mbar_init(&ms->sync, 4);
        ms->raise_tile[0] = 0; ms->raise_tile[1] = 0;
        mbar_fence_init();
        if (n_tiles > 0) {
            // the maps were rewritten by a host copy since the last launch that used these addresses
            asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(k_map) : "memory");
            asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(v_map) : "memory");
            for (uint32_t kc = 0; kc < (uint32_t)kKSlots && kc < n_kchunks; ++kc) load_k(kc);
            for (uint32_t vb = 0; vb < (uint32_t)kVSlots && vb < n_vblocks; ++vb) load_v(vb);
        }
    }
    if (warp == 1) tmem_alloc(&ms->tmem_base, kTmemCols);

    // ---- stage Q^T's operand: packed row r = w*G + g -> q[w][kv_head*G + g][:], K-major, 128-byte
    // swizzle; asynchronous 16-byte copies so that all of a thread's chunks are in flight together
    if (warp != 0) {
        const T *q = reinterpret_cast<const T *>(ses.q);
        for (uint32_t c = threadIdx.x - 32; c < kRows * (kHD / 8); c += kThreads - 32) {
            const uint32_t r = c / (kHD / 8), chunk = c % (kHD / 8);       // 16-byte chunk of the row
            const uint32_t sub = chunk >> 3, cc = chunk & 7;
            unsigned char *dst = q_s + sub * kQSub + r * 128 + ((cc ^ (r & 7)) << 4);
            if (r < n_rows) {
                const uint32_t w = r / group, g = r - w * group;
                const T *src = q + (size_t)w * p.q_row_stride + (size_t)(item.kv_head * group + g) * kHD + chunk * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
            } else {
                *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        const uint32_t one2 = std::is_same<T, __half>::value ? 0x3C003C00u : 0x3F803F80u;   // 1.0 twice
        for (uint32_t c = threadIdx.x - 32; c < kOnesBytes / 16; c += kThreads - 32)
            *reinterpret_cast<uint4 *>(ones_s + c * 16) = make_uint4(one2, one2, one2, one2);
        for (uint32_t r = threadIdx.x - 32; r < kRows; r += kThreads - 32) {
            const uint32_t w = r / group, g = r - w * group;
            ms->mref[r] = -INFINITY;
            ms->factor[r] = 1.f;
            ms->limit[r] = r < n_rows ? ses.seq_len - (ses.q_rows - 1 - w) : 0u;
            const uint32_t rho = w * p.n_q_heads + item.kv_head * group + g;
            ms->prow[r] = item.partial_base + item.part_index * rows_total + rho;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ms->tmem_base;
    bool failed = false;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producers
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kc = kKSlots; ok && kc < n_kchunks; ++kc) {
                ok = mbar_wait(&ms->k_empty[kc % kKSlots], ((kc / kKSlots) - 1) & 1);
                if (ok) load_k(kc);
            }
            failed = !ok;
        } else if (lane == 1) {
            bool ok = true;
            for (uint32_t vb = kVSlots; ok && vb < n_vblocks; ++vb) {
                ok = mbar_wait(&ms->v_empty[vb % kVSlots], ((vb / kVSlots) - 1) & 1);
                if (ok) load_v(vb);
            }
            failed = !ok;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_tiles > 0) {
            const uint32_t k_a = smem_u32(k_ring), v_a = smem_u32(v_ring), q_a = smem_u32(q_s), p_a = smem_u32(p_s),
                           ones_a = smem_u32(ones_s);
            // S^T(j) = K_j . Q^T, one 64-wide head-dim slice at a time as the chunks land
            auto issue_qk = [&](uint32_t j) {
                const uint32_t d = tmem + kColS + (j & 1) * kRows;
                for (uint32_t c = 0; c < 4; ++c) {
                    const uint32_t kc = 4 * j + c, slot = kc % kKSlots;
                    if (!mbar_wait(&ms->k_full[slot], (kc / kKSlots) & 1)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t ad = make_desc(k_a + slot * kChunkBytes + ks * 32, 16, 1024);
                        const uint64_t bd = make_desc(q_a + c * kQSub + ks * 32, 16, 1024);
                        mma_ss(d, ad, bd, p.idesc_qk, (c > 0 || ks > 0) ? 1u : 0u);
                    }
                    mma_commit(&ms->k_empty[slot]);
                }
                mma_commit(&ms->s_full[j & 1]);
                return true;
            };
            bool ok = issue_qk(0);
            for (uint32_t j = 0; ok && j < n_tiles; ++j) {
                if (j + 1 < n_tiles) ok = issue_qk(j + 1);
                if (ok) ok = mbar_wait(&ms->p_ready, j & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc0 = j > 0 ? 1u : 0u;
                // l^T += 1 . P^T_j: every 8-row group of the A operand is the same 1 KB of ones (SBO 0)
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk) {
                    const uint64_t ad = make_desc(ones_a + (kk & 3) * 32, 16, 0);
                    const uint64_t bd = make_desc(p_a + kk * 2048, kPBytes, 1024);
                    mma_ss(tmem + kColL, ad, bd, p.idesc_l, (acc0 || kk > 0) ? 1u : 0u);
                }
                // O^T(half) += V_j(half)^T . P^T_j
                for (uint32_t half = 0; ok && half < 2; ++half) {
                    const uint32_t vb = 2 * j + half, slot = vb % kVSlots;
                    ok = mbar_wait(&ms->v_full[slot], (vb / kVSlots) & 1);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        // V block as the M-major A operand: 64-wide head-dim atoms kChunkBytes apart (LBO),
                        // 8-key groups 1024 B apart (SBO); P^T as the N-major B operand, one atom wide
                        const uint64_t ad = make_desc(v_a + slot * kVBlockBytes + kk * 2048, kChunkBytes, 1024);
                        const uint64_t bd = make_desc(p_a + kk * 2048, kPBytes, 1024);
                        mma_ss(tmem + kColO + half * kRows, ad, bd, p.idesc_pv, (acc0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&ms->v_empty[slot]);
                }
                if (!ok) break;
                mma_commit(&ms->p_free);
                mma_commit(&ms->o_ready);
            }
            failed = !ok;
        }
    } else {
        // ------------------------------------------------------------------ softmax: one key per thread
        const uint32_t quarter = warp & 3;                       // TMEM lane quarter this warp may touch
        const uint32_t i = quarter * 32 + lane;                  // key inside the tile == TMEM lane
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t min_limit = 0xffffffffu;
        for (uint32_t r = 0; r < n_rows; r += group) min_limit = min(min_limit, ms->limit[r]);
        bool ok = true;
        uint32_t sync_phase = 0;

        for (uint32_t j = 0; j < n_tiles; ++j) {
            const uint32_t st = j & 1;
            ok = warp_all(mbar_wait(&ms->s_full[st], (j >> 1) & 1));
            if (!ok) break;
            tc_fence_after();
            uint32_t raw[2][32];
            tmem_ld32(tmem + lane_addr + kColS + st * kRows, raw[0]);
            tmem_ld32(tmem + lane_addr + kColS + st * kRows + 32, raw[1]);
            tmem_wait_ld();

            const uint32_t key0 = item.key_begin + j * kBK, key = key0 + i;
            const bool need_mask = key0 + kBK > min_limit || key0 + kBK > item.key_end;
            bool exceed = false;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    const float4 m4 = *reinterpret_cast<const float4 *>(&ms->mref[h * 32 + c]);
                    const float mm[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float s = __uint_as_float(raw[h][c + u]) * p.scale_log2;
                        if (need_mask && (key >= ms->limit[h * 32 + c + u] || key >= item.key_end)) s = -INFINITY;
                        raw[h][c + u] = __float_as_uint(s);
                        exceed |= (s - mm[u]) > kRaiseThreshold;     // -inf - -inf is NaN: compares false
                    }
                }

            if (__any_sync(0xffffffffu, exceed) && lane == 0) atomicMax(&ms->raise_tile[st], j + 1);
            ok = softmax_sync(&ms->sync, sync_phase, lane);
            if (!ok) break;
            if (ms->raise_tile[st] == j + 1) {
                // raise the reference maxima to the true maxima so far, rescale what is accumulated
                float m0, m1;
                warp_colmax64(raw, lane, m0, m1);
                *reinterpret_cast<float2 *>(&ms->tile_max[quarter][2 * lane]) = make_float2(m0, m1);
                ok = softmax_sync(&ms->sync, sync_phase, lane);
                if (!ok) break;
                if (i < kRows) {
                    const float m_old = ms->mref[i];
                    const float tm = fmaxf(fmaxf(ms->tile_max[0][i], ms->tile_max[1][i]),
                                           fmaxf(ms->tile_max[2][i], ms->tile_max[3][i]));
                    const float m_new = fmaxf(m_old, tm);
                    ms->factor[i] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_old - m_new);   // exp2(-inf) == 0
                    ms->mref[i] = m_new;
                }
                ok = softmax_sync(&ms->sync, sync_phase, lane);
                if (!ok) break;
                if (j > 0) {
                    // everything accumulated so far must have retired before it is touched
                    ok = warp_all(mbar_wait(&ms->o_ready, (j - 1) & 1));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (uint32_t c0 = kColO; c0 < kColL + kRows; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem + lane_addr + c0, o);
                        tmem_wait_ld();
                        const float *f = &ms->factor[c0 & 63];      // columns repeat every 64: O lo, O hi, l
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f[c]);
                        tmem_st32(tmem + lane_addr + c0, o);
                    }
                    tmem_wait_st();
                }
            }

            // P^T row of this key: 64 weights -> 128 bytes, chunk c at (c ^ (key & 7)); the exponentials are
            // formed first, the single P buffer is only waited for when they are ready to be stored
            uint4 w[8];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    const float4 ma = *reinterpret_cast<const float4 *>(&ms->mref[h * 32 + c]);
                    const float4 mb = *reinterpret_cast<const float4 *>(&ms->mref[h * 32 + c + 4]);
                    const float mm[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
                    float e[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float m_use = (mm[u] == -INFINITY) ? 0.f : mm[u];
                        e[u] = fast_exp2(__uint_as_float(raw[h][c + u]) - m_use);
                    }
                    uint4 &o = w[h * 4 + (c >> 3)];
                    o.x = pack2<T>(e[0], e[1]); o.y = pack2<T>(e[2], e[3]);
                    o.z = pack2<T>(e[4], e[5]); o.w = pack2<T>(e[6], e[7]);
                }
            if (j >= 1) {
                ok = warp_all(mbar_wait(&ms->p_free, (j - 1) & 1));
                if (!ok) break;
            }
            unsigned char *prow = p_s + i * 128;
#pragma unroll
            for (uint32_t chunk = 0; chunk < 8; ++chunk)
                *reinterpret_cast<uint4 *>(prow + ((chunk ^ (i & 7)) << 4)) = w[chunk];
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(&ms->p_ready);
        }

        // ---- partial of this item: O^T (transposed back on the way out), m, l
        if (ok && n_tiles > 0) ok = warp_all(mbar_wait(&ms->o_ready, (n_tiles - 1) & 1));
        if (ok) {
            tc_fence_after();
            if (n_tiles > 0 && quarter == 0) {   // every lane of l^T holds the 64 sums; the load is warp-wide
                uint32_t l0[32], l1[32];
                tmem_ld32(tmem + lane_addr + kColL, l0);
                tmem_ld32(tmem + lane_addr + kColL + 32, l1);
                tmem_wait_ld();
                if (lane == 0) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) { ms->lsum[c] = __uint_as_float(l0[c]); ms->lsum[32 + c] = __uint_as_float(l1[c]); }
                }
            }
            ok = softmax_sync(&ms->sync, sync_phase, lane);
        }
        if (ok && p.direct) {
            // the item covers the session's whole key range: normalise and store the output rows
            T *out = reinterpret_cast<T *>(ses.out);
#pragma unroll 1
            for (uint32_t half = 0; half < 2; ++half) {
                uint32_t o0[32], o1[32];
                if (n_tiles > 0) {
                    tmem_ld32(tmem + lane_addr + kColO + half * kRows, o0);
                    tmem_ld32(tmem + lane_addr + kColO + half * kRows + 32, o1);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) { o0[c] = 0u; o1[c] = 0u; }
                }
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    if ((uint32_t)c < n_rows) {
                        const float l = n_tiles > 0 ? ms->lsum[c] : 0.f;
                        const float inv = l > 0.f ? 1.f / l : 0.f;          // no visible key: zeros
                        const uint32_t w = (uint32_t)c / group, g = (uint32_t)c - w * group;
                        const float v = __uint_as_float(c < 32 ? o0[c & 31] : o1[c & 31]) * inv;
                        out[(size_t)w * p.out_row_stride + (size_t)(item.kv_head * group + g) * kHD + half * 128 + i] = (T)v;
                    }
                }
            }
        } else if (ok) {
            if (i < n_rows) {
                const float m = ms->mref[i];
                p.part_m[ms->prow[i]] = n_tiles > 0 ? m * kLn2 : -INFINITY;   // natural-log domain
                p.part_l[ms->prow[i]] = (n_tiles > 0 && m != -INFINITY) ? ms->lsum[i] : 0.f;
            }
#pragma unroll 1
            for (uint32_t half = 0; half < 2; ++half) {
                uint32_t o0[32], o1[32];
                if (n_tiles > 0) {
                    tmem_ld32(tmem + lane_addr + kColO + half * kRows, o0);
                    tmem_ld32(tmem + lane_addr + kColO + half * kRows + 32, o1);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) { o0[c] = 0u; o1[c] = 0u; }
                }
                float *dst = p.part_o + half * 128 + i;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    if ((uint32_t)c < n_rows) dst[(size_t)ms->prow[c] * kHD] = __uint_as_float(o0[c]);
                    if ((uint32_t)(32 + c) < n_rows) dst[(size_t)ms->prow[32 + c] * kHD] = __uint_as_float(o1[c]);
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

}  // namespace

// One K and one V tensor map per session of a verify batch ([seq_len rows][n_kv_heads * 256], box
// 128 x 64, keys past seq_len read as zero), written into the staging table that the caller uploads
// together with the session and item tables.
int tt_verify_tc_encode_maps(tt_context *ctx, uint32_t n_sessions, const tt_attn_batch_params *p) {
    CUtensorMap *maps = reinterpret_cast<CUtensorMap *>(ctx->h_tensor_maps);
    for (uint32_t i = 0; i < n_sessions; ++i) {
        const TTDecodeSession &s = ctx->h_sessions[i];
        const uint64_t rows = s.seq_len > 0 ? s.seq_len : 1;
        const bool ok = tt_make_tensor_map_2d(&maps[2 * i], s.k, p->io_dtype, (uint64_t)p->n_kv_heads * kHD, rows,
                                              p->kv_token_stride_elements, kBK) &&
                        tt_make_tensor_map_2d(&maps[2 * i + 1], s.v, p->io_dtype, (uint64_t)p->n_kv_heads * kHD, rows,
                                              p->kv_token_stride_elements, kBK);
        if (!ok) return tt_set_error(ctx, TT_ERR_CUDA, "cuTensorMapEncodeTiled failed for session %u", i);
    }
    return TT_OK;
}

// Pass 1 of a verify batch on the tensor cores: the items (one per (session, kv head, key range), all
// packed rows at once), the sessions and the tensor maps are already on the device.
int tt_launch_verify_tc(tt_context *ctx, cudaStream_t stream, uint32_t n_sessions, uint32_t n_items, float *part_o,
                        float *part_m, float *part_l, const tt_attn_batch_params *p, bool direct) {
    (void)n_sessions;
    cudaError_t e;
    VerifyParams kp;
    kp.items = ctx->items; kp.sessions = ctx->sessions;
    kp.maps = reinterpret_cast<const CUtensorMap *>(ctx->tensor_maps);
    kp.part_o = part_o; kp.part_m = part_m; kp.part_l = part_l;
    kp.n_q_heads = p->n_q_heads; kp.n_kv_heads = p->n_kv_heads; kp.q_row_stride = p->q_row_stride_elements;
    kp.out_row_stride = p->out_row_stride_elements; kp.direct = direct ? 1u : 0u;
    kp.scale_log2 = p->scale * kLog2e;
    kp.idesc_qk = tt_make_idesc_f16(p->io_dtype, kRows, false, false);
    kp.idesc_pv = tt_make_idesc_f16(p->io_dtype, kRows, true, true);
    kp.idesc_l = tt_make_idesc_f16(p->io_dtype, kRows, true, false);
    if (p->io_dtype == TT_F16) {
        auto kernel = attn_verify_tc_kernel<__half>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "verify smem attribute");
        kernel<<<n_items, kThreads, kSmemBytes, stream>>>(kp, ctx->status);
    } else {
        auto kernel = attn_verify_tc_kernel<__nv_bfloat16>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "verify smem attribute");
        kernel<<<n_items, kThreads, kSmemBytes, stream>>>(kp, ctx->status);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_verify_tc launch");
    return TT_OK;
}
