// Few-token ("verify") decode attention on the sm_100a tensor cores, head_dim 256.
//
// With W draft rows and G query heads per KV head, W*G packed query rows (17..128) share every K/V
// row of a KV head. The mma.sync decode kernel serves 16 packed rows per pass and re-reads the key
// range for the rest; here one CTA computes all of them against each K/V row it streams. A packed
// row is a TMEM lane, so a softmax thread owns a whole row of the score tile and nothing of the
// softmax crosses threads:
//
//   S[j%2]  = Q . K_j^T        SS MMA  M128 N128 (keys) K16 x16    TMEM columns   0..255 (two tiles)
//   P_j     = exp2(S - m)      tcgen05.ld -> registers -> tcgen05.st over the first 64 columns of the
//                              same score tile (two 16-bit weights per column)
//   O      += P_j . V_j        TS MMA  M128 N128 (head-dim half) K16 x8, twice      columns 256..511
//
// Two geometries. Up to 64 packed rows: only those rows exist; the M128 instructions read rows 64..127
// of the Q operand from whatever follows Q in shared memory and leave the result in TMEM lanes
// 64..127, which nothing reads. Keeping Q as the only resident operand in shared memory (32 KB) and
// P in TMEM leaves 192 KB for ONE ring of twelve 16 KB slots that K ([128 keys][64 head-dim] chunks)
// and V (the same boxes, consumed in adjacent pairs) travel through in the order the MMAs consume
// them: K(0) K(1) V(0) K(2) V(1) ... The kernel is bound by the bytes it keeps in flight per SM, and
// this ring holds a tile and a half more than separate K and V rings next to a P buffer did.
// 65..128 packed rows: Q takes 64 KB, the ring ten slots, and four softmax warps own the 128 lanes.
//
// One softmax warp per 32 packed rows (row = thread), then the producer warp (lane 0 issues the TMA
// loads; the warp owns the TMEM allocation) and the MMA warp (lane 0 issues). The reference maximum
// of a row is only raised when a score exceeds it by more than 2^8; the raise rescales the row of O
// in TMEM (after P.V of the previous tile has retired). The row sum is taken on the ROUNDED weights.
// Each CTA writes one unnormalised (m, l, o) partial per packed row, in the layout the split-KV
// combine kernel merges, or the finished rows when its item is the whole key range of the session.
//
// Semantics: attention.metal:162-269 (partial pass over a key range, row r of a W-row group
// masked at seq_len - (W-1-r)); every mbarrier wait is bounded.
#include "tt_sm100.h"

#include <type_traits>

namespace {

constexpr int kHD = 256;
constexpr int kBK = 128;                   // keys per tile
constexpr int kMaxSlots = 12;
constexpr int kUnitsPerTile = 8;           // 4 K chunks + 4 V chunks
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRaiseThreshold = 8.0f;

constexpr int kSlotBytes = kBK * 64 * 2;       // [128 keys][64 head-dim], 128-byte rows: 16384
// Geometry for ROWS packed query rows (64 or 128): one softmax warp per 32 rows, then the producer warp
// and the MMA warp; Q and the ring share the shared memory, so 128 rows leave ten slots instead of twelve.
template <int ROWS>
struct VerifyGeom {
    static constexpr int kSoftmaxWarps = ROWS / 32;
    static constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1;
    static constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
    static constexpr int kSlots = ROWS == 64 ? 12 : 10;        // even: a V pair never wraps
    static constexpr int kQBytes = ROWS * kHD * 2;             // 4 sub-tiles [ROWS][64 head-dim]
    static constexpr int kQSub = ROWS * 64 * 2;
    static constexpr int kOffRing = kQBytes;
    static constexpr int kOffMisc = kOffRing + kSlots * kSlotBytes;
};

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;     // S: two tiles of 128 columns

struct Misc {
    uint64_t full[kMaxSlots], empty[kMaxSlots];
    uint64_t s_full[2];
    uint64_t p_ready[2];        // count 2: one arrive per softmax warp
    uint64_t o_ready[2];        // [tile parity]: P.V of the tile has retired. Two barriers, because the softmax threads
                                // may be two P.V products ahead of the tensor pipe when they reach the epilogue and
                                // a single barrier's parity cannot tell tile n-1 from tile n-3
    uint32_t tmem_base;
    uint32_t pad;
};
template <int ROWS>
constexpr int verify_smem_bytes() { return VerifyGeom<ROWS>::kOffMisc + (int)sizeof(Misc) + 1024 /*align*/; }
static_assert(verify_smem_bytes<64>() <= 232448 && verify_smem_bytes<128>() <= 232448,
              "the verify kernel's shared memory exceeds the per-CTA limit");

struct VerifyParams {
    const TTDecodeItem *items;
    const TTDecodeSession *sessions;
    const CUtensorMap *maps;     // [2 * session]: K map (box 128 x 64), V map (box 128 x 64)
    float *part_o, *part_m, *part_l;
    uint32_t n_q_heads, n_kv_heads, q_row_stride;
    uint32_t out_row_stride;     // elements
    uint32_t direct;             // every session is one part: write the normalised rows, no partials
    float scale_log2;
    uint32_t idesc_qk, idesc_pv;
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Up to kVerifyParamSessions sessions travel in the kernel parameters together with their tensor maps
// (table.n != 0): nothing is uploaded before the launch, a CTA derives its item from the block index,
// and the maps need no proxy fence. Larger batches read the tables the host copied to device memory.
template <typename T, int ROWS>
__global__ void __launch_bounds__(VerifyGeom<ROWS>::kThreads, 1)
attn_verify_tc_kernel(VerifyParams p, uint32_t *__restrict__ status, const __grid_constant__ TTSessionTable table,
                      const __grid_constant__ TTVerifyMaps pmaps) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *q_s = smem;
    using G = VerifyGeom<ROWS>;
    constexpr int kSlots = G::kSlots, kThreads = G::kThreads, kQSub = G::kQSub;
    unsigned char *ring = smem + G::kOffRing;
    Misc *ms = reinterpret_cast<Misc *>(smem + G::kOffMisc);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();       // the kernel before this one may have produced the query rows or the newest K/V rows
    TTDecodeItem item;
    TTDecodeSession ses;
    const bool in_params = table.n != 0;
    if (in_params) {
        uint32_t i = 0;
        while (i + 1 < table.n && table.item_prefix[i + 1] <= blockIdx.x) ++i;
        ses = table.s[i];
        const uint32_t local = blockIdx.x - table.item_prefix[i];
        const uint32_t part = local / p.n_kv_heads;
        const uint32_t keys = ses.seq_len > ses.kv_start ? ses.seq_len - ses.kv_start : 0u;
        const uint32_t len = ((keys + ses.n_parts - 1) / ses.n_parts + 127) / 128 * 128;   // the host planner's part length
        item.session = i;
        item.kv_head = local - part * p.n_kv_heads;
        item.key_begin = ses.kv_start + part * len;
        item.key_end = min(ses.seq_len, item.key_begin + len);
        if (item.key_end < item.key_begin) item.key_end = item.key_begin;
        item.part_index = part;
        item.partial_base = ses.partial_base;
    } else {
        item = p.items[blockIdx.x];
        ses = p.sessions[item.session];
    }
    const uint32_t group = p.n_q_heads / p.n_kv_heads;
    const uint32_t n_rows = ses.q_rows * group;                    // packed rows in use (<= ROWS)
    const uint32_t n_tiles = (item.key_end - item.key_begin + kBK - 1) / kBK;
    const uint32_t rows_total = ses.q_rows * p.n_q_heads;

    // Ring unit u (16 KB) in consumption order: K(0) | K(1) V(0) | K(2) V(1) | ... | V(n-1), four units each.
    const CUtensorMap *k_map = in_params ? reinterpret_cast<const CUtensorMap *>(pmaps.m[2 * item.session])
                                         : p.maps + 2 * item.session;
    const CUtensorMap *v_map = k_map + 1;
    const uint32_t n_units = kUnitsPerTile * n_tiles;
    auto load_unit = [&](uint32_t u) {
        // block of four: 0 -> K(0); odd 2t+1 -> K(t+1) (while it exists); even 2t+2 -> V(t); the last block is V(n-1)
        const uint32_t blk = u >> 2, c = u & 3;
        bool is_k; uint32_t tile;
        if (blk == 0) { is_k = true; tile = 0; }
        else if (blk == 2 * n_tiles - 1) { is_k = false; tile = n_tiles - 1; }
        else if (blk & 1) { is_k = true; tile = (blk + 1) >> 1; }
        else { is_k = false; tile = (blk >> 1) - 1; }
        const uint32_t slot = u % kSlots;
        mbar_expect_tx(&ms->full[slot], kSlotBytes);
        tma_load_2d(ring + slot * kSlotBytes, is_k ? k_map : v_map, (int)(item.kv_head * kHD + c * 64),
                    (int)(item.key_begin + tile * kBK), &ms->full[slot]);
    };
    // ---- stage Q: packed row r = w*G + g -> q[w][kv_head*G + g][:], K-major, 128-byte swizzle;
    // asynchronous 16-byte copies so that all of a thread's chunks are in flight together, issued
    // ahead of the ring fill because the first product waits for Q as well as for K(0)
    {
        const T *q = reinterpret_cast<const T *>(ses.q);
        for (uint32_t c = threadIdx.x; c < ROWS * (kHD / 8); c += kThreads) {
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
    }
    // The first ring fill leaves before the CTA-wide sync so that it overlaps the arrival of Q (the
    // thread that initialises the barriers is the one that uses them first).
    if (threadIdx.x == G::kProducerWarp * 32) {
        for (int s = 0; s < kSlots; ++s) { mbar_init(&ms->full[s], 1); mbar_init(&ms->empty[s], 1); }
        mbar_init(&ms->s_full[0], 1); mbar_init(&ms->s_full[1], 1);
        mbar_init(&ms->p_ready[0], G::kSoftmaxWarps); mbar_init(&ms->p_ready[1], G::kSoftmaxWarps);
        mbar_init(&ms->o_ready[0], 1); mbar_init(&ms->o_ready[1], 1);
        mbar_fence_init();
        if (n_tiles > 0) {
            if (!in_params) {
                // the maps were rewritten by a host copy since the last launch that used these addresses
                asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(k_map) : "memory");
                asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(v_map) : "memory");
            }
            for (uint32_t u = 0; u < (uint32_t)kSlots && u < n_units; ++u) load_unit(u);
        }
    }
    if (warp == G::kProducerWarp) {
        __syncwarp();
        tmem_alloc(&ms->tmem_base, kTmemCols);
    }

    asm volatile("cp.async.wait_group 0;" ::: "memory");
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ms->tmem_base;
    bool failed = false;

    if (warp == G::kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            uint32_t u = kSlots;
            for (; ok && u < n_units; ++u) {
                ok = mbar_wait(&ms->empty[u % kSlots], ((u / kSlots) - 1) & 1);
                if (ok) load_unit(u);
            }
            if (!ok) {
                // give the copies still in flight a bounded chance to land before the shared memory is released
                --u;
                for (uint32_t v = u > (uint32_t)kSlots ? u - kSlots : 0; v < u; ++v)
                    mbar_wait(&ms->full[v % kSlots], (v / kSlots) & 1, 1u << 16);
            }
            failed = !ok;
        }
    } else if (warp == G::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_tiles > 0) {
            const uint32_t ring_a = smem_u32(ring), q_a = smem_u32(q_s);
            uint32_t u = 0;
            // S(j) = Q . K_j^T, one 64-wide head-dim chunk at a time as the chunks land
            auto issue_qk = [&](uint32_t j) {
                const uint32_t d = tmem + kColS + (j & 1) * kBK;
                for (uint32_t c = 0; c < 4; ++c, ++u) {
                    const uint32_t slot = u % kSlots;
                    if (!mbar_wait(&ms->full[slot], (u / kSlots) & 1)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t ad = make_desc(q_a + c * kQSub + ks * 32, 16, 1024);
                        const uint64_t bd = make_desc(ring_a + slot * kSlotBytes + ks * 32, 16, 1024);
                        mma_ss(d, ad, bd, p.idesc_qk, (c > 0 || ks > 0) ? 1u : 0u);
                    }
                    mma_commit(&ms->empty[slot]);
                }
                mma_commit(&ms->s_full[j & 1]);
                return true;
            };
            bool ok = issue_qk(0);
            for (uint32_t j = 0; ok && j < n_tiles; ++j) {
                if (j + 1 < n_tiles) ok = issue_qk(j + 1);
                if (ok) ok = mbar_wait(&ms->p_ready[j & 1], (j >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t p_t = tmem + kColS + (j & 1) * kBK;    // P_j: 64 columns of 16-bit pairs over S_j
                // O(half) += P_j . V_j(half): V as the MN-major B operand, two 64-wide head-dim atoms one
                // slot apart (LBO), 8-key groups 1024 B apart (SBO), 16 keys (2048 B) per step
                for (uint32_t half = 0; ok && half < 2; ++half, u += 2) {
                    const uint32_t slot = u % kSlots;
                    ok = mbar_wait(&ms->full[slot], (u / kSlots) & 1) && mbar_wait(&ms->full[slot + 1], (u / kSlots) & 1);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        const uint64_t bd = make_desc(ring_a + slot * kSlotBytes + kk * 2048, kSlotBytes, 1024);
                        mma_ts(tmem + kColO + half * 128, p_t + kk * 8, bd, p.idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&ms->empty[slot]);
                    mma_commit(&ms->empty[slot + 1]);
                }
                if (!ok) break;
                mma_commit(&ms->o_ready[j & 1]);
            }
            failed = !ok;
        }
    } else {
        // ------------------------------------------------------------------ softmax: one packed row per thread
        const uint32_t row = warp * 32 + lane;                   // packed row == TMEM lane
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const bool row_valid = row < n_rows;
        const uint32_t w_idx = row / group, g_idx = row - w_idx * group;
        // first key this row may not see: its causal limit inside the draft rows, cut at the item's end
        const uint32_t lim = row_valid ? min(ses.seq_len - (ses.q_rows - 1 - w_idx), item.key_end) : 0u;
        float m_ref = -INFINITY, l_run = 0.f;                    // log2-domain reference maximum, running row sum
        bool ok = true;

        for (uint32_t j = 0; j < n_tiles; ++j) {
            const uint32_t st = j & 1;
            ok = warp_all(mbar_wait(&ms->s_full[st], (j >> 1) & 1));
            if (!ok) break;
            tc_fence_after();
            const uint32_t s_addr = tmem + lane_addr + kColS + st * kBK;
            uint32_t raw[4][32];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) tmem_ld32(s_addr + c4 * 32, raw[c4]);
            tmem_wait_ld();

            const uint32_t key0 = item.key_begin + j * kBK;
            if (key0 + kBK > lim) {          // masked keys become -inf before the (positive) scale
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4)
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (key0 + c4 * 32 + c >= lim) raw[c4][c] = 0xff800000u;
            }
            float mx4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(__uint_as_float(raw[0][u]), __uint_as_float(raw[1][u]));
#pragma unroll
            for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], fmaxf(__uint_as_float(raw[2][u]), __uint_as_float(raw[3][u])));
#pragma unroll
            for (int c = 4; c < 32; ++c)
                mx4[c & 3] = fmaxf(mx4[c & 3], fmaxf(fmaxf(__uint_as_float(raw[0][c]), __uint_as_float(raw[1][c])),
                                                     fmaxf(__uint_as_float(raw[2][c]), __uint_as_float(raw[3][c]))));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            const float m_new = fmaxf(m_ref, mx);
            // lazy rescale: keep the stale reference while it is within 2^8 of the true maximum
            const bool raise = (m_new - m_ref > kRaiseThreshold) || (m_ref == -INFINITY && m_new != -INFINITY);
            if (j == 0) {
                m_ref = m_new;
            } else if (__any_sync(0xffffffffu, raise)) {
                // O holds the sum over tiles < j; it may only be touched once P.V of tile j-1 has retired
                ok = warp_all(mbar_wait(&ms->o_ready[(j - 1) & 1], ((j - 1) >> 1) & 1));
                if (!ok) break;
                tc_fence_after();
                const float factor = raise ? fast_exp2(m_ref - m_new) : 1.f;   // exp2(-inf) == 0: the row of O was zero
                if (raise) { l_run *= factor; m_ref = m_new; }
#pragma unroll 1
                for (int c0 = 0; c0 < kHD; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem + lane_addr + kColO + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                    tmem_st32(tmem + lane_addr + kColO + c0, o);
                }
            }
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    // one FMA per exponent argument: raw * scale - m
                    const float p0 = fast_exp2(fmaf(__uint_as_float(raw[c4][2 * c]), p.scale_log2, neg_m));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(raw[c4][2 * c + 1]), p.scale_log2, neg_m));
                    pk[c] = pack2<T>(p0, p1);       // P takes V's type: A and B of one tcgen05.mma share a format
                    rs4[c & 3] += sum2<T>(pk[c]);   // the row sum uses the ROUNDED weights the MMA will see
                }
                // keys 32*c4 .. 32*c4+31 of the row -> columns 16*c4 .. of the score tile they came from (every
                // column written here has been read above)
                tmem_st16(s_addr + c4 * 16, pk);
            }
            l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            tmem_wait_st();
            tc_fence_before();                 // orders P and a rescale of O before the P.V they precede
            __syncwarp();
            if (lane == 0) mbar_arrive(&ms->p_ready[st]);
        }

        // ---- this item's rows: O, m, l
        if (ok && n_tiles > 0) ok = warp_all(mbar_wait(&ms->o_ready[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1));
        if (ok) {
            tc_fence_after();
            const uint32_t rho = w_idx * p.n_q_heads + item.kv_head * group + g_idx;
            if (p.direct) {
                // the item covers the session's whole key range: normalise and store the output row
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;          // no visible key: zeros
                T *orow = reinterpret_cast<T *>(ses.out) + (size_t)w_idx * p.out_row_stride +
                          (size_t)(item.kv_head * group + g_idx) * kHD;
#pragma unroll 1
                for (int c0 = 0; c0 < kHD; c0 += 32) {
                    uint32_t o[32];
                    if (n_tiles > 0) {
                        tmem_ld32(tmem + lane_addr + kColO + c0, o);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = 0u;
                    }
                    if (row_valid) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 v;
                            v.x = pack2<T>(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                            v.y = pack2<T>(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                            v.z = pack2<T>(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                            v.w = pack2<T>(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                            *reinterpret_cast<uint4 *>(orow + c0 + c) = v;
                        }
                    }
                }
            } else {
                const size_t prow = (size_t)item.partial_base + (size_t)item.part_index * rows_total + rho;
                if (row_valid) {
                    p.part_m[prow] = (n_tiles > 0 && m_ref != -INFINITY) ? m_ref * kLn2 : -INFINITY;   // natural-log domain
                    p.part_l[prow] = (n_tiles > 0 && m_ref != -INFINITY) ? l_run : 0.f;
                }
                float *dst = p.part_o + prow * kHD;
#pragma unroll 1
                for (int c0 = 0; c0 < kHD; c0 += 32) {
                    uint32_t o[32];
                    if (n_tiles > 0) {
                        tmem_ld32(tmem + lane_addr + kColO + c0, o);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = 0u;
                    }
                    if (row_valid) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4)
                            *reinterpret_cast<float4 *>(dst + c0 + c) =
                                make_float4(__uint_as_float(o[c]), __uint_as_float(o[c + 1]), __uint_as_float(o[c + 2]),
                                            __uint_as_float(o[c + 3]));
                    }
                }
            }
        }
        failed = !ok;
    }

    if (failed) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == G::kProducerWarp) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

// One K and one V tensor map per session of a verify batch ([seq_len rows][n_kv_heads * 256], box
// 128 x 64, keys past seq_len read as zero), written to `dst_maps`: the context's parameter block for a
// small batch, else the staging table that the caller uploads together with the session and item tables.
int tt_verify_tc_encode_maps(tt_context *ctx, uint32_t n_sessions, const tt_attn_batch_params *p, void *dst_maps) {
    CUtensorMap *maps = reinterpret_cast<CUtensorMap *>(dst_maps);
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
                        float *part_m, float *part_l, const tt_attn_batch_params *p, bool direct, bool in_params,
                        bool rows128) {
    (void)n_sessions;
    static thread_local TTSessionTable no_table;       // n == 0: the kernel reads the device tables
    no_table.n = 0;
    const TTSessionTable &table = in_params ? ctx->session_table : no_table;
    cudaError_t e;
    VerifyParams kp;
    kp.items = ctx->items; kp.sessions = ctx->sessions;
    kp.maps = reinterpret_cast<const CUtensorMap *>(ctx->tensor_maps);
    kp.part_o = part_o; kp.part_m = part_m; kp.part_l = part_l;
    kp.n_q_heads = p->n_q_heads; kp.n_kv_heads = p->n_kv_heads; kp.q_row_stride = p->q_row_stride_elements;
    kp.out_row_stride = p->out_row_stride_elements; kp.direct = direct ? 1u : 0u;
    kp.scale_log2 = p->scale * kLog2e;
    kp.idesc_qk = tt_make_idesc_f16(p->io_dtype, kBK, false);        // Q (K-major) x K rows (K-major), N = 128 keys
    kp.idesc_pv = tt_make_idesc_f16(p->io_dtype, kHD / 2, true);     // P (TMEM) x V (MN-major), N = 128 head dims
    auto launch = [&](auto kernel, int threads, int smem) {
        cudaError_t err = tt_set_smem_once(kernel, smem);
        if (err != cudaSuccess) return err;
        return tt_launch_pdl(kernel, dim3(n_items), dim3(threads), (size_t)smem, stream, kp, ctx->status, table, ctx->verify_maps);
    };
    if (rows128) {
        constexpr int kT = VerifyGeom<128>::kThreads, kS = verify_smem_bytes<128>();
        e = p->io_dtype == TT_F16 ? launch(attn_verify_tc_kernel<__half, 128>, kT, kS)
                                  : launch(attn_verify_tc_kernel<__nv_bfloat16, 128>, kT, kS);
    } else {
        constexpr int kT = VerifyGeom<64>::kThreads, kS = verify_smem_bytes<64>();
        e = p->io_dtype == TT_F16 ? launch(attn_verify_tc_kernel<__half, 64>, kT, kS)
                                  : launch(attn_verify_tc_kernel<__nv_bfloat16, 64>, kT, kS);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_verify_tc launch");
    return TT_OK;
}
