// Split-KV decode attention for sm_100a: batched over sessions, GQA-packed.
//
// Replaces attention_decode_partial / attention_decode_combine
// (sources/TinyTitanCore/Metal/Attention/attention.metal:162-269, :395-437) and the host
// dispatch Attention.encodeSplit (sources/TinyTitan/Kernels/Attention/Attention.swift:314-470).
//
// HBM-bound design. A work item is (session, kv head, 16-row tile of packed query rows, key
// range). Every K/V row of the range is read from HBM once per KV head and serves all query
// rows of the group (the reference re-reads it per q head). A CTA is one warp pair: both warps
// stream the same 16-key blocks through a 3-stage shared-memory ring filled by bulk async
// copies (cp.async.bulk + mbarrier complete_tx), each warp owns one half of the head dimension
// (its half of Q in registers, its half of the output columns), Q.K^T and P.V run on
// mma.sync m16n8k16 with fp32 accumulation, the softmax is done on the accumulator fragments
// with quad shuffles. Pass 2 merges the items of a session by log-sum-exp. A call with one
// session carries it in the kernel parameters (no table upload), which also makes that call
// capturable in a CUDA graph.
#include "tt_sm100.h"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace {

constexpr int kKeysPerBlock = 16;   // keys per warp pipeline stage
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1);

template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4],
                                                  uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4],
                                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared memory of the fp16/bf16 pass-1 kernel for HPC KV heads per CTA.
template <int HD, int HPC>
struct DecodeSmem {
    static constexpr int kPitch = HPC * HD + 8;                    // elements per staged row (all HPC heads of a key)
    static constexpr int kRowBytes = kPitch * 2;
    static constexpr int kTileBytes = kKeysPerBlock * kRowBytes;   // one K (or V) block
    static constexpr int kVRing = kStages * kTileBytes;            // K ring first, V ring behind it
    static constexpr int kRingBytes = 2 * kStages * kTileBytes;
    static constexpr int kScorePitch = 24;                         // floats per query row of a handed-over score tile
    static constexpr int kScoreTile = 16 * kScorePitch;            // [query row][key]
    static constexpr int kScoreBytes = HPC * 2 * kScoreTile * 4;   // [head][buffer]
    static constexpr int kBars = 4 * kStages + 4 * HPC;            // k_full, v_full, k_empty, v_empty [kStages]; s_full, s_empty [HPC][2]
    static constexpr int kTotal = kRingBytes + kScoreBytes + kBars * 8;
};

__device__ __forceinline__ void pair_barrier() { asm volatile("bar.sync 1, 64;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// Pass 1. grid = items, block = 2 * HPC warps; 4 / HPC CTAs per SM.
//
// A work item is (session, HPC adjacent KV heads, up to 16 packed query rows per head, key range).
// With HPC = 2 a CTA streams whole cache rows (both KV heads of a key, 1 KB at head_dim 256) so
// that DRAM is read in long contiguous pieces; a pure streaming read of 512-byte pieces at a 1 KB
// pitch measured 6.6 TB/s on this part against 7.1 TB/s for whole rows.
//
// The warps of a CTA have different jobs and run one block apart. Both products are TRANSPOSED so
// that the 8-wide N dimension of mma.m16n8k16 is the query rows of one KV head (8 with a GQA group
// of 8, two n-tiles for up to 16 packed rows) and the 16-wide M dimension is filled by keys
// (Q.K^T) or head dimensions (P.V) -- nothing is padding:
//   warps 0 .. HPC-1      (one per KV head) form S^T = K . Q^T from the K ring (A = the K block read
//                         with ldmatrix, B = the query rows held in registers) and hand the
//                         16 x 8 score tile over through shared memory;
//   warps HPC .. 2 HPC-1  take the score tile in the B-operand layout (one query row per lane
//                         quad-row, so a row's maximum is two shuffles), run the online softmax
//                         and accumulate O^T += V^T . P^T from the V ring (A = the V block read
//                         with ldmatrix.trans); they end with (m, l) and the whole output tile.
// K and V have their own 3-stage rings of bulk copies (one per key row, completion on the stage's
// mbarrier). Warp 0 refills a K stage once every K.Q^T warp has released it, warp HPC a V stage
// once every P.V warp has; the score tiles are double buffered per head. Every wait is bounded.
// ---------------------------------------------------------------------------------------
template <int HD, int NT, int HPC, typename T>
__global__ void __launch_bounds__(64 * HPC, 4 / HPC)
attn_decode_partial_kernel(const TTDecodeItem *__restrict__ items,
                           const TTDecodeSession *__restrict__ sessions, float *__restrict__ part_o,
                           float *__restrict__ part_m, float *__restrict__ part_l,
                           uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t kv_stride_bytes,
                           uint32_t q_row_stride, float scale_log2, uint32_t *__restrict__ status,
                           const __grid_constant__ TTSessionTable table, uint32_t table_keys_per_item) {
    using S = DecodeSmem<HD, HPC>;
    constexpr int KS = HD / 16;         // k-steps of K.Q^T and m-tiles of V^T.P^T
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int role = warp / HPC, head = warp % HPC;   // role 0: K.Q^T, role 1: softmax + V^T.P^T

    const uint32_t group = n_q_heads / n_kv_heads;
    const uint32_t n_kv_groups = n_kv_heads / HPC;
    // Calls with up to kParamSessions sessions carry them in the kernel parameters and derive the
    // work item from the block index (the items of a session are equal slices, item_prefix says
    // where each session's items start), so no table is copied to the device and a CTA starts
    // without two dependent global loads.
    pdl_launch_dependents();
    TTDecodeItem item;
    TTDecodeSession ses;
    if (table.n != 0) {
        uint32_t lo = 0, hi = table.n;
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (table.item_prefix[mid] <= blockIdx.x) lo = mid; else hi = mid;
        }
        ses = table.s[lo];
        const uint32_t local = blockIdx.x - table.item_prefix[lo];
        const uint32_t packed_rows = ses.q_rows * group;
        const uint32_t row_tiles = (packed_rows + 15) / 16;
        const uint32_t rt = local % row_tiles, kvg = (local / row_tiles) % n_kv_groups;
        const uint32_t part = local / (row_tiles * n_kv_groups);
        item.session = lo; item.kv_head = kvg * HPC; item.part_index = part; item.partial_base = ses.partial_base;
        item.key_begin = min(ses.seq_len, ses.kv_start + part * table_keys_per_item);
        item.key_end = min(ses.seq_len, item.key_begin + table_keys_per_item);
        item.row_begin = rt * 16;
        item.row_count = min(16u, packed_rows - rt * 16);
    } else {
        item = items[blockIdx.x];
        ses = sessions[item.session];
    }
    const uint32_t kv_head = item.kv_head + head;      // the head this warp serves

    unsigned char *k_ring = smem;
    unsigned char *v_ring = smem + S::kVRing;
    float *score = reinterpret_cast<float *>(smem + S::kRingBytes) + head * 2 * S::kScoreTile;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::kRingBytes + S::kScoreBytes);
    uint64_t *k_full = bars, *v_full = bars + kStages, *k_empty = bars + 2 * kStages, *v_empty = bars + 3 * kStages;
    uint64_t *s_full = bars + 4 * kStages + head * 4, *s_empty = s_full + 2;

    if (threadIdx.x == 0) {
        for (int b = 0; b < 2 * kStages; ++b) mbar_init(&bars[b], 1);                   // filled by one expect_tx arrival
        for (int b = 2 * kStages; b < 4 * kStages; ++b) mbar_init(&bars[b], HPC);       // released by every reader warp
        for (int b = 4 * kStages; b < S::kBars; ++b) mbar_init(&bars[b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // everything above overlapped the tail of the kernel before this one in the stream; its
    // results (the query rows, the newest K/V rows, partials being merged) are read from here on
    pdl_wait();

    const uint32_t n_keys = item.key_end - item.key_begin;
    const uint32_t n_blocks = (n_keys + kKeysPerBlock - 1) / kKeysPerBlock;
    auto block_valid = [&](uint32_t i) { return min((uint32_t)kKeysPerBlock, n_keys - i * kKeysPerBlock); };
    // lanes 0..15 of the issuing warp fetch one row each (all HPC heads of the key) of block i
    auto issue = [&](uint32_t i, unsigned char *ring, const unsigned char *base, uint64_t *full, bool zero_fill) {
        const uint32_t valid = block_valid(i), stage = i % kStages;
        if (lane == 0) mbar_expect_tx(&full[stage], valid * (uint32_t)(HPC * HD * 2));
        __syncwarp();
        if (lane < kKeysPerBlock) {
            unsigned char *dst = ring + stage * S::kTileBytes + lane * S::kRowBytes;
            if ((uint32_t)lane < valid) {
                uint32_t p = item.key_begin + i * kKeysPerBlock + lane;
                if (ses.row_index != nullptr) p = ses.row_index[p];
                if (ses.ring_capacity) p %= ses.ring_capacity;
                // read once: evict-first in L2, so that the stream does not push out the partials, the query
                // rows and what the neighbouring kernels of the step keep there (measured on the config-2
                // step: 0.1854 -> 0.1778 ms)
                bulk_copy_g2s_stream(dst, base + (size_t)p * kv_stride_bytes, HPC * HD * 2, &full[stage]);
            } else if (zero_fill) {
                // a V row that is never fetched must still be finite: it meets p == 0 in P.V
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                for (int c = 0; c < HPC * HD / 8; ++c) reinterpret_cast<uint4 *>(dst)[c] = z;
            }
        }
    };
    bool timed_out = false;
    uint32_t consumed = 0, issued = 0;      // blocks of the ring this warp fills (warps 0 and HPC only)

    if (role == 0) {
        // ================= K . Q^T =================
        const unsigned char *kbase = reinterpret_cast<const unsigned char *>(ses.k) + (size_t)item.kv_head * HD * 2;
        // the query rows as B fragments: lane (g, t) holds dims 2t, 2t+1 (+8) of row g of every n-tile
        uint32_t qf[NT][KS][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t r = nt * 8 + g;
            const T *qp = nullptr;
            if (r < item.row_count) {
                const uint32_t packed = item.row_begin + r;
                qp = reinterpret_cast<const T *>(ses.q) + (size_t)(packed / group) * q_row_stride +
                     (size_t)(kv_head * group + packed % group) * HD + t * 2;
            }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                qf[nt][ks][0] = qp ? *reinterpret_cast<const uint32_t *>(qp + ks * 16) : 0u;
                qf[nt][ks][1] = qp ? *reinterpret_cast<const uint32_t *>(qp + ks * 16 + 8) : 0u;
            }
        }
        if (head == 0)
            for (; issued < n_blocks && issued < (uint32_t)kStages; ++issued) issue(issued, k_ring, kbase, k_full, false);
        // A fragment of a K block: matrix j = lane / 8 covers keys 8 (j & 1) .. +7, dims 8 (j >> 1) .. +7
        const uint32_t k_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * S::kRowBytes + (lane >> 4) * 16 + head * HD * 2;
        for (uint32_t i = 0; i < n_blocks; ++i) {
            if (!warp_all(mbar_wait(&k_full[i % kStages], (i / kStages) & 1))) { timed_out = true; break; }
            const uint32_t stage = smem_u32(k_ring + (i % kStages) * S::kTileBytes);
            // two accumulator chains per n-tile (even / odd k-steps) halve the dependent MMA depth
            float s0[NT][4], s1[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { s0[nt][0] = s0[nt][1] = s0[nt][2] = s0[nt][3] = 0.f; s1[nt][0] = s1[nt][1] = s1[nt][2] = s1[nt][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ks += 2) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, stage + k_off + ks * 32);
                ldmatrix_x4(b, stage + k_off + (ks + 1) * 32);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_16816<T>(s0[nt], a, qf[nt][ks][0], qf[nt][ks][1]);
                    mma_16816<T>(s1[nt], b, qf[nt][ks + 1][0], qf[nt][ks + 1][1]);
                }
            }
            __syncwarp();                                   // every lane has its fragments: this warp releases the stage
            if (lane == 0) mbar_arrive(&k_empty[i % kStages]);
            if (head == 0) consumed = i + 1;
            // hand the tile over: element (query row r, key k) at score[buffer][r][k]
            if (i >= 2 && !warp_all(mbar_wait(&s_empty[i & 1], ((i >> 1) - 1) & 1))) { timed_out = true; break; }
            float *sb = score + (i & 1) * S::kScoreTile;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float *r0 = sb + (nt * 8 + 2 * t) * S::kScorePitch, *r1 = r0 + S::kScorePitch;
                r0[g] = s0[nt][0] + s1[nt][0]; r1[g] = s0[nt][1] + s1[nt][1];
                r0[g + 8] = s0[nt][2] + s1[nt][2]; r1[g + 8] = s0[nt][3] + s1[nt][3];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_full[i & 1]);
            if (head == 0 && issued < n_blocks) {           // block i + kStages goes into the stage block i just left
                if (!warp_all(mbar_wait(&k_empty[i % kStages], (i / kStages) & 1))) { timed_out = true; break; }
                issue(issued, k_ring, kbase, k_full, false);
                ++issued;
            }
        }
        if (timed_out) {
            // blocks issued into the ring and not yet waited for may still be landing
            for (uint32_t b = consumed; b < issued; ++b) mbar_wait(&k_full[b % kStages], (b / kStages) & 1, 1u << 16);
            if (lane == 0) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
        }
        return;
    }

    // ================= softmax and V^T . P^T =================
    const unsigned char *vbase = reinterpret_cast<const unsigned char *>(ses.v) + (size_t)item.kv_head * HD * 2;
    if (head == 0)
        for (; issued < n_blocks && issued < (uint32_t)kStages; ++issued) issue(issued, v_ring, vbase, v_full, true);

    float acc[NT][KS][4];               // O^T: dims 16 mt + g (+8) x query rows 2t, 2t+1 of n-tile nt
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mt = 0; mt < KS; ++mt) acc[nt][mt][0] = acc[nt][mt][1] = acc[nt][mt][2] = acc[nt][mt][3] = 0.f;
    float m_run[NT], l_run[NT];         // of query row 8 nt + g; l is this lane's share (keys 2t, 2t+1, 2t+8, 2t+9)
    uint32_t limit[NT];                 // visible-key limit of that row
    const uint32_t w_first = item.row_begin / group;
    const uint32_t limit_min = ses.seq_len - (ses.q_rows - 1 - w_first);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m_run[nt] = -INFINITY; l_run[nt] = 0.f;
        const uint32_t r = nt * 8 + g;
        // rows past row_count are never written: they take the tile's smallest limit and need no masking of their own
        limit[nt] = r < item.row_count ? ses.seq_len - (ses.q_rows - 1 - (item.row_begin + r) / group) : limit_min;
    }
    // A fragment of V^T: matrix j = lane / 8 covers keys 8 (j >> 1) .. +7, dims 8 (j & 1) .. +7 (read transposed)
    const uint32_t v_off = ((lane & 7) + (lane >> 4) * 8) * S::kRowBytes + ((lane >> 3) & 1) * 16 + head * HD * 2;

    for (uint32_t i = 0; i < n_blocks; ++i) {
        if (!warp_all(mbar_wait(&s_full[i & 1], (i >> 1) & 1))) { timed_out = true; break; }
        const float *sb = score + (i & 1) * S::kScoreTile;
        float sv[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float2 lo = *reinterpret_cast<const float2 *>(sb + (nt * 8 + g) * S::kScorePitch + 2 * t);
            const float2 hi = *reinterpret_cast<const float2 *>(sb + (nt * 8 + g) * S::kScorePitch + 2 * t + 8);
            sv[nt][0] = lo.x; sv[nt][1] = lo.y; sv[nt][2] = hi.x; sv[nt][3] = hi.y;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[i & 1]);

        // ---- mask + online softmax of row 8 nt + g over this lane's four keys ----
        const uint32_t blk_key0 = item.key_begin + i * kKeysPerBlock;
        const bool plain = (blk_key0 + kKeysPerBlock <= limit_min) && (blk_key0 + kKeysPerBlock <= item.key_end) &&
                           (ses.keep == nullptr);
        uint32_t pb[NT][2];
        float alpha[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float s = sv[nt][j] * scale_log2;
                if (!plain) {
                    const uint32_t key = blk_key0 + 2 * t + (j >> 1) * 8 + (j & 1);
                    bool ok = key < limit[nt] && key < item.key_end;
                    if (ok && ses.keep != nullptr) ok = ses.keep[key] != 0;
                    s = ok ? s : -INFINITY;
                }
                sv[nt][j] = s;
                mx = fmaxf(mx, s);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[nt], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[nt] = fast_exp2(m_run[nt] - m_use);
            m_run[nt] = m_new;
            pb[nt][0] = pack2<T>(fast_exp2(sv[nt][0] - m_use), fast_exp2(sv[nt][1] - m_use));
            pb[nt][1] = pack2<T>(fast_exp2(sv[nt][2] - m_use), fast_exp2(sv[nt][3] - m_use));
            // row sums from the ROUNDED weights the MMA consumes: O / l stays a convex combination
            l_run[nt] = l_run[nt] * alpha[nt] + sum2<T>(pb[nt][0]) + sum2<T>(pb[nt][1]);
        }
        // the accumulators hold query rows 2t, 2t+1: their factors live in the lanes of quad rows 2t and 2t+1
        bool rescale = false;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) rescale |= alpha[nt] != 1.f;
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float a0 = __shfl_sync(0xffffffffu, alpha[nt], 8 * t), a1 = __shfl_sync(0xffffffffu, alpha[nt], 8 * t + 4);
#pragma unroll
                for (int mt = 0; mt < KS; ++mt) {
                    acc[nt][mt][0] *= a0; acc[nt][mt][1] *= a1;
                    acc[nt][mt][2] *= a0; acc[nt][mt][3] *= a1;
                }
            }
        }

        // ---- O^T += V^T P^T ----
        if (!warp_all(mbar_wait(&v_full[i % kStages], (i / kStages) & 1))) { timed_out = true; break; }
        const uint32_t stage = smem_u32(v_ring + (i % kStages) * S::kTileBytes);
#pragma unroll
        for (int mt = 0; mt < KS; ++mt) {
            uint32_t a[4];
            ldmatrix_x4_trans(a, stage + v_off + mt * 32);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_16816<T>(acc[nt][mt], a, pb[nt][0], pb[nt][1]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&v_empty[i % kStages]);
        if (head == 0) {
            consumed = i + 1;
            if (issued < n_blocks) {
                if (!warp_all(mbar_wait(&v_empty[i % kStages], (i / kStages) & 1))) { timed_out = true; break; }
                issue(issued, v_ring, vbase, v_full, true);
                ++issued;
            }
        }
    }

    if (timed_out) {
        for (uint32_t b = consumed; b < issued; ++b) mbar_wait(&v_full[b % kStages], (b / kStages) & 1, 1u << 16);
        if (lane == 0) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
    }

    // ---- write the partial: (m, l) of row 8 nt + g by the quad's first lane, O^T by everyone ----
    const uint32_t rows_total = ses.q_rows * n_q_heads;
    auto partial_row = [&](uint32_t r) {
        const uint32_t packed = item.row_begin + r;
        const uint32_t rho = (packed / group) * n_q_heads + kv_head * group + packed % group;
        return (size_t)ses.partial_base + (size_t)item.part_index * rows_total + rho;
    };
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        float l = l_run[nt];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const uint32_t r = nt * 8 + g;
        if (t == 0 && r < item.row_count) {
            const size_t prow = partial_row(r);
            part_m[prow] = m_run[nt] * kLn2;   // natural-log domain, the reference's partial format
            part_l[prow] = l;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t ro = nt * 8 + 2 * t + h;
            if (ro >= item.row_count) continue;
            float *dst = part_o + partial_row(ro) * HD + g;
#pragma unroll
            for (int mt = 0; mt < KS; ++mt) {
                dst[mt * 16] = acc[nt][mt][h];
                dst[mt * 16 + 8] = acc[nt][mt][2 + h];
            }
        }
    }
}

// Shared memory of the quantised-KV variant: a ring of RAW rows (this head's packed values followed by
// the row's scale/bias block), plus one private fp16 tile pair per warp holding the dequantised halves.
template <int HD, int BITS>
struct QuantSmem {
    static constexpr int kValBytes = HD * BITS / 8;                // packed values of one head in a row
    static constexpr int kRowBytes = kValBytes + 64;               // + up to 64 B of scales and biases
    static constexpr int kTileBytes = kKeysPerBlock * kRowBytes;   // K (or V) raw block
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kRingBytes = kStages * kStageBytes;
    static constexpr int kHalfRowBytes = (HD / 2 + 8) * 2;         // fp16 half-row, padded for ldmatrix
    static constexpr int kHalfTileBytes = kKeysPerBlock * kHalfRowBytes;
    static constexpr int kWarpTileBytes = 2 * kHalfTileBytes;      // K half + V half
    static constexpr int kXchgBytes = 2 * 2 * 32 * 9 * 4;
    static constexpr int kTotal = kRingBytes + 2 * kWarpTileBytes + kXchgBytes + 64;
};

// ---------------------------------------------------------------------------------------
// Pass 1 over affine-quantised K/V rows (8 or 4 bits, 64-element groups, fp16 scale and bias
// stored after the packed values of each row: KVCacheManager.rowLayout,
// KVCacheManager+Validation.swift:30-41; loader semantics attn_load_kv, attention.metal:89-117).
// Same structure as the fp16 kernel above; the ring carries the raw rows (half or a quarter of
// the bytes), and each warp dequantises its own head-dim halves of the landed K and V block into
// private fp16 tiles before the MMAs: value = code * scale + bias in fp32, rounded to fp16.
// ---------------------------------------------------------------------------------------
template <int HD, int BITS>
__global__ void __launch_bounds__(64, 4)
attn_decode_partial_quant_kernel(const TTDecodeItem *__restrict__ items,
                           const TTDecodeSession *__restrict__ sessions, float *__restrict__ part_o,
                           float *__restrict__ part_m, float *__restrict__ part_l,
                           uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t kv_stride_bytes,
                           uint32_t q_row_stride, float scale_log2, uint32_t *__restrict__ status,
                           const __grid_constant__ TTSessionTable table, uint32_t table_keys_per_item,
                           uint32_t value_bytes, uint32_t meta_bytes) {
    using T = __half;
    using S = QuantSmem<HD, BITS>;
    constexpr int HH = HD / 2;          // head-dim half per warp
    constexpr int KS = HH / 16;         // k-steps of the partial Q.K^T
    constexpr int NT = HH / 8;          // n-tiles of this warp's half of O
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t group = n_q_heads / n_kv_heads;
    // Calls with up to kParamSessions sessions carry them in the kernel parameters and derive the
    // work item from the block index (the items of a session are equal slices, item_prefix says
    // where each session's items start), so no table is copied to the device and a CTA starts
    // without two dependent global loads.
    pdl_launch_dependents();
    TTDecodeItem item;
    TTDecodeSession ses;
    if (table.n != 0) {
        uint32_t lo = 0, hi = table.n;
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (table.item_prefix[mid] <= blockIdx.x) lo = mid; else hi = mid;
        }
        ses = table.s[lo];
        const uint32_t local = blockIdx.x - table.item_prefix[lo];
        const uint32_t packed_rows = ses.q_rows * group;
        const uint32_t row_tiles = (packed_rows + 15) / 16;
        const uint32_t rt = local % row_tiles, kvh = (local / row_tiles) % n_kv_heads;
        const uint32_t part = local / (row_tiles * n_kv_heads);
        item.session = lo; item.kv_head = kvh; item.part_index = part; item.partial_base = ses.partial_base;
        item.key_begin = min(ses.seq_len, ses.kv_start + part * table_keys_per_item);
        item.key_end = min(ses.seq_len, item.key_begin + table_keys_per_item);
        item.row_begin = rt * 16;
        item.row_count = min(16u, packed_rows - rt * 16);
    } else {
        item = items[blockIdx.x];
        ses = sessions[item.session];
    }

    unsigned char *ring = smem;                                   // raw (quantised) K/V rows, 3 stages
    unsigned char *tiles = smem + S::kRingBytes + warp * S::kWarpTileBytes;   // this warp's fp16 K and V halves
    float *xchg = reinterpret_cast<float *>(smem + S::kRingBytes + 2 * S::kWarpTileBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::kRingBytes + 2 * S::kWarpTileBytes + S::kXchgBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    // everything above overlapped the tail of the kernel before this one in the stream; its
    // results (the query rows, the newest K/V rows, partials being merged) are read from here on
    pdl_wait();
    // ---- this warp's half of the Q tile, straight into mma A fragments ----
    uint32_t qf[KS][4];
    {
        const uint32_t r0 = lane >> 2, r1 = r0 + 8;
        const T *q0 = nullptr, *q1 = nullptr;
        if (r0 < item.row_count) {
            const uint32_t packed = item.row_begin + r0;
            q0 = reinterpret_cast<const T *>(ses.q) + (size_t)(packed / group) * q_row_stride +
                 (size_t)(item.kv_head * group + packed % group) * HD + warp * HH + (lane & 3) * 2;
        }
        if (r1 < item.row_count) {
            const uint32_t packed = item.row_begin + r1;
            q1 = reinterpret_cast<const T *>(ses.q) + (size_t)(packed / group) * q_row_stride +
                 (size_t)(item.kv_head * group + packed % group) * HD + warp * HH + (lane & 3) * 2;
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = q0 ? *reinterpret_cast<const uint32_t *>(q0 + ks * 16) : 0u;
            qf[ks][1] = q1 ? *reinterpret_cast<const uint32_t *>(q1 + ks * 16) : 0u;
            qf[ks][2] = q0 ? *reinterpret_cast<const uint32_t *>(q0 + ks * 16 + 8) : 0u;
            qf[ks][3] = q1 ? *reinterpret_cast<const uint32_t *>(q1 + ks * 16 + 8) : 0u;
        }
    }

    const uint32_t n_keys = item.key_end - item.key_begin;
    const uint32_t n_blocks = (n_keys + kKeysPerBlock - 1) / kKeysPerBlock;
    // a key's row: [packed values of all heads | fp16 scale per 64-element group | fp16 bias per group]
    const unsigned char *kbase = reinterpret_cast<const unsigned char *>(ses.k);
    const unsigned char *vbase = reinterpret_cast<const unsigned char *>(ses.v);
    const uint32_t head_value_offset = item.kv_head * S::kValBytes;
    const uint32_t groups_total = n_kv_heads * HD / 64;

    auto block_valid = [&](uint32_t i) {
        return min((uint32_t)kKeysPerBlock, n_keys - i * kKeysPerBlock);
    };
    // thread 0 announces the bytes of block i; ordered before the copies by a barrier
    auto announce = [&](uint32_t i) {
        mbar_expect_tx(&bars[i % kStages], block_valid(i) * 2u * (uint32_t)(S::kValBytes + meta_bytes));
    };
    // warp 0 fetches the K rows of block i, warp 1 the V rows (lanes 0..15, one row each)
    auto issue = [&](uint32_t i) {
        if (lane < kKeysPerBlock) {
            const uint32_t valid = block_valid(i);
            unsigned char *dst = ring + (i % kStages) * S::kStageBytes + warp * S::kTileBytes + lane * S::kRowBytes;
            if ((uint32_t)lane < valid) {
                uint32_t p = item.key_begin + i * kKeysPerBlock + lane;
                if (ses.row_index != nullptr) p = ses.row_index[p];
                if (ses.ring_capacity) p %= ses.ring_capacity;
                const unsigned char *src = (warp ? vbase : kbase) + (size_t)p * kv_stride_bytes;
                bulk_copy_g2s_stream(dst, src + head_value_offset, S::kValBytes, &bars[i % kStages]);
                bulk_copy_g2s_stream(dst + S::kValBytes, src + value_bytes, meta_bytes, &bars[i % kStages]);
            }
        }
    };

    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }

    // visible-key limit of the two rows this thread owns; rows past row_count are never
    // written, so they take the tile's smallest limit and need no masking of their own
    const uint32_t w_first = item.row_begin / group;
    const uint32_t limit_min = ses.seq_len - (ses.q_rows - 1 - w_first);
    uint32_t limit[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = (lane >> 2) + 8 * h;
        limit[h] = r < item.row_count ? ses.seq_len - (ses.q_rows - 1 - (item.row_begin + r) / group) : limit_min;
    }

    const uint32_t prologue = min(n_blocks, (uint32_t)(kStages - 1));
    if (threadIdx.x == 0)
        for (uint32_t i = 0; i < prologue; ++i) announce(i);
    __syncthreads();
    for (uint32_t i = 0; i < prologue; ++i) issue(i);

    bool timed_out = false;
    uint32_t timed_block = 0;
    const uint32_t k_off = ((lane & 7) + ((lane >> 4) << 3)) * S::kHalfRowBytes + ((lane >> 3) & 1) * 16;
    const uint32_t v_off = S::kHalfTileBytes + ((lane & 7) + ((lane >> 3) & 1) * 8) * S::kHalfRowBytes + (lane >> 4) * 16;
    // dequantisation duty of this lane: key lane/2, E = HH/2 consecutive elements of this warp's half
    constexpr int E = HH / 2;
    const uint32_t dq_key = lane >> 1, dq_sub = lane & 1;
    const uint32_t dq_group = (item.kv_head * HD + warp * HH + dq_sub * E) / 64;
    const uint32_t dq_src = dq_key * S::kRowBytes + (warp * HH + dq_sub * E) * BITS / 8;
    const uint32_t dq_dst = dq_key * S::kHalfRowBytes + dq_sub * E * 2;

    for (uint32_t i = 0; i < n_blocks; ++i) {
        const uint32_t nxt = i + kStages - 1;
        if (threadIdx.x == 0 && nxt < n_blocks) announce(nxt);
        const bool got = __all_sync(0xffffffffu, mbar_wait(&bars[i % kStages], (i / kStages) & 1)) != 0;

        // ---- dequantise this warp's halves of the landed K and V rows into its fp16 tiles ----
        if (got) {
            const uint32_t valid = block_valid(i);
#pragma unroll
            for (int kv = 0; kv < 2; ++kv) {
                const unsigned char *raw = ring + (i % kStages) * S::kStageBytes + kv * S::kTileBytes;
                unsigned char *dst = tiles + kv * S::kHalfTileBytes + dq_dst;
                if (dq_key < valid) {
                    const unsigned char *row = raw + dq_key * S::kRowBytes;
                    const float sc = __half2float(*reinterpret_cast<const __half *>(row + S::kValBytes + dq_group * 2));
                    const float bi = __half2float(*reinterpret_cast<const __half *>(row + S::kValBytes + (groups_total + dq_group) * 2));
                    const unsigned char *src = raw + dq_src;
#pragma unroll
                    for (int c = 0; c < E * BITS / 8 / 16; ++c) {
                        const uint4 pk = *reinterpret_cast<const uint4 *>(src + c * 16);
                        const uint32_t wds[4] = {pk.x, pk.y, pk.z, pk.w};
                        if constexpr (BITS == 8) {
                            uint32_t o[8];
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                const uint32_t u = wds[q4];
                                o[2 * q4] = pack2<__half>(fmaf((float)(u & 0xffu), sc, bi), fmaf((float)((u >> 8) & 0xffu), sc, bi));
                                o[2 * q4 + 1] = pack2<__half>(fmaf((float)((u >> 16) & 0xffu), sc, bi), fmaf((float)(u >> 24), sc, bi));
                            }
                            reinterpret_cast<uint4 *>(dst)[2 * c] = make_uint4(o[0], o[1], o[2], o[3]);
                            reinterpret_cast<uint4 *>(dst)[2 * c + 1] = make_uint4(o[4], o[5], o[6], o[7]);
                        } else {
                            uint32_t o[16];
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                const uint32_t u = wds[q4];
#pragma unroll
                                for (int b2 = 0; b2 < 4; ++b2) {   // byte b2: low nibble = even element, high = odd
                                    const uint32_t byte = (u >> (8 * b2)) & 0xffu;
                                    o[4 * q4 + b2] = pack2<__half>(fmaf((float)(byte & 0xfu), sc, bi), fmaf((float)(byte >> 4), sc, bi));
                                }
                            }
#pragma unroll
                            for (int v4 = 0; v4 < 4; ++v4)
                                reinterpret_cast<uint4 *>(dst)[4 * c + v4] = make_uint4(o[4 * v4], o[4 * v4 + 1], o[4 * v4 + 2], o[4 * v4 + 3]);
                        }
                    }
                } else {
                    // keys past the end of the item: finite zeros (their scores are masked, P is 0)
                    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int c = 0; c < E * 2 / 16; ++c) reinterpret_cast<uint4 *>(dst)[c] = z;
                }
            }
        }
        __syncwarp();
        const uint32_t stage = smem_u32(tiles);
        // ---- partial S over this warp's head-dim half: two independent chains per n-tile ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KS; ks += 2) {
            uint32_t b[4], c[4];
            ldmatrix_x4(b, stage + k_off + ks * 32);
            ldmatrix_x4(c, stage + k_off + (ks + 1) * 32);
            mma_16816<T>(s0, qf[ks], b[0], b[1]);
            mma_16816<T>(s1, qf[ks], b[2], b[3]);
            mma_16816<T>(t0, qf[ks + 1], c[0], c[1]);
            mma_16816<T>(t1, qf[ks + 1], c[2], c[3]);
        }
        float *mine = xchg + (((i & 1) * 2 + warp) * 32 + lane) * 9;
        const float *theirs = xchg + (((i & 1) * 2 + (warp ^ 1)) * 32 + lane) * 9;
#pragma unroll
        for (int j = 0; j < 4; ++j) { mine[j] = s0[j] + t0[j]; mine[4 + j] = s1[j] + t1[j]; }
        mine[8] = got ? 1.f : 0.f;
        pair_barrier();
        if (!(got && theirs[8] != 0.f)) { timed_out = true; timed_block = i; break; }   // same decision in both warps
        float sv[2][4];  // [row half][key: n0c0 n0c1 n1c0 n1c1]
        sv[0][0] = mine[0] + theirs[0]; sv[0][1] = mine[1] + theirs[1];
        sv[1][0] = mine[2] + theirs[2]; sv[1][1] = mine[3] + theirs[3];
        sv[0][2] = mine[4] + theirs[4]; sv[0][3] = mine[5] + theirs[5];
        sv[1][2] = mine[6] + theirs[6]; sv[1][3] = mine[7] + theirs[7];

        // every lane of the pair is past block i-1 now: its stage may be refilled
        if (nxt < n_blocks) issue(nxt);

        // ---- mask + online softmax (identical in both warps) ----
        const uint32_t blk_key0 = item.key_begin + i * kKeysPerBlock;
        const bool plain = (blk_key0 + kKeysPerBlock <= limit_min) && (blk_key0 + kKeysPerBlock <= item.key_end) &&
                           (ses.keep == nullptr);
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float s = sv[h][j] * scale_log2;
                if (!plain) {
                    const uint32_t key = blk_key0 + (lane & 3) * 2 + (j >> 1) * 8 + (j & 1);
                    bool ok = key < limit[h] && key < item.key_end;
                    if (ok && ses.keep != nullptr) ok = ses.keep[key] != 0;
                    s = ok ? s : -INFINITY;
                }
                sv[h][j] = s;
                mx = fmaxf(mx, s);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[h] = fast_exp2(m_run[h] - m_use);
            m_run[h] = m_new;
#pragma unroll
            for (int j = 0; j < 4; ++j) sv[h][j] = fast_exp2(sv[h][j] - m_use);
        }
        uint32_t pa[4];
        pa[0] = pack2<T>(sv[0][0], sv[0][1]);
        pa[1] = pack2<T>(sv[1][0], sv[1][1]);
        pa[2] = pack2<T>(sv[0][2], sv[0][3]);
        pa[3] = pack2<T>(sv[1][2], sv[1][3]);
        // row sums from the ROUNDED weights the MMA consumes: O / l stays a convex combination
        l_run[0] = l_run[0] * alpha[0] + sum2<T>(pa[0]) + sum2<T>(pa[2]);
        l_run[1] = l_run[1] * alpha[1] + sum2<T>(pa[1]) + sum2<T>(pa[3]);

        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                acc[n][0] *= alpha[0]; acc[n][1] *= alpha[0];
                acc[n][2] *= alpha[1]; acc[n][3] *= alpha[1];
            }
        }

        // ---- O(own half) += P V ----
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, stage + v_off + np * 32);
            mma_16816<T>(acc[2 * np], pa, b[0], b[1]);
            mma_16816<T>(acc[2 * np + 1], pa, b[2], b[3]);
        }
    }

    if (timed_out) {
        // the block that gave up and the one issued behind it may still be landing in this CTA's
        // shared memory: give them a short, bounded chance to finish before the CTA exits
        for (uint32_t b = timed_block; b < n_blocks && b < timed_block + 2; ++b)
            mbar_wait(&bars[b % kStages], (b / kStages) & 1, 1u << 16);
        if (lane == 0) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }

    // ---- write the partial: this warp's half of O, and (warp 0) m and l ----
    const uint32_t rows_total = ses.q_rows * n_q_heads;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = (lane >> 2) + 8 * h;
        if (r >= item.row_count) continue;
        const uint32_t packed = item.row_begin + r;
        const uint32_t rho = (packed / group) * n_q_heads + item.kv_head * group + packed % group;
        const size_t prow = (size_t)ses.partial_base + (size_t)item.part_index * rows_total + rho;
        float *dst = part_o + prow * HD + warp * HH + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n)
            *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(acc[n][2 * h], acc[n][2 * h + 1]);
        if (warp == 0 && (lane & 3) == 0) {
            part_m[prow] = m_run[h] * kLn2;   // natural-log domain, the reference's partial format
            part_l[prow] = l_run[h];
        }
    }
}

// ---------------------------------------------------------------------------------------
// Pass 2. grid = (sessions, rows per session), block = HD/4 threads (one float4 column each).
// mode 0: normalised output in the I/O dtype; mode 1: merged unnormalised (m, d, o) triple.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
attn_decode_combine_kernel(const TTDecodeSession *__restrict__ sessions, const float *__restrict__ part_o,
                           const float *__restrict__ part_m, const float *__restrict__ part_l,
                           uint32_t n_q_heads, uint32_t head_dim, uint32_t out_row_stride, int mode,
                           float *__restrict__ m_out, float *__restrict__ d_out, float *__restrict__ o_out,
                           const __grid_constant__ TTSessionTable table, uint32_t col_threads) {
    // 256 threads = G groups of `col_threads` column threads (one float4 of the row each); group g
    // merges parts g, g+G, ... so that a long session's hundreds of parts are read with many loads
    // in flight instead of one after another. Batches with many (session, row) pairs use one CTA per
    // row (64 column threads, G = 4); a few long sessions split the columns over gridDim.z CTAs
    // (down to 8 column threads, G = 32) so that the merge still fills the machine.
    // One pass: every group keeps an online (max, sum, output) triple over its parts and the groups'
    // triples are merged at the end, so no block-wide reduction over the parts' maxima and sums has
    // to finish before the first output load is issued.
    __shared__ float grp_m[32], grp_d[32];
    __shared__ float4 accs[256];
    pdl_launch_dependents();
    pdl_wait();                       // pass 1 has finished and its partials are visible
    const TTDecodeSession ses = table.n != 0 ? table.s[blockIdx.x] : sessions[blockIdx.x];
    const uint32_t rows_total = ses.q_rows * n_q_heads;
    const uint32_t rho = blockIdx.y;
    if (rho >= rows_total) return;
    const uint32_t n_parts = ses.n_parts;
    const size_t base = (size_t)ses.partial_base + rho;
    const uint32_t grp = threadIdx.x / col_threads, ct = threadIdx.x % col_threads;
    const uint32_t n_groups = 256 / col_threads;
    const uint32_t col = (blockIdx.z * col_threads + ct) * 4;

    float m_run = -INFINITY, d_run = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < head_dim) {
        uint32_t c = grp;
        for (; c + 3 * n_groups < n_parts; c += 4 * n_groups) {   // four independent loads in flight per thread
            float e[4], l[4]; float4 o[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const size_t pr = base + (size_t)(c + n_groups * u) * rows_total;
                e[u] = part_m[pr];
                l[u] = part_l[pr];
                o[u] = *reinterpret_cast<const float4 *>(part_o + pr * head_dim + col);
            }
            const float m_new = fmaxf(m_run, fmaxf(fmaxf(e[0], e[1]), fmaxf(e[2], e[3])));
            if (m_new != -INFINITY) {                              // exp(-inf - -inf) would be NaN
                const float sc = __expf(m_run - m_new);            // 0 for the first finite maximum
                acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc; d_run *= sc;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float wgt = __expf(e[u] - m_new);
                    acc.x += o[u].x * wgt; acc.y += o[u].y * wgt; acc.z += o[u].z * wgt; acc.w += o[u].w * wgt;
                    d_run += l[u] * wgt;
                }
                m_run = m_new;
            }
        }
        for (; c < n_parts; c += n_groups) {
            const size_t pr = base + (size_t)c * rows_total;
            const float e = part_m[pr], l = part_l[pr];
            const float4 o = *reinterpret_cast<const float4 *>(part_o + pr * head_dim + col);
            const float m_new = fmaxf(m_run, e);
            if (m_new != -INFINITY) {
                const float sc = __expf(m_run - m_new), wgt = __expf(e - m_new);
                acc.x = acc.x * sc + o.x * wgt; acc.y = acc.y * sc + o.y * wgt;
                acc.z = acc.z * sc + o.z * wgt; acc.w = acc.w * sc + o.w * wgt;
                d_run = d_run * sc + l * wgt;
                m_run = m_new;
            }
        }
    }
    accs[grp * col_threads + ct] = acc;
    if (ct == 0) { grp_m[grp] = m_run; grp_d[grp] = d_run; }
    __syncthreads();
    if (grp != 0 || col >= head_dim) return;
    float mg = grp_m[0];
    for (uint32_t g = 1; g < n_groups; ++g) mg = fmaxf(mg, grp_m[g]);
    float D = 0.f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mg != -INFINITY)
        for (uint32_t g = 0; g < n_groups; ++g) {
            const float wgt = __expf(grp_m[g] - mg);              // 0 for a group that saw no finite maximum
            const float4 o = accs[g * col_threads + ct];
            acc.x += o.x * wgt; acc.y += o.y * wgt; acc.z += o.z * wgt; acc.w += o.w * wgt;
            D += grp_d[g] * wgt;
        }
    const uint32_t w = rho / n_q_heads, h = rho % n_q_heads;
    if (mode == 0) {
        const float inv = D > 0.f ? 1.f / D : 0.f;
        T *dst = reinterpret_cast<T *>(ses.out) + (size_t)w * out_row_stride + (size_t)h * head_dim + col;
        uint2 packed;
        packed.x = pack2<T>(acc.x * inv, acc.y * inv);
        packed.y = pack2<T>(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2 *>(dst) = packed;
    } else {
        *reinterpret_cast<float4 *>(o_out + (size_t)rho * head_dim + col) = acc;
        if (ct == 0 && blockIdx.z == 0) {
            m_out[rho] = mg;
            d_out[rho] = D;
        }
    }
}

// Merge of externally supplied triples: m,d [n_parts][H]; o [n_parts][H][hd].
template <typename T>
__global__ void attn_combine_parts_kernel(const float *__restrict__ m, const float *__restrict__ d,
                                          const float *__restrict__ o, uint32_t n_parts,
                                          uint32_t n_q_heads, uint32_t head_dim, T *__restrict__ out) {
    const uint32_t h = blockIdx.x;
    float mg = -INFINITY;
    for (uint32_t c = 0; c < n_parts; ++c) mg = fmaxf(mg, m[(size_t)c * n_q_heads + h]);
    float D = 0.f;
    if (mg != -INFINITY)
        for (uint32_t c = 0; c < n_parts; ++c)
            D += d[(size_t)c * n_q_heads + h] * __expf(m[(size_t)c * n_q_heads + h] - mg);
    const float inv = D > 0.f ? 1.f / D : 0.f;
    for (uint32_t col = threadIdx.x; col < head_dim; col += blockDim.x) {
        float acc = 0.f;
        if (mg != -INFINITY)
            for (uint32_t c = 0; c < n_parts; ++c)
                acc += o[((size_t)c * n_q_heads + h) * head_dim + col] *
                       __expf(m[(size_t)c * n_q_heads + h] - mg);
        out[(size_t)h * head_dim + col] = static_cast<T>(acc * inv);
    }
}

template <int HD, int NT, int HPC, typename T>
cudaError_t launch_partial_nt(cudaStream_t stream, uint32_t n_items, const TTDecodeItem *items,
                              const TTDecodeSession *sessions, float *part_o, float *part_m,
                              float *part_l, const tt_attn_batch_params *p, uint32_t *status,
                              const TTSessionTable &table, uint32_t table_keys) {
    auto kernel = attn_decode_partial_kernel<HD, NT, HPC, T>;
    const int smem = DecodeSmem<HD, HPC>::kTotal;
    cudaError_t e = tt_set_smem_once(kernel, smem);
    if (e != cudaSuccess) return e;
    return tt_launch_pdl(kernel, dim3(n_items), dim3(64 * HPC), (size_t)smem, stream, items, sessions, part_o, part_m, part_l,
                         p->n_q_heads, p->n_kv_heads, p->kv_token_stride_elements * 2u, p->q_row_stride_elements,
                         p->scale * kLog2e, status, table, table_keys);
}

// `wide_rows`: some session has more than 8 packed query rows per KV head (two n-tiles per item);
// `hpc`: KV heads served by one CTA (tt_decode_heads_per_cta)
template <int HD, typename T>
cudaError_t launch_partial(cudaStream_t stream, uint32_t n_items, const TTDecodeItem *items,
                           const TTDecodeSession *sessions, float *part_o, float *part_m,
                           float *part_l, const tt_attn_batch_params *p, uint32_t *status,
                           const TTSessionTable &table, uint32_t table_keys, bool wide_rows, uint32_t hpc) {
#define TT_P(NT, HPC) launch_partial_nt<HD, NT, HPC, T>(stream, n_items, items, sessions, part_o, part_m, part_l, p, status, table, table_keys)
    if (hpc == 2) return wide_rows ? TT_P(2, 2) : TT_P(1, 2);
    return wide_rows ? TT_P(2, 1) : TT_P(1, 1);
#undef TT_P
}

template <int HD, int BITS>
cudaError_t launch_partial_quant_one(cudaStream_t stream, uint32_t n_items, const TTDecodeItem *items,
                                     const TTDecodeSession *sessions, float *part_o, float *part_m, float *part_l,
                                     const tt_attn_batch_params *p, uint32_t *status, const TTSessionTable &table,
                                     uint32_t table_keys, const TTKvQuant *quant, uint32_t meta_bytes) {
    auto kernel = attn_decode_partial_quant_kernel<HD, BITS>;
    const int smem = QuantSmem<HD, BITS>::kTotal;
    cudaError_t e = tt_set_smem_once(kernel, smem);
    if (e != cudaSuccess) return e;
    return tt_launch_pdl(kernel, dim3(n_items), dim3(64), (size_t)smem, stream, items, sessions, part_o, part_m, part_l,
                         p->n_q_heads, p->n_kv_heads, quant->stride_bytes, p->q_row_stride_elements, p->scale * kLog2e,
                         status, table, table_keys, quant->value_bytes, meta_bytes);
}

cudaError_t launch_partial_quant(cudaStream_t stream, uint32_t n_items, const TTDecodeItem *items,
                                 const TTDecodeSession *sessions, float *part_o, float *part_m, float *part_l,
                                 const tt_attn_batch_params *p, uint32_t *status, const TTSessionTable &table,
                                 uint32_t table_keys, const TTKvQuant *quant, uint32_t meta_bytes) {
#define TT_Q(HD, BITS) launch_partial_quant_one<HD, BITS>(stream, n_items, items, sessions, part_o, part_m, part_l, p, \
                                                          status, table, table_keys, quant, meta_bytes)
    if (p->head_dim == 256) return quant->bits == 8 ? TT_Q(256, 8) : TT_Q(256, 4);
    return quant->bits == 8 ? TT_Q(128, 8) : TT_Q(128, 4);
#undef TT_Q
}

template <typename T>
cudaError_t launch_partial_hd(cudaStream_t stream, uint32_t n_items, const TTDecodeItem *items,
                              const TTDecodeSession *sessions, float *part_o, float *part_m,
                              float *part_l, const tt_attn_batch_params *p, uint32_t *status,
                              const TTSessionTable &table, uint32_t table_keys, bool wide_rows, uint32_t hpc) {
    switch (p->head_dim) {
        case 64: return launch_partial<64, T>(stream, n_items, items, sessions, part_o, part_m, part_l, p, status, table, table_keys, wide_rows, hpc);
        case 128: return launch_partial<128, T>(stream, n_items, items, sessions, part_o, part_m, part_l, p, status, table, table_keys, wide_rows, hpc);
        case 256: return launch_partial<256, T>(stream, n_items, items, sessions, part_o, part_m, part_l, p, status, table, table_keys, wide_rows, hpc);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Host side: split planning (pure arithmetic) and the launcher.
// ---------------------------------------------------------------------------------------
static uint32_t ceil_div_u32(uint64_t a, uint64_t b) { return (uint32_t)((a + b - 1) / b); }

// KV heads one pass-1 CTA of the fp16/bf16 kernel serves: adjacent pairs when the head count is
// even, so that whole cache rows are streamed (quantised rows keep one head per CTA).
static uint32_t tt_decode_heads_per_cta(uint32_t n_kv_heads, bool quantised) {
    return (!quantised && n_kv_heads % 2 == 0) ? 2u : 1u;
}

static int plan_splits(const uint32_t *keys_per_session, const uint32_t *q_rows_per_session,
                       uint32_t n_sessions, uint32_t head_dim, uint32_t n_q_heads,
                       uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes, uint32_t heads_per_cta,
                       uint32_t *out_keys_per_item, uint32_t *out_n_items);

TT_API int tt_attn_plan_splits(const uint32_t *keys_per_session, const uint32_t *q_rows_per_session,
                               uint32_t n_sessions, uint32_t head_dim, uint32_t n_q_heads,
                               uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes,
                               uint32_t *out_keys_per_item, uint32_t *out_n_items) {
    return plan_splits(keys_per_session, q_rows_per_session, n_sessions, head_dim, n_q_heads, n_kv_heads, sm_count,
                       workspace_bytes, n_kv_heads ? tt_decode_heads_per_cta(n_kv_heads, false) : 1u, out_keys_per_item,
                       out_n_items);
}

static int plan_splits(const uint32_t *keys_per_session, const uint32_t *q_rows_per_session,
                       uint32_t n_sessions, uint32_t head_dim, uint32_t n_q_heads,
                       uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes, uint32_t heads_per_cta,
                       uint32_t *out_keys_per_item, uint32_t *out_n_items) {
    if (keys_per_session == nullptr || n_sessions == 0 || n_kv_heads == 0 || n_q_heads % n_kv_heads != 0 ||
        head_dim == 0 || sm_count == 0)
        return TT_ERR_INVALID_ARG;
    const uint32_t group = n_q_heads / n_kv_heads;
    const uint32_t rows_per_item = 16u;
    const uint32_t units_per_part = n_kv_heads / heads_per_cta;      // CTAs per (session, part, row tile)
    // Items and partial rows of a candidate item length.
    auto count = [&](uint32_t keys, uint64_t *items, uint64_t *prows) {
        *items = 0; *prows = 0;
        for (uint32_t i = 0; i < n_sessions; ++i) {
            const uint32_t qr = q_rows_per_session ? q_rows_per_session[i] : 1u;
            const uint32_t tiles = ceil_div_u32((uint64_t)qr * group, rows_per_item);
            uint32_t parts = ceil_div_u32(keys_per_session[i], keys);
            if (parts == 0) parts = 1;  // an empty range still produces its (-inf, 0, 0) partial
            *items += (uint64_t)parts * units_per_part * tiles;
            *prows += (uint64_t)parts * qr * n_q_heads;
        }
    };
    // The kernel is HBM-bound and its items are equal slices, so what matters is how the items fill the
    // CTA slots of the machine (4 / heads_per_cta per SM): a launch of exactly `waves` full waves ends
    // with every SM busy, one of 1.5 waves leaves half the machine idle for a third of the time
    // (measured on one 262,144-key session: 90 us at one wave, 120 us at 1.5, 104 us at three). The item
    // length is therefore the SHORTEST multiple of the 16-key block for which the items fit `waves`
    // waves: one wave when a handful of long streams divide evenly (fewest partials to merge), three
    // when many ragged sessions need the scheduler to even them out. TT_DECODE_WAVES overrides the
    // choice (an experiment knob).
    const uint64_t slots = (uint64_t)sm_count * (4u / heads_per_cta);
    static const uint32_t waves_env = getenv("TT_DECODE_WAVES") ? (uint32_t)atoi(getenv("TT_DECODE_WAVES")) : 0u;
    uint64_t streams = 0, max_keys = 0;
    for (uint32_t i = 0; i < n_sessions; ++i) {
        const uint32_t qr = q_rows_per_session ? q_rows_per_session[i] : 1u;
        streams += (uint64_t)units_per_part * ceil_div_u32((uint64_t)qr * group, rows_per_item);
        if (keys_per_session[i] > max_keys) max_keys = keys_per_session[i];
    }
    uint32_t waves = waves_env ? waves_env : (streams * 8 <= slots ? 1u : 3u);
    uint32_t keys = 64;
    if (streams >= waves * slots) {
        keys = 1u << 30;                    // more streams than slots: one item per stream, nothing to split
    } else {
        // smallest multiple of 16 (at least 64) whose item count fits: the count falls as the length grows
        uint32_t lo = 4, hi = (uint32_t)((max_keys + 15) / 16);      // in 16-key blocks
        if (hi < lo) hi = lo;
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2;
            uint64_t items, prows;
            count(mid * 16, &items, &prows);
            if (items <= waves * slots) hi = mid; else lo = mid + 1;
        }
        keys = lo * 16;
    }
    for (;;) {
        uint64_t items, prows;
        count(keys, &items, &prows);
        const uint64_t need = prows * ((uint64_t)head_dim + 2) * sizeof(float);
        if (workspace_bytes == 0 || need <= workspace_bytes || keys >= (1u << 30)) {
            if (workspace_bytes != 0 && need > workspace_bytes) return TT_ERR_OOM;
            if (out_keys_per_item) *out_keys_per_item = keys;
            if (out_n_items) *out_n_items = (uint32_t)items;
            return TT_OK;
        }
        keys *= 2;
    }
}

TT_API void tt_attn_reference_split_geometry(uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t seq_len,
                                             uint32_t kv_start, int prefer_gqa_swa,
                                             tt_split_geometry *out) {
    // Attention.swift:59-64 (defaultFullChunks 16, defaultGQASWAChunks 8, maxChunks 64), :196-227.
    if (out == nullptr || n_kv_heads == 0) return;
    const int q_per_kv = (int)(n_q_heads / n_kv_heads);
    const bool swa_grouped = prefer_gqa_swa && q_per_kv <= 2;
    const int eff = (int)seq_len - (int)kv_start;
    const int eff1 = eff < 1 ? 1 : eff;
    const int def = swa_grouped ? 8 : 16;
    int base = def < 64 ? def : 64;
    if (eff1 < base) base = eff1;
    if (base < 1) base = 1;
    int chunks = base;
    if (swa_grouped) {
        int widened = base * q_per_kv;
        if (widened > 64) widened = 64;
        if (widened > chunks) chunks = widened;
    }
    out->effective_length = (uint32_t)eff;
    out->num_chunks = (uint32_t)chunks;
    out->chunk_length = (uint32_t)((eff1 + chunks - 1) / chunks);
    out->partial_threadgroups = (uint32_t)((swa_grouped ? (int)n_kv_heads : (int)n_q_heads) * chunks);
    out->use_swa_grouped_partial = swa_grouped ? 1u : 0u;
}

int tt_verify_tc_encode_maps(tt_context *ctx, uint32_t n_sessions, const tt_attn_batch_params *p, void *dst_maps);
int tt_launch_verify_tc(tt_context *ctx, cudaStream_t stream, uint32_t n_sessions, uint32_t n_items, float *part_o,
                        float *part_m, float *part_l, const tt_attn_batch_params *p, bool direct, bool in_params,
                        bool rows128);

// Split plan of the tensor-core verify pass: one item per (session, kv head, key range) serving all
// packed rows, the parts of one session of equal length (a multiple of the 128-key tile). One CTA is
// resident per SM and an item costs about two tiles of start-up on top of its own tiles, so the part
// length is picked by simulating the hardware's in-order dispatch of the items over the SMs for a
// few candidate lengths and keeping the shortest makespan. False when the partials or the items do
// not fit the context.
static uint64_t wide_makespan(const uint32_t *keys, uint32_t n_sessions, uint32_t n_kv_heads, uint32_t len,
                              uint32_t sm_count, std::vector<uint32_t> &heap) {
    constexpr uint32_t kStartupTiles = 2;
    heap.assign(sm_count, 0u);   // min-heap of SM finish times (in tiles)
    auto sift_down = [&](uint32_t i) {
        const uint32_t n = (uint32_t)heap.size();
        for (;;) {
            uint32_t l = 2 * i + 1, r = l + 1, m = i;
            if (l < n && heap[l] < heap[m]) m = l;
            if (r < n && heap[r] < heap[m]) m = r;
            if (m == i) return;
            std::swap(heap[i], heap[m]);
            i = m;
        }
    };
    uint32_t makespan = 0;
    for (uint32_t i = 0; i < n_sessions; ++i) {
        uint32_t parts = ceil_div_u32(keys[i], len);
        if (parts == 0) parts = 1;
        const uint32_t part_len = (ceil_div_u32(keys[i], parts) + 127) / 128 * 128;
        for (uint32_t part = 0; part < parts; ++part) {
            const uint32_t begin = part * part_len;
            const uint32_t n = keys[i] > begin ? (keys[i] - begin < part_len ? keys[i] - begin : part_len) : 0u;
            const uint32_t cost = kStartupTiles + (n + 127) / 128;
            for (uint32_t h = 0; h < n_kv_heads; ++h) {
                heap[0] += cost;
                if (heap[0] > makespan) makespan = heap[0];
                sift_down(0);
            }
        }
    }
    return makespan;
}

// Part length (a multiple of 128) of the tensor-core verify pass, 0 when nothing fits.
static uint32_t wide_part_length(const uint32_t *keys, const uint32_t *q_rows, uint32_t n_sessions, uint32_t head_dim,
                                 uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes,
                                 uint32_t max_items) {
    uint32_t max_keys = 0;
    for (uint32_t i = 0; i < n_sessions; ++i) max_keys = keys[i] > max_keys ? keys[i] : max_keys;
    // Part counts tried for the longest session (every candidate costs a simulation on the host, so
    // there are few). Few streams (fewer than SMs) are best cut so that ONE wave of items just fills
    // the machine, i.e. into about SMs / streams parts: the counts around that value are tried next
    // to the coarse ladder.
    static const uint32_t kCoarse[] = {1, 2, 3, 4, 5, 6, 8, 10, 12, 16, 20, 24, 32, 48, 64};
    std::vector<uint32_t> choices;
    const uint32_t streams = n_sessions * n_kv_heads;
    if (streams < sm_count) {
        const uint32_t fill = sm_count / streams;
        for (uint32_t c = fill > 2 ? fill - 2 : 1; c <= fill + 1 && c <= 64; ++c) choices.push_back(c);
        for (uint32_t c : kCoarse)
            if (c < fill && std::find(choices.begin(), choices.end(), c) == choices.end()) choices.push_back(c);
    } else {
        choices.assign(kCoarse, kCoarse + sizeof(kCoarse) / sizeof(kCoarse[0]));
    }
    std::sort(choices.begin(), choices.end());
    std::vector<uint32_t> heap;
    uint64_t best = ~(uint64_t)0;
    uint32_t target = 0;
    for (uint32_t parts : choices) {
        uint32_t len = (ceil_div_u32(max_keys, parts) + 127) / 128 * 128;
        if (len < 512) len = 512;                 // at least four tiles per item
        uint64_t items = 0, prows = 0;
        for (uint32_t i = 0; i < n_sessions; ++i) {
            uint32_t np = ceil_div_u32(keys[i], len);
            if (np == 0) np = 1;
            items += (uint64_t)np * n_kv_heads;
            prows += (uint64_t)np * (q_rows ? q_rows[i] : 1u) * n_q_heads;
        }
        if ((workspace_bytes != 0 && prows * ((uint64_t)head_dim + 2) * sizeof(float) > workspace_bytes) ||
            items > max_items || items > 8192) {
            if (len == 512) break;
            continue;
        }
        const uint64_t span = wide_makespan(keys, n_sessions, n_kv_heads, len, sm_count, heap);
        if (span < best) { best = span; target = len; }
        if (len == 512) break;
    }
    return target;
}

// The verify plan as pure arithmetic (what the launcher uses): for every session the number of
// parts and their common length; sum(parts) * n_kv_heads items in all.
TT_API int tt_attn_plan_verify_splits(const uint32_t *keys_per_session, const uint32_t *q_rows_per_session,
                                      uint32_t n_sessions, uint32_t head_dim, uint32_t n_q_heads,
                                      uint32_t n_kv_heads, uint32_t sm_count, size_t workspace_bytes,
                                      uint32_t *out_parts, uint32_t *out_part_len, uint32_t *out_n_items) {
    if (keys_per_session == nullptr || n_sessions == 0 || n_kv_heads == 0 || n_q_heads % n_kv_heads != 0 ||
        head_dim == 0 || sm_count == 0)
        return TT_ERR_INVALID_ARG;
    const uint32_t target = wide_part_length(keys_per_session, q_rows_per_session, n_sessions, head_dim, n_q_heads,
                                             n_kv_heads, sm_count, workspace_bytes, 65536u);
    if (target == 0) return TT_ERR_OOM;
    uint32_t items = 0;
    for (uint32_t i = 0; i < n_sessions; ++i) {
        uint32_t parts = ceil_div_u32(keys_per_session[i], target);
        if (parts == 0) parts = 1;
        if (out_parts) out_parts[i] = parts;
        if (out_part_len) out_part_len[i] = (ceil_div_u32(keys_per_session[i], parts) + 127) / 128 * 128;
        items += parts * n_kv_heads;
    }
    if (out_n_items) *out_n_items = items;
    return TT_OK;
}

static bool plan_wide(tt_context *ctx, const TTDecodeSession *in_sessions, uint32_t n_sessions,
                      const tt_attn_batch_params *p, const uint32_t *keys, uint32_t *out_items,
                      uint32_t *out_partial_rows, uint32_t *out_max_rows) {
    // the simulation behind the part length costs tens of microseconds on the host: reuse the last
    // plan while its inputs (tile counts, row counts, head geometry) are unchanged
    std::vector<uint32_t> &key = ctx->verify_plan_key;
    bool same = key.size() == 2 * (size_t)n_sessions + 3 && key[0] == p->n_q_heads && key[1] == p->n_kv_heads &&
                key[2] == p->head_dim;
    for (uint32_t i = 0; same && i < n_sessions; ++i)
        same = key[3 + 2 * i] == (keys[i] + 127) / 128 && key[4 + 2 * i] == ctx->h_rows[i];
    if (!same) {
        ctx->verify_plan_target = wide_part_length(keys, ctx->h_rows, n_sessions, p->head_dim, p->n_q_heads,
                                                   p->n_kv_heads, (uint32_t)ctx->sm_count, ctx->workspace_bytes,
                                                   ctx->max_items);
        key.resize(2 * (size_t)n_sessions + 3);
        key[0] = p->n_q_heads; key[1] = p->n_kv_heads; key[2] = p->head_dim;
        for (uint32_t i = 0; i < n_sessions; ++i) {
            key[3 + 2 * i] = (keys[i] + 127) / 128;
            key[4 + 2 * i] = ctx->h_rows[i];
        }
    }
    const uint32_t target = ctx->verify_plan_target;
    if (target == 0) return false;
    uint32_t partial_cursor = 0, item_cursor = 0, max_rows = 0;
    const uint32_t group = p->n_q_heads / p->n_kv_heads;
    for (uint32_t i = 0; i < n_sessions; ++i) {
        TTDecodeSession s = in_sessions[i];
        uint32_t parts = ceil_div_u32(keys[i], target);
        if (parts == 0) parts = 1;
        const uint32_t len = (ceil_div_u32(keys[i], parts) + 127) / 128 * 128;
        const uint32_t rows_total = s.q_rows * p->n_q_heads;
        s.n_parts = parts;
        s.partial_base = partial_cursor;
        ctx->h_sessions[i] = s;
        if (n_sessions <= kVerifyParamSessions) {      // the parameter form: the kernel derives the same items
            ctx->session_table.s[i] = s;
            ctx->session_table.item_prefix[i] = item_cursor;
        }
        if (rows_total > max_rows) max_rows = rows_total;
        for (uint32_t part = 0; part < parts; ++part) {
            const uint32_t kb = s.kv_start + part * len;
            uint32_t ke = kb + len;
            if (ke > s.seq_len) ke = s.seq_len;
            if (ke < kb) ke = kb;
            for (uint32_t kvh = 0; kvh < p->n_kv_heads; ++kvh) {
                TTDecodeItem &it = ctx->h_items[item_cursor++];
                it.session = i; it.kv_head = kvh; it.key_begin = kb; it.key_end = ke;
                it.part_index = part; it.row_begin = 0; it.row_count = s.q_rows * group;
                it.partial_base = s.partial_base;
            }
        }
        partial_cursor += parts * rows_total;
    }
    if (n_sessions <= kVerifyParamSessions) {
        ctx->session_table.item_prefix[n_sessions] = item_cursor;
        ctx->session_table.n = n_sessions;
    }
    *out_items = item_cursor; *out_partial_rows = partial_cursor; *out_max_rows = max_rows;
    return true;
}

// mode 0: write normalised outputs to the sessions' `out`; mode 1: one merged triple for a
// single session (m_out/d_out/o_out); mode 2: a single one-row session whose local merge is fused
// with the cross-GPU exchange (`exchange`).
int tt_launch_decode(tt_context *ctx, cudaStream_t stream, const TTDecodeSession *in_sessions,
                     uint32_t n_sessions, const tt_attn_batch_params *p, int mode, float *m_out,
                     float *d_out, float *o_out, const TTKvQuant *quant, const tt_attn_exchange *exchange) {
    if (n_sessions == 0) return TT_OK;
    if (mode == 2 && (exchange == nullptr || n_sessions != 1 || in_sessions[0].q_rows != 1))
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "the fused exchange serves one session with one query row");
    if (n_sessions > ctx->max_sessions)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_sessions %u exceeds the context's max_sessions %u",
                            n_sessions, ctx->max_sessions);
    if (p->n_kv_heads == 0 || p->n_q_heads == 0 || p->n_q_heads % p->n_kv_heads != 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_q_heads must be a multiple of n_kv_heads");
    if (p->head_dim != 64 && p->head_dim != 128 && p->head_dim != 256)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "decode attention supports head_dim 64/128/256, got %u",
                            p->head_dim);
    if (p->io_dtype != TT_F16 && p->io_dtype != TT_BF16)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "io_dtype must be TT_F16 or TT_BF16");
    const bool quantised = quant != nullptr && quant->bits != 16;
    uint32_t meta_bytes = 0;
    if (quantised) {
        if (quant->bits != 8 && quant->bits != 4) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "KV bits must be 4, 8, or 16");
        if (p->head_dim != 128 && p->head_dim != 256)
            return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "quantised KV rows need head_dim 128 or 256");
        if (p->io_dtype != TT_F16) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "quantised KV rows need fp16 queries");
        const uint32_t groups = p->n_kv_heads * p->head_dim / 64;
        meta_bytes = (groups * 4 + 15) / 16 * 16;
        const uint32_t packed = p->n_kv_heads * p->head_dim * quant->bits / 8;
        if (meta_bytes > 64 || quant->value_bytes != packed || quant->value_bytes % 16 != 0 ||
            quant->stride_bytes % 16 != 0 || quant->stride_bytes < quant->value_bytes + meta_bytes)
            return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE,
                                "quantised KV row layout not supported (stride %u, values %u, %u groups)",
                                quant->stride_bytes, quant->value_bytes, groups);
    }
    if ((!quantised && p->kv_token_stride_elements < p->n_kv_heads * p->head_dim) ||
        p->q_row_stride_elements < p->n_q_heads * p->head_dim ||
        p->out_row_stride_elements < p->n_q_heads * p->head_dim)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "a row stride is smaller than its tight width");
    if ((p->kv_token_stride_elements % 8) || (p->q_row_stride_elements % 8) || (p->out_row_stride_elements % 4))
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "row strides must keep rows 16-byte aligned");
    const uint32_t group = p->n_q_heads / p->n_kv_heads;

    uint32_t *keys = ctx->h_keys, *rows = ctx->h_rows;
    for (uint32_t i = 0; i < n_sessions; ++i) {
        const TTDecodeSession &s = in_sessions[i];
        if (s.q == nullptr || s.k == nullptr || s.v == nullptr || (mode == 0 && s.out == nullptr))
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "session %u has a null buffer", i);
        if (s.q_rows == 0 || s.q_rows > 64)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "session %u: q_rows must be in 1..64", i);
        if (s.seq_len + 1 < s.q_rows)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "session %u: seq_len %u cannot hold %u query rows", i,
                                s.seq_len, s.q_rows);
        if (((uintptr_t)s.q | (uintptr_t)s.k | (uintptr_t)s.v | (uintptr_t)s.out) & 15)
            return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "session %u: buffers must be 16-byte aligned", i);
        keys[i] = s.seq_len > s.kv_start ? s.seq_len - s.kv_start : 0u;
        rows[i] = s.q_rows;
    }
    // Verify batches (17..128 packed rows per KV head, head_dim 256, plain 16-bit rows) take the
    // tensor-core pass 1: one item serves all packed rows of a (session, kv head, key range).
    bool wide = !quantised && p->head_dim == 256 && getenv("TT_VERIFY_FORCE_MMA_SYNC") == nullptr;
    bool wide128 = false;       // some session has more than 64 packed rows: the 128-row form of the kernel
    for (uint32_t i = 0; wide && i < n_sessions; ++i) {
        const TTDecodeSession &s = in_sessions[i];
        const uint32_t packed = s.q_rows * group;
        wide = packed > 16 && packed <= 128 && s.ring_capacity == 0 && s.keep == nullptr && s.row_index == nullptr;
        wide128 |= packed > 64;
    }

    tt_bind_decode_tables(ctx, n_sessions, wide);
    uint32_t keys_per_item = 0, n_items = 0;
    uint32_t partial_cursor = 0, item_cursor = 0, max_rows = 0;
    TTSessionTable &table = ctx->session_table;
    table.n = 0;
    if (wide) wide = plan_wide(ctx, in_sessions, n_sessions, p, keys, &n_items, &partial_cursor, &max_rows);
    if (!wide) table.n = 0;
    // Up to kParamSessions sessions (kVerifyParamSessions of a verify batch, whose tensor maps travel
    // too) go in the kernel parameters: nothing is uploaded and the item table is not read (a CTA
    // derives its item from the block index).
    const bool in_params = wide ? n_sessions <= kVerifyParamSessions : n_sessions <= kParamSessions;
    const uint32_t hpc = tt_decode_heads_per_cta(p->n_kv_heads, quantised);
    if (!wide) {
        int rc = plan_splits(keys, rows, n_sessions, p->head_dim, p->n_q_heads, p->n_kv_heads, (uint32_t)ctx->sm_count,
                             ctx->workspace_bytes, hpc, &keys_per_item, &n_items);
        if (rc != TT_OK) return tt_set_error(ctx, rc, "split-KV partials do not fit the context workspace");
        if (!in_params && n_items > ctx->max_items)
            return tt_set_error(ctx, TT_ERR_OOM, "%u work items exceed the context's item table (%u)", n_items,
                                ctx->max_items);

        const uint32_t rows_per_item = 16u;
        // Build the session table and, for the device-table form, the item table.
        for (uint32_t i = 0; i < n_sessions; ++i) {
            TTDecodeSession s = in_sessions[i];
            uint32_t parts = ceil_div_u32(keys[i], keys_per_item);
            if (parts == 0) parts = 1;
            const uint32_t rows_total = s.q_rows * p->n_q_heads;
            s.n_parts = parts;
            s.partial_base = partial_cursor;
            ctx->h_sessions[i] = s;
            if (rows_total > max_rows) max_rows = rows_total;
            const uint32_t packed_rows = s.q_rows * group;
            if (in_params) {
                table.s[i] = s;
                table.item_prefix[i] = item_cursor;
                item_cursor += parts * (p->n_kv_heads / hpc) * ceil_div_u32(packed_rows, rows_per_item);
            } else {
                for (uint32_t part = 0; part < parts; ++part) {
                    const uint32_t kb = s.kv_start + part * keys_per_item;
                    uint32_t ke = kb + keys_per_item;
                    if (ke > s.seq_len) ke = s.seq_len;
                    if (ke < kb) ke = kb;
                    for (uint32_t kvh = 0; kvh < p->n_kv_heads; kvh += hpc)
                        for (uint32_t rb = 0; rb < packed_rows; rb += rows_per_item) {
                            TTDecodeItem &it = ctx->h_items[item_cursor++];
                            it.session = i; it.kv_head = kvh; it.key_begin = kb; it.key_end = ke;
                            it.part_index = part; it.row_begin = rb;
                            it.row_count = packed_rows - rb < rows_per_item ? packed_rows - rb : rows_per_item;
                            it.partial_base = s.partial_base;
                        }
                }
            }
            partial_cursor += parts * rows_total;
        }
        if (item_cursor != n_items) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "internal: item count mismatch");
        if (in_params) {
            table.item_prefix[n_sessions] = item_cursor;
            table.n = n_sessions;
        }
    }

    float *part_o = ctx->partials;
    float *part_m = part_o + (size_t)partial_cursor * p->head_dim;
    float *part_l = part_m + partial_cursor;

    const uint32_t table_keys = in_params ? keys_per_item : 0u;
    bool wide_rows = false;             // more than 8 packed query rows per KV head somewhere: two n-tiles per item
    for (uint32_t i = 0; i < n_sessions; ++i) wide_rows |= in_sessions[i].q_rows * group > 8;
    cudaError_t e = cudaSuccess;
    if (wide) {
        const int rc = tt_verify_tc_encode_maps(ctx, n_sessions, p, in_params ? (void *)ctx->verify_maps.m : ctx->h_tensor_maps);
        if (rc != TT_OK) return rc;
    }
    if (!in_params) {
        // sessions, maps and items sit back to back: one upload
        const size_t bytes = (size_t)(reinterpret_cast<unsigned char *>(ctx->h_items + n_items) - ctx->h_tables);
        e = cudaMemcpyAsync(ctx->tables, ctx->h_tables, bytes, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "copy decode tables");
    }

    TTLaunchTimer timer(ctx, stream, TT_PROFILE_DECODE_PARTIAL);
    // a verify batch whose sessions are all one part needs no merge: pass 1 stores the output rows
    bool direct = wide && mode == 0;
    for (uint32_t i = 0; direct && i < n_sessions; ++i) direct = ctx->h_sessions[i].n_parts == 1;
    if (wide) {
        const int rc = tt_launch_verify_tc(ctx, stream, n_sessions, n_items, part_o, part_m, part_l, p, direct, in_params, wide128);
        if (rc != TT_OK) return rc;
    } else if (quantised)
        e = launch_partial_quant(stream, n_items, ctx->items, ctx->sessions, part_o, part_m, part_l, p, ctx->status,
                                 table, table_keys, quant, meta_bytes);
    else if (p->io_dtype == TT_F16)
        e = launch_partial_hd<__half>(stream, n_items, ctx->items, ctx->sessions, part_o, part_m, part_l, p, ctx->status,
                                      table, table_keys, wide_rows, hpc);
    else
        e = launch_partial_hd<__nv_bfloat16>(stream, n_items, ctx->items, ctx->sessions, part_o, part_m, part_l, p,
                                             ctx->status, table, table_keys, wide_rows, hpc);
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_decode_partial launch");
    timer.stop();
    ctx->launches++;
    if (direct) return TT_OK;
    if (mode == 2)
        return tt_launch_merge_exchange(ctx, stream, part_o, part_m, part_l, ctx->h_sessions[0].n_parts, exchange,
                                        p->n_q_heads, p->head_dim, p->io_dtype);

    // few (session, row) pairs: split the row's columns over several CTAs so the merge fills the GPU
    uint32_t col_threads = 64;
    while (col_threads > 8 && (uint64_t)n_sessions * max_rows * (64 / col_threads) * 2 <= (uint64_t)ctx->sm_count)
        col_threads /= 2;
    const dim3 grid(n_sessions, max_rows, (p->head_dim / 4 + col_threads - 1) / col_threads);
    const dim3 threads(256);
    if (p->io_dtype == TT_F16)
        e = tt_launch_pdl(attn_decode_combine_kernel<__half>, grid, threads, 0, stream, ctx->sessions, part_o, part_m, part_l,
                          p->n_q_heads, p->head_dim, p->out_row_stride_elements, mode, m_out, d_out, o_out, table, col_threads);
    else
        e = tt_launch_pdl(attn_decode_combine_kernel<__nv_bfloat16>, grid, threads, 0, stream, ctx->sessions, part_o, part_m,
                          part_l, p->n_q_heads, p->head_dim, p->out_row_stride_elements, mode, m_out, d_out, o_out, table,
                          col_threads);
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_decode_combine launch");
    e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_decode_combine launch");
    ctx->launches++;
    return TT_OK;
}

// ---------------------------------------------------------------------------------------
// C entry points.
// ---------------------------------------------------------------------------------------
TT_API int tt_attn_decode_batched(tt_context *ctx, tt_stream stream, const tt_attn_session *sessions,
                                  uint32_t n_sessions, const tt_attn_batch_params *params) {
    TT_ENTER(ctx);
    if (sessions == nullptr || params == nullptr)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "sessions and params must not be null");
    if (n_sessions > ctx->max_sessions)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_sessions %u exceeds the context's max_sessions %u",
                            n_sessions, ctx->max_sessions);
    TTDecodeSession *tmp = ctx->h_sessions_in;
    for (uint32_t i = 0; i < n_sessions; ++i) {
        TTDecodeSession &d = tmp[i];
        d.q = sessions[i].q; d.out = sessions[i].out; d.k = sessions[i].k; d.v = sessions[i].v;
        d.seq_len = sessions[i].seq_len; d.q_rows = sessions[i].q_rows; d.kv_start = sessions[i].kv_start;
        d.n_parts = 0; d.partial_base = 0; d.ring_capacity = 0; d.keep = nullptr; d.row_index = nullptr;
    }
    return tt_launch_decode(ctx, (cudaStream_t)stream, tmp, n_sessions, params, 0, nullptr, nullptr, nullptr);
}

static int decode_one(tt_context *ctx, tt_stream stream, const void *q, const void *k, const void *v,
                      void *out, uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads,
                      uint32_t seq_len, uint32_t kv_start, float scale, const tt_kv_format *kv_format,
                      const uint8_t *keep_mask, uint32_t ring_capacity, const uint32_t *row_index) {
    if (head_dim > 512) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "head_dim must be <= 512");
    if (n_kv_heads == 0 || n_q_heads % n_kv_heads != 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_q_heads must be a multiple of n_kv_heads for GQA");
    if (n_q_heads > 96) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "n_q_heads exceeds 96");
    uint32_t stride_elems = n_kv_heads * head_dim;
    TTKvQuant quant;
    if (kv_format != nullptr) {
        if (kv_format->bits != 16 && kv_format->bits != 8 && kv_format->bits != 4)
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "KV bits must be 4, 8, or 16");
        if (kv_format->bits != 16) {
            if (kv_format->group_size != 64)
                return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "quantisation group size must be 64");
            quant.bits = kv_format->bits; quant.stride_bytes = kv_format->stride_bytes; quant.value_bytes = kv_format->value_bytes;
        }
        if (kv_format->stride_bytes != 0) {
            if (kv_format->stride_bytes % 2) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "odd KV stride");
            stride_elems = kv_format->stride_bytes / 2;
        }
    }
    tt_attn_batch_params p;
    p.head_dim = head_dim; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
    p.kv_token_stride_elements = stride_elems; p.q_row_stride_elements = n_q_heads * head_dim;
    p.out_row_stride_elements = n_q_heads * head_dim; p.scale = scale; p.io_dtype = TT_F16;
    TTDecodeSession s;
    s.q = q; s.out = out; s.k = k; s.v = v; s.seq_len = seq_len; s.q_rows = 1;
    s.kv_start = kv_start < seq_len ? kv_start : seq_len;
    s.n_parts = 0; s.partial_base = 0; s.ring_capacity = ring_capacity; s.keep = keep_mask; s.row_index = row_index;
    return tt_launch_decode(ctx, (cudaStream_t)stream, &s, 1, &p, 0, nullptr, nullptr, nullptr, &quant);
}

TT_API int tt_attn_decode(tt_context *ctx, tt_stream stream, const void *q, const void *k, const void *v,
                          void *out, uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads,
                          uint32_t seq_len, uint32_t kv_start, float scale, const tt_kv_format *kv_format,
                          const uint8_t *keep_mask, uint32_t ring_capacity) {
    TT_ENTER(ctx);
    return decode_one(ctx, stream, q, k, v, out, head_dim, n_q_heads, n_kv_heads, seq_len, kv_start, scale, kv_format,
                      keep_mask, ring_capacity, nullptr);
}

TT_API int tt_attn_decode_window(tt_context *ctx, tt_stream stream, const void *q, const void *k, const void *v,
                                 void *out, uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads,
                                 uint32_t sel_count, float scale, const tt_kv_format *kv_format,
                                 const uint32_t *sel_rows) {
    TT_ENTER(ctx);
    if (sel_rows == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "a windowed selection needs its row list");
    return decode_one(ctx, stream, q, k, v, out, head_dim, n_q_heads, n_kv_heads, sel_count, 0, scale, kv_format,
                      nullptr, 0, sel_rows);
}

TT_API int tt_attn_decode_partial(tt_context *ctx, tt_stream stream, const void *q, const void *k,
                                  const void *v, uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads,
                                  uint32_t seq_len, uint32_t kv_start, float scale,
                                  uint32_t kv_token_stride_elements, uint32_t io_dtype, float *m_out,
                                  float *d_out, float *o_out) {
    TT_ENTER(ctx);
    if (m_out == nullptr || d_out == nullptr || o_out == nullptr)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "partial outputs must not be null");
    tt_attn_batch_params p;
    p.head_dim = head_dim; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
    p.kv_token_stride_elements = kv_token_stride_elements ? kv_token_stride_elements : n_kv_heads * head_dim;
    p.q_row_stride_elements = n_q_heads * head_dim; p.out_row_stride_elements = n_q_heads * head_dim;
    p.scale = scale; p.io_dtype = io_dtype;
    TTDecodeSession s;
    s.q = q; s.out = nullptr; s.k = k; s.v = v; s.seq_len = seq_len; s.q_rows = 1;
    s.kv_start = kv_start < seq_len ? kv_start : seq_len;
    s.n_parts = 0; s.partial_base = 0; s.ring_capacity = 0; s.keep = nullptr; s.row_index = nullptr;
    return tt_launch_decode(ctx, (cudaStream_t)stream, &s, 1, &p, 1, m_out, d_out, o_out);
}

TT_API int tt_attn_decode_exchange(tt_context *ctx, tt_stream stream, const void *q, const void *k, const void *v,
                                   uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t seq_len,
                                   uint32_t kv_start, float scale, uint32_t kv_token_stride_elements,
                                   uint32_t io_dtype, const tt_attn_exchange *x) {
    TT_ENTER(ctx);
    if (x == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange descriptor must not be null");
    tt_attn_batch_params p;
    p.head_dim = head_dim; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
    p.kv_token_stride_elements = kv_token_stride_elements ? kv_token_stride_elements : n_kv_heads * head_dim;
    p.q_row_stride_elements = n_q_heads * head_dim; p.out_row_stride_elements = n_q_heads * head_dim;
    p.scale = scale; p.io_dtype = io_dtype;
    TTDecodeSession s;
    s.q = q; s.out = nullptr; s.k = k; s.v = v; s.seq_len = seq_len; s.q_rows = 1;
    s.kv_start = kv_start < seq_len ? kv_start : seq_len;
    s.n_parts = 0; s.partial_base = 0; s.ring_capacity = 0; s.keep = nullptr; s.row_index = nullptr;
    return tt_launch_decode(ctx, (cudaStream_t)stream, &s, 1, &p, 2, nullptr, nullptr, nullptr, nullptr, x);
}

TT_API int tt_attn_combine(tt_context *ctx, tt_stream stream, const float *m, const float *d, const float *o,
                           uint32_t n_parts, uint32_t n_q_heads, uint32_t head_dim, void *out,
                           uint32_t io_dtype) {
    TT_ENTER(ctx);
    if (m == nullptr || d == nullptr || o == nullptr || out == nullptr || n_parts == 0 || n_q_heads == 0 ||
        head_dim == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "combine needs non-null buffers and positive sizes");
    const uint32_t threads = head_dim < 256 ? ((head_dim + 31) / 32) * 32 : 256;
    if (io_dtype == TT_F16)
        attn_combine_parts_kernel<__half><<<n_q_heads, threads, 0, (cudaStream_t)stream>>>(
            m, d, o, n_parts, n_q_heads, head_dim, reinterpret_cast<__half *>(out));
    else if (io_dtype == TT_BF16)
        attn_combine_parts_kernel<__nv_bfloat16><<<n_q_heads, threads, 0, (cudaStream_t)stream>>>(
            m, d, o, n_parts, n_q_heads, head_dim, reinterpret_cast<__nv_bfloat16 *>(out));
    else
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "io_dtype must be TT_F16 or TT_BF16");
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_combine launch");
    ctx->launches++;
    return TT_OK;
}

// ---------------------------------------------------------------------------------------
// Single-query decode attention that allocates nothing.
//
// Some callers cannot allocate device memory: a plugin that runs inside another process's
// real-time or capture-restricted section, a host whose memory budget was handed out in full
// before this library was loaded (the reference sizes every buffer up front against a memory
// budget and treats a later allocation as a bug), or a thread that must not take the driver's
// allocation lock. For them this one entry point runs the same two kernels as tt_attn_decode
// with the split-KV scratch (partial triples, status word) carved out of a fixed array that
// lives in the library image on every device that loads it.
//
// The array's name is only a stand-in on the host side, so the device address is looked up
// once per device with cudaGetSymbolAddress while that device is current. That lookup happens
// inside the first call on a device: make that first call outside any stream capture.
// The session travels in the kernel parameters and every work item is derived from the block
// index, so nothing is copied from host memory and no table lives on the caller's stack.
// All calls on a device share the array and it keeps what the last call left behind; nothing
// in it has to start at zero except the status word, which every call clears. Two calls that
// overlap on the GPU (different streams, no ordering) race on the array and give wrong
// results: order them.
// ---------------------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocScratchBytes = (size_t)8 << 20;   // 8 MiB per device, held until exit
constexpr size_t kNoAllocPartialOffset = 256;              // the status word has the first 256 bytes
constexpr uint32_t kNoAllocMaxKeys = 1u << 22;             // longest key range served (TT_NOALLOC_MAX_KEYS)
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

unsigned char *g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
volatile int g_noalloc_lock = 0;

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t noalloc_scratch(int device, unsigned char **out) {
    while (__sync_lock_test_and_set(&g_noalloc_lock, 1)) {}
    cudaError_t e = cudaSuccess;
    if (g_noalloc_ptr[device] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e == cudaSuccess) g_noalloc_ptr[device] = static_cast<unsigned char *>(p);
    }
    *out = g_noalloc_ptr[device];
    __sync_lock_release(&g_noalloc_lock);
    return e;
}

}  // namespace

TT_API int tt_attn_decode_noalloc(tt_stream stream, const void *q, const void *k, const void *v, void *out,
                                  uint32_t head_dim, uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t seq_len,
                                  uint32_t kv_start, float scale) {
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return TT_ERR_INVALID_ARG;
    if (n_kv_heads == 0 || n_q_heads == 0 || n_q_heads % n_kv_heads != 0 || n_q_heads > 96) return TT_ERR_INVALID_ARG;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return TT_ERR_UNSUPPORTED_SHAPE;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) != 0) return TT_ERR_UNSUPPORTED_SHAPE;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return TT_ERR_CUDA;
    if (device < 0 || device >= kNoAllocMaxDevices) return TT_ERR_UNSUPPORTED_SHAPE;
    int sm_count = 0;
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return TT_ERR_CUDA;
    unsigned char *scratch = nullptr;
    if (noalloc_scratch(device, &scratch) != cudaSuccess || scratch == nullptr) return TT_ERR_CUDA;

    if (kv_start > seq_len) kv_start = seq_len;
    const uint32_t keys = seq_len - kv_start, one = 1;
    if (keys > kNoAllocMaxKeys) return TT_ERR_UNSUPPORTED_SHAPE;   // beyond the stated maximum
    uint32_t keys_per_item = 0, n_items = 0;
    // the planner lengthens the items until the partial triples fit the fixed array
    int rc = tt_attn_plan_splits(&keys, &one, 1, head_dim, n_q_heads, n_kv_heads, (uint32_t)sm_count,
                                 kNoAllocScratchBytes - kNoAllocPartialOffset, &keys_per_item, &n_items);
    if (rc != TT_OK) return TT_ERR_UNSUPPORTED_SHAPE;       // does not fit the 8 MiB array
    uint32_t parts = ceil_div_u32(keys, keys_per_item);
    if (parts == 0) parts = 1;
    const size_t partial_rows = (size_t)parts * n_q_heads;
    if (partial_rows * (head_dim + 2) * sizeof(float) > kNoAllocScratchBytes - kNoAllocPartialOffset)
        return TT_ERR_UNSUPPORTED_SHAPE;
    // one session in the kernels' parameter table (a member of a thread-local object: no allocation,
    // and no 5 KB object on the caller's stack)
    static thread_local TTSessionTable table;
    TTDecodeSession &ses = table.s[0];
    ses.q = q; ses.out = out; ses.k = k; ses.v = v;
    ses.seq_len = seq_len; ses.q_rows = 1; ses.kv_start = kv_start;
    ses.n_parts = parts; ses.partial_base = 0; ses.ring_capacity = 0; ses.keep = nullptr; ses.row_index = nullptr;
    const uint32_t group = n_q_heads / n_kv_heads;
    const uint32_t hpc = tt_decode_heads_per_cta(n_kv_heads, false);
    const uint32_t grid = parts * (n_kv_heads / hpc) * ceil_div_u32(group, 16);
    table.item_prefix[0] = 0; table.item_prefix[1] = grid; table.n = 1;

    cudaStream_t s = (cudaStream_t)stream;
    uint32_t *status = reinterpret_cast<uint32_t *>(scratch);
    float *part_o = reinterpret_cast<float *>(scratch + kNoAllocPartialOffset);
    float *part_m = part_o + partial_rows * head_dim;
    float *part_l = part_m + partial_rows;
    if (cudaMemsetAsync(status, 0, sizeof(uint32_t), s) != cudaSuccess) return TT_ERR_CUDA;
    tt_attn_batch_params p;
    p.head_dim = head_dim; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
    p.kv_token_stride_elements = n_kv_heads * head_dim; p.q_row_stride_elements = n_q_heads * head_dim;
    p.out_row_stride_elements = n_q_heads * head_dim; p.scale = scale; p.io_dtype = TT_F16;
    if (launch_partial_hd<__half>(s, grid, nullptr, nullptr, part_o, part_m, part_l, &p, status, table, keys_per_item,
                                  group > 8, hpc) != cudaSuccess)
        return TT_ERR_CUDA;
    attn_decode_combine_kernel<__half><<<dim3(1, n_q_heads, (head_dim / 4 + 15) / 16), 256, 0, s>>>(
        nullptr, part_o, part_m, part_l, n_q_heads, head_dim, n_q_heads * head_dim, 0, nullptr, nullptr, nullptr, table,
        16u);
    return cudaGetLastError() == cudaSuccess ? TT_OK : TT_ERR_CUDA;
}

// The status word of the allocation-free entry point on the current device: waits for `stream`,
// then reads the word the last tt_attn_decode_noalloc call on this device cleared and its kernels
// may have set (bit 0: a bounded wait inside a kernel ran out and that call's output is not valid).
TT_API int tt_attn_decode_noalloc_status(tt_stream stream, uint32_t *out_flags) {
    if (out_flags == nullptr) return TT_ERR_INVALID_ARG;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return TT_ERR_CUDA;
    if (device < 0 || device >= kNoAllocMaxDevices) return TT_ERR_UNSUPPORTED_SHAPE;
    unsigned char *scratch = nullptr;
    if (noalloc_scratch(device, &scratch) != cudaSuccess || scratch == nullptr) return TT_ERR_CUDA;
    if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return TT_ERR_CUDA;
    if (cudaMemcpy(out_flags, scratch, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) return TT_ERR_CUDA;
    return TT_OK;
}
