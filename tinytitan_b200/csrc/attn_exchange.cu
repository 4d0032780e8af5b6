// Cross-GPU log-sum-exp merge of split-KV partials, exchange and merge in one kernel.
//
// One long session's KV rows are split along the sequence over the GPUs of a node; each GPU ends
// pass 1 with one unnormalised (m, d, o) triple per q head (the chunk-partial format of
// sources/TinyTitanCore/Metal/Attention/attention.metal:146-159). Instead of an all-gather
// followed by the merge (attention.metal:395-437), every rank's kernel
//   1. stores its triple into slot `rank` of EVERY rank's exchange buffer through peer mappings
//      (plain 16-byte stores over NVLink; remote memory is only ever written, never read). Every
//      8 bytes on the wire are one value and the step's epoch, so a word validates itself: there is
//      no flag behind the data, hence no system-scope release that has to wait for the peer stores
//      to be acknowledged first (measured: 4.5 us per step on two GPUs for that release alone),
//   2. polls its OWN buffer until every word of every rank's cell carries this epoch (volatile
//      16-byte loads, bounded),
//   3. merges the `world` triples of its head from the words it polled and writes the output row.
// CTA (h, column block) handles its part of q head h alone, so heads never wait for one another.
// Slots are double buffered on the epoch's parity: a rank can run at most one step ahead of the
// slowest one (it needs that rank's data of the current step to finish), so the step after next
// never lands in a slot that is still being read, and a slot's previous epoch differs by two.
#include "tt_sm100.h"

namespace {

constexpr uint32_t kMaxWorld = 16;
constexpr uint32_t kPollLimit = 1u << 22;   // polls of ~0.25 us before the wait gives up (about a second)
constexpr uint32_t kColBlock = 64;          // columns per CTA: 16 threads x float4
constexpr uint32_t kCellValues = kColBlock + 2;   // o slice, m, d
constexpr uint32_t kCellUnits = kCellValues / 2;  // 16-byte words {value, epoch, value, epoch}: 33
constexpr uint32_t kCellBytes = kCellUnits * 16;

// One parity of an exchange buffer: cells [world][H][col blocks] of kCellUnits self-validating words,
// padded to 256 B. A cell is one rank's (m, d) and 64 columns of o for one head; every (head, col block)
// is exchanged and merged by one CTA on its own.
struct ExchangeLayout {
    uint32_t col_blocks;
    size_t parity_bytes;
};

__host__ __device__ inline ExchangeLayout exchange_layout(uint32_t world, uint32_t n_q_heads, uint32_t head_dim) {
    ExchangeLayout l;
    l.col_blocks = (head_dim + kColBlock - 1) / kColBlock;
    const size_t cells = (size_t)world * n_q_heads * l.col_blocks;
    l.parity_bytes = (cells * kCellBytes + 255) / 256 * 256;
    return l;
}

struct ExchangeParams {
    unsigned char *peer[kMaxWorld];
    // input form 1: one merged triple per head
    const float *m, *d, *o;
    // input form 2: the split partials of pass 1 ([part][head] rows of head_dim, m, l), merged here first
    const float *part_o, *part_m, *part_l;
    uint32_t n_parts;
    uint32_t rank, world, n_q_heads, head_dim, epoch;
    uint32_t poll_limit;   // polls of ~0.25 us before the flag wait gives up
};

__device__ __forceinline__ void st_word_sys(void *p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_word_sys(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Shared memory of one exchange: this rank's cell on the way out, every rank's cell on the way in.
constexpr uint32_t kCellPitch = (kCellValues + 3) / 4 * 4;   // rows of 16-byte multiples: the merge reads them as float4
struct ExchangeSmem {
    float mine[kCellPitch];
    float recv[kMaxWorld][kCellPitch];
    int all_arrived;
};
static_assert(kCellPitch % 4 == 0 && sizeof(float) * kCellPitch % 16 == 0, "cell rows must stay 16-byte aligned");

// Steps 1-3 of the header comment for one (head, col block): threads 0..15 hold this rank's 64
// columns (`acc`, unnormalised) and everyone its (m, d). All threads of the CTA call this.
template <typename T>
__device__ __forceinline__ void exchange_and_merge(const ExchangeParams &p, uint32_t h, uint32_t cb, float4 acc, float m,
                                                   float d, T *__restrict__ out, uint32_t *__restrict__ status,
                                                   ExchangeSmem *sm) {
    const uint32_t tid = threadIdx.x;
    const ExchangeLayout l = exchange_layout(p.world, p.n_q_heads, p.head_dim);
    const size_t parity_off = (size_t)(p.epoch & 1u) * l.parity_bytes;
    const size_t my_cell = ((size_t)p.rank * p.n_q_heads + h) * l.col_blocks + cb;
    const uint32_t col = cb * kColBlock + tid * 4;

    // 1. this rank's cell, re-cut into {value, epoch} pairs, into slot `rank` of every buffer
    if (tid < 16) *reinterpret_cast<float4 *>(&sm->mine[tid * 4]) = acc;
    if (tid == 16) { sm->mine[kColBlock] = m; sm->mine[kColBlock + 1] = d; }
    if (tid == 0) sm->all_arrived = 1;
    __syncthreads();
    for (uint32_t u = tid; u < kCellUnits; u += blockDim.x) {       // the one-warp form of the kernel has fewer threads than words
        const uint4 word = make_uint4(__float_as_uint(sm->mine[2 * u]), p.epoch, __float_as_uint(sm->mine[2 * u + 1]), p.epoch);
        for (uint32_t r = 0; r < p.world; ++r)
            st_word_sys(p.peer[r] + parity_off + my_cell * kCellBytes + u * 16, word);
    }
    // 2. every rank's cell of this epoch from the local buffer, word by word
    const unsigned char *mine = p.peer[p.rank] + parity_off;
    for (uint32_t idx = tid; idx < p.world * kCellUnits; idx += blockDim.x) {
        const uint32_t r = idx / kCellUnits, u = idx - r * kCellUnits;
        const unsigned char *src = mine + (((size_t)r * p.n_q_heads + h) * l.col_blocks + cb) * kCellBytes + u * 16;
        bool ok = false;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        for (uint32_t it = 0; it < p.poll_limit; ++it) {
            v = ld_word_sys(src);
            if (v.y == p.epoch && v.w == p.epoch) { ok = true; break; }
            __nanosleep(32);
        }
        if (!ok) sm->all_arrived = 0;
        sm->recv[r][2 * u] = __uint_as_float(v.x);
        sm->recv[r][2 * u + 1] = __uint_as_float(v.z);
    }
    __syncthreads();
    if (!sm->all_arrived) {
        if (tid == 0) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
        return;     // the output columns are left untouched
    }
    // 3. merge (attention.metal:395-437)
    if (tid >= 16 || col >= p.head_dim) return;
    float mg = -INFINITY;
    for (uint32_t r = 0; r < p.world; ++r) mg = fmaxf(mg, sm->recv[r][kColBlock]);
    float dsum = 0.f;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mg != -INFINITY)
        for (uint32_t r = 0; r < p.world; ++r) {
            const float *cell = sm->recv[r];
            const float wgt = __expf(cell[kColBlock] - mg);
            const float4 o = *reinterpret_cast<const float4 *>(cell + tid * 4);
            dsum += cell[kColBlock + 1] * wgt;
            sum.x += o.x * wgt; sum.y += o.y * wgt; sum.z += o.z * wgt; sum.w += o.w * wgt;
        }
    const float inv = dsum > 0.f ? 1.f / dsum : 0.f;
    uint2 packed;
    packed.x = pack2<T>(sum.x * inv, sum.y * inv);
    packed.y = pack2<T>(sum.z * inv, sum.w * inv);
    *reinterpret_cast<uint2 *>(out + (size_t)h * p.head_dim + col) = packed;
}

// Input form 1. grid = (n_q_heads, col blocks), block = 32
template <typename T>
__global__ void __launch_bounds__(32) attn_exchange_combine_kernel(ExchangeParams p, T *__restrict__ out,
                                                                  uint32_t *__restrict__ status) {
    __shared__ __align__(16) ExchangeSmem xs;
    const uint32_t h = blockIdx.x, cb = blockIdx.y, tid = threadIdx.x;
    const uint32_t col = cb * kColBlock + tid * 4;
    pdl_launch_dependents();
    pdl_wait();                       // the kernel that produced (m, d, o) has completed
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid < 16 && col < p.head_dim) acc = *reinterpret_cast<const float4 *>(p.o + (size_t)h * p.head_dim + col);
    exchange_and_merge<T>(p, h, cb, acc, p.m[h], p.d[h], out, status, &xs);
}

// Input form 2: the local log-sum-exp merge of this rank's split partials (one session, one query
// row) and the cross-GPU exchange and merge in the same kernel. grid = (n_q_heads, col blocks),
// block = 256 = 16 part groups x 16 column threads.
template <typename T>
__global__ void __launch_bounds__(256) attn_merge_exchange_kernel(ExchangeParams p, T *__restrict__ out,
                                                                 uint32_t *__restrict__ status) {
    __shared__ __align__(16) ExchangeSmem xs;
    __shared__ float grp_m[16], grp_d[16];
    __shared__ float4 accs[256];
    const uint32_t h = blockIdx.x, cb = blockIdx.y, tid = threadIdx.x;
    const uint32_t grp = tid >> 4, ct = tid & 15;
    const uint32_t H = p.n_q_heads;
    const uint32_t col = cb * kColBlock + ct * 4;
    pdl_launch_dependents();
    pdl_wait();                       // pass 1 has completed and its partials are visible

    // One pass over this rank's parts: group g (16 column threads) walks parts g, g+16, ... four loads at
    // a time with an online (max, sum, output) triple; the 16 triples are merged below. Nothing
    // block-wide has to finish before the first load is issued.
    float m_run = -INFINITY, d_run = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < p.head_dim) {
        uint32_t c = grp;
        for (; c + 48 < p.n_parts; c += 64) {
            float e[4], l[4]; float4 o[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const size_t pr = (size_t)(c + 16 * u) * H + h;
                e[u] = p.part_m[pr];
                l[u] = p.part_l[pr];
                o[u] = *reinterpret_cast<const float4 *>(p.part_o + pr * p.head_dim + col);
            }
            const float m_new = fmaxf(m_run, fmaxf(fmaxf(e[0], e[1]), fmaxf(e[2], e[3])));
            if (m_new != -INFINITY) {                              // exp(-inf - -inf) would be NaN
                const float sc = __expf(m_run - m_new);
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
        for (; c < p.n_parts; c += 16) {
            const size_t pr = (size_t)c * H + h;
            const float e = p.part_m[pr], l = p.part_l[pr];
            const float4 o = *reinterpret_cast<const float4 *>(p.part_o + pr * p.head_dim + col);
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
    accs[tid] = acc;
    if (ct == 0) { grp_m[grp] = m_run; grp_d[grp] = d_run; }
    __syncthreads();
    float mg = grp_m[0];
#pragma unroll
    for (int g = 1; g < 16; ++g) mg = fmaxf(mg, grp_m[g]);
    float D = 0.f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid < 17 && mg != -INFINITY)      // threads 0-15 carry the columns on, thread 16 the (max, sum) pair
        for (uint32_t g = 0; g < 16; ++g) {
            const float wgt = __expf(grp_m[g] - mg);              // 0 for a group that saw no finite maximum
            const float4 o = accs[g * 16 + (tid & 15)];
            acc.x += o.x * wgt; acc.y += o.y * wgt; acc.z += o.z * wgt; acc.w += o.w * wgt;
            D += grp_d[g] * wgt;
        }
    exchange_and_merge<T>(p, h, cb, acc, mg, D, out, status, &xs);
}

int fill_params(tt_context *ctx, ExchangeParams &p, void *const *peer_buffers, uint32_t rank, uint32_t world,
                uint32_t n_q_heads, uint32_t head_dim, uint32_t epoch, const void *out, uint32_t io_dtype) {
    if (!peer_buffers || !out) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: null argument");
    if (world == 0 || world > kMaxWorld || rank >= world)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: world must be 1..%u and rank below it", kMaxWorld);
    if (n_q_heads == 0 || head_dim == 0 || head_dim % 4 != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "exchange: head_dim must be a positive multiple of 4");
    if (epoch == 0) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: epochs start at 1");
    if (io_dtype != TT_F16 && io_dtype != TT_BF16) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "io_dtype must be TT_F16 or TT_BF16");
    if ((uintptr_t)out & 15) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "exchange: buffers must be 16-byte aligned");
    for (uint32_t r = 0; r < kMaxWorld; ++r) p.peer[r] = nullptr;
    for (uint32_t r = 0; r < world; ++r) {
        if (peer_buffers[r] == nullptr || ((uintptr_t)peer_buffers[r] & 255))
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: peer buffer %u is null or not 256-byte aligned", r);
        p.peer[r] = reinterpret_cast<unsigned char *>(peer_buffers[r]);
    }
    p.m = p.d = p.o = p.part_o = p.part_m = p.part_l = nullptr;
    p.n_parts = 0;
    p.rank = rank; p.world = world; p.n_q_heads = n_q_heads; p.head_dim = head_dim; p.epoch = epoch;
    p.poll_limit = ctx->exchange_poll_limit ? ctx->exchange_poll_limit : kPollLimit;
    return TT_OK;
}

}  // namespace

// Local merge of one session's split partials fused with the cross-GPU exchange and merge (the
// second launch of tt_attn_decode_exchange).
int tt_launch_merge_exchange(tt_context *ctx, cudaStream_t stream, const float *part_o, const float *part_m,
                             const float *part_l, uint32_t n_parts, const tt_attn_exchange *x, uint32_t n_q_heads,
                             uint32_t head_dim, uint32_t io_dtype) {
    ExchangeParams p;
    int rc = fill_params(ctx, p, x->peer_buffers, x->rank, x->world, n_q_heads, head_dim, x->epoch, x->out, io_dtype);
    if (rc != TT_OK) return rc;
    p.part_o = part_o; p.part_m = part_m; p.part_l = part_l; p.n_parts = n_parts;
    const dim3 grid(n_q_heads, exchange_layout(x->world, n_q_heads, head_dim).col_blocks);
    cudaError_t e;
    TTLaunchTimer timer(ctx, stream, TT_PROFILE_EXCHANGE);
    if (io_dtype == TT_F16)
        e = tt_launch_pdl(attn_merge_exchange_kernel<__half>, grid, dim3(256), 0, stream, p, reinterpret_cast<__half *>(x->out), ctx->status);
    else
        e = tt_launch_pdl(attn_merge_exchange_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, p,
                          reinterpret_cast<__nv_bfloat16 *>(x->out), ctx->status);
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_merge_exchange launch");
    timer.stop();
    ctx->launches++;
    return TT_OK;
}

TT_API int tt_ctx_set_exchange_poll_limit(tt_context *ctx, uint32_t polls) {
    if (ctx == nullptr) return TT_ERR_INVALID_ARG;
    ctx->exchange_poll_limit = polls;   // 0 selects the default
    return TT_OK;
}

TT_API size_t tt_attn_exchange_bytes(uint32_t world, uint32_t n_q_heads, uint32_t head_dim) {
    return 2 * exchange_layout(world, n_q_heads, head_dim).parity_bytes;
}

TT_API int tt_peer_buffer_create(tt_context *ctx, size_t bytes, void **out_ptr, unsigned char out_handle[64]) {
    TT_ENTER(ctx);
    if (out_ptr == nullptr || out_handle == nullptr || bytes == 0)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "peer buffer: null output or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    void *ptr = nullptr;
    cudaError_t e = cudaMalloc(&ptr, bytes);
    if (e != cudaSuccess) { cudaGetLastError(); return tt_set_error(ctx, TT_ERR_OOM, "peer buffer of %zu bytes", bytes); }
    e = cudaMemset(ptr, 0, bytes);      // flags start below every epoch
    cudaIpcMemHandle_t handle;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&handle, ptr);
    if (e != cudaSuccess) { cudaFree(ptr); return tt_check_cuda(ctx, e, "peer buffer handle"); }
    memcpy(out_handle, &handle, 64);
    *out_ptr = ptr;
    return TT_OK;
}

TT_API int tt_peer_buffer_open(tt_context *ctx, const unsigned char handle[64], void **out_ptr) {
    TT_ENTER(ctx);
    if (out_ptr == nullptr || handle == nullptr) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "peer buffer: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    return tt_check_cuda(ctx, cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess), "open peer buffer");
}

TT_API int tt_peer_buffer_close(tt_context *ctx, void *ptr) {
    TT_ENTER(ctx);
    return ptr ? tt_check_cuda(ctx, cudaIpcCloseMemHandle(ptr), "close peer buffer") : TT_OK;
}

TT_API int tt_peer_buffer_destroy(tt_context *ctx, void *ptr) {
    TT_ENTER(ctx);
    return ptr ? tt_check_cuda(ctx, cudaFree(ptr), "free peer buffer") : TT_OK;
}

TT_API int tt_attn_exchange_combine(tt_context *ctx, tt_stream stream, const float *m, const float *d,
                                    const float *o, void *const *peer_buffers, uint32_t rank, uint32_t world,
                                    uint32_t n_q_heads, uint32_t head_dim, uint32_t epoch, void *out,
                                    uint32_t io_dtype) {
    TT_ENTER(ctx);
    if (!m || !d || !o) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: null argument");
    if ((uintptr_t)o & 15) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "exchange: buffers must be 16-byte aligned");
    ExchangeParams p;
    int rc = fill_params(ctx, p, peer_buffers, rank, world, n_q_heads, head_dim, epoch, out, io_dtype);
    if (rc != TT_OK) return rc;
    p.m = m; p.d = d; p.o = o;
    const dim3 grid(n_q_heads, exchange_layout(world, n_q_heads, head_dim).col_blocks);
    if (io_dtype == TT_F16)
        attn_exchange_combine_kernel<__half><<<grid, 32, 0, (cudaStream_t)stream>>>(p, reinterpret_cast<__half *>(out), ctx->status);
    else
        attn_exchange_combine_kernel<__nv_bfloat16><<<grid, 32, 0, (cudaStream_t)stream>>>(p, reinterpret_cast<__nv_bfloat16 *>(out), ctx->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_exchange_combine launch");
    ctx->launches++;
    return TT_OK;
}
