// Cross-GPU log-sum-exp merge of split-KV partials, exchange and merge in one kernel.
//
// One long session's KV rows are split along the sequence over the GPUs of a node; each GPU ends
// pass 1 with one unnormalised (m, d, o) triple per q head (the chunk-partial format of
// sources/TinyTitanCore/Metal/Attention/attention.metal:146-159). Instead of an all-gather
// followed by the merge (attention.metal:395-437), every rank's kernel
//   1. stores its triple into slot `rank` of EVERY rank's exchange buffer through peer mappings
//      (plain 16-byte stores over NVLink; remote memory is only ever written, never read),
//   2. publishes it: __syncthreads, a system-scope fence and a release store of the step's epoch
//      into flag[rank][head] of every buffer,
//   3. waits until flag[r][head] == epoch for all r in its OWN buffer (acquire loads, bounded),
//   4. merges the `world` triples of its head from local memory and writes the output row.
// CTA h handles q head h alone, so heads never wait for one another. Slots and flags are double
// buffered on the epoch's parity: a rank can run at most one step ahead of the slowest one (it
// needs that rank's data of the current step to finish), so the step after next never lands in a
// slot that is still being read.
#include "tt_sm100.h"

namespace {

constexpr uint32_t kMaxWorld = 16;
constexpr uint32_t kPollLimit = 1u << 22;   // polls of ~0.25 us before the wait gives up (about a second)

struct ExchangeLayout {
    uint32_t row_floats;     // head_dim + 4: o[head_dim], m, d, two pads (rows stay 16-byte aligned)
    size_t parity_bytes;     // data [world][H][row_floats] fp32, then flags [world][H] u32, padded to 256 B
    size_t flags_offset;
};

__host__ __device__ inline ExchangeLayout exchange_layout(uint32_t world, uint32_t n_q_heads, uint32_t head_dim) {
    ExchangeLayout l;
    l.row_floats = head_dim + 4;
    l.flags_offset = (size_t)world * n_q_heads * l.row_floats * sizeof(float);
    l.parity_bytes = (l.flags_offset + (size_t)world * n_q_heads * sizeof(uint32_t) + 255) / 256 * 256;
    return l;
}

struct ExchangeParams {
    unsigned char *peer[kMaxWorld];
    const float *m, *d, *o;
    uint32_t rank, world, n_q_heads, head_dim, epoch;
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// grid = n_q_heads, block = 128
template <typename T>
__global__ void __launch_bounds__(128) attn_exchange_combine_kernel(ExchangeParams p, T *__restrict__ out,
                                                                   uint32_t *__restrict__ status) {
    __shared__ int all_arrived;
    const uint32_t h = blockIdx.x, tid = threadIdx.x;
    const ExchangeLayout l = exchange_layout(p.world, p.n_q_heads, p.head_dim);
    const size_t parity_off = (size_t)(p.epoch & 1u) * l.parity_bytes;
    const size_t my_row = ((size_t)p.rank * p.n_q_heads + h) * l.row_floats;

    // 1. this rank's triple of head h into slot `rank` of every buffer
    for (uint32_t r = 0; r < p.world; ++r) {
        float *dst = reinterpret_cast<float *>(p.peer[r] + parity_off) + my_row;
        for (uint32_t c = tid * 4; c < p.head_dim; c += blockDim.x * 4)
            *reinterpret_cast<float4 *>(dst + c) = *reinterpret_cast<const float4 *>(p.o + (size_t)h * p.head_dim + c);
        if (tid == 0) *reinterpret_cast<float4 *>(dst + p.head_dim) = make_float4(p.m[h], p.d[h], 0.f, 0.f);
    }
    // 2. publish
    __syncthreads();
    if (tid < p.world) {
        __threadfence_system();
        uint32_t *flags = reinterpret_cast<uint32_t *>(p.peer[tid] + parity_off + l.flags_offset);
        st_release_sys(flags + (size_t)p.rank * p.n_q_heads + h, p.epoch);
    }
    // 3. wait for every rank's triple of this epoch in the local buffer
    if (tid == 0) all_arrived = 1;
    __syncthreads();
    unsigned char *mine = p.peer[p.rank] + parity_off;
    if (tid < p.world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(mine + l.flags_offset) + (size_t)tid * p.n_q_heads + h;
        bool ok = false;
        for (uint32_t it = 0; it < kPollLimit; ++it) {
            if (ld_acquire_sys(flag) == p.epoch) { ok = true; break; }
            __nanosleep(64);
        }
        if (!ok) all_arrived = 0;
    }
    __syncthreads();
    if (!all_arrived) {
        if (tid == 0) atomicOr(status, TT_DEV_WAIT_TIMEOUT);
        return;     // the output row is left untouched
    }
    // 4. merge (attention.metal:395-437)
    const float *rows = reinterpret_cast<const float *>(mine);
    float mg = -INFINITY;
    for (uint32_t r = 0; r < p.world; ++r)
        mg = fmaxf(mg, rows[((size_t)r * p.n_q_heads + h) * l.row_floats + p.head_dim]);
    float dsum = 0.f;
    if (mg != -INFINITY)
        for (uint32_t r = 0; r < p.world; ++r) {
            const float *row = rows + ((size_t)r * p.n_q_heads + h) * l.row_floats;
            dsum += row[p.head_dim + 1] * __expf(row[p.head_dim] - mg);
        }
    const float inv = dsum > 0.f ? 1.f / dsum : 0.f;
    for (uint32_t c = tid; c < p.head_dim; c += blockDim.x) {
        float acc = 0.f;
        if (mg != -INFINITY)
            for (uint32_t r = 0; r < p.world; ++r) {
                const float *row = rows + ((size_t)r * p.n_q_heads + h) * l.row_floats;
                acc += row[c] * __expf(row[p.head_dim] - mg);
            }
        out[(size_t)h * p.head_dim + c] = static_cast<T>(acc * inv);
    }
}

}  // namespace

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
    if (!m || !d || !o || !peer_buffers || !out) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: null argument");
    if (world == 0 || world > kMaxWorld || rank >= world)
        return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: world must be 1..%u and rank below it", kMaxWorld);
    if (n_q_heads == 0 || head_dim == 0 || head_dim % 4 != 0)
        return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "exchange: head_dim must be a positive multiple of 4");
    if (epoch == 0) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: epochs start at 1");
    if (io_dtype != TT_F16 && io_dtype != TT_BF16) return tt_set_error(ctx, TT_ERR_INVALID_ARG, "io_dtype must be TT_F16 or TT_BF16");
    if (((uintptr_t)o | (uintptr_t)out) & 15) return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "exchange: buffers must be 16-byte aligned");
    ExchangeParams p;
    for (uint32_t r = 0; r < kMaxWorld; ++r) p.peer[r] = nullptr;
    for (uint32_t r = 0; r < world; ++r) {
        if (peer_buffers[r] == nullptr || ((uintptr_t)peer_buffers[r] & 255))
            return tt_set_error(ctx, TT_ERR_INVALID_ARG, "exchange: peer buffer %u is null or not 256-byte aligned", r);
        p.peer[r] = reinterpret_cast<unsigned char *>(peer_buffers[r]);
    }
    p.m = m; p.d = d; p.o = o;
    p.rank = rank; p.world = world; p.n_q_heads = n_q_heads; p.head_dim = head_dim; p.epoch = epoch;
    if (io_dtype == TT_F16)
        attn_exchange_combine_kernel<__half><<<n_q_heads, 128, 0, (cudaStream_t)stream>>>(p, reinterpret_cast<__half *>(out), ctx->status);
    else
        attn_exchange_combine_kernel<__nv_bfloat16><<<n_q_heads, 128, 0, (cudaStream_t)stream>>>(p, reinterpret_cast<__nv_bfloat16 *>(out), ctx->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "attn_exchange_combine launch");
    ctx->launches++;
    return TT_OK;
}
