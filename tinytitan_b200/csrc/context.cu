// Context: device binding, one-time scratch allocation, error reporting.
#include <mutex>
#include "tt_common.h"

#include <cstdlib>
#include <new>

int tt_set_error(tt_context *ctx, int code, const char *fmt, ...) {
    if (ctx != nullptr) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

bool tt_pdl_enabled() {
    static const bool enabled = getenv("TT_NO_PDL") == nullptr;
    return enabled;
}

int tt_check_cuda(tt_context *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return TT_OK;
    const int code = (e == cudaErrorMemoryAllocation) ? TT_ERR_OOM : TT_ERR_CUDA;
    return tt_set_error(ctx, code, "%s: %s", what, cudaGetErrorString(e));
}

TT_API const char *tt_status_string(int status) {
    switch (status) {
        case TT_OK: return "ok";
        case TT_ERR_INVALID_ARG: return "invalid argument";
        case TT_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
        case TT_ERR_OOM: return "out of memory";
        case TT_ERR_CUDA: return "CUDA error";
        case TT_ERR_TIMEOUT: return "device wait timed out";
        case TT_ERR_BUSY: return "context busy";
        default: return "unknown status";
    }
}

TT_API const char *tt_last_error_string(const tt_context *ctx) { return ctx ? ctx->err : "null context"; }

// Lays the three tables of a decode call out back to back (128-byte aligned) in the host staging
// buffer and, identically, in the device buffer: sessions, then (verify batches) two tensor maps per
// session, then the items.
cudaError_t tt_set_smem_once_impl(const void *kernel, int smem) {
    struct Entry { const void *fn; int dev; int smem; };
    static Entry table[256];
    static int n = 0;
    static std::mutex lock;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> guard(lock);
    for (int i = 0; i < n; ++i)
        if (table[i].fn == kernel && table[i].dev == dev) {
            if (table[i].smem >= smem) return cudaSuccess;
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e == cudaSuccess) table[i].smem = smem;
            return e;
        }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess && n < 256) table[n++] = Entry{kernel, dev, smem};
    return e;
}

void tt_bind_decode_tables(tt_context *ctx, uint32_t n_sessions, bool with_maps) {
    const size_t off_maps = (sizeof(TTDecodeSession) * n_sessions + 127) / 128 * 128;
    const size_t off_items = off_maps + (with_maps ? (size_t)256 * n_sessions : 0);
    ctx->sessions = reinterpret_cast<TTDecodeSession *>(ctx->tables);
    ctx->tensor_maps = ctx->tables + off_maps;
    ctx->items = reinterpret_cast<TTDecodeItem *>(ctx->tables + off_items);
    ctx->h_sessions = reinterpret_cast<TTDecodeSession *>(ctx->h_tables);
    ctx->h_tensor_maps = ctx->h_tables + off_maps;
    ctx->h_items = reinterpret_cast<TTDecodeItem *>(ctx->h_tables + off_items);
}

static void context_free(tt_context *ctx) {
    if (ctx == nullptr) return;
    cudaFree(ctx->partials);
    cudaFree(ctx->tables);
    cudaFree(ctx->gdn_sessions);
    cudaFree(ctx->status);
    if (ctx->profile_begin) {
        for (uint32_t i = 0; i < tt_context::kProfileSlots; ++i) {
            if (ctx->profile_begin[i]) cudaEventDestroy(ctx->profile_begin[i]);
            if (ctx->profile_end[i]) cudaEventDestroy(ctx->profile_end[i]);
        }
        free(ctx->profile_begin);
        free(ctx->profile_end);
    }
    free(ctx->h_tables);
    free(ctx->h_sessions_in);
    free(ctx->h_keys);
    free(ctx->h_rows);
    delete ctx;
}

TT_API tt_context *tt_context_create(int device, const tt_context_options *options, int *out_err) {
    int err_local = TT_OK;
    int *err = out_err ? out_err : &err_local;
    *err = TT_OK;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) { *err = TT_ERR_CUDA; return nullptr; }
    if (device < 0 || device >= count) { *err = TT_ERR_INVALID_ARG; return nullptr; }
    if (cudaSetDevice(device) != cudaSuccess) { *err = TT_ERR_CUDA; return nullptr; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { *err = TT_ERR_CUDA; return nullptr; }
    if (prop.major != 10) { *err = TT_ERR_UNSUPPORTED_SHAPE; return nullptr; }  // sm_100a code only

    tt_context *ctx = new (std::nothrow) tt_context();
    if (ctx == nullptr) { *err = TT_ERR_OOM; return nullptr; }
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    ctx->workspace_bytes = (options && options->workspace_bytes) ? options->workspace_bytes : ((size_t)256 << 20);
    ctx->max_sessions = (options && options->max_sessions) ? options->max_sessions : 1024u;
    ctx->max_items = 65536u;

    bool ok = true;
    ok = ok && cudaMalloc(&ctx->partials, ctx->workspace_bytes) == cudaSuccess;
    ctx->table_bytes = (sizeof(TTDecodeSession) * ctx->max_sessions + 127) / 128 * 128 + (size_t)256 * ctx->max_sessions +
                       sizeof(TTDecodeItem) * ctx->max_items;
    ok = ok && cudaMalloc(&ctx->tables, ctx->table_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->gdn_sessions, sizeof(tt_gdn_session) * ctx->max_sessions) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->status, sizeof(uint32_t)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->status, 0, sizeof(uint32_t)) == cudaSuccess;
    ctx->h_tables = (unsigned char *)aligned_alloc(128, (ctx->table_bytes + 127) / 128 * 128);
    ctx->h_sessions_in = (TTDecodeSession *)malloc(sizeof(TTDecodeSession) * ctx->max_sessions);
    ctx->h_keys = (uint32_t *)malloc(sizeof(uint32_t) * ctx->max_sessions);
    ctx->h_rows = (uint32_t *)malloc(sizeof(uint32_t) * ctx->max_sessions);
    ok = ok && ctx->h_tables && ctx->h_sessions_in && ctx->h_keys && ctx->h_rows;
    if (ok) tt_bind_decode_tables(ctx, ctx->max_sessions, true);
    if (!ok) {
        cudaGetLastError();
        context_free(ctx);
        *err = TT_ERR_OOM;
        return nullptr;
    }
    return ctx;
}

TT_API void tt_context_destroy(tt_context *ctx) {
    if (ctx == nullptr) return;
    cudaSetDevice(ctx->device);
    context_free(ctx);
}

TT_API int tt_stream_synchronize(tt_context *ctx, tt_stream stream) {
    TT_ENTER(ctx);
    return tt_check_cuda(ctx, cudaStreamSynchronize((cudaStream_t)stream), "cudaStreamSynchronize");
}

TT_API int tt_ctx_poll_status(tt_context *ctx, tt_stream stream, uint32_t *out_flags) {
    TT_ENTER(ctx);
    uint32_t flags = 0;
    cudaError_t e = cudaMemcpyAsync(&flags, ctx->status, sizeof(flags), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return tt_check_cuda(ctx, e, "poll status");
    if (out_flags) *out_flags = flags;
    if (flags & TT_DEV_WAIT_TIMEOUT) return tt_set_error(ctx, TT_ERR_TIMEOUT, "a bounded device-side wait ran out");
    if (flags) return tt_set_error(ctx, TT_ERR_CUDA, "device status flags 0x%x", flags);
    return TT_OK;
}

TT_API uint64_t tt_ctx_launch_count(const tt_context *ctx) { return ctx ? ctx->launches : 0; }

TT_API int tt_ctx_profile_enable(tt_context *ctx, int enabled) {
    TT_ENTER(ctx);
    if (enabled && ctx->profile_begin == nullptr) {
        ctx->profile_begin = (cudaEvent_t *)calloc(tt_context::kProfileSlots, sizeof(cudaEvent_t));
        ctx->profile_end = (cudaEvent_t *)calloc(tt_context::kProfileSlots, sizeof(cudaEvent_t));
        if (!ctx->profile_begin || !ctx->profile_end) return tt_set_error(ctx, TT_ERR_OOM, "profile events");
        for (uint32_t i = 0; i < tt_context::kProfileSlots; ++i) {
            cudaError_t e = cudaEventCreate(&ctx->profile_begin[i]);
            if (e == cudaSuccess) e = cudaEventCreate(&ctx->profile_end[i]);
            if (e != cudaSuccess) return tt_check_cuda(ctx, e, "cudaEventCreate");
        }
    }
    ctx->profiling = enabled;
    ctx->profile_count = 0;
    return TT_OK;
}

TT_API int tt_ctx_profile_collect(tt_context *ctx, float *out_ms, uint32_t capacity, uint32_t *out_count) {
    TT_ENTER(ctx);
    uint32_t n = ctx->profile_count < capacity ? ctx->profile_count : capacity;
    for (uint32_t i = 0; i < n; ++i) {
        cudaError_t e = cudaEventSynchronize(ctx->profile_end[i]);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&out_ms[i], ctx->profile_begin[i], ctx->profile_end[i]);
        if (e != cudaSuccess) return tt_check_cuda(ctx, e, "profile collect");
    }
    if (out_count) *out_count = n;
    ctx->profile_count = 0;
    return TT_OK;
}
