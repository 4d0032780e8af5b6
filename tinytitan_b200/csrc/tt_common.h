// Internal declarations shared by the translation units of libtinytitan_cuda.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdarg>
#include <cstdint>
#include <vector>
#include <cstdio>
#include <cstring>

#include "tinytitan_cuda.h"

#define TT_API extern "C" __attribute__((visibility("default")))

// Device-side status bits (tt_ctx_poll_status).
enum : uint32_t {
    TT_DEV_WAIT_TIMEOUT = 1u,   // a bounded mbarrier / flag wait ran out
    TT_DEV_BAD_ITEM = 2u,       // a work item failed its own bounds check
};

// One split-KV work item of the batched decode kernel (device + host view).
struct TTDecodeItem {
    uint32_t session;
    uint32_t kv_head;
    uint32_t key_begin;   // first key of this item (absolute position)
    uint32_t key_end;     // one past the last key
    uint32_t part_index;  // index of this item's partial among the session's parts
    uint32_t row_begin;   // first packed row (w*G + g) this item serves
    uint32_t row_count;   // rows served (<= 16 per CTA pass)
    uint32_t partial_base; // first partial row of this item in the workspace
};

// One session of the batched decode kernel (device view).
struct TTDecodeSession {
    const void *q;
    void *out;
    const void *k;
    const void *v;
    uint32_t seq_len;
    uint32_t q_rows;
    uint32_t kv_start;
    uint32_t n_parts;        // key splits of this session
    uint32_t partial_base;   // first partial row of this session in the workspace
    uint32_t ring_capacity;
    const uint8_t *keep;     // nullable
    const uint32_t *row_index;  // nullable: key s lives at row row_index[s] (compact selection)
};

// Sessions of a batched decode call that travel in the kernel parameters instead of a device
// table: calls with up to kParamSessions sessions upload nothing (the work item of a CTA is derived
// from its block index and item_prefix). n == 0 selects the device tables.
constexpr uint32_t kParamSessions = 64;
struct TTSessionTable {
    TTDecodeSession s[kParamSessions];
    uint32_t item_prefix[kParamSessions + 1];   // work items of the sessions before session i
    uint32_t n;
};

// Tensor maps of a verify batch that travel in the kernel parameters next to its TTSessionTable: the K and
// the V map of session i at [2 * i], [2 * i + 1]. 128 bytes each, 64-byte aligned as the copy engine wants.
constexpr uint32_t kVerifyParamSessions = 16;
struct alignas(64) TTVerifyMaps {
    unsigned char m[2 * kVerifyParamSessions][128];
};

struct tt_context {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    size_t workspace_bytes = 0;
    uint32_t max_sessions = 0;
    uint32_t max_items = 0;
    // device scratch, allocated once at creation
    unsigned char *tables = nullptr;    // session table | tensor maps | item table of the current decode call,
    unsigned char *h_tables = nullptr;  // packed back to back so that one copy uploads them. Pageable on
                                        // purpose: the driver stages small pageable copies inline in the
                                        // command stream, which measured faster than a pinned staging ring
                                        // (whose DMA fetch sits on the stream's critical path).
    size_t table_bytes = 0;
    float *partials = nullptr;          // [rows][head_dim + 2] fp32 split partials
    TTDecodeItem *items = nullptr;      // views into `tables`, rebound by every decode call
    TTDecodeSession *sessions = nullptr;
    void *gdn_sessions = nullptr;       // tt_gdn_session[max_sessions]
    void *tensor_maps = nullptr;        // CUtensorMap[2 * max_sessions]: per-session K and V maps (verify kernel)
    uint32_t *status = nullptr;         // device status word
    // host staging (pageable; async copies from it are staged by the driver before returning)
    TTDecodeItem *h_items = nullptr;
    TTDecodeSession *h_sessions = nullptr;
    TTDecodeSession *h_sessions_in = nullptr;
    uint32_t *h_keys = nullptr;
    uint32_t *h_rows = nullptr;
    void *h_tensor_maps = nullptr;
    TTSessionTable session_table;       // the parameter form of the current decode call's sessions
    TTVerifyMaps verify_maps;           // ... and of a verify batch's tensor maps
    uint64_t launches = 0;
    uint32_t exchange_poll_limit = 0;   // 0: the exchange kernels' default (about a second)
    // last verify split plan: the part length only depends on the sessions' 128-key tile counts and
    // row counts, which stay the same for up to 128 consecutive decode steps
    std::vector<uint32_t> verify_plan_key;
    uint32_t verify_plan_target = 0;
    // optional per-launch timing of the selected kernel classes (mask of TT_PROFILE_*)
    static constexpr uint32_t kProfileSlots = 256;
    int profiling = 0;
    uint32_t profile_count = 0;
    cudaEvent_t *profile_begin = nullptr;
    cudaEvent_t *profile_end = nullptr;
    volatile int busy = 0;
    char err[512] = {0};
};

int tt_set_error(tt_context *ctx, int code, const char *fmt, ...);
void tt_bind_decode_tables(tt_context *ctx, uint32_t n_sessions, bool with_maps);
// Brackets one kernel launch with an event pair when the context profiles its class.
struct TTLaunchTimer {
    tt_context *ctx;
    cudaStream_t stream;
    bool timed;
    TTLaunchTimer(tt_context *c, cudaStream_t s, int kernel_class)
        : ctx(c), stream(s),
          timed((c->profiling & kernel_class) != 0 && c->profile_count < tt_context::kProfileSlots) {
        if (timed) cudaEventRecord(c->profile_begin[c->profile_count], s);
    }
    void stop() {
        if (timed) cudaEventRecord(ctx->profile_end[ctx->profile_count++], stream);
        timed = false;
    }
};
int tt_check_cuda(tt_context *ctx, cudaError_t e, const char *what);

// Launch with programmatic stream serialization: the kernel may start while its predecessor in the
// stream drains and must call pdl_wait() before it touches anything the predecessor wrote.
// TT_NO_PDL=1 in the environment launches plainly (an A/B switch).
bool tt_pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t tt_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tt_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Opt-in dynamic shared memory of a kernel, set once per (kernel, device) instead of on every launch: the
// attribute call is a host round trip of its own at the start of every decode step. Implemented in context.cu.
cudaError_t tt_set_smem_once_impl(const void *kernel, int smem);
template <typename K>
cudaError_t tt_set_smem_once(K kernel, int smem) { return tt_set_smem_once_impl(reinterpret_cast<const void *>(kernel), smem); }

struct TTBusyGuard {
    tt_context *ctx;
    bool ok;
    explicit TTBusyGuard(tt_context *c) : ctx(c) {
        ok = (__sync_lock_test_and_set(&c->busy, 1) == 0);
    }
    ~TTBusyGuard() { if (ok) __sync_lock_release(&ctx->busy); }
};

#define TT_ENTER(ctx)                                                                 \
    if ((ctx) == nullptr) return TT_ERR_INVALID_ARG;                                  \
    TTBusyGuard tt_guard_(ctx);                                                       \
    if (!tt_guard_.ok) return TT_ERR_BUSY;                                            \
    {                                                                                 \
        cudaError_t tt_e_ = cudaSetDevice((ctx)->device);                             \
        if (tt_e_ != cudaSuccess) return tt_check_cuda((ctx), tt_e_, "cudaSetDevice"); \
    }

// Host-side planner shared by the C entry point and the launcher.
struct TTPlan {
    uint32_t keys_per_item;
    uint32_t n_items;
    uint32_t n_partial_rows;
};

// Affine-quantised KV rows (8 or 4 bits); bits == 16 means plain fp16/bf16 rows.
struct TTKvQuant {
    uint32_t bits = 16;
    uint32_t stride_bytes = 0;   // bytes per token row
    uint32_t value_bytes = 0;    // packed values of the whole row; scales and biases follow
};

// Launchers implemented in the .cu files.
int tt_launch_decode(tt_context *ctx, cudaStream_t stream, const TTDecodeSession *h_sessions,
                     uint32_t n_sessions, const tt_attn_batch_params *p, int mode,
                     float *m_out, float *d_out, float *o_out, const TTKvQuant *quant = nullptr,
                     const tt_attn_exchange *exchange = nullptr);
int tt_launch_merge_exchange(tt_context *ctx, cudaStream_t stream, const float *part_o, const float *part_m,
                             const float *part_l, uint32_t n_parts, const tt_attn_exchange *x, uint32_t n_q_heads,
                             uint32_t head_dim, uint32_t io_dtype);
