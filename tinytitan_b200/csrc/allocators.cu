// KV-cache and Gated-DeltaNet state managers.
//
// Re-statement of the bookkeeping of KVCacheManager
// (sources/TinyTitan/Runtime/KVCache/KVCacheManager.swift:62-333, +Storage.swift:18-339,
// +Views.swift:11-72, +Validation.swift:12-81) and GDNStateManager
// (sources/TinyTitan/Runtime/KVCache/GDNStateManager.swift:18-354) over plain device
// allocations: the byte layouts (slot regions, strides, doubling growth, zero-initialised
// state) are the reference's, so the kernels read exactly what the reference's would.
// Memory comes through a tt_allocator so the same code runs on host memory in CPU-only tests.
#include "tt_common.h"

#include <new>
#include <vector>

namespace {

void *cuda_alloc(void *, size_t bytes) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
void cuda_release(void *, void *p) { cudaFree(p); }

// The stream a manager backed by the built-in CUDA allocator orders its copies and fills on. Unbound
// (the default) they are synchronous calls on the legacy default stream, which only blocking streams
// wait for; once bound (tt_kv_cache_bind_stream / tt_gdn_state_bind_stream) they are enqueued on that
// stream, in order with the kernels the caller launches there. `user` of the built-in allocator
// points at the manager's own CudaBinding.
struct CudaBinding {
    cudaStream_t stream = nullptr;
    bool bound = false;
};

int cuda_copy(void *user, void *dst, const void *src, size_t bytes) {
    const CudaBinding *b = static_cast<const CudaBinding *>(user);
    if (b != nullptr && b->bound)
        return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, b->stream) == cudaSuccess ? 0 : 1;
    return cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice) == cudaSuccess ? 0 : 1;
}
int cuda_zero(void *user, void *dst, size_t bytes) {
    const CudaBinding *b = static_cast<const CudaBinding *>(user);
    if (b != nullptr && b->bound) return cudaMemsetAsync(dst, 0, bytes, b->stream) == cudaSuccess ? 0 : 1;
    return cudaMemset(dst, 0, bytes) == cudaSuccess ? 0 : 1;
}

int cuda_download(void *, void *host_dst, const void *src, size_t bytes) {
    return cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
int cuda_upload(void *, void *dst, const void *host_src, size_t bytes) {
    return cudaMemcpy(dst, host_src, bytes, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : 1;
}

const tt_allocator kCudaAllocator = {nullptr, cuda_alloc, cuda_release, cuda_copy, cuda_zero, cuda_download, cuda_upload};

// Up to kMaxWriteRows cache rows written by one launch: block i copies row i of the K and V sources to
// the byte offsets the host worked out (slot region + position), 16 bytes per thread and step.
constexpr uint32_t kMaxWriteRows = 256;
struct WriteRowsTable { unsigned long long offset[kMaxWriteRows]; };
__global__ void __launch_bounds__(128)
kv_write_rows_kernel(unsigned char *__restrict__ k_dst, unsigned char *__restrict__ v_dst, const unsigned char *__restrict__ k_src,
                     const unsigned char *__restrict__ v_src, uint32_t row_bytes, uint32_t src_stride_bytes,
                     const __grid_constant__ WriteRowsTable table) {
    const size_t off = table.offset[blockIdx.x];
    const uint4 *ks = reinterpret_cast<const uint4 *>(k_src + (size_t)blockIdx.x * src_stride_bytes);
    const uint4 *vs = reinterpret_cast<const uint4 *>(v_src + (size_t)blockIdx.x * src_stride_bytes);
    uint4 *kd = reinterpret_cast<uint4 *>(k_dst + off), *vd = reinterpret_cast<uint4 *>(v_dst + off);
    for (uint32_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) { kd[i] = ks[i]; vd[i] = vs[i]; }
}

constexpr uint32_t kMaximumSlots = 256;            // KVCacheManager.maximumSlots
constexpr uint32_t kInitialCapacityTokens = 8192;  // KVCacheManager.initialCapacityTokens
constexpr uint32_t kQuantGroup = 64;               // KVCacheManager.quantizationGroupSize

bool allocator_ok(const tt_allocator *a) {
    return a->alloc != nullptr && a->release != nullptr && a->copy != nullptr && a->zero != nullptr;
}

}  // namespace

TT_API void tt_kv_row_layout(uint32_t elements, uint32_t precision_bits, uint32_t *out_stride,
                             uint32_t *out_value_bytes) {
    uint32_t stride, value_bytes;
    if (precision_bits == 16) {
        stride = value_bytes = elements * 2;
    } else {
        const uint32_t packed = (elements * precision_bits + 7) / 8;
        const uint32_t aligned = (packed + 1) & ~1u;
        const uint32_t groups = (elements + kQuantGroup - 1) / kQuantGroup;
        stride = aligned + groups * 2 * 2;  // fp16 scale + fp16 bias per group, after the values
        value_bytes = aligned;
    }
    if (out_stride) *out_stride = stride;
    if (out_value_bytes) *out_value_bytes = value_bytes;
}

struct tt_kv_cache {
    tt_allocator alloc;
    CudaBinding binding;   // used when `alloc` is the built-in CUDA allocator
    bool builtin = false;
    uint32_t max_context = 0, slots = 0, precision_bits = 16;
    bool ring = false;
    std::vector<void *> k, v;
    std::vector<uint32_t> stride, value_bytes, capacity;
    std::vector<uint8_t> kind;  // 0 swa, 1 full, 2 linear
    std::vector<uint32_t> position;
};

TT_API tt_kv_cache *tt_kv_cache_create(const tt_arch *arch, uint32_t max_context, uint32_t slots,
                                       uint32_t precision_bits, int fp16_ring_enabled,
                                       uint32_t max_prefill_chunk_tokens, const tt_allocator *allocator,
                                       int *out_err) {
    int err_local;
    int *err = out_err ? out_err : &err_local;
    *err = TT_OK;
    if (arch == nullptr || arch->layer_kind == nullptr || arch->n_layers == 0 || max_context == 0 ||
        max_prefill_chunk_tokens == 0 || slots == 0 || slots > kMaximumSlots ||
        (precision_bits != 16 && precision_bits != 8 && precision_bits != 4) ||
        (allocator != nullptr && !allocator_ok(allocator))) {
        *err = TT_ERR_INVALID_ARG;
        return nullptr;
    }
    tt_kv_cache *c = new (std::nothrow) tt_kv_cache();
    if (c == nullptr) { *err = TT_ERR_OOM; return nullptr; }
    c->alloc = allocator ? *allocator : kCudaAllocator;
    c->builtin = allocator == nullptr;
    if (c->builtin) c->alloc.user = &c->binding;
    c->max_context = max_context;
    c->slots = slots;
    c->precision_bits = precision_bits;
    c->ring = fp16_ring_enabled != 0;
    c->position.assign(slots, 0);
    const uint32_t swa_elems = arch->n_kv_heads * arch->head_dim;
    const uint32_t full_elems = arch->n_full_kv_heads * arch->full_head_dim;
    uint32_t swa_capacity = arch->sliding_window + max_prefill_chunk_tokens;
    if (swa_capacity < 1) swa_capacity = 1;
    if (swa_capacity > max_context) swa_capacity = max_context;
    for (uint32_t layer = 0; layer < arch->n_layers; ++layer) {
        const uint8_t kind = arch->layer_kind[layer];
        if (kind == 2) {  // linear layers keep no per-token rows
            c->k.push_back(nullptr); c->v.push_back(nullptr);
            c->stride.push_back(0); c->value_bytes.push_back(0); c->capacity.push_back(0);
            c->kind.push_back(2);
            continue;
        }
        const bool full = kind != 0;
        uint32_t stride, vbytes;
        tt_kv_row_layout(full ? full_elems : swa_elems, precision_bits, &stride, &vbytes);
        uint32_t capacity = (c->ring && !full) ? swa_capacity
                                               : (max_context < kInitialCapacityTokens ? max_context
                                                                                       : kInitialCapacityTokens);
        const size_t length = (size_t)slots * capacity * stride;
        void *kb = c->alloc.alloc(c->alloc.user, length);
        void *vb = kb ? c->alloc.alloc(c->alloc.user, length) : nullptr;
        if (kb == nullptr || vb == nullptr) {
            if (kb) c->alloc.release(c->alloc.user, kb);
            tt_kv_cache_destroy(c);
            *err = TT_ERR_OOM;
            return nullptr;
        }
        c->k.push_back(kb); c->v.push_back(vb);
        c->stride.push_back(stride); c->value_bytes.push_back(vbytes); c->capacity.push_back(capacity);
        c->kind.push_back(full ? 1 : 0);
    }
    return c;
}

TT_API void tt_kv_cache_destroy(tt_kv_cache *c) {
    if (c == nullptr) return;
    for (size_t i = 0; i < c->k.size(); ++i) {
        if (c->k[i]) c->alloc.release(c->alloc.user, c->k[i]);
        if (c->v[i]) c->alloc.release(c->alloc.user, c->v[i]);
    }
    delete c;
}

TT_API int tt_kv_cache_reserve(tt_kv_cache *c, uint32_t tokens, uint32_t slot) {
    if (c == nullptr || slot >= c->slots) return TT_ERR_INVALID_ARG;
    uint32_t needed = tokens < 1 ? 1 : tokens;
    if (needed > c->max_context) needed = c->max_context;
    for (size_t layer = 0; layer < c->kind.size(); ++layer) {
        if (c->kind[layer] == 2) continue;
        if (c->ring && c->kind[layer] == 0) continue;  // a ring's capacity is its window
        const uint32_t current = c->capacity[layer];
        if (current >= needed) continue;
        uint64_t target = current;
        while (target < needed) target *= 2;
        if (target > c->max_context) target = c->max_context;
        const uint32_t stride = c->stride[layer];
        const size_t length = (size_t)c->slots * target * stride;
        void *nk = c->alloc.alloc(c->alloc.user, length);
        void *nv = nk ? c->alloc.alloc(c->alloc.user, length) : nullptr;
        if (nk == nullptr || nv == nullptr) {
            if (nk) c->alloc.release(c->alloc.user, nk);
            return TT_ERR_OOM;
        }
        for (uint32_t s = 0; s < c->slots; ++s) {
            const uint32_t live = c->position[s] < current ? c->position[s] : current;
            const size_t used = (size_t)live * stride;
            if (used == 0) continue;
            int bad = c->alloc.copy(c->alloc.user, (char *)nk + (size_t)s * target * stride,
                                    (const char *)c->k[layer] + (size_t)s * current * stride, used);
            bad |= c->alloc.copy(c->alloc.user, (char *)nv + (size_t)s * target * stride,
                                 (const char *)c->v[layer] + (size_t)s * current * stride, used);
            if (bad) {
                c->alloc.release(c->alloc.user, nk);
                c->alloc.release(c->alloc.user, nv);
                return TT_ERR_CUDA;
            }
        }
        // the row copies above may still be in flight on the bound stream, and kernels enqueued
        // there earlier may still read the old buffers
        if (c->builtin && c->binding.bound && cudaStreamSynchronize(c->binding.stream) != cudaSuccess) {
            c->alloc.release(c->alloc.user, nk);
            c->alloc.release(c->alloc.user, nv);
            return TT_ERR_CUDA;
        }
        c->alloc.release(c->alloc.user, c->k[layer]);
        c->alloc.release(c->alloc.user, c->v[layer]);
        c->k[layer] = nk; c->v[layer] = nv;
        c->capacity[layer] = (uint32_t)target;
    }
    return TT_OK;
}

TT_API int tt_kv_cache_write_rows(tt_kv_cache *c, tt_stream stream, uint32_t layer, const uint32_t *slots,
                                  const uint32_t *positions, uint32_t n, const void *k_rows, const void *v_rows,
                                  uint32_t src_stride_bytes) {
    if (c == nullptr || layer >= c->kind.size() || c->kind[layer] == 2 || slots == nullptr || positions == nullptr ||
        k_rows == nullptr || v_rows == nullptr)
        return TT_ERR_INVALID_ARG;
    const uint32_t stride = c->stride[layer], cap = c->capacity[layer];
    if (src_stride_bytes < stride) return TT_ERR_INVALID_ARG;
    const bool ring_layer = c->ring && c->kind[layer] == 0;
    for (uint32_t base = 0; base < n; base += kMaxWriteRows) {
        const uint32_t count = n - base < kMaxWriteRows ? n - base : kMaxWriteRows;
        static thread_local WriteRowsTable table;
        for (uint32_t i = 0; i < count; ++i) {
            const uint32_t slot = slots[base + i], position = positions[base + i];
            if (slot >= c->slots || (uint64_t)position + 1 > c->max_context) return TT_ERR_INVALID_ARG;
            if (!ring_layer && position >= cap) return TT_ERR_INVALID_ARG;      // reserve() first
            table.offset[i] = ((size_t)slot * cap + position % cap) * stride;
        }
        const unsigned char *ks = static_cast<const unsigned char *>(k_rows) + (size_t)base * src_stride_bytes;
        const unsigned char *vs = static_cast<const unsigned char *>(v_rows) + (size_t)base * src_stride_bytes;
        if (!c->builtin) {     // caller-supplied memory (host memory in the CPU tests): plain copies through the allocator
            for (uint32_t i = 0; i < count; ++i) {
                int bad = c->alloc.copy(c->alloc.user, (char *)c->k[layer] + table.offset[i], ks + (size_t)i * src_stride_bytes, stride);
                bad |= c->alloc.copy(c->alloc.user, (char *)c->v[layer] + table.offset[i], vs + (size_t)i * src_stride_bytes, stride);
                if (bad) return TT_ERR_CUDA;
            }
            continue;
        }
        if (stride % 16 != 0 || src_stride_bytes % 16 != 0 || (((uintptr_t)k_rows | (uintptr_t)v_rows) & 15))
            return TT_ERR_UNSUPPORTED_SHAPE;
        kv_write_rows_kernel<<<count, 128, 0, (cudaStream_t)stream>>>(static_cast<unsigned char *>(c->k[layer]),
                                                                     static_cast<unsigned char *>(c->v[layer]), ks, vs, stride,
                                                                     src_stride_bytes, table);
        if (cudaGetLastError() != cudaSuccess) return TT_ERR_CUDA;
    }
    return TT_OK;
}

TT_API int tt_kv_cache_bind_stream(tt_kv_cache *c, tt_stream stream) {
    if (c == nullptr) return TT_ERR_INVALID_ARG;
    if (!c->builtin) return TT_ERR_UNSUPPORTED_SHAPE;   // a caller-supplied allocator orders its own copies
    c->binding.stream = (cudaStream_t)stream;
    c->binding.bound = true;
    return TT_OK;
}

static int kv_slot(tt_kv_cache *c, bool value, uint32_t layer, uint32_t position, uint32_t slot, void **out) {
    if (c == nullptr || out == nullptr || layer >= c->kind.size() || slot >= c->slots) return TT_ERR_INVALID_ARG;
    if (c->kind[layer] == 2) return TT_ERR_INVALID_ARG;  // linear layers have no KV slots
    if ((uint64_t)position + 1 > c->max_context) return TT_ERR_INVALID_ARG;
    const uint32_t cap = c->capacity[layer];
    const bool ring_layer = c->ring && c->kind[layer] == 0;
    if (!ring_layer && position >= cap) return TT_ERR_INVALID_ARG;  // reserve() first
    const size_t token = (size_t)slot * cap + position % cap;
    *out = (char *)(value ? c->v[layer] : c->k[layer]) + token * c->stride[layer];
    return TT_OK;
}

TT_API int tt_kv_cache_k_slot(tt_kv_cache *c, uint32_t layer, uint32_t position, uint32_t slot, void **out) {
    return kv_slot(c, false, layer, position, slot, out);
}
TT_API int tt_kv_cache_v_slot(tt_kv_cache *c, uint32_t layer, uint32_t position, uint32_t slot, void **out) {
    return kv_slot(c, true, layer, position, slot, out);
}

static int kv_view(tt_kv_cache *c, bool value, uint32_t layer, uint32_t slot, uint32_t valid, tt_kv_view *out) {
    if (c == nullptr || out == nullptr || layer >= c->kind.size() || slot >= c->slots) return TT_ERR_INVALID_ARG;
    if (valid > c->max_context) return TT_ERR_INVALID_ARG;
    out->buffer = value ? c->v[layer] : c->k[layer];
    out->offset = (size_t)slot * c->capacity[layer] * c->stride[layer];
    out->stride = c->stride[layer];
    out->valid_token_count = valid;
    out->precision_bits = c->precision_bits;
    out->value_bytes = c->value_bytes[layer];
    out->group_size = kQuantGroup;
    out->ring_capacity = (c->ring && c->kind[layer] == 0) ? c->capacity[layer] : 0;
    return TT_OK;
}

TT_API int tt_kv_cache_key_view(tt_kv_cache *c, uint32_t layer, uint32_t slot, uint32_t valid, tt_kv_view *out) {
    return kv_view(c, false, layer, slot, valid, out);
}
TT_API int tt_kv_cache_value_view(tt_kv_cache *c, uint32_t layer, uint32_t slot, uint32_t valid, tt_kv_view *out) {
    return kv_view(c, true, layer, slot, valid, out);
}

TT_API int tt_kv_cache_advance(tt_kv_cache *c, uint32_t slot, uint32_t count) {
    if (c == nullptr || slot >= c->slots) return TT_ERR_INVALID_ARG;
    if ((uint64_t)c->position[slot] + count > c->max_context) return TT_ERR_INVALID_ARG;
    c->position[slot] += count;
    return TT_OK;
}

TT_API int tt_kv_cache_rewind(tt_kv_cache *c, uint32_t slot, uint32_t new_position) {
    if (c == nullptr || slot >= c->slots) return TT_ERR_INVALID_ARG;
    if (new_position > c->position[slot]) return TT_ERR_INVALID_ARG;
    c->position[slot] = new_position;  // rows stay; a later pass overwrites them
    return TT_OK;
}

TT_API int tt_kv_cache_reset(tt_kv_cache *c) {
    if (c == nullptr) return TT_ERR_INVALID_ARG;
    for (auto &p : c->position) p = 0;
    return TT_OK;
}

TT_API int tt_kv_cache_reset_slot(tt_kv_cache *c, uint32_t slot) {
    if (c == nullptr || slot >= c->slots) return TT_ERR_INVALID_ARG;
    c->position[slot] = 0;
    return TT_OK;
}

TT_API uint32_t tt_kv_cache_position(const tt_kv_cache *c, uint32_t slot) {
    return (c && slot < c->slots) ? c->position[slot] : 0;
}
TT_API uint32_t tt_kv_cache_capacity(const tt_kv_cache *c, uint32_t layer) {
    return (c && layer < c->capacity.size()) ? c->capacity[layer] : 0;
}
TT_API uint32_t tt_kv_cache_stride(const tt_kv_cache *c, uint32_t layer) {
    return (c && layer < c->stride.size()) ? c->stride[layer] : 0;
}
TT_API uint32_t tt_kv_cache_layer_kind(const tt_kv_cache *c, uint32_t layer) {
    return (c && layer < c->kind.size()) ? c->kind[layer] : 2;
}
TT_API size_t tt_kv_cache_buffer_length(const tt_kv_cache *c, uint32_t layer) {
    return (c && layer < c->kind.size()) ? (size_t)c->slots * c->capacity[layer] * c->stride[layer] : 0;
}

TT_API size_t tt_kv_cache_worst_case_bytes(const tt_arch *arch, uint32_t max_context, uint32_t precision_bits,
                                           uint32_t slots) {
    if (arch == nullptr || arch->layer_kind == nullptr) return 0;
    size_t total = 0;
    for (uint32_t layer = 0; layer < arch->n_layers; ++layer) {
        const uint8_t kind = arch->layer_kind[layer];
        if (kind == 2) continue;
        uint32_t stride, vb;
        tt_kv_row_layout(kind ? arch->n_full_kv_heads * arch->full_head_dim : arch->n_kv_heads * arch->head_dim,
                         precision_bits, &stride, &vb);
        total += (size_t)slots * max_context * stride * 2;
    }
    return total;
}

TT_API size_t tt_kv_cache_snapshot_bytes(const tt_kv_cache *c, uint32_t position) {
    if (c == nullptr) return 0;
    size_t total = 0;
    for (size_t layer = 0; layer < c->kind.size(); ++layer) {
        if (c->kind[layer] == 2) continue;
        const uint32_t stored = position < c->capacity[layer] ? position : c->capacity[layer];
        total += (size_t)stored * c->stride[layer] * 2;
    }
    return total;
}

TT_API int tt_kv_cache_snapshot_export(tt_kv_cache *c, void *host_dst, size_t capacity, size_t *out_bytes) {
    if (c == nullptr || host_dst == nullptr) return TT_ERR_INVALID_ARG;
    if (c->alloc.download == nullptr) return TT_ERR_UNSUPPORTED_SHAPE;
    const uint32_t position = c->position[0];
    if (position == 0 || position > c->max_context) return TT_ERR_INVALID_ARG;   // invalidPosition
    const size_t need = tt_kv_cache_snapshot_bytes(c, position);
    if (capacity < need) return TT_ERR_INVALID_ARG;
    char *dst = static_cast<char *>(host_dst);
    for (size_t layer = 0; layer < c->kind.size(); ++layer) {
        if (c->kind[layer] == 2) continue;
        const uint32_t stored = position < c->capacity[layer] ? position : c->capacity[layer];
        const size_t len = (size_t)stored * c->stride[layer];
        // slot 0's region starts at offset 0 of the layer's buffers
        if (c->alloc.download(c->alloc.user, dst, c->k[layer], len)) return TT_ERR_CUDA;
        dst += len;
        if (c->alloc.download(c->alloc.user, dst, c->v[layer], len)) return TT_ERR_CUDA;
        dst += len;
    }
    if (out_bytes) *out_bytes = need;
    return TT_OK;
}

TT_API int tt_kv_cache_snapshot_restore(tt_kv_cache *c, uint32_t position, const void *host_src, size_t bytes) {
    if (c == nullptr || host_src == nullptr) return TT_ERR_INVALID_ARG;
    if (c->alloc.upload == nullptr) return TT_ERR_UNSUPPORTED_SHAPE;
    if (position == 0 || position > c->max_context) return TT_ERR_INVALID_ARG;
    // grow first: the segment lengths are a function of capacity
    int rc = tt_kv_cache_reserve(c, position, 0);
    if (rc != TT_OK) return rc;
    if (bytes != tt_kv_cache_snapshot_bytes(c, position)) return TT_ERR_INVALID_ARG;   // invalidLayout
    tt_kv_cache_reset(c);
    const char *src = static_cast<const char *>(host_src);
    for (size_t layer = 0; layer < c->kind.size(); ++layer) {
        if (c->kind[layer] == 2) continue;
        const uint32_t stored = position < c->capacity[layer] ? position : c->capacity[layer];
        const size_t len = (size_t)stored * c->stride[layer];
        if (c->alloc.upload(c->alloc.user, c->k[layer], src, len)) return TT_ERR_CUDA;
        src += len;
        if (c->alloc.upload(c->alloc.user, c->v[layer], src, len)) return TT_ERR_CUDA;
        src += len;
    }
    c->position[0] = position;
    return TT_OK;
}

// ------------------------------------------------------------------ GDN state

struct tt_gdn_state {
    tt_allocator alloc;
    CudaBinding binding;   // used when `alloc` is the built-in CUDA allocator
    bool builtin = false;
    uint32_t slots = 0;
    size_t state_bytes = 0, tail_bytes = 0;
    std::vector<void *> state, tail, spec_state, spec_tail;  // null for non-linear layers
};

TT_API size_t tt_gdn_state_worst_case_bytes(const tt_arch *arch, uint32_t slots) {
    if (arch == nullptr || arch->layer_kind == nullptr) return 0;
    const size_t sb = (size_t)arch->gdn_v_heads * arch->gdn_value_dim * arch->gdn_key_dim * 4;
    const uint32_t qkv = 2 * arch->gdn_k_heads * arch->gdn_key_dim + arch->gdn_v_heads * arch->gdn_value_dim;
    const size_t tb = (size_t)(arch->gdn_conv_kernel > 0 ? arch->gdn_conv_kernel - 1 : 0) * qkv * 2;
    size_t linear = 0;
    for (uint32_t i = 0; i < arch->n_layers; ++i) linear += arch->layer_kind[i] == 2;
    return (size_t)slots * linear * (sb + tb);
}

TT_API tt_gdn_state *tt_gdn_state_create(const tt_arch *arch, uint32_t slots, int enable_speculative_checkpoint,
                                         const tt_allocator *allocator, int *out_err) {
    int err_local;
    int *err = out_err ? out_err : &err_local;
    *err = TT_OK;
    if (arch == nullptr || arch->layer_kind == nullptr || slots == 0 || slots > kMaximumSlots ||
        (allocator != nullptr && !allocator_ok(allocator))) {
        *err = TT_ERR_INVALID_ARG;
        return nullptr;
    }
    tt_gdn_state *g = new (std::nothrow) tt_gdn_state();
    if (g == nullptr) { *err = TT_ERR_OOM; return nullptr; }
    g->alloc = allocator ? *allocator : kCudaAllocator;
    g->builtin = allocator == nullptr;
    if (g->builtin) g->alloc.user = &g->binding;
    g->slots = slots;
    g->state_bytes = (size_t)arch->gdn_v_heads * arch->gdn_value_dim * arch->gdn_key_dim * 4;
    const uint32_t qkv = 2 * arch->gdn_k_heads * arch->gdn_key_dim + arch->gdn_v_heads * arch->gdn_value_dim;
    g->tail_bytes = (size_t)(arch->gdn_conv_kernel > 0 ? arch->gdn_conv_kernel - 1 : 0) * qkv * 2;
    for (uint32_t layer = 0; layer < arch->n_layers; ++layer) {
        void *s = nullptr, *t = nullptr, *ss = nullptr, *st = nullptr;
        if (arch->layer_kind[layer] == 2) {
            if (g->state_bytes == 0 || g->tail_bytes == 0) {  // linear layer with an empty config
                tt_gdn_state_destroy(g);
                *err = TT_ERR_INVALID_ARG;
                return nullptr;
            }
            s = g->alloc.alloc(g->alloc.user, g->state_bytes * slots);
            t = g->alloc.alloc(g->alloc.user, g->tail_bytes * slots);
            if (enable_speculative_checkpoint) {
                ss = g->alloc.alloc(g->alloc.user, g->state_bytes * slots);
                st = g->alloc.alloc(g->alloc.user, g->tail_bytes * slots);
            }
            const bool ok = s && t && (!enable_speculative_checkpoint || (ss && st));
            g->state.push_back(s); g->tail.push_back(t); g->spec_state.push_back(ss); g->spec_tail.push_back(st);
            if (!ok) {
                tt_gdn_state_destroy(g);
                *err = TT_ERR_OOM;
                return nullptr;
            }
        } else {
            g->state.push_back(nullptr); g->tail.push_back(nullptr);
            g->spec_state.push_back(nullptr); g->spec_tail.push_back(nullptr);
        }
    }
    if (tt_gdn_state_reset(g) != TT_OK) {
        tt_gdn_state_destroy(g);
        *err = TT_ERR_CUDA;
        return nullptr;
    }
    return g;
}

TT_API void tt_gdn_state_destroy(tt_gdn_state *g) {
    if (g == nullptr) return;
    for (size_t i = 0; i < g->state.size(); ++i) {
        if (g->state[i]) g->alloc.release(g->alloc.user, g->state[i]);
        if (g->tail[i]) g->alloc.release(g->alloc.user, g->tail[i]);
        if (g->spec_state[i]) g->alloc.release(g->alloc.user, g->spec_state[i]);
        if (g->spec_tail[i]) g->alloc.release(g->alloc.user, g->spec_tail[i]);
    }
    delete g;
}

static int gdn_slot(tt_gdn_state *g, const std::vector<void *> &bufs, size_t bytes, uint32_t layer, uint32_t slot,
                    void **out) {
    if (g == nullptr || out == nullptr || layer >= bufs.size() || slot >= g->slots) return TT_ERR_INVALID_ARG;
    if (bufs[layer] == nullptr) return TT_ERR_INVALID_ARG;  // not a linear layer / no checkpoint twin
    *out = (char *)bufs[layer] + (size_t)slot * bytes;
    return TT_OK;
}

TT_API int tt_gdn_state_state_slot(tt_gdn_state *g, uint32_t layer, uint32_t slot, void **out) {
    return g ? gdn_slot(g, g->state, g->state_bytes, layer, slot, out) : TT_ERR_INVALID_ARG;
}
TT_API int tt_gdn_state_conv_tail_slot(tt_gdn_state *g, uint32_t layer, uint32_t slot, void **out) {
    return g ? gdn_slot(g, g->tail, g->tail_bytes, layer, slot, out) : TT_ERR_INVALID_ARG;
}
TT_API int tt_gdn_state_speculative_state_slot(tt_gdn_state *g, uint32_t layer, uint32_t slot, void **out) {
    return g ? gdn_slot(g, g->spec_state, g->state_bytes, layer, slot, out) : TT_ERR_INVALID_ARG;
}

TT_API int tt_gdn_state_reset(tt_gdn_state *g) {
    if (g == nullptr) return TT_ERR_INVALID_ARG;
    int bad = 0;
    for (size_t i = 0; i < g->state.size(); ++i) {
        if (g->state[i]) bad |= g->alloc.zero(g->alloc.user, g->state[i], g->state_bytes * g->slots);
        if (g->tail[i]) bad |= g->alloc.zero(g->alloc.user, g->tail[i], g->tail_bytes * g->slots);
        if (g->spec_state[i]) bad |= g->alloc.zero(g->alloc.user, g->spec_state[i], g->state_bytes * g->slots);
        if (g->spec_tail[i]) bad |= g->alloc.zero(g->alloc.user, g->spec_tail[i], g->tail_bytes * g->slots);
    }
    return bad ? TT_ERR_CUDA : TT_OK;
}

TT_API int tt_gdn_state_reset_slot(tt_gdn_state *g, uint32_t slot) {
    if (g == nullptr || slot >= g->slots) return TT_ERR_INVALID_ARG;
    int bad = 0;
    for (size_t i = 0; i < g->state.size(); ++i) {
        if (g->state[i]) bad |= g->alloc.zero(g->alloc.user, (char *)g->state[i] + slot * g->state_bytes, g->state_bytes);
        if (g->tail[i]) bad |= g->alloc.zero(g->alloc.user, (char *)g->tail[i] + slot * g->tail_bytes, g->tail_bytes);
    }
    return bad ? TT_ERR_CUDA : TT_OK;
}

TT_API int tt_gdn_state_bind_stream(tt_gdn_state *g, tt_stream stream) {
    if (g == nullptr) return TT_ERR_INVALID_ARG;
    if (!g->builtin) return TT_ERR_UNSUPPORTED_SHAPE;
    g->binding.stream = (cudaStream_t)stream;
    g->binding.bound = true;
    return TT_OK;
}

TT_API int tt_gdn_state_speculative_restore(tt_gdn_state *g, tt_stream stream) {
    if (g == nullptr) return TT_ERR_INVALID_ARG;
    for (size_t i = 0; i < g->state.size(); ++i)
        if (g->state[i] && (!g->spec_state[i] || !g->spec_tail[i])) return TT_ERR_INVALID_ARG;  // invalidLayout
    // Enqueued on the caller's stream like the reference's blit, which is encoded into the same command
    // buffer as the verify pass (GDNStateManager.swift:265-292): it runs after the step kernels that wrote
    // the checkpoint and before whatever the caller enqueues next. A caller-supplied allocator copies in
    // its own way (the host allocator of the CPU tests is synchronous).
    CudaBinding on_stream;
    on_stream.stream = (cudaStream_t)stream;
    on_stream.bound = true;
    void *user = g->builtin ? &on_stream : g->alloc.user;
    int bad = 0;
    for (size_t i = 0; i < g->state.size(); ++i) {
        if (!g->state[i]) continue;
        // slot 0's segment, as the reference copies stateBytesPerLayer from offset 0
        bad |= g->alloc.copy(user, g->state[i], g->spec_state[i], g->state_bytes);
        bad |= g->alloc.copy(user, g->tail[i], g->spec_tail[i], g->tail_bytes);
    }
    return bad ? TT_ERR_CUDA : TT_OK;
}

TT_API size_t tt_gdn_state_bytes_per_layer(const tt_gdn_state *g) { return g ? g->state_bytes : 0; }
TT_API size_t tt_gdn_state_conv_tail_bytes_per_layer(const tt_gdn_state *g) { return g ? g->tail_bytes : 0; }
TT_API int tt_gdn_state_is_linear(const tt_gdn_state *g, uint32_t layer) {
    return (g && layer < g->state.size() && g->state[layer] != nullptr) ? 1 : 0;
}

TT_API size_t tt_gdn_state_snapshot_bytes(const tt_gdn_state *g) {
    if (g == nullptr) return 0;
    size_t linear = 0;
    for (void *p : g->state) linear += p != nullptr;
    return linear * (g->state_bytes + g->tail_bytes);
}

TT_API int tt_gdn_state_snapshot_export(tt_gdn_state *g, void *host_dst, size_t capacity, size_t *out_bytes) {
    if (g == nullptr || host_dst == nullptr) return TT_ERR_INVALID_ARG;
    if (g->alloc.download == nullptr) return TT_ERR_UNSUPPORTED_SHAPE;
    const size_t need = tt_gdn_state_snapshot_bytes(g);
    if (capacity < need) return TT_ERR_INVALID_ARG;
    char *dst = static_cast<char *>(host_dst);
    for (size_t i = 0; i < g->state.size(); ++i) {
        if (!g->state[i]) continue;
        if (g->alloc.download(g->alloc.user, dst, g->state[i], g->state_bytes)) return TT_ERR_CUDA;
        dst += g->state_bytes;
        if (g->alloc.download(g->alloc.user, dst, g->tail[i], g->tail_bytes)) return TT_ERR_CUDA;
        dst += g->tail_bytes;
    }
    if (out_bytes) *out_bytes = need;
    return TT_OK;
}

TT_API int tt_gdn_state_snapshot_restore(tt_gdn_state *g, const void *host_src, size_t bytes) {
    if (g == nullptr || host_src == nullptr) return TT_ERR_INVALID_ARG;
    if (g->alloc.upload == nullptr) return TT_ERR_UNSUPPORTED_SHAPE;
    if (bytes != tt_gdn_state_snapshot_bytes(g)) return TT_ERR_INVALID_ARG;   // invalidLayout
    int rc = tt_gdn_state_reset(g);
    if (rc != TT_OK) return rc;
    const char *src = static_cast<const char *>(host_src);
    for (size_t i = 0; i < g->state.size(); ++i) {
        if (!g->state[i]) continue;
        if (g->alloc.upload(g->alloc.user, g->state[i], src, g->state_bytes)) return TT_ERR_CUDA;
        src += g->state_bytes;
        if (g->alloc.upload(g->alloc.user, g->tail[i], src, g->tail_bytes)) return TT_ERR_CUDA;
        src += g->tail_bytes;
    }
    return TT_OK;
}
