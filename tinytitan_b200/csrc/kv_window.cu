// Host-KV streaming tier: the authoritative K/V rows of the full-attention layers live in a host
// arena, device memory holds a small window of rows per (layer, slot), and an attention call reads
// the window through an indirection list (logical key -> window row).
//
// Re-statement of the bookkeeping of KVCacheManager+HostStreaming.swift:33-364 and
// KVCacheManager+HostStreamingPrefill.swift:12-436 (sources/TinyTitan/Runtime/KVCache/) over a
// tt_allocator: windowRowMap / windowOccupant / windowCursor / windowDirty / windowPinned /
// windowProtected, ensureWindowRow's clock-hand eviction with write-back, prepareDecodeWindow,
// the prefill staging + union + indirection (preparePrefillWindow), commitStreamedRows and
// resetStreamedWindow. The consumers are tt_attn_decode_window (sel_rows) and
// tt_attn_prefill_causal_selected (keep_rows). Window memory comes through the allocator (device
// memory by default, host memory in the CPU tests); arena <-> window copies use its
// upload / download, window <-> staging copies its copy.
#include "tt_common.h"

#include <cstdlib>
#include <new>
#include <unordered_set>
#include <vector>

namespace {

constexpr uint32_t kNone = 0xFFFFFFFFu;

void *cuda_alloc(void *, size_t bytes) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
void cuda_release(void *, void *p) { cudaFree(p); }
int cuda_copy(void *, void *dst, const void *src, size_t bytes) {
    return cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice) == cudaSuccess ? 0 : 1;
}
int cuda_zero(void *, void *dst, size_t bytes) { return cudaMemset(dst, 0, bytes) == cudaSuccess ? 0 : 1; }
int cuda_download(void *, void *host_dst, const void *src, size_t bytes) {
    return cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
int cuda_upload(void *, void *dst, const void *host_src, size_t bytes) {
    return cudaMemcpy(dst, host_src, bytes, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : 1;
}
const tt_allocator kCudaAllocator = {nullptr, cuda_alloc, cuda_release, cuda_copy, cuda_zero, cuda_download, cuda_upload};

struct Layer {
    unsigned char *host_k = nullptr, *host_v = nullptr;      // [slots][max_context][stride], host arena
    unsigned char *win_k = nullptr, *win_v = nullptr;        // [slots][window][stride], allocator memory
    std::vector<uint32_t> row_map;                           // [slots][max_context] -> window row or kNone
    std::vector<uint32_t> occupant;                          // [slots][window] -> logical position or kNone
    std::vector<uint32_t> cursor;                            // [slots] clock hand
    std::vector<uint8_t> dirty;                              // [slots][window]
    std::vector<int64_t> pinned;                             // [slots] position written this step, or -1
    // prefill staging, per slot
    std::vector<unsigned char *> stage_k, stage_v;
    std::vector<uint32_t> stage_capacity, stage_start, stage_count;
    std::vector<uint8_t> stage_active;
};

}  // namespace

struct tt_kv_window {
    tt_allocator alloc;
    uint32_t stride = 0, max_context = 0, slots = 0, window = 0;
    std::vector<Layer> layers;
    std::vector<uint8_t> needed;                             // [max_context] scratch of the prefill union
    std::unordered_set<uint64_t> protect;                    // rows of the selection being gathered
    uint64_t evictions = 0, row_copies = 0, copy_bytes = 0;
};

namespace {

bool valid(const tt_kv_window *w, uint32_t layer, uint32_t slot) {
    return w != nullptr && layer < w->layers.size() && slot < w->slots;
}

// windowRow (KVCacheManager+HostStreaming.swift:120-130): the row that holds `position`, or -1
int64_t window_row(const tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position) {
    const Layer &l = w->layers[layer];
    const uint32_t value = l.row_map[(size_t)slot * w->max_context + position];
    if (value == kNone) return -1;
    if (l.occupant[(size_t)slot * w->window + value] != position) return -1;
    return value;
}

unsigned char *arena_row(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position, bool key) {
    Layer &l = w->layers[layer];
    return (key ? l.host_k : l.host_v) + ((size_t)slot * w->max_context + position) * w->stride;
}
unsigned char *win_row(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t row, bool key) {
    Layer &l = w->layers[layer];
    return (key ? l.win_k : l.win_v) + ((size_t)slot * w->window + row) * w->stride;
}

// flushWindowRow (:213-232): a dirty row goes back to the arena
int flush_row(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t row) {
    Layer &l = w->layers[layer];
    const size_t index = (size_t)slot * w->window + row;
    if (!l.dirty[index]) return TT_OK;
    const uint32_t occupant = l.occupant[index];
    if (occupant == kNone) { l.dirty[index] = 0; return TT_OK; }
    int bad = w->alloc.download(w->alloc.user, arena_row(w, layer, slot, occupant, true), win_row(w, layer, slot, row, true), w->stride);
    bad |= w->alloc.download(w->alloc.user, arena_row(w, layer, slot, occupant, false), win_row(w, layer, slot, row, false), w->stride);
    l.dirty[index] = 0;
    return bad ? TT_ERR_CUDA : TT_OK;
}

// ensureWindowRow (:152-209): the row of `position`, evicting round-robin when it is not resident.
// Rows of the selection being gathered and the row of the token written this step are skipped.
// TT_ERR_OOM when every row is protected ("the selection plus the in-flight token must fit").
int ensure_row(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position, bool for_write, uint32_t *out_row) {
    Layer &l = w->layers[layer];
    const int64_t resident = window_row(w, layer, slot, position);
    if (resident >= 0) {
        if (for_write) {
            l.pinned[slot] = position;
            l.dirty[(size_t)slot * w->window + resident] = 1;
        }
        *out_row = (uint32_t)resident;
        return TT_OK;
    }
    const uint32_t rows = w->window;
    int64_t chosen = -1;
    for (uint32_t tries = 0; tries < rows; ++tries) {
        const uint32_t row = l.cursor[slot];
        l.cursor[slot] = (row + 1) % rows;
        const size_t index = (size_t)slot * rows + row;
        const uint32_t occupant = l.occupant[index];
        const uint64_t key = ((uint64_t)layer * w->slots + slot) * rows + row;
        if (w->protect.count(key)) continue;
        if (occupant != kNone && l.pinned[slot] >= 0 && occupant == (uint32_t)l.pinned[slot]) continue;
        if (occupant != kNone) {
            const int rc = flush_row(w, layer, slot, row);
            if (rc != TT_OK) return rc;
            l.row_map[(size_t)slot * w->max_context + occupant] = kNone;
            l.occupant[index] = kNone;
            l.dirty[index] = 0;
            w->evictions++;
        }
        chosen = row;
        break;
    }
    if (chosen < 0) return TT_ERR_OOM;
    const size_t index = (size_t)slot * rows + chosen;
    l.occupant[index] = position;
    l.row_map[(size_t)slot * w->max_context + position] = (uint32_t)chosen;
    l.dirty[index] = for_write ? 1 : 0;
    if (for_write) l.pinned[slot] = position;
    *out_row = (uint32_t)chosen;
    return TT_OK;
}

int fetch_row(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position, uint32_t row) {
    int bad = w->alloc.upload(w->alloc.user, win_row(w, layer, slot, row, true), arena_row(w, layer, slot, position, true), w->stride);
    bad |= w->alloc.upload(w->alloc.user, win_row(w, layer, slot, row, false), arena_row(w, layer, slot, position, false), w->stride);
    w->copy_bytes += (uint64_t)w->stride * 2;
    w->row_copies++;
    return bad ? TT_ERR_CUDA : TT_OK;
}

}  // namespace

TT_API tt_kv_window *tt_kv_window_create(uint32_t n_layers, uint32_t stride_bytes, uint32_t max_context, uint32_t slots,
                                         uint32_t window_tokens, const tt_allocator *allocator, int *out_err) {
    int err_local;
    int *err = out_err ? out_err : &err_local;
    *err = TT_OK;
    if (n_layers == 0 || stride_bytes == 0 || max_context == 0 || slots == 0 || slots > 256 || window_tokens == 0 ||
        (allocator != nullptr && (!allocator->alloc || !allocator->release || !allocator->copy || !allocator->download ||
                                  !allocator->upload))) {
        *err = TT_ERR_INVALID_ARG;
        return nullptr;
    }
    tt_kv_window *w = new (std::nothrow) tt_kv_window();
    if (w == nullptr) { *err = TT_ERR_OOM; return nullptr; }
    w->alloc = allocator ? *allocator : kCudaAllocator;
    w->stride = stride_bytes; w->max_context = max_context; w->slots = slots;
    w->window = window_tokens < max_context ? window_tokens : max_context;      // windowTokens.map { min($0, maxContext) }
    w->needed.assign(max_context, 0);
    w->layers.resize(n_layers);
    for (Layer &l : w->layers) {
        const size_t arena = (size_t)slots * max_context * stride_bytes, win = (size_t)slots * w->window * stride_bytes;
        l.host_k = static_cast<unsigned char *>(calloc(arena, 1));
        l.host_v = static_cast<unsigned char *>(calloc(arena, 1));
        l.win_k = static_cast<unsigned char *>(w->alloc.alloc(w->alloc.user, win));
        l.win_v = static_cast<unsigned char *>(w->alloc.alloc(w->alloc.user, win));
        if (!l.host_k || !l.host_v || !l.win_k || !l.win_v) {
            tt_kv_window_destroy(w);
            *err = TT_ERR_OOM;
            return nullptr;
        }
        l.row_map.assign((size_t)slots * max_context, kNone);
        l.occupant.assign((size_t)slots * w->window, kNone);
        l.cursor.assign(slots, 0);
        l.dirty.assign((size_t)slots * w->window, 0);
        l.pinned.assign(slots, -1);
        l.stage_k.assign(slots, nullptr); l.stage_v.assign(slots, nullptr);
        l.stage_capacity.assign(slots, 0); l.stage_start.assign(slots, 0); l.stage_count.assign(slots, 0);
        l.stage_active.assign(slots, 0);
    }
    return w;
}

TT_API void tt_kv_window_destroy(tt_kv_window *w) {
    if (w == nullptr) return;
    for (Layer &l : w->layers) {
        free(l.host_k); free(l.host_v);
        if (l.win_k) w->alloc.release(w->alloc.user, l.win_k);
        if (l.win_v) w->alloc.release(w->alloc.user, l.win_v);
        for (unsigned char *p : l.stage_k) if (p) w->alloc.release(w->alloc.user, p);
        for (unsigned char *p : l.stage_v) if (p) w->alloc.release(w->alloc.user, p);
    }
    delete w;
}

TT_API size_t tt_kv_window_bytes(const tt_kv_window *w) {
    return w ? (size_t)w->layers.size() * 2 * w->slots * w->window * w->stride : 0;
}
TT_API size_t tt_kv_window_host_arena_bytes(const tt_kv_window *w) {
    return w ? (size_t)w->layers.size() * 2 * w->slots * w->max_context * w->stride : 0;
}
TT_API uint32_t tt_kv_window_tokens(const tt_kv_window *w) { return w ? w->window : 0; }

// streamingPrefillChunkTokens (:96-107)
TT_API uint32_t tt_kv_window_prefill_chunk_tokens(const tt_kv_window *w, uint32_t configured, uint32_t selection_width) {
    if (w == nullptr || selection_width == 0) return configured;
    uint32_t bound = w->window / selection_width;
    if (bound > configured) bound = configured;
    return bound < 1 ? 1 : bound;
}

TT_API int tt_kv_window_base(tt_kv_window *w, uint32_t layer, uint32_t slot, void **out_k, void **out_v) {
    if (!valid(w, layer, slot)) return TT_ERR_INVALID_ARG;
    if (out_k) *out_k = win_row(w, layer, slot, 0, true);
    if (out_v) *out_v = win_row(w, layer, slot, 0, false);
    return TT_OK;
}

// kSlot / vSlot of a streamed layer (KVCacheManager+Storage.swift:173-201): where the projection
// writes position's row -- a window row, marked dirty and pinned for this step; a row inside an
// active prefill staging range goes to the staging buffers instead (stagedRange, :47-62).
TT_API int tt_kv_window_write_slot(tt_kv_window *w, uint32_t layer, uint32_t position, uint32_t slot, void **out_k,
                                   void **out_v) {
    if (!valid(w, layer, slot) || position >= w->max_context) return TT_ERR_INVALID_ARG;
    Layer &l = w->layers[layer];
    if (l.stage_active[slot] && position >= l.stage_start[slot] && position < l.stage_start[slot] + l.stage_count[slot]) {
        const size_t off = (size_t)(position - l.stage_start[slot]) * w->stride;
        if (out_k) *out_k = l.stage_k[slot] + off;
        if (out_v) *out_v = l.stage_v[slot] + off;
        return TT_OK;
    }
    uint32_t row = 0;
    const int rc = ensure_row(w, layer, slot, position, true, &row);
    if (rc != TT_OK) return rc;
    if (out_k) *out_k = win_row(w, layer, slot, row, true);
    if (out_v) *out_v = win_row(w, layer, slot, row, false);
    return TT_OK;
}

TT_API int tt_kv_window_row_of(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position, int64_t *out_row) {
    if (!valid(w, layer, slot) || position >= w->max_context || out_row == nullptr) return TT_ERR_INVALID_ARG;
    *out_row = window_row(w, layer, slot, position);
    return TT_OK;
}

// prepareDecodeWindow (:299-363): gather the keys a decode step reads into the window; returns the
// indirection lists (logical key, window row). `indices` NULL = every key 0..count-1 (dense path).
TT_API int tt_kv_window_prepare_decode(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position,
                                       const uint32_t *indices, uint32_t count, uint32_t *out_indices,
                                       uint32_t *out_rows) {
    if (!valid(w, layer, slot) || position >= w->max_context || out_indices == nullptr || out_rows == nullptr)
        return TT_ERR_INVALID_ARG;
    if (count == 0) return TT_ERR_INVALID_ARG;            // "decode selection is empty"
    if (count > w->window) return TT_ERR_OOM;            // "does not fit the KV window"
    for (uint32_t i = 0; i < count; ++i)
        if ((indices ? indices[i] : i) > position) return TT_ERR_INVALID_ARG;   // past the current position
    uint32_t row = 0;
    int rc = ensure_row(w, layer, slot, position, false, &row);      // pinForDecode
    if (rc != TT_OK) return rc;
    w->layers[layer].pinned[slot] = position;
    w->protect.clear();
    for (uint32_t i = 0; i < count; ++i) {
        const uint32_t logical = indices ? indices[i] : i;
        const bool resident = window_row(w, layer, slot, logical) >= 0;
        rc = ensure_row(w, layer, slot, logical, false, &row);
        if (rc != TT_OK) { w->protect.clear(); return rc; }
        w->protect.insert(((uint64_t)layer * w->slots + slot) * w->window + row);
        if (!resident && logical != position) {
            rc = fetch_row(w, layer, slot, logical, row);
            if (rc != TT_OK) { w->protect.clear(); return rc; }
        }
        out_indices[i] = logical;
        out_rows[i] = row;
    }
    w->protect.clear();
    return TT_OK;
}

// beginPrefillWrite (+HostStreamingPrefill.swift:14-45): the chunk's rows are projected into a
// staging buffer, [token_count][stride] per slot.
TT_API int tt_kv_window_begin_prefill(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t start_position,
                                      uint32_t token_count, void **out_stage_k, void **out_stage_v) {
    if (!valid(w, layer, slot) || token_count == 0 || (uint64_t)start_position + token_count > w->max_context)
        return TT_ERR_INVALID_ARG;
    Layer &l = w->layers[layer];
    if (l.stage_capacity[slot] < token_count) {
        if (l.stage_k[slot]) w->alloc.release(w->alloc.user, l.stage_k[slot]);
        if (l.stage_v[slot]) w->alloc.release(w->alloc.user, l.stage_v[slot]);
        l.stage_k[slot] = static_cast<unsigned char *>(w->alloc.alloc(w->alloc.user, (size_t)token_count * w->stride));
        l.stage_v[slot] = static_cast<unsigned char *>(w->alloc.alloc(w->alloc.user, (size_t)token_count * w->stride));
        if (!l.stage_k[slot] || !l.stage_v[slot]) { l.stage_capacity[slot] = 0; return TT_ERR_OOM; }
        l.stage_capacity[slot] = token_count;
    }
    l.stage_start[slot] = start_position; l.stage_count[slot] = token_count; l.stage_active[slot] = 1;
    if (out_stage_k) *out_stage_k = l.stage_k[slot];
    if (out_stage_v) *out_stage_v = l.stage_v[slot];
    return TT_OK;
}

// preparePrefillWindow (:72-115): the union of the chunk's per-row selections is made resident
// (markPrefillUnion + assignPrefillRows), the per-row indirection is filled (fillPrefillIndirection)
// and the chunk's own needed rows are copied from staging into the window
// (encodePrefillStagingBlits). `sel_indices` NULL = dense: row t keeps keys 0..start+t.
TT_API int tt_kv_window_prepare_prefill(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t start_position,
                                        uint32_t token_count, const uint32_t *sel_indices, uint32_t sel_index_stride,
                                        const uint32_t *sel_counts, uint32_t *out_indices, uint32_t *out_rows,
                                        uint32_t *out_counts, uint32_t out_index_stride) {
    if (!valid(w, layer, slot) || token_count == 0 || out_indices == nullptr || out_rows == nullptr || out_counts == nullptr)
        return TT_ERR_INVALID_ARG;
    const uint64_t visible64 = (uint64_t)start_position + token_count;
    if (visible64 > w->max_context) return TT_ERR_INVALID_ARG;
    const uint32_t visible = (uint32_t)visible64;
    const bool sparse = sel_indices != nullptr;
    if (sparse && (sel_counts == nullptr || sel_index_stride == 0)) return TT_ERR_INVALID_ARG;
    if (!sparse && visible > w->window) return TT_ERR_OOM;     // dense prefill does not fit the window
    if (out_index_stride < (sparse ? sel_index_stride : visible)) return TT_ERR_INVALID_ARG;
    Layer &l = w->layers[layer];
    // union
    std::fill(w->needed.begin(), w->needed.begin() + visible, 0);
    for (uint32_t t = 0; t < token_count; ++t) {
        const uint32_t count = sparse ? sel_counts[t] : start_position + t + 1;
        if (sparse && count > sel_index_stride) return TT_ERR_INVALID_ARG;
        for (uint32_t i = 0; i < count; ++i) {
            const uint32_t logical = sparse ? sel_indices[(size_t)t * sel_index_stride + i] : i;
            if (logical >= visible) return TT_ERR_INVALID_ARG;  // "prefill selection exceeds visible"
            w->needed[logical] = 1;
        }
    }
    uint32_t needed = 0;
    for (uint32_t p = 0; p < visible; ++p) needed += w->needed[p];
    if (needed > w->window) return TT_ERR_OOM;                  // "selection union exceeds the KV window"
    // rows
    w->protect.clear();
    for (uint32_t p = 0; p < visible; ++p) {
        if (!w->needed[p]) continue;
        const bool resident = window_row(w, layer, slot, p) >= 0;
        uint32_t row = 0;
        int rc = ensure_row(w, layer, slot, p, false, &row);
        if (rc != TT_OK) { w->protect.clear(); return rc; }
        w->protect.insert(((uint64_t)layer * w->slots + slot) * w->window + row);
        if (!resident && p < start_position) {
            rc = fetch_row(w, layer, slot, p, row);
            if (rc != TT_OK) { w->protect.clear(); return rc; }
        }
    }
    w->protect.clear();
    // indirection
    for (uint32_t t = 0; t < token_count; ++t) {
        const uint32_t count = sparse ? sel_counts[t] : start_position + t + 1;
        out_counts[t] = count;
        for (uint32_t i = 0; i < count; ++i) {
            const uint32_t logical = sparse ? sel_indices[(size_t)t * sel_index_stride + i] : i;
            const int64_t row = window_row(w, layer, slot, logical);
            out_indices[(size_t)t * out_index_stride + i] = logical;
            out_rows[(size_t)t * out_index_stride + i] = row >= 0 ? (uint32_t)row : 0u;
        }
    }
    // the chunk's own rows: staging -> window
    if (l.stage_active[slot]) {
        for (uint32_t p = start_position; p < visible; ++p) {
            if (!w->needed[p] || p < l.stage_start[slot] || p >= l.stage_start[slot] + l.stage_count[slot]) continue;
            const int64_t row = window_row(w, layer, slot, p);
            if (row < 0) continue;
            const size_t off = (size_t)(p - l.stage_start[slot]) * w->stride;
            int bad = w->alloc.copy(w->alloc.user, win_row(w, layer, slot, (uint32_t)row, true), l.stage_k[slot] + off, w->stride);
            bad |= w->alloc.copy(w->alloc.user, win_row(w, layer, slot, (uint32_t)row, false), l.stage_v[slot] + off, w->stride);
            if (bad) return TT_ERR_CUDA;
            l.dirty[(size_t)slot * w->window + row] = 0;
        }
    }
    return TT_OK;
}

// commitStreamedRows (:288-339), called by advance: staged chunk rows go to the arena in one copy
// per layer, rows written straight into the window are flushed; the step's pin is released.
TT_API int tt_kv_window_commit(tt_kv_window *w, uint32_t slot, uint32_t position, uint32_t count) {
    if (w == nullptr || slot >= w->slots || (uint64_t)position + count > w->max_context) return TT_ERR_INVALID_ARG;
    for (uint32_t layer = 0; layer < w->layers.size(); ++layer) {
        Layer &l = w->layers[layer];
        if (l.stage_active[slot]) {
            const uint32_t start = l.stage_start[slot], staged = l.stage_count[slot];
            const uint32_t end = start + staged;
            const uint32_t available = position >= start && end > position ? (count < end - position ? count : end - position) : 0u;
            if (available > 0) {
                const size_t off = (size_t)(position - start) * w->stride;
                int bad = w->alloc.download(w->alloc.user, arena_row(w, layer, slot, position, true), l.stage_k[slot] + off,
                                            (size_t)available * w->stride);
                bad |= w->alloc.download(w->alloc.user, arena_row(w, layer, slot, position, false), l.stage_v[slot] + off,
                                         (size_t)available * w->stride);
                if (bad) return TT_ERR_CUDA;
            }
            l.stage_active[slot] = 0; l.stage_start[slot] = 0; l.stage_count[slot] = 0;
        } else {
            for (uint32_t p = position; p < position + count; ++p) {
                const int64_t row = window_row(w, layer, slot, p);
                if (row < 0) continue;
                const int rc = flush_row(w, layer, slot, (uint32_t)row);
                if (rc != TT_OK) return rc;
            }
        }
        l.pinned[slot] = -1;
    }
    return TT_OK;
}

// resetStreamedWindow (:341-366): walks the window, not the logical map
TT_API int tt_kv_window_reset_slot(tt_kv_window *w, uint32_t slot) {
    if (w == nullptr || slot >= w->slots) return TT_ERR_INVALID_ARG;
    for (Layer &l : w->layers) {
        for (uint32_t row = 0; row < w->window; ++row) {
            const size_t index = (size_t)slot * w->window + row;
            if (l.occupant[index] != kNone) l.row_map[(size_t)slot * w->max_context + l.occupant[index]] = kNone;
            l.occupant[index] = kNone;
            l.dirty[index] = 0;
        }
        l.cursor[slot] = 0; l.pinned[slot] = -1;
        l.stage_active[slot] = 0; l.stage_start[slot] = 0; l.stage_count[slot] = 0;
    }
    return TT_OK;
}

// hostRowBytes: one authoritative row of the arena
TT_API int tt_kv_window_host_row(tt_kv_window *w, uint32_t layer, uint32_t slot, uint32_t position, int key, void *dst) {
    if (!valid(w, layer, slot) || position >= w->max_context || dst == nullptr) return TT_ERR_INVALID_ARG;
    memcpy(dst, arena_row(w, layer, slot, position, key != 0), w->stride);
    return TT_OK;
}

TT_API void tt_kv_window_counters(const tt_kv_window *w, uint64_t *out_evictions, uint64_t *out_row_copies,
                                  uint64_t *out_copy_bytes) {
    if (w == nullptr) return;
    if (out_evictions) *out_evictions = w->evictions;
    if (out_row_copies) *out_row_copies = w->row_copies;
    if (out_copy_bytes) *out_copy_bytes = w->copy_bytes;
}
