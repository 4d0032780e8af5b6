"""Host-side mirror of KVCacheManager and GDNStateManager over the C ABI.

  KVCacheManager   sources/TinyTitan/Runtime/KVCache/KVCacheManager.swift:62-333 (+Storage, +Views)
  GDNStateManager  sources/TinyTitan/Runtime/KVCache/GDNStateManager.swift:18-354

Accessors return integer device addresses (the reference returns MTLBuffer + byte offset).
`allocator="host"` backs the managers with host memory so that the bookkeeping can be tested
without a GPU; the default is CUDA device memory.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

from . import _lib as L
from .operators import LinearAttentionConfig, _stream

SWA, FULL, LINEAR = 0, 1, 2


@dataclass
class ArchConfig:
    """The fields of ArchConfig the two managers read."""
    layer_kinds: List[int]                      # fullAttentionLayerMask: 0 swa, 1 full, 2 linear
    num_kv_heads: int = 0
    head_dim: int = 0
    num_full_kv_heads: int = 0
    full_head_dim: int = 0
    sliding_window: int = 0
    linear_attention: LinearAttentionConfig = field(default_factory=lambda: LinearAttentionConfig(0, 0, 0, 0, 0))

    @property
    def num_layers(self) -> int:
        return len(self.layer_kinds)

    def to_c(self):
        kinds = (C.c_uint8 * len(self.layer_kinds))(*self.layer_kinds)
        la = self.linear_attention
        arch = L.Arch(len(self.layer_kinds), kinds, self.num_kv_heads, self.head_dim, self.num_full_kv_heads,
                      self.full_head_dim, self.sliding_window, la.num_k_heads, la.num_v_heads, la.key_head_dim,
                      la.value_head_dim, la.conv_kernel_size)
        arch._keepalive = kinds
        return arch

    @staticmethod
    def qwen36_35b_a3b() -> "ArchConfig":
        """Qwen3.6-35B-A3B geometry (sources/TinyTitan/Infrastructure/ModelIO/ModelTypes.swift:9-43)."""
        kinds = [FULL if (i + 1) % 4 == 0 else LINEAR for i in range(40)]
        return ArchConfig(kinds, 2, 256, 2, 256, 0, LinearAttentionConfig(16, 32, 128, 128, 4))


@dataclass
class KVView:
    buffer: int
    offset: int
    stride: int
    valid_token_count: int
    precision_bits: int
    value_bytes: int
    group_size: int
    ring_capacity: int

    @property
    def address(self) -> int:
        return self.buffer + self.offset


def _host_allocator():
    libc = C.CDLL(None)
    libc.malloc.restype = C.c_void_p
    libc.malloc.argtypes = [C.c_size_t]
    libc.free.argtypes = [C.c_void_p]
    live = {}

    def alloc(_user, n):
        p = libc.malloc(max(int(n), 1))
        live[p] = int(n)
        return p

    def release(_user, p):
        live.pop(p, None)
        libc.free(p)

    def copy(_user, dst, src, n):
        C.memmove(dst, src, n)
        return 0

    def zero(_user, dst, n):
        C.memset(dst, 0, n)
        return 0

    a = L.Allocator(None, L.ALLOC_FN(alloc), L.RELEASE_FN(release), L.COPY_FN(copy), L.ZERO_FN(zero), L.COPY_FN(copy),
                    L.COPY_FN(copy))
    a._live = live
    return a


class KVCacheManager:
    maximum_slots = 256
    initial_capacity_tokens = 8192
    quantization_group_size = 64

    def __init__(self, config: ArchConfig, max_context: int, slots: int = 1, fp16_ring_enabled: bool = False,
                 precision: int = 16, max_prefill_chunk_tokens: int = 128, allocator: Optional[str] = None):
        if max_context <= 0:
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, "maxContext must be positive")
        if not (0 < slots <= self.maximum_slots):
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, f"slots must be between 1 and {self.maximum_slots}")
        self.config, self.max_context, self.slots, self.precision = config, max_context, slots, precision
        self._allocator = _host_allocator() if allocator == "host" else None
        self._arch = config.to_c()
        err = C.c_int(0)
        self.handle = L.lib().tt_kv_cache_create(
            C.byref(self._arch), max_context, slots, precision, int(fp16_ring_enabled), max_prefill_chunk_tokens,
            C.byref(self._allocator) if self._allocator is not None else None, C.byref(err))
        if not self.handle:
            L.check(err.value or L.TT_ERR_OOM)

    def close(self):
        if getattr(self, "handle", None):
            L.lib().tt_kv_cache_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def row_layout(elements: int, precision: int):
        s, v = C.c_uint32(0), C.c_uint32(0)
        L.lib().tt_kv_row_layout(elements, precision, C.byref(s), C.byref(v))
        return s.value, v.value

    @staticmethod
    def worst_case_bytes(config: ArchConfig, max_context: int, precision: int = 16, slots: int = 1) -> int:
        arch = config.to_c()
        return int(L.lib().tt_kv_cache_worst_case_bytes(C.byref(arch), max_context, precision, slots))

    def bind_stream(self, command_buffer):
        """Row copies of reserve() are enqueued on this stream from now on instead of the legacy default stream."""
        L.check(L.lib().tt_kv_cache_bind_stream(self.handle, _stream(command_buffer)))

    def write_rows(self, layer: int, slots, positions, k_rows, v_rows, src_stride_bytes: int, command_buffer=None):
        """kSlot / vSlot for a decode batch: row i of k_rows / v_rows goes to (slots[i], positions[i]); one launch.
        slots / positions: numpy uint32 arrays (kept by the caller between steps when they do not change)."""
        L.check(L.lib().tt_kv_cache_write_rows(
            self.handle, 0 if self._allocator is not None else _stream(command_buffer), layer, slots.ctypes.data,
            positions.ctypes.data, len(slots), k_rows.data_ptr() if hasattr(k_rows, "data_ptr") else int(k_rows),
            v_rows.data_ptr() if hasattr(v_rows, "data_ptr") else int(v_rows), src_stride_bytes))

    def reserve(self, tokens: int, slot: int = 0):
        L.check(L.lib().tt_kv_cache_reserve(self.handle, tokens, slot))

    def k_slot(self, layer: int, position: int, slot: int = 0) -> int:
        p = C.c_void_p(0)
        L.check(L.lib().tt_kv_cache_k_slot(self.handle, layer, position, slot, C.byref(p)))
        return p.value or 0

    def v_slot(self, layer: int, position: int, slot: int = 0) -> int:
        p = C.c_void_p(0)
        L.check(L.lib().tt_kv_cache_v_slot(self.handle, layer, position, slot, C.byref(p)))
        return p.value or 0

    def _view(self, fn, layer, slot, valid) -> KVView:
        v = L.KVViewC()
        L.check(fn(self.handle, layer, slot, self.position(slot) if valid is None else valid, C.byref(v)))
        return KVView(v.buffer or 0, v.offset, v.stride, v.valid_token_count, v.precision_bits, v.value_bytes,
                      v.group_size, v.ring_capacity)

    def key_view(self, layer: int, slot: int = 0, valid_token_count: Optional[int] = None) -> KVView:
        return self._view(L.lib().tt_kv_cache_key_view, layer, slot, valid_token_count)

    def value_view(self, layer: int, slot: int = 0, valid_token_count: Optional[int] = None) -> KVView:
        return self._view(L.lib().tt_kv_cache_value_view, layer, slot, valid_token_count)

    def advance(self, slot: int = 0, by: int = 1):
        L.check(L.lib().tt_kv_cache_advance(self.handle, slot, by))

    def rewind(self, to: int, slot: int = 0):
        L.check(L.lib().tt_kv_cache_rewind(self.handle, slot, to))

    def reset(self, slot: Optional[int] = None):
        if slot is None:
            L.check(L.lib().tt_kv_cache_reset(self.handle))
        else:
            L.check(L.lib().tt_kv_cache_reset_slot(self.handle, slot))

    def position(self, slot: int = 0) -> int:
        if not (0 <= slot < self.slots):
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, f"slot {slot} is out of range 0..<{self.slots}")
        return int(L.lib().tt_kv_cache_position(self.handle, slot))

    def capacity(self, layer: int) -> int:
        return int(L.lib().tt_kv_cache_capacity(self.handle, layer))

    def stride(self, layer: int) -> int:
        return int(L.lib().tt_kv_cache_stride(self.handle, layer))

    def layer_kind(self, layer: int) -> int:
        return int(L.lib().tt_kv_cache_layer_kind(self.handle, layer))

    def buffer_length(self, layer: int) -> int:
        return int(L.lib().tt_kv_cache_buffer_length(self.handle, layer))

    def snapshot(self) -> bytes:
        """Slot 0's K/V prefix at its cursor (KVCacheManager+Snapshot.swift:38-65)."""
        n = int(L.lib().tt_kv_cache_snapshot_bytes(self.handle, self.position(0)))
        buf = C.create_string_buffer(max(n, 1))
        out = C.c_size_t(0)
        L.check(L.lib().tt_kv_cache_snapshot_export(self.handle, buf, n, C.byref(out)))
        return buf.raw[:out.value]

    def restore_snapshot(self, position: int, payload: bytes):
        """restoreSnapshot (KVCacheManager+Snapshot.swift:67-121)."""
        L.check(L.lib().tt_kv_cache_snapshot_restore(self.handle, position, payload, len(payload)))


class GDNStateManager:
    maximum_slots = KVCacheManager.maximum_slots

    def __init__(self, config: ArchConfig, slots: int = 1, enable_speculative_checkpoint: bool = False,
                 allocator: Optional[str] = None):
        if not (0 < slots <= self.maximum_slots):
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, f"slots must be between 1 and {self.maximum_slots}")
        self.config, self.slots = config, slots
        self._allocator = _host_allocator() if allocator == "host" else None
        self._arch = config.to_c()
        err = C.c_int(0)
        self.handle = L.lib().tt_gdn_state_create(
            C.byref(self._arch), slots, int(enable_speculative_checkpoint),
            C.byref(self._allocator) if self._allocator is not None else None, C.byref(err))
        if not self.handle:
            L.check(err.value or L.TT_ERR_OOM)

    def close(self):
        if getattr(self, "handle", None):
            L.lib().tt_gdn_state_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def worst_case_bytes(config: ArchConfig, slots: int = 1) -> int:
        arch = config.to_c()
        return int(L.lib().tt_gdn_state_worst_case_bytes(C.byref(arch), slots))

    @property
    def state_bytes_per_layer(self) -> int:
        return int(L.lib().tt_gdn_state_bytes_per_layer(self.handle))

    @property
    def conv_tail_bytes_per_layer(self) -> int:
        return int(L.lib().tt_gdn_state_conv_tail_bytes_per_layer(self.handle))

    def is_linear(self, layer: int) -> bool:
        return bool(L.lib().tt_gdn_state_is_linear(self.handle, layer))

    def _slot(self, fn, layer, slot) -> int:
        p = C.c_void_p(0)
        L.check(fn(self.handle, layer, slot, C.byref(p)))
        return p.value or 0

    def state_slot(self, layer: int, slot: int = 0) -> int:
        return self._slot(L.lib().tt_gdn_state_state_slot, layer, slot)

    def conv_tail_slot(self, layer: int, slot: int = 0) -> int:
        return self._slot(L.lib().tt_gdn_state_conv_tail_slot, layer, slot)

    def speculative_state_slot(self, layer: int, slot: int = 0) -> int:
        return self._slot(L.lib().tt_gdn_state_speculative_state_slot, layer, slot)

    def reset(self, slot: Optional[int] = None):
        if slot is None:
            L.check(L.lib().tt_gdn_state_reset(self.handle))
        else:
            L.check(L.lib().tt_gdn_state_reset_slot(self.handle, slot))

    def speculative_restore(self, command_buffer=None):
        """encodeSpeculativeRestore(commandBuffer:): enqueued on the verify pass's stream."""
        stream = 0 if self._allocator is not None else _stream(command_buffer)   # host-backed: no stream
        L.check(L.lib().tt_gdn_state_speculative_restore(self.handle, stream))

    def bind_stream(self, command_buffer):
        """Zero fills (reset) are enqueued on this stream from now on instead of the legacy default stream."""
        L.check(L.lib().tt_gdn_state_bind_stream(self.handle, _stream(command_buffer)))

    def snapshot(self) -> bytes:
        """[state, conv tail] of slot 0 for every linear layer (GDNStateManager.swift:228-261)."""
        n = int(L.lib().tt_gdn_state_snapshot_bytes(self.handle))
        buf = C.create_string_buffer(max(n, 1))
        out = C.c_size_t(0)
        L.check(L.lib().tt_gdn_state_snapshot_export(self.handle, buf, n, C.byref(out)))
        return buf.raw[:out.value]

    def restore_snapshot(self, payload: bytes):
        L.check(L.lib().tt_gdn_state_snapshot_restore(self.handle, payload, len(payload)))


class KVWindow:
    """Host-KV streaming tier of KVCacheManager (KVCacheManager+HostStreaming.swift,
    +HostStreamingPrefill.swift) for `layers` streamed layers: host arena + device window + the
    (logical key, window row) lists attention reads. numpy uint32 arrays cross the boundary."""

    def __init__(self, layers: int, stride_bytes: int, max_context: int, window_tokens: int, slots: int = 1,
                 allocator: Optional[str] = None):
        self._allocator = _host_allocator() if allocator == "host" else None
        err = C.c_int(0)
        self.handle = L.lib().tt_kv_window_create(
            layers, stride_bytes, max_context, slots, window_tokens,
            C.byref(self._allocator) if self._allocator is not None else None, C.byref(err))
        if not self.handle:
            L.check(err.value or L.TT_ERR_OOM)
        self.stride, self.max_context, self.slots = stride_bytes, max_context, slots
        self.window_tokens = int(L.lib().tt_kv_window_tokens(self.handle))

    def close(self):
        if getattr(self, "handle", None):
            L.lib().tt_kv_window_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def window_bytes(self) -> int:
        return int(L.lib().tt_kv_window_bytes(self.handle))

    @property
    def host_arena_bytes(self) -> int:
        return int(L.lib().tt_kv_window_host_arena_bytes(self.handle))

    def streaming_prefill_chunk_tokens(self, configured: int, selection_width: int) -> int:
        return int(L.lib().tt_kv_window_prefill_chunk_tokens(self.handle, configured, selection_width))

    def base(self, layer: int, slot: int = 0):
        k, v = C.c_void_p(), C.c_void_p()
        L.check(L.lib().tt_kv_window_base(self.handle, layer, slot, C.byref(k), C.byref(v)))
        return k.value, v.value

    def write_slot(self, layer: int, position: int, slot: int = 0):
        """kSlot / vSlot of a streamed layer: addresses the projection writes this position's row to."""
        k, v = C.c_void_p(), C.c_void_p()
        L.check(L.lib().tt_kv_window_write_slot(self.handle, layer, position, slot, C.byref(k), C.byref(v)))
        return k.value, v.value

    def window_row(self, layer: int, position: int, slot: int = 0):
        row = C.c_int64(-1)
        L.check(L.lib().tt_kv_window_row_of(self.handle, layer, slot, position, C.byref(row)))
        return None if row.value < 0 else int(row.value)

    def prepare_decode_window(self, layer: int, position: int, indices=None, count: Optional[int] = None, slot: int = 0):
        """prepareDecodeWindow: (indices, rows) uint32 arrays of the step's selection."""
        import numpy as np
        if indices is not None:
            indices = np.ascontiguousarray(indices, dtype=np.uint32)
            count = len(indices) if count is None else count
        out_i, out_r = np.empty(count, np.uint32), np.empty(count, np.uint32)
        L.check(L.lib().tt_kv_window_prepare_decode(
            self.handle, layer, slot, position, indices.ctypes.data if indices is not None else None, count,
            out_i.ctypes.data, out_r.ctypes.data))
        return out_i, out_r

    def begin_prefill_write(self, layer: int, start_position: int, token_count: int, slot: int = 0):
        k, v = C.c_void_p(), C.c_void_p()
        L.check(L.lib().tt_kv_window_begin_prefill(self.handle, layer, slot, start_position, token_count, C.byref(k), C.byref(v)))
        return k.value, v.value

    def prepare_prefill_window(self, layer: int, start_position: int, token_count: int, indices=None, counts=None,
                               slot: int = 0):
        """preparePrefillWindow: (indices, rows, counts) with the [token, index_stride] layout of the selection."""
        import numpy as np
        if indices is not None:
            indices = np.ascontiguousarray(indices, dtype=np.uint32)
            counts = np.ascontiguousarray(counts, dtype=np.uint32)
            stride = indices.shape[1]
        else:
            stride = start_position + token_count
        out_i = np.zeros((token_count, stride), np.uint32); out_r = np.zeros((token_count, stride), np.uint32)
        out_c = np.zeros(token_count, np.uint32)
        L.check(L.lib().tt_kv_window_prepare_prefill(
            self.handle, layer, slot, start_position, token_count, indices.ctypes.data if indices is not None else None,
            stride if indices is not None else 0, counts.ctypes.data if indices is not None else None,
            out_i.ctypes.data, out_r.ctypes.data, out_c.ctypes.data, stride))
        return out_i, out_r, out_c

    def commit(self, position: int, count: int = 1, slot: int = 0):
        L.check(L.lib().tt_kv_window_commit(self.handle, slot, position, count))

    def reset_slot(self, slot: int = 0):
        L.check(L.lib().tt_kv_window_reset_slot(self.handle, slot))

    def host_row(self, layer: int, position: int, key: bool = True, slot: int = 0) -> bytes:
        buf = C.create_string_buffer(self.stride)
        L.check(L.lib().tt_kv_window_host_row(self.handle, layer, slot, position, int(key), buf))
        return buf.raw

    def counters(self):
        e, r, b = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
        L.lib().tt_kv_window_counters(self.handle, C.byref(e), C.byref(r), C.byref(b))
        return {"evictions": e.value, "row_copies": r.value, "copy_bytes": b.value}
