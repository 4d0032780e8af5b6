"""Host-side logic and the C ABI surface, without a GPU."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import tinytitan_b200 as tt
from tinytitan_b200 import _lib as L
from tinytitan_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "tinytitan_cuda.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(tt_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 45
    handle = ctypes.CDLL(L.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} is declared but not exported"
    assert declared == set(L.SIGNATURES), declared ^ set(L.SIGNATURES)


def test_header_is_strict_c99():
    # the reference's own flag set for its C target (Package.swift:108-118)
    src = '#include "tinytitan_cuda.h"\nint main(void) { tt_prefill_params p; (void)p; return (int)TT_OK; }\n'
    r = subprocess.run(["gcc", "-std=c99", "-pedantic-errors", "-Wall", "-Wextra", "-Werror", "-fsyntax-only",
                        "-I", os.path.join(ROOT, "include"), "-x", "c", "-"], input=src.encode(), capture_output=True)
    assert r.returncode == 0, r.stderr.decode()


def test_reference_split_geometry_numbers():
    # tests/TinyTitan/Kernels/Attention/AttentionTests.swift:27-51
    g = tt.Attention.split_geometry(16, 2, 1536, 0, False)
    assert (g.num_chunks, g.chunk_length, g.partial_threadgroups) == (16, 96, 256)
    g = tt.Attention.split_geometry(16, 2, 5, 0, False)
    assert (g.num_chunks, g.chunk_length) == (5, 1)
    g = tt.Attention.split_geometry(4, 2, 1024, 0, True)       # q_per_kv 2 -> grouped SWA partial
    assert g.use_swa_grouped_partial and g.num_chunks == 16 and g.partial_threadgroups == 2 * 16
    g = tt.Attention.split_geometry(16, 2, 1024, 512, True)    # q_per_kv 8 -> per-q-head split
    assert not g.use_swa_grouped_partial and g.effective_length == 512 and g.num_chunks == 16


def _plan(keys, rows, hd=256, hq=16, hkv=2, sms=148, ws=192 << 20):
    n = len(keys)
    k = (ctypes.c_uint32 * n)(*keys); r = (ctypes.c_uint32 * n)(*rows)
    per, items = ctypes.c_uint32(0), ctypes.c_uint32(0)
    rc = L.lib().tt_attn_plan_splits(k, r, n, hd, hq, hkv, sms, ws, ctypes.byref(per), ctypes.byref(items))
    return rc, per.value, items.value


def test_split_planner():
    rng = np.random.default_rng(0)
    keys = [int(x) for x in rng.integers(1024, 32769, size=32)]
    rc, per, items = _plan(keys, [1] * 32)
    assert rc == 0 and per % 16 == 0 and 64 <= per <= 16384
    # an item serves a PAIR of adjacent KV heads when the head count is even (whole cache rows are streamed)
    assert items == sum(-(-k // per) for k in keys)
    # 32 streams on 148 SMs x 2 resident CTAs: the items fill ONE wave as tightly as the ragged lengths allow,
    # and a shorter item length would spill into a second, mostly empty wave
    assert 0.9 * 296 <= items <= 296
    assert sum(-(-k // (per - 16)) for k in keys) > 296
    # a single short session is not split below the minimum item length
    rc, per, items = _plan([4096], [1], hq=8)
    assert rc == 0 and per == 64 and items == 64
    # an odd head count keeps one head per item
    rc, per, items = _plan([4096], [1], hq=9, hkv=3)
    assert rc == 0 and items == 3 * (-(-4096 // per))
    # an empty range still yields one (empty) item per KV head pair
    rc, per, items = _plan([0], [1])
    assert rc == 0 and items == 1
    # 64 packed rows (4 draft rows x group 16) -> 4 row tiles per KV head pair; 256 streams take three waves
    rc, per, items = _plan([16384] * 64, [4] * 64, hq=32)
    assert rc == 0 and items == 64 * 4 * (-(-16384 // per)) and 2 * 296 < items <= 3 * 296
    # one long session: exactly one wave
    rc, per, items = _plan([262144], [1])
    assert rc == 0 and 0.95 * 296 <= items <= 296
    # workspace too small for even one part per session -> OOM status, never a silent truncation
    rc, _, _ = _plan([100000] * 8, [1] * 8, ws=1024)
    assert rc == L.TT_ERR_OOM


def _plan_verify(keys, rows, hd=256, hq=32, hkv=2, sms=148, ws=192 << 20):
    n = len(keys)
    k = (ctypes.c_uint32 * n)(*keys); r = (ctypes.c_uint32 * n)(*rows)
    parts, lens = (ctypes.c_uint32 * n)(), (ctypes.c_uint32 * n)()
    items = ctypes.c_uint32(0)
    rc = L.lib().tt_attn_plan_verify_splits(k, r, n, hd, hq, hkv, sms, ws, parts, lens, ctypes.byref(items))
    return rc, list(parts), list(lens), items.value


def test_verify_split_planner():
    # config 5 on one GPU: 64 sessions x 2 kv heads = 128 streams for 148 SMs: one item per stream
    # (a second wave of half-length items would not finish sooner)
    rc, parts, lens, items = _plan_verify([16387] * 64, [4] * 64)
    assert rc == 0 and parts == [1] * 64 and lens == [16512] * 64 and items == 128
    # its per-GPU share on 8 GPUs: 16 streams are cut so that one wave fills the SMs
    rc, parts, lens, items = _plan_verify([16387] * 8, [4] * 8)
    assert rc == 0 and len(set(parts)) == 1 and 100 <= items <= 148
    # ragged batch: equal parts inside a session, tile multiples, every key covered exactly once
    rng = np.random.default_rng(1)
    keys = [int(x) for x in rng.integers(1, 40000, size=23)] + [0]
    rc, parts, lens, items = _plan_verify(keys, [4] * 24)
    assert rc == 0 and items == 2 * sum(parts)
    for k, p, l in zip(keys, parts, lens):
        assert p >= 1 and l % 128 == 0 and p * l >= k and (p - 1) * l < max(k, 1)
        assert l >= 128 or k == 0
    # short contexts stay one part (the pass then stores the outputs itself)
    rc, parts, lens, items = _plan_verify([500, 300, 4, 129], [4] * 4)
    assert rc == 0 and parts == [1, 1, 1, 1]
    # partials that cannot fit the workspace are refused, not truncated
    rc, _, _, _ = _plan_verify([100000] * 8, [4] * 8, ws=1024)
    assert rc == L.TT_ERR_OOM


def test_exchange_buffer_size_is_pure_arithmetic():
    # two parities of [world][heads][64-column blocks] cells; a cell is 66 values (64 columns, max, sum), each
    # travelling as 8 bytes {value, epoch}: 33 words of 16 bytes; each parity padded to 256 bytes
    cells = 8 * 16 * 4
    assert L.lib().tt_attn_exchange_bytes(8, 16, 256) == 2 * ((cells * 33 * 16 + 255) // 256 * 256)
    assert L.lib().tt_attn_exchange_bytes(2, 16, 256) < L.lib().tt_attn_exchange_bytes(4, 16, 256)
    assert L.lib().tt_attn_exchange_bytes(2, 8, 64) % 512 == 0


def test_context_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(tt.TinyTitanError):
        tt.Context(0)


def test_kv_row_layout_pins():
    # tests/TinyTitan/Kernels/Attention/KVCacheQuantizedAttentionTests.swift:86-101 (2 heads x 256)
    assert tt.KVCacheManager.row_layout(512, 16) == (1024, 1024)
    assert tt.KVCacheManager.row_layout(512, 8) == (544, 512)
    assert tt.KVCacheManager.row_layout(512, 4) == (288, 256)
    assert tt.KVCacheManager.row_layout(65, 4) == (34 + 2 * 4, 34)


def _read(ptr, n):
    return bytes((ctypes.c_ubyte * n).from_address(ptr))


def _write(ptr, data: bytes):
    ctypes.memmove(ptr, data, len(data))


def test_kv_cache_manager_bookkeeping_on_host_memory():
    # KVCacheManagerTests / KVCacheGrowthTests (tests/TinyTitan/Runtime/KVCache): strides, disjoint
    # linear slot regions, independent cursors, doubling growth that keeps every slot's rows,
    # rewind moves only the cursor, per-slot reset.
    cfg = tt.ArchConfig.qwen36_35b_a3b()
    kv = tt.KVCacheManager(cfg, max_context=40000, slots=3, allocator="host")
    full = [i for i, k in enumerate(cfg.layer_kinds) if k == tt.FULL]
    assert len(full) == 10 and kv.layer_kind(0) == tt.LINEAR and kv.stride(0) == 0
    layer = full[0]
    assert kv.stride(layer) == 1024 and kv.capacity(layer) == 8192
    assert kv.buffer_length(layer) == 3 * 8192 * 1024
    base = kv.key_view(layer, 0).buffer
    assert kv.k_slot(layer, 0, 1) - base == 8192 * 1024              # slot regions are linear in the slot
    assert kv.k_slot(layer, 5, 2) - base == (2 * 8192 + 5) * 1024
    assert kv.v_slot(layer, 0, 0) != kv.k_slot(layer, 0, 0)           # K and V never alias
    with pytest.raises(tt.InvalidArgument):
        kv.k_slot(0, 0, 0)                                            # linear layers have no KV slots
    with pytest.raises(tt.InvalidArgument):
        kv.k_slot(layer, 8192, 0)                                     # beyond capacity: reserve first
    with pytest.raises(tt.InvalidArgument):
        kv.k_slot(layer, 0, 3)
    rows = {0: b"\x11" * 1024, 1: b"\x22" * 1024, 2: b"\x33" * 1024}
    for slot, n in ((0, 3), (1, 8192), (2, 1)):
        _write(kv.k_slot(layer, n - 1, slot), rows[slot]); _write(kv.v_slot(layer, n - 1, slot), rows[slot][::-1])
        kv.advance(slot, n)
    assert [kv.position(s) for s in range(3)] == [3, 8192, 1]
    kv.reserve(8193, slot=1)
    assert kv.capacity(layer) == 16384 and kv.capacity(full[-1]) == 16384
    for slot, n in ((0, 3), (1, 8192), (2, 1)):
        assert _read(kv.k_slot(layer, n - 1, slot), 1024) == rows[slot]
        view = kv.key_view(layer, slot)
        assert view.offset == slot * 16384 * 1024 and view.valid_token_count == n and view.stride == 1024
    kv.reserve(10 ** 9, slot=0)                                       # clamped to maxContext
    assert kv.capacity(layer) == 40000
    kv.rewind(2, slot=0)
    assert kv.position(0) == 2 and _read(kv.k_slot(layer, 2, 0), 1024) == rows[0]   # rows stay
    with pytest.raises(tt.InvalidArgument):
        kv.rewind(5, slot=0)
    kv.reset(slot=1)
    assert [kv.position(s) for s in range(3)] == [2, 0, 1]
    kv.reset()
    assert [kv.position(s) for s in range(3)] == [0, 0, 0]
    with pytest.raises(tt.InvalidArgument):
        kv.advance(0, 40001)
    assert tt.KVCacheManager.worst_case_bytes(cfg, 32768, 16, 32) == 10 * 2 * 32 * 32768 * 1024
    kv.close()
    with pytest.raises(tt.InvalidArgument):
        tt.KVCacheManager(cfg, 1024, slots=257, allocator="host")


def test_kv_cache_ring_and_quantised_strides():
    cfg = tt.ArchConfig([tt.SWA, tt.FULL], 8, 256, 2, 512, sliding_window=1024)
    kv = tt.KVCacheManager(cfg, max_context=100000, fp16_ring_enabled=True, max_prefill_chunk_tokens=128,
                           allocator="host")
    assert kv.capacity(0) == 1024 + 128 and kv.capacity(1) == 8192
    assert kv.key_view(0, 0, 10).ring_capacity == 1152 and kv.key_view(1, 0, 10).ring_capacity == 0
    base = kv.key_view(0).buffer
    assert kv.k_slot(0, 1152 + 7, 0) - base == 7 * kv.stride(0)       # physicalSlot = position % capacity
    kv.reserve(20000)
    assert kv.capacity(0) == 1152 and kv.capacity(1) == 32768         # rings never grow
    kv.close()
    kv8 = tt.KVCacheManager(cfg, 4096, precision=8, allocator="host")
    assert kv8.stride(1) == tt.KVCacheManager.row_layout(2 * 512, 8)[0] == 1024 + 16 * 4
    assert kv8.key_view(1, 0, 0).value_bytes == 1024
    kv8.close()


def test_gdn_state_manager_on_host_memory():
    # GDNStateManagerTests (tests/TinyTitan/Runtime/KVCache/GDNStateManagerTests.swift:29-95)
    cfg = tt.ArchConfig.qwen36_35b_a3b()
    g = tt.GDNStateManager(cfg, slots=3, enable_speculative_checkpoint=True, allocator="host")
    assert g.state_bytes_per_layer == 32 * 128 * 128 * 4 == 2 << 20
    assert g.conv_tail_bytes_per_layer == 3 * 8192 * 2 == 49152
    assert g.is_linear(0) and not g.is_linear(3)
    with pytest.raises(tt.InvalidArgument):
        g.state_slot(3, 0)
    with pytest.raises(tt.InvalidArgument):
        g.state_slot(0, 3)
    s0, s2 = g.state_slot(0, 0), g.state_slot(0, 2)
    assert s2 - s0 == 2 * g.state_bytes_per_layer
    assert g.conv_tail_slot(0, 1) - g.conv_tail_slot(0, 0) == g.conv_tail_bytes_per_layer
    assert _read(s0, 4096) == b"\0" * 4096                            # the empty state is all zeros
    _write(s0, b"\x7f" * 64); _write(s2, b"\x55" * 64)
    g.reset(slot=0)
    assert _read(s0, 64) == b"\0" * 64 and _read(s2, 64) == b"\x55" * 64
    _write(g.speculative_state_slot(0, 0), b"\x42" * 64)
    g.speculative_restore()
    assert _read(s0, 64) == b"\x42" * 64 and _read(s2, 64) == b"\x55" * 64
    g.reset()
    assert _read(s2, 64) == b"\0" * 64
    assert tt.GDNStateManager.worst_case_bytes(cfg, 2) == 2 * 30 * ((2 << 20) + 49152)
    g.close()
    g2 = tt.GDNStateManager(cfg, slots=1, allocator="host")
    with pytest.raises(tt.InvalidArgument):
        g2.speculative_restore()                                      # no checkpoint twins: invalid layout
    g2.close()


def test_session_sharding_and_kv_ranges():
    rng = np.random.default_rng(1)
    lens = [int(x) for x in rng.integers(1024, 32769, size=32)]
    for world in (1, 2, 4, 8):
        shards = sharding.shard_sessions(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(32))
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)                   # greedy balance bound
        rr = sharding.shard_sessions(lens, world, "round_robin")
        assert all(i % world == r for r, s in enumerate(rr) for i in s)
    for world in (1, 2, 4, 8, 3):
        ranges = sharding.kv_split_ranges(262144, world)
        assert ranges[0][0] == 0 and ranges[-1][1] == 262144
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    assert sharding.kv_split_ranges(3, 8)[4:] == [(3, 3)] * 4             # empty trailing ranks
    assert sharding.kv_split_ranges(10, 2, kv_start=4) == [(4, 7), (7, 10)]


def test_snapshot_round_trip_on_host_memory():
    # KVCacheManager+Snapshot.swift:12-121 and GDNStateManager.swift:228-344: slot 0's prefix, per layer K then
    # V; restore grows the receiver first; a payload of another size is refused.
    cfg = tt.ArchConfig([tt.LINEAR, tt.FULL, tt.LINEAR, tt.FULL], 2, 64, 2, 64, 0, tt.LinearAttentionConfig(2, 4, 32, 32, 4))
    a = tt.KVCacheManager(cfg, max_context=20000, slots=2, allocator="host")
    n = 9000
    a.reserve(n)
    stride = a.stride(1)
    rng = np.random.default_rng(0)
    blobs = {}
    for layer in (1, 3):
        for name, fn in (("k", a.k_slot), ("v", a.v_slot)):
            data = rng.integers(0, 256, size=n * stride, dtype=np.uint8).tobytes()
            _write(fn(layer, 0, 0), data)
            blobs[(layer, name)] = data
    a.advance(0, n)
    payload = a.snapshot()
    assert len(payload) == 2 * 2 * n * stride
    assert payload[:n * stride] == blobs[(1, "k")] and payload[n * stride:2 * n * stride] == blobs[(1, "v")]
    b = tt.KVCacheManager(cfg, max_context=20000, slots=2, allocator="host")     # fresh receiver at capacity 8192
    b.advance(1, 5)
    b.restore_snapshot(n, payload)
    assert b.capacity(1) == 16384 and b.position(0) == n and b.position(1) == 0
    assert _read(b.v_slot(3, 0, 0), n * stride) == blobs[(3, "v")]
    with pytest.raises(tt.InvalidArgument):
        b.restore_snapshot(n, payload[:-1])
    with pytest.raises(tt.InvalidArgument):
        b.restore_snapshot(0, payload)
    g = tt.GDNStateManager(cfg, slots=2, allocator="host")
    _write(g.state_slot(0, 0), b"\x21" * 100); _write(g.conv_tail_slot(2, 0), b"\x43" * 50); _write(g.state_slot(0, 1), b"\x99" * 8)
    snap = g.snapshot()
    assert len(snap) == 2 * (g.state_bytes_per_layer + g.conv_tail_bytes_per_layer)
    g2 = tt.GDNStateManager(cfg, slots=2, allocator="host")
    _write(g2.state_slot(2, 1), b"\x77" * 8)
    g2.restore_snapshot(snap)
    assert _read(g2.state_slot(0, 0), 100) == b"\x21" * 100 and _read(g2.conv_tail_slot(2, 0), 50) == b"\x43" * 50
    assert _read(g2.state_slot(2, 1), 8) == b"\0" * 8                            # restore resets everything first
    with pytest.raises(tt.InvalidArgument):
        g2.restore_snapshot(snap + b"x")
    for m in (a, b, g, g2):
        m.close()


def test_kv_cache_write_rows_on_host_memory():
    # the batched kSlot / vSlot write: row i lands at (slots[i], positions[i]), other rows untouched
    import numpy as np
    cfg = tt.ArchConfig([tt.FULL], 2, 256, 2, 256, 0, tt.LinearAttentionConfig(16, 32, 128, 128, 4))
    kv = tt.KVCacheManager(cfg, max_context=100, slots=4, allocator="host")
    stride = kv.stride(0)
    src_stride = stride + 32
    n = 3
    ksrc = (ctypes.c_ubyte * (n * src_stride))(*([0] * (n * src_stride))); vsrc = (ctypes.c_ubyte * (n * src_stride))()
    for i in range(n):
        ctypes.memset(ctypes.addressof(ksrc) + i * src_stride, 0x10 + i, stride)
        ctypes.memset(ctypes.addressof(vsrc) + i * src_stride, 0x20 + i, stride)
    slots = np.array([3, 0, 2], np.uint32); positions = np.array([7, 99, 0], np.uint32)
    kv.write_rows(0, slots, positions, ctypes.addressof(ksrc), ctypes.addressof(vsrc), src_stride)
    for i in range(n):
        assert _read(kv.k_slot(0, int(positions[i]), int(slots[i])), stride) == bytes([0x10 + i]) * stride
        assert _read(kv.v_slot(0, int(positions[i]), int(slots[i])), stride) == bytes([0x20 + i]) * stride
    assert kv.position(3) == 0                                        # cursors do not move
    with pytest.raises(tt.InvalidArgument):
        kv.write_rows(0, np.array([4], np.uint32), np.array([0], np.uint32), ctypes.addressof(ksrc), ctypes.addressof(vsrc), src_stride)
    with pytest.raises(tt.InvalidArgument):
        kv.write_rows(0, np.array([0], np.uint32), np.array([100], np.uint32), ctypes.addressof(ksrc), ctypes.addressof(vsrc), src_stride)
    kv.close()
