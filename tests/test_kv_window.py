"""Host-KV streaming tier on host memory (no GPU): the bookkeeping of
KVCacheManager+HostStreaming.swift / +HostStreamingPrefill.swift, checked the way the reference's
tests/TinyTitan/Runtime/KVCache/HostKVStreamingTests.swift checks it -- rows written through the
window reach the arena intact however often the window is recycled, a step's copies are bounded
by its selection, the device cost is the window."""
import ctypes as C

import numpy as np
import pytest

import tinytitan_b200 as tt
from tinytitan_b200 import _lib as L

STRIDE = 64


def row_bytes(position, seed, key=True):
    """Finite fp16 rows that differ per position (HostKVStreamingTests.swift:84-99)."""
    i = np.arange(STRIDE // 2)
    phase = (seed * 31 + i * 7 + position * 3) * 0.001
    return ((np.sin(phase) if key else np.cos(phase)) * 0.25).astype(np.float16).tobytes()


def write(w, layer, position, seed, slot=0):
    k, v = w.write_slot(layer, position, slot)
    C.memmove(k, row_bytes(position, seed, True), STRIDE)
    C.memmove(v, row_bytes(position, seed, False), STRIDE)


def window_bytes_at(w, layer, row, key=True, slot=0):
    k, v = w.base(layer, slot)
    return C.string_at((k if key else v) + row * STRIDE, STRIDE)


def test_rows_reach_the_arena_across_thousands_of_evictions():
    # :243-330: a 64-row window over a long context; every row written is read back from the arena
    w = tt.KVWindow(2, STRIDE, max_context=5000, window_tokens=64, allocator="host")
    assert w.window_tokens == 64
    assert w.window_bytes == 2 * 2 * 64 * STRIDE and w.host_arena_bytes == 2 * 2 * 5000 * STRIDE   # :332-375
    for position in range(5000):
        for layer in range(2):
            write(w, layer, position, seed=5 + layer)
        w.commit(position, 1)
    for position in (0, 63, 64, 65, 4096, 4999):
        for layer in range(2):
            assert w.host_row(layer, position, True) == row_bytes(position, 5 + layer, True)
            assert w.host_row(layer, position, False) == row_bytes(position, 5 + layer, False)
    assert w.counters()["evictions"] >= 2 * (5000 - 64)
    w.close()


def test_decode_window_gathers_the_selection_and_only_the_selection():
    w = tt.KVWindow(1, STRIDE, max_context=3000, window_tokens=32, allocator="host")
    for position in range(2000):
        write(w, 0, position, seed=9)
        w.commit(position, 1)
    position = 2000
    write(w, 0, position, seed=9)                       # this step's token: pinned, must survive the gather
    keys = np.array(sorted({0, 8, 512, 1024, 1500} | set(range(position - 7, position + 1))), np.uint32)
    before = w.counters()
    idx, rows = w.prepare_decode_window(0, position, keys)
    after = w.counters()
    assert np.array_equal(idx, keys) and len(set(rows.tolist())) == len(keys)
    for key, row in zip(idx, rows):
        assert window_bytes_at(w, 0, int(row), True) == row_bytes(int(key), 9, True)
        assert window_bytes_at(w, 0, int(row), False) == row_bytes(int(key), 9, False)
    # copies are bounded by the selection, not by the context (:377-440)
    assert after["row_copies"] - before["row_copies"] <= len(keys)
    assert after["copy_bytes"] - before["copy_bytes"] <= len(keys) * 2 * STRIDE
    # the same selection again costs nothing: every row is resident
    idx2, rows2 = w.prepare_decode_window(0, position, keys)
    assert w.counters()["row_copies"] == after["row_copies"] and np.array_equal(rows, rows2)
    w.commit(position, 1)
    assert w.host_row(0, position) == row_bytes(position, 9)
    # dense path: indices None means keys 0..count-1, which must fit the window
    with pytest.raises(tt.TinyTitanError):
        w.prepare_decode_window(0, position, None, count=33)
    with pytest.raises(tt.InvalidArgument):
        w.prepare_decode_window(0, 10, np.array([11], np.uint32))          # a key past the current position
    w.close()


def test_short_context_allocation_order_is_logical_order():
    # :186-241: with no eviction window row == logical position, so the windowed read is the dense read
    w = tt.KVWindow(1, STRIDE, max_context=128, window_tokens=128, allocator="host")
    for position in range(128):
        write(w, 0, position, seed=11)
        w.commit(position, 1)
    idx, rows = w.prepare_decode_window(0, 127, None, count=128)
    assert np.array_equal(idx, np.arange(128)) and np.array_equal(rows, np.arange(128))
    assert w.counters()["evictions"] == 0
    w.close()


def test_prefill_staging_union_and_indirection():
    w = tt.KVWindow(1, STRIDE, max_context=400, window_tokens=48, slots=2, allocator="host")
    slot = 1
    for position in range(200):
        write(w, 0, position, seed=3, slot=slot)
        w.commit(position, 1, slot=slot)
    start, tokens = 200, 6
    sk, sv = w.begin_prefill_write(0, start, tokens, slot=slot)
    for t in range(tokens):                                              # the chunk's projection writes staging rows
        k, v = w.write_slot(0, start + t, slot)
        assert k == sk + t * STRIDE and v == sv + t * STRIDE
        C.memmove(k, row_bytes(start + t, 3, True), STRIDE); C.memmove(v, row_bytes(start + t, 3, False), STRIDE)
    stride = 10
    sel = np.zeros((tokens, stride), np.uint32); cnt = np.zeros(tokens, np.uint32)
    for t in range(tokens):
        keys = sorted({0, 17, 100 + t, 150} | set(range(start + t - 3, start + t + 1)))
        sel[t, :len(keys)] = keys; cnt[t] = len(keys)
    idx, rows, counts = w.prepare_prefill_window(0, start, tokens, sel, cnt, slot=slot)
    assert np.array_equal(counts, cnt)
    for t in range(tokens):
        for i in range(cnt[t]):
            assert idx[t, i] == sel[t, i]
            assert window_bytes_at(w, 0, int(rows[t, i]), True, slot) == row_bytes(int(sel[t, i]), 3, True)
            assert window_bytes_at(w, 0, int(rows[t, i]), False, slot) == row_bytes(int(sel[t, i]), 3, False)
    # the same logical key maps to the same window row in every query row
    assert rows[0, 0] == rows[5, 0]
    w.commit(start, tokens, slot=slot)                                    # staged rows reach the arena in one copy
    for t in range(tokens):
        assert w.host_row(0, start + t, True, slot) == row_bytes(start + t, 3, True)
    # a union larger than the window is refused
    wide = np.arange(60, dtype=np.uint32)[None].repeat(2, 0)
    with pytest.raises(tt.TinyTitanError):
        w.prepare_prefill_window(0, 206, 2, wide, np.array([60, 60], np.uint32), slot=slot)
    # slot 0 was never touched
    assert w.window_row(0, 5, slot=0) is None
    w.reset_slot(slot)
    assert w.window_row(0, 150, slot=slot) is None
    assert w.streaming_prefill_chunk_tokens(128, 2051) == 1 and w.streaming_prefill_chunk_tokens(8, 4) == 8
    w.close()
