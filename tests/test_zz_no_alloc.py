"""The allocation-free decode entry point against the regular one and the oracle (B200 only).

tt_attn_decode_noalloc exists for callers that may not allocate device memory at the moment
they need attention (no cudaMalloc allowed where they run, or no memory budget left): it takes
no context and keeps its split-KV scratch in a fixed array inside the library. This file is
collected last on purpose, so a run that stops at the first failure has already exercised
everything else. It must pass alone in a fresh process and after the other tests: the first
call on the device does the one-time address lookup either way.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from tinytitan_b200 import _lib as L

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _case(hq, hkv, hd, s, seed):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    q = torch.randn(hq, hd, device="cuda", generator=g).half()
    k = torch.randn(s, hkv, hd, device="cuda", generator=g).half()
    v = torch.randn(s, hkv, hd, device="cuda", generator=g).half()
    want = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    got = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    return q, k, v, want, got


def _both(ctx, hq, hkv, hd, s, kv_start, seed):
    q, k, v, want, got = _case(hq, hkv, hd, s, seed)
    stream = torch.cuda.current_stream().cuda_stream
    ctx.check(L.lib().tt_attn_decode(ctx.handle, stream, _ptr(q), _ptr(k), _ptr(v), _ptr(want), hd, hq, hkv, s,
                                     kv_start, 0.0625, None, None, 0))
    rc = L.lib().tt_attn_decode_noalloc(stream, _ptr(q), _ptr(k), _ptr(v), _ptr(got), hd, hq, hkv, s, kv_start, 0.0625)
    assert rc == L.TT_OK
    flags = C.c_uint32(0xFFFF)
    assert L.lib().tt_attn_decode_noalloc_status(stream, C.byref(flags)) == L.TT_OK and flags.value == 0
    torch.cuda.synchronize()
    ref = np.zeros((hq, hd), np.float32)
    if s > kv_start:
        f = lambda t: t.float().cpu().numpy()
        ref = oracle.attn_decode(f(q), f(k)[kv_start:], f(v)[kv_start:], hkv, 0.0625)
    return got.float().cpu().numpy(), want.float().cpu().numpy(), ref


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    ctx = tt.Context(0)
    # two calls back to back with different inputs and split counts: the second must not see
    # anything the first left in the shared scratch
    for seed, (hq, hkv, hd, s, kv_start) in enumerate([(16, 2, 256, 9000, 0), (8, 2, 256, 4096, 100)]):
        got, want, ref = _both(ctx, hq, hkv, hd, s, kv_start, seed)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 2e-3      # the suite's fp16 bar; the two planners may split differently
        assert np.abs(got - ref).max() <= 2e-3       # and the CPU oracle on the same inputs
    got, want, ref = _both(ctx, 4, 2, 64, 33, 0, 7)
    assert np.abs(got - want).max() <= 2e-3 and np.abs(got - ref).max() <= 2e-3
    # empty range -> zeros, like the regular entry point
    got, want, _ = _both(ctx, 16, 2, 256, 50, 50, 9)
    assert np.all(got == 0) and np.all(want == 0)
    ctx.close()


def test_noalloc_leaves_free_device_memory_unchanged():
    # Everything the call touches is allocated beforehand and one warm call has done the address
    # lookup; across the next call (and the wait for it) the driver's free-memory figure must not move.
    hq, hkv, hd, s = 16, 2, 256, 20000
    q, k, v, _, got = _case(hq, hkv, hd, s, 21)
    stream = torch.cuda.current_stream().cuda_stream
    f = L.lib().tt_attn_decode_noalloc
    assert f(stream, _ptr(q), _ptr(k), _ptr(v), _ptr(got), hd, hq, hkv, s, 0, 0.0625) == L.TT_OK
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert f(stream, _ptr(q), _ptr(k), _ptr(v), _ptr(got), hd, hq, hkv, s, 0, 0.0625) == L.TT_OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_noalloc_rejects_what_does_not_fit():
    x = torch.zeros(1 << 16, device="cuda", dtype=torch.float16)
    stream = torch.cuda.current_stream().cuda_stream
    f = L.lib().tt_attn_decode_noalloc
    assert f(stream, _ptr(x), _ptr(x), _ptr(x), _ptr(x), 96, 16, 2, 8, 0, 1.0) == L.TT_ERR_UNSUPPORTED_SHAPE
    assert f(stream, _ptr(x), _ptr(x), _ptr(x), _ptr(x), 256, 16, 3, 8, 0, 1.0) == L.TT_ERR_INVALID_ARG
    assert f(stream, None, _ptr(x), _ptr(x), _ptr(x), 256, 16, 2, 8, 0, 1.0) == L.TT_ERR_INVALID_ARG
    assert f(stream, C.c_void_p(x.data_ptr() + 2), _ptr(x), _ptr(x), _ptr(x), 256, 16, 2, 8, 0, 1.0) == L.TT_ERR_UNSUPPORTED_SHAPE
    # a key range beyond TT_NOALLOC_MAX_KEYS is refused before anything is launched or read
    assert f(stream, _ptr(x), _ptr(x), _ptr(x), _ptr(x), 256, 16, 2, (1 << 22) + 1, 0, 1.0) == L.TT_ERR_UNSUPPORTED_SHAPE
