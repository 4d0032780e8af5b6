"""Causal prefill SDPA (generic kernel and the tcgen05 kernel) against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from oracle.prng import seed_tree_key
from gpu_util import TOL, context, dev, host, rounded, bf16_tol

pytestmark = pytest.mark.gpu


def run_prefill(q, k, v, p: tt.PrefillAttentionParams, dtype=torch.float16, prefix=(0, 0, 0, 0), expect=None):
    """q/k/v flat fp32 arrays laid out with the strides in p; prefix = element offsets of the four
    buffers inside their allocations (the reference tests bind non-zero buffer offsets)."""
    def place(a, off):
        buf = torch.zeros(off + a.size, device="cuda", dtype=dtype)
        buf[off:] = dev(a.ravel(), dtype)
        return buf
    qb, kb, vb = place(q, prefix[0]), place(k, prefix[1]), place(v, prefix[2])
    n_out = p.query_count * p.o_token_stride_elements
    ob = torch.full((prefix[3] + n_out,), float("nan"), device="cuda", dtype=dtype)
    pa = tt.PrefillAttention(context())
    path = pa.selected_path(qb, kb, vb, ob, p, q_offset=prefix[0] * 2, k_offset=prefix[1] * 2,
                            v_offset=prefix[2] * 2, out_offset=prefix[3] * 2)
    if expect is not None:
        assert path == expect
    pa.encode_causal(qb, kb, vb, ob, p, q_offset=prefix[0] * 2, k_offset=prefix[1] * 2, v_offset=prefix[2] * 2,
                     out_offset=prefix[3] * 2)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    o = host(ob[prefix[3]:]).reshape(p.query_count, p.o_token_stride_elements)
    return o[:, :p.num_q_heads * p.head_dim].reshape(p.query_count, p.num_q_heads, p.head_dim)


def reference_case(root, start, chunk, window, hd, hq, hkv):
    # Layout of tests/TinyTitan/Kernels/Attention/PrefillAttentionTests.swift:306-346: padded
    # strides Hq*hd+3 / Hkv*hd+5 / Hq*hd+7, scale 1.0, U(-0.35, 0.35); q per (t,h,d), then per
    # (pos,h,d) k and v interleaved.
    g = seed_tree_key(root, f"prefill-attn-start{start}-chunk{chunk}-window{window}")
    qs, kvs, os_ = hq * hd + 3, hkv * hd + 5, hq * hd + 7
    kv_valid = start + chunk
    q = np.zeros((chunk, qs), np.float32); k = np.zeros((kv_valid, kvs), np.float32); v = np.zeros((kv_valid, kvs), np.float32)
    for t in range(chunk):
        q[t, :hq * hd] = g.uniform_array(hq * hd, -0.35, 0.35)
    for pos in range(kv_valid):
        kvrow = g.uniform_array(2 * hkv * hd, -0.35, 0.35).reshape(hkv * hd, 2)
        k[pos, :hkv * hd] = kvrow[:, 0]; v[pos, :hkv * hd] = kvrow[:, 1]
    p = tt.PrefillAttentionParams(start, chunk, hd, hq, hkv, kv_valid, window, kvs, qs, os_, 1.0)
    return rounded(q), rounded(k), rounded(v), p


@pytest.mark.parametrize("i,start,chunk,window,hd,hq,hkv", [
    (0, 0, 5, 0, 8, 4, 2), (1, 3, 4, 0, 32, 4, 1), (2, 7, 6, 4, 8, 2, 2), (3, 0, 9, 3, 32, 8, 2),
    (4, 2, 3, 0, 256, 16, 8), (5, 1, 2, 0, 512, 16, 2)])
def test_generic_kernel_reference_layouts(i, start, chunk, window, hd, hq, hkv):
    q, k, v, p = reference_case(0xA510 + i, start, chunk, window, hd, hq, hkv)
    want = oracle.attn_prefill(q, k, v, p.q_token_stride_elements, p.kv_token_stride_elements, hd, hq, hkv, start,
                               chunk, p.kv_valid_count, window, 1.0)
    got = run_prefill(q, k, v, p, prefix=(17, 19, 23, 29), expect="generic")
    # reference bar: maxAbs and rel <= 2e-2 (PrefillAttentionTests.swift:353-354); ours is tighter
    assert np.abs(got - want).max() <= TOL


def test_future_rows_are_masked():
    # PrefillAttentionTests.swift:74-93: rows after the query position must not leak in
    r = np.random.default_rng(1)
    hd, hq, hkv, start, chunk = 64, 4, 2, 4, 6
    kv_valid = start + chunk
    q = rounded(r.normal(size=(chunk, hq * hd))); k = rounded(r.normal(size=(kv_valid, hkv * hd))); v = rounded(r.normal(size=(kv_valid, hkv * hd)))
    p = tt.PrefillAttentionParams(start, chunk, hd, hq, hkv, kv_valid, 0, hkv * hd, hq * hd, hq * hd, 0.125)
    a = run_prefill(q, k, v, p)
    k2, v2 = k.copy(), v.copy()
    k2[start + 3:] = 100.0; v2[start + 3:] = -100.0           # poison the future of row 2
    b = run_prefill(q, k2, v2, p)
    assert np.array_equal(a[:3], b[:3])


def tc_case(r, start, chunk, hq, hkv, window=0, dtype=torch.float16, pad=0, extra_valid=0):
    hd = 256
    kv_valid = start + chunk + extra_valid
    qs, kvs, os_ = hq * hd + pad, hkv * hd + pad, hq * hd + pad
    q = np.zeros((chunk, qs), np.float32); k = np.zeros((kv_valid, kvs), np.float32); v = np.zeros((kv_valid, kvs), np.float32)
    q[:, :hq * hd] = r.normal(size=(chunk, hq * hd)); k[:, :hkv * hd] = r.normal(size=(kv_valid, hkv * hd))
    v[:, :hkv * hd] = r.normal(size=(kv_valid, hkv * hd))
    p = tt.PrefillAttentionParams(start, chunk, hd, hq, hkv, kv_valid, window, kvs, qs, os_, 0.0625)
    return rounded(q, dtype), rounded(k, dtype), rounded(v, dtype), p


@pytest.mark.parametrize("start,chunk,hq,hkv,window,pad,extra", [
    (0, 128, 2, 1, 0, 0, 0), (0, 64, 2, 2, 0, 0, 0), (0, 1, 2, 1, 0, 0, 0), (0, 300, 4, 2, 0, 8, 0),
    (77, 200, 2, 1, 0, 0, 0), (0, 513, 2, 1, 0, 0, 0), (130, 129, 4, 1, 100, 0, 5), (0, 1024, 16, 2, 0, 0, 0),
    # around the 128-key tile and the 64-key halves the two softmax groups and the V loads work in
    (0, 127, 2, 1, 0, 0, 0), (0, 255, 2, 1, 0, 0, 0), (0, 257, 2, 2, 0, 0, 0), (128, 128, 2, 1, 0, 0, 0),
    (65, 190, 2, 1, 0, 0, 0), (0, 600, 2, 1, 200, 0, 0), (300, 77, 2, 1, 65, 8, 3),
    # the last boundary of PrefillAttentionTests.swift:144-180 (1 ... 1025 keys)
    (0, 1025, 2, 1, 0, 0, 0)])
def test_tcgen05_kernel_matches_oracle(start, chunk, hq, hkv, window, pad, extra):
    r = np.random.default_rng(start * 7 + chunk)
    q, k, v, p = tc_case(r, start, chunk, hq, hkv, window, pad=pad, extra_valid=extra)
    want = oracle.attn_prefill(q, k, v, p.q_token_stride_elements, p.kv_token_stride_elements, 256, hq, hkv, start,
                               chunk, p.kv_valid_count, window, 0.0625)
    got = run_prefill(q, k, v, p, expect="tcgen05")
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= TOL


def test_tcgen05_kernel_bf16():
    r = np.random.default_rng(99)
    q, k, v, p = tc_case(r, 0, 384, 4, 2, dtype=torch.bfloat16)
    want = oracle.attn_prefill(q, k, v, p.q_token_stride_elements, p.kv_token_stride_elements, 256, 4, 2, 0, 384,
                               p.kv_valid_count, 0, 0.0625)
    got = run_prefill(q, k, v, p, dtype=torch.bfloat16, expect="tcgen05")
    assert np.all(np.abs(got - want) <= bf16_tol(want))


def test_tcgen05_large_scores_rescale_path():
    # scores far apart force the running maximum to move by more than the lazy threshold
    r = np.random.default_rng(4)
    q, k, v, p = tc_case(r, 0, 256, 2, 1)
    k[100] *= 6.0; k[200] *= 12.0
    k = rounded(k)
    want = oracle.attn_prefill(q, k, v, p.q_token_stride_elements, p.kv_token_stride_elements, 256, 2, 1, 0, 256,
                               p.kv_valid_count, 0, 0.0625)
    got = run_prefill(q, k, v, p, expect="tcgen05")
    assert np.abs(got - want).max() <= TOL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tcgen05_equals_generic_at_config3_size_and_is_byte_stable(dtype):
    # Full config-3 shape (8192 tokens, 16/2/256, bf16). The oracle would need minutes; the two
    # independent CUDA kernels must agree, and the tcgen05 kernel must be run-to-run byte-stable
    # (PrefillAttentionTests.swift:144-180).
    import os
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    T, hq, hkv, hd = 8192, 16, 2, 256
    q = torch.randn(T, hq * hd, device="cuda", generator=g).to(dtype)
    k = torch.randn(T, hkv * hd, device="cuda", generator=g).to(dtype)
    v = torch.randn(T, hkv * hd, device="cuda", generator=g).to(dtype)
    p = tt.PrefillAttentionParams(0, T, hd, hq, hkv, T, 0, hkv * hd, hq * hd, hq * hd, 0.0625)
    pa = tt.PrefillAttention(context())
    o1 = torch.empty(T, hq * hd, device="cuda", dtype=dtype); o2 = torch.empty_like(o1); o3 = torch.empty_like(o1)
    pa.encode_causal(q, k, v, o1, p)
    pa.encode_causal(q, k, v, o2, p)
    os.environ["TT_PREFILL_FORCE_GENERIC"] = "1"
    try:
        pa.encode_causal(q, k, v, o3, p)
    finally:
        del os.environ["TT_PREFILL_FORCE_GENERIC"]
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    assert torch.equal(o1, o2)
    # bf16 I/O: both outputs carry one bf16 rounding (2^-8 relative each) and the tensor-core
    # kernel's probabilities are bf16 (2^-9 relative on |v| <= ~4.5); fp16 I/O is held to 2e-3.
    if dtype == torch.bfloat16:
        excess = (o1.float() - o3.float()).abs() - (1e-2 + o3.float().abs() * 2.0 ** -7)
    else:
        excess = (o1.float() - o3.float()).abs() - (2e-3 + o3.float().abs() * 2.0 ** -10)
    assert excess.max().item() <= 0, excess.max().item()
    assert (o1.float() - o3.float()).abs().mean().item() < 5e-4
    # causality as a property: the first 128 rows only depend on the first 128 keys
    k2 = k.clone(); k2[128:] = 0
    o4 = torch.empty_like(o1)
    pa.encode_causal(q, k2, v, o4, p)
    torch.cuda.synchronize()
    assert torch.equal(o1[:128], o4[:128])


def test_validation_errors():
    pa = tt.PrefillAttention(context())
    x = torch.zeros(1 << 16, device="cuda", dtype=torch.float16)
    ok = dict(start_position=0, query_count=4, head_dim=64, num_q_heads=4, num_kv_heads=2, kv_valid_count=4,
              sliding_window=0, kv_token_stride_elements=128, q_token_stride_elements=256,
              o_token_stride_elements=256, scale=0.125)
    for bad in (dict(query_count=0), dict(num_kv_heads=3), dict(q_token_stride_elements=255),
                dict(o_token_stride_elements=1), dict(kv_token_stride_elements=127), dict(kv_valid_count=3),
                dict(kv_bits=5)):
        with pytest.raises(tt.InvalidArgument):
            pa.encode_causal(x, x, x, x, tt.PrefillAttentionParams(**{**ok, **bad}))
    with pytest.raises(tt.InvalidArgument):   # quantised stride without room for the values and groups
        pa.encode_causal(x, x, x, x, tt.PrefillAttentionParams(**{**ok, "kv_bits": 8, "kv_token_stride_bytes": 72}))


def test_non_positive_scale_takes_the_generic_kernel():
    # the tensor-core kernel takes row maxima before scaling, which needs a positive scale
    r = np.random.default_rng(8)
    q, k, v, p = tc_case(r, 0, 130, 2, 1)
    p = tt.PrefillAttentionParams(p.start_position, p.query_count, p.head_dim, p.num_q_heads, p.num_kv_heads,
                                  p.kv_valid_count, p.sliding_window, p.kv_token_stride_elements,
                                  p.q_token_stride_elements, p.o_token_stride_elements, -0.0625)
    want = oracle.attn_prefill(q, k, v, p.q_token_stride_elements, p.kv_token_stride_elements, 256, 2, 1, 0, 130,
                               p.kv_valid_count, 0, -0.0625)
    got = run_prefill(q, k, v, p, expect="generic")
    assert np.abs(got - want).max() <= TOL
