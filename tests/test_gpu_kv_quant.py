"""Affine-quantised KV rows (int8 / int4): quantiser, decode attention and prefill attention."""
import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from gpu_util import TOL, context, dev, host, rounded

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [8, 4])
def test_row_layout_and_quantiser_bytes(bits):
    # tests/TinyTitan/Kernels/Attention/KVCacheQuantizedAttentionTests.swift:86-101: 544 / 288 byte rows at 2 x 256
    r = np.random.default_rng(bits)
    tokens, n = 37, 512
    x = rounded(r.normal(size=(tokens, n)))
    x[3] = 0.25                       # a constant group: scale 0, every code 0
    want, deq, stride, value_bytes = oracle.kv_quantize_rows(x, bits)
    assert (stride, value_bytes) == tt.KVCacheManager.row_layout(n, bits)
    dst = torch.zeros(tokens, stride, device="cuda", dtype=torch.uint8)
    tt.quantize_kv_rows(context(), dev(x), dst, n, bits, tokens)
    torch.cuda.synchronize()
    got = dst.cpu().numpy()
    assert np.array_equal(got[:, value_bytes:], want[:, value_bytes:])        # scales and biases, bit for bit
    codes_equal = (got[:, :value_bytes] == want[:, :value_bytes]).mean()
    assert codes_equal > 0.999        # a code may differ by one where (x-bias)/scale sits on a .5 boundary
    assert np.abs(deq - x).max() <= (x.max() - x.min()) / (15 if bits == 4 else 255) * 0.51 + 2e-3


@pytest.mark.parametrize("bits,hd,hq,hkv,s", [(8, 256, 16, 2, 3000), (4, 256, 24, 2, 700), (8, 128, 8, 4, 513), (4, 128, 8, 2, 64)])
def test_decode_attention_over_quantised_rows(bits, hd, hq, hkv, s):
    r = np.random.default_rng(bits * 1000 + s)
    q = rounded(r.normal(size=(hq, hd)))
    k = rounded(r.normal(size=(s, hkv * hd))); v = rounded(r.uniform(0, 1, size=(s, hkv * hd)))
    kq, kdeq, stride, vb = oracle.kv_quantize_rows(k, bits)
    vq, vdeq, _, _ = oracle.kv_quantize_rows(v, bits)
    scale = 1.0 / np.sqrt(hd)
    want = oracle.attn_decode(q, kdeq.reshape(s, hkv, hd), vdeq.reshape(s, hkv, hd), hkv, scale)
    out = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    kd, vd = torch.from_numpy(kq).cuda(), torch.from_numpy(vq).cuda()
    tt.Attention(context()).encode_full(dev(q), kd, vd, out, hd, hq, hkv, s, scale=scale,
                                        kv_format=tt.KVFormat(bits, stride, vb, 64))
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    got = host(out)
    # reference bar for quantised rows: rel < 2e-2 (SimdPartialAttentionTests.swift:128-155); ours: the fp16 bar
    assert np.abs(got - want).max() <= TOL
    # and the quantiser on the device feeds the same kernel
    kd2 = torch.zeros_like(kd); vd2 = torch.zeros_like(vd)
    tt.quantize_kv_rows(context(), dev(k), kd2, hkv * hd, bits, s)
    tt.quantize_kv_rows(context(), dev(v), vd2, hkv * hd, bits, s)
    out2 = torch.empty_like(out)
    tt.Attention(context()).encode_full(dev(q), kd2, vd2, out2, hd, hq, hkv, s, scale=scale,
                                        kv_format=tt.KVFormat(bits, stride, vb, 64))
    torch.cuda.synchronize()
    assert np.abs(host(out2) - want).max() <= 3 * TOL     # a handful of codes may differ by one


@pytest.mark.parametrize("bits", [8, 4])
def test_prefill_attention_over_quantised_rows(bits):
    r = np.random.default_rng(bits)
    hd, hq, hkv, start, chunk = 64, 4, 2, 9, 20
    kv_valid = start + chunk
    q = rounded(r.normal(size=(chunk, hq * hd)))
    k = rounded(r.normal(size=(kv_valid, hkv * hd))); v = rounded(r.normal(size=(kv_valid, hkv * hd)))
    kq, kdeq, stride, vb = oracle.kv_quantize_rows(k, bits)
    vq, vdeq, _, _ = oracle.kv_quantize_rows(v, bits)
    want = oracle.attn_prefill(q, kdeq, vdeq, hq * hd, hkv * hd, hd, hq, hkv, start, chunk, kv_valid, 0, 0.125)
    p = tt.PrefillAttentionParams(start, chunk, hd, hq, hkv, kv_valid, 0, 0, hq * hd, hq * hd, 0.125, kv_bits=bits,
                                  kv_token_stride_bytes=stride, kv_value_bytes=vb, kv_group_size=64)
    out = torch.empty(chunk, hq * hd, device="cuda", dtype=torch.float16)
    tt.PrefillAttention(context()).encode_causal(dev(q), torch.from_numpy(kq).cuda(), torch.from_numpy(vq).cuda(), out, p)
    torch.cuda.synchronize()
    assert np.abs(host(out).reshape(chunk, hq, hd) - want).max() <= TOL


def test_quantised_rows_refusals():
    attn = tt.Attention(context())
    x = torch.zeros(16, 256, device="cuda", dtype=torch.float16)
    kv = torch.zeros(8, 544, device="cuda", dtype=torch.uint8)
    with pytest.raises(tt.UnsupportedShape):      # wrong value_bytes for the shape
        attn.encode_full(x, kv, kv, x, 256, 16, 2, 8, kv_format=tt.KVFormat(8, 544, 500, 64))
    with pytest.raises(tt.UnsupportedShape):      # group size other than 64
        attn.encode_full(x, kv, kv, x, 256, 16, 2, 8, kv_format=tt.KVFormat(8, 544, 512, 32))
    with pytest.raises(tt.InvalidArgument):
        attn.encode_full(x, kv, kv, x, 256, 16, 2, 8, kv_format=tt.KVFormat(5, 544, 512, 64))


@pytest.mark.parametrize("seq,keep_fraction,seed", [(4096, 0.55, 0x51AD), (700, 1.0, 0x51AE), (2048, 0.02, 0x51AF)])
def test_reference_sparse_int8_cases(seq, keep_fraction, seed):
    # tests/TinyTitan/Kernels/Attention/SimdPartialAttentionTests.swift:15-155: Qwen3.8 full-attention geometry
    # (24 q heads, 2 KV heads, head_dim 256), int8 KV quantised on the device, a sparse keep mask (the last key
    # always kept); q, k ~ U(-0.5, 0.5), v ~ U(0, 1), then the keep draws, all from SeedTree(seed).key("simd-partial-<S>").
    # The reference compares with fp32 attention over the UNQUANTISED kept keys at rel < 0.02 (RelError:
    # max |diff| / max |reference|) and wants no NaN when most chunks hold no kept key.
    from oracle.prng import seed_tree_key
    hq, hkv, hd = 24, 2, 256
    g = seed_tree_key(seed, f"simd-partial-{seq}")
    q = rounded(g.uniform_array(hq * hd, -0.5, 0.5)).reshape(hq, hd)
    k = rounded(g.uniform_array(seq * hkv * hd, -0.5, 0.5)).reshape(seq, hkv * hd)
    v = rounded(g.uniform_array(seq * hkv * hd, 0.0, 1.0)).reshape(seq, hkv * hd)
    keep = (g.uniform_array(seq, 0.0, 1.0) < np.float32(keep_fraction)).astype(np.uint8)
    keep[seq - 1] = 1
    stride, vb = tt.KVCacheManager.row_layout(hkv * hd, 8)
    kd = torch.zeros(seq, stride, device="cuda", dtype=torch.uint8); vd = torch.zeros_like(kd)
    tt.quantize_kv_rows(context(), dev(k), kd, hkv * hd, 8, seq)
    tt.quantize_kv_rows(context(), dev(v), vd, hkv * hd, 8, seq)
    out = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    tt.Attention(context()).encode_full(dev(q), kd, vd, out, hd, hq, hkv, seq, kv_format=tt.KVFormat(8, stride, vb, 64),
                                        keep_mask=torch.as_tensor(keep).cuda())
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    got = host(out)
    assert np.isfinite(got).all()
    kept = np.nonzero(keep)[0]
    scale = 1.0 / np.sqrt(hd)
    reference = oracle.attn_decode(q, k[kept].reshape(-1, hkv, hd), v[kept].reshape(-1, hkv, hd), hkv, scale)
    rel = np.abs(got - reference).max() / max(np.abs(reference).max(), 1e-6)
    assert rel < 0.02                                            # the reference's own bar
    # and against the oracle on what the kernel actually reads (the dequantised rows): the fp16 bar
    _, kdeq, _, _ = oracle.kv_quantize_rows(k, 8)
    _, vdeq, _, _ = oracle.kv_quantize_rows(v, 8)
    want = oracle.attn_decode(q, kdeq[kept].reshape(-1, hkv, hd), vdeq[kept].reshape(-1, hkv, hd), hkv, scale)
    assert np.abs(got - want).max() <= 3 * TOL                   # a handful of device-side codes may differ by one


def test_quantised_rows_in_a_ring_with_a_window():
    # int8 rows of a sliding-window layer: logical position p lives at ring row p % capacity
    r = np.random.default_rng(77)
    hq, hkv, hd, cap, seq, window = 8, 2, 128, 96, 250, 64
    q = rounded(r.normal(size=(hq, hd)))
    k = rounded(r.normal(size=(seq, hkv * hd))); v = rounded(r.uniform(0, 1, size=(seq, hkv * hd)))
    kq, kdeq, stride, vb = oracle.kv_quantize_rows(k, 8)
    vq, vdeq, _, _ = oracle.kv_quantize_rows(v, 8)
    ring_k = np.zeros((cap, stride), np.uint8); ring_v = np.zeros((cap, stride), np.uint8)
    for p in range(seq):
        ring_k[p % cap] = kq[p]; ring_v[p % cap] = vq[p]
    out = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    tt.Attention(context()).encode_swa(dev(q), torch.from_numpy(ring_k).cuda(), torch.from_numpy(ring_v).cuda(), out, hd, hq, hkv,
                                       seq, window, scale=0.09, ring_capacity=cap, kv_format=tt.KVFormat(8, stride, vb, 64))
    torch.cuda.synchronize()
    want = oracle.attn_decode(q, kdeq.reshape(seq, hkv, hd), vdeq.reshape(seq, hkv, hd), hkv, 0.09, window=window)
    assert np.abs(host(out) - want).max() <= TOL
