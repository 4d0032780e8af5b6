"""Decode SDPA through the C ABI against the CPU oracle (B200 only)."""
import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from oracle.prng import seed_tree_key
from gpu_util import TOL, context, dev, host, rounded, bf16_tol

pytestmark = pytest.mark.gpu


def _decode(q, k, v, hkv, scale=None, seq_len=None, **kw):
    hq, hd = q.shape
    s = k.shape[0] if seq_len is None else seq_len
    qd, kd, vd = dev(q), dev(k), dev(v)
    out = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    attn = tt.Attention(context())
    window = kw.pop("window", None)
    if window is not None:
        attn.encode_swa(qd, kd, vd, out, hd, hq, hkv, s, window, scale=scale, **kw)
    else:
        attn.encode_full(qd, kd, vd, out, hd, hq, hkv, s, scale=scale, **kw)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    return host(out)


@pytest.mark.parametrize("root,label,hd,hq,hkv,s,aliased", [
    (0x174, "attn-h8-kv1-d64-T128-kv=false", 64, 8, 1, 128, False),
    (0x175, "attn-h16-kv2-d256-T128-kv=false", 256, 16, 2, 128, False),
    (0x176, "attn-h8-kv1-d64-T128-kv=true", 64, 8, 1, 128, True),
    (0x177, "attn-h16-kv2-d256-T128-kv=true", 256, 16, 2, 128, True),
])
def test_reference_seeded_cases(root, label, hd, hq, hkv, s, aliased):
    # tests/TinyTitan/Kernels/Attention/AttentionTests.swift:399-425 (reference bar: rel < 1e-2)
    g = seed_tree_key(root, label)
    q = rounded(g.uniform_array(hq * hd, -0.5, 0.5).reshape(hq, hd))
    k = rounded(g.uniform_array(s * hkv * hd, -0.5, 0.5).reshape(s, hkv, hd))
    v = k if aliased else rounded(g.uniform_array(s * hkv * hd, -0.5, 0.5).reshape(s, hkv, hd))
    want = oracle.attn_decode(q, k, v, hkv, 1.0 / np.sqrt(hd))
    got = _decode(q, k, v, hkv)
    assert np.abs(got - want).max() <= TOL
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-2


def test_runtime_scale_is_honoured():
    # AttentionTests.swift:59-123: scale 1.0 differs from the default-scale result
    g = seed_tree_key(0x501, "attn-scale1-swa")
    hd, hq, hkv, s = 64, 4, 2, 8
    q = rounded(g.uniform_array(hq * hd, -0.5, 0.5).reshape(hq, hd))
    k = rounded(g.uniform_array(s * hkv * hd, -0.5, 0.5).reshape(s, hkv, hd))
    v = rounded(g.uniform_array(s * hkv * hd, -0.5, 0.5).reshape(s, hkv, hd))
    got1 = _decode(q, k, v, hkv, scale=1.0, window=8)
    want1 = oracle.attn_decode(q, k, v, hkv, 1.0, window=8)
    assert np.abs(got1 - want1).max() <= TOL
    got_default = _decode(q, k, v, hkv, window=8)
    assert np.abs(got1 - got_default).max() > 1e-3


@pytest.mark.parametrize("hd,hq,hkv,s", [(256, 8, 2, 4096), (256, 16, 2, 1), (256, 16, 2, 17), (128, 8, 8, 300),
                                          (64, 4, 2, 1000), (256, 24, 2, 700), (256, 32, 2, 2049)])
def test_shapes_normal_inputs(hd, hq, hkv, s):
    r = np.random.default_rng(hd + hq + s)
    q = rounded(r.normal(size=(hq, hd))); k = rounded(r.normal(size=(s, hkv, hd))); v = rounded(r.normal(size=(s, hkv, hd)))
    scale = 1.0 / np.sqrt(hd)
    want = oracle.attn_decode(q, k, v, hkv, scale)
    got = _decode(q, k, v, hkv, scale=scale)
    assert np.abs(got - want).max() <= TOL


def test_gqa_head_mapping_by_permutation():
    # CPUEngineTests.swift:730-825: query head h reads KV head h / (Hq / Hkv). Swapping the KV heads of the cache
    # must give exactly the outputs of the original cache with the two query-head groups swapped (same kernel,
    # same arithmetic per head, so bit for bit), on the decode kernel and on the tensor-core verify kernel.
    r = np.random.default_rng(730)
    hq, hkv, hd, s = 16, 2, 256, 777
    g = hq // hkv
    q = rounded(r.normal(size=(hq, hd)))
    k = rounded(r.normal(size=(s, hkv, hd))); v = rounded(r.normal(size=(s, hkv, hd)))
    base = _decode(q, k.reshape(s, -1), v.reshape(s, -1), hkv, scale=0.0625)
    q_swapped = np.concatenate([q[g:], q[:g]])
    swapped = _decode(q_swapped, k[:, ::-1].reshape(s, -1).copy(), v[:, ::-1].reshape(s, -1).copy(), hkv, scale=0.0625)
    assert np.array_equal(np.concatenate([swapped[g:], swapped[:g]]), base)
    # a changed KV head 1 leaves the outputs of the heads that read KV head 0 alone
    v2 = v.copy(); v2[:, 1] += 1.0
    moved = _decode(q, k.reshape(s, -1), rounded(v2).reshape(s, -1), hkv, scale=0.0625)
    assert np.array_equal(moved[:g], base[:g]) and not np.array_equal(moved[g:], base[g:])
    # the same through the verify kernel (4 draft rows x 32 heads: 64 packed rows per KV head)
    rr = np.random.default_rng(731)
    got, want = _verify_batch(rr, 32, 2, 4, [900])
    assert np.all(np.abs(got[0] - want[0]) <= TOL)


def test_sliding_window_ring_and_keep_mask():
    r = np.random.default_rng(7)
    hd, hq, hkv, s = 256, 16, 2, 900
    q = rounded(r.normal(size=(hq, hd))); k = rounded(r.normal(size=(s, hkv, hd))); v = rounded(r.normal(size=(s, hkv, hd)))
    scale = 0.0625
    # window
    want = oracle.attn_decode(q, k, v, hkv, scale, window=129)
    assert np.abs(_decode(q, k, v, hkv, scale=scale, window=129) - want).max() <= TOL
    # ring: logical p at row p % cap
    cap = 160
    rk = np.zeros((cap, hkv, hd), np.float32); rv = np.zeros((cap, hkv, hd), np.float32)
    for p in range(s):
        rk[p % cap] = k[p]; rv[p % cap] = v[p]
    want = oracle.attn_decode(q, k, v, hkv, scale, window=128)
    got = _decode(q, rk, rv, hkv, scale=scale, seq_len=s, window=128, ring_capacity=cap)
    assert np.abs(got - want).max() <= TOL
    # sparse keep mask (SimdPartialAttentionTests.swift:15-35: empty chunks must not NaN)
    for frac in (0.55, 0.02):
        keep = (r.uniform(size=s) < frac).astype(np.uint8); keep[-1] = 1
        want = oracle.attn_decode_split(q, k, v, hkv, scale, s, keep=keep)
        got = _decode(q, k, v, hkv, scale=scale, keep_mask=torch.as_tensor(keep).cuda())
        assert np.isfinite(got).all() and np.abs(got - want).max() <= TOL
    # everything masked -> zeros (attention.metal:418-424)
    got = _decode(q, k, v, hkv, scale=scale, keep_mask=torch.zeros(s, dtype=torch.uint8, device="cuda"))
    assert np.all(got == 0)


def test_long_session_merge_with_empty_parts():
    # One long session, two rows: the merge pass splits the row's columns over several CTAs and walks
    # hundreds of parts in groups, each group keeping an online (max, sum, output) triple. The keep mask
    # leaves long stretches without any key, so whole parts (the first ones of most groups among them)
    # arrive with a maximum of -inf and a zero sum, and must neither produce NaN nor weigh in.
    r = np.random.default_rng(41)
    hd, hq, hkv, s = 128, 2, 1, 60000
    q = rounded(r.normal(size=(hq, hd))); k = rounded(r.normal(size=(s, hkv, hd))); v = rounded(r.normal(size=(s, hkv, hd)))
    keep = np.zeros(s, np.uint8)
    keep[20000:20300] = 1; keep[41000:41007] = 1; keep[59990:] = 1
    keep[r.integers(30000, 36000, size=40)] = 1
    want = oracle.attn_decode_split(q, k, v, hkv, 0.09, s, keep=keep)
    launches = context().launch_count
    got = _decode(q, k, v, hkv, scale=0.09, keep_mask=torch.as_tensor(keep).cuda())
    assert context().launch_count - launches == 2
    assert np.isfinite(got).all() and np.abs(got - want).max() <= TOL


def _batched_case(r, n, hq, hkv, hd, lens, q_rows, dtype=torch.float16, stride_pad=0):
    """Sessions packed into one KV store of the reference layout: slot s at row s*capacity."""
    cap = max(lens) + 8
    stride = hkv * hd + stride_pad
    kbuf = np.zeros((n * cap, stride), np.float32); vbuf = np.zeros((n * cap, stride), np.float32)
    kbuf[:, :hkv * hd] = r.normal(size=(n * cap, hkv * hd)); vbuf[:, :hkv * hd] = r.normal(size=(n * cap, hkv * hd))
    kbuf = rounded(kbuf, dtype); vbuf = rounded(vbuf, dtype)
    q = rounded(r.normal(size=(n, q_rows, hq * hd)), dtype)
    return cap, stride, kbuf, vbuf, q


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_batched_ragged_sessions(dtype):
    r = np.random.default_rng(11)
    n, hq, hkv, hd = 9, 16, 2, 256
    lens = [int(x) for x in r.integers(1, 3000, size=n)]
    lens[0], lens[1] = 1, 2999
    cap, stride, kbuf, vbuf, q = _batched_case(r, n, hq, hkv, hd, lens, 1, dtype, stride_pad=8)
    kd, vd, qd = dev(kbuf, dtype), dev(vbuf, dtype), dev(q, dtype)
    out = torch.full((n, 1, hq * hd), float("nan"), device="cuda", dtype=dtype)
    esz = 2
    sessions = [tt.DecodeSession(qd, out, kd, vd, lens[i], 1, 0, q_offset=i * hq * hd * esz,
                                 out_offset=i * hq * hd * esz, k_offset=i * cap * stride * esz,
                                 v_offset=i * cap * stride * esz) for i in range(n)]
    tt.Attention(context()).encode_batched(sessions, hd, hq, hkv, kv_token_stride_elements=stride, scale=0.0625)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    got = host(out)
    for i in range(n):
        kk = kbuf[i * cap:i * cap + lens[i], :hkv * hd].reshape(lens[i], hkv, hd)
        vv = vbuf[i * cap:i * cap + lens[i], :hkv * hd].reshape(lens[i], hkv, hd)
        want = oracle.attn_decode(q[i, 0].reshape(hq, hd), kk, vv, hkv, 0.0625).reshape(-1)
        tol = TOL if dtype == torch.float16 else bf16_tol(want)
        assert np.all(np.abs(got[i, 0] - want) <= tol), (i, lens[i], np.abs(got[i, 0] - want).max())


@pytest.mark.parametrize("hq,q_rows", [(16, 4), (32, 4), (8, 2), (24, 3)])
def test_few_token_verify_rows(hq, q_rows):
    # Row r of W at base position P attends keys [0, P + r]
    # (RealForwardRunner+VerifyDecodeOrderAttention.swift:84-105): equal to W single-row decodes.
    r = np.random.default_rng(hq * 10 + q_rows)
    n, hkv, hd = 3, 2, 256
    lens = [600 + q_rows, 64 + q_rows, q_rows]   # seq_len counts the draft rows themselves
    cap, stride, kbuf, vbuf, q = _batched_case(r, n, hq, hkv, hd, lens, q_rows)
    kd, vd, qd = dev(kbuf), dev(vbuf), dev(q)
    out = torch.full((n, q_rows, hq * hd), float("nan"), device="cuda", dtype=torch.float16)
    sessions = [tt.DecodeSession(qd, out, kd, vd, lens[i], q_rows, 0, q_offset=i * q_rows * hq * hd * 2,
                                 out_offset=i * q_rows * hq * hd * 2, k_offset=i * cap * stride * 2,
                                 v_offset=i * cap * stride * 2) for i in range(n)]
    tt.Attention(context()).encode_batched(sessions, hd, hq, hkv, scale=0.0625)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    got = host(out)
    for i in range(n):
        for w in range(q_rows):
            vis = lens[i] - (q_rows - 1 - w)
            kk = kbuf[i * cap:i * cap + vis].reshape(vis, hkv, hd); vv = vbuf[i * cap:i * cap + vis].reshape(vis, hkv, hd)
            want = oracle.attn_decode(q[i, w].reshape(hq, hd), kk, vv, hkv, 0.0625).reshape(-1)
            assert np.abs(got[i, w] - want).max() <= TOL, (i, w)


def test_partial_and_combine_across_shards():
    # A KV range split over G "devices": each produces one (m, d, o) triple per head, the merge
    # equals attention over the whole range (config 4's exchange, done here on one GPU).
    r = np.random.default_rng(3)
    hq, hkv, hd, s, shards = 16, 2, 256, 5000, 4
    q = rounded(r.normal(size=(hq, hd))); k = rounded(r.normal(size=(s, hkv, hd))); v = rounded(r.normal(size=(s, hkv, hd)))
    qd, kd, vd = dev(q), dev(k), dev(v)
    m = torch.zeros(shards, hq, device="cuda"); d = torch.zeros(shards, hq, device="cuda")
    o = torch.zeros(shards, hq, hd, device="cuda")
    attn = tt.Attention(context())
    bounds = [0, 1300, 1300, 3700, s]   # shard 1 is empty on purpose
    for g in range(shards):
        lo, hi = bounds[g], bounds[g + 1]
        attn.encode_partial(qd, kd, vd, hd, hq, hkv, hi, lo, m[g], d[g], o[g], scale=0.0625)
    out = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
    attn.encode_combine(m, d, o, shards, hq, hd, out)
    torch.cuda.synchronize()
    want = oracle.attn_decode(q, k, v, hkv, 0.0625)
    assert np.abs(host(out) - want).max() <= TOL
    assert np.isinf(host(m[1])).all() and np.all(host(d[1]) == 0)   # empty shard: (-inf, 0, 0)
    # the partial format is the reference's: m = max score, d = sum exp(s - m)
    mo, do_, oo = oracle.attn_partial(q[3], k.reshape(s, -1), v.reshape(s, -1), hkv, 0, 0, 1300, 0.0625)
    assert abs(host(m[0])[3] - mo) < 1e-3 and abs(host(d[0])[3] - do_) / do_ < 2e-3


def test_rejects_bad_arguments():
    attn = tt.Attention(context())
    x = torch.zeros(16, 256, device="cuda", dtype=torch.float16)
    kv = torch.zeros(8, 2, 256, device="cuda", dtype=torch.float16)
    with pytest.raises(tt.InvalidArgument):
        attn.encode_full(x, kv, kv, x, 256, 16, 3, 8)          # 16 % 3 != 0
    with pytest.raises(tt.InvalidArgument):
        attn.encode_full(x, kv, kv, x, 256, 16, 2, 0)          # needs one KV position
    with pytest.raises(tt.UnsupportedShape):
        attn.encode_full(x, kv, kv, x, 256, 16, 2, 8, kv_format=tt.KVFormat(bits=8, stride=544))
    with pytest.raises(tt.UnsupportedShape):
        attn.encode_full(x, kv, kv, x, 96, 16, 2, 8)           # head_dim without a kernel: refused, not skipped


def test_large_batch_property_partition_invariance():
    # At full config-2 size the oracle is too slow; the result must not depend on how the key
    # range is partitioned: one batched call (library split) vs explicit shards merged by combine.
    r = torch.Generator(device="cuda"); r.manual_seed(5)
    hq, hkv, hd, s = 16, 2, 256, 32768
    q = torch.randn(hq, hd, device="cuda", generator=r).half()
    k = torch.randn(s, hkv, hd, device="cuda", generator=r).half()
    v = torch.randn(s, hkv, hd, device="cuda", generator=r).half()
    attn = tt.Attention(context())
    out_a = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
    attn.encode_full(q, k, v, out_a, hd, hq, hkv, s, scale=0.0625)
    m = torch.zeros(3, hq, device="cuda"); d = torch.zeros(3, hq, device="cuda"); o = torch.zeros(3, hq, hd, device="cuda")
    for g, (lo, hi) in enumerate([(0, 10000), (10000, 10001), (10001, s)]):
        attn.encode_partial(q, k, v, hd, hq, hkv, hi, lo, m[g], d[g], o[g], scale=0.0625)
    out_b = torch.empty_like(out_a)
    attn.encode_combine(m, d, o, 3, hq, hd, out_b)
    torch.cuda.synchronize()
    assert (out_a.float() - out_b.float()).abs().max().item() <= 1e-3
    # and against a float64 statement of the same softmax on the device
    sc = torch.einsum("hd,shd->hs", q.double(), k.double().repeat_interleave(hq // hkv, dim=1)) * 0.0625
    ref = torch.einsum("hs,shd->hd", torch.softmax(sc, dim=1), v.double().repeat_interleave(hq // hkv, dim=1))
    assert (out_a.double() - ref).abs().max().item() <= TOL


def test_windowed_selection_with_row_indirection():
    # attention_decode_window_partial (attention.metal:612-870): key s of the selection lives at row sel_row[s]
    r = np.random.default_rng(13)
    hq, hkv, hd, rows, count = 16, 2, 256, 5000, 2049
    q = rounded(r.normal(size=(hq, hd)))
    k = rounded(r.normal(size=(rows, hkv, hd))); v = rounded(r.normal(size=(rows, hkv, hd)))
    sel = r.permutation(rows)[:count].astype(np.uint32)
    out = torch.full((hq, hd), float("nan"), device="cuda", dtype=torch.float16)
    tt.Attention(context()).encode_window(dev(q), dev(k), dev(v), out, hd, hq, hkv,
                                          torch.from_numpy(sel.astype(np.int64)).to(torch.int32).cuda(), count, scale=0.0625)
    torch.cuda.synchronize()
    want = oracle.attn_decode(q, k[sel], v[sel], hkv, 0.0625)
    assert np.abs(host(out) - want).max() <= TOL


def _verify_batch(r, hq, hkv, q_rows, lens, dtype=torch.float16, kv_start=None, stride_pad=0, k_gain=None,
                  scale=0.0625):
    """Runs one few-token batch through the C ABI; returns (outputs, per-row oracle outputs)."""
    n, hd = len(lens), 256
    cap, stride, kbuf, vbuf, q = _batched_case(r, n, hq, hkv, hd, lens, q_rows, dtype, stride_pad)
    if k_gain is not None:
        for i in range(n):   # scores that keep growing along the sequence: the reference maxima are raised again and again
            kbuf[i * cap:(i + 1) * cap, :hkv * hd] *= k_gain(np.arange(cap))[:, None]
        kbuf = rounded(kbuf, dtype)
    kd, vd, qd = dev(kbuf, dtype), dev(vbuf, dtype), dev(q, dtype)
    out = torch.full((n, q_rows, hq * hd), float("nan"), device="cuda", dtype=dtype)
    starts = kv_start or [0] * n
    sessions = [tt.DecodeSession(qd, out, kd, vd, lens[i], q_rows, starts[i], q_offset=i * q_rows * hq * hd * 2,
                                 out_offset=i * q_rows * hq * hd * 2, k_offset=i * cap * stride * 2,
                                 v_offset=i * cap * stride * 2) for i in range(n)]
    tt.Attention(context()).encode_batched(sessions, hd, hq, hkv, kv_token_stride_elements=stride, scale=scale,
                                           io_dtype=tt.TT_F16 if dtype == torch.float16 else tt.TT_BF16)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    want = np.zeros((n, q_rows, hq * hd), np.float32)
    for i in range(n):
        for w in range(q_rows):
            vis = lens[i] - (q_rows - 1 - w)
            lo = starts[i]
            kk = kbuf[i * cap + lo:i * cap + vis, :hkv * hd].reshape(vis - lo, hkv, hd)
            vv = vbuf[i * cap + lo:i * cap + vis, :hkv * hd].reshape(vis - lo, hkv, hd)
            want[i, w] = oracle.attn_decode(q[i, w].reshape(hq, hd), kk, vv, hkv, scale).reshape(-1)
    return host(out), want


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_verify_tensor_core_ragged_multi_part(dtype):
    # 64 and 32 packed rows per KV head over ragged contexts long enough to be cut into several
    # parts per session, a padded row stride, and a context shorter than one 128-key tile.
    r = np.random.default_rng(501)
    for hq, q_rows in [(32, 4), (16, 4)]:
        lens = [4100, 2977, 131, 128 + q_rows, q_rows, 1500]
        got, want = _verify_batch(r, hq, 2, q_rows, lens, dtype, stride_pad=16)
        for i in range(len(lens)):
            tol = TOL if dtype == torch.float16 else bf16_tol(want[i])
            if dtype == torch.bfloat16 and lens[i] < 64:
                # bf16 softmax weights carry 8 mantissa bits; over a handful of keys their rounding does
                # not average out (error up to |v| * 2^-8). The reference's own bar is 2e-2 absolute.
                tol = 2e-2
            assert np.all(np.abs(got[i] - want[i]) <= tol), (hq, i, np.abs(got[i] - want[i]).max())


def test_verify_batches_on_both_sides_of_the_parameter_table_limit():
    # up to 16 sessions travel in the kernel parameters with their tensor maps (the CTA derives its item from the
    # block index), 17 and more go through the uploaded tables: both against the oracle, and the first 16 sessions
    # of the larger batch bit-identical to the smaller one when the split plan is the same
    r = np.random.default_rng(1617)
    lens = [int(x) for x in r.integers(200, 2500, size=17)]
    lens[3], lens[16] = 5, 4097
    for n in (16, 17):
        rr = np.random.default_rng(99)
        got, want = _verify_batch(rr, 32, 2, 4, lens[:n])
        for i in range(n):
            assert np.all(np.abs(got[i] - want[i]) <= TOL), (n, i, np.abs(got[i] - want[i]).max())


@pytest.mark.parametrize("hq,q_rows", [(32, 8), (32, 5), (16, 16)])
def test_verify_tensor_core_up_to_128_packed_rows(hq, q_rows):
    # 128, 80 and 128 packed rows per KV head: the 128-row form of the tensor-core kernel (four softmax warps, Q in
    # 64 KB, ten ring slots), several parts per session and a single-part session, against the oracle
    r = np.random.default_rng(128 + q_rows)
    lens = [3000, 700 + q_rows, q_rows, 1290]
    got, want = _verify_batch(r, hq, 2, q_rows, lens)
    for i in range(len(lens)):
        assert np.all(np.abs(got[i] - want[i]) <= TOL), (i, np.abs(got[i] - want[i]).max())


def test_verify_tensor_core_repeated_raises_and_window_start():
    # Key norms grow along the sequence, so later tiles keep exceeding the reference maxima by more
    # than the lazy threshold and O^T / l^T are rescaled in TMEM several times; sessions also start
    # their window at a position that is not a multiple of the tile.
    r = np.random.default_rng(502)
    lens = [2300, 1111, 700]
    got, want = _verify_batch(r, 32, 2, 4, lens, kv_start=[0, 77, 301], k_gain=lambda t: 1.0 + t / 150.0, scale=0.0625)
    for i in range(len(lens)):
        assert np.abs(got[i] - want[i]).max() <= TOL, (i, np.abs(got[i] - want[i]).max())


def test_verify_tensor_core_agrees_with_mma_sync_path(monkeypatch):
    # Two independent CUDA kernels on the same batch at a size the oracle would take minutes for:
    # the tcgen05 pass and (forced by the A/B switch) the mma.sync pass that serves 16 rows at a time.
    r = np.random.default_rng(503)
    n, hq, hkv, hd, q_rows = 6, 32, 2, 256, 4
    lens = [16384 + 3, 9000, 12001, 300, 16000, 7777]
    cap, stride, kbuf, vbuf, q = _batched_case(r, n, hq, hkv, hd, lens, q_rows)
    kd, vd, qd = dev(kbuf), dev(vbuf), dev(q)
    outs = []
    for force in (False, True):
        if force:
            monkeypatch.setenv("TT_VERIFY_FORCE_MMA_SYNC", "1")
        out = torch.full((n, q_rows, hq * hd), float("nan"), device="cuda", dtype=torch.float16)
        sessions = [tt.DecodeSession(qd, out, kd, vd, lens[i], q_rows, 0, q_offset=i * q_rows * hq * hd * 2,
                                     out_offset=i * q_rows * hq * hd * 2, k_offset=i * cap * stride * 2,
                                     v_offset=i * cap * stride * 2) for i in range(n)]
        launches = context().launch_count
        tt.Attention(context()).encode_batched(sessions, hd, hq, hkv, scale=0.0625)
        torch.cuda.synchronize()
        assert context().poll_status() == 0
        assert context().launch_count - launches in (1, 2)   # pass 1, and the merge unless every session is one part
        outs.append(host(out))
    assert np.isfinite(outs[0]).all()
    assert np.abs(outs[0] - outs[1]).max() <= 2 * TOL
    assert not np.array_equal(outs[0], outs[1])   # different kernels: agreement to rounding, not by construction


def test_verify_tensor_core_single_part_writes_outputs_directly():
    # Contexts that fit one part each: the tensor-core pass normalises and stores the rows itself
    # (one launch, no merge pass); rows with a single visible key and a padded output stride included.
    r = np.random.default_rng(504)
    lens = [500, 300, 4, 129]
    launches = context().launch_count
    got, want = _verify_batch(r, 32, 2, 4, lens)
    assert context().launch_count - launches == 1
    for i in range(len(lens)):
        assert np.abs(got[i] - want[i]).max() <= TOL, (i, np.abs(got[i] - want[i]).max())


def test_exchange_wait_runs_out_and_reports_timeout():
    # The cross-GPU merge waits for every rank's flag with a poll limit. Here "rank 1" never
    # publishes (both exchange buffers are plain local allocations of this one GPU and nothing ever
    # writes rank 1's flag), the limit is tiny, so the wait gives up: the kernel returns, the status
    # word reads TT_ERR_TIMEOUT on the host and the output row is left untouched. A context of its
    # own, so the suite's shared context keeps a clean status word.
    import ctypes as C
    from tinytitan_b200 import _lib as L
    ctx = tt.Context(0)
    try:
        ctx.set_exchange_poll_limit(1000)
        hq, hd, world = 4, 128, 2
        nbytes = L.lib().tt_attn_exchange_bytes(world, hq, hd)
        bufs = [torch.zeros(nbytes + 256, device="cuda", dtype=torch.uint8) for _ in range(world)]
        ptrs = (C.c_void_p * world)(*[(b.data_ptr() + 255) // 256 * 256 for b in bufs])
        m = torch.zeros(hq, device="cuda"); d = torch.ones(hq, device="cuda"); o = torch.ones(hq, hd, device="cuda")
        out = torch.full((hq, hd), 7.0, device="cuda", dtype=torch.float16)
        stream = torch.cuda.current_stream().cuda_stream
        ctx.check(L.lib().tt_attn_exchange_combine(ctx.handle, stream, m.data_ptr(), d.data_ptr(), o.data_ptr(), ptrs, 0,
                                                   world, hq, hd, 1, out.data_ptr(), tt.TT_F16))
        flags = C.c_uint32(0)
        rc = L.lib().tt_ctx_poll_status(ctx.handle, stream, C.byref(flags))
        assert rc == L.TT_ERR_TIMEOUT and flags.value & 1
        assert torch.all(out == 7.0)
    finally:
        ctx.close()
