"""The sparse-attention block indexer and prefill attention over a key selection on B200."""
import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from gpu_util import TOL, context, dev, host, rounded

pytestmark = pytest.mark.gpu
CFG = tt.SparseIndexerConfig(num_heads=4, head_dim=128, budget=64, compress_ratio=4)   # QSAIndexerTests.swift:17-19


def select(indexer, scores_rows, start, keep_stride=None, index_stride=None):
    """Runs tt_qsa_select_keys on [rows, blocks] scores; returns (keep [rows, stride], indices, counts)."""
    rows, stride = scores_rows.shape
    ks = keep_stride or (start + rows)
    ix = index_stride or indexer.selection_width
    keep = torch.full((rows, ks), 9, device="cuda", dtype=torch.uint8)
    idx = torch.full((rows, ix), 0xFFFFFFF, device="cuda", dtype=torch.int32)
    cnt = torch.zeros(rows, device="cuda", dtype=torch.int32)
    indexer.encode_select_keys(dev(scores_rows, torch.float32), stride, start, rows, keep, ks, idx, ix, cnt)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    return keep.cpu().numpy(), idx.cpu().numpy().astype(np.int64), cnt.cpu().numpy()


def check_rows(indexer, scores_rows, start):
    keep, idx, cnt = select(indexer, scores_rows, start)
    width, ratio = indexer.selection_width, indexer.compress_ratio
    for r in range(scores_rows.shape[0]):
        visible = start + r + 1
        want_keep, want_idx = oracle.qsa_select_keys(scores_rows[r], visible, ratio, width)
        assert np.array_equal(keep[r, :visible], want_keep), (r, visible)
        assert not keep[r, visible:].any()
        assert cnt[r] == len(want_idx) and np.array_equal(idx[r, :cnt[r]], want_idx), (r, visible)
    return keep, idx, cnt


def test_reference_selection_cases():
    # the four cases of tests/TinyTitan/Kernels/Attention/QSAIndexerTests.swift, same scores
    ix = tt.QSAIndexer(context(), CFG)
    assert ix.selection_width == 67
    keep, idx, cnt = check_rows(ix, np.zeros((1, 17), np.float32), 66)        # 67 visible: inside the window
    assert keep[0].all() and cnt[0] == 67
    keep, _, cnt = check_rows(ix, np.zeros((1, 18), np.float32), 67)          # 68 visible: a real selection
    assert keep[0].sum() == 67
    keep, _, cnt = check_rows(ix, np.full((1, 26), 1000, np.float32), 102)    # 103 visible: tail cells 100..102 survive
    assert keep[0, 100] and keep[0, 101] and keep[0, 102] and cnt[0] == 67
    scores = np.zeros((1, 18), np.float32); scores[0, :17] = 17 - np.arange(17)
    keep, _, _ = check_rows(ix, scores, 67)                                   # the budget cuts block 16 after 3 cells
    assert keep[0, 64] and keep[0, 66] and not keep[0, 67] and keep[0].sum() == 67
    keep, idx, cnt = check_rows(ix, np.full((1, 19), 5, np.float32), 71)      # ties go to the lower block index
    assert idx[0, 0] == 0 and idx[0, cnt[0] - 1] == 66


def test_selection_of_a_prefill_chunk_with_ties_and_signed_zeros():
    # every row of a chunk at once (selectKeysPrefill): rows inside the dense window, rows past it,
    # heavy ties (scores drawn from five values) and both zeros
    r = np.random.default_rng(5)
    ix = tt.QSAIndexer(context(), CFG)
    start, rows = 40, 300
    blocks = (start + rows) // CFG.compress_ratio + 1
    scores = r.choice(np.array([0.0, -0.0, 1.5, 1.5, 7.25, 0.125], np.float32), size=(rows, blocks))
    check_rows(ix, scores, start)
    scores = r.normal(size=(rows, blocks)).astype(np.float32)
    check_rows(ix, np.maximum(scores, 0), start)


def test_selection_at_production_geometry_long_context():
    # budget 2048, ratio 4 (ModelTypes.swift:131-132) at 100,003 visible keys: 25,000 scored blocks
    big = tt.QSAIndexer(context(), tt.SparseIndexerConfig(4, 128, 2048, 4))
    r = np.random.default_rng(6)
    visible = 100003
    scores = np.maximum(r.normal(size=(2, visible // 4 + 1)), 0).astype(np.float32)
    keep, idx, cnt = check_rows(big, scores, visible - 2)
    assert cnt[1] == big.selection_width and keep[1].sum() == big.selection_width
    assert np.all(np.diff(idx[1, :cnt[1]]) > 0)


def test_pool_norm_rope_matches_oracle():
    r = np.random.default_rng(7)
    d, ratio, n_kv = 128, 4, 1003
    ix = tt.QSAIndexer(context(), tt.SparseIndexerConfig(4, d, 2048, ratio))
    raw = rounded(r.normal(size=(n_kv, d)))
    w = rounded(r.uniform(0.5, 1.5, size=d), torch.bfloat16)
    blocks = (n_kv + ratio - 1) // ratio
    pooled = torch.full((blocks + 1, d), float("nan"), device="cuda", dtype=torch.float16)
    ix.encode_pool_prefill(dev(raw), pooled, 0, n_kv, dev(w, torch.bfloat16))
    torch.cuda.synchronize()
    got = host(pooled)
    want = oracle.qsa_pool_blocks(raw, ratio, n_kv, 0, blocks, w, 1e-6, 1e7)
    for b in (0, 1, 57, blocks - 2, blocks - 1):                  # the last block has 3 of 4 members
        assert np.abs(got[b] - want[b]).max() <= TOL + np.abs(want[b]).max() * 2.0 ** -9, b
    assert np.isnan(got[blocks]).all()                            # nothing past the last block is written
    # pooling alone (no norm weight): the mean, bit for bit after the fp16 store
    plain = torch.zeros((blocks, d), device="cuda", dtype=torch.float16)
    ix.encode_pool(dev(raw), plain, 0, blocks, n_kv)
    torch.cuda.synchronize()
    want_plain = oracle.qsa_pool_blocks(raw, ratio, n_kv, 0, blocks)
    assert np.array_equal(host(plain)[blocks - 1], want_plain[blocks - 1])
    assert np.abs(host(plain)[3] - want_plain[3]).max() <= 2.0 ** -10 * np.abs(want_plain[3]).max()
    # a decode step repools only the block the new token joined
    one = pooled.clone()
    raw2 = raw.copy(); raw2[n_kv - 1] = rounded(r.normal(size=d))
    ix.encode_append_key(dev(raw2), one, n_kv - 1, dev(w, torch.bfloat16))
    torch.cuda.synchronize()
    assert torch.equal(one[:blocks - 1], pooled[:blocks - 1]) and not torch.equal(one[blocks - 1], pooled[blocks - 1])


def test_query_norm_rope_and_block_scores_match_oracle():
    r = np.random.default_rng(8)
    d, h, rows, blocks, pos = 128, 4, 37, 1500, 2900
    ix = tt.QSAIndexer(context(), tt.SparseIndexerConfig(h, d, 2048, 4))
    q = rounded(r.normal(size=(rows, h, d)))
    w = rounded(r.uniform(0.5, 1.5, size=d), torch.bfloat16)
    qd = dev(q)
    ix.encode_query(qd, rows, pos, dev(w, torch.bfloat16))
    torch.cuda.synchronize()
    got_q = host(qd)
    for t in (0, 17, rows - 1):
        for head in range(h):
            want = oracle.attn_norm_rope(q[t, head], w, 1e-6, d, 1e7, pos + t)
            assert np.abs(got_q[t, head] - want).max() <= TOL + np.abs(want).max() * 2.0 ** -9
    pooled = rounded(r.normal(size=(blocks, d)))
    scores = torch.full((rows, blocks + 3), float("nan"), device="cuda")
    ix.encode_scores(qd, dev(pooled), scores, blocks, rows=rows, score_stride=blocks + 3)
    torch.cuda.synchronize()
    want = oracle.qsa_block_scores(got_q, pooled)
    got = scores.cpu().numpy()
    assert np.abs(got[:, :blocks] - want).max() <= 1e-3 * max(1.0, np.abs(want).max())
    assert np.isnan(got[:, blocks:]).all()


def _prefill_case(r, t_count, start, hq, hkv, hd, extra_rows=0):
    kv_valid = start + t_count
    q = rounded(r.normal(size=(t_count, hq * hd)))
    k = rounded(r.normal(size=(kv_valid + extra_rows, hkv * hd)))
    v = rounded(r.normal(size=(kv_valid + extra_rows, hkv * hd)))
    p = tt.PrefillAttentionParams(start, t_count, hd, hq, hkv, kv_valid, 0, hkv * hd, hq * hd, hq * hd, 0.0625)
    return q, k, v, p


@pytest.mark.parametrize("hd,hq,hkv", [(256, 16, 2), (64, 4, 1)])
def test_prefill_over_a_selection_mask_and_compact_forms_agree_with_oracle(hd, hq, hkv):
    # A chunk of 48 queries at positions 300..347 with the indexer's own selection (budget 64): the
    # byte mask and the compact list are the same selection, so the two calls must agree with the
    # oracle and with each other (PrefillAttention.swift:206-218).
    r = np.random.default_rng(hd)
    start, t_count = 300, 48
    q, k, v, p = _prefill_case(r, t_count, start, hq, hkv, hd)
    ix = tt.QSAIndexer(context(), CFG)
    blocks = (start + t_count) // CFG.compress_ratio + 1
    scores = np.maximum(r.normal(size=(t_count, blocks)), 0).astype(np.float32)
    keep, idx, cnt = select(ix, scores, start)
    keys_of_row = [idx[t, :cnt[t]] for t in range(t_count)]
    want = oracle.attn_prefill_selected(q, k, v, hd, hq, hkv, start, start + t_count, 0, 0.0625, keys_of_row)
    pa = tt.PrefillAttention(context())
    qd, kd, vd = dev(q), dev(k), dev(v)
    keep_d = torch.as_tensor(keep).cuda(); idx_d = torch.as_tensor(idx.astype(np.int32)).cuda(); cnt_d = torch.as_tensor(cnt).cuda()
    outs = []
    for kwargs in (dict(keep_mask=keep_d, keep_stride=keep.shape[1]),
                   dict(keep_mask=keep_d, keep_stride=keep.shape[1], keep_indices=idx_d, keep_index_stride=idx.shape[1],
                        keep_counts=cnt_d)):
        o = torch.full((t_count, hq * hd), float("nan"), device="cuda", dtype=torch.float16)
        pa.encode_causal(qd, kd, vd, o, p, **kwargs)
        torch.cuda.synchronize()
        assert context().poll_status() == 0
        got = host(o).reshape(t_count, hq, hd)
        assert np.abs(got - want).max() <= TOL
        outs.append(got)
    assert np.abs(outs[0] - outs[1]).max() <= 1e-3
    # the selection matters: dense attention over all keys is a different result
    dense = oracle.attn_prefill(q, k, v, hq * hd, hkv * hd, hd, hq, hkv, start, t_count, start + t_count, 0, 0.0625)
    assert np.abs(dense - want).max() > 1e-2


def test_prefill_over_window_rows_and_dropped_entries():
    # useKeep == 3: the list holds logical keys, a parallel list the cache rows that hold them (a
    # shuffled window); entries beyond a row's own position are dropped, a row with nothing visible
    # in its list is written as zeros (prefill.metal:967-985, :1051-1053).
    r = np.random.default_rng(11)
    hd, hq, hkv, start, t_count = 128, 8, 2, 90, 12
    kv_valid = start + t_count
    q, k_logical, v_logical, p = _prefill_case(r, t_count, start, hq, hkv, hd)
    window_rows = 150
    perm = r.permutation(window_rows)[:kv_valid]                 # logical key j lives in window row perm[j]
    k_win = np.zeros((window_rows, hkv * hd), np.float32); v_win = np.zeros_like(k_win)
    k_win[perm] = k_logical; v_win[perm] = v_logical
    stride = 40
    idx = np.zeros((t_count, stride), np.int64); cnt = np.zeros(t_count, np.int32)
    for t in range(t_count):
        n = 30 + t % 5
        chosen = np.sort(r.choice(kv_valid, size=n, replace=False))   # some lie beyond position start + t: dropped
        idx[t, :n] = chosen; cnt[t] = n
    idx[3, :cnt[3]] = np.arange(kv_valid - cnt[3], kv_valid)[::1]     # row 3 (position 93): mostly future keys
    idx[5, :cnt[5]] = kv_valid - 1; cnt[5] = 4                        # row 5: only a future key -> zeros
    rows = perm[idx]
    keys_of_row = [idx[t, :cnt[t]] for t in range(t_count)]
    want = oracle.attn_prefill_selected(q, k_logical, v_logical, hd, hq, hkv, start, kv_valid, 0, 0.0625, keys_of_row)
    o = torch.full((t_count, hq * hd), float("nan"), device="cuda", dtype=torch.float16)
    tt.PrefillAttention(context()).encode_causal(
        dev(q), dev(k_win), dev(v_win), o, p, keep_indices=torch.as_tensor(idx.astype(np.int32)).cuda(),
        keep_index_stride=stride, keep_counts=torch.as_tensor(cnt).cuda(), keep_rows=torch.as_tensor(rows.astype(np.int32)).cuda())
    torch.cuda.synchronize()
    got = host(o).reshape(t_count, hq, hd)
    assert np.abs(got - want).max() <= TOL
    assert np.all(got[5] == 0) and np.all(want[5] == 0)


def test_host_kv_window_matches_contiguous_attention_over_the_same_selection():
    # HostKVStreamingTests.swift:243-330 on device memory: a 64-row window over a 3000-token context;
    # at a few positions a sparse selection read through the window (tt_attn_decode_window with the
    # rows prepareDecodeWindow returned) equals contiguous attention under the same keep mask.
    from gpu_util import device_view
    r = np.random.default_rng(21)
    hq, hkv, hd, max_context, window = 8, 2, 128, 3000, 64
    stride = hkv * hd * 2
    kd = dev(r.normal(size=(max_context, hkv * hd))); vd = dev(r.normal(size=(max_context, hkv * hd)))
    w = tt.KVWindow(1, stride, max_context, window)
    attn = tt.Attention(context())
    q = dev(r.normal(size=(hq, hd)))
    wk, wv = w.base(0)
    win_k = device_view(wk, window * hkv * hd, torch.float16); win_v = device_view(wv, window * hkv * hd, torch.float16)
    checked = {65, 700, 2999}
    for position in range(max_context):
        pk, pv = w.write_slot(0, position)
        device_view(pk, hkv * hd, torch.float16).copy_(kd[position]); device_view(pv, hkv * hd, torch.float16).copy_(vd[position])
        if position in checked:
            keys = sorted({0, position} | set(range(0, position + 1, 512)) | set(range(max(0, position - 7), position + 1)))
            mask = np.zeros(position + 1, np.uint8); mask[keys] = 1
            a = torch.empty(hq, hd, device="cuda", dtype=torch.float16); b = torch.empty_like(a)
            attn.encode_full(q, kd, vd, a, hd, hq, hkv, position + 1, scale=0.09, keep_mask=torch.as_tensor(mask).cuda())
            torch.cuda.synchronize()
            idx, rows = w.prepare_decode_window(0, position, np.array(keys, np.uint32))
            attn.encode_window(q, win_k, win_v, b, hd, hq, hkv, torch.as_tensor(rows.astype(np.int32)).cuda(), len(keys), scale=0.09)
            torch.cuda.synchronize()
            want = oracle.attn_decode(host(q), host(kd)[keys].reshape(-1, hkv, hd), host(vd)[keys].reshape(-1, hkv, hd), hkv, 0.09)
            assert np.abs(host(b) - want).max() <= TOL and np.abs(host(a) - host(b)).max() <= 1e-3
        torch.cuda.synchronize()
        w.commit(position, 1)
    # the arena holds every row although the window was recycled dozens of times
    for position in (0, 64, 1234, 2999):
        got = np.frombuffer(w.host_row(0, position, True), np.float16)
        assert np.array_equal(got, kd[position].cpu().numpy())
    assert w.window_bytes == 2 * window * stride
    w.close()
