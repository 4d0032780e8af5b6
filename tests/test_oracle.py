"""The CPU oracle against the reference's golden outputs and known-answer cases (no GPU)."""
import os

import numpy as np
import pytest

import oracle
from oracle.prng import SplitMix64, seed_tree_key, LCG
import make_golden as mg

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_splitmix64_known_sequence():
    # First outputs of SplitMix64(seed=0) are a published known-answer sequence.
    g = SplitMix64(0)
    assert [g.next() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    # FNV-1a offset basis: an empty label leaves the root XORed with the basis.
    assert seed_tree_key(0, "").state == 0xCBF29CE484222325
    u = seed_tree_key(0x174, "attn-h8-kv1-d64-T128-kv=false").uniform(-0.5, 0.5)
    assert -0.5 <= float(u) < 0.5


def test_lcg_range():
    vals = LCG(0x55AA1234).array(1000)
    assert vals.min() >= -1.0 and vals.max() <= 1.0
    assert len(np.unique(vals)) > 300


def test_delta_rule_matches_reference_golden():
    c = mg.lcg_delta_rule_inputs()
    gold = np.load(os.path.join(GOLD, "delta_rule_lcg.npz"))
    ro, st = oracle.delta_rule(c["query"], c["key"], c["value"], c["a"], c["b"], c["decay_log"],
                               c["decay_bias"], c["key_heads"], c["inverse"], c["state"])
    # the reference's own bar for this case is 1e-5 (CPUBatchedPrefillTests.swift:242)
    assert np.abs(ro - gold["readout"]).max() < 1e-6
    assert np.abs(st - gold["state"]).max() < 1e-6


@pytest.mark.parametrize("tokens", [8, 16, 32])
def test_chunk_rule_matches_reference_golden(tokens):
    c = mg.lcg_chunk_inputs(tokens)
    gold = np.load(os.path.join(GOLD, "delta_chunk_lcg.npz"))
    ro, st = oracle.delta_rule_chunk(c["queries"], c["keys"], c["values"], c["alphas"], c["betas"],
                                     np.zeros((4, 8), np.float32))
    assert np.abs(ro - gold[f"chunk_readout_{tokens}"]).max() < 1e-6
    assert np.abs(st - gold[f"chunk_state_{tokens}"]).max() < 1e-6
    # the reference's own test: chunked vs token kernel < 1e-4 (CPUBatchedPrefillTests.swift:320)
    assert np.abs(ro - gold[f"token_readout_{tokens}"]).max() < 1e-4
    assert np.abs(st - gold[f"token_state_{tokens}"]).max() < 1e-4


@pytest.mark.parametrize("chunk", [16, 64])
def test_chunk_algebra_matches_python_spec(chunk):
    # Inputs as benchmark/gdn_chunked_scan.py:46-55 draws them (default_rng(7)).
    r = np.random.default_rng(7)
    state = r.normal(size=(8, 8)); keys = r.normal(size=(chunk, 8)); values = r.normal(size=(chunk, 8))
    queries = r.normal(size=(chunk, 8)); alphas = r.uniform(0.5, 1.0, size=chunk)
    betas = r.uniform(0.1, 0.9, size=chunk)
    gold = np.load(os.path.join(GOLD, "chunk_algebra.npz"))
    ro, st = oracle.delta_rule_chunk(queries, keys, values, alphas, betas, state)
    scale = max(1.0, np.abs(gold[f"scalar_readouts_{chunk}"]).max())
    assert np.abs(ro - gold[f"scalar_readouts_{chunk}"]).max() < 2e-5 * scale
    assert np.abs(st - gold[f"scalar_state_{chunk}"]).max() < 2e-5 * max(1.0, np.abs(gold[f"scalar_state_{chunk}"]).max())
    assert np.abs(gold[f"scalar_readouts_{chunk}"] - gold[f"chunked_readouts_{chunk}"]).max() < 1e-9 * scale * 100


def test_delta_rule_d128_golden():
    c = mg.d128_inputs()
    gold = np.load(os.path.join(GOLD, "delta_rule_d128.npz"))
    state = c["state"].copy()
    for t in range(c["value"].shape[0]):
        ro, state = oracle.delta_rule(c["query"][t], c["key"][t], c["value"][t], c["a"][t], c["b"][t],
                                      c["decay_log"], c["decay_bias"], c["key_heads"], c["inverse"], state)
        assert np.abs(ro - gold["readout"][t]).max() < 1e-5
    assert np.abs(state[0, :4] - gold["state_head0_rows"]).max() < 1e-5
    assert abs(state.astype(np.float64).sum() - gold["state_checksum"][0]) < 1e-2


@pytest.mark.skipif(oracle.ref() is None, reason="oracle/_ref not built")
def test_restatement_equals_compiled_reference_random():
    r = np.random.default_rng(3)
    for heads, kh, dk, dv in [(4, 2, 16, 8), (6, 3, 32, 32), (2, 2, 128, 128)]:
        q = r.normal(size=(kh, dk)); k = r.normal(size=(kh, dk)); v = r.normal(size=(heads, dv))
        a = r.normal(size=heads); b = r.normal(size=heads)
        dl = r.uniform(-1, 1, size=heads); db = r.uniform(-0.5, 0.5, size=heads)
        st = 0.1 * r.normal(size=(heads, dv, dk))
        got = oracle.delta_rule(q, k, v, a, b, dl, db, kh, 0.5, st)
        want = oracle.ref_delta_rule(q, k, v, a, b, dl, db, kh, 0.5, st)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    T, dk, dv = 24, 16, 8
    q = r.normal(size=(T, dk)); k = r.normal(size=(T, dk)) / 4; v = r.normal(size=(T, dv))
    al = r.uniform(0.5, 1, size=T); be = r.uniform(0.1, 0.9, size=T); st = r.normal(size=(dv, dk))
    got = oracle.delta_rule_chunk(q, k, v, al, be, st)
    want = oracle.ref_delta_rule_chunk(q, k, v, al, be, st)
    assert np.abs(got[0] - want[0]).max() < 1e-5 and np.abs(got[1] - want[1]).max() < 1e-5


def test_gdn_gpu_form_equals_cpu_form():
    # The kernel form (conv_out row, softplus shortcut) and the CPU-engine form agree when the
    # readout scale is folded the same way (Dk == Dv).
    r = np.random.default_rng(11)
    hk, hv, d, rows = 2, 4, 32, 3
    conv = r.normal(size=(rows, 2 * hk * d + hv * d)).astype(np.float32)
    a = r.normal(size=(rows, hv)); b = r.normal(size=(rows, hv))
    a_log = r.uniform(-1, 1.5, size=hv); dtb = r.uniform(-0.5, 0.5, size=hv)
    st0 = (0.1 * r.normal(size=(hv, d, d))).astype(np.float32)
    y, st, ck = oracle.gdn_step_rows(conv, a, b, a_log, dtb, hk, hv, d, d, st0, want_checkpoint=True)
    state = st0.copy()
    for t in range(rows):
        q = conv[t, :hk * d]; k = conv[t, hk * d:2 * hk * d]; v = conv[t, 2 * hk * d:].reshape(hv, d)
        ro, state = oracle.delta_rule(q, k, v, a[t], b[t], a_log, dtb, hk, 1.0, state)
        assert np.abs(ro.ravel() - y[t]).max() < 1e-4
        if t == 0:
            assert np.abs(ck - state).max() < 1e-5
    assert np.abs(st - state).max() < 1e-4


def _reference_attention_case(root, label, hd, hq, hkv, s, aliased=False):
    g = seed_tree_key(root, label)
    q = g.uniform_array(hq * hd, -0.5, 0.5).astype(np.float16).astype(np.float32).reshape(hq, hd)
    k = g.uniform_array(s * hkv * hd, -0.5, 0.5).astype(np.float16).astype(np.float32).reshape(s, hkv, hd)
    v = k if aliased else g.uniform_array(s * hkv * hd, -0.5, 0.5).astype(np.float16).astype(np.float32).reshape(s, hkv, hd)
    return q, k, v


@pytest.mark.parametrize("root,label,hd,hq,hkv,s,aliased", [
    (0x174, "attn-h8-kv1-d64-T128-kv=false", 64, 8, 1, 128, False),
    (0x175, "attn-h16-kv2-d256-T128-kv=false", 256, 16, 2, 128, False),
    (0x176, "attn-h8-kv1-d64-T128-kv=true", 64, 8, 1, 128, True),
])
def test_attention_two_statements_agree(root, label, hd, hq, hkv, s, aliased):
    # Seeded cases of tests/TinyTitan/Kernels/Attention/AttentionTests.swift:399-425; the
    # materialised-softmax reference and the split/merge kernel form must agree (reference bar
    # rel < 1e-2; fp32 forms agree far tighter).
    q, k, v = _reference_attention_case(root, label, hd, hq, hkv, s, aliased)
    scale = 1.0 / np.sqrt(hd)
    full = oracle.attn_decode(q, k, v, hkv, scale)
    for chunks in (1, 16, 64):
        split = oracle.attn_decode_split(q, k, v, hkv, scale, s, n_chunks=chunks)
        assert np.abs(full - split).max() < 2e-6
    win = oracle.attn_decode(q, k, v, hkv, scale, window=64)
    split = oracle.attn_decode_split(q, k, v, hkv, scale, s, kv_start=s - 64)
    assert np.abs(win - split).max() < 2e-6
    eng = oracle.cpu_engine_attention(q, k.reshape(s, -1), v.reshape(s, -1), hkv, scale)
    assert np.abs(full - eng).max() < 2e-6


def test_attention_edges():
    r = np.random.default_rng(5)
    q = r.normal(size=(4, 32)).astype(np.float32); k = r.normal(size=(40, 2, 32)).astype(np.float32)
    v = r.normal(size=(40, 2, 32)).astype(np.float32)
    # all keys masked -> zero row (attention.metal:418-424)
    out = oracle.attn_decode_split(q, k, v, 2, 0.2, 40, keep=np.zeros(40, np.uint8))
    assert np.all(out == 0)
    # empty range
    out = oracle.attn_decode_split(q, k, v, 2, 0.2, 7, kv_start=7)
    assert np.all(out == 0)
    # keep mask == dropping the keys
    keep = (r.uniform(size=40) < 0.5).astype(np.uint8); keep[-1] = 1
    got = oracle.attn_decode_split(q, k, v, 2, 0.2, 40, keep=keep, n_chunks=16)
    idx = np.nonzero(keep)[0]
    want = oracle.attn_decode(q, k[idx], v[idx], 2, 0.2)
    assert np.abs(got - want).max() < 2e-6
    # ring: logical position p lives at row p % cap
    cap = 16
    ring_k = np.zeros((cap, 2, 32), np.float32); ring_v = np.zeros((cap, 2, 32), np.float32)
    for p in range(40):
        ring_k[p % cap] = k[p]; ring_v[p % cap] = v[p]
    got = oracle.attn_decode_split(q, ring_k, ring_v, 2, 0.2, 40, kv_start=40 - cap, ring_capacity=cap)
    want = oracle.attn_decode(q, k, v, 2, 0.2, window=cap)
    assert np.abs(got - want).max() < 2e-6


def test_prefill_reference_vs_decode_reference():
    r = np.random.default_rng(9)
    hd, hq, hkv, start, chunk = 32, 4, 2, 5, 7
    kv_valid = start + chunk
    qs, kvs = hq * hd + 3, hkv * hd + 5
    q = r.normal(size=(chunk, qs)).astype(np.float32)
    k = r.normal(size=(kv_valid, kvs)).astype(np.float32); v = r.normal(size=(kv_valid, kvs)).astype(np.float32)
    out = oracle.attn_prefill(q, k, v, qs, kvs, hd, hq, hkv, start, chunk, kv_valid, 0, 0.3)
    for t in range(chunk):
        n = start + t + 1
        want = oracle.attn_decode(q[t, :hq * hd].reshape(hq, hd), k[:n, :hkv * hd].reshape(n, hkv, hd),
                                  v[:n, :hkv * hd].reshape(n, hkv, hd), hkv, 0.3)
        assert np.abs(out[t] - want).max() < 2e-6
    # sliding window
    out = oracle.attn_prefill(q, k, v, qs, kvs, hd, hq, hkv, start, chunk, kv_valid, 4, 0.3)
    t = 3; n = start + t + 1
    want = oracle.attn_decode(q[t, :hq * hd].reshape(hq, hd), k[:n, :hkv * hd].reshape(n, hkv, hd),
                              v[:n, :hkv * hd].reshape(n, hkv, hd), hkv, 0.3, window=4)
    assert np.abs(out[t] - want).max() < 2e-6
    # CPU-engine batched form
    eng = oracle.cpu_engine_attention_batch(q[:, :hq * hd].reshape(chunk, hq, hd), k[:, :hkv * hd].copy(),
                                            v[:, :hkv * hd].copy(), hkv, start, 0.3)
    full = oracle.attn_prefill(q, k, v, qs, kvs, hd, hq, hkv, start, chunk, kv_valid, 0, 0.3)
    assert np.abs(eng - full).max() < 2e-6


def test_threaded_drivers_equal_serial():
    r = np.random.default_rng(21)
    T, hk, hv, d = 40, 2, 4, 16
    q = r.normal(size=(T, hk * d)) / 4; k = r.normal(size=(T, hk * d)) / 4; v = r.normal(size=(T, hv * d))
    al = r.uniform(0.5, 1, size=(T, hv)); be = r.uniform(0.1, 0.9, size=(T, hv)); st = r.normal(size=(hv, d, d)) * 0.1
    y1, s1 = oracle.gdn_scan_heads(q, k, v, al, be, hk, hv, d, d, 8, st, threads=1)
    y4, s4 = oracle.gdn_scan_heads(q, k, v, al, be, hk, hv, d, d, 8, st, threads=4)
    assert np.array_equal(y1, y4) and np.array_equal(s1, s4)
    y64, s64 = oracle.gdn_scan_heads(q, k, v, al, be, hk, hv, d, d, 64, st, threads=2)
    assert np.abs(y1 - y64).max() < 1e-4
    if oracle.ref() is not None:
        yr, sr = oracle.gdn_scan_heads(q, k, v, al, be, hk, hv, d, d, 8, st, threads=2, use_ref=True)
        assert np.abs(y1 - yr).max() < 1e-5
