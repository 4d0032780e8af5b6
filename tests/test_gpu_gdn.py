"""Gated delta rule (decode step, sequential rows, batched sessions) against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
import make_golden as mg
from gpu_util import TOL, context, dev, host, rounded, device_view

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _unit(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def make_inputs(r, rows, hk, hv, dk, dv, extra_stride=0):
    """conv_out rows [q | k | v] with q,k L2-normalised per head (q additionally * dk^-0.5, the
    folded scale of gdn.metal:466-521), fp16-rounded; a,b fp16; A_log, dt_bias bf16."""
    q = _unit(r.normal(size=(rows, hk, dk))) / np.sqrt(dk)
    k = _unit(r.normal(size=(rows, hk, dk)))
    v = r.normal(size=(rows, hv, dv))
    conv = np.concatenate([q.reshape(rows, -1), k.reshape(rows, -1), v.reshape(rows, -1),
                           np.zeros((rows, extra_stride))], axis=1)
    conv = rounded(conv)
    a = rounded(r.normal(size=(rows, hv))); b = rounded(r.normal(size=(rows, hv)))
    a_log = rounded(r.uniform(-1, 1.5, size=hv), torch.bfloat16)
    dt_bias = rounded(r.uniform(-0.5, 0.5, size=hv), torch.bfloat16)
    state = (0.02 * r.normal(size=(hv, dv, dk))).astype(np.float32)
    return conv, a, b, a_log, dt_bias, state


def run_step(cfg, conv, a, b, a_log, dt_bias, state, rows, checkpoint=False, **gdn_kw):
    gdn = tt.GDN(context(), cfg, **gdn_kw)
    conv_d, a_d, b_d = dev(conv), dev(a), dev(b)
    al_d, dt_d = dev(a_log, torch.bfloat16), dev(dt_bias, torch.bfloat16)
    st_d = dev(state, torch.float32)
    y = torch.full((rows, cfg.value_dim), float("nan"), device="cuda", dtype=torch.float16)
    ck = torch.zeros_like(st_d) if checkpoint else None
    gdn.encode_delta_step_prefill(conv_d, a_d, b_d, al_d, dt_d, st_d, y, rows, checkpoint_state=ck,
                                  row_stride=conv.shape[1])
    torch.cuda.synchronize()
    return host(y), host(st_d), (host(ck) if ck is not None else None)


@pytest.mark.parametrize("hk,hv,dk,dv,rows", [(16, 16, 128, 128, 1), (16, 32, 128, 128, 1), (2, 4, 32, 32, 6),
                                               (16, 64, 128, 128, 4), (4, 8, 64, 72, 3)])
def test_step_matches_oracle(hk, hv, dk, dv, rows):
    r = np.random.default_rng(hv * 100 + rows)
    cfg = tt.LinearAttentionConfig(hk, hv, dk, dv)
    conv, a, b, a_log, dt_bias, state = make_inputs(r, rows, hk, hv, dk, dv, extra_stride=4)
    want_y, want_s, want_ck = oracle.gdn_step_rows(conv, a, b, a_log, dt_bias, hk, hv, dk, dv, state,
                                                   want_checkpoint=True)
    got_y, got_s, got_ck = run_step(cfg, conv, a, b, a_log, dt_bias, state, rows, checkpoint=True)
    assert np.abs(got_y - want_y).max() <= TOL
    assert np.abs(got_s - want_s).max() <= 1e-5
    assert np.abs(got_ck - want_ck).max() <= 1e-5


def test_prefill_rows_equal_sequential_decode_bitwise():
    # tests/TinyTitan/Kernels/GDN/GDNKernelTests.swift:279-392: the multi-row kernel must be
    # bit-identical (y and state) to decode steps applied one after another.
    r = np.random.default_rng(42)
    hk, hv, d, rows = 16, 32, 128, 5
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, a, b, a_log, dt_bias, state = make_inputs(r, rows, hk, hv, d, d)
    y_all, s_all, _ = run_step(cfg, conv, a, b, a_log, dt_bias, state, rows)
    s = state
    for t in range(rows):
        y1, s, _ = run_step(cfg, conv[t:t + 1], a[t:t + 1], b[t:t + 1], a_log, dt_bias, s, 1)
        assert np.array_equal(y1[0], y_all[t])
    assert np.array_equal(s, s_all)


def test_storage_conventions():
    # GDNStorageConvention.swift:7-25: pre-exponentiated A and tiled value heads
    r = np.random.default_rng(8)
    hk, hv, d = 4, 8, 64
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, a, b, a_log, dt_bias, state = make_inputs(r, 2, hk, hv, d, d)
    pre = rounded(-np.exp(a_log), torch.bfloat16)
    want_y, want_s, _ = oracle.gdn_step_rows(conv, a, b, pre, dt_bias, hk, hv, d, d, state, a_preexp=True, v_tiled=True)
    got_y, got_s, _ = run_step(cfg, conv, a, b, pre, dt_bias, state, 2, a_log_preexp=True, v_tiled=True)
    assert np.abs(got_y - want_y).max() <= TOL and np.abs(got_s - want_s).max() <= 1e-5


def test_batched_sessions_and_slots_untouched():
    # GDNKernelTests.swift:206-277: a slot offset is honoured and other slots are not written.
    r = np.random.default_rng(5)
    cfgA = tt.ArchConfig.qwen36_35b_a3b()
    la = cfgA.linear_attention
    slots = 5
    mgr = tt.GDNStateManager(cfgA, slots=slots)
    layer = 0
    assert mgr.is_linear(layer) and not mgr.is_linear(3)
    n_state = la.num_v_heads * la.value_head_dim * la.key_head_dim
    states0 = (0.02 * r.normal(size=(slots, n_state))).astype(np.float32)
    base = mgr.state_slot(layer, 0)
    assert mgr.state_slot(layer, 3) - base == 3 * mgr.state_bytes_per_layer
    live = device_view(base, slots * n_state).view(slots, n_state)   # the manager's own buffer
    assert torch.count_nonzero(live).item() == 0                     # zero-initialised (GDNStateManager.swift:207)
    live.copy_(torch.from_numpy(states0).cuda())
    active = [1, 3, 4]
    ins = [make_inputs(r, 1, la.num_k_heads, la.num_v_heads, la.key_head_dim, la.value_head_dim) for _ in active]
    a_log, dt_bias = ins[0][3], ins[0][4]
    keep = []
    sessions = []
    ys = []
    for (conv, a, b, _, _, _), slot in zip(ins, active):
        cd, ad, bd = dev(conv), dev(a), dev(b)
        y = torch.zeros(1, la.value_dim, device="cuda", dtype=torch.float16)
        keep += [cd, ad, bd]; ys.append(y)
        sessions.append(tt.GDNSession(cd, ad, bd, mgr.state_slot(layer, slot), y))
    gdn = tt.GDN(context(), la)
    al_d, dt_d = dev(a_log, torch.bfloat16), dev(dt_bias, torch.bfloat16)
    gdn.encode_delta_step_batched(sessions, al_d, dt_d)
    torch.cuda.synchronize()
    after = host(live)
    for idx, slot in enumerate(active):
        conv, a, b = ins[idx][0], ins[idx][1], ins[idx][2]
        wy, ws, _ = oracle.gdn_step_rows(conv, a, b, a_log, dt_bias, la.num_k_heads, la.num_v_heads, la.key_head_dim,
                                         la.value_head_dim, states0[slot])
        assert np.abs(host(ys[idx]) - wy).max() <= TOL
        assert np.abs(after[slot] - ws.reshape(-1)).max() <= 1e-5
    for slot in (0, 2):
        assert np.array_equal(after[slot], states0[slot])
    mgr.reset(slot=1)
    torch.cuda.synchronize()
    z = host(live)
    assert np.all(z[1] == 0) and np.array_equal(z[3], after[3])
    mgr.close()


def test_cpu_engine_convention_matches_reference_golden():
    # The CPU engine's convention (unit-L2 q, readout * 1/sqrt(dv)) through the explicit
    # readout_scale, on the reference kernel's own outputs (tests/golden/delta_rule_d128.npz).
    c = mg.d128_inputs()
    gold = np.load(os.path.join(GOLD, "delta_rule_d128.npz"))
    tokens, heads = c["value"].shape[:2]
    kh, d = c["key_heads"], 128
    cfg = tt.LinearAttentionConfig(kh, heads, d, d)
    conv = np.concatenate([c["query"].reshape(tokens, -1), c["key"].reshape(tokens, -1), c["value"].reshape(tokens, -1)], 1)
    conv16 = rounded(conv); a16 = rounded(c["a"]); b16 = rounded(c["b"])
    al = rounded(c["decay_log"], torch.bfloat16); db = rounded(c["decay_bias"], torch.bfloat16)
    got_y, got_s, _ = run_step(cfg, conv16, a16, b16, al, db, c["state"], tokens, readout_scale=float(c["inverse"]))
    # inputs were rounded to the GPU path's storage types, so compare at the storage-rounding level
    assert np.abs(got_y - gold["readout"].reshape(tokens, -1)).max() <= 1e-2
    want_y, want_s, _ = oracle.gdn_step_rows(conv16, a16, b16, al, db, kh, heads, d, d, c["state"],
                                             readout_scale=float(c["inverse"]))
    assert np.abs(got_y - want_y).max() <= TOL and np.abs(got_s - want_s).max() <= 1e-5


def test_precomputed_gates_form():
    # the tinytitan_delta_rule_chunk calling form: per-token alpha, beta given as fp32
    r = np.random.default_rng(77)
    hk, hv, d, rows = 2, 4, 128, 7
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, _, _, _, _, state = make_inputs(r, rows, hk, hv, d, d)
    alpha = r.uniform(0.5, 1.0, size=(rows, hv)).astype(np.float32)
    beta = r.uniform(0.1, 0.9, size=(rows, hv)).astype(np.float32)
    gdn = tt.GDN(context(), cfg, gates_f32=True)
    st = dev(state, torch.float32)
    y = torch.zeros(rows, cfg.value_dim, device="cuda", dtype=torch.float16)
    gdn.encode_delta_step_prefill(dev(conv), dev(alpha, torch.float32), dev(beta, torch.float32), None, None, st, y, rows)
    torch.cuda.synchronize()
    q = conv[:, :hk * d]; k = conv[:, hk * d:2 * hk * d]; v = conv[:, 2 * hk * d:]
    want_y, want_s = oracle.gdn_scan_heads(q, k, v, alpha, beta, hk, hv, d, d, 1, state, threads=4)
    assert np.abs(host(y) - want_y).max() <= TOL and np.abs(host(st) - want_s).max() <= 1e-4


def test_rejects_bad_shapes():
    cfg = tt.LinearAttentionConfig(3, 8, 128, 128)
    gdn = tt.GDN(context(), cfg)
    x = torch.zeros(4096, device="cuda", dtype=torch.float16)
    s = torch.zeros(8 * 128 * 128, device="cuda")
    with pytest.raises(tt.InvalidArgument):
        gdn.encode_delta_step_decode(x, x, x, x, x, s, x)
    gdn = tt.GDN(context(), tt.LinearAttentionConfig(2, 4, 48, 64))
    with pytest.raises(tt.UnsupportedShape):
        gdn.encode_delta_step_decode(x, x, x, x, x, s, x)


# ------------------------------------------------------------------ chunk-parallel scan
def run_scan(cfg, conv, a, b, a_log, dt_bias, state, rows, **gdn_kw):
    gdn = tt.GDN(context(), cfg, **gdn_kw)
    f32 = gdn_kw.get("gates_f32", False)
    conv_d = dev(conv)
    a_d, b_d = (dev(a, torch.float32), dev(b, torch.float32)) if f32 else (dev(a), dev(b))
    al_d = dev(a_log, torch.bfloat16) if a_log is not None else None
    dt_d = dev(dt_bias, torch.bfloat16) if dt_bias is not None else None
    st_d = dev(state, torch.float32)
    y = torch.full((rows, cfg.value_dim), float("nan"), device="cuda", dtype=torch.float16)
    gdn.encode_delta_scan_chunked(conv_d, a_d, b_d, al_d, dt_d, st_d, y, rows, row_stride=conv.shape[1])
    torch.cuda.synchronize()
    assert context().poll_status() == 0   # no bounded wait ran out, no alignment check failed
    return host(y), host(st_d)


@pytest.mark.parametrize("rows,hk,hv", [(64, 1, 1), (200, 2, 4), (1, 1, 2), (513, 2, 2)])
def test_chunked_scan_matches_sequential_oracle(rows, hk, hv):
    r = np.random.default_rng(rows + hv)
    d = 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, a, b, a_log, dt_bias, state = make_inputs(r, rows, hk, hv, d, d, extra_stride=8)
    want_y, want_s, _ = oracle.gdn_step_rows(conv, a, b, a_log, dt_bias, hk, hv, d, d, state)
    got_y, got_s = run_scan(cfg, conv, a, b, a_log, dt_bias, state, rows)
    assert np.isfinite(got_y).all()
    assert np.abs(got_y - want_y).max() <= TOL
    assert np.abs(got_s - want_s).max() <= 2e-3 * max(1.0, np.abs(want_s).max())


def test_chunked_scan_against_reference_chunk_kernel():
    # the tinytitan_delta_rule_chunk calling form (alpha, beta given), checked against the
    # reference's own chunk kernel at chunk 64 and its token kernel (via the oracle drivers)
    r = np.random.default_rng(31)
    hk, hv, d, rows = 2, 4, 128, 256
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, _, _, _, _, state = make_inputs(r, rows, hk, hv, d, d)
    alpha = r.uniform(0.5, 1.0, size=(rows, hv)).astype(np.float32)
    beta = r.uniform(0.1, 0.9, size=(rows, hv)).astype(np.float32)
    got_y, got_s = run_scan(cfg, conv, alpha, beta, None, None, state, rows, gates_f32=True)
    q = conv[:, :hk * d]; k = conv[:, hk * d:2 * hk * d]; v = conv[:, 2 * hk * d:]
    use_ref = oracle.ref() is not None
    want_y, want_s = oracle.gdn_scan_heads(q, k, v, alpha, beta, hk, hv, d, d, 64, state, threads=4, use_ref=use_ref)
    assert np.abs(got_y - want_y).max() <= TOL
    assert np.abs(got_s - want_s).max() <= 2e-3 * max(1.0, np.abs(want_s).max())


def test_chunked_scan_equals_sequential_kernel_at_config3_size():
    # 8192 tokens, 16/32 heads (config 3): the oracle needs minutes, so the exact sequential
    # CUDA kernel is the comparison; also the scan over [0,T) equals two scans over [0,T1),[T1,T)
    g = torch.Generator(device="cuda"); g.manual_seed(17)
    T, hk, hv, d = 8192, 16, 32, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    qk = torch.randn(T, 2 * hk, d, device="cuda", generator=g)
    qk = qk / qk.norm(dim=-1, keepdim=True); qk[:, :hk] *= d ** -0.5
    conv = torch.cat([qk.reshape(T, -1), torch.randn(T, hv * d, device="cuda", generator=g)], 1).half().contiguous()
    a = (-torch.randn(T, hv, device="cuda", generator=g)).half(); b = torch.randn(T, hv, device="cuda", generator=g).half()
    z = torch.zeros(hv, device="cuda", dtype=torch.bfloat16)
    s0 = (0.02 * torch.randn(hv, d, d, device="cuda", generator=g))
    gdn = tt.GDN(context(), cfg)
    s_seq, s_scan, s_two = s0.clone(), s0.clone(), s0.clone()
    y_seq = torch.empty(T, hv * d, device="cuda", dtype=torch.float16); y_scan = torch.empty_like(y_seq); y_two = torch.empty_like(y_seq)
    gdn.encode_delta_step_prefill(conv, a, b, z, z, s_seq, y_seq, T)
    gdn.encode_delta_scan_chunked(conv, a, b, z, z, s_scan, y_scan, T)
    T1 = 3000   # not a multiple of the chunk: the second call starts mid-chunk of the first
    gdn.encode_delta_scan_chunked(conv, a, b, z, z, s_two, y_two, T1)
    gdn.encode_delta_scan_chunked(conv[T1:], a[T1:], b[T1:], z, z, s_two, y_two[T1:], T - T1)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    assert (y_scan.float() - y_seq.float()).abs().max().item() <= TOL
    assert (s_scan - s_seq).abs().max().item() <= 2e-3 * max(1.0, s_seq.abs().max().item())
    assert (y_two.float() - y_seq.float()).abs().max().item() <= TOL
    assert (s_two - s_seq).abs().max().item() <= 2e-3 * max(1.0, s_seq.abs().max().item())


def test_chunked_scan_tcgen05_and_mma_sync_recurrences_agree(monkeypatch):
    # TT_GDN_SCAN_FORCE_MMA_SYNC=1 runs the state recurrence on the mma.sync kernel (fp32 state in
    # accumulator registers) instead of the tcgen05 one (state transposed in tensor memory); a ragged
    # tail, tiled value heads and more than one Dv block per head are all in this case
    r = np.random.default_rng(77)
    rows, hk, hv, d = 333, 2, 4, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, a, b, a_log, dt_bias, state = make_inputs(r, rows, hk, hv, d, d)
    want_y, want_s, _ = oracle.gdn_step_rows(conv, a, b, a_log, dt_bias, hk, hv, d, d, state)
    got = []
    for force in (False, True):
        if force:
            monkeypatch.setenv("TT_GDN_SCAN_FORCE_MMA_SYNC", "1")
        launches = context().launch_count
        got.append(run_scan(cfg, conv, a, b, a_log, dt_bias, state, rows))
        assert context().launch_count - launches == 2
    for y, s in got:
        assert np.abs(y - want_y).max() <= TOL
        assert np.abs(s - want_s).max() <= 2e-3 * max(1.0, np.abs(want_s).max())
    # The two tensor-core generations round a 16-deep step the same way, so the states may even agree
    # bit for bit; y is formed in a different order (A_t R added after M C rather than before).
    assert np.abs(got[0][0] - got[1][0]).max() <= TOL
    assert np.abs(got[0][1] - got[1][1]).max() <= 1e-5 * max(1.0, np.abs(want_s).max())


def test_chunked_scan_in_segments_equals_one_segment(monkeypatch):
    # A context whose workspace holds 8 chunk records per head runs a 23-chunk prompt (ragged tail) in
    # three segments: the state goes through global memory between them and the record indices
    # restart, but chunk boundaries are the same, so both recurrences must reproduce the
    # one-segment result exactly.
    r = np.random.default_rng(91)
    rows, hk, hv, d = 23 * 64 - 17, 2, 4, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    conv, a, b, a_log, dt_bias, state = make_inputs(r, rows, hk, hv, d, d)
    record_bytes = 64 * 128 * 4 + 64 * 128 * 2 + 64 * 64 * 2 + 2 * 64 * 4
    small = tt.Context(0, workspace_bytes=8 * hv * record_bytes + 100)
    try:
        for force in (False, True):
            if force:
                monkeypatch.setenv("TT_GDN_SCAN_FORCE_MMA_SYNC", "1")
            want_y, want_s = run_scan(cfg, conv, a, b, a_log, dt_bias, state, rows)
            cd, ad, bd = dev(conv), dev(a), dev(b)
            al, dt, st = dev(a_log, torch.bfloat16), dev(dt_bias, torch.bfloat16), dev(state, torch.float32)
            y = torch.full((rows, cfg.value_dim), float("nan"), device="cuda", dtype=torch.float16)
            launches = small.launch_count
            tt.GDN(small, cfg).encode_delta_scan_chunked(cd, ad, bd, al, dt, st, y, rows, row_stride=conv.shape[1])
            torch.cuda.synchronize()
            assert small.poll_status() == 0
            assert small.launch_count - launches == 6
            assert np.array_equal(host(y), want_y)
            assert np.array_equal(host(st), want_s)
    finally:
        small.close()


def test_chunked_scan_rejects_other_shapes():
    gdn = tt.GDN(context(), tt.LinearAttentionConfig(2, 4, 64, 64))
    x = torch.zeros(1 << 14, device="cuda", dtype=torch.float16); s = torch.zeros(4 * 64 * 64, device="cuda")
    with pytest.raises(tt.UnsupportedShape):
        gdn.encode_delta_scan_chunked(x, x, x, x, x, s, x, 64)
    gdn = tt.GDN(context(), tt.LinearAttentionConfig(2, 4, 128, 128))
    with pytest.raises(tt.UnsupportedShape):
        gdn.encode_delta_scan_chunked(x, x, x, x, x, torch.zeros(4 * 128 * 128, device="cuda"), x, 64, chunk=32)


@pytest.mark.parametrize("n,hk,hv,dk,dv,rows", [(70, 3, 6, 64, 24, 3), (3, 2, 132, 32, 8, 2), (40, 16, 32, 128, 128, 1)])
def test_persistent_step_other_paths(n, hk, hv, dk, dv, rows):
    # More sessions than the kernel stages in shared memory (70 > 64), more value heads than it
    # stages decay parameters for (132 > 128), head and row-block counts that are not powers of two
    # (the division path of the item decode), and enough items that every warp walks several.
    r = np.random.default_rng(n * 1000 + hv)
    cfg = tt.LinearAttentionConfig(hk, hv, dk, dv)
    ctx = tt.Context(0, max_sessions=128)
    try:
        gdn = tt.GDN(ctx, cfg)
        ins = [make_inputs(r, rows, hk, hv, dk, dv) for _ in range(n)]
        a_log, dt_bias = ins[0][3], ins[0][4]
        al_d, dt_d = dev(a_log, torch.bfloat16), dev(dt_bias, torch.bfloat16)
        keep, sessions, ys, sts = [], [], [], []
        for conv, a, b, _, _, state in ins:
            cd, ad, bd, sd = dev(conv), dev(a), dev(b), dev(state, torch.float32)
            y = torch.full((rows, cfg.value_dim), float("nan"), device="cuda", dtype=torch.float16)
            keep += [cd, ad, bd]; ys.append(y); sts.append(sd)
            sessions.append(tt.GDNSession(cd, ad, bd, sd, y))
        gdn.encode_delta_step_batched(sessions, al_d, dt_d, rows=rows)
        torch.cuda.synchronize()
        assert ctx.poll_status() == 0
        for i in (0, n // 2, n - 1):
            conv, a, b, _, _, state = ins[i]
            wy, ws, _ = oracle.gdn_step_rows(conv, a, b, a_log, dt_bias, hk, hv, dk, dv, state)
            assert np.abs(host(ys[i]) - wy).max() <= TOL, i
            assert np.abs(host(sts[i]) - ws).max() <= 1e-5, i
    finally:
        ctx.close()
