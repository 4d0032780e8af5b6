"""Oracle parity at the sizes the benchmark configurations are stated at.

Each case runs the CUDA path through the C ABI at the FULL configuration size and compares a
sample of its output rows with the CPU oracle evaluated at that same full size (query rows, heads
or sessions are sampled, never the key range: every compared row attends over all of its keys).
Two bars are asserted and printed: the north star's (max abs error 2e-3 on fp16 I/O, plus one
rounding step of the value for bf16 outputs) and the reference's own test tolerances (decode rel
1e-2, Tolerances.swift:15; prefill max abs and rel 2e-2, PrefillAttentionTests.swift:353-354).
"""
import os

import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from gpu_util import TOL, context, dev, host, bf16_tol

pytestmark = pytest.mark.gpu
SCALE = 0.0625


def report(name, got, want, tol=TOL, ref_abs=2e-2, ref_rel=1e-2):
    err = np.abs(got - want)
    rel = err.max() / max(np.abs(want).max(), 1e-30)
    print(f"{name}: max abs error {err.max():.2e} (bar {np.max(tol):.1e}); relative to max |want| {rel:.2e} "
          f"(reference bar {ref_rel:.0e})")
    assert np.all(err <= tol), name
    assert err.max() <= ref_abs and rel <= ref_rel, name


def randn(gen, *shape, dtype=torch.float16):
    return torch.randn(*shape, device="cuda", generator=gen).to(dtype)


def f32(t):
    return t.float().cpu().numpy()


# ------------------------------------------------------------------------------------------
# config 1: one decode step at the 2B shape (8/2/256, 4096 keys; GDN 16/16/128)
# ------------------------------------------------------------------------------------------
def test_config1_decode_step():
    g = torch.Generator(device="cuda"); g.manual_seed(101)
    hq, hkv, hd, s = 8, 2, 256, 4096
    q, k, v = randn(g, hq, hd), randn(g, s, hkv, hd), randn(g, s, hkv, hd)
    out = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
    tt.Attention(context()).encode_full(q, k, v, out, hd, hq, hkv, s, scale=SCALE)
    torch.cuda.synchronize()
    report("config 1 attention", f32(out), oracle.attn_decode(f32(q), f32(k), f32(v), hkv, SCALE))

    hk, hv, d = 16, 16, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    qk = torch.randn(2 * hk, d, device="cuda", generator=g)
    qk = qk / qk.norm(dim=-1, keepdim=True); qk[:hk] *= d ** -0.5
    conv = torch.cat([qk.reshape(-1), torch.randn(hv * d, device="cuda", generator=g)]).half()[None].contiguous()
    a, b = -randn(g, 1, hv), randn(g, 1, hv)                     # A_log = dt_bias = 0: decay = sigmoid(n)
    z = torch.zeros(hv, device="cuda", dtype=torch.bfloat16)
    state = 0.02 * torch.randn(hv, d, d, device="cuda", generator=g)
    want_y, want_s, _ = oracle.gdn_step_rows(f32(conv), f32(a), f32(b), np.zeros(hv), np.zeros(hv), hk, hv, d, d, f32(state))
    y = torch.empty(1, hv * d, device="cuda", dtype=torch.float16)
    tt.GDN(context(), cfg).encode_delta_step_decode(conv, a, b, z, z, state, y)
    torch.cuda.synchronize()
    report("config 1 GDN y", f32(y), want_y)
    assert np.abs(f32(state) - want_s).max() <= 1e-5


# ------------------------------------------------------------------------------------------
# config 2: the benchmark's own 32 drawn sessions in one batched call (16/2/256; GDN 16/32/128)
# ------------------------------------------------------------------------------------------
def test_config2_batched_decode_sampled_sessions():
    lens = [int(x) for x in np.random.default_rng(20261125).integers(1024, 32769, size=32)]   # bench.py's draw
    g = torch.Generator(device="cuda"); g.manual_seed(202)
    hq, hkv, hd = 16, 2, 256
    n, cap = len(lens), 32768
    k = randn(g, n * cap, hkv * hd); v = randn(g, n * cap, hkv * hd)           # slot i at row i * capacity
    q = randn(g, n, hq * hd)
    out = torch.full((n, hq * hd), float("nan"), device="cuda", dtype=torch.float16)
    row = hkv * hd * 2
    sessions = [tt.DecodeSession(q, out, k, v, lens[i], 1, 0, q_offset=i * hq * hd * 2, out_offset=i * hq * hd * 2,
                                 k_offset=i * cap * row, v_offset=i * cap * row) for i in range(n)]
    tt.Attention(context()).encode_batched(sessions, hd, hq, hkv, scale=SCALE)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    assert torch.isfinite(out.float()).all()
    order = np.argsort(lens)
    for i in (int(order[-1]), int(order[0]), int(order[len(order) // 2]), 5):   # longest, shortest, median, one more
        kk = f32(k[i * cap:i * cap + lens[i]]).reshape(lens[i], hkv, hd)
        vv = f32(v[i * cap:i * cap + lens[i]]).reshape(lens[i], hkv, hd)
        want = oracle.attn_decode(f32(q[i]).reshape(hq, hd), kk, vv, hkv, SCALE).reshape(-1)
        report(f"config 2 session {i} ({lens[i]} keys)", f32(out[i]), want)


def test_config2_gdn_step_sampled_sessions():
    g = torch.Generator(device="cuda"); g.manual_seed(203)
    n, hk, hv, d = 32, 16, 32, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    qk = torch.randn(n, 2 * hk, d, device="cuda", generator=g)
    qk = qk / qk.norm(dim=-1, keepdim=True); qk[:, :hk] *= d ** -0.5
    conv = torch.cat([qk.reshape(n, -1), torch.randn(n, hv * d, device="cuda", generator=g)], 1).half().contiguous()
    a, b = -randn(g, n, hv), randn(g, n, hv)
    z = torch.zeros(hv, device="cuda", dtype=torch.bfloat16)
    state = 0.02 * torch.randn(n, hv, d, d, device="cuda", generator=g)
    before = f32(state)
    y = torch.empty(n, hv * d, device="cuda", dtype=torch.float16)
    ses = [tt.GDNSession(conv[i], a[i], b[i], state[i], y[i]) for i in range(n)]
    tt.GDN(context(), cfg).encode_delta_step_batched(ses, z, z)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    for i in (0, 13, 31):
        want_y, want_s, _ = oracle.gdn_step_rows(f32(conv[i:i + 1]), f32(a[i:i + 1]), f32(b[i:i + 1]), np.zeros(hv),
                                                 np.zeros(hv), hk, hv, d, d, before[i])
        report(f"config 2 GDN session {i}", f32(y[i:i + 1]), want_y)
        assert np.abs(f32(state[i]) - want_s).max() <= 1e-5


# ------------------------------------------------------------------------------------------
# config 3: causal prefill over 8192 tokens (16/2/256) on both kernels; GDN scan over 8192 tokens
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_config3_prefill_sampled_rows_both_kernels(dtype):
    g = torch.Generator(device="cuda"); g.manual_seed(303)
    T, hq, hkv, hd = 8192, 16, 2, 256
    q, k, v = randn(g, T, hq * hd, dtype=dtype), randn(g, T, hkv * hd, dtype=dtype), randn(g, T, hkv * hd, dtype=dtype)
    p = tt.PrefillAttentionParams(0, T, hd, hq, hkv, T, 0, hkv * hd, hq * hd, hq * hd, SCALE)
    pa = tt.PrefillAttention(context())
    assert pa.selected_path(q, k, v, q, p) == "tcgen05"
    outs = {}
    for name in ("tcgen05", "generic"):
        o = torch.full((T, hq * hd), float("nan"), device="cuda", dtype=dtype)
        if name == "generic":
            os.environ["TT_PREFILL_FORCE_GENERIC"] = "1"
        try:
            pa.encode_causal(q, k, v, o, p)
        finally:
            os.environ.pop("TT_PREFILL_FORCE_GENERIC", None)
        torch.cuda.synchronize()
        assert context().poll_status() == 0
        outs[name] = o
    kf, vf = f32(k), f32(v)
    for start in (0, 4000, 8128):                                   # 64 query rows each, all 16 heads
        want = oracle.attn_prefill(f32(q[start:start + 64]), kf, vf, hq * hd, hkv * hd, hd, hq, hkv, start, 64, T, 0,
                                   SCALE).reshape(64, -1)
        for name, o in outs.items():
            # bf16 I/O: the output carries one bf16 rounding of its own value, and the tensor-core kernel's
            # softmax weights are bf16 too (both operands of one tcgen05.mma share a format): 2^-9
            # relative on each weight, which over a row's few keys does not average out
            tol = TOL if dtype == torch.float16 else bf16_tol(want) + 2.0 ** -9 * np.abs(vf).max()
            report(f"config 3 prefill {name} {str(dtype)[6:]} rows {start}..{start + 63}", f32(o[start:start + 64]), want,
                   tol=tol, ref_abs=2e-2, ref_rel=2e-2)


def test_config3_gdn_scan_sampled_heads():
    g = torch.Generator(device="cuda"); g.manual_seed(304)
    T, hk, hv, d = 8192, 16, 32, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    qk = torch.randn(T, 2 * hk, d, device="cuda", generator=g)
    qk = qk / qk.norm(dim=-1, keepdim=True); qk[:, :hk] *= d ** -0.5
    conv = torch.cat([qk.reshape(T, -1), torch.randn(T, hv * d, device="cuda", generator=g)], 1).half().contiguous()
    a, b = -randn(g, T, hv), randn(g, T, hv)
    z = torch.zeros(hv, device="cuda", dtype=torch.bfloat16)
    s0 = 0.02 * torch.randn(hv, d, d, device="cuda", generator=g)
    state = s0.clone()
    y = torch.empty(T, hv * d, device="cuda", dtype=torch.float16)
    tt.GDN(context(), cfg).encode_delta_scan_chunked(conv, a, b, z, z, state, y, T)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    convf = f32(conv)
    for h in (3, 30):                                               # heads are independent: carry two of the 32
        kh = h // (hv // hk)
        sub = np.concatenate([convf[:, kh * d:(kh + 1) * d], convf[:, (hk + kh) * d:(hk + kh + 1) * d],
                              convf[:, (2 * hk + h) * d:(2 * hk + h + 1) * d]], 1)
        want_y, want_s, _ = oracle.gdn_step_rows(sub, f32(a[:, h:h + 1]), f32(b[:, h:h + 1]), np.zeros(1), np.zeros(1),
                                                 1, 1, d, d, f32(s0[h:h + 1]))
        report(f"config 3 GDN scan head {h}, 8192 tokens", f32(y[:, h * d:(h + 1) * d]), want_y)
        assert np.abs(f32(state[h]) - want_s[0]).max() <= 2e-3 * max(1.0, np.abs(want_s).max())


# ------------------------------------------------------------------------------------------
# config 4: one 262,144-key session (16/2/256) on one GPU
# ------------------------------------------------------------------------------------------
def test_config4_long_context_single_gpu():
    g = torch.Generator(device="cuda"); g.manual_seed(404)
    hq, hkv, hd, s = 16, 2, 256, 262144
    q, k, v = randn(g, hq, hd), randn(g, s, hkv, hd), randn(g, s, hkv, hd)
    out = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
    tt.Attention(context()).encode_full(q, k, v, out, hd, hq, hkv, s, scale=SCALE)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    want = oracle.attn_decode_split(f32(q), f32(k), f32(v), hkv, SCALE, s, n_chunks=64)
    report("config 4 attention, 262144 keys", f32(out), want)


# ------------------------------------------------------------------------------------------
# config 5: 64 sessions x 4 draft rows at context 16384 (32/2/256); paired 4-row GDN step 16/64/128
# ------------------------------------------------------------------------------------------
def test_config5_verify_batch_sampled_session():
    g = torch.Generator(device="cuda"); g.manual_seed(505)
    n, w, hq, hkv, hd = 64, 4, 32, 2, 256
    s = 16384 + w - 1                                              # the draft rows are in the cache too
    cap = s + 5
    k = randn(g, n * cap, hkv * hd); v = randn(g, n * cap, hkv * hd)
    q = randn(g, n, w, hq * hd)
    out = torch.full((n, w, hq * hd), float("nan"), device="cuda", dtype=torch.float16)
    row = hkv * hd * 2
    sessions = [tt.DecodeSession(q, out, k, v, s, w, 0, q_offset=i * w * hq * hd * 2, out_offset=i * w * hq * hd * 2,
                                 k_offset=i * cap * row, v_offset=i * cap * row) for i in range(n)]
    tt.Attention(context()).encode_batched(sessions, hd, hq, hkv, scale=SCALE)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    assert torch.isfinite(out.float()).all()
    i = 37
    kk, vv = f32(k[i * cap:i * cap + s]).reshape(s, hkv, hd), f32(v[i * cap:i * cap + s]).reshape(s, hkv, hd)
    for r in range(w):
        vis = s - (w - 1 - r)
        want = oracle.attn_decode(f32(q[i, r]).reshape(hq, hd), kk[:vis], vv[:vis], hkv, SCALE).reshape(-1)
        report(f"config 5 session {i} draft row {r} ({vis} keys)", f32(out[i, r]), want)


def test_config5_gdn_four_row_step_sampled_session():
    g = torch.Generator(device="cuda"); g.manual_seed(506)
    n, w, hk, hv, d = 64, 4, 16, 64, 128
    cfg = tt.LinearAttentionConfig(hk, hv, d, d)
    qk = torch.randn(n, w, 2 * hk, d, device="cuda", generator=g)
    qk = qk / qk.norm(dim=-1, keepdim=True); qk[:, :, :hk] *= d ** -0.5
    conv = torch.cat([qk.reshape(n, w, -1), torch.randn(n, w, hv * d, device="cuda", generator=g)], 2).half().contiguous()
    a, b = -randn(g, n, w, hv), randn(g, n, w, hv)
    z = torch.zeros(hv, device="cuda", dtype=torch.bfloat16)
    state = 0.02 * torch.randn(n, hv, d, d, device="cuda", generator=g)
    ck = torch.zeros_like(state)
    i = 21
    before = f32(state[i])
    y = torch.empty(n, w, hv * d, device="cuda", dtype=torch.float16)
    ses = [tt.GDNSession(conv[j], a[j], b[j], state[j], y[j], checkpoint_state=ck[j]) for j in range(n)]
    tt.GDN(context(), cfg).encode_delta_step_batched(ses, z, z, rows=w)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    want_y, want_s, want_ck = oracle.gdn_step_rows(f32(conv[i]), f32(a[i]), f32(b[i]), np.zeros(hv), np.zeros(hv), hk, hv,
                                                   d, d, before, want_checkpoint=True)
    report(f"config 5 GDN session {i}, 4 rows", f32(y[i]), want_y)
    assert np.abs(f32(state[i]) - want_s).max() <= 1e-5
    assert np.abs(f32(ck[i]) - want_ck).max() <= 1e-5
