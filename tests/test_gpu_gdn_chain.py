"""The Gated-DeltaNet chain around the delta rule (conv, q/k norm, gated norm) on B200."""
import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from oracle.prng import seed_tree_key
from gpu_util import TOL, context, dev, host, rounded

pytestmark = pytest.mark.gpu
CFG = tt.LinearAttentionConfig(2, 4, 32, 32, 4)   # tests/TinyTitan/Kernels/GDN/GDNKernelTests.swift:18-20


def bf16_trunc(x):
    """bf16 by truncation, as the reference's fixture does (GDNKernelTests.swift:24-30)."""
    bits = np.asarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFF0000)
    return bits.view(np.float32)


def fixture(rows, seed):
    # GDNKernelTests.swift:59-99: draw order convW, aLog, dtBias, normW, then all qkv rows, all a, all b, all z
    g = seed_tree_key(seed, f"gdn-fixture-{rows}")
    c = CFG.qkv_dim
    conv_w = bf16_trunc(g.uniform_array(c * CFG.conv_kernel_size, -0.4, 0.4))
    a_log = bf16_trunc(g.uniform_array(CFG.num_v_heads, -1.0, 1.5))
    dt_bias = bf16_trunc(g.uniform_array(CFG.num_v_heads, -0.5, 0.5))
    norm_w = bf16_trunc(g.uniform_array(CFG.value_head_dim, 0.5, 1.5))
    qkv = rounded(g.uniform_array(rows * c, -1, 1).reshape(rows, c))
    a = rounded(g.uniform_array(rows * CFG.num_v_heads, -1, 1).reshape(rows, -1))
    b = rounded(g.uniform_array(rows * CFG.num_v_heads, -1, 1).reshape(rows, -1))
    z = rounded(g.uniform_array(rows * CFG.value_dim, -1, 1).reshape(rows, -1))
    return conv_w, a_log, dt_bias, norm_w, qkv, a, b, z


class Device:
    def __init__(self, fx):
        conv_w, a_log, dt_bias, norm_w, qkv, a, b, z = fx
        self.gdn = tt.GDN(context(), CFG)
        self.conv_w, self.a_log = dev(conv_w, torch.bfloat16), dev(a_log, torch.bfloat16)
        self.dt_bias, self.norm_w = dev(dt_bias, torch.bfloat16), dev(norm_w, torch.bfloat16)
        self.qkv, self.a, self.b, self.z = dev(qkv), dev(a), dev(b), dev(z)
        self.tail = torch.zeros(CFG.conv_kernel_size - 1, CFG.qkv_dim, device="cuda", dtype=torch.float16)
        self.state = torch.zeros(CFG.num_v_heads, CFG.value_head_dim, CFG.key_head_dim, device="cuda")


@pytest.mark.parametrize("rows,seed", [(6, 0x51D), (7, 0xBEEF), (2, 0xC11E), (1, 0x5107)])
def test_decode_chain_matches_reference(rows, seed):
    # GDNKernelTests.swift:144-200: per-row gated output within max(2e-2, 4e-2*|want|), state within 5e-2
    fx = fixture(rows, seed)
    ref = oracle.GDNChainReference(2, 4, 32, 32, 4, *fx[:4])
    d = Device(fx)
    c = CFG.qkv_dim
    conv = torch.empty(c, device="cuda", dtype=torch.float16)
    y = torch.empty(CFG.value_dim, device="cuda", dtype=torch.float16)
    out = torch.empty(CFG.value_dim, device="cuda", dtype=torch.float16)
    for t in range(rows):
        d.gdn.encode_conv_decode(d.tail, d.qkv[t], d.conv_w, conv)
        d.gdn.encode_qk_norm(conv)
        d.gdn.encode_delta_step_decode(conv, d.a[t], d.b[t], d.a_log, d.dt_bias, d.state, y)
        d.gdn.encode_gated_norm(y, d.z[t], d.norm_w, out)
        torch.cuda.synchronize()
        want, want_y, want_conv = ref.step(fx[4][t], fx[5][t], fx[6][t], fx[7][t])
        assert np.abs(host(conv) - want_conv).max() <= 2e-3
        assert np.abs(host(y) - want_y).max() <= TOL
        got = host(out)
        assert np.all(np.abs(got - want) <= np.maximum(2e-2, 4e-2 * np.abs(want)))
    assert np.abs(host(d.state) - ref.state).max() <= 1e-3
    assert np.array_equal(host(d.tail), ref.tail)


def test_prefill_chunk_equals_sequential_decode_bitwise():
    # GDNKernelTests.swift:279-392: the prefill kernels over a chunk give exactly the decode chain's
    # outputs, state and tail; plus the short-chunk tail carry (:681-721) with rows < taps-1
    for rows, seed in [(7, 0xBEEF), (2, 0xC11E)]:
        fx = fixture(rows, seed)
        c = CFG.qkv_dim
        a, bdev = Device(fx), Device(fx)
        outs = []
        conv = torch.empty(c, device="cuda", dtype=torch.float16)
        y = torch.empty(CFG.value_dim, device="cuda", dtype=torch.float16)
        for t in range(rows):
            o = torch.empty(CFG.value_dim, device="cuda", dtype=torch.float16)
            a.gdn.encode_conv_decode(a.tail, a.qkv[t], a.conv_w, conv)
            a.gdn.encode_qk_norm(conv)
            a.gdn.encode_delta_step_decode(conv, a.a[t], a.b[t], a.a_log, a.dt_bias, a.state, y)
            a.gdn.encode_gated_norm(y, a.z[t], a.norm_w, o)
            outs.append(o)
        convs = torch.empty(rows, c, device="cuda", dtype=torch.float16)
        ys = torch.empty(rows, CFG.value_dim, device="cuda", dtype=torch.float16)
        os_ = torch.empty(rows, CFG.value_dim, device="cuda", dtype=torch.float16)
        ck_tail = torch.empty_like(bdev.tail); ck_state = torch.empty_like(bdev.state)
        g = bdev.gdn
        g.encode_conv_prefill(bdev.tail, bdev.qkv, bdev.conv_w, convs, rows)
        g.encode_conv_tail_checkpoint(bdev.tail, bdev.qkv, ck_tail)
        g.encode_conv_tail_update(bdev.tail, bdev.qkv, rows)
        g.encode_qk_norm(convs, rows=rows)
        g.encode_delta_step_prefill(convs, bdev.a, bdev.b, bdev.a_log, bdev.dt_bias, bdev.state, ys, rows,
                                    checkpoint_state=ck_state)
        g.encode_gated_norm(ys, bdev.z, bdev.norm_w, os_, rows=rows)
        torch.cuda.synchronize()
        assert torch.equal(os_, torch.stack(outs))
        assert torch.equal(bdev.state, a.state) and torch.equal(bdev.tail, a.tail)
        # speculative checkpoint == state / tail after row 0 (GDNKernelTests.swift:394-500)
        one = Device(fx)
        one.gdn.encode_conv_decode(one.tail, one.qkv[0], one.conv_w, conv)
        one.gdn.encode_qk_norm(conv)
        one.gdn.encode_delta_step_decode(conv, one.a[0], one.b[0], one.a_log, one.dt_bias, one.state, y)
        torch.cuda.synchronize()
        assert torch.equal(ck_state, one.state) and torch.equal(ck_tail, one.tail)


def test_gated_norm_sigmoid_gate_and_production_width():
    r = np.random.default_rng(2)
    cfg = tt.LinearAttentionConfig(16, 32, 128, 128, 4)
    gdn = tt.GDN(context(), cfg)
    rows = 5
    y = rounded(r.normal(size=(rows, cfg.value_dim))); z = rounded(r.normal(size=(rows, cfg.value_dim)))
    w = rounded(r.uniform(0.5, 1.5, size=128), torch.bfloat16)
    ref = oracle.GDNChainReference(16, 32, 128, 128, 4, np.zeros(cfg.qkv_dim * 4), np.zeros(32), np.zeros(32), w)
    out = torch.empty(rows, cfg.value_dim, device="cuda", dtype=torch.float16)
    for sig in (False, True):
        gdn.encode_gated_norm(dev(y), dev(z), dev(w, torch.bfloat16), out, rows=rows, sigmoid_gate=sig)
        torch.cuda.synchronize()
        want = np.stack([ref.gated_norm(y[t], z[t], sigmoid_gate=sig) for t in range(rows)])
        assert np.abs(host(out) - want).max() <= TOL + 2.0 ** -10 * np.abs(want).max()
    conv = rounded(r.normal(size=(rows, cfg.qkv_dim + 8)))
    cd = dev(conv)
    gdn.encode_qk_norm(cd, rows=rows, row_stride=cfg.qkv_dim + 8)
    torch.cuda.synchronize()
    got = host(cd)
    for t in range(rows):
        want = ref.qk_norm(conv[t, :cfg.qkv_dim])
        assert np.abs(got[t, :cfg.qkv_dim] - want).max() <= 1e-3
    assert np.array_equal(got[:, cfg.qkv_dim:], conv[:, cfg.qkv_dim:])      # padding untouched
    assert np.array_equal(got[:, 2 * 16 * 128:cfg.qkv_dim], conv[:, 2 * 16 * 128:cfg.qkv_dim])   # v slice untouched


def test_batched_decode_prologue_is_bit_identical_to_the_separate_kernels():
    # conv + tail shift + q/k norm of a whole batch in one launch (tt_gdn_decode_pre) against
    # tt_gdn_conv_mix(update_tail) + tt_gdn_qk_norm per session, at the production widths, over several steps
    r = np.random.default_rng(19)
    cfg = tt.LinearAttentionConfig(16, 32, 128, 128, 4)
    gdn = tt.GDN(context(), cfg)
    n, c = 5, cfg.qkv_dim
    conv_w = dev(rounded(r.uniform(-0.4, 0.4, size=(c, 4)), torch.bfloat16), torch.bfloat16)
    tails_a = dev(rounded(r.normal(size=(n, 3, c)))); tails_b = tails_a.clone()
    out_a = torch.empty(n, c, device="cuda", dtype=torch.float16); out_b = torch.empty_like(out_a)
    for step in range(3):
        qkv = dev(rounded(r.normal(size=(n, c))))
        for i in range(n):
            gdn.encode_conv_decode(tails_a[i], qkv[i], conv_w, out_a[i])
            gdn.encode_qk_norm(out_a[i])
        launches = context().launch_count
        gdn.encode_decode_prologue([(tails_b[i], qkv[i], out_b[i]) for i in range(n)], conv_w)
        assert context().launch_count - launches == 1
        torch.cuda.synchronize()
        assert torch.equal(out_a, out_b) and torch.equal(tails_a, tails_b)


@pytest.mark.parametrize("cfg,rows", [(CFG, 7), (CFG, 2), (tt.LinearAttentionConfig(16, 32, 128, 128, 4), 70),
                                      (tt.LinearAttentionConfig(16, 32, 128, 128, 4), 1),
                                      (tt.LinearAttentionConfig(4, 8, 64, 64, 3), 33)])
def test_prefill_prologue_is_bit_identical_to_the_separate_kernels(cfg, rows):
    # conv + SiLU over the chunk, the tail checkpoint after row 0, the tail update and the q/k norm in ONE launch
    # against the four separate launches, at the fixture width (one channel per lane) and at production width
    # (vector loads, several row blocks per channel group, a chunk longer and shorter than the conv history)
    g = torch.Generator(device="cuda"); g.manual_seed(911 + rows)
    c, taps = cfg.qkv_dim, cfg.conv_kernel_size
    gdn = tt.GDN(context(), cfg)
    conv_w = (torch.rand(c, taps, device="cuda", generator=g) * 0.8 - 0.4).bfloat16()
    qkv = (torch.rand(rows, c, device="cuda", generator=g) * 2 - 1).half()
    tail0 = (torch.rand(taps - 1, c, device="cuda", generator=g) * 2 - 1).half()

    tail_a, out_a, ck_a = tail0.clone(), torch.empty_like(qkv), torch.empty_like(tail0)
    gdn.encode_conv_prefill(tail_a, qkv, conv_w, out_a, rows)
    gdn.encode_conv_tail_checkpoint(tail_a, qkv, ck_a)
    gdn.encode_conv_tail_update(tail_a, qkv, rows)
    gdn.encode_qk_norm(out_a, rows=rows)

    tail_b, out_b, ck_b = tail0.clone(), torch.empty_like(qkv), torch.empty_like(tail0)
    launches = context().launch_count
    gdn.encode_prefill_prologue(tail_b, qkv, conv_w, out_b, rows, checkpoint_tail=ck_b)
    assert context().launch_count - launches == 1
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b) and torch.equal(tail_a, tail_b) and torch.equal(ck_a, ck_b)

    # the conv + SiLU itself against a float64 statement of the same sum (rounded once to fp16), q/k slices aside
    full = torch.cat([tail0, qkv]).double()
    want = sum(full[j:j + rows] * conv_w.double()[:, j] for j in range(taps))
    want = want / (1 + torch.exp(-want))
    lo = 2 * cfg.num_k_heads * cfg.key_head_dim
    assert (out_b[:, lo:].double() - want[:, lo:]).abs().max().item() <= 2e-3
    # the read-only form leaves the tail alone
    tail_c = tail0.clone()
    gdn.encode_prefill_prologue(tail_c, qkv, conv_w, out_b, rows, update_tail=False)
    torch.cuda.synchronize()
    assert torch.equal(tail_c, tail0)


@pytest.mark.parametrize("cfg", [tt.LinearAttentionConfig(16, 32, 128, 128, 4), tt.LinearAttentionConfig(1, 1, 32, 36, 4),
                                 tt.LinearAttentionConfig(1, 1, 8, 18, 4), tt.LinearAttentionConfig(1, 1, 8, 17, 4)])
def test_conv_mix_lane_chunks_and_decode_order(cfg):
    # every lane-chunk width of the conv kernel (8192, 100, 34 and 33 channels: 8, 4, 2 and 1 channels per lane,
    # the last with a partial group), prefill and decode forms, against float64
    channels = cfg.qkv_dim
    g = torch.Generator(device="cuda"); g.manual_seed(channels)
    taps, rows = 4, 19
    gdn = tt.GDN(context(), cfg)
    conv_w = (torch.rand(channels, taps, device="cuda", generator=g) * 0.8 - 0.4).bfloat16()
    qkv = (torch.rand(rows, channels, device="cuda", generator=g) * 2 - 1).half()
    tail = (torch.rand(taps - 1, channels, device="cuda", generator=g) * 2 - 1).half()
    out = torch.empty_like(qkv)
    gdn.encode_conv_prefill(tail, qkv, conv_w, out, rows)
    full = torch.cat([tail, qkv]).double()
    want = sum(full[j:j + rows] * conv_w.double()[:, j] for j in range(taps))
    want = want / (1 + torch.exp(-want))
    torch.cuda.synchronize()
    assert (out.double() - want).abs().max().item() <= 2e-3
    one = torch.empty(channels, device="cuda", dtype=torch.float16)
    t2 = tail.clone()
    gdn.encode_conv_decode(t2, qkv[0], conv_w, one)
    torch.cuda.synchronize()
    assert (one.double() - want[0]).abs().max().item() <= 2e-3
    assert torch.equal(t2, torch.cat([tail[1:], qkv[:1]]))
