"""The fused pre-attention step (split, q/k norm, partial NeoX RoPE) and the output gate."""
import numpy as np
import pytest
import torch

import tinytitan_b200 as tt
from gpu_util import context, dev, host, rounded

pytestmark = pytest.mark.gpu


def h(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def ref_norm_rope(x, w, eps, rotary, theta, pos):
    """rmsnorm_bf16w_perhead then rope_neox_subdim on one head, with the fp16 store in between
    (Primitives/rmsnorm.metal:101-128, Primitives/rope.metal:32-49, :80-108)."""
    x = x.astype(np.float32)
    inv = np.float32(1) / np.sqrt(np.float32((x * x).sum(dtype=np.float32) / x.size + eps))
    y = h(x * inv * w)
    half = rotary // 2
    pair = np.arange(half, dtype=np.float32)
    angle = np.float32(pos) * np.power(np.float32(theta), -(2 * pair) / np.float32(rotary)).astype(np.float32)
    c, s = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    out = y.copy()
    out[:half] = h(y[:half] * c - y[half:rotary] * s)
    out[half:rotary] = h(y[:half] * s + y[half:rotary] * c)
    return out


@pytest.mark.parametrize("hd,hq,hkv,rotary,rows,pos", [(256, 16, 2, 64, 1, 4097), (256, 16, 2, 64, 5, 100), (128, 8, 4, 128, 3, 7),
                                                        (64, 4, 2, 24, 2, 31)])
def test_pre_attention_step(hd, hq, hkv, rotary, rows, pos):
    r = np.random.default_rng(hd + rows)
    theta, eps = 1e7, 1e-6
    packed = rounded(r.normal(size=(rows, hq, 2 * hd)))
    stride = hkv * hd + 16
    krows = rounded(r.normal(size=(rows, stride)))
    qw = rounded(r.uniform(0.5, 1.5, size=hd), torch.bfloat16); kw = rounded(r.uniform(0.5, 1.5, size=hd), torch.bfloat16)
    kd = dev(krows)
    q_out = torch.empty(rows, hq, hd, device="cuda", dtype=torch.float16); g_out = torch.empty_like(q_out)
    tt.Attention(context()).encode_pre(dev(packed), q_out, g_out, kd, dev(qw, torch.bfloat16), dev(kw, torch.bfloat16), hd, hq,
                                       hkv, rotary, theta, eps, pos, rows=rows, k_row_stride_elements=stride)
    torch.cuda.synchronize()
    got_q, got_g, got_k = host(q_out), host(g_out), host(kd)
    assert np.array_equal(got_g, packed[:, :, hd:])                        # the gate half is a plain copy
    assert np.array_equal(got_k[:, hkv * hd:], krows[:, hkv * hd:])         # row padding untouched
    for t in range(rows):
        for head in range(hq):
            want = ref_norm_rope(packed[t, head, :hd], qw, eps, rotary, theta, pos + t)
            assert np.abs(got_q[t, head] - want).max() <= 2e-3 + np.abs(want).max() * 2.0 ** -9
        for head in range(hkv):
            want = ref_norm_rope(krows[t, head * hd:(head + 1) * hd], kw, eps, rotary, theta, pos + t)
            assert np.abs(got_k[t, head * hd:(head + 1) * hd] - want).max() <= 2e-3 + np.abs(want).max() * 2.0 ** -9
            # beyond the rotary window the value is the normed one, bit for bit
            assert np.array_equal(got_k[t, head * hd + rotary:(head + 1) * hd], want[rotary:])


def test_output_gate():
    r = np.random.default_rng(0)
    out = rounded(r.normal(size=4096)); gate = rounded(r.normal(size=4096) * 3)
    od = dev(out)
    tt.Attention(context()).encode_gate_mul(od, dev(gate), 4096)
    torch.cuda.synchronize()
    want = h(out / (1 + np.exp(-gate)))
    assert np.abs(host(od) - want).max() <= 2.0 ** -10 * np.abs(want).max() + 1e-6
