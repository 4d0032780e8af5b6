"""The CUDA decode chains against outputs of the reference's own numpy model.

Fixtures: tests/golden/qwen35_attention.npz and qwen35_gdn.npz, written by
tests/golden/make_golden_qwen35.py from `Reference.attention` / `Reference.gdn` of the reference's
tools/qwen35_reference.py (:292-322, :231-290) on seeded synthetic weights. Here the same inputs
go through the library the way the decode path runs it:

  attention  tt_attn_pre (split [query;gate], q/k RMS norm, partial NeoX RoPE; the K row is normed
             in place inside the KV cache manager's slot) -> V row copied into the cache ->
             tt_attn_decode over the manager's views -> tt_attn_gate_mul
  GDN        tt_gdn_conv_mix -> tt_gdn_qk_norm -> tt_gdn_step -> tt_gdn_gated_norm on the state
             manager's state and conv-tail slots

fp16 rounding points of the GPU path (the reference model is fp32/float64 throughout): the normed
q/k, the rotated q/k, the cached K/V rows, the attention row, the gated row; conv output, normed
q/k, y and the gated-norm output on the GDN side.
"""
import os

import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
import make_golden_qwen35 as mq
from gpu_util import TOL, context, dev, host, device_view
from test_oracle import _oracle_attention_chain, _oracle_gdn_chain, gdn_chain_bar

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", list(mq.ATTENTION_CASES))
def test_attention_decode_chain_matches_reference_model(name):
    c = mq.attention_inputs(name)
    gold = np.load(os.path.join(GOLD, "qwen35_attention.npz"))
    want_out, want_keys = gold[f"{name}.out"], gold[f"{name}.keys"]
    hq, hkv, hd, cached, steps = c["hq"], c["hkv"], c["hd"], c["cached"], c["steps"]
    row = hkv * hd
    cfg = tt.ArchConfig([tt.FULL], hkv, hd, hkv, hd, 0, tt.LinearAttentionConfig(16, 32, 128, 128, 4))
    kv = tt.KVCacheManager(cfg, max_context=cached + steps)
    if cached:
        device_view(kv.k_slot(0, 0), cached * row, torch.float16).copy_(dev(c["cache_k"]).view(-1))
        device_view(kv.v_slot(0, 0), cached * row, torch.float16).copy_(dev(c["cache_v"]).view(-1))
        kv.advance(0, cached)
    attn = tt.Attention(context())
    packed, kproj, vproj = dev(c["packed"]), dev(c["k"]), dev(c["v"])
    qw, kw = dev(c["q_norm"], torch.bfloat16), dev(c["k_norm"], torch.bfloat16)
    q = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
    gate = torch.empty_like(q)
    out = torch.empty(steps, hq, hd, device="cuda", dtype=torch.float16)
    for t in range(steps):
        pos = kv.position(0)
        assert pos == cached + t
        kv.reserve(pos + 1)
        krow = device_view(kv.k_slot(0, pos), row, torch.float16)
        krow.copy_(kproj[t].view(-1))                                  # the K projection writes its row into the cache
        device_view(kv.v_slot(0, pos), row, torch.float16).copy_(vproj[t].view(-1))
        attn.encode_pre(packed[t], q, gate, krow, qw, kw, hd, hq, hkv, mq.ROTARY, mq.ROPE_THETA, mq.EPS, pos)
        kv.advance(0, 1)
        kview, vview = kv.key_view(0), kv.value_view(0)
        assert kview.valid_token_count == pos + 1
        attn.encode_full(q, kview.address, vview.address, out[t], hd, hq, hkv, pos + 1, scale=1.0 / np.sqrt(hd),
                         kv_format=tt.KVFormat(16, kview.stride))
        attn.encode_gate_mul(out[t], gate, hq * hd)
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    got = host(out).reshape(steps, -1)
    got_keys = host(device_view(kv.k_slot(0, cached), steps * row, torch.float16)).reshape(steps, hkv, hd)
    # against the reference model's outputs: the north star's bar
    err = np.abs(got - want_out).max()
    key_err = np.abs(got_keys - want_keys)
    print(f"{name}: max abs error vs reference model {err:.2e} (bar {TOL}); K rows {key_err.max():.2e}")
    assert err <= TOL
    assert (key_err <= TOL + np.abs(want_keys) * 2.0 ** -9).all()
    # and against the oracle's statements chained with the same fp16 stores
    o_out, o_keys = _oracle_attention_chain(c, fp16_points=True)
    assert np.abs(got - o_out).max() <= TOL
    assert (np.abs(got_keys - o_keys) <= np.abs(o_keys) * 2.0 ** -9 + 1e-4).all()
    kv.close()


def test_gdn_decode_chain_matches_reference_model():
    c = mq.gdn_inputs()
    gold = np.load(os.path.join(GOLD, "qwen35_gdn.npz"))
    lin = tt.LinearAttentionConfig(c["hk"], c["hv"], c["dk"], c["dv"], c["conv_k"])
    cfg = tt.ArchConfig([tt.LINEAR], 2, 256, 2, 256, 0, lin)
    states = tt.GDNStateManager(cfg)
    n_state, n_tail = c["hv"] * c["dv"] * c["dk"], (c["conv_k"] - 1) * lin.qkv_dim
    state = device_view(states.state_slot(0), n_state)
    tail = device_view(states.conv_tail_slot(0), n_tail, torch.float16)
    gdn = tt.GDN(context(), lin)
    conv_w, a_log, dt_bias, norm_w = (dev(c[k], torch.bfloat16) for k in ("conv_w", "a_log", "dt_bias", "norm_w"))
    qkv, z, a, b = dev(c["qkv"]), dev(c["z"]), dev(c["a"]), dev(c["b"])
    conv = torch.empty(lin.qkv_dim, device="cuda", dtype=torch.float16)
    y = torch.empty(c["tokens"], lin.value_dim, device="cuda", dtype=torch.float16)
    out = torch.empty(c["tokens"], lin.value_dim, device="cuda", dtype=torch.float16)
    for t in range(c["tokens"]):
        gdn.encode_conv_decode(tail, qkv[t], conv_w, conv)
        gdn.encode_qk_norm(conv)
        gdn.encode_delta_step_decode(conv, a[t], b[t], a_log, dt_bias, state, y[t])
        gdn.encode_gated_norm(y[t], z[t], norm_w, out[t])
    torch.cuda.synchronize()
    assert context().poll_status() == 0
    got = host(out)
    err = np.abs(got - gold["out"])
    print(f"gdn chain: max abs error vs reference model {err.max():.2e}, max |want| {np.abs(gold['out']).max():.2f}")
    # bars explained in tests/test_oracle.py::test_gdn_oracle_matches_reference_model
    assert (err <= gdn_chain_bar(c, gold["out"]) + np.abs(gold["out"]) * 2.0 ** -10).all()
    assert (err <= np.maximum(2e-2, 4e-2 * np.abs(gold["out"]))).all()
    got_state = host(state).reshape(c["hv"], c["dv"], c["dk"])
    assert np.abs(got_state[::8, ::32, :] - gold["state_rows"]).max() < 5e-4
    assert np.array_equal(host(tail).reshape(c["conv_k"] - 1, -1), gold["tail"])
    # against the oracle chain with the same fp16 stores: y within the bar, output within the bar
    # times the gated norm's gain
    o_out, ch = _oracle_gdn_chain(c, fp16_points=True)
    assert np.abs(got_state - ch.state).max() <= 1e-4
    assert (np.abs(got - o_out) <= gdn_chain_bar(c, o_out)).all()
    states.close()
