"""KV-cache manager on device memory: rows survive growth, slots stay disjoint (B200 only)."""
import numpy as np
import pytest
import torch

import oracle
import tinytitan_b200 as tt
from gpu_util import TOL, context, dev, host, rounded, device_view

pytestmark = pytest.mark.gpu


def test_growth_preserves_rows_and_attention_reads_views():
    cfg = tt.ArchConfig([tt.LINEAR, tt.FULL], 2, 256, 2, 256, 0, tt.LinearAttentionConfig(16, 32, 128, 128, 4))
    kv = tt.KVCacheManager(cfg, max_context=40000, slots=3)
    layer, hq, hkv, hd = 1, 16, 2, 256
    stride = kv.stride(layer)
    assert stride == 1024 and kv.capacity(layer) == 8192
    r = np.random.default_rng(0)
    lens = {0: 50, 2: 8192}
    data = {}
    for slot, n in lens.items():
        k = rounded(r.normal(size=(n, hkv * hd))); v = rounded(r.normal(size=(n, hkv * hd)))
        data[slot] = (k, v)
        kdst = device_view(kv.k_slot(layer, 0, slot), n * hkv * hd, torch.float16)
        vdst = device_view(kv.v_slot(layer, 0, slot), n * hkv * hd, torch.float16)
        kdst.copy_(dev(k).view(-1)); vdst.copy_(dev(v).view(-1))
        kv.advance(slot, n)
    torch.cuda.synchronize()
    kv.reserve(8193, slot=2)                     # doubles to 16384; every slot's live rows move
    assert kv.capacity(layer) == 16384
    attn = tt.Attention(context())
    for slot, n in lens.items():
        kview, vview = kv.key_view(layer, slot), kv.value_view(layer, slot)
        assert kview.offset == slot * 16384 * stride and kview.valid_token_count == n
        q = rounded(r.normal(size=(hq, hd)))
        out = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
        attn.encode_full(dev(q), kview.address, vview.address, out, hd, hq, hkv, n, scale=0.0625,
                         kv_format=tt.KVFormat(16, kview.stride))
        torch.cuda.synchronize()
        k, v = data[slot]
        want = oracle.attn_decode(q, k.reshape(n, hkv, hd), v.reshape(n, hkv, hd), hkv, 0.0625)
        assert np.abs(host(out) - want).max() <= TOL
    kv.rewind(10, slot=0)
    assert kv.position(0) == 10 and kv.position(2) == 8192
    kv.close()


def test_snapshot_round_trip_on_device_memory():
    cfg = tt.ArchConfig([tt.FULL, tt.LINEAR], 2, 256, 2, 256, 0, tt.LinearAttentionConfig(16, 32, 128, 128, 4))
    a = tt.KVCacheManager(cfg, max_context=4096)
    g = tt.GDNStateManager(cfg)
    n = 300
    k = torch.randn(n, 512, device="cuda").half(); v = torch.randn(n, 512, device="cuda").half()
    device_view(a.k_slot(0, 0), n * 512, torch.float16).copy_(k.view(-1))
    device_view(a.v_slot(0, 0), n * 512, torch.float16).copy_(v.view(-1))
    a.advance(0, n)
    st = torch.randn(32 * 128 * 128, device="cuda")
    device_view(g.state_slot(1, 0), st.numel()).copy_(st)
    torch.cuda.synchronize()
    kv_payload, gdn_payload = a.snapshot(), g.snapshot()
    assert len(kv_payload) == 2 * n * 1024 and len(gdn_payload) == g.state_bytes_per_layer + g.conv_tail_bytes_per_layer
    b = tt.KVCacheManager(cfg, max_context=4096); g2 = tt.GDNStateManager(cfg)
    b.restore_snapshot(n, kv_payload); g2.restore_snapshot(gdn_payload)
    assert b.position(0) == n
    assert torch.equal(device_view(b.k_slot(0, 0), n * 512, torch.float16), k.view(-1))
    assert torch.equal(device_view(b.v_slot(0, 0), n * 512, torch.float16), v.view(-1))
    assert torch.equal(device_view(g2.state_slot(1, 0), st.numel()), st)
    for m in (a, b, g, g2):
        m.close()
