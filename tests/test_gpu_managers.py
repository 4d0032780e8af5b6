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


def test_speculative_restore_is_ordered_on_a_non_blocking_stream():
    # GDNStateManager.encodeSpeculativeRestore(commandBuffer:) (GDNStateManager.swift:265-292) is a blit
    # in the verify pass's command buffer. Here: a 3-row verify step that checkpoints the state after
    # row 0, then the restore, then a read-back, all enqueued on one NON-blocking stream with no host
    # synchronisation in between -- the legacy default stream would not be ordered with any of it.
    r = np.random.default_rng(77)
    lin = tt.LinearAttentionConfig(2, 4, 128, 128, 4)
    cfg = tt.ArchConfig([tt.LINEAR], 2, 256, 2, 256, 0, lin)
    g = tt.GDNStateManager(cfg, enable_speculative_checkpoint=True)
    n_state = 4 * 128 * 128
    rows = 3
    unit = lambda x: x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)
    conv = rounded(np.concatenate([unit(r.normal(size=(rows, 2, 128))).reshape(rows, -1) / np.sqrt(128),
                                   unit(r.normal(size=(rows, 2, 128))).reshape(rows, -1),
                                   r.normal(size=(rows, 4 * 128))], 1))
    a, b = rounded(r.normal(size=(rows, 4))), rounded(r.normal(size=(rows, 4)))
    s0 = (0.02 * r.normal(size=(4, 128, 128))).astype(np.float32)
    state = device_view(g.state_slot(0), n_state)
    spec = device_view(g.speculative_state_slot(0), n_state)
    conv_d, a_d, b_d = dev(conv), dev(a), dev(b)
    z = torch.zeros(4, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(rows, 4 * 128, device="cuda", dtype=torch.float16)
    after = torch.empty(n_state, device="cuda")
    big = torch.empty(64 << 20, device="cuda")
    torch.cuda.synchronize()
    side = torch.cuda.Stream()            # torch side streams are created non-blocking
    with torch.cuda.stream(side):
        state.copy_(dev(s0, torch.float32).view(-1))
        big.normal_()                     # keeps the stream busy so that an unordered copy would run early
        tt.GDN(context(), lin).encode_delta_step_prefill(conv_d, a_d, b_d, z, z, state, y, rows, checkpoint_state=spec)
        g.speculative_restore(side)
        after.copy_(state)
    side.synchronize()
    assert context().poll_status() == 0
    _, want_all, want_ck = oracle.gdn_step_rows(conv, a, b, np.zeros(4), np.zeros(4), 2, 4, 128, 128, s0, want_checkpoint=True)
    got = host(after).reshape(4, 128, 128)
    assert np.abs(got - want_ck).max() <= 1e-5            # the state after row 0 alone, not after all three rows
    assert np.abs(got - want_all).max() > 1e-4
    g.close()


def test_reserve_on_a_bound_stream_keeps_rows_written_there():
    cfg = tt.ArchConfig([tt.FULL], 2, 256, 2, 256, 0, tt.LinearAttentionConfig(16, 32, 128, 128, 4))
    kv = tt.KVCacheManager(cfg, max_context=20000)
    side = torch.cuda.Stream()
    kv.bind_stream(side)
    n = 8192
    rows = torch.randn(n, 512, device="cuda").half()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        device_view(kv.k_slot(0, 0), n * 512, torch.float16).copy_(rows.view(-1))   # enqueued, not yet done
        kv.advance(0, n)
        kv.reserve(n + 1)                                                            # grows: the copy must follow the write
        assert kv.capacity(0) == 16384
        back = device_view(kv.k_slot(0, 0), n * 512, torch.float16).clone()
    side.synchronize()
    assert torch.equal(back.view(n, 512), rows)
    kv.close()


def test_write_rows_scatters_a_decode_batch_in_one_launch():
    cfg = tt.ArchConfig([tt.FULL], 2, 256, 2, 256, 0, tt.LinearAttentionConfig(16, 32, 128, 128, 4))
    slots_n = 40
    kv = tt.KVCacheManager(cfg, max_context=5000, slots=slots_n)
    r = np.random.default_rng(4)
    k = torch.randn(slots_n, 512, device="cuda").half(); v = torch.randn(slots_n, 512, device="cuda").half()
    slots = r.permutation(slots_n).astype(np.uint32); positions = r.integers(0, 5000, size=slots_n).astype(np.uint32)
    before = device_view(kv.k_slot(0, 0, 0), slots_n * 5000 * 512, torch.float16).clone()
    kv.write_rows(0, slots, positions, k, v, 1024)
    torch.cuda.synchronize()
    after = device_view(kv.k_slot(0, 0, 0), slots_n * 5000 * 512, torch.float16).view(slots_n, 5000, 512)
    changed = torch.zeros(slots_n, 5000, dtype=torch.bool, device="cuda")
    for i in range(slots_n):
        s, p = int(slots[i]), int(positions[i])
        assert torch.equal(after[s, p], k[i])
        assert torch.equal(device_view(kv.v_slot(0, p, s), 512, torch.float16), v[i])
        changed[s, p] = True
    assert torch.equal(after[~changed], before.view(slots_n, 5000, 512)[~changed])   # nothing else was touched
    kv.close()
