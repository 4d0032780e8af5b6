"""Worker of tests/test_gpu_multi.py: one process per GPU (launched by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tinytitan_b200 as tt
from tinytitan_b200 import sharding


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = tt.Context(local)
    attn = tt.Attention(ctx)
    hq, hkv, hd, s = 16, 2, 256, int(os.environ.get("TT_TEST_SEQ", "50001"))

    # the same seeded session on every rank; each rank then keeps only its slice of the rows
    g = torch.Generator(device="cuda"); g.manual_seed(99)
    q = torch.randn(hq, hd, device="cuda", generator=g).half()
    k = torch.randn(s, hkv * hd, device="cuda", generator=g).half()
    v = torch.randn(s, hkv * hd, device="cuda", generator=g).half()
    lo, hi = sharding.kv_split_ranges(s, world)[rank]
    k_local, v_local = k[lo:hi].contiguous(), v[lo:hi].contiguous()

    lc = sharding.LongContextDecode(attn, hd, hq, hkv, 0.0625)
    out = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
    for _ in range(3):
        lc.step(q, k_local, v_local, hi - lo, out)
    torch.cuda.synchronize()

    # the CPU oracle over ALL rows, computed once on rank 0 and broadcast: the bar every path below is held to
    want = torch.empty(hq, hd, device="cuda")
    if rank == 0:
        import oracle
        f = lambda t: t.float().cpu().numpy()
        want.copy_(torch.from_numpy(oracle.attn_decode_split(f(q), f(k).reshape(s, hkv, hd), f(v).reshape(s, hkv, hd), hkv,
                                                             0.0625, s, n_chunks=64)))
    dist.broadcast(want, 0)
    TOL = 2e-3
    err = (out.float() - want).abs().max().item()
    assert err <= TOL, f"rank {rank}: split-KV merge over NCCL differs from the oracle by {err}"
    full = torch.empty_like(out)
    attn.encode_full(q, k, v, full, hd, hq, hkv, s, scale=0.0625)      # single-GPU answer over all rows
    torch.cuda.synchronize()
    err = (out.float() - full.float()).abs().max().item()
    assert err <= 1e-3, f"rank {rank}: split-KV merge differs from single-GPU attention by {err}"
    # every rank ends with the same merged row
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    assert all(torch.equal(gathered[0], t) for t in gathered)

    # the same merge with exchange and merge fused in one kernel over peer memory: bit-identical
    # inputs per rank, so the result may differ from the all-gather path only by summation order
    fused = sharding.LongContextDecode(attn, hd, hq, hkv, 0.0625, fused=True)
    out_f = torch.empty_like(out)
    for _ in range(5):     # several steps: both parities of the double-buffered slots are reused
        out_f.zero_()
        fused.step(q, k_local, v_local, hi - lo, out_f)
    torch.cuda.synchronize()
    assert ctx.poll_status() == 0
    err = (out_f.float() - want).abs().max().item()
    assert err <= TOL, f"rank {rank}: fused exchange differs from the oracle by {err}"
    err = (out_f.float() - full.float()).abs().max().item()
    assert err <= 1e-3, f"rank {rank}: fused exchange differs from single-GPU attention by {err}"
    assert (out_f.float() - out.float()).abs().max().item() <= 1e-3
    # the exchange kernel alone, fed with a triple computed beforehand (the two-call form)
    m_l = torch.empty(hq, device="cuda"); d_l = torch.empty(hq, device="cuda"); o_l = torch.empty(hq, hd, device="cuda")
    out_t = torch.zeros_like(out)
    for _ in range(3):
        attn.encode_partial(q, k_local, v_local, hd, hq, hkv, hi - lo, 0, m_l, d_l, o_l, scale=0.0625)
        attn.encode_exchange_combine(m_l, d_l, o_l, fused.exchange, hq, hd, out_t)
    torch.cuda.synchronize()
    assert ctx.poll_status() == 0
    assert (out_t.float() - full.float()).abs().max().item() <= 1e-3
    assert (out_t.float() - want).abs().max().item() <= TOL
    if rank == 0:
        print(f"ORACLE_MAX_ABS_ERR world={world} S={s} nccl={(out.float() - want).abs().max().item():.2e} "
              f"fused={(out_f.float() - want).abs().max().item():.2e}")
    # device time of one step, both ways (max over ranks is taken by the reader of the log)
    def timed(fn, reps=50):
        for _ in range(5):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    t_nccl = timed(lambda: lc.step(q, k_local, v_local, hi - lo, out))
    t_fused = timed(lambda: fused.step(q, k_local, v_local, hi - lo, out_f))
    if rank == 0:
        print(f"SPLIT_KV_STEP_MS world={world} S={s} nccl={t_nccl:.4f} fused={t_fused:.4f}")
    fused.close()

    # independent sessions: each is decoded on exactly one rank, nothing is exchanged on the data path
    lens = [257 * (i + 1) for i in range(8)]
    mine = sharding.shard_sessions(lens, world)[rank]
    done = torch.zeros(len(lens), device="cuda")
    for i in mine:
        kk = torch.randn(lens[i], hkv * hd, device="cuda", generator=g).half()
        o = torch.empty(hq, hd, device="cuda", dtype=torch.float16)
        attn.encode_full(q, kk, kk, o, hd, hq, hkv, lens[i], scale=0.0625)
        done[i] = 1
    dist.all_reduce(done)
    assert torch.all(done == 1)
    assert ctx.poll_status() == 0
    dist.barrier()
    dist.destroy_process_group()
    print(f"RANK_OK {rank}")


if __name__ == "__main__":
    main()
