"""The multi-rank plumbing of the path on CPU: two gloo ranks (no GPU needed)."""
import os
import socket
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["TT_ROOT"])
import oracle
from tinytitan_b200 import sharding

dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['TT_PORT']}",
                        rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()

# (1) one long session, KV split along the sequence; per-rank partial -> all-gather -> merge
r = np.random.default_rng(123)
hq, hkv, hd, s = 8, 2, 64, 1001
q = r.normal(size=(hq, hd)).astype(np.float32)
k = r.normal(size=(s, hkv * hd)).astype(np.float32)
v = r.normal(size=(s, hkv * hd)).astype(np.float32)
lo, hi = sharding.kv_split_ranges(s, world)[rank]
m = np.zeros(hq, np.float32); d = np.zeros(hq, np.float32); o = np.zeros((hq, hd), np.float32)
for h in range(hq):
    # the rank only holds rows [lo, hi): local row 0 is logical position lo
    m[h], d[h], o[h] = oracle.attn_partial(q[h], k[lo:hi], v[lo:hi], hkv, h // (hq // hkv), 0, hi - lo, 0.125)
mg, dg, og = sharding.exchange_partials(torch.from_numpy(m), torch.from_numpy(d), torch.from_numpy(o))
assert mg.shape == (world, hq) and og.shape == (world, hq, hd) and og.is_contiguous()
out = np.stack([oracle.attn_combine(mg[:, h].numpy(), dg[:, h].numpy(), og[:, h].numpy()) for h in range(hq)])
want = oracle.attn_decode(q, k.reshape(s, hkv, hd), v.reshape(s, hkv, hd), hkv, 0.125)
assert np.abs(out - want).max() < 2e-6, np.abs(out - want).max()

# (2) independent sessions: every session is owned by exactly one rank, no exchange on the data path
lens = [int(x) for x in np.random.default_rng(5).integers(1024, 32769, size=32)]
mine = sharding.shard_sessions(lens, world)[rank]
owned = torch.zeros(32, dtype=torch.int64); owned[mine] = 1
dist.all_reduce(owned)
assert torch.all(owned == 1)
keys = torch.tensor([float(sum(lens[i] for i in mine))])
allk = [torch.zeros(1) for _ in range(world)]
dist.all_gather(allk, keys)
assert abs(sum(x.item() for x in allk) - sum(lens)) < 1
dist.barrier()
dist.destroy_process_group()
print("RANK_OK", rank)
'''


def test_two_gloo_ranks_kv_split_and_session_sharding(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", TT_PORT=str(port), TT_ROOT=ROOT,
                   CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out.decode())
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"RANK_OK {rank}" in out, out
