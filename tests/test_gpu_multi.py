"""Two or more B200s: KV split of one long session with the NCCL merge, and session sharding."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("seq", ["50001", "262144"])       # a ragged split, and the long-context configuration's size
def test_kv_split_merge_and_session_sharding_over_nccl(seq, monkeypatch):
    monkeypatch.setenv("TT_TEST_SEQ", seq)
    world = min(torch.cuda.device_count(), 8)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multi_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for rank in range(world):
        assert f"RANK_OK {rank}" in r.stdout
