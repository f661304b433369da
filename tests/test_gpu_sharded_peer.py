"""Column-sharded linear with the library-free gather on two real GPUs (skipped on a one-GPU box)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_two_rank_peer_gather_matches_single_gpu():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                           "--master-port", "29533", os.path.join(here, "peer_worker.py")], capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0 and "PEER_GATHER_OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-2000:]
