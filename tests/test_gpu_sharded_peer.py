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


def test_one_process_drives_two_devices():
    """One host process, one session per GPU (the reference's model: a CudaExecutionContext binds to whatever device is
    current when it is created, src/kernel/cuda/runtime.cu:318-321): every kernel family that raises its dynamic
    shared-memory limit must do so on each device it runs on, and the SM count and status word are per device."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import numpy as np

    import infer_b200 as B
    import oracle as O
    from tests import util
    shapes = [(1, 1024, 2048), (16, 8192, 4096), (64, 1024, 1024), (300, 512, 640), (3, 96, 80)]  # cluster, swapped + reduce, swapped 64, pair, CUDA cores
    try:
        for device in (0, 1, 0):
            torch.cuda.set_device(device)
            for m, k, n in shapes:
                case = util.make_fp8_linear(O.E4M3, m, k, n, seed=m + k + n)
                a, w = torch.from_numpy(case["a"]).cuda(), torch.from_numpy(case["w"]).cuda()
                out = torch.zeros((m, n), dtype=torch.uint8, device="cuda")
                d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=out, a_scale=case["sa"],
                                      w_scale=case["sw"], out_scale=case["so"])
                keep = B.linear_workspace(torch, d)
                B.fp8_linear(d, stream=B.current_stream())
                torch.cuda.synchronize()
                want = O.fp8_linear(O.OP_MATMUL, O.E4M3, case["a"], case["sa"], case["w"], case["sw"], case["so"])
                assert util.fp8_code_distance(out.cpu().numpy(), want).max() <= 1, (device, m, k, n)
                assert B.device_status() == 0
                del keep
    finally:
        torch.cuda.set_device(0)
