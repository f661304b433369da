"""One rank of the multi-GPU gather test (launched by tests/test_gpu_sharded_peer.py through torch.distributed.run).

Every rank holds the full seeded problem, computes the single-GPU result locally as the oracle for the gather, then
runs several gathered steps through PeerGather / forward_peer and compares bytes."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import infer_b200 as B  # noqa: E402
from infer_b200.sharded import PeerGather, ShardedLinear, forward_peer, slice_weight  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    lib = B.lib()
    failures = 0
    for m, k, n in ((1, 2048, 4096), (16, 1024, 2048 + 128), (200, 512, 1024)):
        rng = np.random.default_rng(1000 + m)
        a = torch.from_numpy(rng.integers(0, 0x78, (m, k), dtype=np.uint8)).cuda()
        w = torch.from_numpy(rng.integers(0, 0x78, (k, n), dtype=np.uint8)).cuda()
        full = torch.empty((m, n), dtype=torch.uint8, device="cuda")
        d_full = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=full, a_scale=0.5, w_scale=2.0 ** -6,
                                   out_scale=float(k) / 64)
        ws_full = B.linear_workspace(torch, d_full)
        B.fp8_linear(d_full)
        torch.cuda.synchronize()
        shard = ShardedLinear(n, world, rank, compute=None, dist=dist)
        w_local = slice_weight(w, shard.n0, shard.n1, False)
        d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=shard.n1 - shard.n0, a=a, w=w_local, out=None, a_scale=0.5,
                              w_scale=2.0 ** -6, out_scale=float(k) / 64, weights_static=True)
        d.out = full.data_ptr()  # any valid pointer: workspace sizing only looks at shapes
        ws = B.linear_workspace(torch, d)
        stream = B.current_stream()
        for fold_signal in (False, True):  # a signal / wait kernel behind every step; signalling folded into the linear kernels
            gather = PeerGather(lib, dist, world, rank, m, n)
            for step in range(6):
                parity = forward_peer(shard, gather, d, lambda desc, s: lib.fth_b200_fp8_linear(C.byref(desc), s), stream,
                                      fold_signal=fold_signal)
                if fold_signal and step % 2 == 1:
                    continue  # let the next step's kernel do the waiting: its result is checked below all the same
                if fold_signal:
                    gather.wait(stream)
                torch.cuda.synchronize()
                got = gather.view(torch, parity)
                if not torch.equal(got, full):
                    failures += 1
                    print(f"rank {rank}: M={m} fold={fold_signal} step {step}: {(got != full).sum().item()} bytes differ", flush=True)
            if B.device_status() != 0:
                failures += 1
            torch.cuda.synchronize()
            dist.barrier()
            gather.close()
        del ws, ws_full
    t = torch.tensor([failures], device="cuda")
    dist.all_reduce(t)
    if rank == 0:
        print("PEER_GATHER_OK" if int(t.item()) == 0 else f"PEER_GATHER_FAILED {int(t.item())}", flush=True)
    dist.destroy_process_group()
    return 0 if int(t.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
