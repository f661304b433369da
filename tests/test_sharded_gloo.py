"""CPU, world size 2 over gloo: the column-sharding host logic (bounds, padded all-gather, interleave) of
infer_b200/sharded.py.  The per-rank compute is injected (here: the CPU oracle), so what is under test is the
partition and the exchange; the single-process result is the expected output, byte for byte."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from infer_b200.sharded import ShardedLinear, shard_bounds, slice_weight
from tests import util


def test_shard_bounds_cover_and_align():
    for n, world in [(28672, 8), (28672, 4), (3072, 2), (1000, 4), (128, 8), (77, 2)]:
        bounds = [shard_bounds(n, world, r) for r in range(world)]
        assert bounds[0][0] == 0 and bounds[-1][1] == n
        for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
            assert a1 == b0 and a0 <= a1
        assert all(b0 % 128 == 0 for b0, b1 in bounds if b1 > b0)
    assert [shard_bounds(28672, 8, r)[1] - shard_bounds(28672, 8, r)[0] for r in range(8)] == [3584] * 8
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def _worker(rank, world, port, m, n, trans_b, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = util.make_int8_linear(m, 256, n, seed=11, trans_b=trans_b)
        n0, n1 = shard_bounds(n, world, rank)
        w = slice_weight(case["w"], n0, n1, trans_b)

        def compute(a, out_block):
            if n1 > n0:
                y = O.int8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, a.numpy(), case["sa"], 0, w, case["ws"][n0:n1], None,
                                  case["so"], 0, trans_b=trans_b)
                out_block[:, : n1 - n0] = torch.from_numpy(y)

        sl = ShardedLinear(n, world, rank, compute, dist)
        local = torch.zeros((m, sl.width), dtype=torch.int8)
        gathered = torch.zeros((world, m, sl.width), dtype=torch.int8)
        full = torch.zeros((m, n), dtype=torch.int8)
        out = sl.forward(torch.from_numpy(case["a"]), local, gathered, full)
        want = O.int8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, case["a"], case["sa"], 0, case["w"], case["ws"], None, case["so"], 0,
                             trans_b=trans_b)
        results[rank] = bool(np.array_equal(out.numpy().reshape(m, n), want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,n,trans_b", [(1, 512, False), (4, 512, False), (3, 1000, True), (1, 384, False)])
def test_two_rank_sharded_linear_equals_single_process(m, n, trans_b):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, m, n, trans_b, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}


def test_forward_peer_points_the_descriptor_at_every_rank(monkeypatch):
    """Host logic of the library-free gather, no GPU: the step's parity picks the buffers, this rank's column
    offset is applied to its own and to every peer's address, and the step ends with a sync of that epoch."""
    import infer_b200 as B
    from infer_b200.sharded import ShardedLinear, forward_peer

    class FakeGather:
        world, rank, n, elem = 4, 2, 1024, 1
        epoch = 0
        synced = []

        def buffer(self, r, parity):
            return 0x10000000 * (r + 1) + parity * 0x100000

        def sync(self, stream):
            self.synced.append(self.epoch)

    shard = ShardedLinear(1024, 4, 2, compute=None)
    gather = FakeGather()
    d = B.Fp8LinearDesc()
    seen = []
    for step in (1, 2, 3):
        parity = forward_peer(shard, gather, d, lambda desc, s: seen.append((desc.out, desc.ldo, desc.gather_peers, list(desc.gather_out[:3]))) or 0, None)
        assert parity == step & 1
        out, ldo, peers, others = seen[-1]
        assert out == gather.buffer(2, parity) + shard.n0 and ldo == 1024 and peers == 3
        assert others == [gather.buffer(r, parity) + shard.n0 for r in (0, 1, 3)]
    assert gather.synced == [1, 2, 3]
    with pytest.raises(RuntimeError):
        forward_peer(shard, gather, d, lambda desc, s: -3, None)
