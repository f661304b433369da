"""Column-sharded linear for large-N projections: the only multi-GPU part of the path.

A weight [K, N] (or [N, K] when trans_b) is split along N, the output-channel axis, across the ranks of one
box; per-output-channel scales / zero points / vector bias split the same way.  Every rank computes
``Y[:, n0:n1]`` from the full (replicated) activation with the same kernels as a single GPU — the K split
inside the kernels depends on K and M alone, so the bytes equal the single-GPU result — and ONE all-gather of
the 1-byte outputs follows.  There is no other data-path collective.

The reference has no multi-device code at all (one ``CudaExecutionContext`` = one device,
src/kernel/cuda/runtime.cu:318-321, 453-472); the single-GPU result is the oracle for this module.
"""
from __future__ import annotations

from typing import Callable, Tuple


def shard_bounds(n: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """Columns [n0, n1) owned by `rank`: equal blocks of `align` columns, the remainder spread over the first
    ranks, so every shard starts on a TMA-friendly boundary.  Ranks beyond the last block get an empty range."""
    if world <= 0 or not 0 <= rank < world or n < 0:
        raise ValueError("bad shard request")
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * align, n), min(b1 * align, n)


def slice_weight(w, n0: int, n1: int, trans_b: bool):
    """The rank's dense slice of the weight (a copy: the kernels take dense row-major weights)."""
    part = w[n0:n1] if trans_b else w[:, n0:n1]
    return part.contiguous() if hasattr(part, "contiguous") else part.copy()


class ShardedLinear:
    """Y = gather_n(f(A, W[:, shard])) on `world` ranks.

    compute(a, out_block) runs this rank's slice (on the GPU: one C-ABI call writing [M, n1-n0] bytes with row
    stride `width`); `dist` is ``torch.distributed`` (NCCL on the GPUs, gloo in the CPU tests).  One
    ``all_gather_into_tensor`` of equal, padded blocks follows.  For M == 1 and equal shards the gathered
    buffer IS the row-major [1, N] output; otherwise the [world, M, width] blocks are interleaved by one copy.
    """

    def __init__(self, n: int, world: int, rank: int, compute: Callable, dist=None, align: int = 128):
        self.n, self.world, self.rank = n, world, rank
        self.bounds = [shard_bounds(n, world, r, align) for r in range(world)]
        self.n0, self.n1 = self.bounds[rank]
        self.compute = compute
        self.dist = dist
        self.equal = len({b[1] - b[0] for b in self.bounds}) == 1

    @property
    def width(self) -> int:
        """Width of the padded per-rank block: the widest shard."""
        return max(b1 - b0 for b0, b1 in self.bounds)

    def forward(self, a, local_out, gathered, full_out=None):
        """local_out: [M, width] (this rank fills its first n1-n0 columns); gathered: [world, M, width];
        full_out: [M, N] destination, needed unless M == 1 with equal shards."""
        self.compute(a, local_out)
        if self.world == 1:
            return local_out[:, : self.n1 - self.n0]
        m = local_out.shape[0]
        # concatenation along dim 0: rank r's [M, width] block lands at rows r*M .. (r+1)*M
        self.dist.all_gather_into_tensor(gathered.view(self.world * m, self.width), local_out)
        if self.equal and m == 1:
            return gathered.view(1, self.n)
        if self.equal:
            full_out.view(m, self.world, self.width).copy_(gathered.transpose(0, 1))
            return full_out
        for r, (b0, b1) in enumerate(self.bounds):
            full_out[:, b0:b1].copy_(gathered[r, :, : b1 - b0])
        return full_out
