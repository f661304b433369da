"""Column-sharded linear for large-N projections: the only multi-GPU part of the path.

A weight [K, N] (or [N, K] when trans_b) is split along N, the output-channel axis, across the ranks of one
box; per-output-channel scales / zero points / vector bias split the same way.  Every rank computes
``Y[:, n0:n1]`` from the full (replicated) activation with the same kernels as a single GPU — the K split
inside the kernels depends on K and M alone, so the bytes equal the single-GPU result — and ONE all-gather of
the 1-byte outputs follows.  There is no other data-path collective.

On the GPUs the gather needs no collective library at all: ``PeerGather`` maps every rank's output buffer into
every rank (CUDA IPC), the linear kernels store their columns into all of them from their own epilogue, and one
small signal / wait kernel ends the step (``ShardedLinear.forward_peer``).  The NCCL path stays for hosts where
peer mapping is not available and for the CPU (gloo) tests of the host logic.

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


class PeerGather:
    """Every rank's [M, N] output buffer, mapped into every rank of one box, with the flags that end a step.

    Two buffers per rank, used by step parity: a rank can run at most one step ahead of the slowest one (it
    cannot pass step s before every rank has signalled s), so the buffer of step s is not written again until
    everybody has consumed it.  `dist` is only used to exchange the 64-byte handles at set-up.

    With `torch` given (and world > 1) the buffers are first tried as torch symmetric memory
    (torch.distributed._symmetric_memory): the same peer-mapped addresses, plus — where the box has NVLink multicast
    (NVLS) — one multicast address per buffer (`multicast`, 0 if there is none), which the dense kernel stores to once
    instead of once per peer.  If that set-up is not available the CUDA IPC path below is used.
    """

    def __init__(self, lib, dist, world: int, rank: int, m: int, n: int, elem_bytes: int = 1, torch=None):
        import ctypes as C
        self.lib, self.world, self.rank = lib, world, rank
        self.m, self.n, self.elem = m, n, elem_bytes
        self.block = (m * n * elem_bytes + 255) // 256 * 256
        total = 2 * self.block + 256  # two output buffers, then uint32 flags[world]
        self.multicast = 0
        self._symmetric = None
        if torch is not None and world > 1 and self._try_symmetric(torch, dist, total):
            self.flags = (C.c_void_p * world)(*[b + 2 * self.block for b in self.base])
            self._world, self._rank = C.c_int32(world), C.c_int32(rank)
            self.epoch = 0
            dist.barrier()
            return
        own = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        created = lib.fth_b200_peer_buffer_create(C.c_size_t(total), C.byref(own), handle) == 0
        # every rank takes part in every exchange, whatever happened locally, so that a failure on one rank ends in the
        # same exception on all of them instead of a collective that never completes
        handles = [bytes(handle) if created else None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle) if created else None)
        self.base = [0] * world
        self.base[rank] = own.value if created else 0
        opened = created and all(h is not None for h in handles)
        if opened:
            for r in range(world):
                if r == rank:
                    continue
                ptr = C.c_void_p()
                peer_handle = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                if lib.fth_b200_peer_buffer_open(peer_handle, C.byref(ptr)) != 0:
                    opened = False
                    break
                self.base[r] = ptr.value
        verdicts = [opened] * world
        if world > 1:
            dist.all_gather_object(verdicts, opened)
        if not all(verdicts):
            self.close()
            raise RuntimeError("peer-mapped output buffers are not available on this box (CUDA IPC create / open failed on some rank)")
        self.flags = (C.c_void_p * world)(*[b + 2 * self.block for b in self.base])
        self._world, self._rank = C.c_int32(world), C.c_int32(rank)
        self.epoch = 0
        if world > 1:
            dist.barrier()  # nobody stores into a buffer before every rank has mapped it

    def _try_symmetric(self, torch, dist, total: int) -> bool:
        """Allocates the buffers as symmetric memory; every rank reports, and all ranks take the same branch."""
        ok, tensor, handle = True, None, None
        try:
            import torch.distributed._symmetric_memory as symm
            tensor = symm.empty(total, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            tensor.zero_()
            torch.cuda.synchronize()
            handle = symm.rendezvous(tensor, dist.group.WORLD)
            base = [int(p) for p in handle.buffer_ptrs]
            ok = len(base) == self.world and all(base)
        except Exception:  # set-up not available here: the IPC path takes over, on every rank alike
            ok = False
        verdicts = [ok] * self.world
        dist.all_gather_object(verdicts, ok)
        if not all(verdicts):
            return False
        self.base = base
        multicast = int(handle.multicast_ptr) if getattr(handle, "has_multicast_support", False) or getattr(handle, "multicast_ptr", 0) else 0
        present = [multicast != 0] * self.world
        dist.all_gather_object(present, multicast != 0)
        self.multicast = multicast if all(present) else 0
        self._symmetric = (tensor, handle)
        return True

    def buffer(self, r: int, parity: int) -> int:
        """Device address of rank r's output buffer for steps of this parity, as seen from this rank."""
        return self.base[r] + parity * self.block

    def multicast_buffer(self, parity: int) -> int:
        """The multicast address of the buffers of this parity (a store there lands in every rank's), or 0."""
        return self.multicast + parity * self.block if self.multicast else 0

    def view(self, torch, parity: int):
        """This rank's gathered [M, N] buffer as a uint8 tensor of M * N * elem_bytes bytes per row block."""
        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.m, self.n * self.elem), "typestr": "|u1",
                                        "data": (self.buffer(self.rank, parity), False), "version": 3}
        return torch.as_tensor(raw, device="cuda")

    def sync(self, stream) -> None:
        """Signals this step to every rank and waits (on the stream) for theirs."""
        # step numbers are kept on the device (epoch 0), which makes the step replayable from a CUDA graph; the host
        # counter only picks the buffer parity
        if self.lib.fth_b200_gather_sync(self.flags, self._world, self._rank, 0, stream) != 0:
            raise RuntimeError("fth_b200_gather_sync failed")

    def wait(self, stream) -> None:
        """Consumer side of the signalling the linear kernels do themselves (gather_world in their descriptors): waits,
        on the stream, until every rank has published the step this rank published last."""
        if self.lib.fth_b200_gather_wait(self.flags, self._world, self._rank, stream) != 0:
            raise RuntimeError("fth_b200_gather_wait failed")

    def close(self) -> None:
        if self._symmetric is not None:
            self._symmetric = None  # torch frees the allocation with the tensor
            self.base = [0] * self.world
            self.multicast = 0
            return
        for r, b in enumerate(self.base):
            if b and r != self.rank:
                self.lib.fth_b200_peer_buffer_close(b)
        if self.base[self.rank]:
            self.lib.fth_b200_peer_buffer_destroy(self.base[self.rank])
        self.base = [0] * self.world


def point_at_step_buffers(shard: "ShardedLinear", gather: PeerGather, desc, parity: int, fold_signal: bool = False):
    """Points `desc` (this rank's linear descriptor, weights = its column slice) at the buffers of steps with this
    parity: its own block in its own buffer, and the same block in every other rank's.  fold_signal: the kernel also
    does the step signalling itself (no fth_b200_gather_sync behind it; consumers use PeerGather.wait)."""
    if fold_signal:
        desc.gather_world, desc.gather_rank = gather.world, gather.rank
        for r in range(gather.world):
            desc.gather_flags[r] = gather.flags[r]
    else:
        desc.gather_world = 0
    offset = shard.n0 * gather.elem
    desc.out = gather.buffer(gather.rank, parity) + offset
    desc.ldo = gather.n
    others = [r for r in range(gather.world) if r != gather.rank]
    desc.gather_peers = len(others)
    for i, r in enumerate(others):
        desc.gather_out[i] = gather.buffer(r, parity) + offset
    multicast = gather.multicast_buffer(parity) if hasattr(gather, "multicast_buffer") else 0
    desc.gather_multicast_out = multicast + offset if multicast else None
    return desc


def forward_peer(shard: "ShardedLinear", gather: PeerGather, desc, call, stream, prepared=None, fold_signal: bool = False):
    """One gathered step: `call(desc, stream)` launches the C ABI with the output pointed at the step's buffers, then
    the step is signalled.  `prepared` = (desc for even steps, desc for odd steps) from point_at_step_buffers saves
    the per-step pointer set-up (a decode step is a few microseconds of GPU time).  fold_signal: the kernel signals by
    itself and nothing else is launched; whoever reads the gathered buffer calls gather.wait(stream) first (the next
    step's kernel does that on its own).  Returns the parity of the buffer that holds the [M, N] result."""
    gather.epoch += 1
    parity = gather.epoch & 1
    step_desc = prepared[parity] if prepared is not None else point_at_step_buffers(shard, gather, desc, parity, fold_signal)
    rc = call(step_desc, stream)
    if rc != 0:
        raise RuntimeError(f"linear call failed: {rc}")
    if not fold_signal:
        gather.sync(stream)
    return parity
