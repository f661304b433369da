"""Peer replicas of the output on ONE GPU: the "peers" are two more local buffers, so every kernel family's way of
writing them (from its own epilogue, or through the block copy behind it) is checked without a second device."""
import ctypes as C

import numpy as np
import pytest

import infer_b200 as B
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch


# (m, k, n, variant): cluster kernel, two-kernel split path, folded split (one launch; ragged last tile), CTA-pair dense kernel (ragged tile; four tiles per CTA pair, so
# the shared-memory tile behind its tile stores is reused), CUDA-core kernels
CASES = [(1, 1024, 2048, B.VARIANT_AUTO), (16, 8192, 8192, B.VARIANT_AUTO), (5, 1024, 128 * 119 + 48, B.VARIANT_AUTO), (48, 2048, 4096, B.VARIANT_AUTO),
         (300, 512, 640, B.VARIANT_AUTO), (512, 256, 256 * 74 * 2, B.VARIANT_AUTO), (4, 256, 384, B.VARIANT_SKINNY),
         (3, 96, 80, B.VARIANT_SIMT)]


@pytest.mark.parametrize("m,k,n,variant", CASES)
def test_fp8_output_reaches_every_replica(cuda, m, k, n, variant):
    torch = cuda
    rng = np.random.default_rng(m * 7 + n)
    a = torch.from_numpy(rng.integers(0, 0x78, (m, k), dtype=np.uint8)).cuda()
    w = torch.from_numpy(rng.integers(0, 0x78, (k, n), dtype=np.uint8)).cuda()
    width, col0 = n + 256, 128  # the block sits inside a wider row, as a column shard does
    bufs = [torch.full((m + 2, width), 0x5A, dtype=torch.uint8, device="cuda") for _ in range(3)]
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=None, a_scale=0.5, w_scale=2.0 ** -6,
                          out_scale=float(k) / 64, ldo=width, variant=variant, weights_static=True)
    d.out = bufs[0].data_ptr() + width + col0
    d.gather_peers = 2
    d.gather_out[0] = bufs[1].data_ptr() + width + col0
    d.gather_out[1] = bufs[2].data_ptr() + width + col0
    ws = B.linear_workspace(torch, d)
    if B.lib().fth_b200_fp8_linear_supported(C.byref(d)) != 0:
        pytest.skip("variant declines this shape")
    B.fp8_linear(d)
    torch.cuda.synchronize()
    assert B.device_status() == 0
    host = [b.cpu().numpy() for b in bufs]
    # the same call without replicas is the reference for the block
    plain = torch.full((m + 2, width), 0x5A, dtype=torch.uint8, device="cuda")
    d.out = plain.data_ptr() + width + col0
    d.gather_peers = 0
    B.fp8_linear(d)
    torch.cuda.synchronize()
    want = plain.cpu().numpy()
    assert (want[1:m + 1, col0:col0 + n] != 0x5A).any()
    for h in host:
        assert np.array_equal(h, want), "a replica differs from the local output (or bytes outside the block moved)"
    del ws


@pytest.mark.parametrize("m,k,n", [(8, 1024, 1024), (300, 512, 1280)])
def test_int8_output_reaches_every_replica(cuda, m, k, n):
    torch = cuda
    rng = np.random.default_rng(5)
    a = torch.from_numpy(rng.integers(-127, 128, (m, k), dtype=np.int8)).cuda()
    w = torch.from_numpy(rng.integers(-127, 128, (k, n), dtype=np.int8)).cuda()
    scales = torch.full((n,), 0.004, dtype=torch.float32, device="cuda")
    bufs = [torch.full((m, n), 77, dtype=torch.int8, device="cuda") for _ in range(3)]
    d = B.int8_linear_desc(op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=bufs[0], a_scale=0.02, a_zp=0, w_scales=scales,
                           w_zps=None, w_params=n, out_scale=1.5, out_zp=0)
    d.gather_peers = 2
    d.gather_out[0], d.gather_out[1] = bufs[1].data_ptr(), bufs[2].data_ptr()
    ws = B.linear_workspace(torch, d)
    B.int8_linear(d)
    torch.cuda.synchronize()
    host = [b.cpu().numpy() for b in bufs]
    assert (host[0] != 77).any() and np.array_equal(host[0], host[1]) and np.array_equal(host[0], host[2])
    d.gather_peers = 0  # the same call without replicas (stores from registers) gives the same block
    plain = torch.full((m, n), 77, dtype=torch.int8, device="cuda")
    d.out = plain.data_ptr()
    B.int8_linear(d)
    torch.cuda.synchronize()
    assert np.array_equal(plain.cpu().numpy(), host[0])
    del ws


def test_gather_sync_single_rank(cuda):
    torch = cuda
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    ptrs = (C.c_void_p * 1)(flags.data_ptr())
    for epoch in (1, 2, 3):
        assert B.lib().fth_b200_gather_sync(ptrs, C.c_int32(1), C.c_int32(0), C.c_uint32(epoch), B.current_stream()) == 0
        torch.cuda.synchronize()
        assert int(flags[0].item()) == epoch and B.device_status() == 0
    assert B.lib().fth_b200_gather_sync(ptrs, C.c_int32(9), C.c_int32(0), C.c_uint32(1), B.current_stream()) == B.ERR_INVALID


def test_gather_sync_gives_up_when_a_peer_never_signals(cuda):
    """Failure detection without a fault: rank 0 of a two-rank gather whose peer never raises its flag.  The wait runs
    out after its one-second budget, the kernel returns, the status word names the wait (site 40) and the silent rank,
    and the device keeps working."""
    torch = cuda
    mine = torch.zeros(8, dtype=torch.int32, device="cuda")
    peer = torch.zeros(8, dtype=torch.int32, device="cuda")   # stands in for rank 1's flag array; rank 1 does not exist
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    assert B.device_status() == 0
    assert B.lib().fth_b200_gather_sync(ptrs, C.c_int32(2), C.c_int32(0), C.c_uint32(1), B.current_stream()) == 0
    torch.cuda.synchronize()
    status = B.device_status()
    assert status >> 16 == 40 and status & 0xffff == 1
    assert int(peer[0].item()) == 1 and int(mine[0].item()) == 1   # this rank did signal both arrays
    # the context is intact: the next step, with the peer "answering", completes cleanly
    mine[1] = 2
    assert B.lib().fth_b200_gather_sync(ptrs, C.c_int32(2), C.c_int32(0), C.c_uint32(2), B.current_stream()) == 0
    torch.cuda.synchronize()
    assert B.device_status() == 0


# ---- gather signalling folded into the linear kernels ----------------------------------------------------------------
# Two "ranks" on one GPU take turns on one stream (kernels of different ranks never have to run at the same time: every
# wait finds its condition already true, except in the test that lets one run out on purpose).
FOLD_CASES = [(1, 1024, 2048, B.VARIANT_AUTO, "cluster kernel"), (16, 8192, 32768, B.VARIANT_AUTO, "folded split-K, one launch"),
              (16, 8192, 16384, B.VARIANT_AUTO, "split-K reduce pass"),
              (4, 8192, 14336, B.VARIANT_AUTO, "cluster kernel, two tiles per CTA"),
              (300, 512, 640, B.VARIANT_AUTO, "CTA-pair dense kernel"), (4, 256, 384, B.VARIANT_SKINNY, "small kernels around a CUDA-core kernel")]


def _rank_desc(torch, a, w, out_bufs, flags, rank, m, k, n, n0, n1, variant):
    """Descriptor of `rank` (columns n0:n1 of the [k, n] problem) writing into both ranks' [m, n] buffers."""
    w_local = w[:, n0:n1].contiguous()
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n1 - n0, a=a, w=w_local, out=None, a_scale=0.5, w_scale=2.0 ** -6,
                          out_scale=float(k) / 64, ldo=n, variant=variant, weights_static=True)
    d.out = out_bufs[rank].data_ptr() + n0
    d.gather_peers = 1
    d.gather_out[0] = out_bufs[1 - rank].data_ptr() + n0
    d.gather_world, d.gather_rank = 2, rank
    d.gather_flags[0], d.gather_flags[1] = flags[0].data_ptr(), flags[1].data_ptr()
    keep = B.linear_workspace(torch, d)
    return d, (w_local, keep)


@pytest.mark.parametrize("m,k,n,variant,what", FOLD_CASES)
def test_folded_gather_signalling_two_ranks_in_turn(cuda, m, k, n, variant, what):
    torch = cuda
    rng = np.random.default_rng(m + k + n)
    a = torch.from_numpy(rng.integers(0, 0x78, (m, k), dtype=np.uint8)).cuda()
    w = torch.from_numpy(rng.integers(0, 0x78, (k, n), dtype=np.uint8)).cuda()
    full = torch.zeros((m, n), dtype=torch.uint8, device="cuda")
    d_full = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=full, a_scale=0.5, w_scale=2.0 ** -6,
                               out_scale=float(k) / 64, variant=variant)
    keep_full = B.linear_workspace(torch, d_full)
    if B.lib().fth_b200_fp8_linear_supported(C.byref(d_full)) != 0:
        pytest.skip("variant declines this shape")
    B.fp8_linear(d_full)
    half = (n // 2 + 127) // 128 * 128
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    outs = [torch.zeros((m, n), dtype=torch.uint8, device="cuda") for _ in range(2)]
    descs = [_rank_desc(torch, a, w, outs, flags, r, m, k, n, 0 if r == 0 else half, half if r == 0 else n, variant) for r in range(2)]
    B.lib().fth_b200_reset_launch_count()
    for step in range(1, 4):
        for r in range(2):
            B.fp8_linear(descs[r][0])
        torch.cuda.synchronize()
        for r in range(2):
            f = flags[r].cpu().numpy()
            assert f[0] == step and f[1] == step, f"{what}: rank {r} flags {f[:4]} after step {step}"
            assert f[2] == step and f[3] == 0, f"{what}: step counter / arrival counter {f[2:4]}"
            assert torch.equal(outs[r], full), f"{what}: rank {r} buffer differs from the single-GPU result"
            outs[r].zero_()
    folded = "CUDA-core" not in what
    per_call = B.lib().fth_b200_launch_count() / 6
    assert (per_call <= 2) if folded else (per_call >= 3), f"{what}: {per_call} launches per call"
    # the consumer-side wait: both ranks have published step 3
    ptrs = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    for r in range(2):
        assert B.lib().fth_b200_gather_wait(ptrs, C.c_int32(2), C.c_int32(r), B.current_stream()) == 0
    torch.cuda.synchronize()
    assert B.device_status() == 0
    del keep_full


def test_folded_gather_wait_gives_up_when_a_peer_is_a_step_behind(cuda):
    """Failure detection without a fault: rank 0 starts step 2 although rank 1 never ran step 1.  Its kernel waits one
    second for rank 1's flag before storing into rank 1's buffer, reports the wait (site 41, rank 1) in the status
    word, and still completes; once rank 1 has caught up the next step is clean."""
    torch = cuda
    m, k, n = 1, 1024, 2048
    rng = np.random.default_rng(3)
    a = torch.from_numpy(rng.integers(0, 0x78, (m, k), dtype=np.uint8)).cuda()
    w = torch.from_numpy(rng.integers(0, 0x78, (k, n), dtype=np.uint8)).cuda()
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    outs = [torch.zeros((m, n), dtype=torch.uint8, device="cuda") for _ in range(2)]
    descs = [_rank_desc(torch, a, w, outs, flags, r, m, k, n, 0 if r == 0 else 1024, 1024 if r == 0 else n, B.VARIANT_AUTO) for r in range(2)]
    assert B.device_status() == 0
    B.fp8_linear(descs[0][0])   # rank 0, step 1: nothing to wait for
    torch.cuda.synchronize()
    assert B.device_status() == 0
    B.fp8_linear(descs[0][0])   # rank 0, step 2: rank 1 has not published step 1
    torch.cuda.synchronize()
    status = B.device_status()
    assert status >> 16 == 41 and status & 0xffff == 1
    assert flags[0].cpu().numpy()[0] == 2   # the kernel finished and published its step all the same
    B.fp8_linear(descs[1][0])   # rank 1 catches up: steps 1 and 2
    B.fp8_linear(descs[1][0])
    B.fp8_linear(descs[0][0])   # rank 0, step 3
    torch.cuda.synchronize()
    assert B.device_status() == 0
    ptrs = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    assert B.lib().fth_b200_gather_wait(ptrs, C.c_int32(2), C.c_int32(0), B.current_stream()) == 0   # rank 1 is at step 2, rank 0 at 3
    torch.cuda.synchronize()
    status = B.device_status()
    assert status >> 16 == 41 and status & 0xffff == 1   # the consumer-side wait reports the rank that is behind
