"""Host-buffer plans (fth_b200_plan_*): the convenience layer bench.py's end-to-end figure goes through.  The result
must be the bytes of the direct device call, for pageable and for pinned host buffers."""
import ctypes

import numpy as np
import pytest

import infer_b200 as B

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch


@pytest.mark.parametrize("m,k,n", [(1, 1024, 2048), (16, 8192, 8192), (200, 512, 768)])
def test_fp8_plan_matches_device_call(cuda, m, k, n):
    torch = cuda
    rng = np.random.default_rng(m + n)
    a = rng.integers(0, 0x78, (m, k), dtype=np.uint8)
    w = rng.integers(0, 0x78, (k, n), dtype=np.uint8)
    a_dev, w_dev = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    out_dev = torch.empty((m, n), dtype=torch.uint8, device="cuda")
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=a_dev, w=w_dev, out=out_dev, a_scale=0.5, w_scale=2.0 ** -6,
                          out_scale=float(k) / 64)
    ws = B.linear_workspace(torch, d)
    B.fp8_linear(d)
    torch.cuda.synchronize()
    want = out_dev.cpu().numpy()
    hd = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=None, w=None, out=None, a_scale=0.5, w_scale=2.0 ** -6,
                           out_scale=float(k) / 64)
    hd.w = w.ctypes.data
    plan = B.Plan(hd)
    pageable = np.zeros((m, n), dtype=np.uint8)
    plan.run(a, pageable)
    assert np.array_equal(pageable, want)
    pinned_in = torch.from_numpy(a).pin_memory()
    pinned_out = torch.zeros((m, n), dtype=torch.uint8).pin_memory()
    for _ in range(2):
        pinned_out.zero_()
        plan.run(pinned_in, pinned_out)
        assert np.array_equal(pinned_out.numpy(), want)
    # Decode-sized plans replay a recorded step for the pair of page-locked buffers of the last call: other data in the
    # same buffers must be read afresh, another pair of buffers must be recorded again, and a mixed pair too.
    a2 = rng.integers(0, 0x78, (m, k), dtype=np.uint8)
    a_dev.copy_(torch.from_numpy(a2).cuda())
    B.fp8_linear(d)
    torch.cuda.synchronize()
    want2 = out_dev.cpu().numpy()
    assert not np.array_equal(want, want2)
    pinned_in.copy_(torch.from_numpy(a2))
    pinned_out.zero_()
    plan.run(pinned_in, pinned_out)
    assert np.array_equal(pinned_out.numpy(), want2)
    other_in = torch.from_numpy(a).pin_memory()
    other_out = torch.zeros((m, n), dtype=torch.uint8).pin_memory()
    plan.run(other_in, other_out)
    assert np.array_equal(other_out.numpy(), want)
    other_out.zero_()
    plan.run(pinned_in, other_out)
    assert np.array_equal(other_out.numpy(), want2)
    plan.run(a, pageable)  # and pageable memory still goes through the copy engine
    assert np.array_equal(pageable, want)
    plan.close()
    assert B.device_status() == 0
    del ws


def test_int8_plan_matches_device_call(cuda):
    torch = cuda
    m, k, n = 4, 1024, 1024
    rng = np.random.default_rng(11)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-127, 128, (k, n), dtype=np.int8)
    scales = np.full(n, 0.004, dtype=np.float32)
    a_dev, w_dev, s_dev = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(scales).cuda()
    out_dev = torch.empty((m, n), dtype=torch.int8, device="cuda")
    d = B.int8_linear_desc(op=B.OP_MATMUL, m=m, k=k, n=n, a=a_dev, w=w_dev, out=out_dev, a_scale=0.02, a_zp=0, w_scales=s_dev, w_zps=None,
                           w_params=n, out_scale=1.5, out_zp=0)
    ws = B.linear_workspace(torch, d)
    B.int8_linear(d)
    torch.cuda.synchronize()
    want = out_dev.cpu().numpy()
    hd = B.int8_linear_desc(op=B.OP_MATMUL, m=m, k=k, n=n, a=None, w=None, out=None, a_scale=0.02, a_zp=0, w_scales=None, w_zps=None,
                            w_params=n, out_scale=1.5, out_zp=0)
    hd.w, hd.w_scales = w.ctypes.data, scales.ctypes.data
    plan = B.Plan(hd)
    pageable = np.zeros((m, n), dtype=np.int8)
    plan.run(a, pageable)
    pinned_out = torch.zeros((m, n), dtype=torch.int8).pin_memory()
    plan.run(torch.from_numpy(a).pin_memory(), pinned_out)
    plan.close()
    assert np.array_equal(pageable, want) and np.array_equal(pinned_out.numpy(), want)
    del ws


@pytest.mark.parametrize("nbytes", [1, 17, 8192, 28672, 100003])
def test_small_copy_between_pinned_host_and_device(cuda, nbytes):
    torch = cuda
    rng = np.random.default_rng(nbytes)
    src = torch.from_numpy(rng.integers(0, 256, nbytes, dtype=np.uint8)).pin_memory()
    mid = torch.zeros(nbytes + 32, dtype=torch.uint8, device="cuda")
    back = torch.zeros(nbytes + 2, dtype=torch.uint8).pin_memory()
    B.small_copy(mid[16:], src, nbytes)                       # host -> device (16-byte aligned destination)
    B.small_copy(back.data_ptr() + 1, mid.data_ptr() + 16, nbytes)   # device -> host, unaligned destination
    torch.cuda.synchronize()
    assert torch.equal(back[1:nbytes + 1], src) and int(back[0]) == 0 and int(back[-1]) == 0
    assert int(mid[:16].sum()) == 0 and int(mid[16 + nbytes:].sum()) == 0
    pageable = np.zeros(nbytes, dtype=np.uint8)
    assert B.lib().fth_b200_small_copy(ctypes.c_void_p(pageable.ctypes.data), ctypes.c_void_p(mid.data_ptr()), ctypes.c_int64(nbytes),
                                       B.current_stream()) == B.ERR_UNSUPPORTED
