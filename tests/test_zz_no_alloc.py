"""GPU: the allocation-free FP8 linear entry point (scratch inside the library image) against the ordinary one.

Collected last on purpose: a run that stops at the first failure has then already exercised every other test.
The two entry points must agree byte for byte, on two calls in a row that differ in shape and data (the
built-in scratch keeps the previous call's partial sums; a call may only ever read what it wrote itself)."""
import ctypes as C

import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests import util
from tests.gpu_helpers import dev

pytestmark = pytest.mark.gpu


def both_entry_points(torch, dtype, m, k, n, seed, trans_b=False):
    case = util.make_fp8_linear(dtype, m, k, n, seed=seed, trans_b=trans_b)
    a, w = dev(torch, case["a"]), dev(torch, case["w"])
    outs = []
    for noalloc in (False, True):
        out = torch.full((m, n), 0x5A, dtype=torch.uint8, device="cuda")
        d = B.fp8_linear_desc(dtype=dtype, op=B.OP_GEMM if trans_b else B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=out,
                              a_scale=case["sa"], w_scale=case["sw"], out_scale=case["so"], trans_b=trans_b,
                              variant=B.VARIANT_TCGEN05)
        # the shape must be one whose split-K partial sums really go through scratch memory (decode-sized shapes
        # that fit one wave of CTAs run on a kernel that needs none, and would not touch the built-in array at all)
        need = B.lib().fth_b200_fp8_linear_workspace_bytes(C.byref(d))
        assert 0 < need <= B.lib().fth_b200_noalloc_scratch_bytes()
        B.lib().fth_b200_reset_launch_count()
        if noalloc:
            rc = B.lib().fth_b200_fp8_linear_noalloc(C.byref(d), B.current_stream())
        else:
            keep = B.linear_workspace(torch, d)
            rc = B.lib().fth_b200_fp8_linear(C.byref(d), B.current_stream())
        assert rc == B.OK, rc
        assert B.lib().fth_b200_launch_count() == 2  # weight-streaming pass + the pass that adds the partial sums
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    want = O.fp8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"], trans_b=trans_b)
    return outs[0], outs[1], want, need


def test_noalloc_matches_ordinary_entry_point_twice_in_a_row(cuda):
    assert B.lib().fth_b200_noalloc_scratch_bytes() == 4 << 20
    # first call: 1 MiB of partial sums (8 K chunks x 4 rows x 8192 channels); second call: other data, other format,
    # other weight layout and a smaller footprint, so the first call's partial sums still lie under and behind the
    # region it uses — a call may only ever read what it wrote itself
    needs = []
    for (dtype, m, k, n, seed, trans_b) in [(O.E4M3, 4, 4096, 8192, 101, False), (O.E5M2, 1, 2048, 8192, 202, True)]:
        ordinary, noalloc, want, need = both_entry_points(cuda, dtype, m, k, n, seed, trans_b)
        needs.append(need)
        assert np.array_equal(ordinary, noalloc)
        assert util.fp8_code_distance(noalloc, want).max() <= 1
    assert needs[1] < needs[0]
    assert B.device_status() == 0


def test_noalloc_rejects_what_does_not_fit(cuda):
    tiny = cuda.zeros(4096, dtype=cuda.uint8, device="cuda")
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=16, k=8192, n=28672, a=tiny, w=tiny, out=tiny, a_scale=1.0,
                          w_scale=1.0, out_scale=1.0)
    assert B.lib().fth_b200_fp8_linear_workspace_bytes(C.byref(d)) > B.lib().fth_b200_noalloc_scratch_bytes()
    assert B.lib().fth_b200_fp8_linear_noalloc(C.byref(d), B.current_stream()) == B.ERR_SCRATCH_LIMIT  # nothing is launched
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=1, k=100, n=64, a=tiny, w=tiny, out=tiny, a_scale=1.0, w_scale=1.0,
                          out_scale=1.0)
    assert B.lib().fth_b200_fp8_linear_noalloc(C.byref(d), B.current_stream()) == B.ERR_UNSUPPORTED  # K % 16 != 0
    assert B.lib().fth_b200_fp8_linear_noalloc(None, B.current_stream()) == B.ERR_INVALID
