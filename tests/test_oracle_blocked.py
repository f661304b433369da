"""CPU: the column-blocked oracle loops (the ones every test calls) against the plain one-output-at-a-time loops that
restate the reference's Common kernels line by line — byte for byte, on shapes with ragged blocks, both weight
layouts, every bias mode, Gemm alpha / beta, zero points, and an INT8 shape outside the int32 bound (which must take
the plain loop and report the overflow)."""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from tests import util


def _plain_fp8(op, dtype, case, trans_b, alpha, beta):
    a, w, bias = case["a"], case["w"], case["bias"]
    m, k = a.shape
    n = w.shape[0] if trans_b else w.shape[1]
    mode = 0 if bias is None else (1 if bias.ndim == 1 else 2)
    out = np.empty((m, n), np.uint8)
    rc = O.port().fo_fp8_linear_plain(C.c_int(op), C.c_int(dtype), O._p(a), C.c_float(case["sa"]), O._p(w), C.c_float(case["sw"]),
                                      O._p(bias), C.c_float(case["sb"]), C.c_int(mode), O._p(out), C.c_float(case["so"]),
                                      C.c_int64(m), C.c_int64(k), C.c_int64(n), C.c_int(int(trans_b)), C.c_float(alpha), C.c_float(beta))
    assert rc == 0
    return out


def _plain_int8(op, case, trans_b, alpha, beta):
    a, w, bias = case["a"], case["w"], case["bias"]
    m, k = a.shape
    n = w.shape[0] if trans_b else w.shape[1]
    ws = np.atleast_1d(case["ws"])
    zps = case["w_zps"]
    mode = 0 if bias is None else (1 if bias.ndim == 1 else 2)
    out = np.empty((m, n), np.int8)
    rc = O.port().fo_int8_linear_plain(C.c_int(op), O._p(a), C.c_float(case["sa"]), C.c_int32(case["a_zp"]), O._p(w), O._p(ws), O._p(zps),
                                       C.c_int64(0 if ws.size == 1 else n), O._p(bias), C.c_int(mode), O._p(out), C.c_float(case["so"]),
                                       C.c_int32(case["out_zp"]), C.c_int64(m), C.c_int64(k), C.c_int64(n), C.c_int(int(trans_b)),
                                       C.c_float(alpha), C.c_float(beta))
    return rc, out


@pytest.mark.parametrize("dtype", [O.E4M3, O.E5M2])
@pytest.mark.parametrize("m,k,n,trans_b,bias_mode", [(3, 257, 130, False, 1), (5, 100, 64, True, 2), (1, 1024, 3072, False, 0),
                                                     (17, 64, 63, True, 0), (2, 8192, 65, False, 1)])
def test_blocked_fp8_equals_plain(dtype, m, k, n, trans_b, bias_mode):
    case = util.make_fp8_linear(dtype, m, k, n, seed=m + k + n, trans_b=trans_b, bias_mode=bias_mode)
    for op, alpha, beta in [(O.OP_FC, 1.0, 1.0), (O.OP_GEMM, 0.5, 2.0)]:
        got = O.fp8_linear(op, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"], bias=case["bias"],
                           bias_scale=case["sb"], trans_b=trans_b, alpha=alpha, beta=beta)
        assert np.array_equal(got, _plain_fp8(op, dtype, case, trans_b, alpha, beta))


def test_blocked_fp8_non_finite_inputs():
    case = util.make_fp8_linear(O.E5M2, 4, 96, 70, seed=9)
    case["a"][1, 5] = 0x7C   # +Inf
    case["a"][2, 7] = 0x7D   # NaN
    case["w"][3, 11] = 0xFC  # -Inf
    got = O.fp8_linear(O.OP_MATMUL, O.E5M2, case["a"], case["sa"], case["w"], case["sw"], case["so"])
    assert np.array_equal(got, _plain_fp8(O.OP_MATMUL, O.E5M2, case, False, 1.0, 1.0))


@pytest.mark.parametrize("m,k,n,trans_b,zero_points,bias_mode,per_channel", [
    (3, 257, 130, False, False, 1, True), (5, 100, 64, True, True, 2, True), (128, 1024, 200, False, False, 0, True),
    (2, 64, 63, True, True, 0, False)])
def test_blocked_int8_equals_plain(m, k, n, trans_b, zero_points, bias_mode, per_channel):
    case = util.make_int8_linear(m, k, n, seed=m + k + n, trans_b=trans_b, per_channel=per_channel, zero_points=zero_points,
                                 bias_mode=bias_mode)
    for op, alpha, beta in [(O.OP_FC, 1.0, 1.0), (O.OP_GEMM, 0.75, 1.25)]:
        got = O.int8_linear(op, case["a"], case["sa"], case["a_zp"], case["w"], case["ws"], case["w_zps"], case["so"], case["out_zp"],
                            bias=case["bias"], trans_b=trans_b, alpha=alpha, beta=beta)
        rc, want = _plain_int8(op, case, trans_b, alpha, beta)
        assert rc == 0 and np.array_equal(got, want)


def test_blocked_int8_overflow_takes_the_plain_loop():
    k = 140000  # 140000 * 128 * 128 > 2^31 - 1: a running sum may leave int32, which the contract reports as failure
    a = np.full((1, k), -128, np.int8)
    w = np.full((k, 2), -128, np.int8)
    w[:, 1] = 1
    rc, _ = O.int8_linear(O.OP_MATMUL, a, 1.0, 0, w, np.ones(1, np.float32), None, 1.0, 0, check=False)
    assert rc == -1
