"""GPU: the exact launches the ncu summaries under profiles/ were captured from — four calls of one kernel on the
named workload (ncu: `-s 3 -c 1`).  As tests they check that the call runs on the expected kernel family, leaves the
device status word clean, and that a seeded slice of what it wrote (the conv: all of it) is the oracle's result."""
import ctypes as C

import numpy as np
import pytest

import infer_b200 as B
import oracle as O

pytestmark = pytest.mark.gpu
K, N = 8192, 28672


def _linear(torch, kind, m):
    ws = torch.zeros(16 << 20, dtype=torch.uint8, device="cuda")
    if kind == "fp8":
        w = torch.randint(0, 120, (K, N), dtype=torch.uint8, device="cuda")
        a = torch.randint(0, 120, (m, K), dtype=torch.uint8, device="cuda")
        out = torch.empty((m, N), dtype=torch.uint8, device="cuda")
        d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=K, n=N, a=a, w=w, out=out, a_scale=1.0, w_scale=1.0,
                              out_scale=64.0, variant=B.VARIANT_TCGEN05, workspace=ws, workspace_bytes=ws.numel())
        call = B.lib().fth_b200_fp8_linear
    else:
        w = torch.randint(-127, 127, (K, N), dtype=torch.int8, device="cuda")
        a = torch.randint(-127, 127, (m, K), dtype=torch.int8, device="cuda")
        sc = torch.full((N,), 0.005, dtype=torch.float32, device="cuda")
        out = torch.empty((m, N), dtype=torch.int8, device="cuda")
        d = B.int8_linear_desc(op=B.OP_MATMUL, m=m, k=K, n=N, a=a, w=w, out=out, a_scale=0.02, a_zp=0, w_scales=sc, w_zps=None,
                               w_params=N, out_scale=1.0, out_zp=0, variant=B.VARIANT_TCGEN05, workspace=ws, workspace_bytes=ws.numel())
        call = B.lib().fth_b200_int8_linear
    for _ in range(4):
        assert call(C.byref(d), B.current_stream()) == B.OK
    torch.cuda.synchronize()
    assert B.last_variant() == "tcgen05"
    # 16 rows x 64 columns of the output against the oracle on the sliced operands
    rng = np.random.default_rng(m)
    rows = np.sort(rng.choice(m, min(16, m), replace=False))
    cols = np.sort(rng.choice(N, 64, replace=False))
    a_h = np.ascontiguousarray(a.cpu().numpy()[rows])
    w_h = np.ascontiguousarray(w[:, torch.from_numpy(cols).cuda()].cpu().numpy())
    got = out.cpu().numpy()[np.ix_(rows, cols)]
    if kind == "fp8":
        want = O.fp8_linear(O.OP_MATMUL, O.E4M3, a_h, 1.0, w_h, 1.0, 64.0)
        dist = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert dist.max() <= 1
    else:
        want = O.int8_linear(O.OP_MATMUL, a_h, 0.02, 0, w_h, np.full(64, 0.005, np.float32), None, 1.0, 0)
        assert np.array_equal(got, want)


def _conv(torch):
    from tests import util
    from tests.gpu_helpers import dev
    case = util.make_int8_conv(1, 64, 160, 160, 64, 3, 3, seed=3)
    x, w, b, ws = dev(torch, case["x"]), dev(torch, case["w"]), dev(torch, case["bias"]), dev(torch, case["ws"])
    out = torch.empty((1, 64, 160, 160), dtype=torch.int8, device="cuda")
    lut = dev(torch, B.int8_relu_table(case["so"], 0, case["so"], 0))
    d = B.int8_conv2d_desc(batch=1, ic=64, ih=160, iw=160, oc=64, kh=3, kw=3, x=x, w=w, out=out, x_scale=case["sx"], x_zp=0,
                           w_scales=ws, w_zps=None, w_params=64, out_scale=case["so"], out_zp=0, bias=b, relu_lut=lut,
                           bias_max_abs=1 << 15)
    need = B.lib().fth_b200_int8_conv2d_workspace_bytes(C.byref(d))
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = scratch.data_ptr(), need
    for _ in range(4):
        assert B.lib().fth_b200_int8_conv2d(C.byref(d), B.current_stream()) == B.OK
        d.weights_packed = 1
    torch.cuda.synchronize()
    assert B.last_variant() == "conv_tcgen05"
    want = O.int8_conv2d(case["x"], case["sx"], 0, case["w"], case["ws"], None, case["bias"], case["so"], 0)
    want = O.int8_relu(want, case["so"], 0, case["so"], 0)
    assert np.array_equal(out.cpu().numpy(), want)


def _decode_projection(torch):
    """Config-4 projection (hidden 1024 -> intermediate 3584, FP8 E5M2, BF16 in and out) on the single-launch cluster
    kernel: 40 different weights (147 MB, more than L2) in turn, then one more round for the capture."""
    k, n = 1024, 3584
    a = torch.randn((1, k), device="cuda").to(torch.bfloat16)
    out = torch.empty((1, n), dtype=torch.bfloat16, device="cuda")
    weights = [torch.randint(0, 120, (k, n), dtype=torch.uint8, device="cuda") for _ in range(40)]
    descs = [B.fp8_linear_desc(dtype=B.E5M2, op=B.OP_MATMUL, m=1, k=k, n=n, a=a, w=w, out=out, a_scale=2.0 ** -9, w_scale=2.0 ** -20,
                               out_scale=2.0 ** -9, a_dtype=B.BF16, out_dtype=B.BF16, weights_static=True) for w in weights]
    assert B.lib().fth_b200_fp8_linear_workspace_bytes(C.byref(descs[0])) == 0  # no scratch on this path
    for _ in range(2):
        for d in descs:
            assert B.lib().fth_b200_fp8_linear(C.byref(d), B.current_stream()) == B.OK
    torch.cuda.synchronize()
    assert B.last_variant() == "tcgen05"
    # the last weight's projection against the oracle: Cast -> MatMul -> Cast, at most one E5M2 code apart
    a_bits = a.view(torch.int16).cpu().numpy().view(np.uint16)
    codes = O.cast(O.BF16, a_bits, 1.0, O.E5M2, 2.0 ** -9).reshape(1, k)
    y = O.fp8_linear(O.OP_MATMUL, O.E5M2, codes, 2.0 ** -9, weights[-1].cpu().numpy(), 2.0 ** -20, 2.0 ** -9)
    got = O.cast(O.BF16, out.view(torch.int16).cpu().numpy().view(np.uint16), 1.0, O.E5M2, 2.0 ** -9).reshape(1, n)
    assert np.abs(got.astype(np.int32) - y.astype(np.int32)).max() <= 1


@pytest.mark.parametrize("case", ["gemv_m1_fp8", "dense_m4096_fp8", "dense_m4096_int8", "conv_c3", "decode_projection"])
def test_profile_case(cuda, case):
    if case == "decode_projection":
        _decode_projection(cuda)
    elif case == "gemv_m1_fp8":
        _linear(cuda, "fp8", 1)
    elif case == "dense_m4096_fp8":
        _linear(cuda, "fp8", 4096)
    elif case == "dense_m4096_int8":
        _linear(cuda, "int8", 4096)
    else:
        _conv(cuda)
    assert B.device_status() == 0
