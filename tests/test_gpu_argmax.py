"""Fused linear + greedy selection (fth_b200_fp8_linear_argmax): the index must be what an ArgMax node would pick from
the linear's own output — largest decoded value, NaN skipped, ties to the lowest column — and the chosen value must be
the oracle's row maximum to within one FP8 code (the linear's own parity bound)."""
import ctypes as C

import numpy as np
import pytest

import infer_b200 as B
import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch


def _greedy(values):
    """Reference rule (src/kernel/cuda/qwen_gemm_argmax.cu:55-64): first strictly larger non-NaN value wins."""
    best, index = None, -1
    for i, v in enumerate(values):
        if np.isnan(v):
            continue
        if index < 0 or v > best:
            best, index = v, i
    return index


# (m, k, n, trans_b, dtype): cluster kernel; two-kernel split path with an lm-head-like [N,K] weight; several rows
CASES = [(1, 1024, 2048, False, B.E5M2), (1, 1024, 16384 + 64, True, B.E4M3), (4, 2048, 8192, True, B.E5M2), (16, 8192, 8192, False, B.E4M3)]


@pytest.mark.parametrize("m,k,n,trans_b,dtype", CASES)
def test_fused_argmax_matches_argmax_of_the_output(cuda, m, k, n, trans_b, dtype):
    torch = cuda
    rng = np.random.default_rng(k + n + m)
    a_f = rng.standard_normal((m, k)).astype(np.float32)
    w_f = (rng.standard_normal((n, k) if trans_b else (k, n)) * 0.05).astype(np.float32)
    sa, sw = float(np.abs(a_f).max() / 200.0), float(np.abs(w_f).max() / 200.0)
    a = O.fp8_encode(dtype, a_f / sa)
    w = O.fp8_encode(dtype, w_f / sw)
    so = float(np.sqrt(k) * 0.05 * 4.0 / 200.0)
    a_dev, w_dev = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    out = torch.zeros((m, n), dtype=torch.uint8, device="cuda")
    idx = torch.full((m,), -7, dtype=torch.int64, device="cuda")
    d = B.fp8_linear_desc(dtype=dtype, op=B.OP_GEMM if trans_b else B.OP_MATMUL, m=m, k=k, n=n, a=a_dev, w=w_dev, out=out, a_scale=sa,
                          w_scale=sw, out_scale=so, trans_b=trans_b, weights_static=True)
    ws = B.linear_workspace(torch, d)
    for _ in range(2):  # the selection state is rebuilt by every call
        rc = B.lib().fth_b200_fp8_linear_argmax(C.byref(d), C.c_void_p(idx.data_ptr()), B.current_stream())
        assert rc == 0
        torch.cuda.synchronize()
    assert B.device_status() == 0
    codes = out.cpu().numpy()
    got = idx.cpu().numpy()
    decoded = O.fp8_decode(dtype, codes)
    want_codes = O.fp8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, dtype, a, sa, w, sw, so, trans_b=trans_b)
    want = O.fp8_decode(dtype, want_codes)
    for row in range(m):
        assert got[row] == _greedy(decoded[row]), f"row {row}: fused index {got[row]} is not the argmax of the output"
        top = np.nanmax(want[row])
        chosen = want_codes[row, got[row]]
        assert abs(int(chosen & 0x7f) - int(O.fp8_encode(dtype, np.array([top], np.float32))[0] & 0x7f)) <= 1
    del ws


def test_fused_argmax_skips_nan_and_declines_dense_shapes(cuda):
    torch = cuda
    m, k, n = 2, 256, 1024
    a = np.full((m, k), 0x38, dtype=np.uint8)       # 1.0 in E4M3
    w = np.full((k, n), 0x30, dtype=np.uint8)       # 0.5
    w[:, 5] = 0x7f                                   # a NaN weight column: its outputs are NaN codes
    w[:, 700] = 0x38                                 # the largest finite column
    w[:, 900] = 0x38                                 # equal to column 700: the lower column must win
    a[1, :] = 0x7f                                   # a row of NaN activations: no candidate at all
    a_dev, w_dev = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    out = torch.zeros((m, n), dtype=torch.uint8, device="cuda")
    idx = torch.zeros((m,), dtype=torch.int64, device="cuda")
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=k, n=n, a=a_dev, w=w_dev, out=out, a_scale=1.0, w_scale=1.0, out_scale=2.0)
    ws = B.linear_workspace(torch, d)
    assert B.lib().fth_b200_fp8_linear_argmax(C.byref(d), C.c_void_p(idx.data_ptr()), B.current_stream()) == 0
    torch.cuda.synchronize()
    assert idx.cpu().tolist() == [700, -1]
    big = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=300, k=k, n=n, a=a_dev, w=w_dev, out=out, a_scale=1.0, w_scale=1.0, out_scale=2.0)
    assert B.lib().fth_b200_fp8_linear_argmax(C.byref(big), C.c_void_p(idx.data_ptr()), B.current_stream()) == B.ERR_UNSUPPORTED
    del ws


def test_fused_argmax_against_the_reference_x86_lm_head_kernel(cuda):
    """Pinned to the reference: the seeded lm-head cases of tests/golden/cases.py were run through the reference's own
    fused FP8 kernel (QwenGemmArgmaxKernel<X86, FP8*>, src/kernel/x86/linear_fp8.cc:733-1004) when the fixtures were
    made.  On the exact-integer cases (ties between rows, a NaN row, output scale != 1) the selected index must be the
    same.  On random data the two kernels add the 256 .. 512 products in different orders, so output codes may differ
    by one and with them the winner among near-equal rows: there the row picked here must hold, in the reference's
    materialised output, a code within one step of the code of the row the reference picked."""
    import os
    from tests.golden import cases as G
    from tests import util
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))
    torch = cuda
    for entry in G.ARGMAX:
        name, dtype = entry[0], entry[1]
        c = G.argmax_case(entry)
        n, k = c["b"].shape
        a_dev, w_dev = torch.from_numpy(c["a"]).cuda(), torch.from_numpy(c["b"]).cuda()
        out = torch.zeros((1, n), dtype=torch.uint8, device="cuda")
        idx = torch.full((1,), -7, dtype=torch.int64, device="cuda")
        d = B.fp8_linear_desc(dtype=dtype, op=B.OP_GEMM, m=1, k=k, n=n, a=a_dev, w=w_dev, out=out, a_scale=c["sa"], w_scale=c["sb"],
                              out_scale=c["so"], trans_b=True, weights_static=True)
        ws = B.linear_workspace(torch, d)
        assert B.lib().fth_b200_fp8_linear_argmax(C.byref(d), C.c_void_p(idx.data_ptr()), B.current_stream()) == 0
        torch.cuda.synchronize()
        got, want = int(idx.item()), int(gold[f"argmax/{name}/x86_index"])
        codes = gold[f"argmax/{name}/common_codes"][0]
        if entry[5] == "random":
            assert util.fp8_code_distance(codes[got:got + 1], codes[want:want + 1]).max() <= 1, (name, got, want)
        else:
            assert got == want, (name, got, want)
        print(f"{name}: fused index {got}, reference x86 kernel {want}")
        del ws
    assert B.device_status() == 0
