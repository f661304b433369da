"""INT8 FC / MatMul / Gemm on the GPU: bit-exact against the CPU oracle (Common semantics: int32
accumulation, FP64 requantisation, round-half-away, saturation)."""
import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests import util
from tests.gpu_helpers import run_int8_linear

pytestmark = pytest.mark.gpu


def oracle_int8(op, case, **kw):
    return O.int8_linear(op, case["a"], case["sa"], case["a_zp"], case["w"], case["ws"], case["w_zps"], case["so"],
                         case["out_zp"], bias=case["bias"], **kw)


@pytest.mark.parametrize("variant", [B.VARIANT_SIMT, B.VARIANT_SKINNY, B.VARIANT_STREAM, B.VARIANT_TCGEN05])
@pytest.mark.parametrize("m,k,n", [(1, 1024, 3072), (2, 1024, 1024), (4, 8192, 512), (16, 512, 256), (3, 100, 48), (1, 4, 16), (3, 8192, 1040)])
@pytest.mark.parametrize("zero_points", [False, True])
def test_matmul_kn(cuda, variant, m, k, n, zero_points):
    if variant == B.VARIANT_STREAM and m > 4:
        pytest.skip("the TMA-ring GEMV takes M <= 4 for INT8")
    case = util.make_int8_linear(m, k, n, seed=m + k + n, zero_points=zero_points)
    want = oracle_int8(O.OP_MATMUL, case)
    got = run_int8_linear(cuda, B.OP_MATMUL, case, variant=variant)
    assert np.array_equal(got, want), f"{int((got != want).sum())} of {want.size} bytes differ"


@pytest.mark.parametrize("variant", [B.VARIANT_SIMT, B.VARIANT_SKINNY, B.VARIANT_TCGEN05])
@pytest.mark.parametrize("m,k,n", [(1, 1024, 3072), (2, 2048, 1000), (5, 528, 19), (16, 256, 77)])
@pytest.mark.parametrize("zero_points", [False, True])
def test_gemm_trans_b(cuda, variant, m, k, n, zero_points):
    case = util.make_int8_linear(m, k, n, seed=k + n, trans_b=True, zero_points=zero_points, bias_mode=1)
    want = oracle_int8(O.OP_GEMM, case, trans_b=True, alpha=0.5, beta=2.0)
    got = run_int8_linear(cuda, B.OP_GEMM, case, trans_b=True, variant=variant, alpha=0.5, beta=2.0)
    assert np.array_equal(got, want)


def test_config2_shape_m128(cuda):
    """M=128, K=1024, N=1024, per-channel weight scales, a few percent of outputs saturating."""
    case = util.make_int8_linear(128, 1024, 1024, seed=2)
    want = oracle_int8(O.OP_MATMUL, case)
    got = run_int8_linear(cuda, B.OP_MATMUL, case)
    assert np.array_equal(got, want)
    sat = float((np.abs(want.astype(np.int32)) >= 127).mean())
    assert 0.002 < sat < 0.2


@pytest.mark.parametrize("op,bias_mode", [(B.OP_FC, 1), (B.OP_FC, 2), (B.OP_GEMM, 2), (B.OP_FC, 0)])
@pytest.mark.parametrize("per_channel", [True, False])
def test_bias_and_granularity(cuda, op, bias_mode, per_channel):
    case = util.make_int8_linear(6, 192, 144, seed=5 + bias_mode, per_channel=per_channel, zero_points=True, bias_mode=bias_mode)
    want = oracle_int8(op, case)
    got = run_int8_linear(cuda, op, case)
    assert np.array_equal(got, want)


def test_ragged_shapes(cuda):
    for m, k, n in [(1, 1, 1), (2, 3, 5), (17, 33, 65), (63, 64, 65), (65, 127, 129)]:
        case = util.make_int8_linear(m, k, n, seed=m * k + n, zero_points=True, bias_mode=1)
        want = oracle_int8(O.OP_FC, case)
        got = run_int8_linear(cuda, B.OP_FC, case)
        assert np.array_equal(got, want), (m, k, n)


def test_reference_known_answers(cuda):
    """test/common_int8_kernel_test.cc:103-140 — zero points, per-channel weights, bias → {8, 14};
    127·127 at scale 0.01 saturates to 127."""
    case = dict(a=np.array([[5, 1]], np.int8), w=np.array([[2, 3], [6, -1]], np.int8), bias=np.array([4, -4], np.int32),
                sa=0.5, a_zp=3, ws=np.array([0.25, 0.5], np.float32), w_zps=np.array([-2, 1], np.int32), so=0.25, out_zp=10)
    assert run_int8_linear(cuda, B.OP_FC, case).tolist() == [[8, 14]]
    case = dict(a=np.array([[127]], np.int8), w=np.array([[127]], np.int8), bias=None, sa=1.0, a_zp=0,
                ws=np.array([1.0], np.float32), w_zps=None, so=0.01, out_zp=0)
    assert run_int8_linear(cuda, B.OP_MATMUL, case).tolist() == [[127]]


def test_exact_ties_round_away_from_zero(cuda):
    """Crafted .5 cases: scale 1, out scale 2 → acc/2; odd accumulators tie and must round away from zero
    (std::round), e.g. 3 → 2, -3 → -2, 1 → 1, -1 → -1; round-half-even would give 2, -2, 0, 0."""
    a = np.array([[1, 0], [3, 0], [-1, 0], [-3, 0], [5, 0], [-5, 0]], np.int8)
    w = np.array([[1, 1], [0, 0]], np.int8)
    case = dict(a=a, w=w, bias=None, sa=1.0, a_zp=0, ws=np.array([1.0], np.float32), w_zps=None, so=2.0, out_zp=0)
    want = oracle_int8(O.OP_MATMUL, case)
    assert want[:, 0].tolist() == [1, 2, -1, -2, 3, -3]
    for variant in (B.VARIANT_SIMT,):
        got = run_int8_linear(cuda, B.OP_MATMUL, case, variant=variant)
        assert np.array_equal(got, want)


def test_fused_quantize_and_dequantize(cuda):
    """QuantizeLinear → MatMul → DequantizeLinear in one call equals the three reference nodes."""
    rng = np.random.default_rng(8)
    case = util.make_int8_linear(3, 512, 256, seed=8, zero_points=True)
    x = (case["a"].astype(np.float32) - case["a_zp"]) * np.float32(case["sa"]) + rng.uniform(-0.49, 0.49, case["a"].shape).astype(np.float32) * np.float32(case["sa"])
    q = O.quantize_linear(O.FP32, x, [case["sa"]], [case["a_zp"]])
    case_q = dict(case, a=q)
    mid = oracle_int8(O.OP_MATMUL, case_q)
    want = O.dequantize_linear(mid, [case["so"]], [case["out_zp"]], O.FP32)
    got = run_int8_linear(cuda, B.OP_MATMUL, case_q, a_dtype=B.FP32, out_dtype=B.FP32, a_raw=x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("m", [1, 4, 16, 64, 300])
@pytest.mark.parametrize("op,bias_mode", [(B.OP_MATMUL, 0), (B.OP_GEMM, 1), (B.OP_FC, 1)])
def test_fused_quantize_and_dequantize_symmetric(cuda, m, op, bias_mode):
    """The chain a statically quantised plan holds around a classifier layer — QuantizeLinear -> FC / MatMul / Gemm ->
    DequantizeLinear with all zero points 0 — as one call on the kernel family AUTO picks (tensor cores), against the
    three reference nodes."""
    rng = np.random.default_rng(80 + m)
    case = util.make_int8_linear(m, 512, 256, seed=8 + m, bias_mode=bias_mode)
    x = case["a"].astype(np.float32) * np.float32(case["sa"]) + rng.uniform(-0.49, 0.49, case["a"].shape).astype(np.float32) * np.float32(case["sa"])
    q = O.quantize_linear(O.FP32, x, [case["sa"]], [0])
    case_q = dict(case, a=q)
    mid = oracle_int8(op, case_q)
    want = O.dequantize_linear(mid, [case["so"]], [0], O.FP32)
    got = run_int8_linear(cuda, op, case_q, a_dtype=B.FP32, out_dtype=B.FP32, a_raw=x)
    bad = int((got.view(np.uint32) != want.view(np.uint32)).sum())
    assert bad == 0, f"{bad} of {want.size} outputs differ on kernel {B.last_variant()}"


def test_overflow_and_rejections(cuda):
    import ctypes as C
    from tests.gpu_helpers import dev
    case = util.make_int8_linear(1, 64, 64, seed=1)
    a, w, ws = dev(cuda, case["a"]), dev(cuda, case["w"]), dev(cuda, case["ws"])
    out = cuda.empty((1, 64), dtype=cuda.int8, device="cuda")
    base = dict(op=B.OP_MATMUL, m=1, k=64, n=64, a=a, w=w, out=out, a_scale=1.0, a_zp=0, w_scales=ws, w_zps=None,
                w_params=64, out_scale=1.0, out_zp=0)
    f = B.lib().fth_b200_int8_linear_supported
    assert f(C.byref(B.int8_linear_desc(**base))) == B.OK
    # K·128·128 beyond int32 → declined up front instead of a device-side error flag
    assert f(C.byref(B.int8_linear_desc(**{**base, "k": 200000}))) == B.ERR_OVERFLOW
    assert f(C.byref(B.int8_linear_desc(**{**base, "bias_max_abs": 2 ** 31}))) == B.ERR_OVERFLOW
    for bad in (dict(a_scale=-1.0), dict(out_zp=200), dict(w_params=3), dict(w_scales=None), dict(trans_b=True)):
        assert f(C.byref(B.int8_linear_desc(**{**base, **bad}))) == B.ERR_INVALID, bad


@pytest.mark.parametrize("m,k,n,trans_b", [(16, 8192, 2048, False), (64, 1024, 1024, False), (128, 1024, 1024, True),
                                           (300, 512, 528, False), (257, 2048, 272, True), (33, 4096, 640, False)])
@pytest.mark.parametrize("per_channel", [True, False])
def test_tensor_core_path_shapes(cuda, m, k, n, trans_b, per_channel):
    """kind::i8 MMA with int32 TMEM accumulators and the estimate-plus-exact-fallback requantisation: bit-exact."""
    case = util.make_int8_linear(m, k, n, seed=m + n, trans_b=trans_b, per_channel=per_channel)
    op = B.OP_GEMM if trans_b else B.OP_MATMUL
    want = oracle_int8(op, case, trans_b=trans_b)
    got = run_int8_linear(cuda, op, case, trans_b=trans_b, variant=B.VARIANT_TCGEN05)
    assert B.last_variant() == "tcgen05" and B.device_status() == 0
    assert np.array_equal(got, want), f"{int((got != want).sum())} of {want.size} bytes differ"


def test_tensor_core_requant_near_ties(cuda):
    """Accumulators that land exactly on and right next to x.5 after scaling: the FP32 estimate must hand
    them to the exact double sequence (ties round away from zero)."""
    k, n = 64, 128
    a = np.zeros((130, k), np.int8)
    a[:, 0] = np.arange(-65, 65)
    a[:, 1] = 1
    w = np.zeros((k, n), np.int8)
    w[0, :] = 1
    w[1, :] = np.arange(n) % 3
    case = dict(a=a, w=w, bias=None, sa=1.0, a_zp=0, ws=np.full(n, 1.0, np.float32), w_zps=None, so=2.0, out_zp=0)
    want = oracle_int8(O.OP_MATMUL, case)
    got = run_int8_linear(cuda, B.OP_MATMUL, case, variant=B.VARIANT_TCGEN05)
    assert np.array_equal(got, want)
    case["ws"] = np.full(n, np.float32(1.0000001), np.float32)
    want = oracle_int8(O.OP_MATMUL, case)
    got = run_int8_linear(cuda, B.OP_MATMUL, case, variant=B.VARIANT_TCGEN05)
    assert np.array_equal(got, want)
