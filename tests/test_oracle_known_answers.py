"""CPU: the known-answer values of the reference's own unit tests, asserted on the C restatement."""
import numpy as np

import oracle as O


def enc(dt, v):
    return int(O.port().fo_fp8_encode(dt, float(v)))


def dec(dt, c):
    return float(O.port().fo_fp8_decode(dt, c))


def test_fp8_codec_exact_codes():
    """test/fp8_test.cc:230-279 — exact codes and round-to-nearest-even ties."""
    assert enc(O.E4M3, 1.0) == 0x38 and enc(O.E4M3, 0.001953125) == 0x01 and enc(O.E4M3, 0.015625) == 0x08
    assert enc(O.E4M3, 448.0) == 0x7E and enc(O.E4M3, 1e9) == 0x7E and enc(O.E4M3, float("inf")) == 0x7E
    assert enc(O.E4M3, float("nan")) == 0x7F
    assert enc(O.E5M2, 1.0) == 0x3C and enc(O.E5M2, 2.0 ** -16) == 0x01 and enc(O.E5M2, 2.0 ** -14) == 0x04
    assert enc(O.E5M2, 57344.0) == 0x7B and enc(O.E5M2, 1e9) == 0x7B and enc(O.E5M2, float("inf")) == 0x7C
    assert enc(O.E5M2, float("nan")) == 0x7D
    # ties to even on E4M3 (3 mantissa bits): 1.0625 → 1.0, 1.1875 → 1.25, and E5M2 (2 bits): 1.125 → 1.0, 1.375 → 1.5
    assert enc(O.E4M3, 1.0625) == 0x38 and enc(O.E4M3, 1.1875) == 0x3A
    assert enc(O.E5M2, 1.125) == 0x3C and enc(O.E5M2, 1.375) == 0x3E
    assert enc(O.E4M3, -1.0) == 0xB8 and enc(O.E4M3, -0.0) == 0x80


def test_fp8_round_trip_all_codes():
    for dt, nan_codes in ((O.E4M3, {0x7F, 0xFF}), (O.E5M2, {0x7D, 0x7E, 0x7F, 0xFD, 0xFE, 0xFF})):
        for c in range(256):
            v = dec(dt, c)
            if c in nan_codes:
                assert np.isnan(v)
            else:
                assert enc(dt, v) == c, (dt, c)


def test_fp8_matmul_small_integers():
    """test/fp8_test.cc:768-820 — {1,2,3,4} x {5,6,7,8} = {19,22,43,50} through MatMul, Gemm and FC."""
    a = O.fp8_encode(O.E4M3, np.array([[1, 2], [3, 4]], np.float32) / 0.25)
    w = O.fp8_encode(O.E4M3, np.array([[5, 6], [7, 8]], np.float32) / 0.5)
    for op in (O.OP_MATMUL, O.OP_GEMM, O.OP_FC):
        out = O.fp8_linear(op, O.E4M3, a, 0.25, w, 0.5, 0.25)
        val = O.fp8_decode(O.E4M3, out) * 0.25
        assert np.allclose(val, [[19, 22], [43, 50]], atol=2.0)
        # 19 → 20 and 43 → 44 are the nearest E4M3 values at scale 0.25; 22 → 22, 50 → 48 or 52 (tie to even: 48)
        assert val.tolist() == [[20.0, 22.0], [44.0, 48.0]]


def test_fp8_linear_pattern_case():
    """test/x86_fp8_linear_test.cc:60-101 — M2 K17 N64 pattern inputs with a vector bias, checked against the
    plain double-precision value within the reference's own tolerance of 2.0."""
    m, k, n = 2, 17, 64
    for dt in (O.E4M3, O.E5M2):
        a = O.fp8_encode(dt, ((np.arange(m * k) % 7) - 3).astype(np.float32)).reshape(m, k)
        w = O.fp8_encode(dt, ((np.arange(k * n) % 9) - 4).astype(np.float32)).reshape(k, n)
        b = O.fp8_encode(dt, ((np.arange(n) % 5) - 2).astype(np.float32))
        out = O.fp8_linear(O.OP_FC, dt, a, 0.25, w, 0.5, 0.25, bias=b, bias_scale=0.25)
        want = (O.fp8_decode(dt, a) * 0.25).astype(np.float64) @ (O.fp8_decode(dt, w) * 0.5).astype(np.float64) + O.fp8_decode(dt, b) * 0.25
        assert np.abs(O.fp8_decode(dt, out) * 0.25 - want).max() <= 2.0


def test_e5m2_infinity_propagates():
    """test/x86_fp8_linear_test.cc:142-156."""
    a = O.fp8_encode(O.E5M2, np.ones((1, 8), np.float32))
    w = O.fp8_encode(O.E5M2, np.ones((8, 8), np.float32))
    w[3, 2] = 0x7C
    out = O.fp8_linear(O.OP_MATMUL, O.E5M2, a, 1.0, w, 1.0, 1.0)
    assert out[0, 2] == 0x7C and out[0, 0] == O.fp8_encode(O.E5M2, np.float32(8.0))


def test_int8_known_answers():
    """test/common_int8_kernel_test.cc:103-184."""
    out = O.int8_linear(O.OP_FC, np.array([[5, 1]], np.int8), 0.5, 3, np.array([[2, 3], [6, -1]], np.int8),
                        np.array([0.25, 0.5], np.float32), np.array([-2, 1], np.int32), 0.25, 10, bias=np.array([4, -4], np.int32))
    assert out.tolist() == [[8, 14]]
    out = O.int8_linear(O.OP_MATMUL, np.array([[127]], np.int8), 1.0, 0, np.array([[127]], np.int8), [1.0], None, 0.01, 0)
    assert out.tolist() == [[127]]


def test_int8_overflow_is_an_error():
    """Any running sum outside int32 fails the kernel (src/kernel/common/int8_kernel_utils.h:99-114)."""
    k = 140000
    a = np.full((1, k), -128, np.int8)
    w = np.full((k, 1), -128, np.int8)
    rc, _ = O.int8_linear(O.OP_MATMUL, a, 1.0, 0, w, [1.0], None, 1.0, 0, check=False)
    assert rc == -1


def test_quantize_value_rounds_half_away_from_zero():
    """include/quant/quantization.h:94-99 and test/quantization_math_test.cc."""
    q = O.port().fo_quantize_int8_value
    assert [q(v, 1.0, 0) for v in (0.5, -0.5, 1.5, 2.5, -2.5, 0.49999997)] == [1, -1, 2, 3, -3, 0]
    assert q(1000.0, 1.0, 0) == 127 and q(-1000.0, 1.0, 0) == -128 and q(1.0, 0.5, 3) == 5


def test_conv_known_answer_and_padding():
    """test/common_int8_kernel_test.cc:186-211 (bias enters before requantisation) and a 3x3 pad-1 case against
    a naive integer loop (the pattern of :326-443)."""
    out = O.int8_conv2d(np.array([[[[4]]]], np.int8), 0.5, 0, np.array([[[[3]]]], np.int8), [0.5], None, np.array([12], np.int32), 1.0, 0, pad=(0, 0))
    assert out.tolist() == [[[[6]]]]
    rng = np.random.default_rng(0)
    x = rng.integers(-128, 128, (1, 3, 5, 6)).astype(np.int8)
    w = rng.integers(-128, 128, (2, 3, 3, 3)).astype(np.int8)
    out = O.int8_conv2d(x, 1.0, 0, w, [1.0], None, None, 4096.0, 0)
    xp = np.pad(x.astype(np.int64), ((0, 0), (0, 0), (1, 1), (1, 1)))
    for o in range(2):
        for y in range(5):
            for z in range(6):
                acc = int((xp[0, :, y:y + 3, z:z + 3] * w[o].astype(np.int64)).sum())
                t = acc / 4096.0
                want = int(np.clip(np.sign(t) * np.floor(abs(t) + 0.5), -128, 127))
                assert out[0, o, y, z] == want


def test_fp8_per_channel_weight_scales_are_the_per_tensor_kernel_column_by_column():
    """The per-channel extension has no reference kernel (include/util/types.h:96-101 keeps FP8 per-tensor); its
    definition is the reference's kernel applied to each column with that column's scale — on both implementations."""
    from tests import util
    case = util.make_fp8_linear(O.E4M3, 3, 256, 96, seed=7, pow2=True)
    same = np.full(96, case["sw"], np.float32)
    plain = O.fp8_linear(O.OP_MATMUL, O.E4M3, case["a"], case["sa"], case["w"], case["sw"], case["so"])
    assert np.array_equal(O.fp8_linear_per_channel(O.OP_MATMUL, O.E4M3, case["a"], case["sa"], case["w"], same, case["so"]), plain)
    scales = (case["sw"] * np.exp2(np.arange(96) % 4 - 1)).astype(np.float32)
    port = O.fp8_linear_per_channel(O.OP_MATMUL, O.E4M3, case["a"], case["sa"], case["w"], scales, case["so"])
    ref = O.fp8_linear_per_channel(O.OP_MATMUL, O.E4M3, case["a"], case["sa"], case["w"], scales, case["so"], impl="ref")
    assert np.array_equal(port, ref)
    for n in (0, 1, 2, 3, 95):
        col = O.fp8_linear(O.OP_MATMUL, O.E4M3, case["a"], case["sa"], np.ascontiguousarray(case["w"][:, n:n + 1]), float(scales[n]), case["so"])
        assert np.array_equal(port[:, n:n + 1], col)
    assert not np.array_equal(port, plain)
