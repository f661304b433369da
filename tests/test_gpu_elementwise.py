"""FP8 codec, Cast, QuantizeLinear, DequantizeLinear and the INT8 ReLU table on the GPU: bit-exact."""
import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests.gpu_helpers import dev

pytestmark = pytest.mark.gpu
NP = {B.FP32: np.float32, B.BF16: np.uint16, B.FP16: np.uint16, B.E4M3: np.uint8, B.E5M2: np.uint8}


def gpu_cast(torch, in_dtype, x, in_scale, out_dtype, out_scale):
    xd = dev(torch, x)
    out = torch.zeros(x.size * np.dtype(NP[out_dtype]).itemsize + 16, dtype=torch.uint8, device="cuda")
    B.cast(in_dtype, xd, in_scale, out_dtype, out, out_scale, x.size)
    torch.cuda.synchronize()
    host = out.cpu().numpy()
    assert (host[-16:] == 0).all()
    return host[:-16].view(NP[out_dtype]).copy()


def lcg_floats(count):
    """The bit-pattern generator of test/x86_fp8_linear_test.cc:268-292: state = state*1664525 + 1013904223."""
    state = np.uint64(0x12345678)
    out = np.empty(count, np.uint32)
    for i in range(count):
        state = (state * np.uint64(1664525) + np.uint64(1013904223)) & np.uint64(0xFFFFFFFF)
        out[i] = state
    return out.view(np.float32)


@pytest.mark.parametrize("dtype", [B.E4M3, B.E5M2])
def test_encode_matches_reference_codec(cuda, dtype):
    rng = np.random.default_rng(0)
    with np.errstate(all="ignore"):
        specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, -np.nan, 448.0, 449.0, 464.0, 480.0, 57344.0, 61440.0,
                             65536.0, 2.0 ** -9, 2.0 ** -10, 2.0 ** -16, 2.0 ** -17, 1.0625, 1.1875, 1.125, 1.375,
                             0.015625, 0.0146484375, 6.103515625e-05, 3.0e-05], np.float32)
        values = np.concatenate([specials, -specials, lcg_floats(100000),
                                 rng.standard_normal(200000).astype(np.float32) * 100.0,
                                 (rng.standard_normal(200000) * 1e-3).astype(np.float32)])
    got = gpu_cast(cuda, B.FP32, values, 1.0, dtype, 1.0)
    want = O.fp8_encode(dtype, values)
    assert np.array_equal(got, want), f"{int((got != want).sum())} codes differ"


@pytest.mark.parametrize("dtype", [B.E4M3, B.E5M2])
def test_decode_all_codes(cuda, dtype):
    codes = np.arange(256, dtype=np.uint8)
    got = gpu_cast(cuda, dtype, codes, 0.75, B.FP32, 1.0)
    want = O.cast(dtype, codes, 0.75, O.FP32, 1.0)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


@pytest.mark.parametrize("pair", [(B.FP32, B.E4M3), (B.FP32, B.E5M2), (B.BF16, B.E5M2), (B.BF16, B.E4M3), (B.E5M2, B.BF16),
                                  (B.E4M3, B.BF16), (B.E4M3, B.FP32), (B.FP32, B.BF16), (B.BF16, B.FP32), (B.FP16, B.E4M3),
                                  (B.E5M2, B.FP16)])
@pytest.mark.parametrize("count", [1, 15, 4096, 100003])
def test_cast_pairs(cuda, pair, count):
    i, o = pair
    rng = np.random.default_rng(count)
    xf = (rng.standard_normal(count) * 3).astype(np.float32)
    if i == B.FP32: x = xf
    elif i == B.BF16: x = (xf.view(np.uint32) >> 16).astype(np.uint16)
    elif i == B.FP16: x = xf.astype(np.float16).view(np.uint16)
    else: x = O.fp8_encode(i, xf / 0.25)
    got = gpu_cast(cuda, i, x, 0.25, o, 0.125)
    want = O.cast(i, x, 0.25, o, 0.125)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("x_dtype", [B.FP32, B.BF16, B.FP16])
@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("rows,channels", [(1, 1), (7, 33), (128, 1024)])
def test_quantize_linear(cuda, x_dtype, per_channel, rows, channels):
    rng = np.random.default_rng(rows + channels)
    xf = (rng.standard_normal((rows, channels)) * 2).astype(np.float32)
    xf.flat[0] = 0.5 * 0.05  # an exact tie on a per-tensor scale of 0.05
    x = xf if x_dtype == B.FP32 else (xf.view(np.uint32) >> 16).astype(np.uint16) if x_dtype == B.BF16 else xf.astype(np.float16).view(np.uint16)
    p = channels if per_channel else 1
    scales = rng.uniform(0.01, 0.1, p).astype(np.float32)
    zps = rng.integers(-20, 20, p).astype(np.int32)
    want = O.quantize_linear(x_dtype, x, scales, zps)
    out = cuda.zeros((rows, channels), dtype=cuda.int8, device="cuda")
    B.quantize_linear(x_dtype, dev(cuda, x), dev(cuda, scales), dev(cuda, zps), p, out, rows, channels)
    cuda.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("to", [B.FP32, B.BF16, B.FP16])
@pytest.mark.parametrize("per_channel", [False, True])
def test_dequantize_linear(cuda, to, per_channel):
    rng = np.random.default_rng(3)
    rows, channels = 9, 130
    q = rng.integers(-128, 128, (rows, channels)).astype(np.int8)
    p = channels if per_channel else 1
    scales = rng.uniform(0.01, 0.1, p).astype(np.float32)
    zps = rng.integers(-20, 20, p).astype(np.int32)
    want = O.dequantize_linear(q, scales, zps, to)
    out = cuda.zeros(rows * channels * want.itemsize, dtype=cuda.uint8, device="cuda")
    B.dequantize_linear(dev(cuda, q), dev(cuda, scales), dev(cuda, zps), p, out, to, rows, channels)
    cuda.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(want.dtype).reshape(rows, channels), want)


@pytest.mark.parametrize("outer,channels,inner", [(2, 5, 7), (1, 64, 400), (3, 17, 1)])
def test_quantize_dequantize_per_channel_on_an_inner_axis(cuda, outer, channels, inner):
    """Parameters along the middle extent of [outer, channels, inner] (QuantizeLinearParam::axis on an NCHW activation):
    the oracle sees the same tensor with the channel axis moved last."""
    rng = np.random.default_rng(outer * 100 + channels + inner)
    x = (rng.standard_normal((outer, channels, inner)) * 2).astype(np.float32)
    scales = rng.uniform(0.01, 0.1, channels).astype(np.float32)
    zps = rng.integers(-20, 20, channels).astype(np.int32)
    moved = np.ascontiguousarray(np.moveaxis(x, 1, 2)).reshape(-1, channels)
    want_q = np.moveaxis(O.quantize_linear(O.FP32, moved, scales, zps).reshape(outer, inner, channels), 2, 1)
    q = cuda.zeros((outer, channels, inner), dtype=cuda.int8, device="cuda")
    B.quantize_linear(B.FP32, dev(cuda, x), dev(cuda, scales), dev(cuda, zps), channels, q, outer, channels, inner=inner)
    cuda.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), want_q)
    want_f = np.moveaxis(O.dequantize_linear(np.ascontiguousarray(np.moveaxis(want_q, 1, 2)).reshape(-1, channels), scales, zps, B.FP32)
                         .reshape(outer, inner, channels), 2, 1)
    f = cuda.zeros((outer, channels, inner), dtype=cuda.float32, device="cuda")
    B.dequantize_linear(q, dev(cuda, scales), dev(cuda, zps), channels, f, B.FP32, outer, channels, inner=inner)
    cuda.cuda.synchronize()
    assert np.array_equal(f.cpu().numpy().view(np.uint32), np.ascontiguousarray(want_f).view(np.uint32))


def test_quantize_known_answers(cuda):
    """include/quant/quantization.h:94-99 ties away from zero: 0.5 → 1, -0.5 → -1, 2.5 → 3; saturation."""
    x = np.array([[0.5, -0.5, 1.5, 2.5, -2.5, 1000.0, -1000.0, np.nan, np.inf, -np.inf]], np.float32)
    want = O.quantize_linear(O.FP32, x, [1.0], [0])
    assert want[0, :7].tolist() == [1, -1, 2, 3, -3, 127, -128]
    out = cuda.zeros((1, 10), dtype=cuda.int8, device="cuda")
    B.quantize_linear(B.FP32, dev(cuda, x), dev(cuda, np.array([1.0], np.float32)), dev(cuda, np.array([0], np.int32)), 1, out, 1, 10)
    cuda.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)


def test_relu_table_and_lookup(cuda):
    rng = np.random.default_rng(4)
    x = rng.integers(-128, 128, 100003).astype(np.int8)
    for (si, zi, so, zo) in [(0.5, 0, 0.5, 0), (0.05, 3, 0.031, -7), (0.2, -100, 0.01, 5)]:
        lut = B.int8_relu_table(si, zi, so, zo)
        assert np.array_equal(lut, O.int8_relu_lut(si, zi, so, zo))
        out = cuda.zeros(x.size, dtype=cuda.int8, device="cuda")
        B.int8_lookup(dev(cuda, x), out, x.size, dev(cuda, lut))
        cuda.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), O.int8_relu(x, si, zi, so, zo))
