"""CPU: pins the C restatement (oracle/feather_oracle.c) against outputs of the unmodified reference library
stored in tests/golden/reference_outputs.npz, and — where oracle/_ref is present — against the library live."""
import os

import numpy as np
import pytest

import oracle as O
from tests import util
from tests.golden import cases as G

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


def test_codec_matches_reference_outputs():
    vals = G.codec_values()
    assert G.digest(vals) == str(GOLD["codec/digest"])
    for name, dt in (("e4m3", O.E4M3), ("e5m2", O.E5M2)):
        assert np.array_equal(O.fp8_encode(dt, vals), GOLD[f"codec/{name}/encode"])
        assert np.array_equal(O.fp8_decode(dt, np.arange(256, dtype=np.uint8)).view(np.uint32), GOLD[f"codec/{name}/decode"])


@pytest.mark.parametrize("entry", G.FP8_LINEAR, ids=[e[0] for e in G.FP8_LINEAR])
def test_fp8_linear_matches_reference_common(entry):
    case, kw = G.fp8_linear_case(entry)
    name, dtype, op = entry[0], entry[1], entry[2]
    assert G.digest(case["a"], case["w"], case["bias"]) == str(GOLD[f"fp8/{name}/digest"])
    got = O.fp8_linear(op, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"], **kw)
    assert np.array_equal(got, GOLD[f"fp8/{name}/common"])
    if case["bias"] is None:
        # without a bias the reference's x86 path stays within one code of its Common path
        assert util.fp8_code_distance(GOLD[f"fp8/{name}/x86"], GOLD[f"fp8/{name}/common"]).max() <= 1


@pytest.mark.parametrize("entry", G.INT8_LINEAR, ids=[e[0] for e in G.INT8_LINEAR])
def test_int8_linear_matches_reference(entry):
    case, kw = G.int8_linear_case(entry)
    name, op = entry[0], entry[1]
    assert G.digest(case["a"], case["w"], case["bias"], case["ws"]) == str(GOLD[f"int8/{name}/digest"])
    got = O.int8_linear(op, case["a"], case["sa"], case["a_zp"], case["w"], case["ws"], case["w_zps"], case["so"], case["out_zp"], **kw)
    assert np.array_equal(got, GOLD[f"int8/{name}/common"])
    assert np.array_equal(GOLD[f"int8/{name}/x86"], GOLD[f"int8/{name}/common"])  # x86 INT8 linear is the same scalar rule


@pytest.mark.parametrize("entry", G.INT8_CONV, ids=[e[0] for e in G.INT8_CONV])
def test_int8_conv_matches_reference_common(entry):
    case, kw = G.int8_conv_case(entry)
    name = entry[0]
    assert G.digest(case["x"], case["w"], case["bias"], case["ws"]) == str(GOLD[f"conv/{name}/digest"])
    got = O.int8_conv2d(case["x"], case["sx"], case["x_zp"], case["w"], case["ws"], case["w_zps"], case["bias"], case["so"], case["out_zp"], **kw)
    assert np.array_equal(got, GOLD[f"conv/{name}/common"])
    assert np.array_equal(O.int8_relu(got, case["so"], case["out_zp"], case["so"] * 0.7, -3), GOLD[f"conv/{name}/relu"])
    # The reference's x86 kernel is not the oracle: its fast paths requantise in FP32 (a few bytes per million
    # differ from Common) and, with dilation > 1, its outputs disagree with Common almost everywhere
    # (measured: 98 % of bytes on this case) — Common, which matches the direct definition, is canonical.
    if kw["dil"] == (1, 1):
        assert (GOLD[f"conv/{name}/x86"] != GOLD[f"conv/{name}/common"]).mean() < 1e-4


def test_qdq_and_cast_match_reference():
    rng = np.random.default_rng(99)
    x = (rng.standard_normal((9, 130)) * 2).astype(np.float32)
    sc = rng.uniform(0.01, 0.1, 130).astype(np.float32)
    zp = rng.integers(-20, 20, 130).astype(np.int32)
    assert G.digest(x, sc, zp) == str(GOLD["qdq/digest"])
    q = O.quantize_linear(O.FP32, x, sc, zp)
    assert np.array_equal(q, GOLD["qdq/q_per_channel"])
    assert np.array_equal(O.quantize_linear(O.FP32, x, sc[:1], zp[:1]), GOLD["qdq/q_per_tensor"])
    assert np.array_equal(O.dequantize_linear(q, sc, zp, O.FP32).view(np.uint32), GOLD["qdq/dq_fp32"])
    assert np.array_equal(O.dequantize_linear(q, sc, zp, O.BF16), GOLD["qdq/dq_bf16"])
    assert np.array_equal(O.dequantize_linear(q, sc[:1], zp[:1], O.FP16), GOLD["qdq/dq_fp16"])
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)
    c1 = O.cast(O.BF16, xb, 1.0, O.E5M2, 0.125)
    c2 = O.cast(O.FP32, x, 1.0, O.E4M3, 0.03125)
    assert np.array_equal(c1, GOLD["cast/bf16_to_e5m2"]) and np.array_equal(c2, GOLD["cast/fp32_to_e4m3"])
    assert np.array_equal(O.cast(O.E5M2, c1, 0.125, O.BF16, 1.0), GOLD["cast/e5m2_to_bf16"])
    assert np.array_equal(O.cast(O.E4M3, c2, 0.03125, O.FP32, 1.0).view(np.uint32), GOLD["cast/e4m3_to_fp32"])


@pytest.mark.skipif(not O.have_ref(), reason="oracle/_ref/libfeather_ref.so not built (needs a reference checkout)")
def test_port_equals_live_reference_on_random_cases():
    rng = np.random.default_rng(7)
    for dt in (O.E4M3, O.E5M2):
        v = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 1, 100, 1e5)])
        assert np.array_equal(O.fp8_encode(dt, v), O.fp8_encode(dt, v, impl="ref"))
        case = util.make_fp8_linear(dt, 3, 65, 130, seed=5, bias_mode=1)
        kw = dict(bias=case["bias"], bias_scale=case["sb"])
        assert np.array_equal(O.fp8_linear(O.OP_FC, dt, case["a"], case["sa"], case["w"], case["sw"], case["so"], **kw),
                              O.fp8_linear(O.OP_FC, dt, case["a"], case["sa"], case["w"], case["sw"], case["so"], impl="ref", **kw))
    case = util.make_int8_linear(4, 96, 80, seed=6, zero_points=True, bias_mode=2)
    args = (O.OP_FC, case["a"], case["sa"], case["a_zp"], case["w"], case["ws"], case["w_zps"], case["so"], case["out_zp"])
    assert np.array_equal(O.int8_linear(*args, bias=case["bias"]), O.int8_linear(*args, bias=case["bias"], impl="ref"))
