"""Seeded case definitions shared by the fixture generator and the tests that read the fixtures.

Inputs are regenerated from the seed (numpy PCG64 streams are stable across versions); a SHA-256 of the
inputs stored beside each golden output guards against a generator drift."""
from __future__ import annotations

import hashlib

import numpy as np

import oracle as O
from tests import util


def lcg_floats(count: int) -> np.ndarray:
    """Bit patterns from the reference's own encoder-equivalence test (test/x86_fp8_linear_test.cc:268-292):
    state = state * 1664525 + 1013904223 (mod 2^32), seeded with 0x12345678."""
    state = 0x12345678
    out = np.empty(count, np.uint32)
    for i in range(count):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = state
    return out.view(np.float32)


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


FP8_LINEAR = [  # name, dtype, op, m, k, n, trans_b, bias_mode, pow2
    ("e4m3_fc_c1", O.E4M3, O.OP_FC, 1, 1024, 3072, False, 0, False),
    ("e4m3_matmul_pow2", O.E4M3, O.OP_MATMUL, 3, 512, 320, False, 0, True),
    ("e5m2_matmul_c4_gate", O.E5M2, O.OP_MATMUL, 2, 1024, 3584, False, 0, True),
    ("e5m2_gemm_transb_bias", O.E5M2, O.OP_GEMM, 2, 528, 77, True, 1, False),
    ("e4m3_gemm_matrix_bias", O.E4M3, O.OP_GEMM, 5, 130, 272, False, 2, False),
    ("e4m3_fc_vector_bias", O.E4M3, O.OP_FC, 2, 17, 64, False, 1, False),
]

INT8_LINEAR = [  # name, op, m, k, n, trans_b, per_channel, zero_points, bias_mode
    ("int8_matmul_c2", O.OP_MATMUL, 128, 1024, 1024, False, True, False, 0),
    ("int8_fc_zp_bias", O.OP_FC, 6, 192, 144, False, True, True, 1),
    ("int8_gemm_transb", O.OP_GEMM, 5, 528, 19, True, True, True, 1),
    ("int8_fc_per_tensor_matrix_bias", O.OP_FC, 3, 100, 48, False, False, True, 2),
]

INT8_CONV = [  # name, (b, ic, ih, iw, oc, kh, kw), stride, pad, dil, group, zero_points
    ("conv_c3_small", (1, 64, 20, 24, 64, 3, 3), (1, 1), (1, 1), (1, 1), 1, False),
    ("conv_strided_zp", (2, 16, 21, 23, 8, 3, 3), (2, 2), (1, 1), (1, 1), 1, True),
    ("conv_dilated_grouped", (1, 16, 15, 17, 8, 3, 3), (1, 1), (2, 2), (2, 2), 4, True),
    ("conv_1x1", (1, 64, 9, 11, 32, 1, 1), (1, 1), (0, 0), (1, 1), 1, False),
]


def fp8_linear_case(entry):
    name, dtype, op, m, k, n, tb, bias_mode, pow2 = entry
    seed = int(hashlib.sha256(name.encode()).hexdigest()[:8], 16)
    case = util.make_fp8_linear(dtype, m, k, n, seed, trans_b=tb, pow2=pow2, bias_mode=bias_mode)
    kw = dict(bias=case["bias"], bias_scale=case["sb"], trans_b=tb)
    if op == O.OP_GEMM:
        kw.update(alpha=0.75, beta=1.25)
    return case, kw


def int8_linear_case(entry):
    name, op, m, k, n, tb, per_channel, zps, bias_mode = entry
    seed = int(hashlib.sha256(name.encode()).hexdigest()[:8], 16)
    case = util.make_int8_linear(m, k, n, seed, trans_b=tb, per_channel=per_channel, zero_points=zps, bias_mode=bias_mode)
    kw = dict(bias=case["bias"], trans_b=tb)
    if op == O.OP_GEMM:
        kw.update(alpha=0.5, beta=2.0)
    return case, kw


def int8_conv_case(entry):
    name, shape, stride, pad, dil, group, zps = entry
    seed = int(hashlib.sha256(name.encode()).hexdigest()[:8], 16)
    b, ic, ih, iw, oc, kh, kw = shape
    case = util.make_int8_conv(b, ic, ih, iw, oc, kh, kw, seed, zero_points=zps)
    if group > 1:
        case["w"] = np.ascontiguousarray(case["w"][:, :ic // group])
    return case, dict(stride=stride, pad=pad, dil=dil, group=group)


def codec_values() -> np.ndarray:
    with np.errstate(all="ignore"):
        specials = np.array([0.0, np.inf, np.nan, 448.0, 449.0, 464.0, 480.0, 57344.0, 61440.0, 65536.0, 2.0 ** -9,
                             2.0 ** -10, 2.0 ** -16, 2.0 ** -17, 1.0625, 1.1875, 1.125, 1.375, 0.015625,
                             0.0146484375, 6.103515625e-05, 3.0e-05, 1.0, 0.001953125, 0.125, 224.0], np.float32)
        rng = np.random.default_rng(1234)
        return np.concatenate([specials, -specials, lcg_floats(20000), (rng.standard_normal(20000) * 50).astype(np.float32),
                               (rng.standard_normal(20000) * 1e-3).astype(np.float32)])


# ---- the operators between the projections of a decoder block, and the fused lm-head selection ----------------------
def to_bf16(x):
    """float32 -> BF16 bits, round to nearest even (finite inputs)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def decoder_op_inputs():
    rng = np.random.default_rng(0xDEC0DE)
    d = {}
    d["rms_x_bf16"] = to_bf16(rng.standard_normal((5, 1024)).astype(np.float32) * np.float32(3.0))
    d["rms_w_bf16"] = to_bf16(rng.standard_normal(1024).astype(np.float32) * np.float32(0.1))
    d["rms_x_fp32"] = (rng.standard_normal((3, 130)) * 0.5).astype(np.float32)
    d["rms_w_fp32"] = (rng.standard_normal(130) * 0.1 + 1.0).astype(np.float32)
    d["bin_lhs_bf16"] = to_bf16(rng.standard_normal((4, 1030)).astype(np.float32) * np.float32(2.0))
    d["bin_rhs_bf16"] = to_bf16(rng.standard_normal((4, 1030)).astype(np.float32))
    d["bin_row_bf16"] = to_bf16(rng.standard_normal(1030).astype(np.float32))
    d["bin_lhs_fp32"] = rng.standard_normal((2, 77)).astype(np.float32)
    d["bin_rhs_fp32"] = rng.standard_normal((2, 77)).astype(np.float32)
    silu = np.concatenate([rng.standard_normal(7000).astype(np.float32) * np.float32(3.0),
                           np.array([0.0, -0.0, 30.0, -30.0, 88.0, -88.0, 100.0, -100.0, 1e-8, -1e-8], np.float32)])
    d["silu_bf16"] = to_bf16(silu)
    d["silu_fp32"] = silu
    return d


ARGMAX = [  # name, dtype, k, n, output_scale factor, kind
    ("argmax_e4m3_random", O.E4M3, 256, 4096, 1.0, "random"),
    ("argmax_e5m2_random", O.E5M2, 512, 2048, 0.5, "random"),
    ("argmax_e4m3_ties", O.E4M3, 64, 640, 1.0, "ties"),
    ("argmax_e5m2_nan_column", O.E5M2, 64, 256, 2.0, "nan"),
]


def argmax_case(entry):
    """a [1, K] codes, b [N, K] codes (vocabulary rows), scales.  "ties": small integers, so every product sum is exact
    in FP32 and several rows reach the same maximum (the lowest index must win); "nan": the best row holds a NaN code
    and must be skipped."""
    name, dtype, k, n, so_factor, kind = entry
    seed = int(hashlib.sha256(name.encode()).hexdigest()[:8], 16)
    rng = np.random.default_rng(seed)
    if kind == "random":
        case = util.make_fp8_linear(dtype, 1, k, n, seed, trans_b=True)
        return dict(a=case["a"], sa=case["sa"], b=case["w"], sb=case["sw"], so=case["so"] * so_factor)
    a = O.fp8_encode(dtype, rng.integers(-2, 3, (1, k)).astype(np.float32))
    b = O.fp8_encode(dtype, rng.integers(-2, 3, (n, k)).astype(np.float32))
    if kind == "ties":
        best = O.fp8_encode(dtype, np.sign(O.fp8_decode(dtype, a)).astype(np.float32) * 2.0)  # the largest possible sum
        for row in (77, 300, 301, 639):
            b[row] = best[0]
    else:
        best = O.fp8_encode(dtype, np.sign(O.fp8_decode(dtype, a)).astype(np.float32) * 2.0)
        b[10] = best[0]
        b[10, 3] = 0x7D if dtype == O.E5M2 else 0x7F  # NaN: the whole row's sum is NaN and cannot be selected
        b[200] = best[0]
        b[200, :8] = O.fp8_encode(dtype, np.zeros(8, np.float32))
    return dict(a=a, sa=1.0, b=b, sb=1.0, so=float(k) / 32 * so_factor)
