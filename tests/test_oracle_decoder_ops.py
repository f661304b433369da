"""CPU: pins the restatement of QwenRmsNorm / Add / Mul / SiLU (oracle/feather_oracle.c) against outputs of the
unmodified reference's Common kernels stored in tests/golden/reference_outputs.npz, and records how far the reference's
own x86 kernels sit from its Common kernels on the same inputs (the tolerance the GPU tests use is tighter)."""
import os

import numpy as np

import oracle as O
from tests.golden import cases as G

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


def _inputs():
    d = G.decoder_op_inputs()
    assert G.digest(*[d[k] for k in sorted(d)]) == str(GOLD["dec/digest"])
    return d


def test_rms_norm_port_equals_reference_common():
    d = _inputs()
    assert np.array_equal(O.qwen_rms_norm(O.BF16, d["rms_x_bf16"], O.BF16, d["rms_w_bf16"], 1.0, 1e-6, O.BF16), GOLD["dec/rms_bf16/common"])
    assert np.array_equal(O.qwen_rms_norm(O.FP32, d["rms_x_fp32"], O.FP32, d["rms_w_fp32"], 0.0, 1e-5, O.FP32).view(np.uint32),
                          GOLD["dec/rms_fp32/common"])
    w = O.fp8_decode(O.E4M3, np.arange(1024) % 120)
    assert np.array_equal(O.qwen_rms_norm(O.BF16, d["rms_x_bf16"], O.FP32, w, 0.5, 1e-6, O.FP32).view(np.uint32), GOLD["dec/rms_bf16_to_fp32/common"])


def test_reference_x86_rms_norm_is_not_bit_identical_to_its_common_kernel():
    """The reference's kernels reduce and round in different ways: BF16 outputs one code apart, FP32 outputs tens of
    FP32 steps apart.  A parallel reduction on the GPU is held to one BF16 code / 16 + hidden / 32 FP32 steps."""
    bf = np.abs(GOLD["dec/rms_bf16/common"].astype(np.int64) - GOLD["dec/rms_bf16/x86"].astype(np.int64))
    fp = np.abs(GOLD["dec/rms_bf16_to_fp32/common"].astype(np.int64) - GOLD["dec/rms_bf16_to_fp32/x86"].astype(np.int64))
    assert 0 < bf.max() <= 1 and fp.max() > 4


def test_binary_and_silu_port_equals_reference_common_and_x86():
    d = _inputs()
    for name, op in (("add", 0), ("mul", 1)):
        for dev in ("common", "x86"):
            assert np.array_equal(O.binary(op, O.BF16, d["bin_lhs_bf16"], d["bin_rhs_bf16"]), GOLD[f"dec/{name}_bf16/{dev}"])
            assert np.array_equal(O.binary(op, O.BF16, d["bin_lhs_bf16"], d["bin_row_bf16"]), GOLD[f"dec/{name}_row_bf16/{dev}"])
            assert np.array_equal(O.binary(op, O.FP32, d["bin_lhs_fp32"], d["bin_rhs_fp32"]).view(np.uint32), GOLD[f"dec/{name}_fp32/{dev}"])
    for dev in ("common", "x86"):
        assert np.array_equal(O.silu(O.BF16, d["silu_bf16"]), GOLD[f"dec/silu_bf16/{dev}"])
        assert np.array_equal(O.silu(O.FP32, d["silu_fp32"]).view(np.uint32), GOLD[f"dec/silu_fp32/{dev}"])


def test_lm_head_selection_rule_of_the_reference_x86_kernel():
    """The fused FP8 projection + greedy selection exists only as an x86 kernel in the reference
    (src/kernel/x86/linear_fp8.cc:733-1004).  Its answer must be explainable from the materialised Common output row:
    the selected row holds the largest non-NaN decoded code value or is within one code of it (the two kernels
    accumulate in different orders), and on the exact-integer cases it is the lowest index among the maxima."""
    for entry in G.ARGMAX:
        name, dtype = entry[0], entry[1]
        c = G.argmax_case(entry)
        assert G.digest(c["a"], c["b"]) == str(GOLD[f"argmax/{name}/digest"])
        codes = GOLD[f"argmax/{name}/common_codes"][0]
        assert np.array_equal(codes, O.fp8_linear(O.OP_GEMM, dtype, c["a"], c["sa"], c["b"], c["sb"], c["so"], trans_b=True)[0])
        values = O.fp8_decode(dtype, codes).astype(np.float64)
        values[np.isnan(values)] = -np.inf
        index = int(GOLD[f"argmax/{name}/x86_index"])
        if entry[5] == "random":
            from tests import util
            best = int(np.argmax(values))
            assert util.fp8_code_distance(codes[index:index + 1], codes[best:best + 1]).max() <= 1
        else:
            assert index == int(np.argmax(values))  # numpy returns the first maximum
    assert int(GOLD["argmax/argmax_e4m3_ties/x86_index"]) == 77 and int(GOLD["argmax/argmax_e5m2_nan_column/x86_index"]) == 200
