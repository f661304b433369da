"""Generates tests/golden/reference_outputs.npz by running the UNMODIFIED reference CPU library
(oracle/_ref/libfeather_ref.so, built by `make -C oracle ref` next to a reference checkout) on the seeded
cases of tests/golden/cases.py.  Run from the repository root:  python tests/golden/make_golden.py

The fixture holds only outputs (plus input digests), a few hundred KB; the tests regenerate the inputs."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from tests.golden import cases as G  # noqa: E402


def main():
    assert O.have_ref(), "build oracle/_ref first: make -C oracle ref"
    out = {}
    vals = G.codec_values()
    out["codec/digest"] = np.array(G.digest(vals))
    for name, dt in (("e4m3", O.E4M3), ("e5m2", O.E5M2)):
        out[f"codec/{name}/encode"] = O.fp8_encode(dt, vals, impl="ref")
        out[f"codec/{name}/decode"] = O.fp8_decode(dt, np.arange(256, dtype=np.uint8), impl="ref").view(np.uint32)
    for entry in G.FP8_LINEAR:
        case, kw = G.fp8_linear_case(entry)
        name, dtype, op = entry[0], entry[1], entry[2]
        out[f"fp8/{name}/digest"] = np.array(G.digest(case["a"], case["w"], case["bias"]))
        for dev_name, dev in (("common", O.COMMON), ("x86", O.X86)):
            out[f"fp8/{name}/{dev_name}"] = O.fp8_linear(op, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"],
                                                         impl="ref", device=dev, **kw)
    for entry in G.INT8_LINEAR:
        case, kw = G.int8_linear_case(entry)
        name, op = entry[0], entry[1]
        out[f"int8/{name}/digest"] = np.array(G.digest(case["a"], case["w"], case["bias"], case["ws"]))
        for dev_name, dev in (("common", O.COMMON), ("x86", O.X86)):
            out[f"int8/{name}/{dev_name}"] = O.int8_linear(op, case["a"], case["sa"], case["a_zp"], case["w"], case["ws"],
                                                           case["w_zps"], case["so"], case["out_zp"], impl="ref", device=dev, **kw)
    for entry in G.INT8_CONV:
        case, kw = G.int8_conv_case(entry)
        name = entry[0]
        out[f"conv/{name}/digest"] = np.array(G.digest(case["x"], case["w"], case["bias"], case["ws"]))
        for dev_name, dev in (("common", O.COMMON), ("x86", O.X86)):
            y = O.int8_conv2d(case["x"], case["sx"], case["x_zp"], case["w"], case["ws"], case["w_zps"], case["bias"],
                              case["so"], case["out_zp"], impl="ref", device=dev, **kw)
            out[f"conv/{name}/{dev_name}"] = y
        out[f"conv/{name}/relu"] = O.int8_relu(out[f"conv/{name}/common"], case["so"], case["out_zp"], case["so"] * 0.7, -3, impl="ref")
    # QuantizeLinear / DequantizeLinear / Cast
    rng = np.random.default_rng(99)
    x = (rng.standard_normal((9, 130)) * 2).astype(np.float32)
    sc = rng.uniform(0.01, 0.1, 130).astype(np.float32)
    zp = rng.integers(-20, 20, 130).astype(np.int32)
    out["qdq/digest"] = np.array(G.digest(x, sc, zp))
    out["qdq/q_per_channel"] = O.quantize_linear(O.FP32, x, sc, zp, impl="ref")
    out["qdq/q_per_tensor"] = O.quantize_linear(O.FP32, x, sc[:1], zp[:1], impl="ref")
    q = out["qdq/q_per_channel"]
    out["qdq/dq_fp32"] = O.dequantize_linear(q, sc, zp, O.FP32, impl="ref").view(np.uint32)
    out["qdq/dq_bf16"] = O.dequantize_linear(q, sc, zp, O.BF16, impl="ref")
    out["qdq/dq_fp16"] = O.dequantize_linear(q, sc[:1], zp[:1], O.FP16, impl="ref")
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)
    out["cast/bf16_to_e5m2"] = O.cast(O.BF16, xb, 1.0, O.E5M2, 0.125, impl="ref")
    out["cast/fp32_to_e4m3"] = O.cast(O.FP32, x, 1.0, O.E4M3, 0.03125, impl="ref")
    out["cast/e5m2_to_bf16"] = O.cast(O.E5M2, out["cast/bf16_to_e5m2"], 0.125, O.BF16, 1.0, impl="ref")
    out["cast/e4m3_to_fp32"] = O.cast(O.E4M3, out["cast/fp32_to_e4m3"], 0.03125, O.FP32, 1.0, impl="ref").view(np.uint32)
    # QwenRmsNorm / Add / Mul / SiLU (Common and x86) and the fused FP8 lm-head selection (x86 only)
    d = G.decoder_op_inputs()
    out["dec/digest"] = np.array(G.digest(*[d[k] for k in sorted(d)]))
    for dev_name, dev in (("common", O.COMMON), ("x86", O.X86)):
        out[f"dec/rms_bf16/{dev_name}"] = O.qwen_rms_norm(O.BF16, d["rms_x_bf16"], O.BF16, d["rms_w_bf16"], 1.0, 1e-6, O.BF16, impl="ref", device=dev)
        out[f"dec/rms_fp32/{dev_name}"] = O.qwen_rms_norm(O.FP32, d["rms_x_fp32"], O.FP32, d["rms_w_fp32"], 0.0, 1e-5, O.FP32, impl="ref", device=dev).view(np.uint32)
        out[f"dec/rms_bf16_to_fp32/{dev_name}"] = O.qwen_rms_norm(O.BF16, d["rms_x_bf16"], O.FP32, O.fp8_decode(O.E4M3, np.arange(1024) % 120), 0.5, 1e-6, O.FP32,
                                                                 impl="ref", device=dev).view(np.uint32)
        for op_name, op in (("add", 0), ("mul", 1)):
            out[f"dec/{op_name}_bf16/{dev_name}"] = O.binary(op, O.BF16, d["bin_lhs_bf16"], d["bin_rhs_bf16"], impl="ref", device=dev)
            out[f"dec/{op_name}_row_bf16/{dev_name}"] = O.binary(op, O.BF16, d["bin_lhs_bf16"], d["bin_row_bf16"], impl="ref", device=dev)
            out[f"dec/{op_name}_fp32/{dev_name}"] = O.binary(op, O.FP32, d["bin_lhs_fp32"], d["bin_rhs_fp32"], impl="ref", device=dev).view(np.uint32)
        out[f"dec/silu_bf16/{dev_name}"] = O.silu(O.BF16, d["silu_bf16"], impl="ref", device=dev)
        out[f"dec/silu_fp32/{dev_name}"] = O.silu(O.FP32, d["silu_fp32"], impl="ref", device=dev).view(np.uint32)
    for entry in G.ARGMAX:
        c = G.argmax_case(entry)
        name, dtype = entry[0], entry[1]
        out[f"argmax/{name}/digest"] = np.array(G.digest(c["a"], c["b"]))
        out[f"argmax/{name}/x86_index"] = np.array(O.qwen_gemm_argmax(dtype, c["a"], c["sa"], c["b"], c["sb"], c["so"]))
        # the materialised output row of the same projection through the Common Gemm kernel (b is [N, K]: trans_b)
        out[f"argmax/{name}/common_codes"] = O.fp8_linear(O.OP_GEMM, dtype, c["a"], c["sa"], c["b"], c["sb"], c["so"], trans_b=True, impl="ref", device=O.COMMON)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KB")


if __name__ == "__main__":
    main()
