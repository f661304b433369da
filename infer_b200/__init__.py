"""infer_b200 — B200 (sm_100a) backend for Feather's quantized-linear hot path.

The product is ``libfth_b200.so`` (hand-written CUDA behind the C ABI declared in ``include/fth_b200.h``)
plus the C++17 adapter under ``infer_b200/adapter`` that registers it with Feather's ``KernelDispatcher``.
This module is the thin Python host side used by the tests and the benchmark: ctypes mirrors of the C
structs and helpers that take device pointers from torch tensors.  torch is used for device memory and
streams only.  There is no CPU path: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FTH_B200_LIBRARY names another build of the same library (an instrumented or experimental one); default: the in-tree build
LIB_PATH = os.environ.get("FTH_B200_LIBRARY") or os.path.join(_HERE, "libfth_b200.so")

INT8, FP16, FP32, INT32, BF16, E4M3, E5M2 = 1, 3, 4, 5, 11, 12, 13
OP_FC, OP_MATMUL, OP_GEMM = 0, 1, 2
BIAS_NONE, BIAS_VECTOR, BIAS_MATRIX = 0, 1, 2
VARIANT_AUTO, VARIANT_SIMT, VARIANT_SKINNY, VARIANT_TCGEN05, VARIANT_STREAM = 0, 1, 2, 3, 4
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_OVERFLOW, ERR_TIMEOUT, ERR_SCRATCH_LIMIT = 0, -1, -2, -3, -4, -5, -6

EXPORTS = [
    "fth_b200_abi_version", "fth_b200_last_variant", "fth_b200_launch_count", "fth_b200_reset_launch_count",
    "fth_b200_fp8_linear", "fth_b200_fp8_linear_supported", "fth_b200_fp8_linear_workspace_bytes",
    "fth_b200_device_status", "fth_b200_fp8_linear_noalloc", "fth_b200_noalloc_scratch_bytes",
    "fth_b200_int8_linear", "fth_b200_int8_linear_supported", "fth_b200_int8_linear_workspace_bytes",
    "fth_b200_int8_conv2d", "fth_b200_int8_conv2d_supported", "fth_b200_int8_conv2d_workspace_bytes",
    "fth_b200_int8_conv2d_packed_weight_bytes", "fth_b200_int8_conv2d_pack_weights",
    "fth_b200_int8_relu_table", "fth_b200_int8_lookup",
    "fth_b200_quantize_linear", "fth_b200_dequantize_linear", "fth_b200_cast",
    "fth_b200_quantize_linear_axis", "fth_b200_dequantize_linear_axis", "fth_b200_small_copy",
    "fth_b200_plan_create_fp8_linear", "fth_b200_plan_create_int8_linear", "fth_b200_plan_create_int8_conv2d",
    "fth_b200_plan_run", "fth_b200_plan_launch", "fth_b200_plan_input_bytes", "fth_b200_plan_output_bytes",
    "fth_b200_plan_destroy",
    "fth_b200_peer_buffer_create", "fth_b200_peer_buffer_open", "fth_b200_peer_buffer_close", "fth_b200_peer_buffer_destroy",
    "fth_b200_gather_sync", "fth_b200_gather_wait", "fth_b200_fp8_linear_argmax",
    "fth_b200_fp8_lm_head_argmax", "fth_b200_fp8_linear_fused", "fth_b200_fp8_linear_fused_supported", "fth_b200_qwen_rms_norm", "fth_b200_binary", "fth_b200_silu", "fth_b200_silu_mul",
]
BINARY_ADD, BINARY_MUL = 0, 1


class Fp8LinearDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("op", C.c_int32), ("m", C.c_int64), ("k", C.c_int64), ("n", C.c_int64),
        ("trans_b", C.c_int32), ("a_dtype", C.c_int32), ("out_dtype", C.c_int32), ("bias_mode", C.c_int32),
        ("a", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("out", C.c_void_p), ("ldo", C.c_int64),
        ("a_scale", C.c_float), ("w_scale", C.c_float), ("bias_scale", C.c_float), ("out_scale", C.c_float),
        ("w_channel_scales", C.c_void_p), ("alpha", C.c_float), ("beta", C.c_float),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("variant", C.c_int32), ("weights_static", C.c_int32),
        ("gather_peers", C.c_int32), ("gather_out", C.c_void_p * 7),
        ("gather_world", C.c_int32), ("gather_rank", C.c_int32), ("gather_flags", C.c_void_p * 8), ("gather_multicast_out", C.c_void_p),
    ]


class Fp8LinearFusion(C.Structure):
    _fields_ = [
        ("prologue", C.c_int32), ("norm_weight_dtype", C.c_int32), ("norm_weight", C.c_void_p), ("norm_weight_offset", C.c_float),
        ("norm_epsilon", C.c_float), ("a2", C.c_void_p), ("residual", C.c_void_p), ("w2", C.c_void_p), ("w2_scale", C.c_float),
        ("out2", C.c_void_p), ("n2", C.c_int64), ("ldo2", C.c_int64), ("epilogue", C.c_int32), ("out_codes_scale", C.c_float),
        ("out_codes", C.c_void_p), ("ldo_codes", C.c_int64),
    ]


FUSE_NONE, FUSE_RMS_NORM, FUSE_SILU_MUL = 0, 1, 2
FUSE_OUT_NONE, FUSE_OUT_SILU_MUL = 0, 1


class Int8LinearDesc(C.Structure):
    _fields_ = [
        ("op", C.c_int32), ("m", C.c_int64), ("k", C.c_int64), ("n", C.c_int64), ("trans_b", C.c_int32),
        ("a_dtype", C.c_int32), ("out_dtype", C.c_int32), ("bias_mode", C.c_int32),
        ("a", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("out", C.c_void_p), ("ldo", C.c_int64),
        ("a_scale", C.c_float), ("a_zp", C.c_int32), ("w_scales", C.c_void_p), ("w_zps", C.c_void_p),
        ("w_params", C.c_int64), ("w_zp_max_abs", C.c_int32), ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("alpha", C.c_float), ("beta", C.c_float), ("bias_max_abs", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("variant", C.c_int32), ("weights_static", C.c_int32),
        ("gather_peers", C.c_int32), ("gather_out", C.c_void_p * 7),
        ("gather_world", C.c_int32), ("gather_rank", C.c_int32), ("gather_flags", C.c_void_p * 8), ("gather_multicast_out", C.c_void_p),
    ]


class Int8Conv2dDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int64), ("ic", C.c_int64), ("ih", C.c_int64), ("iw", C.c_int64), ("oc", C.c_int64),
        ("kh", C.c_int64), ("kw", C.c_int64),
        ("stride_h", C.c_int32), ("stride_w", C.c_int32), ("pad_h", C.c_int32), ("pad_w", C.c_int32),
        ("dilation_h", C.c_int32), ("dilation_w", C.c_int32), ("group", C.c_int32),
        ("x", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("out", C.c_void_p),
        ("x_scale", C.c_float), ("x_zp", C.c_int32), ("w_scales", C.c_void_p), ("w_zps", C.c_void_p),
        ("w_params", C.c_int64), ("w_zp_max_abs", C.c_int32), ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("relu_lut", C.c_void_p), ("bias_max_abs", C.c_int64), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t), ("weights_packed", C.c_int32), ("variant", C.c_int32), ("packed_w", C.c_void_p),
    ]


_lib = None


def lib():
    """Loads libfth_b200.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m infer_b200.build` (needs nvcc); "
                "this backend has no CPU or library fallback")
        handle = C.CDLL(LIB_PATH)
        handle.fth_b200_last_variant.restype = C.c_char_p
        handle.fth_b200_launch_count.restype = C.c_int64
        handle.fth_b200_int8_conv2d_workspace_bytes.restype = C.c_size_t
        handle.fth_b200_int8_conv2d_packed_weight_bytes.restype = C.c_size_t
        handle.fth_b200_fp8_linear_workspace_bytes.restype = C.c_size_t
        handle.fth_b200_int8_linear_workspace_bytes.restype = C.c_size_t
        handle.fth_b200_noalloc_scratch_bytes.restype = C.c_size_t
        handle.fth_b200_plan_input_bytes.restype = C.c_int64
        handle.fth_b200_plan_output_bytes.restype = C.c_int64
        handle.fth_b200_plan_input_bytes.argtypes = [C.c_void_p]
        handle.fth_b200_plan_output_bytes.argtypes = [C.c_void_p]
        handle.fth_b200_plan_destroy.argtypes = [C.c_void_p]
        handle.fth_b200_plan_destroy.restype = None
        handle.fth_b200_gather_sync.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_uint32, C.c_void_p]
        handle.fth_b200_gather_wait.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
        handle.fth_b200_plan_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        handle.fth_b200_plan_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _lib = handle
    return _lib


class B200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what} failed with status {code}")
        self.code = code


def check(code: int, what: str) -> None:
    if code != OK:
        raise B200Error(code, what)


def last_variant() -> str:
    return lib().fth_b200_last_variant().decode()


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def current_stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def fp8_linear_desc(*, dtype, op, m, k, n, a, w, out, a_scale, w_scale, out_scale, trans_b=False, bias=None,
                    bias_mode=BIAS_NONE, bias_scale=1.0, alpha=1.0, beta=1.0, a_dtype=0, out_dtype=0, ldo=0,
                    w_channel_scales=None, workspace=None, workspace_bytes=0,
                    variant=VARIANT_AUTO, weights_static=False) -> Fp8LinearDesc:
    d = Fp8LinearDesc()
    d.dtype, d.op, d.m, d.k, d.n, d.trans_b = dtype, op, m, k, n, int(trans_b)
    d.a_dtype, d.out_dtype, d.bias_mode = a_dtype, out_dtype, bias_mode
    d.a, d.w, d.bias, d.out, d.ldo = ptr(a), ptr(w), ptr(bias), ptr(out), ldo
    d.a_scale, d.w_scale, d.bias_scale, d.out_scale = a_scale, w_scale, bias_scale, out_scale
    d.w_channel_scales = ptr(w_channel_scales)
    d.alpha, d.beta, d.variant, d.weights_static = alpha, beta, variant, int(weights_static)
    d.workspace, d.workspace_bytes = ptr(workspace), workspace_bytes
    return d


def int8_linear_desc(*, op, m, k, n, a, w, out, a_scale, a_zp, w_scales, w_zps, w_params, out_scale, out_zp,
                     trans_b=False, bias=None, bias_mode=BIAS_NONE, alpha=1.0, beta=1.0, a_dtype=0, out_dtype=0,
                     ldo=0, w_zp_max_abs=0, bias_max_abs=0, workspace=None, workspace_bytes=0,
                     variant=VARIANT_AUTO, weights_static=False) -> Int8LinearDesc:
    d = Int8LinearDesc()
    d.op, d.m, d.k, d.n, d.trans_b = op, m, k, n, int(trans_b)
    d.a_dtype, d.out_dtype, d.bias_mode = a_dtype, out_dtype, bias_mode
    d.a, d.w, d.bias, d.out, d.ldo = ptr(a), ptr(w), ptr(bias), ptr(out), ldo
    d.a_scale, d.a_zp, d.w_scales, d.w_zps, d.w_params = a_scale, a_zp, ptr(w_scales), ptr(w_zps), w_params
    d.w_zp_max_abs, d.out_scale, d.out_zp = w_zp_max_abs, out_scale, out_zp
    d.alpha, d.beta, d.bias_max_abs, d.variant = alpha, beta, bias_max_abs, variant
    d.weights_static = int(weights_static)
    d.workspace, d.workspace_bytes = ptr(workspace), workspace_bytes
    return d


def int8_conv2d_desc(*, batch, ic, ih, iw, oc, kh, kw, x, w, out, x_scale, x_zp, w_scales, w_zps, w_params,
                     out_scale, out_zp, bias=None, stride=(1, 1), pad=(1, 1), dil=(1, 1), group=1, relu_lut=None,
                     w_zp_max_abs=0, bias_max_abs=0, workspace=None, workspace_bytes=0, weights_packed=0,
                     variant=VARIANT_AUTO) -> Int8Conv2dDesc:
    d = Int8Conv2dDesc()
    d.batch, d.ic, d.ih, d.iw, d.oc, d.kh, d.kw = batch, ic, ih, iw, oc, kh, kw
    d.stride_h, d.stride_w, d.pad_h, d.pad_w = stride[0], stride[1], pad[0], pad[1]
    d.dilation_h, d.dilation_w, d.group = dil[0], dil[1], group
    d.x, d.w, d.bias, d.out = ptr(x), ptr(w), ptr(bias), ptr(out)
    d.x_scale, d.x_zp, d.w_scales, d.w_zps, d.w_params = x_scale, x_zp, ptr(w_scales), ptr(w_zps), w_params
    d.w_zp_max_abs, d.out_scale, d.out_zp = w_zp_max_abs, out_scale, out_zp
    d.relu_lut, d.bias_max_abs = ptr(relu_lut), bias_max_abs
    d.workspace, d.workspace_bytes, d.weights_packed, d.variant = ptr(workspace), workspace_bytes, weights_packed, variant
    return d


def fp8_linear(desc: Fp8LinearDesc, stream=None) -> None:
    check(lib().fth_b200_fp8_linear(C.byref(desc), stream or current_stream()), "fth_b200_fp8_linear")


def fp8_linear_fusion(*, prologue=FUSE_NONE, norm_weight=None, norm_weight_dtype=BF16, norm_weight_offset=0.0, norm_epsilon=1e-6, a2=None,
                      residual=None, w2=None, w2_scale=1.0, out2=None, n2=0, ldo2=0, epilogue=FUSE_OUT_NONE, out_codes=None,
                      out_codes_scale=1.0, ldo_codes=0) -> Fp8LinearFusion:
    f = Fp8LinearFusion()
    f.prologue, f.norm_weight_dtype, f.norm_weight = prologue, norm_weight_dtype, ptr(norm_weight)
    f.norm_weight_offset, f.norm_epsilon = norm_weight_offset, norm_epsilon
    f.a2, f.residual, f.w2, f.w2_scale, f.out2, f.n2, f.ldo2 = ptr(a2), ptr(residual), ptr(w2), w2_scale, ptr(out2), n2, ldo2
    f.epilogue = epilogue
    f.out_codes, f.out_codes_scale, f.ldo_codes = ptr(out_codes), out_codes_scale, ldo_codes
    return f


def fp8_linear_fused(desc: Fp8LinearDesc, fusion: Fp8LinearFusion, stream=None) -> None:
    check(lib().fth_b200_fp8_linear_fused(C.byref(desc), C.byref(fusion), stream or current_stream()), "fth_b200_fp8_linear_fused")


def int8_linear(desc: Int8LinearDesc, stream=None) -> None:
    check(lib().fth_b200_int8_linear(C.byref(desc), stream or current_stream()), "fth_b200_int8_linear")


def int8_conv2d(desc: Int8Conv2dDesc, stream=None) -> None:
    check(lib().fth_b200_int8_conv2d(C.byref(desc), stream or current_stream()), "fth_b200_int8_conv2d")


def cast(in_dtype, x, in_scale, out_dtype, out, out_scale, count, stream=None) -> None:
    check(lib().fth_b200_cast(C.c_int32(in_dtype), C.c_void_p(ptr(x)), C.c_float(in_scale), C.c_int32(out_dtype),
                              C.c_void_p(ptr(out)), C.c_float(out_scale), C.c_int64(count),
                              stream or current_stream()), "fth_b200_cast")


def quantize_linear(x_dtype, x, scales, zps, params, out, rows, channels, stream=None, inner=1) -> None:
    """x is [rows, channels, inner]; the parameters run along `channels` (inner = 1: the last axis)."""
    check(lib().fth_b200_quantize_linear_axis(C.c_int32(x_dtype), C.c_void_p(ptr(x)), C.c_void_p(ptr(scales)),
                                              C.c_void_p(ptr(zps)), C.c_int64(params), C.c_void_p(ptr(out)),
                                              C.c_int64(rows), C.c_int64(channels), C.c_int64(inner), stream or current_stream()),
          "fth_b200_quantize_linear_axis")


def dequantize_linear(x, scales, zps, params, out, to_dtype, rows, channels, stream=None, inner=1) -> None:
    check(lib().fth_b200_dequantize_linear_axis(C.c_void_p(ptr(x)), C.c_void_p(ptr(scales)), C.c_void_p(ptr(zps)),
                                                C.c_int64(params), C.c_void_p(ptr(out)), C.c_int32(to_dtype),
                                                C.c_int64(rows), C.c_int64(channels), C.c_int64(inner), stream or current_stream()),
          "fth_b200_dequantize_linear_axis")


def small_copy(dst, src, nbytes, stream=None) -> None:
    """A few KB between a page-locked host buffer and device memory, copied by the SMs on the stream."""
    check(lib().fth_b200_small_copy(C.c_void_p(ptr(dst)), C.c_void_p(ptr(src)), C.c_int64(nbytes), stream or current_stream()),
          "fth_b200_small_copy")


def int8_lookup(x, out, count, lut, stream=None) -> None:
    check(lib().fth_b200_int8_lookup(C.c_void_p(ptr(x)), C.c_void_p(ptr(out)), C.c_int64(count),
                                     C.c_void_p(ptr(lut)), stream or current_stream()), "fth_b200_int8_lookup")


def int8_relu_table(in_scale, in_zp, out_scale, out_zp):
    import numpy as np
    lut = np.empty(256, np.int8)
    check(lib().fth_b200_int8_relu_table(C.c_float(in_scale), C.c_int32(in_zp), C.c_float(out_scale),
                                         C.c_int32(out_zp), C.c_void_p(lut.ctypes.data)), "fth_b200_int8_relu_table")
    return lut


def qwen_rms_norm(x_dtype, x, weight_dtype, weight, weight_offset, epsilon, out_dtype, out, rows, hidden, stream=None) -> None:
    check(lib().fth_b200_qwen_rms_norm(C.c_int32(x_dtype), C.c_void_p(ptr(x)), C.c_int32(weight_dtype), C.c_void_p(ptr(weight)),
                                       C.c_float(weight_offset), C.c_float(epsilon), C.c_int32(out_dtype), C.c_void_p(ptr(out)),
                                       C.c_int64(rows), C.c_int64(hidden), stream or current_stream()), "fth_b200_qwen_rms_norm")


def binary(op, dtype, lhs, rhs, out, count, rhs_count=0, stream=None) -> None:
    check(lib().fth_b200_binary(C.c_int32(op), C.c_int32(dtype), C.c_void_p(ptr(lhs)), C.c_void_p(ptr(rhs)), C.c_void_p(ptr(out)),
                                C.c_int64(count), C.c_int64(rhs_count), stream or current_stream()), "fth_b200_binary")


def silu(dtype, x, out, count, stream=None) -> None:
    check(lib().fth_b200_silu(C.c_int32(dtype), C.c_void_p(ptr(x)), C.c_void_p(ptr(out)), C.c_int64(count),
                              stream or current_stream()), "fth_b200_silu")


def silu_mul(dtype, gate, up, out, count, stream=None) -> None:
    check(lib().fth_b200_silu_mul(C.c_int32(dtype), C.c_void_p(ptr(gate)), C.c_void_p(ptr(up)), C.c_void_p(ptr(out)), C.c_int64(count),
                                  stream or current_stream()), "fth_b200_silu_mul")


def device_status() -> int:
    return lib().fth_b200_device_status()


def linear_workspace(torch, desc):
    """Allocates and zero-fills the scratch a linear descriptor may use and attaches it; returns the tensor."""
    fn = lib().fth_b200_fp8_linear_workspace_bytes if isinstance(desc, Fp8LinearDesc) else lib().fth_b200_int8_linear_workspace_bytes
    fn.restype = C.c_size_t
    need = fn(C.byref(desc))
    if not need:
        return None
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    desc.workspace, desc.workspace_bytes = ws.data_ptr(), need
    return ws


class Plan:
    """Host-buffer plan (Prepare once, compute many): see fth_b200_plan_* in include/fth_b200.h."""

    def __init__(self, desc, keepalive=()):
        self._h = C.c_void_p()
        self._keep = keepalive
        if isinstance(desc, Fp8LinearDesc):
            fn = lib().fth_b200_plan_create_fp8_linear
        elif isinstance(desc, Int8LinearDesc):
            fn = lib().fth_b200_plan_create_int8_linear
        else:
            fn = lib().fth_b200_plan_create_int8_conv2d
        check(fn(C.byref(desc), C.byref(self._h)), "fth_b200_plan_create")

    @property
    def input_bytes(self) -> int:
        return lib().fth_b200_plan_input_bytes(self._h)

    @property
    def output_bytes(self) -> int:
        return lib().fth_b200_plan_output_bytes(self._h)

    def run(self, host_in, host_out, stream=None) -> None:
        check(lib().fth_b200_plan_run(self._h, C.c_void_p(ptr(host_in)), C.c_void_p(ptr(host_out)),
                                      stream or current_stream()), "fth_b200_plan_run")

    def launch(self, device_in, device_out, stream=None) -> None:
        check(lib().fth_b200_plan_launch(self._h, C.c_void_p(ptr(device_in)), C.c_void_p(ptr(device_out)),
                                         stream or current_stream()), "fth_b200_plan_launch")

    def close(self) -> None:
        if self._h:
            lib().fth_b200_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
