"""TEST INFRASTRUCTURE — ctypes bindings for the two CPU checkers.

* ``port``  — ``oracle/libfeather_oracle.so``: this repo's plain-C restatement of the reference's
  portable Common kernels (``oracle/feather_oracle.c``).
* ``ref``   — ``oracle/_ref/libfeather_ref.so``: the unmodified reference CPU library behind
  ``oracle/ref_shim.cc`` (Common = canonical oracle, X86 = timed CPU baseline).  Present only where it
  was built (``make -C oracle ref`` next to a reference checkout); ``have_ref()`` says whether it is.

Nothing in the shipped package imports this module.  Only ``tests/``, the smoke check and the
CPU-baseline leg of ``bench.py`` do, and only as the checker / the CPU number reported beside the GPU one.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "libfeather_oracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libfeather_ref.so")

INT8, FP16, FP32, INT32, BF16, E4M3, E5M2 = 1, 3, 4, 5, 11, 12, 13  # feather::DataType values
OP_FC, OP_MATMUL, OP_GEMM = 0, 1, 2
COMMON, X86 = 0, 1

_port = None
_ref = None


def build_port() -> str:
    """Compile the C restatement if it is missing or older than its source."""
    src = os.path.join(_HERE, "feather_oracle.c")
    if not os.path.exists(PORT_PATH) or os.path.getmtime(PORT_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return PORT_PATH


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _arr(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def port():
    global _port
    if _port is None:
        lib = C.CDLL(build_port())
        lib.fo_fp8_encode.restype = C.c_uint8
        lib.fo_fp8_encode.argtypes = [C.c_int, C.c_float]
        lib.fo_fp8_decode.restype = C.c_float
        lib.fo_fp8_decode.argtypes = [C.c_int, C.c_uint8]
        lib.fo_bf16_encode.restype = C.c_uint16
        lib.fo_bf16_encode.argtypes = [C.c_float]
        lib.fo_bf16_encode_dq.restype = C.c_uint16
        lib.fo_bf16_encode_dq.argtypes = [C.c_float]
        lib.fo_quantize_int8_value.restype = C.c_int8
        lib.fo_quantize_int8_value.argtypes = [C.c_float, C.c_float, C.c_int32]
        _port = lib
    return _port


def have_ref() -> bool:
    return os.path.exists(REF_PATH)


def ref():
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_PATH)
        lib.ref_fp8_encode.restype = C.c_uint8
        lib.ref_fp8_encode.argtypes = [C.c_int, C.c_float]
        lib.ref_fp8_decode.restype = C.c_float
        lib.ref_fp8_decode.argtypes = [C.c_int, C.c_uint8]
        lib.ref_float_to_bf16.restype = C.c_uint16
        lib.ref_float_to_bf16.argtypes = [C.c_float]
        lib.ref_quantize_int8_value.restype = C.c_int8
        lib.ref_quantize_int8_value.argtypes = [C.c_float, C.c_float, C.c_int32]
        for name in ("ref_fp8_linear_create", "ref_int8_linear_create", "ref_int8_conv2d_create",
                     "ref_int8_relu_create", "ref_cast_create", "ref_quantize_linear_create",
                     "ref_dequantize_linear_create"):
            getattr(lib, name).restype = C.c_void_p
        lib.ref_kernel_time_compute.restype = C.c_double
        lib.ref_kernel_output_bytes.restype = C.c_int64
        _ref = lib
    return _ref


# ------------------------------------------------------------------------------------------------
# FP8 codec
# ------------------------------------------------------------------------------------------------
def fp8_encode(dtype: int, values, impl: str = "port") -> np.ndarray:
    v = _arr(values, np.float32).ravel()
    out = np.empty(v.size, np.uint8)
    lib, fn = (port(), "fo_fp8_encode_array") if impl == "port" else (ref(), "ref_fp8_encode_array")
    getattr(lib, fn)(C.c_int(dtype), _p(v), _p(out), C.c_int64(v.size))
    return out.reshape(np.shape(values))


def fp8_decode(dtype: int, bits, impl: str = "port") -> np.ndarray:
    b = _arr(bits, np.uint8).ravel()
    out = np.empty(b.size, np.float32)
    lib, fn = (port(), "fo_fp8_decode_array") if impl == "port" else (ref(), "ref_fp8_decode_array")
    getattr(lib, fn)(C.c_int(dtype), _p(b), _p(out), C.c_int64(b.size))
    return out.reshape(np.shape(bits))


# ------------------------------------------------------------------------------------------------
# reference-handle helper
# ------------------------------------------------------------------------------------------------
class RefKernel:
    """One reference KernelBase instance with its tensors (see oracle/ref_shim.cc)."""

    def __init__(self, handle, out_dtype, out_shape):
        if not handle:
            raise RuntimeError("reference dispatcher returned no kernel")
        self.h = C.c_void_p(handle)
        self.out_dtype = out_dtype
        self.out_shape = out_shape

    def device(self) -> int:
        return ref().ref_kernel_device(self.h)

    def prepare(self) -> int:
        return ref().ref_kernel_prepare(self.h)

    def compute(self) -> int:
        return ref().ref_kernel_compute(self.h)

    def output(self) -> np.ndarray:
        out = np.empty(self.out_shape, self.out_dtype)
        rc = ref().ref_kernel_read_output(self.h, _p(out), C.c_int64(out.nbytes))
        if rc != 0:
            raise RuntimeError("reference output read failed")
        return out

    def time_compute(self, repeats: int) -> float:
        status = C.c_int(0)
        s = ref().ref_kernel_time_compute(self.h, C.c_int(repeats), C.byref(status))
        if status.value != 0:
            raise RuntimeError("reference compute() failed")
        return s

    def run(self) -> np.ndarray:
        if self.prepare() != 0:
            raise RuntimeError("reference Prepare() failed")
        rc = self.compute()
        if rc != 0:
            raise RuntimeError(f"reference compute() returned {rc}")
        return self.output()

    def __del__(self):
        try:
            ref().ref_kernel_destroy(self.h)
        except Exception:
            pass


# ------------------------------------------------------------------------------------------------
# FP8 linear
# ------------------------------------------------------------------------------------------------
def fp8_linear(op, dtype, a, a_scale, w, w_scale, out_scale, *, bias=None, bias_scale=1.0, trans_b=False,
               alpha=1.0, beta=1.0, impl="port", device=COMMON, immutable=True, return_kernel=False):
    a = _arr(a, np.uint8)
    w = _arr(w, np.uint8)
    m, k = a.shape
    n = w.shape[0] if trans_b else w.shape[1]
    bias_mode = 0 if bias is None else (1 if bias.ndim == 1 else 2)
    bias = _arr(bias, np.uint8)
    if impl == "port":
        out = np.empty((m, n), np.uint8)
        rc = port().fo_fp8_linear(C.c_int(op), C.c_int(dtype), _p(a), C.c_float(a_scale), _p(w), C.c_float(w_scale),
                                  _p(bias), C.c_float(bias_scale), C.c_int(bias_mode), _p(out), C.c_float(out_scale),
                                  C.c_int64(m), C.c_int64(k), C.c_int64(n), C.c_int(int(trans_b)), C.c_float(alpha),
                                  C.c_float(beta))
        if rc != 0:
            raise RuntimeError("fo_fp8_linear failed")
        return out
    h = ref().ref_fp8_linear_create(C.c_int(device), C.c_int(op), C.c_int(dtype), _p(a), C.c_float(a_scale), _p(w),
                                    C.c_float(w_scale), _p(bias), C.c_float(bias_scale), C.c_int(bias_mode),
                                    C.c_float(out_scale), C.c_int64(m), C.c_int64(k), C.c_int64(n),
                                    C.c_int(int(trans_b)), C.c_float(alpha), C.c_float(beta), C.c_int(int(immutable)))
    kern = RefKernel(h, np.uint8, (m, n))
    return kern if return_kernel else kern.run()


def fp8_linear_per_channel(op, dtype, a, a_scale, w, w_scales, out_scale, *, bias=None, bias_scale=1.0, trans_b=False,
                           alpha=1.0, beta=1.0, impl="port", device=COMMON):
    """FP8 linear whose weight carries one scale per output channel — a quantisation the reference's FP8 linear
    kernels cannot express (they read the tensor's scalar scale only, include/core/tensor.h:105; per-tensor rule in
    include/util/types.h:96-101), although its tensor metadata and the .fth files can hold the vector
    (src/model/model_io.cc:228-246).  Defined column by column: output
    channel n is what the reference's kernel gives for that column alone with w_scale = w_scales[n].  Channels that
    share a scale are computed in one call."""
    a = _arr(a, np.uint8)
    w = _arr(w, np.uint8)
    w_scales = _arr(w_scales, np.float32).reshape(-1)
    n = w.shape[0] if trans_b else w.shape[1]
    assert w_scales.size == n
    out = np.empty((a.shape[0], n), np.uint8)
    for scale in np.unique(w_scales):
        cols = np.nonzero(w_scales == scale)[0]
        w_part = np.ascontiguousarray(w[cols] if trans_b else w[:, cols])
        b_part = None if bias is None else np.ascontiguousarray(bias[cols] if bias.ndim == 1 else bias[:, cols])
        out[:, cols] = fp8_linear(op, dtype, a, a_scale, w_part, float(scale), out_scale, bias=b_part, bias_scale=bias_scale,
                                  trans_b=trans_b, alpha=alpha, beta=beta, impl=impl, device=device)
    return out


# ------------------------------------------------------------------------------------------------
# INT8 linear
# ------------------------------------------------------------------------------------------------
def int8_linear(op, a, a_scale, a_zp, w, w_scales, w_zps, out_scale, out_zp, *, bias=None, trans_b=False,
                alpha=1.0, beta=1.0, impl="port", device=COMMON, return_kernel=False, check=True):
    a = _arr(a, np.int8)
    w = _arr(w, np.int8)
    m, k = a.shape
    n = w.shape[0] if trans_b else w.shape[1]
    w_scales = np.atleast_1d(_arr(w_scales, np.float32))
    w_channels = 0 if w_scales.size == 1 else n
    w_zps = None if w_zps is None else np.atleast_1d(_arr(w_zps, np.int32))
    if w_zps is not None and w_channels and w_zps.size == 1:
        w_zps = np.full(n, w_zps[0], np.int32)
    bias_mode = 0 if bias is None else (1 if bias.ndim == 1 else 2)
    bias = _arr(bias, np.int32)
    if impl == "port":
        out = np.empty((m, n), np.int8)
        rc = port().fo_int8_linear(C.c_int(op), _p(a), C.c_float(a_scale), C.c_int32(a_zp), _p(w), _p(w_scales),
                                   _p(w_zps), C.c_int64(w_channels), _p(bias), C.c_int(bias_mode), _p(out),
                                   C.c_float(out_scale), C.c_int32(out_zp), C.c_int64(m), C.c_int64(k), C.c_int64(n),
                                   C.c_int(int(trans_b)), C.c_float(alpha), C.c_float(beta))
        if rc != 0 and check:
            raise RuntimeError("fo_int8_linear failed")
        return out if check else (rc, out)
    h = ref().ref_int8_linear_create(C.c_int(device), C.c_int(op), _p(a), C.c_float(a_scale), C.c_int32(a_zp), _p(w),
                                     _p(w_scales), _p(w_zps), C.c_int64(w_channels), _p(bias), C.c_int(bias_mode),
                                     C.c_float(out_scale), C.c_int32(out_zp), C.c_int64(m), C.c_int64(k),
                                     C.c_int64(n), C.c_int(int(trans_b)), C.c_float(alpha), C.c_float(beta))
    kern = RefKernel(h, np.int8, (m, n))
    if return_kernel:
        return kern
    if check:
        return kern.run()
    kern.prepare()
    rc = kern.compute()
    return rc, kern.output()


# ------------------------------------------------------------------------------------------------
# INT8 conv (NCHW / OIHW) and ReLU
# ------------------------------------------------------------------------------------------------
def conv_out_hw(ih, iw, kh, kw, stride, pad, dil):
    oh = (ih + 2 * pad[0] - dil[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (iw + 2 * pad[1] - dil[1] * (kw - 1) - 1) // stride[1] + 1
    return oh, ow


def int8_conv2d(x, x_scale, x_zp, w, w_scales, w_zps, bias, out_scale, out_zp, *, stride=(1, 1), pad=(1, 1),
                dil=(1, 1), group=1, impl="port", device=COMMON, return_kernel=False):
    x = _arr(x, np.int8)
    w = _arr(w, np.int8)
    b, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    oh, ow = conv_out_hw(ih, iw, kh, kw, stride, pad, dil)
    w_scales = np.atleast_1d(_arr(w_scales, np.float32))
    w_channels = 0 if w_scales.size == 1 else oc
    w_zps = None if w_zps is None else np.atleast_1d(_arr(w_zps, np.int32))
    bias = _arr(bias, np.int32)
    if impl == "port":
        out = np.empty((b, oc, oh, ow), np.int8)
        rc = port().fo_int8_conv2d(_p(x), C.c_float(x_scale), C.c_int32(x_zp), _p(w), _p(w_scales), _p(w_zps),
                                   C.c_int64(w_channels), _p(bias), _p(out), C.c_float(out_scale), C.c_int32(out_zp),
                                   C.c_int64(b), C.c_int64(ic), C.c_int64(ih), C.c_int64(iw), C.c_int64(oc),
                                   C.c_int64(kh), C.c_int64(kw), C.c_int32(stride[0]), C.c_int32(stride[1]),
                                   C.c_int32(pad[0]), C.c_int32(pad[1]), C.c_int32(dil[0]), C.c_int32(dil[1]),
                                   C.c_int32(group))
        if rc != 0:
            raise RuntimeError("fo_int8_conv2d failed")
        return out
    h = ref().ref_int8_conv2d_create(C.c_int(device), _p(x), C.c_float(x_scale), C.c_int32(x_zp), _p(w), _p(w_scales),
                                     _p(w_zps), C.c_int64(w_channels), _p(bias), C.c_float(out_scale),
                                     C.c_int32(out_zp), C.c_int64(b), C.c_int64(ic), C.c_int64(ih), C.c_int64(iw),
                                     C.c_int64(oc), C.c_int64(kh), C.c_int64(kw), C.c_int32(stride[0]),
                                     C.c_int32(stride[1]), C.c_int32(pad[0]), C.c_int32(pad[1]), C.c_int32(dil[0]),
                                     C.c_int32(dil[1]), C.c_int32(group))
    kern = RefKernel(h, np.int8, (b, oc, oh, ow))
    return kern if return_kernel else kern.run()


def int8_relu(x, in_scale, in_zp, out_scale, out_zp, *, impl="port", device=COMMON):
    x = _arr(x, np.int8)
    if impl == "port":
        out = np.empty_like(x)
        port().fo_int8_relu(_p(x), _p(out), C.c_int64(x.size), C.c_float(in_scale), C.c_int32(in_zp),
                            C.c_float(out_scale), C.c_int32(out_zp))
        return out
    h = ref().ref_int8_relu_create(C.c_int(device), _p(x), C.c_float(in_scale), C.c_int32(in_zp),
                                   C.c_float(out_scale), C.c_int32(out_zp), C.c_int64(x.size))
    return RefKernel(h, np.int8, x.shape).run()


def int8_relu_lut(in_scale, in_zp, out_scale, out_zp) -> np.ndarray:
    lut = np.empty(256, np.int8)
    port().fo_int8_relu_lut(C.c_float(in_scale), C.c_int32(in_zp), C.c_float(out_scale), C.c_int32(out_zp), _p(lut))
    return lut


# ------------------------------------------------------------------------------------------------
# QuantizeLinear / DequantizeLinear / Cast
# ------------------------------------------------------------------------------------------------
_NP = {FP32: np.float32, FP16: np.uint16, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8, INT8: np.int8}


def quantize_linear(x_dtype, x, scales, zps, *, impl="port"):
    x = _arr(x, _NP[x_dtype])
    rows, channels = x.shape
    scales = np.atleast_1d(_arr(scales, np.float32))
    zps = np.atleast_1d(_arr(zps, np.int32))
    if impl == "port":
        out = np.empty((rows, channels), np.int8)
        rc = port().fo_quantize_linear(C.c_int(x_dtype), _p(x), _p(scales), _p(zps), C.c_int64(scales.size), _p(out),
                                       C.c_int64(rows), C.c_int64(channels))
        if rc != 0:
            raise RuntimeError("fo_quantize_linear failed")
        return out
    h = ref().ref_quantize_linear_create(C.c_int(x_dtype), _p(x), _p(scales), _p(zps), C.c_int64(scales.size),
                                         C.c_int64(rows), C.c_int64(channels))
    return RefKernel(h, np.int8, (rows, channels)).run()


def dequantize_linear(x, scales, zps, to_dtype, *, impl="port"):
    x = _arr(x, np.int8)
    rows, channels = x.shape
    scales = np.atleast_1d(_arr(scales, np.float32))
    zps = np.atleast_1d(_arr(zps, np.int32))
    if impl == "port":
        out = np.empty((rows, channels), _NP[to_dtype])
        rc = port().fo_dequantize_linear(_p(x), _p(scales), _p(zps), C.c_int64(scales.size), _p(out),
                                         C.c_int(to_dtype), C.c_int64(rows), C.c_int64(channels))
        if rc != 0:
            raise RuntimeError("fo_dequantize_linear failed")
        return out
    h = ref().ref_dequantize_linear_create(_p(x), _p(scales), _p(zps), C.c_int64(scales.size), C.c_int64(rows),
                                           C.c_int64(channels), C.c_int(to_dtype))
    return RefKernel(h, _NP[to_dtype], (rows, channels)).run()


def cast(in_dtype, x, in_scale, out_dtype, out_scale, *, impl="port", device=COMMON):
    x = _arr(x, _NP[in_dtype]).ravel()
    if impl == "port":
        out = np.empty(x.size, _NP[out_dtype])
        port().fo_cast(C.c_int(in_dtype), _p(x), C.c_float(in_scale), C.c_int(out_dtype), _p(out),
                       C.c_float(out_scale), C.c_int64(x.size))
        return out
    h = ref().ref_cast_create(C.c_int(device), C.c_int(in_dtype), _p(x), C.c_float(in_scale), C.c_int(out_dtype),
                              C.c_float(out_scale), C.c_int64(x.size))
    return RefKernel(h, _NP[out_dtype], (x.size,)).run()


# ------------------------------------------------------------------------------------------------
# QwenRmsNorm / Add / Mul / SiLU (the operators between the projections of a decoder block)
# ------------------------------------------------------------------------------------------------
def qwen_rms_norm(x_dtype, x, w_dtype, weight, weight_offset, epsilon, out_dtype, *, impl="port", device=COMMON):
    x = _arr(x, _NP[x_dtype])
    weight = _arr(weight, _NP[w_dtype])
    rows, hidden = x.shape
    if impl == "port":
        out = np.empty((rows, hidden), _NP[out_dtype])
        rc = port().fo_qwen_rms_norm(C.c_int(x_dtype), _p(x), C.c_int(w_dtype), _p(weight), C.c_float(weight_offset),
                                     C.c_float(epsilon), C.c_int(out_dtype), _p(out), C.c_int64(rows), C.c_int64(hidden))
        if rc != 0:
            raise RuntimeError("fo_qwen_rms_norm failed")
        return out
    ref().ref_qwen_rms_norm_create.restype = C.c_void_p
    h = ref().ref_qwen_rms_norm_create(C.c_int(device), C.c_int(x_dtype), _p(x), C.c_int(w_dtype), _p(weight), C.c_float(weight_offset),
                                       C.c_float(epsilon), C.c_int(out_dtype), C.c_int64(rows), C.c_int64(hidden))
    return RefKernel(h, _NP[out_dtype], (rows, hidden)).run()


def binary(op, dtype, lhs, rhs, *, impl="port", device=COMMON):
    """op 0 = Add, 1 = Mul; lhs [rows, cols]; rhs the same shape or one row [cols]."""
    lhs = _arr(lhs, _NP[dtype])
    rhs = _arr(rhs, _NP[dtype])
    rows, cols = lhs.shape
    if impl == "port":
        out = np.empty((rows, cols), _NP[dtype])
        rc = port().fo_binary(C.c_int(op), C.c_int(dtype), _p(lhs), _p(rhs), _p(out), C.c_int64(lhs.size), C.c_int64(rhs.size))
        if rc != 0:
            raise RuntimeError("fo_binary failed")
        return out
    ref().ref_binary_create.restype = C.c_void_p
    h = ref().ref_binary_create(C.c_int(device), C.c_int(op), C.c_int(dtype), _p(lhs), _p(rhs), C.c_int64(rows), C.c_int64(cols),
                                C.c_int64(1 if rhs.ndim == 1 else rows))
    return RefKernel(h, _NP[dtype], (rows, cols)).run()


def silu(dtype, x, *, impl="port", device=COMMON):
    x = _arr(x, _NP[dtype])
    if impl == "port":
        out = np.empty(x.shape, _NP[dtype])
        port().fo_silu(C.c_int(dtype), _p(x), _p(out), C.c_int64(x.size))
        return out
    ref().ref_silu_create.restype = C.c_void_p
    h = ref().ref_silu_create(C.c_int(device), C.c_int(dtype), _p(x), C.c_int64(x.size))
    return RefKernel(h, _NP[dtype], x.shape).run()


def qwen_gemm_argmax(dtype, a, a_scale, b, b_scale, output_scale, *, device=X86):
    """The reference's fused FP8 lm-head projection + greedy selection (x86 only: src/kernel/x86/linear_fp8.cc:733-1004).
    a [1, K] codes, b [N, K] codes; returns the selected row of b."""
    a = _arr(a, np.uint8)
    b = _arr(b, np.uint8)
    n, k = b.shape
    ref().ref_qwen_gemm_argmax_create.restype = C.c_void_p
    h = ref().ref_qwen_gemm_argmax_create(C.c_int(device), C.c_int(dtype), _p(a), C.c_float(a_scale), _p(b), C.c_float(b_scale),
                                          C.c_float(output_scale), C.c_int64(k), C.c_int64(n))
    return int(RefKernel(h, np.int64, (1,)).run()[0])
