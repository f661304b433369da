"""CPU: the C-ABI library loads without a GPU, exports every symbol include/fth_b200.h declares, and the
ctypes mirrors of its structs have the C compiler's layout.  No compute call is made here."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import pytest

import infer_b200 as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fth_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fth_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = B.lib()
    names = declared_functions()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/fth_b200.h but not exported"
    assert set(B.EXPORTS) <= set(names)
    assert lib.fth_b200_abi_version() == 5


def test_struct_layouts_match_the_c_compiler():
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "fth_b200.h"
#define P(T, F) printf(#T "." #F " %zu\n", offsetof(T, F))
int main(void) {
  printf("sizeof.fp8 %zu\nsizeof.int8 %zu\nsizeof.conv %zu\nsizeof.fusion %zu\n", sizeof(fth_b200_fp8_linear_desc), sizeof(fth_b200_int8_linear_desc), sizeof(fth_b200_int8_conv2d_desc), sizeof(fth_b200_fp8_linear_fusion));
  P(fth_b200_fp8_linear_fusion, norm_weight); P(fth_b200_fp8_linear_fusion, norm_epsilon); P(fth_b200_fp8_linear_fusion, w2_scale); P(fth_b200_fp8_linear_fusion, ldo2); P(fth_b200_fp8_linear_fusion, epilogue); P(fth_b200_fp8_linear_fusion, out_codes); P(fth_b200_fp8_linear_fusion, ldo_codes);
  P(fth_b200_fp8_linear_desc, a); P(fth_b200_fp8_linear_desc, ldo); P(fth_b200_fp8_linear_desc, w_channel_scales);
  P(fth_b200_fp8_linear_desc, workspace); P(fth_b200_fp8_linear_desc, variant); P(fth_b200_fp8_linear_desc, gather_out);
  P(fth_b200_fp8_linear_desc, gather_world); P(fth_b200_fp8_linear_desc, gather_flags); P(fth_b200_int8_linear_desc, gather_flags);
  P(fth_b200_fp8_linear_desc, gather_multicast_out); P(fth_b200_int8_linear_desc, gather_multicast_out);
  P(fth_b200_int8_linear_desc, a); P(fth_b200_int8_linear_desc, w_scales); P(fth_b200_int8_linear_desc, bias_max_abs);
  P(fth_b200_int8_linear_desc, workspace); P(fth_b200_int8_linear_desc, variant);
  P(fth_b200_int8_conv2d_desc, x); P(fth_b200_int8_conv2d_desc, relu_lut); P(fth_b200_int8_conv2d_desc, workspace_bytes);
  P(fth_b200_int8_conv2d_desc, variant); P(fth_b200_int8_conv2d_desc, packed_w);
  return 0; }
'''
    with tempfile.TemporaryDirectory() as tmp:
        c = os.path.join(tmp, "layout.c")
        open(c, "w").write(src)
        exe = os.path.join(tmp, "layout")
        subprocess.check_call(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        got = dict(line.rsplit(" ", 1) for line in subprocess.check_output([exe], text=True).strip().splitlines())
    py = {"fth_b200_fp8_linear_desc": B.Fp8LinearDesc, "fth_b200_int8_linear_desc": B.Int8LinearDesc,
          "fth_b200_int8_conv2d_desc": B.Int8Conv2dDesc, "fth_b200_fp8_linear_fusion": B.Fp8LinearFusion}
    assert int(got["sizeof.fusion"]) == C.sizeof(B.Fp8LinearFusion)
    assert int(got["sizeof.fp8"]) == C.sizeof(B.Fp8LinearDesc)
    assert int(got["sizeof.int8"]) == C.sizeof(B.Int8LinearDesc)
    assert int(got["sizeof.conv"]) == C.sizeof(B.Int8Conv2dDesc)
    for key, value in got.items():
        if key.startswith("sizeof"):
            continue
        struct, field = key.split(".")
        assert getattr(py[struct], field).offset == int(value), key


def test_validation_needs_no_gpu():
    """Contract checks run on the host before any launch."""
    d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=1, k=64, n=64, a=16, w=16, out=16, a_scale=0.0, w_scale=1.0, out_scale=1.0)
    assert B.lib().fth_b200_fp8_linear_supported(C.byref(d)) == B.ERR_INVALID
    d = B.int8_linear_desc(op=B.OP_MATMUL, m=1, k=300000, n=64, a=16, w=16, out=16, a_scale=1.0, a_zp=0, w_scales=16, w_zps=None,
                           w_params=64, out_scale=1.0, out_zp=0)
    assert B.lib().fth_b200_int8_linear_supported(C.byref(d)) == B.ERR_OVERFLOW
    lut = B.int8_relu_table(0.5, 0, 0.5, 0)
    assert lut[128 + 5] == 5 and lut[128 - 5] == 0
    # K beyond 2^31 is rejected before the worst-case product could wrap
    d = B.int8_linear_desc(op=B.OP_MATMUL, m=1, k=1 << 40, n=64, a=16, w=16, out=16, a_scale=1.0, a_zp=0, w_scales=16, w_zps=None,
                           w_params=64, out_scale=1.0, out_zp=0)
    assert B.lib().fth_b200_int8_linear_supported(C.byref(d)) == B.ERR_OVERFLOW


def test_conv_plan_rejects_degenerate_geometry_before_using_it():
    """A stride, dilation or kernel size of zero returns ERR_INVALID: it must never reach a division or an allocation."""
    import numpy as np
    w = np.zeros((8, 8, 3, 3), np.int8)
    ws = np.ones(8, np.float32)
    for bad in (dict(stride=(0, 1)), dict(stride=(1, 0)), dict(dil=(0, 1)), dict(kh=0), dict(batch=0), dict(group=3)):
        kw = dict(batch=1, ic=8, ih=16, iw=16, oc=8, kh=3, kw=3, x=None, w=w, out=None, x_scale=1.0, x_zp=0, w_scales=ws, w_zps=None,
                  w_params=8, out_scale=1.0, out_zp=0)
        kw.update(bad)
        d = B.int8_conv2d_desc(**kw)
        plan = C.c_void_p()
        assert B.lib().fth_b200_plan_create_int8_conv2d(C.byref(d), C.byref(plan)) == B.ERR_INVALID, bad
        assert not plan.value


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(B, "_lib", None)
    monkeypatch.setattr(B, "LIB_PATH", "/nonexistent/libfth_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or library fallback"):
        B.lib()
