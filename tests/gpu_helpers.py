"""Runs the C ABI on device tensors built from numpy inputs (used by the -m gpu tests)."""
from __future__ import annotations

import numpy as np

import infer_b200 as B


def _skip_if_declined(fn, desc, variant):
    """A forced kernel family may decline a shape (ERR_UNSUPPORTED); the AUTO split never does."""
    import ctypes
    import pytest
    if variant != B.VARIANT_AUTO and fn(ctypes.byref(desc)) == B.ERR_UNSUPPORTED:
        pytest.skip("this kernel family declines the shape")


def dev(torch, arr):
    return None if arr is None else torch.from_numpy(np.ascontiguousarray(arr)).cuda()


_OUT_NP = {0: np.uint8, B.E4M3: np.uint8, B.E5M2: np.uint8, B.BF16: np.uint16, B.FP32: np.float32, B.INT8: np.int8}


def run_fp8_linear(torch, dtype, op, case, *, trans_b=False, variant=B.VARIANT_AUTO, alpha=1.0, beta=1.0,
                   a_dtype=0, out_dtype=0, a_raw=None, w_channel_scales=None, ldo=0, canary=True, workspace=True):
    a_np = case["a"] if a_raw is None else a_raw
    m, k = case["a"].shape
    n = case["w"].shape[0] if trans_b else case["w"].shape[1]
    a, w, bias = dev(torch, a_np), dev(torch, case["w"]), dev(torch, case["bias"])
    wcs = dev(torch, w_channel_scales)
    np_out = _OUT_NP[out_dtype]
    width = ldo or n
    # canary rows around the output catch out-of-bounds writes
    torch_dt = {np.uint8: torch.uint8, np.uint16: torch.int16, np.float32: torch.float32}[np_out]
    fill = 0x5A if np_out is np.uint8 else (0x5A5A if np_out is np.uint16 else 12345.0)
    buf = torch.full((m + 2, width), fill, dtype=torch_dt, device="cuda")
    out = buf[1:m + 1]
    bias_mode = 0 if case["bias"] is None else (1 if case["bias"].ndim == 1 else 2)
    d = B.fp8_linear_desc(dtype=dtype, op=op, m=m, k=k, n=n, a=a, w=w, out=out, a_scale=case["sa"],
                          w_scale=case["sw"], out_scale=case["so"], trans_b=trans_b, bias=bias,
                          bias_mode=bias_mode, bias_scale=case["sb"], alpha=alpha, beta=beta, a_dtype=a_dtype,
                          out_dtype=out_dtype, ldo=ldo, w_channel_scales=wcs, variant=variant)
    ws_keep = B.linear_workspace(torch, d) if workspace else None
    _skip_if_declined(B.lib().fth_b200_fp8_linear_supported, d, variant)
    B.fp8_linear(d)
    torch.cuda.synchronize()
    host = buf.cpu().numpy().view(np_out)
    if m <= 32 and variant in (B.VARIANT_AUTO, B.VARIANT_TCGEN05):
        # decode-sized problems may prefetch weights the caller declares static: same bytes either way
        buf.fill_(fill)
        d.weights_static = 1
        B.fp8_linear(d)
        torch.cuda.synchronize()
        assert np.array_equal(buf.cpu().numpy().view(np.uint8), host.view(np.uint8)), "weights_static changed the result"
    if canary:
        ref_fill = np.full(1, fill).astype(host.dtype if np_out is not np.uint16 else np.int16).view(np_out)[0]
        assert (host[0] == ref_fill).all() and (host[-1] == ref_fill).all(), "write outside the output rows"
        if width > n:
            assert (host[1:m + 1, n:] == ref_fill).all(), "write outside the output columns"
    return host[1:m + 1, :n].copy()


def run_int8_linear(torch, op, case, *, trans_b=False, variant=B.VARIANT_AUTO, alpha=1.0, beta=1.0, a_dtype=0,
                    out_dtype=0, a_raw=None, workspace=True):
    a_np = case["a"] if a_raw is None else a_raw
    m, k = case["a"].shape
    n = case["w"].shape[0] if trans_b else case["w"].shape[1]
    a, w, bias = dev(torch, a_np), dev(torch, case["w"]), dev(torch, case["bias"])
    ws, wz = dev(torch, case["ws"]), dev(torch, case["w_zps"])
    np_out = np.float32 if out_dtype == B.FP32 else np.int8
    buf = torch.full((m + 2, n), 77, dtype=torch.float32 if out_dtype == B.FP32 else torch.int8, device="cuda")
    out = buf[1:m + 1]
    bias_mode = 0 if case["bias"] is None else (1 if case["bias"].ndim == 1 else 2)
    bias_max = 0 if case["bias"] is None else int(np.abs(case["bias"].astype(np.int64)).max())
    zmax = 0 if case["w_zps"] is None else int(np.abs(case["w_zps"]).max())
    d = B.int8_linear_desc(op=op, m=m, k=k, n=n, a=a, w=w, out=out, a_scale=case["sa"], a_zp=case["a_zp"],
                           w_scales=ws, w_zps=wz, w_params=case["ws"].size, out_scale=case["so"],
                           out_zp=case["out_zp"], trans_b=trans_b, bias=bias, bias_mode=bias_mode, alpha=alpha,
                           beta=beta, a_dtype=a_dtype, out_dtype=out_dtype, w_zp_max_abs=zmax,
                           bias_max_abs=bias_max, variant=variant)
    ws_keep = B.linear_workspace(torch, d) if workspace else None
    _skip_if_declined(B.lib().fth_b200_int8_linear_supported, d, variant)
    B.int8_linear(d)
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    if m <= 32 and variant in (B.VARIANT_AUTO, B.VARIANT_TCGEN05):
        buf.fill_(77)
        d.weights_static = 1
        B.int8_linear(d)
        torch.cuda.synchronize()
        assert np.array_equal(buf.cpu().numpy().view(np.uint8), host.view(np.uint8)), "weights_static changed the result"
    assert (host[0] == 77).all() and (host[-1] == 77).all(), "write outside the output rows"
    return host[1:m + 1].astype(np_out)


def run_int8_conv(torch, case, *, stride=(1, 1), pad=(1, 1), dil=(1, 1), group=1, relu_lut=None,
                  variant=B.VARIANT_AUTO):
    import oracle as O
    x, w = case["x"], case["w"]
    b, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    oh, ow = O.conv_out_hw(ih, iw, kh, kw, stride, pad, dil)
    xd, wd, bd = dev(torch, x), dev(torch, w), dev(torch, case["bias"])
    ws, wz = dev(torch, case["ws"]), dev(torch, case["w_zps"])
    lut = dev(torch, relu_lut)
    buf = torch.full((b * oc * oh * ow + 512,), 77, dtype=torch.int8, device="cuda")
    out = buf[256:256 + b * oc * oh * ow]
    bias_max = 0 if case["bias"] is None else int(np.abs(case["bias"].astype(np.int64)).max())
    zmax = 0 if case["w_zps"] is None else int(np.abs(case["w_zps"]).max())
    d = B.int8_conv2d_desc(batch=b, ic=ic, ih=ih, iw=iw, oc=oc, kh=kh, kw=kw, x=xd, w=wd, out=out,
                           x_scale=case["sx"], x_zp=case["x_zp"], w_scales=ws, w_zps=wz, w_params=case["ws"].size,
                           out_scale=case["so"], out_zp=case["out_zp"], bias=bd, stride=stride, pad=pad, dil=dil,
                           group=group, relu_lut=lut, w_zp_max_abs=zmax, bias_max_abs=bias_max, variant=variant)
    need = B.lib().fth_b200_int8_conv2d_workspace_bytes(__import__("ctypes").byref(d))
    wsb = None
    if need:
        wsb = torch.empty(need, dtype=torch.uint8, device="cuda")
        d.workspace, d.workspace_bytes = wsb.data_ptr(), need
    B.int8_conv2d(d)
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    assert (host[:256] == 77).all() and (host[-256:] == 77).all(), "write outside the output"
    return host[256:-256].reshape(b, oc, oh, ow).copy()
