"""Seeded input generators and comparison helpers shared by the tests.

Inputs follow the value distributions of the five benchmark configurations: N(0,1) activations and
N(0,0.02) weights quantised to FP8 with an absmax per-tensor scale (or the exporter's power-of-two rule),
uniform int8 activations/weights with per-output-channel scales in [1e-3, 1e-2]."""
from __future__ import annotations

import numpy as np

import oracle as O

FP8_MAX = {O.E4M3: 448.0, O.E5M2: 57344.0}


def fp8_scale(absmax: float, dtype: int, pow2: bool) -> np.float32:
    s = absmax / FP8_MAX[dtype]
    if pow2:  # exporter rule: 2^ceil(log2(absmax / max))
        s = 2.0 ** np.ceil(np.log2(s))
    return np.float32(s)


def code_index(codes: np.ndarray) -> np.ndarray:
    """Signed, monotone position of each FP8 code on the number line (distance 1 = adjacent codes)."""
    c = codes.astype(np.int32)
    return np.where(c & 0x80, -(c & 0x7F), c & 0x7F)


def fp8_code_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    return np.abs(code_index(a) - code_index(b))


def make_fp8_linear(dtype, m, k, n, seed, *, trans_b=False, pow2=False, bias_mode=0, out_headroom=1.0):
    rng = np.random.default_rng(seed)
    af = rng.standard_normal((m, k)).astype(np.float32)
    wf = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    sa = fp8_scale(float(np.abs(af).max()), dtype, pow2)
    sw = fp8_scale(float(np.abs(wf).max()), dtype, pow2)
    a = O.fp8_encode(dtype, af / sa)
    w = O.fp8_encode(dtype, wf / sw)
    ref = (O.fp8_decode(dtype, a).astype(np.float64) * float(sa)) @ (O.fp8_decode(dtype, w).astype(np.float64) * float(sw))
    bias = None
    sb = np.float32(1.0)
    if bias_mode:
        bf = rng.standard_normal((n,) if bias_mode == 1 else (m, n)).astype(np.float32) * 0.5
        sb = fp8_scale(float(np.abs(bf).max()), dtype, pow2)
        bias = O.fp8_encode(dtype, bf / sb)
        ref = ref + O.fp8_decode(dtype, bias).astype(np.float64) * float(sb)
    so = fp8_scale(float(np.abs(ref).max()) * out_headroom, dtype, pow2)
    if trans_b:
        w = np.ascontiguousarray(w.T)
    return dict(a=a, w=w, bias=bias, sa=float(sa), sw=float(sw), sb=float(sb), so=float(so))


def make_int8_linear(m, k, n, seed, *, trans_b=False, per_channel=True, zero_points=False, bias_mode=0,
                     saturate=0.02):
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w = rng.integers(-127, 128, (k, n)).astype(np.int8)
    sa = np.float32(0.02)
    ws = rng.uniform(1e-3, 1e-2, n if per_channel else 1).astype(np.float32)
    a_zp = int(rng.integers(-8, 9)) if zero_points else 0
    w_zps = rng.integers(-8, 9, n if per_channel else 1).astype(np.int32) if zero_points else None
    out_zp = int(rng.integers(-10, 11)) if zero_points else 0
    bias = None
    if bias_mode:
        bias = rng.integers(-2 ** 15, 2 ** 15, (n,) if bias_mode == 1 else (m, n)).astype(np.int32)
    # output scale such that roughly `saturate` of the outputs clip
    sigma = 73.3 ** 2 * np.sqrt(k) * float(sa) * float(ws.mean())
    z = {0.02: 2.33, 0.05: 1.96, 0.0: 6.0}.get(saturate, 2.33)
    so = np.float32(max(z * sigma / 127.0, 1e-6))
    if trans_b:
        w = np.ascontiguousarray(w.T)
    return dict(a=a, w=w, bias=bias, sa=float(sa), a_zp=a_zp, ws=ws, w_zps=w_zps, so=float(so), out_zp=out_zp)


def make_int8_conv(batch, ic, ih, iw, oc, kh, kw, seed, *, per_channel=True, zero_points=False, bias=True):
    rng = np.random.default_rng(seed)
    x = rng.integers(-128, 128, (batch, ic, ih, iw)).astype(np.int8)
    w = rng.integers(-128, 128, (oc, ic, kh, kw)).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, oc if per_channel else 1).astype(np.float32)
    b = rng.integers(-2 ** 15, 2 ** 15, oc).astype(np.int32) if bias else None
    sx = np.float32(0.05)
    sigma = 74.0 ** 2 * np.sqrt(ic * kh * kw) * float(sx) * float(ws.mean())
    so = np.float32(2.33 * sigma / 127.0)
    x_zp = int(rng.integers(-5, 6)) if zero_points else 0
    w_zps = rng.integers(-5, 6, oc if per_channel else 1).astype(np.int32) if zero_points else None
    out_zp = int(rng.integers(-10, 11)) if zero_points else 0
    return dict(x=x, w=w, bias=b, sx=float(sx), x_zp=x_zp, ws=ws, w_zps=w_zps, so=float(so), out_zp=out_zp)
