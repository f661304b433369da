"""GPU: QwenRmsNorm / Add / Mul / SiLU / SiLU*up against the CPU oracle (the reference's Common kernels).

Add and Mul are bit-exact.  SiLU is compared code for code as well (the kernel evaluates exp in double and rounds once).
QwenRmsNorm reduces the squares in parallel, while the Common kernel adds them one after another in FP32 (a sum whose
own rounding error is a few parts in 10^6 at 1024 terms): BF16 outputs may sit one code from the oracle's, FP32 outputs
16 + hidden / 32 FP32 steps (the sequential sum's error grows with the row length; 6e-6 relative at 1024 elements) — the
reference's own x86 kernel is 29 steps from its Common kernel on the 1024-element fixture
(tests/test_oracle_decoder_ops.py)."""
import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests.golden import cases as G
from tests.gpu_helpers import dev

pytestmark = pytest.mark.gpu
NP = {B.FP32: np.float32, B.BF16: np.uint16, B.FP16: np.uint16}


def _rand(rng, shape, dtype, scale=1.0):
    x = (rng.standard_normal(shape) * scale).astype(np.float32)
    if dtype == B.FP32:
        return x
    if dtype == B.BF16:
        return G.to_bf16(x)
    return x.astype(np.float16).view(np.uint16)


def _steps(a, b):
    """Distance in codes between two arrays of BF16 / FP32 bit patterns (sign-magnitude aware)."""
    bits = 16 if a.dtype == np.uint16 else 32
    def lin(v):
        v = v.astype(np.int64)
        sign = v >> (bits - 1)
        mag = v & ((1 << (bits - 1)) - 1)
        return np.where(sign == 1, -mag, mag)
    return np.abs(lin(a) - lin(b))


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (16, 1024), (3, 3584), (2, 130), (5, 4096), (2, 5000), (1, 7)])
@pytest.mark.parametrize("x_dtype,w_dtype,out_dtype", [(B.BF16, B.BF16, B.BF16), (B.FP32, B.FP32, B.FP32), (B.BF16, B.FP32, B.FP32), (B.FP32, B.BF16, B.BF16)])
def test_qwen_rms_norm(cuda, rows, hidden, x_dtype, w_dtype, out_dtype):
    rng = np.random.default_rng(rows * 31 + hidden)
    x = _rand(rng, (rows, hidden), x_dtype, 3.0)
    w = _rand(rng, (hidden,), w_dtype, 0.1)
    want = O.qwen_rms_norm(x_dtype, x, w_dtype, w, 1.0, 1e-6, out_dtype)
    xd, wd = dev(cuda, x.view(np.int16) if x.dtype == np.uint16 else x), dev(cuda, w.view(np.int16) if w.dtype == np.uint16 else w)
    buf = cuda.full((rows + 2, hidden), 0x5A5A if out_dtype != B.FP32 else 12345.0, dtype=cuda.int16 if out_dtype != B.FP32 else cuda.float32, device="cuda")
    B.qwen_rms_norm(x_dtype, xd, w_dtype, wd, 1.0, 1e-6, out_dtype, buf[1:rows + 1], rows, hidden)
    cuda.cuda.synchronize()
    host = buf.cpu().numpy()
    assert (host[0] == host[0, 0]).all() and (host[-1] == host[0, 0]).all(), "write outside the output rows"
    got = host[1:rows + 1].view(NP[out_dtype])
    want_bits = want.view(np.uint32) if out_dtype == B.FP32 else want
    got_bits = got.view(np.uint32) if out_dtype == B.FP32 else got
    dist = _steps(got_bits, want_bits)
    limit = 16 + hidden // 32 if out_dtype == B.FP32 else 1
    print(f"rms_norm {rows}x{hidden}: {int((dist > 0).sum())} of {dist.size} outputs differ, max {int(dist.max())} step(s)")
    assert dist.max() <= limit
    assert B.last_variant() == "rms_norm"


def test_qwen_rms_norm_golden_inputs(cuda):
    d = G.decoder_op_inputs()
    want = O.qwen_rms_norm(O.BF16, d["rms_x_bf16"], O.BF16, d["rms_w_bf16"], 1.0, 1e-6, O.BF16)
    out = cuda.empty((5, 1024), dtype=cuda.int16, device="cuda")
    B.qwen_rms_norm(B.BF16, dev(cuda, d["rms_x_bf16"].view(np.int16)), B.BF16, dev(cuda, d["rms_w_bf16"].view(np.int16)), 1.0, 1e-6, B.BF16, out, 5, 1024)
    assert _steps(out.cpu().numpy().view(np.uint16), want).max() <= 1


@pytest.mark.parametrize("dtype", [B.BF16, B.FP32, B.FP16])
@pytest.mark.parametrize("rows,cols", [(1, 1024), (16, 3584), (4, 1030), (3, 7)])
def test_add_mul_bit_exact(cuda, dtype, rows, cols):
    rng = np.random.default_rng(rows + cols)
    lhs, rhs, row = _rand(rng, (rows, cols), dtype, 2.0), _rand(rng, (rows, cols), dtype), _rand(rng, (cols,), dtype)
    as_dev = lambda a: dev(cuda, a.view(np.int16) if a.dtype == np.uint16 else a)  # noqa: E731
    for op in (B.BINARY_ADD, B.BINARY_MUL):
        for r, rhs_count in ((rhs, 0), (row, cols)):
            if dtype == B.FP16:  # the oracle's FP16 path is the same read-op-round rule
                want = O.binary(op, O.FP16, lhs, r)
            else:
                want = O.binary(op, dtype, lhs, r)
            out = cuda.zeros((rows, cols), dtype=cuda.float32 if dtype == B.FP32 else cuda.int16, device="cuda")
            B.binary(op, dtype, as_dev(lhs), as_dev(r), out, rows * cols, rhs_count)
            cuda.cuda.synchronize()
            got = out.cpu().numpy().view(NP[dtype])
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (op, rhs_count)


@pytest.mark.parametrize("dtype", [B.BF16, B.FP32])
def test_silu_and_silu_mul(cuda, dtype):
    d = G.decoder_op_inputs()
    x = d["silu_bf16"] if dtype == B.BF16 else d["silu_fp32"]
    rng = np.random.default_rng(3)
    up = _rand(rng, x.shape, dtype, 2.0)
    as_dev = lambda a: dev(cuda, a.view(np.int16) if a.dtype == np.uint16 else a)  # noqa: E731
    want = O.silu(dtype, x)
    out = cuda.zeros(x.size, dtype=cuda.float32 if dtype == B.FP32 else cuda.int16, device="cuda")
    B.silu(dtype, as_dev(x), out, x.size)
    cuda.cuda.synchronize()
    got = out.cpu().numpy().view(NP[dtype])
    bits = (lambda a: a.view(np.uint32)) if dtype == B.FP32 else (lambda a: a)
    dist = _steps(bits(got), bits(want))
    print(f"silu dtype {dtype}: {int((dist > 0).sum())} of {dist.size} outputs differ, max {int(dist.max())} step(s)")
    assert dist.max() <= 1 and (dist > 0).mean() < 1e-3
    # SiLU node followed by Mul node, in one launch: both rounding points
    want2 = O.binary(1, dtype, want.reshape(1, -1), up.reshape(1, -1))[0]
    B.silu_mul(dtype, as_dev(x), as_dev(up), out, x.size)
    cuda.cuda.synchronize()
    got2 = out.cpu().numpy().view(NP[dtype])
    same_silu = dist == 0
    assert np.array_equal(got2[same_silu].view(np.uint8), want2[same_silu].view(np.uint8))
    assert B.last_variant() == "silu_mul" and B.device_status() == 0


def test_silu_bf16_every_input(cuda):
    """All 65536 BF16 inputs.  The BF16 kernels take a short path (FP32 expf, and the exact evaluation only where the
    quotient sits next to a rounding boundary): it must give the bits of the exact evaluation everywhere, and those are
    the oracle's up to the rare last-place difference between the C library's expf and the correctly rounded one."""
    x = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    xf = (x.astype(np.uint32) << 16).view(np.float32)
    finite = np.isfinite(xf)
    out16 = cuda.zeros(x.size, dtype=cuda.int16, device="cuda")
    out32 = cuda.zeros(x.size, dtype=cuda.float32, device="cuda")
    B.silu(B.BF16, dev(cuda, x.view(np.int16)), out16, x.size)
    B.silu(B.FP32, dev(cuda, xf), out32, x.size)
    cuda.cuda.synchronize()
    got = out16.cpu().numpy().view(np.uint16)
    exact = G.to_bf16(out32.cpu().numpy())
    assert np.array_equal(got[finite], exact[finite]), f"{int((got[finite] != exact[finite]).sum())} inputs leave the short path with other bits"
    nan = np.isnan(xf)
    assert np.isnan((got[nan].astype(np.uint32) << 16).view(np.float32)).all()
    want = O.silu(B.BF16, x)
    dist = _steps(got[finite], want[finite])
    print(f"silu over every finite BF16 input: {int((dist > 0).sum())} of {int(finite.sum())} differ from the oracle, max {int(dist.max())} step(s)")
    assert dist.max() <= 1 and (dist > 0).mean() < 1e-3


def test_rejections(cuda):
    t = cuda.zeros(64, dtype=cuda.float32, device="cuda")
    lib = B.lib()
    import ctypes as C
    s = B.current_stream()
    assert lib.fth_b200_qwen_rms_norm(C.c_int32(B.FP32), C.c_void_p(t.data_ptr()), C.c_int32(B.FP32), C.c_void_p(t.data_ptr()), C.c_float(0.0),
                                      C.c_float(-1.0), C.c_int32(B.FP32), C.c_void_p(t.data_ptr()), C.c_int64(1), C.c_int64(64), s) == B.ERR_INVALID
    assert lib.fth_b200_qwen_rms_norm(C.c_int32(B.INT8), C.c_void_p(t.data_ptr()), C.c_int32(B.FP32), C.c_void_p(t.data_ptr()), C.c_float(0.0),
                                      C.c_float(1e-6), C.c_int32(B.FP32), C.c_void_p(t.data_ptr()), C.c_int64(1), C.c_int64(64), s) == B.ERR_UNSUPPORTED
    assert lib.fth_b200_binary(C.c_int32(0), C.c_int32(B.FP32), C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()),
                               C.c_int64(64), C.c_int64(48), s) == B.ERR_INVALID
    assert lib.fth_b200_silu(C.c_int32(B.INT8), C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), C.c_int64(64), s) == B.ERR_UNSUPPORTED
