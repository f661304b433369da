"""FP8 FC / MatMul / Gemm on the GPU against the CPU oracle (Common semantics).

Tolerance: every output byte within ONE FP8 code of the oracle after FP32 accumulation, and the class of
non-finite outputs (NaN / Inf codes) must match exactly."""
import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests import util
from tests.gpu_helpers import run_fp8_linear

pytestmark = pytest.mark.gpu

DTYPES = [O.E4M3, O.E5M2]


def check_codes(got, want, dtype, what, case=None, trans_b=False):
    """Tolerance: one output code.  Near zero the FP8 codes are far denser than FP32 accumulation error
    (two FP32 summation orders of 8192 terms already differ by several subnormal codes there), so an output
    also passes when its value is within the FP32 accumulation bound 2^-20 * sum_k |a_k w_k| of the oracle's."""
    dist = util.fp8_code_distance(got, want)
    # Non-finite class must match exactly: same Inf code, NaN code up to its sign bit (the sign of a NaN made
    # by arithmetic, e.g. 0 x Inf, is a host-FPU convention: x86 generates it negative, the GPU positive).
    special = (want & 0x7F) >= (0x7F if dtype == O.E4M3 else 0x7C)
    nan = (want & 0x7F) >= (0x7F if dtype == O.E4M3 else 0x7D)
    assert np.array_equal(got[special & ~nan], want[special & ~nan]), f"{what}: Inf codes differ"
    assert np.array_equal(got[nan] & 0x7F, want[nan] & 0x7F), f"{what}: NaN codes differ"
    dist = np.where(nan, 0, dist)
    if dist.max() > 1 and case is not None:
        a = np.abs(O.fp8_decode(dtype, case["a"]).astype(np.float64)) * case["sa"]
        w = np.abs(O.fp8_decode(dtype, case["w"]).astype(np.float64)) * case["sw"]
        bound = (a @ (w.T if trans_b else w)) * 2.0 ** -20
        err = np.abs(O.fp8_decode(dtype, got).astype(np.float64) - O.fp8_decode(dtype, want).astype(np.float64)) * case["so"]
        dist = np.where((dist > 1) & (err <= bound), 1, dist)
    assert dist.max() <= 1, f"{what}: max code distance {dist.max()} (> 1), {int((dist > 1).sum())} outputs"
    return int((dist > 0).sum())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("variant", [B.VARIANT_SIMT, B.VARIANT_SKINNY, B.VARIANT_STREAM, B.VARIANT_TCGEN05])
@pytest.mark.parametrize("m,k,n", [(1, 1024, 3072), (2, 1024, 1024), (3, 3584, 1024), (4, 1024, 3584), (16, 512, 256),
                                   (1, 48, 16), (5, 130, 272), (1, 8192, 512), (2, 200, 400), (1, 8192, 1040)])
def test_matmul_kn(cuda, dtype, variant, m, k, n):
    if variant == B.VARIANT_STREAM and m > 2:
        pytest.skip("the TMA-ring GEMV takes M <= 2 for FP8")
    case = util.make_fp8_linear(dtype, m, k, n, seed=m * 7 + k + n)
    want = O.fp8_linear(O.OP_MATMUL, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"])
    got = run_fp8_linear(cuda, dtype, B.OP_MATMUL, case, variant=variant)
    check_codes(got, want, dtype, f"matmul {m}x{k}x{n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("variant", [B.VARIANT_SIMT, B.VARIANT_SKINNY, B.VARIANT_TCGEN05])
@pytest.mark.parametrize("m,k,n", [(1, 1024, 3072), (2, 1024, 1000), (4, 2048, 77), (7, 528, 19), (1, 8192, 640)])
def test_gemm_trans_b(cuda, dtype, variant, m, k, n):
    case = util.make_fp8_linear(dtype, m, k, n, seed=k + n, trans_b=True, bias_mode=1)
    kw = dict(bias=case["bias"], bias_scale=case["sb"], trans_b=True, alpha=0.75, beta=1.25)
    want = O.fp8_linear(O.OP_GEMM, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"], **kw)
    got = run_fp8_linear(cuda, dtype, B.OP_GEMM, case, trans_b=True, variant=variant, alpha=0.75, beta=1.25)
    check_codes(got, want, dtype, f"gemm^T {m}x{k}x{n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op,bias_mode", [(B.OP_FC, 1), (B.OP_FC, 2), (B.OP_GEMM, 2), (B.OP_GEMM, 0)])
def test_bias_modes_auto_variant(cuda, dtype, op, bias_mode):
    case = util.make_fp8_linear(dtype, 3, 256, 320, seed=11 + bias_mode, bias_mode=bias_mode, pow2=True)
    kw = dict(bias=case["bias"], bias_scale=case["sb"])
    want = O.fp8_linear(op, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"], **kw)
    got = run_fp8_linear(cuda, dtype, op, case)
    check_codes(got, want, dtype, f"op {op} bias {bias_mode}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_ragged_shapes_simt(cuda, dtype):
    # every tail of the 64x64x32 tiling, including sizes no TMA / 16-byte path can take
    for m, k, n in [(1, 1, 1), (2, 3, 5), (17, 33, 65), (63, 64, 65), (65, 127, 129), (128, 31, 63)]:
        case = util.make_fp8_linear(dtype, m, k, n, seed=m + k + n, bias_mode=1)
        want = O.fp8_linear(O.OP_FC, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"],
                            bias=case["bias"], bias_scale=case["sb"])
        got = run_fp8_linear(cuda, dtype, B.OP_FC, case)
        assert B.last_variant() == "simt"
        check_codes(got, want, dtype, f"ragged {m}x{k}x{n}")


def test_nonfinite_codes_propagate(cuda):
    """E5M2 Inf in an operand reaches the output as the Inf code 0x7C; E4M3 NaN as 0x7F
    (reference test/x86_fp8_linear_test.cc:142-156)."""
    for dtype, code in ((O.E5M2, 0x7C), (O.E4M3, 0x7F)):
        for variant in (B.VARIANT_SIMT, B.VARIANT_SKINNY, B.VARIANT_STREAM, B.VARIANT_TCGEN05):
            case = util.make_fp8_linear(dtype, 1, 64, 32, seed=9)
            case["a"][:] = O.fp8_encode(dtype, np.ones((1, 64), np.float32))
            case["w"][:] = O.fp8_encode(dtype, np.ones((64, 32), np.float32))
            case["w"][5, 7] = code
            case.update(sa=1.0, sw=1.0, so=1.0)
            want = O.fp8_linear(O.OP_MATMUL, dtype, case["a"], 1.0, case["w"], 1.0, 1.0)
            got = run_fp8_linear(cuda, dtype, B.OP_MATMUL, case, variant=variant)
            assert got[0, 7] == want[0, 7] == code
            assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fused_cast_prologue_and_epilogue(cuda, dtype):
    """Cast(BF16→FP8) → MatMul → Cast(FP8→BF16) in one call equals the three reference nodes."""
    rng = np.random.default_rng(21)
    m, k, n = 2, 1024, 768
    case = util.make_fp8_linear(dtype, m, k, n, seed=21, pow2=True)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x_bf16 = (x.view(np.uint32) >> 16).astype(np.uint16)
    a_codes = O.cast(O.BF16, x_bf16, 1.0, dtype, case["sa"]).reshape(m, k)
    mid = O.fp8_linear(O.OP_MATMUL, dtype, a_codes, case["sa"], case["w"], case["sw"], case["so"])
    want = O.cast(dtype, mid, case["so"], O.BF16, 1.0).reshape(m, n)
    got = run_fp8_linear(cuda, dtype, B.OP_MATMUL, case, a_dtype=B.BF16, out_dtype=B.BF16, a_raw=x_bf16)
    # compare through the FP8 codes the BF16 values stand for
    got_codes = O.cast(O.BF16, got, 1.0, dtype, case["so"]).reshape(m, n)
    check_codes(got_codes, mid, dtype, "fused cast")
    same = got_codes == mid
    assert np.array_equal(got[same], want[same])


@pytest.mark.parametrize("dtype", DTYPES)
def test_output_row_stride(cuda, dtype):
    """ldo > n: a column shard writes its slice straight into a wider [M, N_total] buffer."""
    case = util.make_fp8_linear(dtype, 2, 256, 256, seed=31)
    want = O.fp8_linear(O.OP_MATMUL, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"])
    got = run_fp8_linear(cuda, dtype, B.OP_MATMUL, case, ldo=1024)
    check_codes(got, want, dtype, "ldo")


def test_rejections(cuda):
    """Contract violations the reference kernels answer with -1 (src/kernel/fp8_host.h:150-203)."""
    import ctypes as C
    case = util.make_fp8_linear(O.E4M3, 1, 64, 64, seed=1)
    from tests.gpu_helpers import dev
    a, w = dev(cuda, case["a"]), dev(cuda, case["w"])
    out = cuda.empty((1, 64), dtype=cuda.uint8, device="cuda")
    base = dict(dtype=B.E4M3, op=B.OP_MATMUL, m=1, k=64, n=64, a=a, w=w, out=out, a_scale=1.0, w_scale=1.0, out_scale=1.0)
    assert B.lib().fth_b200_fp8_linear(C.byref(B.fp8_linear_desc(**base, variant=B.VARIANT_STREAM)), B.current_stream()) == B.OK  # K=64: no split, no scratch
    d = B.fp8_linear_desc(**{**base, 'k': 64}, variant=7)
    assert B.lib().fth_b200_fp8_linear(C.byref(d), B.current_stream()) == B.ERR_INVALID
    for bad in (dict(a_scale=0.0), dict(out_scale=float("nan")), dict(w_scale=float("inf")), dict(m=0), dict(dtype=B.INT8),
                dict(trans_b=True), dict(out=None), dict(bias_mode=1)):
        d = B.fp8_linear_desc(**{**base, **bad})
        assert B.lib().fth_b200_fp8_linear(C.byref(d), B.current_stream()) == B.ERR_INVALID, bad


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_workspace_is_left_clean_and_reusable(cuda, dtype):
    """The TMA-ring kernel's arrival counters return to zero, so one zero-filled workspace serves every
    later call; a column shard gives the same bytes as the same columns of the full weight."""
    import ctypes as C
    from tests.gpu_helpers import dev
    m, k, n = 2, 4096, 1024
    case = util.make_fp8_linear(dtype, m, k, n, seed=77)
    want = O.fp8_linear(O.OP_MATMUL, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"])
    a, w = dev(cuda, case["a"]), dev(cuda, case["w"])
    out = cuda.zeros((m, n), dtype=cuda.uint8, device="cuda")
    d = B.fp8_linear_desc(dtype=dtype, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=out, a_scale=case["sa"],
                          w_scale=case["sw"], out_scale=case["so"], variant=B.VARIANT_STREAM)
    ws = B.linear_workspace(cuda, d)
    assert ws is not None
    full = None
    for _ in range(3):
        out.zero_()
        B.fp8_linear(d)
        cuda.cuda.synchronize()
        got = out.cpu().numpy()
        check_codes(got, want, dtype, "stream reuse")
        assert full is None or np.array_equal(full, got)
        full = got
    counters = ws[:256].cpu().numpy().view(np.int32)
    assert (counters == 0).all()
    assert B.device_status() == 0
    # column shard: columns [256, 768) through a strided view of the same weight is not expressible in the
    # ABI (weights are dense), so shard by copying the slice — the bytes must equal the full run's slice
    w_shard = dev(cuda, np.ascontiguousarray(case["w"][:, 256:768]))
    out_s = cuda.zeros((m, 512), dtype=cuda.uint8, device="cuda")
    ds = B.fp8_linear_desc(dtype=dtype, op=B.OP_MATMUL, m=m, k=k, n=512, a=a, w=w_shard, out=out_s, a_scale=case["sa"],
                           w_scale=case["sw"], out_scale=case["so"], variant=B.VARIANT_STREAM)
    ws2 = B.linear_workspace(cuda, ds)
    B.fp8_linear(ds)
    cuda.cuda.synchronize()
    assert np.array_equal(out_s.cpu().numpy(), full[:, 256:768])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,k,n,trans_b", [(16, 8192, 2048, False), (64, 1024, 1024, False), (128, 1024, 1024, True),
                                           (300, 512, 528, False), (257, 2048, 272, True), (33, 4096, 640, False)])
def test_tensor_core_path_shapes(cuda, dtype, m, k, n, trans_b):
    """Dense and mid-size shapes on tcgen05: both weight layouts, swapped (M <= 128) and normal tiling, ragged
    M and N tails handled by TMA zero fill."""
    case = util.make_fp8_linear(dtype, m, k, n, seed=m + n, trans_b=trans_b)
    op = B.OP_GEMM if trans_b else B.OP_MATMUL
    want = O.fp8_linear(op, dtype, case["a"], case["sa"], case["w"], case["sw"], case["so"], trans_b=trans_b)
    got = run_fp8_linear(cuda, dtype, op, case, trans_b=trans_b, variant=B.VARIANT_TCGEN05)
    assert B.last_variant() == "tcgen05" and B.device_status() == 0
    check_codes(got, want, dtype, f"tcgen05 {m}x{k}x{n}", case=case, trans_b=trans_b)


# ---- one weight scale per output channel --------------------------------------------------------------------------------
# The reference's FP8 kernels take per-tensor scales only; its tensor metadata and model files can hold a per-channel
# vector.  The extension is defined column by column (oracle.fp8_linear_per_channel): every kernel family must give, for
# channel n, what the reference gives for that column alone with w_scale = scales[n].
PER_CHANNEL = [(1, 1024, 2048, False, B.VARIANT_AUTO),        # single-launch cluster kernel
               (4, 2048, 128 * 120, False, B.VARIANT_AUTO),   # persistent kernel, K chunks added from tensor memory
               (16, 4096, 4096, True, B.VARIANT_AUTO),        # persistent kernel + reduce pass, [N,K] weights
               (48, 1024, 1024, False, B.VARIANT_AUTO),       # 64-wide swapped tiles
               (300, 512, 640, False, B.VARIANT_AUTO),        # CTA pairs
               (3, 96, 80, False, B.VARIANT_SIMT), (4, 256, 384, False, B.VARIANT_SKINNY), (2, 1024, 1024, False, B.VARIANT_STREAM)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,k,n,trans_b,variant", PER_CHANNEL)
def test_per_channel_weight_scales(cuda, dtype, m, k, n, trans_b, variant):
    case = util.make_fp8_linear(dtype, m, k, n, seed=m * 3 + n, trans_b=trans_b, pow2=True, out_headroom=4.0)
    rng = np.random.default_rng(n + k)
    scales = (case["sw"] * np.exp2(rng.integers(-1, 3, n))).astype(np.float32)  # four powers of two around the tensor's scale
    op = B.OP_GEMM if trans_b else B.OP_MATMUL
    want = O.fp8_linear_per_channel(op, dtype, case["a"], case["sa"], case["w"], scales, case["so"], trans_b=trans_b)
    got = run_fp8_linear(cuda, dtype, op, case, trans_b=trans_b, variant=variant, w_channel_scales=scales)
    assert B.device_status() == 0
    dist = util.fp8_code_distance(got, want)
    if dist.max() > 1:  # near zero: within the FP32 accumulation bound of the oracle's value
        a = np.abs(O.fp8_decode(dtype, case["a"]).astype(np.float64)) * case["sa"]
        w = np.abs(O.fp8_decode(dtype, case["w"]).astype(np.float64))
        w = (w.T if trans_b else w) * scales.astype(np.float64)[None, :]
        err = np.abs(O.fp8_decode(dtype, got).astype(np.float64) - O.fp8_decode(dtype, want).astype(np.float64)) * case["so"]
        dist = np.where((dist > 1) & (err <= (a @ w) * 2.0 ** -20), 1, dist)
    assert dist.max() <= 1, f"per-channel scales {m}x{k}x{n}: max code distance {dist.max()}"
    # and the scales are really applied per channel: the per-tensor result differs
    plain = run_fp8_linear(cuda, dtype, op, case, trans_b=trans_b, variant=variant)
    assert not np.array_equal(plain, got)
