"""INT8 Conv2D (NCHW, int32 bias, requant, optional fused ReLU table) on the GPU: bit-exact."""
import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests import util
from tests.gpu_helpers import run_int8_conv

pytestmark = pytest.mark.gpu


def oracle_conv(case, **kw):
    return O.int8_conv2d(case["x"], case["sx"], case["x_zp"], case["w"], case["ws"], case["w_zps"], case["bias"],
                         case["so"], case["out_zp"], **kw)


@pytest.mark.parametrize("variant", [B.VARIANT_SIMT, B.VARIANT_AUTO])
@pytest.mark.parametrize("shape", [(1, 64, 40, 48, 64, 3, 3), (2, 16, 17, 19, 8, 3, 3), (1, 64, 32, 32, 128, 1, 1), (1, 3, 9, 9, 5, 5, 5)])
def test_conv_same_padding(cuda, variant, shape):
    b, ic, ih, iw, oc, kh, kw = shape
    case = util.make_int8_conv(b, ic, ih, iw, oc, kh, kw, seed=sum(shape))
    pad = (kh // 2, kw // 2)
    want = oracle_conv(case, pad=pad)
    got = run_int8_conv(cuda, case, pad=pad, variant=variant)
    assert np.array_equal(got, want), f"{int((got != want).sum())} of {want.size} bytes differ"


def test_conv_general_geometry(cuda):
    """stride, dilation, groups, asymmetric zero points: the general kernel's contract."""
    for (stride, pad, dil, group) in [((2, 2), (1, 1), (1, 1), 1), ((1, 2), (0, 2), (2, 1), 1), ((1, 1), (1, 1), (1, 1), 4)]:
        case = util.make_int8_conv(2, 16, 21, 23, 8, 3, 3, seed=stride[0] + group, zero_points=True)
        if group > 1:
            case["w"] = case["w"][:, :16 // group].copy()
        want = oracle_conv(case, stride=stride, pad=pad, dil=dil, group=group)
        got = run_int8_conv(cuda, case, stride=stride, pad=pad, dil=dil, group=group)
        assert np.array_equal(got, want), (stride, pad, dil, group)


def test_conv_fused_relu_equals_two_nodes(cuda):
    """Conv → INT8 ReLU node (its own output scale) fused through the 256-entry table."""
    case = util.make_int8_conv(1, 64, 24, 40, 64, 3, 3, seed=12)
    conv = oracle_conv(case)
    for (so2, zo2) in [(case["so"], 0), (case["so"] * 0.7, -3)]:
        want = O.int8_relu(conv, case["so"], case["out_zp"], so2, zo2)
        lut = B.int8_relu_table(case["so"], case["out_zp"], so2, zo2)
        got = run_int8_conv(cuda, case, relu_lut=lut)
        assert np.array_equal(got, want)


def test_conv_reference_known_answer(cuda):
    """test/common_int8_kernel_test.cc:186-211 pattern: 1x1 input, bias added before requantisation."""
    case = dict(x=np.array([[[[4]]]], np.int8), w=np.array([[[[3]]]], np.int8), bias=np.array([12], np.int32), sx=0.5,
                x_zp=0, ws=np.array([0.5], np.float32), w_zps=None, so=1.0, out_zp=0)
    want = oracle_conv(case, pad=(0, 0))
    got = run_int8_conv(cuda, case, pad=(0, 0))
    assert got.tolist() == want.tolist() == [[[[6]]]]


def test_conv_config3_full_size(cuda):
    """1x64x160x160 (*) 64x64x3x3, stride 1, pad 1, per-channel scales, int32 bias, fused ReLU."""
    case = util.make_int8_conv(1, 64, 160, 160, 64, 3, 3, seed=3)
    conv = oracle_conv(case)
    want = O.int8_relu(conv, case["so"], 0, case["so"], 0)
    lut = B.int8_relu_table(case["so"], 0, case["so"], 0)
    got = run_int8_conv(cuda, case, relu_lut=lut)
    assert B.last_variant() == "conv_tcgen05" and B.device_status() == 0
    assert np.array_equal(got, want)
    assert np.array_equal(run_int8_conv(cuda, case), conv)


def test_conv_with_caller_owned_packed_weight(cuda):
    """The weight packed once by fth_b200_int8_conv2d_pack_weights and handed to two different calls (other inputs, own
    workspaces): same bytes as the call that packs into its own workspace, and the workspace need shrinks to the
    channels-last input copy."""
    import ctypes as C
    from tests.gpu_helpers import dev
    case = util.make_int8_conv(1, 64, 24, 40, 64, 3, 3, seed=11)
    want = O.int8_conv2d(case["x"], case["sx"], 0, case["w"], case["ws"], None, case["bias"], case["so"], 0)
    lib = B.lib()
    w, ws, b = dev(cuda, case["w"]), dev(cuda, case["ws"]), dev(cuda, case["bias"])

    def desc(x, out):
        return B.int8_conv2d_desc(batch=1, ic=64, ih=24, iw=40, oc=64, kh=3, kw=3, x=x, w=w, out=out, x_scale=case["sx"], x_zp=0, w_scales=ws,
                                  w_zps=None, w_params=64, out_scale=case["so"], out_zp=0, bias=b, bias_max_abs=1 << 15)
    x = dev(cuda, case["x"])
    out = cuda.zeros((1, 64, 24, 40), dtype=cuda.int8, device="cuda")
    d = desc(x, out)
    own = lib.fth_b200_int8_conv2d_workspace_bytes(C.byref(d))
    need = lib.fth_b200_int8_conv2d_packed_weight_bytes(C.byref(d))
    assert need >= 64 * 64 * 9
    packed = cuda.zeros(need, dtype=cuda.uint8, device="cuda")
    assert lib.fth_b200_int8_conv2d_pack_weights(C.byref(d), C.c_void_p(packed.data_ptr()), B.current_stream()) == B.OK
    d.packed_w = packed.data_ptr()
    shared = lib.fth_b200_int8_conv2d_workspace_bytes(C.byref(d))
    assert shared + need == own
    for seed in (11, 12):  # two calls, two inputs, one packed weight
        c2 = util.make_int8_conv(1, 64, 24, 40, 64, 3, 3, seed=seed)
        x2 = dev(cuda, c2["x"])
        out2 = cuda.zeros((1, 64, 24, 40), dtype=cuda.int8, device="cuda")
        d2 = desc(x2, out2)
        d2.packed_w = packed.data_ptr()
        scratch = cuda.zeros(shared, dtype=cuda.uint8, device="cuda")
        d2.workspace, d2.workspace_bytes = scratch.data_ptr(), shared
        B.int8_conv2d(d2)
        cuda.cuda.synchronize()
        assert B.last_variant() == "conv_tcgen05"
        want2 = O.int8_conv2d(c2["x"], case["sx"], 0, case["w"], case["ws"], None, case["bias"], case["so"], 0)
        assert np.array_equal(out2.cpu().numpy(), want2)
    assert np.array_equal(want, O.int8_conv2d(case["x"], case["sx"], 0, case["w"], case["ws"], None, case["bias"], case["so"], 0))
    # geometries the implicit-GEMM kernel does not take have nothing to pack
    d3 = B.int8_conv2d_desc(batch=1, ic=16, ih=8, iw=8, oc=8, kh=3, kw=3, x=x, w=w, out=out, x_scale=1.0, x_zp=0, w_scales=ws, w_zps=None,
                            w_params=8, out_scale=1.0, out_zp=0)
    assert lib.fth_b200_int8_conv2d_packed_weight_bytes(C.byref(d3)) == 0
    assert lib.fth_b200_int8_conv2d_pack_weights(C.byref(d3), C.c_void_p(packed.data_ptr()), B.current_stream()) == B.ERR_UNSUPPORTED
    assert B.device_status() == 0
