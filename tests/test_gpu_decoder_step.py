"""GPU: a whole decode / prefill-chunk step of the synthetic decoder stack on the device — projections AND the operators
between them — against the CPU oracle, and the six-launch-per-layer fused form against the twelve-launch form.

* fused == unfused, byte for byte: fth_b200_fp8_linear_fused keeps every rounding point of the nodes it absorbs
  (QwenRmsNorm, SiLU, Mul, Add, both Casts) and sums the squares of a row in the stand-alone kernel's order.
* against the oracle (reference Common kernels for every node, tests/decoder_stack.py), layer by layer: every layer run
  on the device from the oracle's own input to that layer gives the oracle's output up to isolated one-code steps
  and what the six projections behind such a step make of it (cosine >= 0.9999, as tools/compare_qwen_logits.py:41-58
  computes it; at most 5 % of the outputs differ at all; tests/test_gpu_decoder_stack.py holds the node-by-node
  comparison, where each projection starts from the oracle's input: at most one code apart).
* the free-running 24-layer step: cosine >= 0.995 and the same greedy index per row.  A row of E5M2 codes has two
  mantissa bits, so one output that lands on the other side of a rounding boundary (the tensor core adds the products
  of a dot product in another order than the sequential CPU loop) moves by 25 % and the layers behind it carry that
  on; the per-layer check above is the one that bounds the kernels."""
import ctypes as C

import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from infer_b200.decoder_step import DecoderStep
from tests import decoder_stack as D
from tests.gpu_helpers import dev

pytestmark = pytest.mark.gpu


def device_layers(torch, weights):
    layers = []
    for layer in weights:
        d = {}
        for name, _, _ in D.PROJ:
            codes, scale = layer[name]
            d[name] = dev(torch, codes)
            d[name + "_scale"] = scale
        d["g1"] = dev(torch, layer["g1"].view(np.int16))
        d["g2"] = dev(torch, layer["g2"].view(np.int16))
        layers.append(d)
    return layers


def oracle_project(h_bits, weight):
    codes, sw = weight
    a = O.cast(O.BF16, h_bits, 1.0, O.E5M2, D.ACT_SCALE).reshape(h_bits.shape)
    y = O.fp8_linear(O.OP_MATMUL, O.E5M2, a, D.ACT_SCALE, codes, sw, D.OUT_SCALE)
    return O.cast(O.E5M2, y, D.OUT_SCALE, O.BF16, 1.0).reshape(y.shape)


def run_device(torch, layers, x0, m, fused):
    step = DecoderStep(torch, layers, m, D.HIDDEN, D.INTER, D.ACT_SCALE, D.OUT_SCALE, fp8_dtype=B.E5M2, epsilon=float(D.EPS), fused=fused)
    step.x.copy_(dev(torch, x0.view(np.int16)))
    step.run()
    torch.cuda.synchronize()
    assert B.device_status() == 0
    return step.result.cpu().numpy().view(np.uint16), step


@pytest.fixture(scope="module")
def stack_weights():
    return D.make_weights(lambda x: O.fp8_encode(O.E5M2, x))


@pytest.mark.parametrize("m", [1, 4, 16])
def test_fused_step_equals_node_by_node_step(cuda, stack_weights, m):
    layers = device_layers(cuda, stack_weights[:3])
    rng = np.random.default_rng(300 + m)
    x0 = D.to_bf16(rng.standard_normal((m, D.HIDDEN)).astype(np.float32))
    plain, step_plain = run_device(cuda, layers, x0, m, fused=False)
    fused, step_fused = run_device(cuda, layers, x0, m, fused=True)
    assert step_plain.launches == 12 * 3 and step_fused.launches == 6 * 3
    assert np.array_equal(fused, plain), f"{int((fused != plain).sum())} of {plain.size} BF16 outputs differ"


@pytest.mark.parametrize("m", [1, 16])
def test_whole_step_on_device_matches_oracle(cuda, stack_weights, m):
    layers = device_layers(cuda, stack_weights)
    rng = np.random.default_rng(100 + m)
    x0 = D.to_bf16(rng.standard_normal((m, D.HIDDEN)).astype(np.float32))
    want = D.from_bf16(D.run_stack(oracle_project, stack_weights, x0)).astype(np.float64)
    got_bits, step = run_device(cuda, layers, x0, m, fused=True)
    got = D.from_bf16(got_bits).astype(np.float64)
    assert step.launches == 6 * D.LAYERS
    assert np.isfinite(got).all() and np.isfinite(want).all()
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    rmse = float(np.sqrt(((got - want) ** 2).mean()))
    print(f"M={m}: whole step on device, {step.launches} launches: cosine {cos:.6f} rmse {rmse:.4g} max|err| {np.abs(got - want).max():.4g} "
          f"argmax equal {bool((got.argmax(axis=1) == want.argmax(axis=1)).all())}")
    assert cos >= 0.995
    assert (got.argmax(axis=1) == want.argmax(axis=1)).all()


@pytest.mark.parametrize("m", [1, 16])
@pytest.mark.parametrize("fused", [True, False])
def test_every_layer_from_the_oracles_input(cuda, stack_weights, m, fused):
    rng = np.random.default_rng(100 + m)
    x0 = D.to_bf16(rng.standard_normal((m, D.HIDDEN)).astype(np.float32))
    states = []
    D.run_stack(oracle_project, stack_weights, x0, states=states)
    worst_cos, worst_frac, total_diff = 1.0, 0.0, 0
    for index in range(D.LAYERS):
        layers = device_layers(cuda, stack_weights[index:index + 1])
        got_bits, _ = run_device(cuda, layers, states[index], m, fused=fused)
        want_bits = states[index + 1]
        got, want = D.from_bf16(got_bits).astype(np.float64), D.from_bf16(want_bits).astype(np.float64)
        cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
        differing = int((got_bits != want_bits).sum())
        worst_cos, worst_frac, total_diff = min(worst_cos, cos), max(worst_frac, differing / want_bits.size), total_diff + differing
        assert cos >= 0.9999, f"layer {index}: cosine {cos}"
        assert differing <= 0.05 * want_bits.size, f"layer {index}: {differing} of {want_bits.size} outputs differ"
    print(f"M={m} {'fused' if fused else 'node by node'}: 24 layers, each from the oracle's input: worst cosine {worst_cos:.7f}, "
          f"{total_diff} of {24 * m * D.HIDDEN} BF16 outputs differ (worst layer {100 * worst_frac:.3f} %)")


@pytest.mark.parametrize("m,k,n", [(1, 1024, 3584), (16, 1024, 3584), (4, 512, 208), (32, 2048, 1024)])
def test_two_weights_in_one_launch(cuda, m, k, n):
    """gate and up on one activation: one launch gives the two separate launches' bytes; with the SiLU * Mul epilogue it
    gives what fth_b200_silu_mul makes of them; and the down projection that starts from SiLU * Mul of two inputs
    (prologue form) gives the bytes of the separate nodes as well."""
    torch = cuda
    rng = np.random.default_rng(m * 7 + n)
    a = dev(torch, D.to_bf16(rng.standard_normal((m, k)).astype(np.float32)).view(np.int16))
    w1 = dev(torch, rng.integers(0, 120, (k, n), dtype=np.uint8) | (rng.integers(0, 2, (k, n), dtype=np.uint8) << 7))
    w2 = dev(torch, rng.integers(0, 120, (k, n), dtype=np.uint8) | (rng.integers(0, 2, (k, n), dtype=np.uint8) << 7))
    outs = [torch.zeros((m, n), dtype=torch.int16, device="cuda") for _ in range(6)]
    common = dict(dtype=B.E5M2, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, a_scale=2.0 ** -7, out_scale=2.0 ** -6, a_dtype=B.BF16, out_dtype=B.BF16)
    keep = []
    for w, ws, out in ((w1, 2.0 ** -18, outs[0]), (w2, 2.0 ** -19, outs[1])):
        d = B.fp8_linear_desc(w=w, w_scale=ws, out=out, **common)
        keep.append(B.linear_workspace(torch, d))
        B.fp8_linear(d)
    B.silu_mul(B.BF16, outs[0], outs[1], outs[2], m * n)
    d = B.fp8_linear_desc(w=w1, w_scale=2.0 ** -18, out=outs[3], **common)
    B.fp8_linear_fused(d, B.fp8_linear_fusion(w2=w2, w2_scale=2.0 ** -19, out2=outs[4], n2=n))
    d5 = B.fp8_linear_desc(w=w1, w_scale=2.0 ** -18, out=outs[5], **common)
    B.fp8_linear_fused(d5, B.fp8_linear_fusion(w2=w2, w2_scale=2.0 ** -19, n2=n, epilogue=B.FUSE_OUT_SILU_MUL))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    h = [o.cpu().numpy() for o in outs]
    assert h[0].any() and h[1].any()
    assert np.array_equal(h[3], h[0]) and np.array_equal(h[4], h[1])
    assert np.array_equal(h[5], h[2]), f"{int((h[5] != h[2]).sum())} of {h[2].size} SiLU * Mul outputs differ"
    # SiLU * Mul in front of a projection (K = n here): prologue form against the separate node
    wd = dev(torch, rng.integers(0, 120, (n, 256), dtype=np.uint8))
    o_plain = torch.zeros((m, 256), dtype=torch.int16, device="cuda")
    o_fused = torch.zeros((m, 256), dtype=torch.int16, device="cuda")
    base = dict(dtype=B.E5M2, op=B.OP_MATMUL, m=m, k=n, n=256, w=wd, a_scale=2.0 ** -7, w_scale=2.0 ** -18, out_scale=2.0 ** -6, a_dtype=B.BF16, out_dtype=B.BF16)
    dp = B.fp8_linear_desc(a=outs[2], out=o_plain, **base)
    keep.append(B.linear_workspace(torch, dp))
    B.fp8_linear(dp)
    B.fp8_linear_fused(B.fp8_linear_desc(a=outs[0], out=o_fused, **base), B.fp8_linear_fusion(prologue=B.FUSE_SILU_MUL, a2=outs[1]))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert np.array_equal(o_fused.cpu().numpy(), o_plain.cpu().numpy())


def test_fused_call_rejections(cuda):
    torch = cuda
    a = torch.zeros((1, 1024), dtype=torch.int16, device="cuda")
    w = torch.zeros((1024, 1024), dtype=torch.uint8, device="cuda")
    out = torch.zeros((1, 1024), dtype=torch.int16, device="cuda")
    base = dict(dtype=B.E5M2, op=B.OP_MATMUL, m=1, k=1024, n=1024, a=a, w=w, out=out, a_scale=1.0, w_scale=1.0, out_scale=1.0)
    ok = B.fp8_linear_desc(a_dtype=B.BF16, out_dtype=B.BF16, **base)
    sup = B.lib().fth_b200_fp8_linear_fused_supported
    f = B.fp8_linear_fusion(residual=out)
    assert sup(C.byref(ok), C.byref(f)) == B.OK
    assert sup(C.byref(B.fp8_linear_desc(**base)), C.byref(f)) == B.ERR_UNSUPPORTED                       # FP8 in / out: nothing to fuse around
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(prologue=B.FUSE_RMS_NORM))) == B.ERR_INVALID       # no norm weight
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(prologue=B.FUSE_SILU_MUL))) == B.ERR_INVALID       # no second input
    big = B.fp8_linear_desc(a_dtype=B.BF16, out_dtype=B.BF16, **dict(base, m=64))
    assert sup(C.byref(big), C.byref(f)) == B.ERR_UNSUPPORTED                                             # not a decode-sized shape
    assert sup(C.byref(ok), None) == B.ERR_INVALID
    w2 = dict(w2=w, w2_scale=1.0, n2=1024)
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(epilogue=B.FUSE_OUT_SILU_MUL))) == B.ERR_INVALID              # needs the second weight
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(epilogue=B.FUSE_OUT_SILU_MUL, residual=out, **w2))) == B.ERR_INVALID
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(epilogue=B.FUSE_OUT_SILU_MUL, **w2))) == B.OK             # out2 not needed
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(**w2))) == B.ERR_INVALID                                  # ... but needed here
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(out2=out, **dict(w2, n2=512)))) == B.ERR_INVALID          # columns must pair up
    codes = torch.zeros((1, 1024), dtype=torch.uint8, device="cuda")
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(out_codes=codes, out_codes_scale=0.5))) == B.OK
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(out_codes=codes, out_codes_scale=0.0))) == B.ERR_INVALID
    assert sup(C.byref(ok), C.byref(B.fp8_linear_fusion(out_codes=codes, out2=out, **w2))) == B.ERR_INVALID       # which of the two outputs?
    from_codes = B.fp8_linear_desc(a_dtype=0, out_dtype=B.BF16, **dict(base, a=codes))
    assert sup(C.byref(from_codes), C.byref(B.fp8_linear_fusion(residual=out))) == B.OK                           # 8-bit activations in
    assert sup(C.byref(from_codes), C.byref(B.fp8_linear_fusion(prologue=B.FUSE_RMS_NORM, norm_weight=a))) == B.ERR_INVALID  # a norm works on BF16
