"""GPU: configuration 4 — the 24-layer E5M2 projection stack as a decode step (M = 1) and prefill chunks
(M = 2, 4, 8, 16).  The GPU runs every projection as ONE fused call (Cast -> MatMul -> Cast through a_dtype /
out_dtype = BF16); the oracle runs the three reference nodes one after another.  Required: cosine of the final
hidden state >= 0.999 (computed in float64 as tools/compare_qwen_logits.py:41-58 does), plus the projection-level
tolerance of one FP8 code when both sides are fed the same inputs."""
import ctypes as C

import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests import decoder_stack as D
from tests import util
from tests.gpu_helpers import dev

pytestmark = pytest.mark.gpu


def oracle_project(h_bits, weight):
    codes, sw = weight
    a = O.cast(O.BF16, h_bits, 1.0, O.E5M2, D.ACT_SCALE).reshape(h_bits.shape)
    y = O.fp8_linear(O.OP_MATMUL, O.E5M2, a, D.ACT_SCALE, codes, sw, D.OUT_SCALE)
    return O.cast(O.E5M2, y, D.OUT_SCALE, O.BF16, 1.0).reshape(y.shape)


class GpuProjector:
    def __init__(self, torch, weights, with_workspace=True):
        self.torch = torch
        self.with_workspace = with_workspace
        self.variants = set()
        self.dev = {id(layer[name][0]): dev(torch, layer[name][0]) for layer in weights for name, _, _ in D.PROJ}
        self.launches = 0

    def __call__(self, h_bits, weight):
        torch = self.torch
        codes, sw = weight
        m, k = h_bits.shape
        n = codes.shape[1]
        a = dev(torch, h_bits.view(np.int16))
        out = torch.empty((m, n), dtype=torch.int16, device="cuda")
        d = B.fp8_linear_desc(dtype=B.E5M2, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=self.dev[id(codes)], out=out,
                              a_scale=D.ACT_SCALE, w_scale=sw, out_scale=D.OUT_SCALE, a_dtype=B.BF16, out_dtype=B.BF16)
        keep = B.linear_workspace(torch, d) if self.with_workspace else None
        B.fp8_linear(d)
        self.variants.add(B.last_variant())
        self.launches += 1
        return out.cpu().numpy().view(np.uint16)


@pytest.fixture(scope="module")
def stack_weights():
    return D.make_weights(lambda x: O.fp8_encode(O.E5M2, x))


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
def test_decoder_stack_matches_oracle(cuda, stack_weights, m):
    rng = np.random.default_rng(100 + m)
    x0 = D.to_bf16(rng.standard_normal((m, D.HIDDEN)).astype(np.float32))
    trace = []
    want = D.from_bf16(D.run_stack(oracle_project, stack_weights, x0, trace)).astype(np.float64)
    gpu = GpuProjector(cuda, stack_weights)
    got = D.from_bf16(D.run_stack(gpu, stack_weights, x0)).astype(np.float64)
    assert gpu.launches == 7 * D.LAYERS and gpu.variants == {"tcgen05"}
    if m in (1, 16):  # the same stack without a workspace: whichever scratch-free kernels run, the result holds
        plain = GpuProjector(cuda, stack_weights, with_workspace=False)
        got_plain = D.from_bf16(D.run_stack(plain, stack_weights, x0)).astype(np.float64)
        assert plain.launches == 7 * D.LAYERS
        cos_plain = float((got_plain * want).sum() / (np.linalg.norm(got_plain) * np.linalg.norm(want)))
        assert cos_plain >= 0.999
    assert np.isfinite(got).all() and np.isfinite(want).all()
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    rmse = float(np.sqrt(((got - want) ** 2).mean()))
    print(f"M={m}: cosine {cos:.6f} rmse {rmse:.4g} max|err| {np.abs(got - want).max():.4g} "
          f"argmax equal {bool((got.argmax(axis=1) == want.argmax(axis=1)).all())} kernel {B.last_variant()}")
    assert cos >= 0.999
    # lockstep: the same inputs into both sides, projection by projection — at most one E5M2 code apart
    layer_of = [layer for layer in stack_weights for _ in range(7)]
    worst, flips, total = 0, 0, 0
    for idx in range(0, len(trace), 9):  # a sample of the 168 projections
        name, h = trace[idx]
        weight = layer_of[idx][name]
        o = O.cast(O.BF16, oracle_project(h, weight), 1.0, O.E5M2, D.OUT_SCALE)
        g = O.cast(O.BF16, gpu(h, weight), 1.0, O.E5M2, D.OUT_SCALE)
        dist = util.fp8_code_distance(g, o)
        worst, flips, total = max(worst, int(dist.max())), flips + int((dist > 0).sum()), total + dist.size
    print(f"M={m}: lockstep projections: {flips} of {total} outputs differ, max distance {worst} code(s)")
    assert worst <= 1
