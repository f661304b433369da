"""GPU: the large-GEMM sweep (K = 8192, N = 28672; FP8 E4M3 and INT8; M = 1, 16, 256, 4096) against the CPU oracle,
plus mid-size cases that make every persistent kernel run many work units per CTA.

These are the shapes the benchmark times.  M = 1 and 16 are compared in full.  M = 256 and 4096 are compared on all M
rows x a seeded 1024-column slice and on 64 seeded rows x all N columns: an output depends only on its own activation
row and weight column, so the oracle run on the sliced operands (same K, same scales) is exact for those outputs.

INT8 must be bit-exact.  FP8 tolerance: one output code; an output farther away passes only when its value lies within
the FP32 accumulation bound 2^-20 * sum_k |a_k w_k| of the oracle's (near zero the FP8 codes are denser than the
rounding error of an 8192-term FP32 sum) — the number of outputs that needed that rule is printed with every case, and
beside it the same statistics for the reference's own x86 kernel against its Common kernel where that library is present.

Inputs follow the benchmark's distributions (tests/util.py): N(0,1) activations, N(0,0.02) weights with an absmax
per-tensor FP8 scale; uniform int8 in [-127,127] with per-output-channel weight scales in [1e-3, 1e-2]."""
import json
import os

import numpy as np
import pytest

import infer_b200 as B
import oracle as O
from tests import util
from tests.gpu_helpers import dev

pytestmark = pytest.mark.gpu
K, N = 8192, 28672
SLICE_COLS, SLICE_ROWS = 1024, 64
REPORT = os.environ.get("FTH_B200_PARITY_REPORT")  # optional: a file that receives one JSON line per compared case


def _note(record):
    print(json.dumps(record))
    if REPORT:
        with open(REPORT, "a") as f:
            f.write(json.dumps(record) + "\n")


@pytest.fixture(scope="module")
def fp8_weight(cuda):
    w, sw = util.make_fp8_weight(O.E4M3, K, N, seed=0xC5)
    return w, sw, dev(cuda, w)


@pytest.fixture(scope="module")
def int8_weight(cuda):
    w, ws = util.make_int8_weight(K, N, seed=0xC5 + 1)
    return w, ws, dev(cuda, w), dev(cuda, ws)


def _run_fp8(torch, a, sa, w_dev, sw, so, m, k, n, trans_b=False, dtype=B.E4M3):
    a_dev = dev(torch, a)
    buf = torch.full((m + 2, n), 0x5A, dtype=torch.uint8, device="cuda")
    d = B.fp8_linear_desc(dtype=dtype, op=B.OP_GEMM if trans_b else B.OP_MATMUL, m=m, k=k, n=n, a=a_dev, w=w_dev, out=buf[1:m + 1],
                          a_scale=sa, w_scale=sw, out_scale=so, trans_b=trans_b)
    keep = B.linear_workspace(torch, d)
    B.fp8_linear(d)
    torch.cuda.synchronize()
    assert B.last_variant() == "tcgen05"
    host = buf.cpu().numpy()
    assert (host[0] == 0x5A).all() and (host[-1] == 0x5A).all(), "write outside the output rows"
    del keep
    return host[1:m + 1]


def _run_int8(torch, a, w_dev, ws_dev, so, m, k, n, trans_b=False):
    a_dev = dev(torch, a)
    buf = torch.full((m + 2, n), 77, dtype=torch.int8, device="cuda")
    d = B.int8_linear_desc(op=B.OP_GEMM if trans_b else B.OP_MATMUL, m=m, k=k, n=n, a=a_dev, w=w_dev, out=buf[1:m + 1], a_scale=0.02,
                           a_zp=0, w_scales=ws_dev, w_zps=None, w_params=n, out_scale=so, out_zp=0, trans_b=trans_b)
    keep = B.linear_workspace(torch, d)
    B.int8_linear(d)
    torch.cuda.synchronize()
    assert B.last_variant() == "tcgen05"
    host = buf.cpu().numpy()
    assert (host[0] == 77).all() and (host[-1] == 77).all(), "write outside the output rows"
    del keep
    return host[1:m + 1]


def _fp8_check(what, got, want, a, sa, w, sw, so, dtype=O.E4M3, trans_b=False):
    def bound():
        aa = np.abs(O.fp8_decode(dtype, a).astype(np.float64)) * sa
        ww = np.abs(O.fp8_decode(dtype, w).astype(np.float64)) * sw
        return (aa @ (ww.T if trans_b else ww)) * 2.0 ** -20
    rep = util.fp8_parity_report(got, want, dtype, bound, so)
    rep["case"] = what
    _note(rep)
    assert rep["class_ok"], f"{what}: non-finite classes differ"
    assert rep["failed"] == 0, f"{what}: {rep}"
    return rep


def _slices(m, seed):
    rng = np.random.default_rng(seed)
    cols = np.sort(rng.choice(N, SLICE_COLS, replace=False))
    rows = np.sort(rng.choice(m, min(SLICE_ROWS, m), replace=False))
    return cols, rows


@pytest.mark.parametrize("m", [1, 16, 256, 4096])
def test_c5_fp8_e4m3(cuda, fp8_weight, m):
    w, sw, w_dev = fp8_weight
    a, sa = util.make_fp8_activation(O.E4M3, m, K, seed=100 + m)
    so = util.fp8_out_scale(O.E4M3, K)
    got = _run_fp8(cuda, a, sa, w_dev, sw, so, m, K, N)
    assert B.device_status() == 0
    if m <= 16:
        want = O.fp8_linear(O.OP_MATMUL, O.E4M3, a, sa, w, sw, so)
        rep = _fp8_check(f"C5 fp8_e4m3 M={m} full", got, want, a, sa, w, sw, so)
        if m == 1 and O.have_ref():
            # the reference's own two implementations on the same inputs, for scale
            x86 = O.fp8_linear(O.OP_MATMUL, O.E4M3, a, sa, w, sw, so, impl="ref", device=O.X86)
            ref_rep = util.fp8_parity_report(x86, want, O.E4M3)
            ref_rep["case"] = "C5 fp8_e4m3 M=1 full: reference x86 kernel vs reference Common contract"
            _note(ref_rep)
        assert rep["exact"] + rep["one_code"] + rep["relaxed"] == rep["outputs"]
        return
    cols, rows = _slices(m, seed=m)
    w_cols = np.ascontiguousarray(w[:, cols])
    want = O.fp8_linear(O.OP_MATMUL, O.E4M3, a, sa, w_cols, sw, so)
    _fp8_check(f"C5 fp8_e4m3 M={m}, all rows x {SLICE_COLS} columns", got[:, cols], want, a, sa, w_cols, sw, so)
    a_rows = np.ascontiguousarray(a[rows])
    want = O.fp8_linear(O.OP_MATMUL, O.E4M3, a_rows, sa, w, sw, so)
    _fp8_check(f"C5 fp8_e4m3 M={m}, {len(rows)} rows x all columns", got[rows], want, a_rows, sa, w, sw, so)


@pytest.mark.parametrize("m", [1, 16, 256, 4096])
def test_c5_int8(cuda, int8_weight, m):
    w, ws, w_dev, ws_dev = int8_weight
    a = np.random.default_rng(200 + m).integers(-127, 128, (m, K), dtype=np.int8)
    so = util.int8_out_scale(K, ws)
    got = _run_int8(cuda, a, w_dev, ws_dev, so, m, K, N)
    assert B.device_status() == 0
    if m <= 16:
        want = O.int8_linear(O.OP_MATMUL, a, 0.02, 0, w, ws, None, so, 0)
        bad = int((got != want).sum())
        _note(dict(case=f"C5 int8 M={m} full", outputs=int(want.size), mismatches=bad, saturated=float((np.abs(want.astype(np.int32)) >= 127).mean())))
        assert bad == 0
        return
    cols, rows = _slices(m, seed=m + 1)
    want = O.int8_linear(O.OP_MATMUL, a, 0.02, 0, np.ascontiguousarray(w[:, cols]), ws[cols], None, so, 0)
    bad_c = int((got[:, cols] != want).sum())
    want_r = O.int8_linear(O.OP_MATMUL, np.ascontiguousarray(a[rows]), 0.02, 0, w, ws, None, so, 0)
    bad_r = int((got[rows] != want_r).sum())
    _note(dict(case=f"C5 int8 M={m} slices", outputs=int(want.size + want_r.size), mismatches=bad_c + bad_r))
    assert bad_c == 0 and bad_r == 0


# ---- many work units per CTA ----------------------------------------------------------------------------------------
# The persistent kernels reuse their tensor-memory accumulator buffers and their shared-memory ring from unit to unit;
# the phase bits of those hand-offs flip only from the second pass over the buffers on.  Small K keeps the oracle cheap
# while N is chosen so that every CTA (296 or 148 of them) / CTA pair (74) runs at least 2 x buffers + 1 units.
SWAPPED = [
    # m, k, n, trans_b        tile width, CTAs, buffers -> units per CTA
    (1, 256, 128 * 296 * 5, False),   # 16 wide, 296 CTAs, 4 buffers: 2960 units, 10 per CTA
    (1, 384, 128 * 296 * 3, True),    # [N,K] weights: chunk index fastest; 3 K blocks -> 3 chunks, 9 per CTA
    (32, 256, 128 * 296 * 5, False),  # 32 wide
    (64, 256, 128 * 148 * 3, False),  # 64 wide, 148 CTAs, 2 buffers: 888 units, 6 per CTA
    (128, 384, 128 * 148 * 3, True),  # 128 wide, ring of 6 stages against 2-block / 1-block chunks
]


@pytest.mark.parametrize("m,k,n,trans_b", SWAPPED)
@pytest.mark.parametrize("kind", ["fp8_e5m2", "int8"])
def test_swapped_kernel_many_units_per_cta(cuda, kind, m, k, n, trans_b):
    rng = np.random.default_rng(m * 7 + k)
    if kind == "int8":
        w, ws = util.make_int8_weight(k, n, seed=k + n)
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        so = util.int8_out_scale(k, ws)
        w_host = np.ascontiguousarray(w.T) if trans_b else w
        got = _run_int8(cuda, a, dev(cuda, w_host), dev(cuda, ws), so, m, k, n, trans_b)
        want = O.int8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, a, 0.02, 0, w_host, ws, None, so, 0, trans_b=trans_b)
        assert int((got != want).sum()) == 0
    else:
        w, sw = util.make_fp8_weight(O.E5M2, k, n, seed=k + n)
        a, sa = util.make_fp8_activation(O.E5M2, m, k, seed=m + k)
        so = util.fp8_out_scale(O.E5M2, k)
        w_host = np.ascontiguousarray(w.T) if trans_b else w
        got = _run_fp8(cuda, a, sa, dev(cuda, w_host), sw, so, m, k, n, trans_b, dtype=B.E5M2)
        want = O.fp8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, O.E5M2, a, sa, w_host, sw, so, trans_b=trans_b)
        _fp8_check(f"swapped kernel {kind} {m}x{k}x{n} trans_b={trans_b}", got, want, a, sa, w_host, sw, so, O.E5M2, trans_b)
    assert B.device_status() == 0


# ---- folded split-K: whole tiles per CTA, the chunks added from tensor memory ----------------------------------------
# With about a hundred tiles or more (and M <= 16) the persistent kernel runs as ONE launch: every CTA takes all K chunks of
# a tile into accumulators of their own and adds them in chunk order itself.  A narrower weight still takes the weight-
# streaming pass plus the pass that adds the partial sums from memory; both must give the same bytes for the same columns.
FOLDED = [(1, 1024, 128 * 224, False), (5, 2048, 128 * 130 + 48, False), (16, 1024, 128 * 224, False), (3, 1024, 128 * 200, True)]


def _count_launches(run):
    B.lib().fth_b200_reset_launch_count()
    out = run()
    return out, B.lib().fth_b200_launch_count()


@pytest.mark.parametrize("m,k,n,trans_b", FOLDED)
@pytest.mark.parametrize("kind", ["fp8_e4m3", "int8"])
def test_folded_split_gives_the_reduce_pass_bytes(cuda, kind, m, k, n, trans_b):
    rng = np.random.default_rng(m * 11 + k + n)
    narrow = 128 * 64  # this many columns alone: too few tiles to fold
    op = O.OP_GEMM if trans_b else O.OP_MATMUL
    if kind == "int8":
        w, ws = util.make_int8_weight(k, n, seed=k + n)
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        so = util.int8_out_scale(k, ws)
        layout = (lambda x: np.ascontiguousarray(x.T)) if trans_b else np.ascontiguousarray
        got, launches = _count_launches(lambda: _run_int8(cuda, a, dev(cuda, layout(w)), dev(cuda, ws), so, m, k, n, trans_b))
        part, launches_part = _count_launches(
            lambda: _run_int8(cuda, a, dev(cuda, layout(w[:, :narrow])), dev(cuda, ws[:narrow]), so, m, k, narrow, trans_b))
        want = O.int8_linear(op, a, 0.02, 0, layout(w), ws, None, so, 0, trans_b=trans_b)
        assert int((got != want).sum()) == 0
    else:
        w, sw = util.make_fp8_weight(O.E4M3, k, n, seed=k + n)
        a, sa = util.make_fp8_activation(O.E4M3, m, k, seed=m + k)
        so = util.fp8_out_scale(O.E4M3, k)
        layout = (lambda x: np.ascontiguousarray(x.T)) if trans_b else np.ascontiguousarray
        got, launches = _count_launches(lambda: _run_fp8(cuda, a, sa, dev(cuda, layout(w)), sw, so, m, k, n, trans_b))
        part, launches_part = _count_launches(lambda: _run_fp8(cuda, a, sa, dev(cuda, layout(w[:, :narrow])), sw, so, m, k, narrow, trans_b))
        want = O.fp8_linear(op, O.E4M3, a, sa, layout(w), sw, so, trans_b=trans_b)
        _fp8_check(f"folded split {kind} {m}x{k}x{n} trans_b={trans_b}", got, want, a, sa, layout(w), sw, so, O.E4M3, trans_b)
    assert launches == 1, "expected the folded form: one launch"
    assert launches_part == 2, "expected the weight-streaming pass plus the reduce pass"
    assert np.array_equal(got[:, :narrow], part), "the folded form and the reduce pass disagree"
    assert B.device_status() == 0


# ---- two weight tiles per CTA in the single-launch kernel ------------------------------------------------------------
# A weight with more tiles than one wave of clusters holds, but at most twice as many, runs as one launch in which every
# CTA takes tile t and tile t + half (the N/4 shard of the headline shape is such a weight).  An odd tile count leaves
# the last cluster with one tile.
TWO_TILES = [(1, 8192, 7168, False), (16, 8192, 7168, False), (4, 8192, 7040, False), (1, 4096, 7168, True)]


@pytest.mark.parametrize("m,k,n,trans_b", TWO_TILES)
@pytest.mark.parametrize("kind", ["fp8_e4m3", "int8"])
def test_cluster_kernel_two_tiles_per_cta(cuda, kind, m, k, n, trans_b):
    rng = np.random.default_rng(m * 11 + n)
    B.lib().fth_b200_reset_launch_count()
    if kind == "int8":
        w, ws = util.make_int8_weight(k, n, seed=k + n + 3)
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        so = util.int8_out_scale(k, ws)
        w_host = np.ascontiguousarray(w.T) if trans_b else w
        got = _run_int8(cuda, a, dev(cuda, w_host), dev(cuda, ws), so, m, k, n, trans_b)
        want = O.int8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, a, 0.02, 0, w_host, ws, None, so, 0, trans_b=trans_b)
        assert int((got != want).sum()) == 0
    else:
        w, sw = util.make_fp8_weight(O.E4M3, k, n, seed=k + n + 2)
        a, sa = util.make_fp8_activation(O.E4M3, m, k, seed=m + k + 2)
        so = util.fp8_out_scale(O.E4M3, k)
        w_host = np.ascontiguousarray(w.T) if trans_b else w
        got = _run_fp8(cuda, a, sa, dev(cuda, w_host), sw, so, m, k, n, trans_b)
        want = O.fp8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, O.E4M3, a, sa, w_host, sw, so, trans_b=trans_b)
        _fp8_check(f"two tiles per CTA {kind} {m}x{k}x{n} trans_b={trans_b}", got, want, a, sa, w_host, sw, so, O.E4M3, trans_b)
    assert B.lib().fth_b200_launch_count() == 1, "expected the single-launch kernel"
    assert B.device_status() == 0


PAIR = [
    # m, k, n, trans_b: 256 x 256 tiles on 74 CTA pairs, two accumulator buffers, ring of 6 stages
    (512, 128, 256 * 74 * 3, False),   # 444 tiles, 6 per pair, one K block per tile: the ring wraps once per 6 tiles
    (512, 384, 256 * 74 * 3, True),    # three K blocks per tile: the ring wraps in the middle of tiles
    (300, 640, 256 * 74 * 2 + 48, False),  # ragged rows and columns, five K blocks: stage index and phase drift apart
]


@pytest.mark.parametrize("m,k,n,trans_b", PAIR)
@pytest.mark.parametrize("kind", ["fp8_e4m3", "int8"])
def test_pair_kernel_many_tiles_per_pair(cuda, kind, m, k, n, trans_b):
    rng = np.random.default_rng(m + k + n)
    if kind == "int8":
        w, ws = util.make_int8_weight(k, n, seed=k + n + 1)
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        so = util.int8_out_scale(k, ws)
        w_host = np.ascontiguousarray(w.T) if trans_b else w
        got = _run_int8(cuda, a, dev(cuda, w_host), dev(cuda, ws), so, m, k, n, trans_b)
        want = O.int8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, a, 0.02, 0, w_host, ws, None, so, 0, trans_b=trans_b)
        assert int((got != want).sum()) == 0
    else:
        w, sw = util.make_fp8_weight(O.E4M3, k, n, seed=k + n)
        a, sa = util.make_fp8_activation(O.E4M3, m, k, seed=m + k)
        so = util.fp8_out_scale(O.E4M3, k)
        w_host = np.ascontiguousarray(w.T) if trans_b else w
        got = _run_fp8(cuda, a, sa, dev(cuda, w_host), sw, so, m, k, n, trans_b)
        want = O.fp8_linear(O.OP_GEMM if trans_b else O.OP_MATMUL, O.E4M3, a, sa, w_host, sw, so, trans_b=trans_b)
        _fp8_check(f"pair kernel {kind} {m}x{k}x{n} trans_b={trans_b}", got, want, a, sa, w_host, sw, so, O.E4M3, trans_b)
    assert B.device_status() == 0
