"""The Feather adapter inside the real reference runtime (oracle/_ref/adapter_e2e, built by `make -C oracle refcuda`
from the unmodified reference sources + infer_b200/adapter/b200_candidates.cu + oracle/adapter_e2e.cc).

* CPU: registration and selection contract — kRequireRequested holds, the new candidates are tried first, a
  declined request moves on to the reference's CUDA kernel (never to a CPU kernel), and QuantizeLinear /
  DequantizeLinear gain the CUDA candidates a statically quantised plan needs.
* GPU: the candidates run through the reference's own CUDA runtime (replica cache, inference stream, deferred
  host sync) and are compared with the reference's COMMON kernels on the same tensors; whole plans — the exporter's
  FP8 projection pattern and a model quantised by the reference's own StaticQuantizeModel — are built for CUDA under
  kRequireRequested, rewritten by this backend's GraphPass (infer_b200/adapter/b200_fusion.cu), run in an
  ExecutionSession and compared with the COMMON run of the unfused plan."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "oracle", "_ref", "adapter_e2e")
needs_binary = pytest.mark.skipif(not os.path.exists(EXE), reason="oracle/_ref/adapter_e2e not built (needs a reference checkout)")


def _run(mode):
    proc = subprocess.run([EXE, mode], capture_output=True, text=True, timeout=600)
    print(proc.stdout)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "FAIL" not in proc.stdout
    return proc.stdout


@needs_binary
def test_selection_contract_inside_reference_dispatcher():
    out = _run("select")
    assert out.count("ok  ") >= 16
    # the graph pass, on the host: chains of a plan become fused nodes (and the plan still builds under kRequireRequested)
    assert "FusedCastMatMulCast FusedCastMatMulCast" in out and "Conv2DRelu" in out and "->  FusedQLinearDQ" in out


@needs_binary
@pytest.mark.gpu
def test_candidates_run_through_reference_cuda_runtime():
    out = _run("run")
    assert not any(line.startswith("skip") for line in out.splitlines())
    assert out.count("ok  ") >= 13


@needs_binary
@pytest.mark.gpu
def test_timing_mode_runs_on_both_candidate_sets():
    """`adapter_e2e time` prints microseconds per compute() for the same MatMul nodes with this backend's candidates
    and, with FEATHER_DISABLE_B200=1, with the reference's own CUDA kernels (cuBLASLt FP8 + a quantise kernel; a scalar
    INT8 kernel): the on-box GPU comparator.  The figures are printed, not asserted."""
    ours = _run("time")
    assert "the b200 candidate" in ours and "no kernel" not in ours
    env = dict(os.environ, FEATHER_DISABLE_B200="1")
    proc = subprocess.run([EXE, "time"], capture_output=True, text=True, timeout=600, env=env)
    print(proc.stdout)
    assert proc.returncode == 0 and "the reference CUDA kernel" in proc.stdout and "the b200 candidate" not in proc.stdout


@needs_binary
@pytest.mark.gpu
def test_sharded_nodes_one_process_several_gpus():
    """`adapter_e2e shard`: one CudaExecutionContext per GPU in one process, a column slice of a MatMul node per rank on
    the B200 candidates, gathered through infer_b200/adapter/b200_shard.h; every rank's gathered buffer must equal the
    unsharded node's output.  Needs two GPUs."""
    out = _run("shard")
    if any(line.startswith("skip") for line in out.splitlines()):
        pytest.skip("needs two GPUs")
    assert out.count("ok  ") >= 4
