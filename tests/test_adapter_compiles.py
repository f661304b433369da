"""CPU: the Feather-side adapter (infer_b200/adapter/b200_candidates.cu) compiles against the unmodified
reference headers.  Needs a reference checkout (FEATHER_REFERENCE or /root/reference); skipped without one."""
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("FEATHER_REFERENCE", "/root/reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src", "kernel", "cuda")), reason="no reference checkout here")
@pytest.mark.parametrize("source,symbol", [("b200_candidates.cu", "feather::kernel::b200::RegisterB200Kernels()"),
                                           ("b200_fusion.cu", "feather::kernel::b200::CreateB200FusionPass()")])
def test_adapter_compiles_against_reference_headers(source, symbol):
    with tempfile.TemporaryDirectory() as tmp:
        cmd = ["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O0", "-arch=sm_100", "-DFEATHER_WITH_CUDA", "-DFEATHER_WITH_X86",
               "-DFEATHER_WITH_OPENMP", "-DFEATHER_WITH_CUBLASLT", "-DFEATHER_WITH_CUDNN", f"-I{REF}/include", f"-I{REF}",
               f"-I{ROOT}/include", "-Xcompiler", "-fopenmp", "-w", "-c",
               os.path.join(ROOT, "infer_b200", "adapter", source), "-o", os.path.join(tmp, "adapter.o")]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        assert proc.returncode == 0, proc.stderr[-3000:]
        syms = subprocess.check_output(["nm", "-C", os.path.join(tmp, "adapter.o")], text=True)
        assert symbol in syms
