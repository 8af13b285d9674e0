"""Builds and runs tests/cpp/kernel_contract_check.cu: a C++ host that calls the launchers through the
drop-in header with the reference's signatures (redline::kernels::Launch*) and links libredline_b200.so."""
import os
import subprocess

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "redline_llm_b200")


def test_cpp_caller_through_the_reference_signatures(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from redline_llm_b200 import build
    lib = build.build()
    exe = str(tmp_path / "kernel_contract_check")
    cmd = ["/usr/local/cuda/bin/nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-cudart", "shared",
           "-I", os.path.join(PKG, "csrc"), "-o", exe, os.path.join(ROOT, "tests", "cpp", "kernel_contract_check.cu"),
           lib, "-Xlinker", f"-rpath,{PKG}", "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "all checks passed" in r.stdout
