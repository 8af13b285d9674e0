"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol
include/redline_kernels.h declares. No compute is launched here."""
import ctypes
import os
import re

from redline_llm_b200 import build, kernels

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "redline_kernels.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rl_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert "rl_launch_paged_attention_decode" in names and len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(kernels.ABI_SYMBOLS) <= set(names)
    assert kernels.version() == "0.1.0"


def test_contract_errors_are_reported_without_a_gpu():
    L = kernels.lib()
    # zero extents return at once (src/kernels/rmsnorm.cu:438-440, kv_scatter.cu:151-153)
    assert L.rl_launch_rmsnorm(0, 0, 0, 0, 1536, 1e-6, 0) == 0
    assert L.rl_launch_silu_mul(0, 0, 0, 8960, 0) == 0
    assert L.rl_launch_kv_scatter(0, 0, 0, 0, 0, 0, 0, 0, 0, 2, 128, 0) == 0
    assert L.rl_launch_paged_attention_decode(0, 0, 0, 0, 0, 0, 0, 0, 1, 12, 2, 128, 0.1, 0) == 0
    # contract violations come back as negative codes with a message
    assert L.rl_launch_paged_attention_decode(8, 1536, 8, 1536, 16, 8, 8, 1, 4, 12, 2, 64, 0.1, 0) == -2
    assert b"head_dim" in L.rl_last_error()
    assert L.rl_launch_paged_attention_decode(0, 1536, 8, 1536, 16, 8, 8, 1, 4, 12, 2, 128, 0.1, 0) == -1
    assert L.rl_launch_rope_inplace(8, 8, 1536, 256, 8, 4, 12, 2, 130, 1e6, 0) == -2
