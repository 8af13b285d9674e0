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


def test_reference_side_comparators_load_where_they_were_built():
    """oracle/_ref holds, where the reference tree was mounted at build time: the reference's CUDA kernels
    behind a C ABI, and the reference's own C++ host (its pybind module) linked once to this library and
    once to its own kernels. Without a GPU they must still load and resolve every symbol; the host module
    must fail a missing model directory with the binding's RuntimeError, before touching CUDA."""
    import subprocess
    import sys

    import pytest

    from oracle import ref_kernels as R
    if not R.available():
        pytest.skip("oracle/_ref was built without the reference tree")
    lib = ctypes.CDLL(R.LIB_PATH)
    for n in R.SYMBOLS:
        assert hasattr(lib, n), n
    for d in (R.HOST_B200_DIR, R.HOST_REF_DIR):
        code = ("import sys; sys.path.insert(0, %r); import redline\n"
                "assert redline.__version__ == '0.1.0'\n"
                "for m in ('add_request', 'step', 'has_capacity', 'stats'): assert hasattr(redline.Engine, m)\n"
                "try:\n    redline.Engine('/nonexistent-model-dir')\nexcept RuntimeError as e:\n    print('RuntimeError', e)\n") % d
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "RuntimeError" in r.stdout, (d, r.stdout, r.stderr[-2000:])


def test_checkpoint_writer_produces_a_well_formed_safetensors_file(tmp_path):
    """tests/ref_host.py writes the checkpoint the reference's loader reads; here its container format is
    checked on a miniature model (header length, JSON, contiguous offsets, names of docs/MODEL_SPEC.md:182-199)."""
    import json
    import struct

    import torch

    from redline_llm_b200.engine import ModelConfig, ModelWeights
    from tests import ref_host
    cfg = ModelConfig(layers=2, hidden=64, inter=96, q_heads=2, kv_heads=1, head_dim=32, vocab=50)
    w = ModelWeights(cfg, torch.device("cpu"), seed=3)
    d = ref_host.write_model_dir(str(tmp_path), cfg, w)
    raw = open(os.path.join(d, "model.safetensors"), "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    assert hdr.pop("__metadata__") == {"format": "pt"} and len(hdr) == 2 + 12 * cfg.layers and n % 8 == 0
    end = 0
    for name, e in hdr.items():
        assert e["dtype"] == "F16" and e["data_offsets"][0] == end
        end = e["data_offsets"][1]
        assert end - e["data_offsets"][0] == 2 * int(torch.tensor(e["shape"]).prod())
    assert len(raw) == 8 + n + end
    q = hdr["model.layers.1.self_attn.q_proj.weight"]
    got = torch.frombuffer(bytearray(raw[8 + n + q["data_offsets"][0]:8 + n + q["data_offsets"][1]]), dtype=torch.float16)
    assert torch.equal(got.view(64, 64), w.layers[1]["qkv"][:64])
    assert hdr["model.layers.0.mlp.up_proj.weight"]["shape"] == [96, 64]
    assert json.load(open(os.path.join(d, "config.json")))["torch_dtype"] == "bfloat16"


def test_prefill_run_length_is_chosen_by_a_replay_of_the_launch():
    """Host arithmetic of the prefill attention launcher, no device: the longest run of 128-key blocks per CTA
    comes from replaying the launch (items in grid order, each onto the SM that frees first) over candidate
    run lengths. Shapes whose measured optimum is known on a 148-SM device pin the model."""
    run = kernels.prefill_attention_run_length
    # 2048 rows at context 8192: 16 tiles of 49-64 blocks x 12 heads = 192 items in two waves when whole;
    # cutting only the longest tiles (runs of at most 56-60 blocks) levels them - measured 120 against 136 us
    assert 56 <= run(6144, 2048, 12, 148) <= 60
    # a prompt's last 128 rows against 32768 keys: 12 pairs of 256 blocks, cut into a dozen runs each
    assert 16 <= run(32640, 128, 12, 148) <= 32
    # the first rows of a prompt and chunks that fill the machine many times over are left whole
    assert run(0, 128, 12, 148) == 1
    assert run(0, 2048, 12, 148) == 16
    assert run(8192, 8192, 12, 148) == 128
    for start, n in ((0, 1), (5, 123), (1000, 257), (31744, 1024), (16384, 4096), (100000, 300)):
        r = run(start, n, 12, 148)
        assert 1 <= r <= (start + n - 1) // 128 + 1
        assert r == run(start, n, 12, 148), "the choice is a pure function of the chunk"
    # fewer SMs, fewer cuts: one SM never cuts anything
    assert run(6144, 2048, 12, 1) == 64
    L = kernels.lib()
    out = ctypes.c_int32(0)
    assert L.rl_prefill_attention_run_length(0, 0, 12, 148, ctypes.byref(out)) == -2
