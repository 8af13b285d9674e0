"""The allocation-free attention entry point, through the C ABI, against the allocating one.

Some callers of this library cannot call cudaMalloc (a process whose device-memory budget is sealed
at start-up, a plugin inside a host that forbids allocation once serving has begun). For them
rl_launch_paged_attention_decode_static keeps its scratch in an array inside the library. This file
is collected last on purpose: if it fails, a stop-at-first-failure run has already run everything else.
It passes alone in a fresh process (the static variant then does its own first-call set-up) and after
the other tests (the allocating launcher's workspace already exists)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host  # noqa: E402


def run(entry, c, sentinel):
    s = len(c["seq_lens"])
    d_out = torch.full((s, 1536), sentinel, dtype=torch.int16, device="cuda")
    entry(d_out, 1536, dev(c["q"]), 1536, dev(c["pool"]), dev(c["tables"]), dev(c["seq_lens"]), s,
          c["tables"].shape[1], 12, 2, 128, c["scale"])
    torch.cuda.synchronize()
    return host(d_out)


def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    # two different batches back to back: the second call meets the first call's leftovers in the array
    cases = [wl.config_attention(lens=[257, 0, 64, 1, 17, 4100, 63, 65, 9000], num_blocks=900, seed=0x5747),
             wl.config_attention(batch=64, lo=900, hi=1400, num_blocks=6000, seed=0x5748)]
    for i, c in enumerate(cases):
        static = run(K.launch_paged_attention_decode_static, c, 0x1234 + i)
        normal = run(K.launch_paged_attention_decode, c, 0x1234 + i)
        # same kernel, same fixed merge order: bit-identical, padded rows untouched in both
        assert np.array_equal(static, normal), f"call {i}: static-scratch result differs"
        pad = np.asarray(c["seq_lens"]) <= 0
        assert (static[pad] == 0x1234 + i).all()
    # and once more on the first batch: results do not depend on what the array held
    again = run(K.launch_paged_attention_decode_static, cases[0], 0x1234)
    assert np.array_equal(again, run(K.launch_paged_attention_decode, cases[0], 0x1234))
    # straight against the CPU checker too (FP64, unrounded), at the attention gate
    c = cases[0]
    lens = np.asarray(c["seq_lens"])
    ref = oracle.own().paged_attention(c["q"], c["pool"], c["tables"], lens, 12, 2, 128, c["scale"], f64out=True)
    err = np.abs(oracle.half_bits_to_f64(again)[lens > 0] - ref[lens > 0])
    assert err.max() <= 2e-3 + 2.0 ** -11, err.max()
    # no bounded wait gave up in either scratch area (the query covers the built-in array as well)
    assert K.attention_health() == 0


def test_static_scratch_entry_allocates_no_device_memory():
    """In a fresh process, where the static entry point does its own first-call set-up, the device's free
    memory is the same before and after the call: nothing was allocated on its behalf. (The inputs are
    allocated beforehand, and the CUDA context and the library's code are already resident.)"""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import subprocess
    import sys
    code = """
import sys
sys.path.insert(0, %r)
import torch
from redline_llm_b200 import kernels as K, workloads as wl
from tests.gpu_util import dev
torch.cuda.init(); torch.zeros(1, device="cuda")
c = wl.config_attention(lens=[300, 17, 5000, 64], num_blocks=500, seed=0x5749)
args = (torch.zeros(4, 1536, dtype=torch.int16, device="cuda"), 1536, dev(c["q"]), 1536, dev(c["pool"]), dev(c["tables"]),
        dev(c["seq_lens"]), 4, c["tables"].shape[1], 12, 2, 128, c["scale"])
K.lib()                                   # load the library (its device code and the array come with it)
def free_bytes():
    return torch.cuda.mem_get_info()[0]       # cudaMemGetInfo
torch.cuda.synchronize()
before = free_bytes()
K.launch_paged_attention_decode_static(*args)
torch.cuda.synchronize()
first = free_bytes()
K.launch_paged_attention_decode_static(*args)
torch.cuda.synchronize()
second = free_bytes()
print("FREE", before, first, second)
""" % (__import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__))),)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    before, first, second = [int(x) for x in r.stdout.strip().splitlines()[-1].split()[1:]]
    # A lazily loaded module may claim its image on the very first launch of any kernel of the library; the
    # steady state must be flat, and the first call may not take more than that image (a few MB at most).
    assert second == first, (before, first, second)
    assert before - first <= 8 << 20, (before, first, second)


def test_static_scratch_entry_rejects_more_than_its_maximum():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    n = 1025
    z16 = torch.zeros(n, 1536, dtype=torch.int16, device="cuda")
    pool = torch.zeros(4 * 2 * 2 * 16 * 128, dtype=torch.int16, device="cuda")
    tab = torch.zeros(n, 1, dtype=torch.int32, device="cuda")
    lens = torch.zeros(n, dtype=torch.int32, device="cuda")
    with pytest.raises(K.KernelError, match="at most 1024"):
        K.launch_paged_attention_decode_static(z16, 1536, z16, 1536, pool, tab, lens, n, 1, 12, 2, 128, 0.088)
