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
