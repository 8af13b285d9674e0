"""The two prefill-only launchers of the contract, through the C ABI. Cases follow the reference's
suite: scatter-then-gather round trip and stride modes (tests/test_kernels.cu:1129-1255), first chunk,
mask boundary with a poisoned masked region, mid-chunk shapes with kv_len > chunk_len, determinism
(:1539-1660). Gather is an exact gate; softmax is held to one FP16 step of the FP64 checker."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host  # noqa: E402


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


# 9601 positions: both kernels move two positions per warp (odd count: the last warp is ragged)
@pytest.mark.parametrize("ctx", [1, 15, 16, 17, 63, 64, 65, 257, 9601])
def test_scatter_then_gather_round_trips_bit_exact(own, ctx):
    nblocks = max(40, (ctx + 15) // 16 + 8)
    k = wl.uniform_half(0x6A1 + ctx, ctx * 256, -1.0, 1.0).reshape(ctx, 256)
    v = wl.uniform_half(0x6B1 + ctx, ctx * 256, -1.0, 1.0).reshape(ctx, 256)
    row = (wl.permutation(0x6C1 + ctx, nblocks - 1)[:(ctx + 15) // 16] + 1).astype(np.int32)
    n = nblocks * 2 * 2 * 16 * 128
    d_pool = dev(np.full(n, 0x7E00, np.uint16))
    d_row = dev(row)
    K.launch_kv_scatter(d_pool, dev(k), dev(v), 256, 256, d_row.view(1, -1), 0, dev(np.arange(ctx, dtype=np.int32)), ctx, 2, 128)
    d_k = torch.zeros(2, ctx, 128, dtype=torch.int16, device="cuda")
    d_v = torch.zeros(2, ctx, 128, dtype=torch.int16, device="cuda")
    K.launch_kv_gather(d_k, d_v, ctx * 128, 128, ctx * 128, 128, d_pool, d_row, ctx, 2, 128)
    assert np.array_equal(host(d_k), k.reshape(ctx, 2, 128).transpose(1, 0, 2))
    assert np.array_equal(host(d_v), v.reshape(ctx, 2, 128).transpose(1, 0, 2))


@pytest.mark.parametrize("head_stride,row_stride,shift", [(300 * 128, 128, 0), (300 * 136, 136, 0), (300 * 133, 133, 0), (300 * 128, 128, 1)])
def test_gather_matches_cpu_mirror_across_stride_modes(own, head_stride, row_stride, shift):
    ctx = 257
    a = wl.config_attention(lens=[ctx], num_blocks=40, seed=0x6A7, fill="uniform")
    total = 2 * head_stride
    sent = wl.uniform_half(0x6A8, total + shift + 8, -1.0, 1.0)
    d_k, d_v = dev(sent), dev(sent)
    L = K.lib()
    st = L.rl_launch_kv_gather(d_k.data_ptr() + 2 * shift, d_v.data_ptr() + 2 * shift, head_stride, row_stride,
                               head_stride, row_stride, dev(a["pool"]).data_ptr(), dev(a["tables"][0]).data_ptr(),
                               ctx, 2, 128, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    mk, mv = sent.copy(), sent.copy()
    own.kv_gather(mk[shift:], mv[shift:], head_stride, row_stride, a["pool"], a["tables"][0], ctx, 2, 128)
    # full-buffer equality: gathered rows exact and every gap / tail untouched
    assert np.array_equal(host(d_k), mk) and np.array_equal(host(d_v), mv)


def run_softmax(scores, chunk_start):
    h, c, kv = scores.shape
    d_p = torch.full((h, c, kv), 0x1234, dtype=torch.int16, device="cuda")
    K.launch_prefill_softmax(d_p, torch.from_numpy(scores).cuda(), h, c, kv, chunk_start)
    return host(d_p)


# the last six shapes take the read-once kernel's five tiers (kv_len a multiple of 8, up to 32768 keys), one
# of them with the causal limit in the middle of the row; the others take the three-pass kernel
@pytest.mark.parametrize("h,c,kv,start", [(12, 8, 8, 0), (12, 17, 300, 283), (2, 1, 1, 0), (3, 64, 2049, 1985), (12, 5, 33000, 32995),
                                          (4, 9, 2048, 2039), (3, 21, 2056, 997), (2, 5, 4096, 4091), (2, 3, 8192, 8189),
                                          (2, 3, 16384, 16381), (1, 2, 32768, 32766)])
def test_prefill_softmax_against_fp64_with_poisoned_masked_region(own, h, c, kv, start):
    rng = np.random.default_rng(h * 1000 + c)
    sc = rng.normal(0, 2.5, (h, c, kv)).astype(np.float32)
    for i in range(c):
        sc[:, i, start + i + 1:] = np.nan      # masked scores must never be read
    got = run_softmax(sc, start)
    ref = own.prefill_softmax(sc, start)
    for i in range(c):
        assert (got[:, i, start + i + 1:] == 0).all(), "masked entries must be exact +0"
    assert not ((got & 0x7FFF) > 0x7C00).any()
    assert oracle.ulp_distance(got, ref).max() <= 1
    assert (got == ref).mean() > 0.99
    if start == 0:
        assert (got[:, 0, 0] == 0x3C00).all()  # the first row attends to itself only: exactly 1.0
    assert np.array_equal(run_softmax(sc, start), got)  # run-to-run identical bits
