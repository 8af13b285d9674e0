"""This library's kernels against the reference's OWN CUDA kernels on the same B200, same device buffers.

oracle/_ref/libredline_refkernels.so is the reference's src/kernels/*.cu compiled for sm_100a where they lie
(make -C oracle gpuref). The CPU checker in oracle/ stays the arbiter of every tolerance; this file adds
the statement a user of the reference cares about: swapping the kernel library changes results by nothing
where the operation is a bit move or FP32 elementwise math with the same rounding points, by at most one
FP16 step where a reduction order differs, and by at most the attention gate for attention."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from oracle import ref_kernels as R  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host  # noqa: E402


@pytest.fixture(scope="module", autouse=True)
def _need():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not R.available():
        pytest.skip("oracle/_ref/libredline_refkernels.so (the reference's CUDA kernels) was never built")
    K.init()


def both(fn):
    """fn(module) -> numpy result, for this library and for the reference's kernels."""
    a = fn(K)
    b = fn(R)
    torch.cuda.synchronize()
    return a, b


@pytest.mark.parametrize("rows", [1, 64, 257, 2048])
def test_fused_rmsnorm_residual(rows):
    c = wl.config_rmsnorm(64)
    x, r = np.tile(c["x"], (rows // 64 + 1, 1))[:rows], np.tile(c["residual"], (rows // 64 + 1, 1))[:rows]

    def run(M):
        d_res, d_out = dev(r), torch.zeros(rows, 1536, dtype=torch.int16, device="cuda")
        M.launch_rms_norm_residual(d_out, d_res, dev(x), dev(c["weight"]), rows, 1536, 1e-6)
        return host(d_out), host(d_res)
    (o1, r1), (o2, r2) = both(run)
    assert np.array_equal(r1, r2), "residual write-back differs from the reference kernel"
    d = oracle.ulp_distance(o1, o2)
    # only sum_sq's FP32 summation order differs; it reaches the output through inv_rms alone
    assert d.max() <= 1 and (d == 0).mean() > 0.995, (d.max(), (d == 0).mean())


@pytest.mark.parametrize("rows", [1, 64, 300])
def test_plain_rmsnorm(rows):
    c = wl.config_rmsnorm(64)
    x = np.tile(c["x"], (rows // 64 + 1, 1))[:rows]

    def run(M):
        d_out = torch.zeros(rows, 1536, dtype=torch.int16, device="cuda")
        M.launch_rms_norm(d_out, dev(x), dev(c["weight"]), rows, 1536, 1e-6)
        return host(d_out)
    o1, o2 = both(run)
    d = oracle.ulp_distance(o1, o2)
    assert d.max() <= 1 and (d == 0).mean() > 0.995


@pytest.mark.parametrize("tokens", [1, 64, 777])
def test_rope_and_scatter(tokens):
    c = wl.config_rope_scatter(tokens if tokens <= 64 else 64)
    reps = tokens // 64 + 1
    qkv = np.tile(c["qkv"], (reps, 1))[:tokens]
    pos = wl.randint(0x40BE + tokens, tokens, 0, 4095)
    # every token writes through a distinct block: a permutation of 1..8191 dealt one per token
    tables = np.zeros((tokens, 256), np.int32)
    tables[np.arange(tokens), pos // 16] = (wl.permutation(0x40BF + tokens, 8191)[:tokens] + 1)

    def run(M):
        d_qkv, d_pos, d_tab = dev(qkv), dev(pos), dev(tables)
        d_pool = torch.full((8192 * 2 * 2 * 16 * 128,), 0x7E01, dtype=torch.int16, device="cuda")
        M.launch_rope_inplace(d_qkv, d_qkv, 2048, 2048, d_pos, tokens, 12, 2, 128, 1e6, k_offset=1536)
        M.launch_kv_scatter(d_pool, d_qkv, d_qkv, 2048, 2048, d_tab, 256, d_pos, tokens, 2, 128,
                            k_offset=1536, v_offset=1792)
        return host(d_qkv), host(d_pool)
    (q1, p1), (q2, p2) = both(run)
    assert np.array_equal(q1, q2), "RoPE differs from the reference kernel (same FP32 steps, same rounding points)"
    assert np.array_equal(p1, p2), "the scattered pool differs from the reference kernel's"


def test_fused_rope_scatter_equals_the_reference_pair():
    c = wl.config_rope_scatter(64)
    d_tab, d_pos = dev(c["tables"]), dev(c["positions"])
    a_qkv, b_qkv = dev(c["qkv"]), dev(c["qkv"])
    a_pool = torch.full((8192 * 2 * 2 * 16 * 128,), 0x7E01, dtype=torch.int16, device="cuda")
    b_pool = a_pool.clone()
    K.launch_rope_kv_scatter(a_qkv, 2048, a_pool, d_tab, 256, d_pos, 64, 12, 2, 128, 1e6)
    R.launch_rope_inplace(b_qkv, b_qkv, 2048, 2048, d_pos, 64, 12, 2, 128, 1e6, k_offset=1536)
    R.launch_kv_scatter(b_pool, b_qkv, b_qkv, 2048, 2048, d_tab, 256, d_pos, 64, 2, 128, k_offset=1536, v_offset=1792)
    assert torch.equal(a_qkv, b_qkv) and torch.equal(a_pool, b_pool)


@pytest.mark.parametrize("tokens,inplace", [(64, True), (512, False), (4096, True)])
def test_silu_mul(tokens, inplace):
    g = np.tile(wl.config_silu(64)["gate_up"], (tokens // 64, 1))

    def run(M):
        d_g = dev(g)
        d_o = d_g if inplace else torch.zeros(tokens, 8960, dtype=torch.int16, device="cuda")
        M.launch_silu_mul(d_o, d_g, tokens, 8960)
        return host(d_o)[:, :8960].copy()
    o1, o2 = both(run)
    assert np.array_equal(o1, o2), "SiLU*mul differs from the reference kernel"


@pytest.mark.parametrize("lens", [None, [4095, 4096, 4097, 1, 0, 16, 8192, 33]])
def test_paged_attention(lens):
    c = wl.config_attention() if lens is None else wl.config_attention(lens=lens, num_blocks=1400, seed=0xA77E)
    n = len(c["seq_lens"])

    def run(M):
        d_out = torch.full((n, 1536), 0x1234, dtype=torch.int16, device="cuda")
        M.launch_paged_attention_decode(d_out, 1536, dev(c["q"]), 1536, dev(c["pool"]), dev(c["tables"]),
                                        dev(c["seq_lens"]), n, c["tables"].shape[1], 12, 2, 128, c["scale"])
        return host(d_out)
    o1, o2 = both(run)
    live = np.asarray(c["seq_lens"]) > 0
    assert np.array_equal(o1[~live], o2[~live]) and (o1[~live] == 0x1234).all()   # padded rows untouched by both
    err = np.abs(oracle.half_bits_to_f64(o1[live]) - oracle.half_bits_to_f64(o2[live]))
    assert err.max() <= 2e-3, err.max()
    assert K.attention_health() == 0


def test_argmax_embed_gather_kv_gather_are_exact():
    lg = wl.normal_half(0xA46, 64 * 151936).reshape(64, 151936)
    lg[3, 100] = lg[3, 90000] = 0x7BFF       # a tie: lowest index wins
    lg[5, :] = 0x7E00                         # all NaN
    t1, t2 = both(lambda M: (lambda t: (M.launch_greedy_argmax(t, dev(lg), 64, 151936), t.cpu().numpy())[1])(
        torch.zeros(64, dtype=torch.int32, device="cuda")))
    assert np.array_equal(t1, t2) and t1[3] == 100
    table = dev(wl.normal_half(0xE1, 4096 * 1536).reshape(4096, 1536))
    ids = dev(wl.randint(0xE2, 64, 0, 4095))
    e1, e2 = both(lambda M: (lambda o: (M.launch_embed_gather(o, 1536, table, ids, 64, 1536), host(o))[1])(
        torch.zeros(64, 1536, dtype=torch.int16, device="cuda")))
    assert np.array_equal(e1, e2)
    ctx = 1000
    pool = dev(wl.normal_half(0x2B4, 128 * 2 * 2 * 16 * 128))
    row = dev((wl.permutation(0x2B3, 127)[:(ctx + 15) // 16] + 1).astype(np.int32))

    def gather(M):
        kh = torch.zeros(2, ctx, 128, dtype=torch.int16, device="cuda")
        vh = torch.zeros(2, ctx, 128, dtype=torch.int16, device="cuda")
        M.launch_kv_gather(kh, vh, ctx * 128, 128, ctx * 128, 128, pool, row, ctx, 2, 128)
        return host(kh), host(vh)
    (k1, v1), (k2, v2) = both(gather)
    assert np.array_equal(k1, k2) and np.array_equal(v1, v2)


def test_prefill_softmax_within_one_step():
    h, c, kv, start = 12, 64, 1024, 960
    sc = torch.randn(h, c, kv, dtype=torch.float32, device="cuda", generator=torch.Generator("cuda").manual_seed(7)) * 2.5

    def run(M):
        pr = torch.zeros(h, c, kv, dtype=torch.int16, device="cuda")
        M.launch_prefill_softmax(pr, sc, h, c, kv, start)
        return host(pr)
    p1, p2 = both(run)
    d = oracle.ulp_distance(p1, p2)
    assert d.max() <= 1 and (d == 0).mean() > 0.99
