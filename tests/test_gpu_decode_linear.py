"""GPU parity of the decode-sized linear layer (tcgen05 weight-streaming kernel), through the C ABI.

The reference runs these products through cuBLASLt (src/gemm/cublaslt_gemm.cpp:569-598) and gates
its GEMM wrapper against an FP64 host product. Here: every output is the FP64 product of the same
FP16 inputs rounded to FP16, up to the error of an FP32 accumulation (2^-20 of sum |x.w|, which only
shows where the sum cancels to almost nothing); rows and columns outside the problem are untouched;
results do not depend on the ring depth or on launch overlap; and the fused SiLU-mul epilogue is
bit-identical to the stand-alone SiLU kernel applied to the stored (unsplit) product."""
import functools

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host, ulp_of  # noqa: E402

SEED = 0xB200C0DE


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    K.init()
    yield
    K.set_decode_linear_stages(6)
    assert K.decode_linear_health() == 0


def f64(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float64)


@functools.lru_cache(maxsize=4)
def weights(N, Kd, scale):
    return wl.normal_half(SEED + 3 * N + Kd, N * Kd, 0.0, scale).reshape(N, Kd)


def vector(seed, n):
    return wl.normal_half(seed, n)


def make(seed, T, N, Kd, scale=None):
    """x [T, Kd] ~ N(0,1) per seed; W [N, Kd] ~ N(0, scale) per shape (products stay O(1) by default)."""
    x = wl.normal_half(seed, T * Kd).reshape(T, Kd)
    return x, weights(N, Kd, scale if scale is not None else Kd ** -0.5)


def run(x, w, T, N, bias=None, epilogue=0, out_stride=None, x_stride=None):
    """x, w: uint16 bit patterns. Returns the [64, N] output buffer (rows >= T keep the 0x7E00 fill)."""
    Kd = x.shape[1]
    xd = torch.zeros(64, x_stride or Kd, dtype=torch.int16, device="cuda")
    xd[:T, :Kd] = dev(x)
    wd = dev(w)
    bd = dev(bias) if bias is not None else None
    out = torch.full((64, out_stride or N), 0x7E00, dtype=torch.int16, device="cuda")
    K.launch_decode_linear(out[:, :N], xd[:, :Kd], wd, bd, num_tokens=T, epilogue=epilogue)
    torch.cuda.synchronize()
    return host(out)


def check_product(got, x, w, T, bias=None):
    """|got - fp64| <= half an FP16 step (one rounding) + 2^-20 * sum |x.w| (FP32 accumulation in the
    tensor core, up to 560 dependent steps for in_features = 8960; the library GEMM needs more).
    Returns the fraction of outputs that are the FP16 value nearest to the FP64 product."""
    xf, wf = f64(x[:T]), f64(w)
    ref = xf @ wf.T
    if bias is not None:
        ref = ref + f64(bias)[None, :]
    g = f64(got[:T])
    assert np.isfinite(g).all()
    err = np.abs(g - ref)
    step = ulp_of(np.maximum(np.abs(ref), np.abs(g)))
    allowance = 2.0 ** -20 * (np.abs(xf) @ np.abs(wf).T)
    bad = err > 0.5 * step * 1.0001 + allowance
    assert not bad.any(), f"{int(bad.sum())} outputs outside the gate (max {(err / step).max():.2f} FP16 steps)"
    return float((err <= 0.5 * ulp_of(ref) * 1.0001).mean())


# the four linear layers of a Qwen2.5-1.5B block, then shapes that leave partial tiles and k-blocks
MODEL_SHAPES = [(2048, 1536, True), (1536, 1536, False), (17920, 1536, False), (1536, 8960, False)]
ODD_SHAPES = [(128, 64, False), (136, 72, True), (1000, 520, False), (264, 8, True), (1536, 2056, True)]


@pytest.mark.parametrize("N,Kd,with_bias", MODEL_SHAPES + ODD_SHAPES)
@pytest.mark.parametrize("T", [1, 3, 16, 17, 33, 48, 64])
def test_product_within_one_step_of_fp64(N, Kd, with_bias, T):
    x, w = make(SEED + N + Kd + T, T, N, Kd)
    bias = vector(SEED + 7, N) if with_bias else None
    got = run(x, w, T, N, bias)
    nearest = check_product(got, x, w, T, bias)
    assert nearest > 0.98, f"only {nearest:.5f} of the outputs are the nearest FP16 value"  # near-ties and tiny sums
    assert (got[T:] == 0x7E00).all(), "rows past num_tokens were written"


@pytest.mark.parametrize("T", [5, 64])
def test_many_row_tiles_take_the_short_ring(T):
    """A vocabulary-sized output (57 000 rows: 446 row tiles, three times the SM count, the last one
    partial) runs with the short ring and several CTAs per SM; same gate as every other shape."""
    N, Kd = 57000, 264
    x, w = make(SEED + N + T, T, N, Kd)
    got = run(x, w, T, N)
    assert check_product(got, x, w, T) > 0.98
    assert (got[T:] == 0x7E00).all()
    assert K.decode_linear_health() == 0


def test_strided_views_and_untouched_columns():
    # the engine's qkv buffer: out rows 2048 wide inside a wider allocation, x rows padded
    T, N, Kd = 64, 2048, 1536
    x, w = make(SEED + 11, T, N, Kd)
    bias = vector(SEED + 12, N)
    got = run(x, w, T, N, bias, out_stride=2304, x_stride=1600)
    check_product(got[:, :N], x, w, T, bias)
    assert (got[:, N:] == 0x7E00).all(), "columns past out_features were written"
    # out rows that are not 16-byte aligned take the scalar store path
    T, N, Kd = 17, 1000, 520
    x, w = make(SEED + 13, T, N, Kd)
    got = run(x, w, T, N, out_stride=1004)
    check_product(got[:, :N], x, w, T)
    assert (got[:, N:] == 0x7E00).all()


@pytest.mark.parametrize("T", [1, 17, 64])
def test_fused_silu_mul_is_bit_identical_to_the_two_step_path(T):
    I, Kd = 8960, 1536
    x, w = make(SEED + 21 + T, T, 2 * I, Kd, scale=0.05)
    fused = run(x, w, T, I, epilogue=K.EPILOGUE_SILU_MUL)
    gate_up = run(x, w, T, 2 * I)                       # the stored product, then the stand-alone SiLU kernel
    gu = dev(gate_up[:T])
    out = torch.zeros(T, I, dtype=torch.int16, device="cuda")
    K.launch_silu_mul(out, gu, T, I)
    torch.cuda.synchronize()
    assert np.array_equal(fused[:T], host(out)), "fused epilogue differs from GEMM + SiLU kernel"
    assert (fused[T:] == 0x7E00).all()
    # odd intermediate size: partial last tile of gate and up rows. The fused product is never split
    # along K, so the stored product it is compared with is made without splits too.
    I2 = 1000
    x2, w2 = make(SEED + 31 + T, T, 2 * I2, 520, scale=0.05)
    fused2 = run(x2, w2, T, I2, epilogue=K.EPILOGUE_SILU_MUL)
    K.set_decode_linear_max_splits(1)
    try:
        gu2 = dev(run(x2, w2, T, 2 * I2)[:T])
    finally:
        K.set_decode_linear_max_splits(8)
    out2 = torch.zeros(T, I2, dtype=torch.int16, device="cuda")
    K.launch_silu_mul(out2, gu2, T, I2)
    torch.cuda.synchronize()
    assert np.array_equal(fused2[:T], host(out2))


@pytest.mark.parametrize("T", [1, 7, 33, 64])
def test_qkv_with_rope_and_scatter_in_the_epilogue_is_bit_identical_to_three_launches(T):
    """Config-2 inputs (positions U[0,4096), permuted block tables, 8192-block pool slice) behind a QKV
    product: the fused launch leaves the qkv buffer and the pool exactly as GEMM -> RoPE + scatter do."""
    q_heads, kv_heads, D, H = 12, 2, 128, 1536
    N = (q_heads + 2 * kv_heads) * D
    c = wl.config_rope_scatter(64)
    pos, tab = dev(c["positions"][:T].copy()), dev(c["tables"][:T].copy())
    mbps = c["tables"].shape[1]
    x, w = make(SEED + 71 + T, T, N, H)
    bias = vector(SEED + 72, N)
    xd, wd, bd = dev(x), dev(w), dev(bias)
    pool_elems = c["num_blocks"] * 2 * kv_heads * 16 * D

    def three_launches():
        qkv = torch.full((64, N), 0x7E00, dtype=torch.int16, device="cuda")
        pool = torch.full((pool_elems,), 0x7D01, dtype=torch.int16, device="cuda")
        K.launch_decode_linear(qkv, xd, wd, bd, num_tokens=T)
        K.launch_rope_kv_scatter(qkv, N, pool, tab, mbps, pos, T, q_heads, kv_heads, D, 1e6)
        torch.cuda.synchronize()
        return host(qkv), host(pool)

    def fused():
        qkv = torch.full((64, N), 0x7E00, dtype=torch.int16, device="cuda")
        pool = torch.full((pool_elems,), 0x7D01, dtype=torch.int16, device="cuda")
        K.launch_qkv_rope_kv_scatter(qkv, xd, wd, bd, pool, tab, mbps, pos, T, q_heads, kv_heads, D, 1e6)
        torch.cuda.synchronize()
        return host(qkv), host(pool)

    want_qkv, want_pool = three_launches()
    got_qkv, got_pool = fused()
    assert np.array_equal(got_qkv, want_qkv), "qkv buffer differs"
    assert np.array_equal(got_pool, want_pool), "pool differs"
    assert (got_qkv[T:] == 0x7E00).all()
    assert int((got_pool != 0x7D01).sum()) <= T * 2 * kv_heads * D   # only the T tokens' K and V cells
    # with splitting capped at 1 the entry point takes the three-launch route itself
    K.set_decode_linear_max_splits(1)
    try:
        ref1_qkv, ref1_pool = three_launches()
        one_qkv, one_pool = fused()
    finally:
        K.set_decode_linear_max_splits(8)
    assert np.array_equal(one_qkv, ref1_qkv) and np.array_equal(one_pool, ref1_pool)
    assert K.decode_linear_health() == 0


def test_ring_depth_and_overlap_change_no_bit():
    cases = [(64, 1536, 8960, False), (33, 2048, 1536, True), (64, 17920, 1536, False)]
    try:
        for T, N, Kd, with_bias in cases:
            x, w = make(SEED + 41 + N, T, N, Kd)
            bias = vector(SEED + 42, N) if with_bias else None
            base = None
            for stages in (2, 4, 7, 8):
                for overlap in (False, True):
                    K.set_decode_linear_stages(stages)
                    K.set_attention_prologue_overlap(overlap)
                    got = run(x, w, T, N, bias)
                    if base is None:
                        base = got
                    assert np.array_equal(got, base), f"stages={stages} overlap={overlap} changed the result"
    finally:
        K.set_decode_linear_stages(6)
        K.set_attention_prologue_overlap(False)


def test_split_cap_is_deterministic_and_within_the_gate():
    T, N, Kd = 64, 1536, 8960
    x, w = make(SEED + 45, T, N, Kd)
    try:
        for cap in (1, 2, 4, 8):
            K.set_decode_linear_max_splits(cap)
            a = run(x, w, T, N)
            b = run(x, w, T, N)
            assert np.array_equal(a, b), f"max_splits={cap}: two runs differ"
            check_product(a, x, w, T)
    finally:
        K.set_decode_linear_max_splits(8)


def test_back_to_back_launches_on_one_stream():
    # a chain as in a decoder block: each product feeds the next, no host sync in between
    T, H, I = 64, 1536, 8960
    x, w1 = make(SEED + 51, T, 2 * I, H, scale=0.05)
    _, w2 = make(SEED + 53, T, H, I)
    xd, w1d, w2d = dev(x), dev(w1), dev(w2)
    act = torch.zeros(T, I, dtype=torch.int16, device="cuda")
    out = torch.zeros(T, H, dtype=torch.int16, device="cuda")
    K.set_attention_prologue_overlap(True)
    try:
        for _ in range(5):
            K.launch_decode_linear(act, xd, w1d, None, epilogue=K.EPILOGUE_SILU_MUL)
            K.launch_decode_linear(out, act, w2d, None)
        torch.cuda.synchronize()
    finally:
        K.set_attention_prologue_overlap(False)
    check_product(host(out), host(act), w2, T)
    assert K.decode_linear_health() == 0


def test_contract_errors():
    x, w = make(SEED + 61, 64, 128, 64)
    xd = torch.zeros(80, 64, dtype=torch.int16, device="cuda")
    wd = dev(w)
    out = torch.zeros(80, 128, dtype=torch.int16, device="cuda")
    with pytest.raises(K.KernelError):      # more than 64 token rows
        K.launch_decode_linear(out, xd, wd, None, num_tokens=65)
    with pytest.raises(K.KernelError):      # in_features not a multiple of 8
        K.launch_decode_linear(out, xd[:, :60], wd[:, :60], None, num_tokens=4)
    with pytest.raises(K.KernelError):      # bias with the gated epilogue
        K.launch_decode_linear(out[:, :64], xd, wd, dev(vector(1, 64)), num_tokens=4,
                               epilogue=K.EPILOGUE_SILU_MUL)
    with pytest.raises(K.KernelError):
        K.set_decode_linear_stages(9)
    with pytest.raises(K.KernelError):
        K.set_decode_linear_max_splits(3)
    K.launch_decode_linear(out, xd, wd, None, num_tokens=0)   # empty: silent return
    torch.cuda.synchronize()
    assert (host(out) == 0).all()
