"""GPU parity of the norm / RoPE / scatter / SiLU kernels, called through the C ABI.

Cases mirror the reference's kernel suite (tests/test_kernels.cu: row sweeps, both stride
modes, the RMSNorm half-ULP boundary fixture with mutants, the HF RoPE capture, full-pool
scatter mirrors, in-place SiLU) with the tighter gates this build is held to: bit moves
exact; norm / RoPE / SiLU within 1 FP16 ulp of FP32-order compute."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import assert_within_one_ulp, dev, host, is_nan_bits, ulp_of  # noqa: E402


def norm_gate(own, got, residual, x, w, what, min_exact=0.995):
    """<= 1 FP16 step at the norm's second rounding point, exact weight product after it."""
    if residual is None:
        h = x
        inv = 1.0 / np.sqrt((oracle.half_bits_to_f64(x) ** 2).mean(axis=1) + EPS)
    else:
        _, h, inv, _ = own.rmsnorm_residual(residual, x, w, EPS)
    ok, exact = oracle.rmsnorm_gate(got, h, inv, w)
    assert ok.all(), f"{what}: {int((~ok).sum())} elements outside the one-step gate"
    assert exact.mean() >= min_exact, f"{what}: only {exact.mean():.5f} bit-exact vs FP64"

EPS = 1e-6
ROWS = [1, 3, 8, 15, 16, 17, 63, 64, 65, 257]  # tests/test_kernels.cu:452


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    K.init()


# ------------------------------------------------------------------ RMSNorm

@pytest.mark.parametrize("rows", ROWS)
def test_rmsnorm_row_sweep(own, rows):
    x = own.uniform_half(0x51C + rows, rows * 1536, -1.0, 1.0).reshape(rows, 1536)
    w = own.uniform_half(0x71C, 1536, 0.5, 1.5)
    d_out = torch.zeros(rows, 1536, dtype=torch.int16, device="cuda")
    K.launch_rms_norm(d_out, dev(x), dev(w), rows, 1536, EPS)
    got = host(d_out)
    norm_gate(own, got, None, x, w, "rmsnorm vs FP64")
    assert (got == own.rmsnorm_f32(None, x, w, EPS)[0]).mean() > 0.999, "rmsnorm vs FP32 order"


@pytest.mark.parametrize("rows", ROWS)
def test_rmsnorm_residual_row_sweep(own, rows):
    x = own.uniform_half(0x52C + rows, rows * 1536, -1.0, 1.0).reshape(rows, 1536)
    r = own.uniform_half(0x62C + rows, rows * 1536, -1.0, 1.0).reshape(rows, 1536)
    w = own.uniform_half(0x72C, 1536, 0.5, 1.5)
    d_res, d_x = dev(r), dev(x)
    d_out = torch.zeros(rows, 1536, dtype=torch.int16, device="cuda")
    K.launch_rms_norm_residual(d_out, d_res, d_x, dev(w), rows, 1536, EPS)
    exp_out, exp_res, _, _ = own.rmsnorm_residual(r, x, w, EPS)
    assert np.array_equal(host(d_res), exp_res), "residual write-back must be bit-exact"
    assert np.array_equal(host(d_x), x), "input must not be written"
    norm_gate(own, host(d_out), r, x, w, "fused rmsnorm vs FP64")


@pytest.mark.parametrize("hidden", [1, 2, 7, 8, 24, 250, 1535, 1544, 2048, 2056, 4100])
def test_rmsnorm_odd_widths_and_unaligned_bases(own, hidden):
    rows = 5
    x = own.uniform_half(0x900 + hidden, rows * hidden, -2.0, 2.0).reshape(rows, hidden)
    r = own.uniform_half(0xA00 + hidden, rows * hidden, -2.0, 2.0).reshape(rows, hidden)
    w = own.uniform_half(0xB00 + hidden, hidden, 0.5, 1.5)
    exp_out, exp_res, _, _ = own.rmsnorm_residual(r, x, w, EPS)
    for shift in (0, 1):  # shift 1: every base is only 2-byte aligned -> scalar kernel
        pad = lambda a: dev(np.concatenate([np.zeros(shift, np.uint16), a.reshape(-1), np.full(8, 0x7E00, np.uint16)]))
        d_x, d_r, d_w = pad(x), pad(r), pad(w)
        d_out = torch.full((shift + rows * hidden + 8,), 0x1234, dtype=torch.int16, device="cuda")
        L = K.lib()
        st = L.rl_launch_rmsnorm_residual(d_out.data_ptr() + 2 * shift, d_r.data_ptr() + 2 * shift,
                                          d_x.data_ptr() + 2 * shift, d_w.data_ptr() + 2 * shift,
                                          rows, hidden, EPS, torch.cuda.current_stream().cuda_stream)
        assert st == 0
        out = host(d_out)
        norm_gate(own, out[shift:shift + rows * hidden].reshape(rows, hidden), r, x, w, f"H={hidden} shift={shift}", 0.98)
        assert np.array_equal(host(d_r)[shift:shift + rows * hidden].reshape(rows, hidden), exp_res)
        assert (out[:shift] == 0x1234).all() and (out[shift + rows * hidden:] == 0x1234).all(), "guard band written"


def test_rmsnorm_zero_row_stays_finite(own):
    x = np.zeros((2, 1536), np.uint16)
    w = own.uniform_half(1, 1536, 0.5, 1.5)
    d_out = torch.full((2, 1536), 0x7E00, dtype=torch.int16, device="cuda")
    K.launch_rms_norm(d_out, dev(x), dev(w), 2, 1536, EPS)
    assert (host(d_out) == 0).all()  # eps inside the rsqrt keeps 0 * rsqrt(eps) = 0


def test_rmsnorm_boundary_fixture_rounding_order(own):
    """tests/test_kernels.cu:602-660: residual bit-exact everywhere, output bit-exact on every
    column whose pre-rounding value is not within 1e-5 (relative) of an FP16 midpoint."""
    res, inp, w, isb = own.boundary_fixture(1)
    exp_out, exp_res, _, exc = own.rmsnorm_residual(res, inp, w, EPS, rel_floor=1e-5)
    d_res = dev(res)
    d_out = torch.zeros(8, 1536, dtype=torch.int16, device="cuda")
    K.launch_rms_norm_residual(d_out, d_res, dev(inp), dev(w), 8, 1536, EPS)
    got = host(d_out)
    assert np.array_equal(host(d_res), exp_res)
    keep = exc == 0
    assert np.array_equal(got[keep], exp_out[keep])
    norm_gate(own, got, res, inp, w, "boundary fixture", 0.9)
    # and the kernel is told apart from both wrong operation orders
    for which in ("unrounded", "single"):
        m = own.rmsnorm_mutant(which, res, inp, w, EPS)
        assert ((got != m) & keep).sum(axis=1).min() >= 16


def test_rmsnorm_deterministic_and_batch_invariant(own):
    """Same row, same bits: run to run, at any batch size, and across the CTA-per-row (few rows) and
    warp-per-row (many rows) kernels, which share one summation order."""
    c = wl.config_rmsnorm(64)
    outs = []
    for rows in (64, 64, 5, 4096):
        reps = -(-rows // 64)
        x = np.tile(c["x"], (reps, 1))[:rows]
        r = np.tile(c["residual"], (reps, 1))[:rows]
        d_res = dev(r)
        d_out = torch.zeros(rows, 1536, dtype=torch.int16, device="cuda")
        K.launch_rms_norm_residual(d_out, d_res, dev(x), dev(c["weight"]), rows, 1536, EPS)
        outs.append(host(d_out))
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[0][:5], outs[2])
    assert np.array_equal(outs[3][:64], outs[0]) and np.array_equal(outs[3][-64:], outs[0])


def test_rmsnorm_config1_shape_and_large_T(own):
    for rows in (64, 4096):
        c = wl.config_rmsnorm(rows)
        d_res = dev(c["residual"])
        d_out = torch.zeros(rows, 1536, dtype=torch.int16, device="cuda")
        K.launch_rms_norm_residual(d_out, d_res, dev(c["x"]), dev(c["weight"]), rows, 1536, EPS)
        exp_out, exp_res, _, _ = own.rmsnorm_residual(c["residual"], c["x"], c["weight"], EPS)
        assert np.array_equal(host(d_res), exp_res)
        norm_gate(own, host(d_out), c["residual"], c["x"], c["weight"], f"config 1 T={rows}")


# --------------------------------------------------------------------- RoPE

def run_rope(q_in, k_in, positions, theta, strided, q_heads=12, kv_heads=2, hd=128):
    t = len(positions)
    qw, kw = q_heads * hd, kv_heads * hd
    d_pos = dev(np.asarray(positions, np.int32))
    if not strided:
        d_q, d_k = dev(q_in), dev(k_in)
        K.launch_rope_inplace(d_q, d_k, qw, kw, d_pos, t, q_heads, kv_heads, hd, theta)
        return host(d_q).reshape(t, qw), host(d_k).reshape(t, kw)
    stride = 2048
    image = wl.uniform_half(0x517AB1E, t * stride, -1.0, 1.0).reshape(t, stride)
    image[:, :qw] = q_in
    image[:, qw:qw + kw] = k_in
    before = image.copy()
    d_img = dev(image)
    K.launch_rope_inplace(d_img, d_img, stride, stride, d_pos, t, q_heads, kv_heads, hd, theta, k_offset=qw)
    after = host(d_img).reshape(t, stride)
    assert np.array_equal(after[:, qw + kw:], before[:, qw + kw:]), "V region / tail must not be touched"
    return after[:, :qw], after[:, qw:qw + kw]


def rope_gate(got, ref_bits, x_in, what):
    """<= 1 FP16 ulp, the ulp taken at the larger magnitude of the rotated pair (the two product
    terms can cancel, so an ulp of a term may be many ulps of a small result)."""
    hd2 = 64
    g = oracle.half_bits_to_f64(got).reshape(-1, 2, hd2)
    r = oracle.half_bits_to_f64(ref_bits).reshape(-1, 2, hd2)
    x = np.abs(oracle.half_bits_to_f64(x_in).reshape(-1, 2, hd2))
    scale = ulp_of(np.maximum(x[:, :1, :], x[:, 1:, :]))
    assert (np.abs(g - r) <= scale + 1e-12).all(), what
    return float((got == ref_bits).mean())


@pytest.mark.parametrize("strided", [False, True])
def test_rope_matches_hf_capture(golden, strided):
    _, cap = golden
    q, k = run_rope(cap["q_in"], cap["k_in"], cap["positions"], float(cap["theta"]), strided)
    eq = rope_gate(q, cap["q_out"], cap["q_in"], "q vs HF capture")
    ek = rope_gate(k, cap["k_out"], cap["k_in"], "k vs HF capture")
    assert eq > 0.999 and ek > 0.999, (eq, ek)


@pytest.mark.parametrize("theta", [1e6, 1e4, 5e5])
@pytest.mark.parametrize("strided", [False, True])
def test_rope_vs_fp32_order_oracle(own, theta, strided):
    t = 64
    c = wl.config_rope_scatter(tokens=t)
    q_in = np.ascontiguousarray(c["qkv"][:, :1536])
    k_in = np.ascontiguousarray(c["qkv"][:, 1536:1792])
    pos = c["positions"]
    q, k = run_rope(q_in, k_in, pos, theta, strided)
    exact = []
    for got, x, heads in ((q, q_in, 12), (k, k_in, 2)):
        exact.append(rope_gate(got, own.rope(x, pos, heads, 128, theta, f32=True), x, "vs FP32 order"))
        err = np.abs(oracle.half_bits_to_f64(got) - oracle.half_bits_to_f64(own.rope(x, pos, heads, 128, theta)))
        assert err.max() <= 1e-2 and err.mean() <= 1e-3  # the reference's own gate vs FP64
    assert min(exact) > 0.999, exact


def test_rope_position_zero_is_identity_and_long_positions(own):
    q_in = wl.uniform_half(7, 4 * 1536, -4.0, 4.0).reshape(4, 1536)
    k_in = wl.uniform_half(8, 4 * 256, -4.0, 4.0).reshape(4, 256)
    q, k = run_rope(q_in, k_in, [0, 0, 0, 0], 1e6, False)
    assert np.array_equal(q, q_in) and np.array_equal(k, k_in)
    pos = [32767, 33023, 100000, 1]
    q, k = run_rope(q_in, k_in, pos, 1e6, True)
    rope_gate(q, own.rope(q_in, pos, 12, 128, 1e6, f32=True), q_in, "long positions")


def test_rope_prompt_sized_batch_equals_decode_sized_launches(own):
    """Thousands of rows take the several-rows-per-block mapping; the same rows fed 64 at a time take the
    one-row mapping. Both must give the same bits (odd row count: the last block is ragged), and a sample
    of rows is checked against the CPU rotation."""
    t = 2401
    q_in = wl.normal_half(0x2E1, t * 1536).reshape(t, 1536)
    k_in = wl.normal_half(0x2E2, t * 256).reshape(t, 256)
    pos = wl.randint(0x2E3, t, 0, 32767)
    q, k = run_rope(q_in, k_in, pos, 1e6, True)
    for lo in range(0, t, 64):
        hi = min(t, lo + 64)
        q1, k1 = run_rope(q_in[lo:hi], k_in[lo:hi], pos[lo:hi], 1e6, True)
        assert np.array_equal(q[lo:hi], q1) and np.array_equal(k[lo:hi], k1), (lo, hi)
    rows = np.r_[0:8, 1196:1204, 2393:2401]
    exact = rope_gate(q[rows], own.rope(q_in[rows], pos[rows], 12, 128, 1e6, f32=True), q_in[rows], "prompt-sized")
    assert exact > 0.999


def test_rope_odd_head_dim_takes_scalar_path(own):
    t, qh, kh, hd = 3, 3, 1, 20
    q_in = wl.uniform_half(17, t * qh * hd, -1.0, 1.0).reshape(t, qh * hd)
    k_in = wl.uniform_half(18, t * kh * hd, -1.0, 1.0).reshape(t, kh * hd)
    pos = np.array([5, 77, 4000], np.int32)
    d_q, d_k = dev(q_in), dev(k_in)
    K.launch_rope_inplace(d_q, d_k, qh * hd, kh * hd, dev(pos), t, qh, kh, hd, 1e4)
    d = oracle.ulp_distance(host(d_q).reshape(t, -1), own.rope(q_in, pos, qh, hd, 1e4, f32=True))
    assert (d <= 1).mean() > 0.99


# --------------------------------------------------------------- KV scatter

def scatter_case(own, tokens, positions, tables, table_stride, k, v, ks, vs, num_blocks, k_off=0, v_off=0, shift=0):
    n = num_blocks * 2 * 2 * 16 * 128
    nan = np.array([0x7E00, 0x7C01, 0x7FFF, 0xFE00, 0xFFFF, 0xFDAB], np.uint16)
    mirror = nan[np.arange(n) % 6].copy()
    pool_img = np.concatenate([np.full(shift, 0x1111, np.uint16), mirror, np.full(8, 0x2222, np.uint16)])
    d_pool = dev(pool_img)
    d_k, d_v = dev(k), dev(v)
    d_tables, d_positions = dev(tables), dev(positions)  # keep the device buffers alive across the launch
    L = K.lib()
    st = L.rl_launch_kv_scatter(d_pool.data_ptr() + 2 * shift, d_k.data_ptr() + 2 * k_off,
                                d_v.data_ptr() + 2 * v_off, ks, vs, d_tables.data_ptr(), table_stride,
                                d_positions.data_ptr(), tokens, 2, 128,
                                torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    kk = k.reshape(-1)[k_off:]
    vv = v.reshape(-1)[v_off:]
    own.kv_scatter(mirror, np.ascontiguousarray(kk), np.ascontiguousarray(vv), ks, vs, tables, table_stride,
                   positions, 2, 128)
    got = host(d_pool)
    assert np.array_equal(got[shift:shift + n], mirror), "pool differs from the CPU mirror (stray or missing writes)"
    assert (got[:shift] == 0x1111).all() and (got[shift + n:] == 0x2222).all()


def test_scatter_decode_mode_config2_strided_and_packed(own):
    c = wl.config_rope_scatter(tokens=64, num_blocks=8192)
    qkv = c["qkv"]
    scatter_case(own, 64, c["positions"], c["tables"], c["tables"].shape[1], qkv, qkv, 2048, 2048, 8192,
                 k_off=1536, v_off=1792)
    k = np.ascontiguousarray(qkv[:, 1536:1792])
    v = np.ascontiguousarray(qkv[:, 1792:2048])
    scatter_case(own, 64, c["positions"], c["tables"], c["tables"].shape[1], k, v, 256, 256, 8192)


def test_scatter_prefill_mode_shares_one_row(own):
    tokens = 257
    k = wl.uniform_half(31, tokens * 256, -1.0, 1.0).reshape(tokens, 256)
    v = wl.uniform_half(32, tokens * 256, -1.0, 1.0).reshape(tokens, 256)
    row = (wl.permutation(33, 40)[:17] + 1).astype(np.int32).reshape(1, 17)
    scatter_case(own, tokens, np.arange(tokens, dtype=np.int32), row, 0, k, v, 256, 256, 48)


@pytest.mark.parametrize("tokens", [2401, 9601])
def test_scatter_prompt_chunks_take_the_wide_mappings(own, tokens):
    """2401 tokens: four warps per block; 9601: also two tokens per warp. Both counts are odd, so the last
    block and the last warp are ragged."""
    k = wl.uniform_half(35, tokens * 256, -1.0, 1.0).reshape(tokens, 256)
    v = wl.uniform_half(36, tokens * 256, -1.0, 1.0).reshape(tokens, 256)
    blocks = -(-tokens // 16)
    row = (wl.permutation(37, 700)[:blocks] + 1).astype(np.int32).reshape(1, blocks)
    scatter_case(own, tokens, np.arange(tokens, dtype=np.int32), row, 0, k, v, 256, 256, 704)


def test_scatter_padded_row_lands_in_block_zero_and_boundaries(own):
    pos = np.array([0, 15, 16, 17, 31, 32, 0], np.int32)  # last row = padded slot (position 0, dummy table)
    tables = np.array([[3, 4, 5]] * 6 + [[0, 0, 0]], np.int32)
    tables[1:6, :] = [[6, 7, 8], [9, 10, 11], [12, 13, 14], [15, 16, 17], [18, 19, 20]]
    k = wl.uniform_half(41, 7 * 256, -1.0, 1.0).reshape(7, 256)
    v = wl.uniform_half(42, 7 * 256, -1.0, 1.0).reshape(7, 256)
    scatter_case(own, 7, pos, tables, 3, k, v, 256, 256, 24)


def test_scatter_odd_strides_and_unaligned_bases(own):
    tokens = 9
    k = wl.uniform_half(51, tokens * 263 + 4, -1.0, 1.0)
    v = wl.uniform_half(52, tokens * 259 + 4, -1.0, 1.0)
    pos = wl.randint(53, tokens, 0, 63)
    tables = (wl.permutation(54, 60)[:tokens * 4] + 1).astype(np.int32).reshape(tokens, 4)
    scatter_case(own, tokens, pos, tables, 4, k, v, 263, 259, 64, k_off=1, v_off=3)
    scatter_case(own, tokens, pos, tables, 4, k, v, 263, 259, 64, k_off=1, v_off=3, shift=1)


# ----------------------------------------------------------------- SiLU*mul

@pytest.mark.parametrize("tokens", [1, 3, 64, 512])
def test_silu_separate_and_in_place(own, tokens):
    gu = wl.config_silu(tokens)["gate_up"]
    exp64 = own.silu_mul(gu)
    exp32 = own.silu_mul(gu, f32=True)
    d_gu = dev(gu)
    d_out = torch.zeros(tokens, 8960, dtype=torch.int16, device="cuda")
    K.launch_silu_mul(d_out, d_gu, tokens, 8960)
    got = host(d_out)
    assert np.array_equal(host(d_gu), gu), "separate mode must not write gate_up"
    assert_within_one_ulp(got, exp64, "silu vs FP64", min_exact=0.999)
    assert_within_one_ulp(got, exp32, "silu vs FP32 order", min_exact=0.9995)
    K.launch_silu_mul(d_gu, d_gu, tokens, 8960)  # aliased: in place over the gate half
    after = host(d_gu)
    assert np.array_equal(after[:, :8960], got), "in-place result differs from the separate one"
    assert np.array_equal(after[:, 8960:], gu[:, 8960:]), "up half must stay untouched"


@pytest.mark.parametrize("inter", [1, 7, 8, 250, 8961])
def test_silu_odd_sizes_take_scalar_path(own, inter):
    rows = 4
    gu = wl.uniform_half(0x5111 + inter, rows * 2 * inter, -3.0, 3.0).reshape(rows, 2 * inter)
    d_out = torch.full((rows * inter + 8,), 0x1234, dtype=torch.int16, device="cuda")
    K.launch_silu_mul(d_out, dev(gu), rows, inter)
    got = host(d_out)
    assert_within_one_ulp(got[:rows * inter].reshape(rows, inter), own.silu_mul(gu), f"I={inter}")
    assert (got[rows * inter:] == 0x1234).all()


def test_silu_every_gate_pattern_matches_the_plain_division_kernel(own):
    """The vector kernel spells its divide out; the scalar kernel uses the compiler's `x / (1 + expf(-x))`
    (the reference kernel's expression). All 65536 gate bit patterns x 48 up values must agree bit for
    bit (NaN results by class), which pins the spelled-out divide to the IEEE one by exhaustion."""
    gates = np.arange(65536, dtype=np.uint16)
    ups = np.concatenate([wl.normal_half(0x51, 40), np.array([0x3C00, 0xBC00, 0x7BFF, 0x0001, 0x8001, 0x0000, 0x7C00, 0x3555], np.uint16)])
    inter = 65536
    rows = len(ups)
    gu = np.empty((rows, 2 * inter), np.uint16)
    gu[:, :inter] = gates[None, :]
    gu[:, inter:] = ups[:, None]
    d_gu = dev(gu)
    fast = torch.zeros(rows, inter, dtype=torch.int16, device="cuda")
    K.launch_silu_mul(fast, d_gu, rows, inter)
    # the scalar kernel: a 2-byte-aligned output base forces it
    slow_img = torch.zeros(rows * inter + 1, dtype=torch.int16, device="cuda")
    st = K.lib().rl_launch_silu_mul(slow_img.data_ptr() + 2, d_gu.data_ptr(), rows, inter,
                                    torch.cuda.current_stream().cuda_stream)
    assert st == 0
    a = host(fast)
    b = host(slow_img)[1:].reshape(rows, inter)
    both_nan = is_nan_bits(a) & is_nan_bits(b)
    assert np.array_equal(a[~both_nan], b[~both_nan])
    assert np.array_equal(is_nan_bits(a), is_nan_bits(b))
    # and the plain kernel itself against the FP64 checker wherever both are finite (FP32 underflows
    # silu(x) to zero below x = -88.7 where FP64 does not, which only shows against an infinite `up`)
    ref = own.silu_mul(gu)
    finite = lambda v: (v & 0x7FFF) < 0x7C00
    both = finite(b) & finite(ref)
    assert both.mean() > 0.9
    assert oracle.ulp_distance(b, ref)[both].max() <= 1


def test_silu_extremes_and_config4_largest(own):
    # saturating gates: silu(+big) = big, silu(-big) = -0 / tiny, NaN propagates
    vals = np.array([0x7BFF, 0xFBFF, 0x4D00, 0xCD00, 0x0001, 0x8001, 0x0000, 0x8000], np.uint16)
    gu = np.concatenate([vals, np.full(8, 0x3C00, np.uint16)]).reshape(1, 16)
    d_out = torch.zeros(1, 8, dtype=torch.int16, device="cuda")
    K.launch_silu_mul(d_out, dev(gu), 1, 8)
    assert_within_one_ulp(host(d_out), own.silu_mul(gu), "extremes")
    # T = 4096 (220 MB of traffic): every row against the CPU checker
    gu = wl.config_silu(4096)["gate_up"]
    d_gu = dev(gu)
    K.launch_silu_mul(d_gu, d_gu, 4096, 8960)
    got = host(d_gu)
    assert np.array_equal(got[:, 8960:], gu[:, 8960:])
    assert_within_one_ulp(got[:, :8960], own.silu_mul(gu, f32=True), "config 4 T=4096", min_exact=0.9995)


# ------------------------------------------------------- RoPE + scatter fused

@pytest.mark.parametrize("tokens,stride_mode", [(64, "decode"), (7, "decode"), (33, "prefill"), (2401, "prefill")])
def test_fused_rope_scatter_equals_the_two_launchers_bit_for_bit(own, tokens, stride_mode):
    # 2401 rows: the several-rows-per-block mappings of all three kernels, with a ragged last block
    c = wl.config_rope_scatter(tokens=min(tokens, 64), num_blocks=1024)
    if tokens > 64:
        c["qkv"] = wl.normal_half(0x2E4, tokens * 2048).reshape(tokens, 2048)
    tables = c["tables"] % 1024
    tables[tables == 0] = 1
    pos = c["positions"]
    if stride_mode == "prefill":            # all tokens share one table row; positions are a run
        pos = np.arange(100, 100 + tokens, dtype=np.int32)
        tables = (wl.permutation(0x77, 1000)[:256] + 1).astype(np.int32).reshape(1, 256)
        tstride = 0
    else:
        # distinct target slots per token
        tables[np.arange(tokens), pos // 16] = (wl.permutation(0x78, 1000)[:tokens] + 1)
        tstride = tables.shape[1]
    n = 1024 * 2 * 2 * 16 * 128
    pool0 = np.full(n, 0x7E00, np.uint16)
    d_tab, d_pos = dev(tables), dev(pos)
    # reference sequence: two launches
    qkv_a, pool_a = dev(c["qkv"]), dev(pool0)
    K.launch_rope_inplace(qkv_a, qkv_a, 2048, 2048, d_pos, tokens, 12, 2, 128, 1e6, k_offset=1536)
    K.launch_kv_scatter(pool_a, qkv_a, qkv_a, 2048, 2048, d_tab, tstride, d_pos, tokens, 2, 128,
                        k_offset=1536, v_offset=1792)
    # fused
    qkv_b, pool_b = dev(c["qkv"]), dev(pool0)
    K.launch_rope_kv_scatter(qkv_b, 2048, pool_b, d_tab, tstride, d_pos, tokens, 12, 2, 128, 1e6)
    assert np.array_equal(host(qkv_a), host(qkv_b))
    assert np.array_equal(host(pool_a), host(pool_b))
    # and the pool against the CPU mirror of the rotated K / raw V
    rot = host(qkv_b).reshape(tokens, 2048)
    mirror = pool0.copy()
    own.kv_scatter(mirror, np.ascontiguousarray(rot[:, 1536:1792]).reshape(-1), np.ascontiguousarray(rot[:, 1792:]).reshape(-1),
                   256, 256, tables, tstride, pos, 2, 128)
    assert np.array_equal(host(pool_b), mirror)
