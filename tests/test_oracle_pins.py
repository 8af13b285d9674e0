"""Pins the CPU checker (oracle/redline_oracle.c) before anything trusts it:
against the committed goldens (outputs of the reference's own CPU code and its
HF RoPE capture), and live against the compiled reference code where present.
Mirrors the CPU-only self-checks of the reference's tests/test_kernels.cu
(:291-350, :552-600, :748-769)."""
import numpy as np
import pytest

import oracle
from redline_llm_b200 import workloads as wl

EPS = 1e-6


def test_widening_all_65536_patterns(own, golden):
    g, _ = golden
    mine = np.array([own.half_to_double(i) for i in range(65536)])
    exp = g["widen_all"]
    nan = np.isnan(exp)
    assert np.array_equal(np.isnan(mine), nan)
    assert np.array_equal(mine[~nan], exp[~nan])
    # and every non-NaN pattern survives widen -> quantise
    for i in np.flatnonzero(~nan)[::7]:
        assert own.quantize(float(exp[i])) == i


def test_quantise_crafted_boundaries(own, golden):
    g, _ = golden
    for x, q in zip(g["quant_probe_in"], g["quant_probe_out"]):
        assert own.quantize(float(x)) == int(q), x
    # landmarks of the boundary fixture (tests/reference/rmsnorm_ref.hpp:192-201)
    assert own.L.rlo_half_add(0x3C00, 0x1000) == 0x3C00
    assert own.L.rlo_half_add(0x3C01, 0x1000) == 0x3C02
    assert own.quantize(float("nan")) == 0x7E00
    assert own.quantize(65519.999) == 0x7BFF and own.quantize(65520.0) == 0x7C00


def test_quantise_random_vs_numpy(own):
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 2000), rng.uniform(-70000, 70000, 2000)])
    with np.errstate(over="ignore"):
        exp = xs.astype(np.float16).view(np.uint16)
    got = np.array([own.quantize(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, exp)


def test_numpy_stream_equals_c_stream(own):
    assert np.array_equal(wl.splitmix64(1234, 100), own.u64(1234, 100))
    assert np.array_equal(wl.uniform_half(99, 5000, -3.0, 3.0), own.uniform_half(99, 5000, -3.0, 3.0))
    assert np.array_equal(wl.normal_half(5, 4001, 1.0, 0.1), own.normal_half(5, 4001, 1.0, 0.1))


def test_boundary_fixture_and_mutants_against_golden(own, golden):
    g, _ = golden
    res, inp, w, isb = own.boundary_fixture(1)
    assert np.array_equal(isb, g["bf_is_boundary"])
    out, res2, _, exc = own.rmsnorm_residual(res, inp, w, EPS, rel_floor=1e-5)
    assert np.array_equal(out, g["bf_out"])
    assert np.array_equal(res2, g["bf_residual"])
    assert np.array_equal(exc, g["bf_excluded"])
    m1 = own.rmsnorm_mutant("unrounded", res, inp, w, EPS)
    m2 = own.rmsnorm_mutant("single", res, inp, w, EPS)
    assert np.array_equal(m1, g["bf_mut_unrounded"])
    assert np.array_equal(m2, g["bf_mut_single"])
    # the fixture must keep its discriminating power: >= 16 flips per row on kept columns
    keep = exc == 0
    for m in (m1, m2):
        flips = ((m != out) & keep).sum(axis=1)
        assert flips.min() >= 16, flips
    # landmark roundings on the boundary columns
    b = isb.astype(bool)
    assert set(np.unique(res2[0][b[0]])) == {0x3C00}
    assert set(np.unique(res2[1][b[1]])) == {0x3C02}


def test_rmsnorm_small_case_against_golden(own, golden):
    g, _ = golden
    assert np.array_equal(own.rmsnorm(g["rn_x"], g["rn_w"], EPS), g["rn_plain"])
    out, res2, _, _ = own.rmsnorm_residual(g["rn_r"], g["rn_x"], g["rn_w"], EPS)
    assert np.array_equal(out, g["rn_fused_out"])
    assert np.array_equal(res2, g["rn_fused_res"])


def test_rope_against_golden_and_hf_capture(own, golden):
    g, cap = golden
    assert np.array_equal(own.rope(g["rope_in"], g["rope_pos"], 14, 128, 1e6), g["rope_out"])
    # the HF capture agrees with the FP64 rotation within the elementwise tolerance the
    # reference uses for this check (max-abs 1e-2, mean-abs 1e-3), and almost always bit-exactly
    for name, heads in (("q", 12), ("k", 2)):
        got = own.rope(cap[f"{name}_in"], cap["positions"], heads, 128, float(cap["theta"]))
        err = np.abs(oracle.half_bits_to_f64(got) - oracle.half_bits_to_f64(cap[f"{name}_out"]))
        assert err.max() <= 1e-2 and err.mean() <= 1e-3
        assert (got == cap[f"{name}_out"]).mean() > 0.99  # FP64 angles differ at positions 2047/4095
        # the FP32 order (the kernels' order: FP32 inv_freq, FP32 angle) reproduces the capture exactly
        got32 = own.rope(cap[f"{name}_in"], cap["positions"], heads, 128, float(cap["theta"]), f32=True)
        assert np.array_equal(got32, cap[f"{name}_out"])
    # position 0 is the identity, bit for bit
    assert np.array_equal(own.rope(g["rope_in"][:1], [0], 14, 128, 1e6), g["rope_in"][:1])


def test_silu_against_golden(own, golden):
    g, _ = golden
    assert np.array_equal(own.silu_mul(g["silu_in"]), g["silu_out"])
    d = oracle.ulp_distance(own.silu_mul(g["silu_in"], f32=True), g["silu_out"])
    assert d.max() <= 1


def test_attention_ragged_nan_poisoned_against_golden(own, golden):
    g, _ = golden
    out = own.paged_attention(g["att_q"], g["att_pool"], g["att_tables"], g["att_lens"], 12, 2, 128,
                              0.088388347648318447)
    live = g["att_lens"] > 0
    assert np.array_equal(out[live], g["att_out"][live])
    assert not ((out[live] & 0x7FFF) > 0x7C00).any()


# ---- live against the compiled reference code (present in the build container)

def test_live_generators_and_helpers(own, ref):
    assert np.array_equal(own.uniform_half(0xA77E, 3000, -1.0, 1.0), ref.uniform_half(0xA77E, 3000, -1.0, 1.0))
    rng = np.random.default_rng(3)
    for x in np.concatenate([rng.normal(0, 1, 500), rng.normal(0, 1e-5, 500), [65519.9, 65520.0, 6e-8, 2.98e-8]]):
        assert own.quantize(float(x)) == ref.quantize(float(x))
        assert own.L.rlo_rel_distance_to_boundary(float(x)) == ref.L.rlr_rel_distance_to_boundary(float(x))


@pytest.mark.parametrize("rows", [1, 3, 8, 65])
def test_live_rmsnorm(own, ref, rows):
    x = own.uniform_half(0x51C + rows, rows * 1536, -1.0, 1.0).reshape(rows, 1536)
    r = own.uniform_half(0x61C + rows, rows * 1536, -1.0, 1.0).reshape(rows, 1536)
    w = own.uniform_half(0x71C, 1536, 0.5, 1.5)
    assert np.array_equal(own.rmsnorm(x, w, EPS), ref.rmsnorm(x, w, EPS))
    a = own.rmsnorm_residual(r, x, w, EPS, rel_floor=1e-5)
    b = ref.rmsnorm_residual(r, x, w, EPS, rel_floor=1e-5)
    for u, v in zip(a, b):
        assert np.array_equal(u, v)


def test_live_rope_and_silu(own, ref):
    heads = own.uniform_half(11, 64 * 14 * 128, -1.0, 1.0).reshape(64, -1)
    pos = wl.randint(12, 64, 0, 4095)
    assert np.array_equal(own.rope(heads, pos, 14, 128, 1e6), ref.rope(heads, pos, 14, 128, 1e6))
    assert np.array_equal(own.rope(heads, pos, 14, 128, 1e4), ref.rope(heads, pos, 14, 128, 1e4))
    gu = wl.normal_half(13, 16 * 2 * 8960).reshape(16, -1)
    assert np.array_equal(own.silu_mul(gu), ref.silu_mul(gu))


def test_live_scatter_and_attention_config_shapes(own, ref):
    c = wl.config_rope_scatter(tokens=64, num_blocks=512, max_pos=4096)
    n = 512 * 2 * 2 * 16 * 128
    k = np.ascontiguousarray(c["qkv"][:, 1536:1792]).reshape(-1)
    v = np.ascontiguousarray(c["qkv"][:, 1792:2048]).reshape(-1)
    tables = np.minimum(c["tables"], 511)
    p1 = np.full(n, 0x7E00, np.uint16)
    p2 = p1.copy()
    own.kv_scatter(p1, k, v, 256, 256, tables, tables.shape[1], c["positions"], 2, 128)
    ref.kv_scatter(p2, k, v, 256, 256, tables, tables.shape[1], c["positions"], 2, 128)
    assert np.array_equal(p1, p2)
    a = wl.config_attention(batch=6, lo=100, hi=400, num_blocks=256)
    o1 = own.paged_attention(a["q"], a["pool"], a["tables"], a["seq_lens"], 12, 2, 128, a["scale"])
    o2 = ref.paged_attention(a["q"], a["pool"], a["tables"], a["seq_lens"], 12, 2, 128, a["scale"], threads=4)
    assert np.array_equal(o1, o2)


def test_live_gather_and_prefill_softmax(own, ref):
    a = wl.config_attention(lens=[257], num_blocks=40, seed=0x6A7, fill="uniform")
    ctx = 257
    for head_stride, row_stride in ((ctx * 128, 128), (300 * 133, 133)):
        sent = own.uniform_half(0x6A8, 2 * head_stride, -1.0, 1.0)
        k1, v1, k2, v2 = sent.copy(), sent.copy(), sent.copy(), sent.copy()
        own.kv_gather(k1, v1, head_stride, row_stride, a["pool"], a["tables"][0], ctx, 2, 128)
        ref.kv_gather(k2, v2, head_stride, row_stride, a["pool"], a["tables"][0], ctx, 2, 128)
        assert np.array_equal(k1, k2) and np.array_equal(v1, v2)
        assert not np.array_equal(k1, sent)
    rng = np.random.default_rng(9)
    for (h, c, kv, start) in ((2, 5, 5, 0), (3, 7, 40, 33), (1, 1, 1, 0), (2, 16, 257, 241)):
        sc = rng.normal(0, 3, (h, c, kv)).astype(np.float32)
        for i in range(c):
            sc[:, i, start + i + 1:] = np.nan  # masked scores are never read
        p1, p2 = own.prefill_softmax(sc, start), ref.prefill_softmax(sc, start)
        assert np.array_equal(p1, p2)
        assert not ((p1 & 0x7FFF) > 0x7C00).any() and (p1[:, 0, start + 1:] == 0).all()
