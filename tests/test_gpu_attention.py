"""GPU parity of paged GQA decode attention (split over the whole grid), through the C ABI.

Mirrors tests/test_kernels.cu:1405-1489 (NaN-poisoned ragged batch, packed batches with padded
rows, primary vs the per-query-head cross-check kernel, determinism) and adds what the reference
suite does not hold: contexts up to 32768, the benchmark's batch-64 shape, thousands of tiny
sequences, and page-permutation invariance. Gate: max-abs 2e-3 against the FP64 checker."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host, is_nan_bits  # noqa: E402

MAX_ABS = 2e-3


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    K.init()
    yield
    assert K.attention_health() == 0, "a bounded wait in the attention kernel gave up"


def run_decode(c, strided=False, check_kernel=False, mbps=None):
    s = len(c["seq_lens"])
    qh, kvh = c["q_heads"], c["kv_heads"]
    width = qh * 128
    stride = 2048 if strided else width
    tables = c["tables"]
    if mbps is not None and mbps > tables.shape[1]:  # wider, dummy-padded table rows
        tables = np.concatenate([tables, np.zeros((s, mbps - tables.shape[1]), np.int32)], axis=1)
    q_img = wl.uniform_half(0x0A7B, s * stride, -1.0, 1.0).reshape(s, stride)
    q_img[:, :width] = c["q"]
    before = wl.uniform_half(0x0A7C, s * stride, -1.0, 1.0).reshape(s, stride)
    d_out = dev(before)
    K.launch_paged_attention_decode(d_out, stride, dev(q_img), stride, dev(c["pool"]), dev(tables),
                                    dev(c["seq_lens"]), s, tables.shape[1], qh, kvh, 128, c["scale"],
                                    check_kernel=check_kernel)
    after = host(d_out).reshape(s, stride)
    assert np.array_equal(after[:, width:], before[:, width:]), "bytes outside the output views changed"
    pad = np.asarray(c["seq_lens"]) <= 0
    assert np.array_equal(after[pad], before[pad]), "a padded row (seq_len 0) was written"
    return after[:, :width]


def expect(own, c, got, what, tol=MAX_ABS):
    live = np.asarray(c["seq_lens"]) > 0
    assert not is_nan_bits(got[live]).any(), f"{what}: NaN leaked into a live row"
    ref = own.paged_attention(c["q"], c["pool"], c["tables"], c["seq_lens"], c["q_heads"], c["kv_heads"],
                              128, c["scale"], f64out=True)
    err = np.abs(oracle.half_bits_to_f64(got[live]) - ref[live])
    # one FP16 rounding of the result is part of the contract: allow half a step on top of the gate
    allow = tol + 0.5 * 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref[live]), 2.0 ** -14))) - 10)
    assert (err <= allow).all(), f"{what}: max-abs {err.max():.3e}"
    assert err.mean() <= 3e-4, f"{what}: mean-abs {err.mean():.3e}"
    return float(err.max())


def case(lens, seed=0xA77E, q_heads=12, kv_heads=2, num_blocks=None, fill="uniform"):
    lens = np.asarray(lens, np.int32)
    need = int(((np.maximum(lens, 0) + 15) // 16).sum()) + 2
    return wl.config_attention(lens=lens, seed=seed, q_heads=q_heads, kv_heads=kv_heads,
                               num_blocks=num_blocks or need, fill=fill)


def test_nan_poisoned_pool_ragged_batch8_strided(own):
    c = case([257, 0, 64, 1, 17, 15, 63, 65])
    expect(own, c, run_decode(c, strided=True), "ragged batch 8")


@pytest.mark.parametrize("lens", [[1], [257], [16, 0, 65], [0, 0, 5], [2], [16], [17]])
def test_packed_small_batches_with_padded_rows(own, lens):
    c = case(lens, seed=0xA801 + len(lens))
    expect(own, c, run_decode(c), f"lens {lens}")


def test_sequence_of_one_token_returns_v_exactly(own):
    c = case([1, 1, 1], seed=0x1111)
    got = run_decode(c)
    pool = c["pool"].reshape(-1, 2, 2, 16, 128)
    for s in range(3):
        b = c["tables"][s, 0]
        for h in range(12):
            assert np.array_equal(got[s, h * 128:(h + 1) * 128], pool[b, 1, h // 6, 0])


def test_primary_matches_cross_check_kernel_on_random_shapes(own):
    draws = wl.splitmix64(0x0AC1E, 64)
    j = 0
    for trial in range(6):
        small = trial % 2 == 1
        n = 1 + int(draws[j] % np.uint64(8)); j += 1
        lens = [int(draws[j + i] % np.uint64(301)) for i in range(n)]; j += n
        lens[0] = max(lens[0], 1)
        c = case(lens, seed=0xF00D + trial, q_heads=6 if small else 12, kv_heads=1 if small else 2)
        primary = run_decode(c, strided=trial % 2 == 0)
        check = run_decode(c, strided=trial % 2 == 0, check_kernel=True)
        expect(own, c, primary, f"trial {trial} primary")
        expect(own, c, check, f"trial {trial} cross-check kernel")
        live = np.asarray(lens) > 0
        d = np.abs(oracle.half_bits_to_f64(primary[live]) - oracle.half_bits_to_f64(check[live]))
        assert d.max() <= MAX_ABS


def test_deterministic_across_repeated_launches(own):
    c = case([65, 0, 17, 257, 1300, 40])
    a, b = run_decode(c), run_decode(c)
    live = np.asarray(c["seq_lens"]) > 0
    assert np.array_equal(a[live], b[live])


@pytest.mark.parametrize("ctx", [4095, 4096, 4097, 8192, 32768])
def test_long_contexts_split_across_the_grid(own, ctx):
    c = case([ctx, 33], seed=0x10C + ctx, fill="normal")
    expect(own, c, run_decode(c, strided=True), f"ctx {ctx}")


def test_benchmark_shape_batch64_ctx_1024_1280(own):
    c = wl.config_attention()  # N(0,1) inputs, 8192-block pool, NaN outside the live slots
    got = run_decode(c, strided=True)
    expect(own, c, got, "config 3")
    # wider dummy-padded table rows must not change a bit
    assert np.array_equal(run_decode(c, strided=True, mbps=2064), got)


def test_mixed_long_and_short_batch(own):
    lens = [32768, 1024, 5000, 0, 8192, 16, 1, 2047] + [1500] * 24
    c = case(lens, seed=0x5151, fill="normal")
    expect(own, c, run_decode(c, strided=True), "mixed batch")


def test_many_tiny_sequences_and_more_than_one_launch_chunk(own):
    lens = wl.randint(0x71, 1100, 0, 40)  # > 1024 sequences: the launcher walks two chunks
    c = case(lens, seed=0x72)
    expect(own, c, run_decode(c), "1100 tiny sequences")


def test_page_permutation_invariance_bit_exact(own):
    """The same logical KV behind a different physical page placement gives the same bits."""
    lens = np.array([1100, 700, 0, 2049, 15], np.int32)
    a = case(lens, seed=0x900, num_blocks=400)
    got_a = run_decode(a)
    pool = a["pool"].reshape(400, -1)
    perm = wl.permutation(0x901, 399) + 1
    remap = np.concatenate([[0], perm]).astype(np.int32)  # block 0 stays the dummy
    pool_b = np.empty_like(pool)
    pool_b[remap] = pool
    b = dict(a, pool=pool_b.reshape(-1), tables=remap[a["tables"]])
    assert np.array_equal(run_decode(b), got_a)


def test_scatter_then_attend_round_trip(own):
    """K/V written by the scatter kernel are what attention reads: decode step t appends a token."""
    c = case([100, 31, 64], seed=0x600, num_blocks=64)
    lens = np.asarray(c["seq_lens"])
    # room for one more token per sequence
    tables = np.concatenate([c["tables"], np.zeros((3, 1), np.int32)], axis=1)
    used = set(tables.reshape(-1).tolist())
    free = [b for b in range(1, 64) if b not in used]
    for s in range(3):
        if lens[s] % 16 == 0:
            tables[s, lens[s] // 16] = free.pop()
    kv = wl.uniform_half(0x601, 3 * 512, -1.0, 1.0).reshape(3, 512)
    d_pool = dev(c["pool"])
    d_kv = dev(kv)
    K.launch_kv_scatter(d_pool, d_kv, d_kv, 512, 512, dev(tables), tables.shape[1], dev(lens.astype(np.int32)),
                        3, 2, 128, v_offset=256)
    mirror = c["pool"].copy()
    own.kv_scatter(mirror, np.ascontiguousarray(kv[:, :256]).reshape(-1), np.ascontiguousarray(kv[:, 256:]).reshape(-1),
                   256, 256, tables, tables.shape[1], lens, 2, 128)
    assert np.array_equal(host(d_pool), mirror)
    c2 = dict(c, pool=mirror, tables=tables, seq_lens=lens + 1)
    d_out = torch.zeros(3, 1536, dtype=torch.int16, device="cuda")
    K.launch_paged_attention_decode(d_out, 1536, dev(c["q"]), 1536, d_pool, dev(tables), dev((lens + 1).astype(np.int32)),
                                    3, tables.shape[1], 12, 2, 128, c["scale"])
    expect(own, c2, host(d_out), "after append")


def test_prologue_overlap_changes_no_bit(own):
    """With programmatic dependent launch on, the kernel's table walk runs under the previous kernel
    (scatter, or the previous attention call); results must stay bit-identical over many back-to-back
    scatter -> attention -> attention rounds that reuse the output, the workspace and the pool."""
    c = case([700, 33, 1300, 0, 257, 2048, 16, 90], seed=0x0F1A, fill="normal")
    lens = np.asarray(c["seq_lens"])
    s = len(lens)
    d_pool, d_tab, d_lens = dev(c["pool"]), dev(c["tables"]), dev(lens)
    d_q = dev(c["q"])
    kv = wl.normal_half(0x0F1B, s * 512).reshape(s, 512)
    d_kv = dev(kv)
    pos = dev(np.maximum(lens - 1, 0).astype(np.int32))
    outs = {}
    try:
        for overlap in (False, True):
            K.set_attention_prologue_overlap(overlap)
            got = []
            for it in range(20):
                d_out = torch.zeros(s, 1536, dtype=torch.int16, device="cuda")
                # the scatter rewrites each sequence's last token (same bytes every time), then two attention calls
                K.launch_kv_scatter(d_pool, d_kv, d_kv, 512, 512, d_tab, c["tables"].shape[1], pos, s, 2, 128, v_offset=256)
                K.launch_paged_attention_decode(d_out, 1536, d_q, 1536, d_pool, d_tab, d_lens, s, c["tables"].shape[1],
                                                12, 2, 128, c["scale"])
                K.launch_paged_attention_decode(d_out, 1536, d_q, 1536, d_pool, d_tab, d_lens, s, c["tables"].shape[1],
                                                12, 2, 128, c["scale"])
                got.append(host(d_out))
            assert all(np.array_equal(g, got[0]) for g in got)
            outs[overlap] = got[0]
    finally:
        K.set_attention_prologue_overlap(False)
    live = lens > 0
    assert np.array_equal(outs[False][live], outs[True][live])


@pytest.mark.parametrize("kv_heads", [1, 3, 4, 8])
def test_other_kv_head_counts(own, kv_heads):
    """The tile stride of the tensor copy follows num_kv_heads (1..8); 6 query heads per KV head throughout."""
    c = case([300, 17, 0, 1025, 64], seed=0x4E0 + kv_heads, q_heads=6 * kv_heads, kv_heads=kv_heads)
    s = len(c["seq_lens"])
    width = 6 * kv_heads * 128
    d_out = torch.zeros(s, width, dtype=torch.int16, device="cuda")
    K.launch_paged_attention_decode(d_out, width, dev(c["q"]), width, dev(c["pool"]), dev(c["tables"]),
                                    dev(c["seq_lens"]), s, c["tables"].shape[1], 6 * kv_heads, kv_heads, 128, c["scale"])
    expect(own, c, host(d_out), f"{kv_heads} kv heads")


def test_seq_len_beyond_the_table_is_clamped_to_it(own):
    """seq_len larger than max_blocks_per_seq * 16 is clamped, as the reference kernel does
    (src/kernels/paged_attention.cu:153): no table entry past the row is ever read."""
    c = case([160, 48], seed=0xC1A, fill="normal")
    lens = np.array([100000, 48], np.int32)  # row 0 claims far more than its 10-entry table row holds
    d_out = torch.zeros(2, 1536, dtype=torch.int16, device="cuda")
    K.launch_paged_attention_decode(d_out, 1536, dev(c["q"]), 1536, dev(c["pool"]), dev(c["tables"]), dev(lens), 2,
                                    c["tables"].shape[1], 12, 2, 128, c["scale"])
    expect(own, c, host(d_out), "clamped row")


def test_second_device_keeps_its_own_state(own):
    """Per-device workspace and attributes: the same case on device 1 after device 0 (needs two GPUs)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU")
    c = case([700, 33, 1300], seed=0xD2, fill="normal")
    outs = []
    for d in (0, 1, 0):
        with torch.cuda.device(d):
            K.init(d)
            to = lambda a: dev(a).to(f"cuda:{d}")
            d_out = torch.zeros(3, 1536, dtype=torch.int16, device=f"cuda:{d}")
            K.launch_paged_attention_decode(d_out, 1536, to(c["q"]), 1536, to(c["pool"]), to(c["tables"]),
                                            to(c["seq_lens"]), 3, c["tables"].shape[1], 12, 2, 128, c["scale"])
            qkv = to(wl.normal_half(0xD3, 3 * 2048).reshape(3, 2048))
            K.launch_rope_inplace(qkv, qkv, 2048, 2048, to(np.array([5, 700, 4000], np.int32)), 3, 12, 2, 128, 1e6,
                                  k_offset=1536)
            torch.cuda.synchronize(d)
            outs.append((host(d_out), host(qkv)))
            assert K.attention_health() == 0
    expect(own, c, outs[1][0], "device 1")
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][0], outs[2][0])
    assert np.array_equal(outs[0][1], outs[1][1])


def test_a_wait_that_runs_out_raises_the_health_flag_and_leaves_the_context_usable(own):
    """The give-up path of the kernel's bounded waits, exercised without any fault: through the test hook one
    warp never requests its first page, so its wait (shortened to about a millisecond) runs out. The launch
    must come back, rl_attention_health must report it once - for the allocating launcher and for the
    launcher with built-in scratch alike - and the next ordinary launch must be correct again."""
    c = wl.config_attention(lens=[700, 33, 1500, 64, 257, 2049], num_blocks=400, seed=0x5A77)
    n = len(c["seq_lens"])

    def launch(entry):
        d_out = torch.zeros(n, 1536, dtype=torch.int16, device="cuda")
        entry(d_out, 1536, dev(c["q"]), 1536, dev(c["pool"]), dev(c["tables"]), dev(c["seq_lens"]), n,
              c["tables"].shape[1], 12, 2, 128, c["scale"])
        torch.cuda.synchronize()
        return host(d_out)

    assert K.attention_health() == 0
    for entry in (K.launch_paged_attention_decode, K.launch_paged_attention_decode_static):
        try:
            K.attention_test_wait_expiry(True, 2_000_000)
            launch(entry)                                # returns: nothing spins without bound
            assert K.attention_health() == 1, "the wait that ran out was not reported"
            assert K.attention_health() == 0, "the flag is cleared by the query that reported it"
        finally:
            K.attention_test_wait_expiry(False, 0)
        expect(own, c, launch(entry), "after a reported give-up")
        assert K.attention_health() == 0
