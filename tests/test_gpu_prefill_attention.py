"""The fused paged prefill attention kernel (TMA page tiles + tcgen05), through the C ABI, against the CPU
checker: every query row of a prompt chunk is one causal attention over the sequence's paged cache up to its
own position - exactly a decode-attention problem with seq_len = position + 1 - so the checker is the paged
attention reference itself (FP64, unrounded), row by row, at the attention gate of 2e-3. Cases cover chunks
at the start of a prompt and deep inside it, lengths that are not multiples of the 128-row tile or the
16-token page, NaN in every slot past the context, rows and columns the kernel must not touch, and agreement
with the reference's composite (gather -> FP32 scores -> causal softmax -> P.V) built from this library's
prefill-side launchers."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host  # noqa: E402

MAX_ABS = 2e-3


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    K.init()


def make_case(chunk_start, chunk_len, seed, spare_pages=3):
    """One sequence of chunk_start + chunk_len cached tokens behind a permuted block table; NaN everywhere else."""
    kv_len = chunk_start + chunk_len
    blocks = (kv_len + 15) // 16
    c = wl.config_attention(lens=[kv_len], num_blocks=blocks + 40, seed=seed)
    row = np.zeros(blocks + spare_pages, np.int32)
    row[:blocks] = c["tables"][0, :blocks]
    q = wl.normal_half(seed + 9, chunk_len * 1536).reshape(chunk_len, 1536)
    return dict(pool=c["pool"], row=row, q=q, kv_len=kv_len, scale=c["scale"])


def reference(own, case, chunk_start, chunk_len):
    lens = np.arange(chunk_start + 1, chunk_start + chunk_len + 1, dtype=np.int32)
    tables = np.ascontiguousarray(np.tile(case["row"], (chunk_len, 1)))
    return own.paged_attention(case["q"], case["pool"], tables, lens, 12, 2, 128, case["scale"], f64out=True)


def run_fused(case, chunk_start, chunk_len, q_stride=2048, out_stride=1536, extra_rows=3):
    qbuf = np.full((chunk_len + extra_rows, q_stride), 0x7E00, np.uint16)      # NaN in the stride gap and past the chunk
    qbuf[:chunk_len, :1536] = case["q"]
    d_out = torch.full((chunk_len + extra_rows, out_stride), 0x1234, dtype=torch.int16, device="cuda")
    K.launch_paged_prefill_attention(d_out, out_stride, dev(qbuf), q_stride, dev(case["pool"]), dev(case["row"]),
                                     len(case["row"]), chunk_start, chunk_len, 12, 2, 128, case["scale"])
    torch.cuda.synchronize()
    return host(d_out)


@pytest.mark.parametrize("chunk_start,chunk_len", [(0, 1), (0, 16), (0, 127), (0, 128), (0, 129), (0, 300), (5, 123),
                                                   (1000, 257), (1024, 256), (4000, 200), (0, 1024), (3000, 1030),
                                                   (8000, 200), (5000, 129), (2040, 40)])
def test_chunk_against_the_cpu_checker(own, chunk_start, chunk_len):
    case = make_case(chunk_start, chunk_len, 0xF00 + chunk_start + chunk_len)
    got = run_fused(case, chunk_start, chunk_len)
    ref = reference(own, case, chunk_start, chunk_len)
    out = oracle.half_bits_to_f64(got[:chunk_len, :1536])
    assert np.isfinite(out).all(), "NaN reached a result: a masked or out-of-context slot was used"
    err = np.abs(out - ref)
    assert err.max() <= MAX_ABS + 2.0 ** -11 * max(1.0, np.abs(ref).max()), err.max()
    assert (got[chunk_len:] == 0x1234).all(), "rows past the chunk were written"
    assert K.prefill_attention_health() == 0


def test_scores_that_outgrow_the_running_reference_late_in_the_context(own):
    """The kernel keeps a stale reference maximum per row: after the first block it only looks at a block's
    maximum - and moves the reference, rescaling its running output in tensor memory - when a half row of
    probabilities sums to 2^15 or more. Keys from position 640 on are made 8, then 24, then 96 times larger, so
    every row's scores jump far beyond the reference three times over the blocks, by more and by less than that
    limit: the result must be that of an exact softmax either way."""
    chunk_start, chunk_len = 900, 200
    case = make_case(chunk_start, chunk_len, 0xFA1)
    pool = case["pool"].reshape(-1, 2, 2, 16, 128)
    for g in range(40, (case["kv_len"] + 15) // 16):
        k = pool[case["row"][g], 0]                     # K tiles of logical page g, both heads
        live = (k & 0x7FFF) < 0x7C00                    # leave the NaN padding of the last page alone
        factor = 8.0 if g < 50 else (24.0 if g < 60 else 96.0)
        k[live] = ((k[live].view(np.float16).astype(np.float32) * factor).astype(np.float16)).view(np.uint16)
    got = run_fused(case, chunk_start, chunk_len)
    ref = reference(own, case, chunk_start, chunk_len)
    out = oracle.half_bits_to_f64(got[:chunk_len, :1536])
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() <= MAX_ABS + 2.0 ** -11 * max(1.0, np.abs(ref).max())
    assert K.prefill_attention_health() == 0


def test_long_contexts_cut_across_ctas_give_the_same_bits_every_time():
    """A (tile, head) pair with more key blocks than the run length is cut into runs on different CTAs whose
    records a second kernel combines, always in run order: two launches must agree bit for bit."""
    chunk_start, chunk_len = 6000, 300
    case = make_case(chunk_start, chunk_len, 0xFB3)
    try:
        K.set_prefill_attention_split_blocks(8)          # 50 key blocks per tile: seven runs each
        a = run_fused(case, chunk_start, chunk_len)
        b = run_fused(case, chunk_start, chunk_len)
        assert np.array_equal(a, b)
        K.set_prefill_attention_split_blocks(1000)       # whole pairs: another summation order, same function
        c = run_fused(case, chunk_start, chunk_len)
    finally:
        K.set_prefill_attention_split_blocks(0)
    assert np.abs(oracle.half_bits_to_f64(a[:chunk_len, :1536]) - oracle.half_bits_to_f64(c[:chunk_len, :1536])).max() <= MAX_ABS


@pytest.mark.parametrize("split", [3, 1000])
def test_forced_run_lengths_against_the_cpu_checker(own, split):
    chunk_start, chunk_len = 2500, 140
    case = make_case(chunk_start, chunk_len, 0xFC1 + split)
    try:
        K.set_prefill_attention_split_blocks(split)
        got = run_fused(case, chunk_start, chunk_len)
    finally:
        K.set_prefill_attention_split_blocks(0)
    ref = reference(own, case, chunk_start, chunk_len)
    assert np.abs(oracle.half_bits_to_f64(got[:chunk_len, :1536]) - ref).max() <= MAX_ABS + 2.0 ** -11


def test_a_long_context_cut_by_the_launchers_own_choice(own):
    """130 rows at position 16000: two query tiles of 126-127 key blocks per head, which the launcher's replay of
    the launch cuts into several runs per pair (24 pairs on 148 SMs otherwise) - records of many runs combined."""
    chunk_start, chunk_len = 16000, 130
    assert K.prefill_attention_run_length(chunk_start, chunk_len, 12, 148) < 64
    case = make_case(chunk_start, chunk_len, 0xFD7)
    got = run_fused(case, chunk_start, chunk_len)
    ref = reference(own, case, chunk_start, chunk_len)
    out = oracle.half_bits_to_f64(got[:chunk_len, :1536])
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() <= MAX_ABS + 2.0 ** -11 * max(1.0, np.abs(ref).max())
    assert K.prefill_attention_health() == 0


@pytest.mark.parametrize("q_heads,kv_heads", [(6, 1), (8, 4), (16, 8)])
def test_other_head_counts(own, q_heads, kv_heads):
    """Any number of query heads that is a multiple of the KV heads (up to 8 KV heads): the page tile of a head is
    picked by the copy's coordinate, the group size only decides which KV head a query head reads."""
    chunk_start, chunk_len = 300, 200
    kv_len = chunk_start + chunk_len
    blocks = (kv_len + 15) // 16
    c = wl.config_attention(lens=[kv_len], num_blocks=blocks + 9, seed=0xFE0 + q_heads, q_heads=q_heads, kv_heads=kv_heads)
    row = np.ascontiguousarray(c["tables"][0, :blocks])
    width = q_heads * 128
    q = wl.normal_half(0xFE9 + kv_heads, chunk_len * width).reshape(chunk_len, width)
    d_out = torch.full((chunk_len, width), 0x1234, dtype=torch.int16, device="cuda")
    K.launch_paged_prefill_attention(d_out, width, dev(q), width, dev(c["pool"]), dev(row), blocks, chunk_start, chunk_len,
                                     q_heads, kv_heads, 128, c["scale"])
    torch.cuda.synchronize()
    lens = np.arange(chunk_start + 1, kv_len + 1, dtype=np.int32)
    tables = np.ascontiguousarray(np.tile(row, (chunk_len, 1)))
    ref = own.paged_attention(q, c["pool"], tables, lens, q_heads, kv_heads, 128, c["scale"], f64out=True)
    out = oracle.half_bits_to_f64(host(d_out))
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() <= MAX_ABS + 2.0 ** -11 * max(1.0, np.abs(ref).max())
    assert K.prefill_attention_health() == 0


@pytest.mark.parametrize("split", [0, 2])
def test_output_stride_gap_and_rows_past_the_chunk_are_untouched(own, split):
    """Whole pairs leave through the kernel's staged row stores, cut pairs (run length 2: two runs per pair) through
    the combining kernel: neither may write the stride gap or a row past the chunk (the last tile has 22 of 128 rows)."""
    chunk_start, chunk_len = 200, 150
    case = make_case(chunk_start, chunk_len, 0xF77)
    try:
        K.set_prefill_attention_split_blocks(split)
        got = run_fused(case, chunk_start, chunk_len, q_stride=2048, out_stride=2048)
    finally:
        K.set_prefill_attention_split_blocks(0)
    assert (got[:, 1536:] == 0x1234).all()
    assert (got[chunk_len:, :] == 0x1234).all()
    ref = reference(own, case, chunk_start, chunk_len)
    assert np.abs(oracle.half_bits_to_f64(got[:chunk_len, :1536]) - ref).max() <= MAX_ABS + 2.0 ** -11


def test_agrees_with_the_gather_softmax_composite():
    """The composite the reference's executor runs (src/core/model_executor.cpp:1219-1290), built from this
    library's gather and causal softmax around FP32 / FP16 torch products: both are within the gate of the
    exact result, so within twice the gate of each other; and identical for a single key."""
    chunk_start, chunk_len = 700, 260
    case = make_case(chunk_start, chunk_len, 0xF99)
    got = oracle.half_bits_to_f64(run_fused(case, chunk_start, chunk_len)[:chunk_len, :1536])
    end = chunk_start + chunk_len
    pool, row = dev(case["pool"]), dev(case["row"])
    khat = torch.empty(2, end, 128, dtype=torch.float16, device="cuda")
    vhat = torch.empty_like(khat)
    K.launch_kv_gather(khat, vhat, end * 128, 128, end * 128, 128, pool, row, end, 2, 128)
    q = dev(case["q"]).view(torch.float16).view(chunk_len, 12, 128).permute(1, 0, 2)
    scores = torch.bmm(q.float(), khat.repeat_interleave(6, 0).float().transpose(1, 2)) * case["scale"]
    probs = torch.empty(12, chunk_len, end, dtype=torch.float16, device="cuda")
    K.launch_prefill_softmax(probs, scores.contiguous(), 12, chunk_len, end, chunk_start)
    comp = torch.bmm(probs, vhat.repeat_interleave(6, 0)).permute(1, 0, 2).reshape(chunk_len, 1536)
    assert np.abs(got - comp.double().cpu().numpy()).max() <= 2 * MAX_ABS


def test_contract_errors():
    z = torch.zeros(16, 1536, dtype=torch.int16, device="cuda")
    pool = torch.zeros(4 * 2 * 2 * 16 * 128, dtype=torch.int16, device="cuda")
    row = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(K.KernelError, match="past the block table"):
        K.launch_paged_prefill_attention(z, 1536, z, 1536, pool, row, 2, 30, 16, 12, 2, 128, 0.088)
    with pytest.raises(K.KernelError, match="head_dim"):
        K.launch_paged_prefill_attention(z, 1536, z, 1536, pool, row, 2, 0, 16, 12, 2, 64, 0.088)
