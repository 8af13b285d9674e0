"""The whole decode on the real architecture (28 layers, hidden 1536, FFN 8960, 12 Q / 2 KV heads, vocabulary
151 936, FP16 ~N(0, 0.02)), at the decode-step benchmark's shapes.

* The gate of the full greedy decode: one admission wave of 64 cached sequences - contexts uniform in
  [1024, 8192] plus one of 32 768 tokens, so many items are cut across CTAs and one is merged from a dozen
  of them - decodes 256 tokens FREE-RUNNING through the shipped path (tcgen05 linear layers, fused
  epilogues, dependent launch, CUDA-graph replay) while an independent engine (the reference's own CUDA
  kernels where oracle/_ref holds them, library GEMMs, eager, unfused) is teacher-forced along
  (oracle/free_run.py). Every disagreement must be a near-tie, the two paths' logits must agree within
  the logit tolerance at all 16 384 (step, sequence) points, and a bounded sample of steps is recomputed
  on the host cores.
* CUDA-graph replay vs eager, dependent launch on vs off, and a sequence alone vs in a batch, on the same
  architecture with sequences that the attention kernel splits; and the step from a real prompt pass to
  the first decode steps with dependent launch on.
"""
import json

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import free_run  # noqa: E402
from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200.engine import Engine, ModelConfig, ModelWeights, blocks_for_tokens  # noqa: E402

LOGIT_TOL_FRAC = 0.01   # of the largest |logit|: what separates a coin flip from a bug in this suite


@pytest.fixture(scope="module")
def model():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    cfg = ModelConfig()
    return cfg, ModelWeights(cfg, torch.device("cuda", 0), seed=0x5EED)


def test_full_greedy_decode_of_a_config5_wave_against_an_independent_path(model):
    cfg, w = model
    contexts = free_run.config5_wave_contexts(0xB200C0F5, 64, long_rows=1)
    assert max(contexts) == 32768 and sum(1 for c in contexts if c > 4096) >= 20
    order = np.argsort(contexts)
    audit_rows = [int(order[2]), int(order[len(order) // 2])]     # a short context and a median one (cut across CTAs)
    rep = free_run.lockstep_decode(cfg, w, contexts, 256, seed=0x5EED0000, cpu_audit_steps=(0, 64, 128, 192, 255),
                                   cpu_audit_rows=audit_rows, cpu_audit_divergences=4,
                                   logit_tol_frac=LOGIT_TOL_FRAC)
    toks = rep.pop("tokens_free_running")
    listed = rep.pop("disagreement_list")
    print("free_running report:", json.dumps(rep))
    assert rep["compared_steps"] == 64 * 256
    assert rep["attention_health"] == 0 and rep["linear_health"] == 0
    # a real greedy stream: inside the vocabulary, not a single repeated token
    assert toks.min() >= 0 and toks.max() < cfg.vocab and len(np.unique(toks)) > 1000
    # the two paths compute the same function: logits agree within the tolerance everywhere ...
    assert rep["logits_max_abs_between_paths"] <= rep["logit_tolerance"], rep
    # ... so they choose the same token except at near-ties, and nearly always
    assert rep["every_disagreement_within_tolerance"], [d for d in listed if d["checker_margin_to_token"] > 2 * rep["logit_tolerance"]]
    assert rep["agreeing_steps"] >= 0.97 * rep["compared_steps"], rep
    # the host cores' opinion on the sampled steps and on the first divergences
    assert len(rep["cpu_audits"]) >= 8
    assert free_run.audits_ok(rep), rep["cpu_audits"]


def _wave(cfg, w, contexts, steps, seed, **kw):
    """Decodes `steps` tokens of cached sequences; returns (tokens [n, steps], logits of every step [steps, n, vocab] on the host as FP16 bits)."""
    n = len(contexts)
    rows = next(b for b in (1, 2, 4, 8, 16, 32, 48, 64) if b >= max(n, kw.get("pad_eager_to_bucket", 0)))
    blocks = sum(blocks_for_tokens(c + steps) for c in contexts) + 8
    args = dict(kv_pool_gb=blocks * cfg.block_bytes() / (1 << 30), max_batch=8, max_seq_len=max(contexts) + steps + 16,
                config=cfg, weights=w, graph_buckets=[rows])
    args.update(kw)
    e = Engine(**args)
    for i, c in enumerate(contexts):
        e.add_synthetic_request(c, steps, seed=seed + i)
    toks, logits = np.zeros((n, steps), np.int64), []
    for s in range(steps):
        res = e.step()
        toks[:, s] = [t for (_, t, _, _) in res]
        logits.append(e.exec.logits[:n].cpu().numpy().view(np.uint16).copy())
    assert K.attention_health() == 0 and K.decode_linear_health() == 0
    return toks, np.stack(logits)


CONTEXTS = [32768, 5000, 1500, 4096, 7777, 16, 8191, 2049]    # 32768 spans ~75 CTAs' shares; most others are cut too


def test_graph_replay_eager_and_dependent_launch_are_bit_identical_on_split_sequences(model):
    cfg, w = model
    base_t, base_l = _wave(cfg, w, CONTEXTS, 8, 0x77000)
    for kw in (dict(enable_cuda_graphs=False), dict(prologue_overlap=False),
               dict(enable_cuda_graphs=False, prologue_overlap=False)):
        t, l = _wave(cfg, w, CONTEXTS, 8, 0x77000, **kw)
        assert np.array_equal(l, base_l), f"logits differ with {kw}"
        assert np.array_equal(t, base_t)
    K.set_attention_prologue_overlap(True)


def test_a_sequence_alone_and_inside_a_batch_agree_on_split_sequences(model):
    """Alone, a sequence's pages are cut into 148 shares; inside a batch, into however many its part of the
    whole page range covers - different merge trees, so logits agree within the tolerance rather than bit
    for bit, and tokens agree wherever the margin is not a coin flip. Both runs use the same bucket (8) so
    the GEMM shapes are equal (the reference's same-shape protocol, docs/DESIGN.md:691-709 there)."""
    cfg, w = model
    bt, bl = _wave(cfg, w, CONTEXTS, 6, 0x78000, enable_cuda_graphs=False, pad_eager_to_bucket=8)
    for i in (0, 1, 6):
        st, sl = _wave(cfg, w, [CONTEXTS[i]], 6, 0x78000 + i, enable_cuda_graphs=False, pad_eager_to_bucket=8)
        a = sl[:, 0].view(np.float16).astype(np.float32)
        b = bl[:, i].view(np.float16).astype(np.float32)
        scale = float(np.abs(b).max())
        assert np.abs(a - b).max() <= LOGIT_TOL_FRAC * scale
        for s in range(6):
            if st[0, s] != bt[i, s]:
                srt = np.sort(b[s])
                assert srt[-1] - srt[-2] <= 2 * LOGIT_TOL_FRAC * scale, (i, s)
                break   # histories differ from here on


def test_prompt_pass_then_first_decode_steps_with_dependent_launch(model):
    """A real prompt pass (chunked, scattering whole chunks into the pool) followed at once by decode steps
    launched with programmatic dependent launch: the first decode step's attention requests pages before the
    previous kernel has finished, which is only sound because the prompt pass has synchronised. Same tokens
    and logits with the option off."""
    cfg, w = model
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (150, 33, 260)]
    outs = []
    for overlap in (True, False):
        e = Engine(kv_pool_gb=0.3, max_batch=4, max_seq_len=512, prefill_chunk=128, config=cfg, weights=w,
                   prologue_overlap=overlap)
        ids = [e.add_request(p, 6, ignore_eos=True) for p in prompts]
        got, logits = {i: [] for i in ids}, []
        while e.stats()["running"] or e.stats()["waiting"]:
            before = e.stats()["decode_tokens"]
            for rid, tok, fin, why in e.step():
                got[rid].append(tok)
            if e.stats()["decode_tokens"] != before:
                logits.append(e.exec.logits[:3].cpu().numpy().view(np.uint16).copy())
        outs.append((got, np.stack(logits)))
        assert all(len(v) == 6 for v in got.values())
    K.set_attention_prologue_overlap(True)
    assert outs[0][0] == outs[1][0]
    assert np.array_equal(outs[0][1], outs[1][1])
    assert K.attention_health() == 0


def test_chunked_prompt_pass_fused_attention_agrees_with_the_composite(model):
    """A 1500-token prompt ingested in chunks of 512 (so later chunks attend to earlier chunks' pages through the
    block table, and the last chunk is ragged) through the fused paged prefill kernel and through the reference's
    composite (gather -> scores -> causal softmax -> P.V around library products): the logits of the first
    generated token agree within the logit tolerance, the greedy tokens of a short continuation agree wherever
    the margin is not a near-tie, and the K/V pages the two passes leave in the pool are identical (both scatter
    the same rotated K and V; attention only reads them) for the first layer and within FP16 noise after it."""
    cfg, w = model
    rng = np.random.default_rng(41)
    prompt = rng.integers(0, cfg.vocab, 1500).tolist()
    runs = {}
    for mode in ("fused", "composite"):
        e = Engine(kv_pool_gb=0.3, max_batch=2, max_seq_len=2048, prefill_chunk=512, config=cfg, weights=w,
                   prefill_attention=mode)
        e.add_request(prompt, 5, ignore_eos=True)
        toks, first_logits = [], None
        while e.stats()["running"] or e.stats()["waiting"]:
            for rid, tok, fin, why in e.step():
                toks.append(tok)
            if first_logits is None and toks:
                first_logits = e.exec.prefill_logits.float().cpu().numpy()[0]
                layer0 = e.exec.pool[0].clone()
        runs[mode] = (toks, first_logits, layer0)
        assert len(toks) == 5
        assert K.prefill_attention_health() == 0
    (tf, lf, p0f), (tc, lc, p0c) = runs["fused"], runs["composite"]
    assert torch.equal(p0f, p0c), "layer 0's pages depend only on the embedding, the norm, the QKV product and RoPE"
    scale = float(np.abs(lc).max())
    assert np.abs(lf - lc).max() <= LOGIT_TOL_FRAC * scale
    srt = np.sort(lc)
    assert tf[0] == tc[0] or srt[-1] - srt[-2] <= 2 * LOGIT_TOL_FRAC * scale
