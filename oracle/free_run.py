"""Whole-decode greedy-token check of the shipped path against an independent GPU path (TEST INFRASTRUCTURE).

Protocol (the reference's own, src/core/request.hpp:33-41, src/core/scheduler.cpp:290-296,
docs/DESIGN.md:655-709 of the reference): the path under test decodes FREE-RUNNING - every sampled
token is fed back - while a second engine over the same weights and the same cache contents is
TEACHER-FORCED onto those tokens (`forced_tokens`), so both see the same history at every step and every
step of every sequence is comparable, not only the prefix before a first disagreement. Per step and
sequence the checker's own greedy choice is compared with the token the path under test produced; the
first step where they differ is that sequence's `first_divergence` (up to and including that step the
checker's choices are exactly what it would have produced free-running, by induction over the shared
history). A disagreement is accepted only where it is a near-tie: the checker's top-1 / runner-up margin
at that step must lie within the logit tolerance, and the two paths' logits must agree within that
tolerance at every step regardless. A bounded sample of steps - every first divergence up to a cap, and a
fixed sparse set of steps for a few sequences - is recomputed on the host cores by the composition of
the reference's CPU functions (oracle/decode_step.py) for a third, independent opinion.

The path under test is `Engine(...)` with its defaults (tcgen05 linear layers, fused epilogues, dependent
launch, CUDA-graph replay). The checker engine runs eagerly with library GEMMs, the unfused launch
sequence of the reference's executor (src/core/model_executor.cpp:908-957) and, where
oracle/_ref/libredline_refkernels.so was built, the REFERENCE'S OWN CUDA KERNELS for every non-GEMM stage;
elsewhere this library's unfused launchers with the one-warp-per-head cross-check attention kernel.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import ref_kernels


class _OwnUnfusedKernels:
    """This library's launchers with attention routed to the textbook cross-check kernel."""

    def __init__(self):
        from redline_llm_b200 import kernels as K
        self._K = K

    def __getattr__(self, name):
        return getattr(self._K, name)

    def launch_paged_attention_decode(self, *a, **kw):
        kw["check_kernel"] = True
        return self._K.launch_paged_attention_decode(*a, **kw)


def checker_kind() -> str:
    return "reference_cuda_kernels" if ref_kernels.available() else "own_unfused_check_kernel"


def make_checker_engine(cfg, weights, kv_pool_gb, max_batch, max_seq_len, device=0, prologue_overlap=True):
    """An engine over the same weights whose every stage is independent of the path under test."""
    from redline_llm_b200.engine import Engine
    e = Engine(kv_pool_gb=kv_pool_gb, max_batch=max_batch, max_seq_len=max_seq_len, config=cfg, weights=weights,
               device=device, enable_cuda_graphs=False, decode_linear="library", vocab_projection="library",
               prologue_overlap=prologue_overlap)
    e.exec.K = ref_kernels if ref_kernels.available() else _OwnUnfusedKernels()
    e.exec.fuse_rope_scatter = False
    e.exec.fuse_qkv_rope = False
    return e


def lockstep_decode(cfg, weights, contexts: Sequence[int], new_tokens: int, seed: int, device: int = 0,
                    engine_kwargs: Optional[dict] = None, cpu_audit_steps: Sequence[int] = (),
                    cpu_audit_rows: Sequence[int] = (), cpu_audit_divergences: int = 0,
                    cpu_row_limit: int = 8192, logit_tol_frac: float = 0.01) -> Dict:
    """Decodes `new_tokens` tokens of len(contexts) cached sequences (synthetic seeded K/V, as the benchmark's)
    free-running through the default engine and teacher-forced through the checker engine; returns the
    report described in the module docstring. `logit_tol_frac` x (largest |logit| seen) is the logit
    tolerance. Sequences longer than `cpu_row_limit` tokens are never recomputed on the host."""
    import torch
    from redline_llm_b200.engine import Engine, blocks_for_tokens
    from redline_llm_b200 import kernels as K

    n = len(contexts)
    rows = 64 if n > 48 else next(b for b in (1, 2, 4, 8, 16, 32, 48) if b >= n)
    max_seq = max(contexts) + new_tokens + 16
    blocks = sum(blocks_for_tokens(c + new_tokens) for c in contexts) + 8
    gb = blocks * cfg.block_bytes() / (1 << 30)
    kw = dict(kv_pool_gb=gb, max_batch=max(n, 1), max_seq_len=max_seq, config=cfg, weights=weights, device=device,
              graph_buckets=[rows])
    kw.update(engine_kwargs or {})
    a = Engine(**kw)
    b = make_checker_engine(cfg, weights, gb, max(n, 1), max_seq, device,
                            prologue_overlap=kw.get("prologue_overlap", True))
    for i, c in enumerate(contexts):
        a.add_synthetic_request(int(c), new_tokens, seed=seed + i)
        b.add_synthetic_request(int(c), new_tokens, seed=seed + i)
    reqs_b = list(b.scheduler.running)
    for r in reqs_b:
        r.forced_tokens = []

    dec = None
    audits: List[dict] = []
    audited_divergences = 0

    def cpu_audit(step: int, rws: List[int], why: str, tok_a, tok_b):
        nonlocal dec
        from oracle.decode_step import CpuDecoder
        rws = [r for r in rws if contexts[r] + step <= cpu_row_limit]
        if not rws:
            return
        if dec is None:
            dec = CpuDecoder(cfg, weights, use_ref=True)
        _, cpu_tok, cpu_logits = dec.step(a.exec, rws)
        got = a.exec.logits[rws].float().cpu().numpy()
        for j, r in enumerate(rws):
            srt = np.sort(cpu_logits[j])
            err = float(np.abs(got[j] - cpu_logits[j]).max())
            audits.append({"step": step, "sequence": r, "why": why, "context": int(contexts[r]) + step,
                           "cpu_token": int(cpu_tok[j]), "token": int(tok_a[r]), "checker_token": int(tok_b[r]),
                           "cpu_top1_top2_margin": float(srt[-1] - srt[-2]),
                           "cpu_margin_to_token": float(srt[-1] - cpu_logits[j, int(tok_a[r])]),
                           "cpu_margin_to_checker_token": float(srt[-1] - cpu_logits[j, int(tok_b[r])]),
                           "logits_max_abs_vs_cpu": err, "cpu_logit_scale": float(np.abs(cpu_logits[j]).max())})

    first_div = [-1] * n
    disagreements: List[dict] = []
    tokens_a = np.zeros((n, new_tokens), np.int32)
    worst_logit_diff, scale = 0.0, 0.0
    t0 = time.perf_counter()
    for step in range(new_tokens):
        out_a = a.step()
        tok_a = np.asarray([t for (_, t, _, _) in out_a], np.int32)
        assert len(tok_a) == n
        tokens_a[:, step] = tok_a
        for r, t in zip(reqs_b, tok_a):
            r.forced_tokens.append(int(t))
        b.step()
        la, lb = a.exec.logits[:n].float(), b.exec.logits[:n].float()
        tok_b = b.exec.tokens[:n].cpu().numpy()
        diff = (la - lb).abs().amax(dim=1)
        worst_logit_diff = max(worst_logit_diff, float(diff.max()))
        scale = max(scale, float(lb.abs().max()))
        bad = np.flatnonzero(tok_a != tok_b)
        new_div = []
        if len(bad):
            top2 = torch.topk(lb[torch.as_tensor(bad, device=lb.device)], 2, dim=1).values.cpu().numpy()
            lb_bad = lb[torch.as_tensor(bad, device=lb.device)].cpu().numpy()
            for j, s in enumerate(bad):
                s = int(s)
                disagreements.append({"step": step, "sequence": s, "context": int(contexts[s]) + step,
                                      "token": int(tok_a[s]), "checker_token": int(tok_b[s]),
                                      "checker_top1_top2_margin": float(top2[j, 0] - top2[j, 1]),
                                      "checker_margin_to_token": float(top2[j, 0] - lb_bad[j, int(tok_a[s])]),
                                      "logit_diff_row": float(diff[s])})
                if first_div[s] < 0:
                    first_div[s] = step
                    new_div.append(s)
        if new_div and audited_divergences < cpu_audit_divergences:
            take = [s for s in new_div if contexts[s] + step <= cpu_row_limit][:cpu_audit_divergences - audited_divergences]
            audited_divergences += len(take)
            cpu_audit(step, take, "first divergence", tok_a, tok_b)
        if step in cpu_audit_steps and cpu_audit_rows:
            cpu_audit(step, list(cpu_audit_rows), "sparse step", tok_a, tok_b)
    wall = time.perf_counter() - t0
    tol = logit_tol_frac * scale
    agree = n * new_tokens - len(disagreements)
    report = {
        "sequences": n, "tokens": new_tokens, "contexts_min_max": [int(min(contexts)), int(max(contexts))],
        "contexts_over_4096": int(sum(1 for c in contexts if c > 4096)),
        "path": {k: str(v) for k, v in dict(decode_linear=a.exec.decode_linear, vocab_projection=a.exec.vocab_projection,
                                            cuda_graph=rows in a.exec.graphs,
                                            prologue_overlap=kw.get("prologue_overlap", True)).items()},
        "checker": checker_kind() + ", library GEMMs, eager, unfused",
        "agreeing_steps": agree, "compared_steps": n * new_tokens,
        "first_divergence": first_div, "sequences_never_diverging": int(sum(1 for f in first_div if f < 0)),
        "disagreements": len(disagreements),
        "max_disagreement_margin": max((d["checker_top1_top2_margin"] for d in disagreements), default=0.0),
        "max_margin_to_token": max((d["checker_margin_to_token"] for d in disagreements), default=0.0),
        "logits_max_abs_between_paths": worst_logit_diff, "logit_scale": scale, "logit_tolerance": tol,
        "every_disagreement_within_tolerance": all(d["checker_margin_to_token"] <= 2 * tol for d in disagreements),
        "cpu_audits": audits, "attention_health": K.attention_health(), "linear_health": K.decode_linear_health(),
        "seconds": round(wall, 2),
        "disagreement_list": disagreements, "tokens_free_running": tokens_a,
    }
    return report


def audits_ok(report: Dict, slack: float = 2.5) -> bool:
    """Every host-recomputed step: each GPU path's token is the host's token, or the host's margin to it is
    within `slack` x that row's logit error against the host (a coin flip, not a kernel bug)."""
    for au in report["cpu_audits"]:
        lim = slack * max(au["logits_max_abs_vs_cpu"], 1e-3)
        if au["token"] != au["cpu_token"] and au["cpu_margin_to_token"] > lim:
            return False
        if au["checker_token"] != au["cpu_token"] and au["cpu_margin_to_checker_token"] > lim:
            return False
    return True


def config5_wave_contexts(seed: int, n: int = 64, long_rows: int = 1) -> List[int]:
    """One admission wave of the benchmark's decode-step workload: contexts uniform in [1024, 8192] plus
    `long_rows` sequences of 32768 tokens (which the attention kernel cuts across many CTAs)."""
    from redline_llm_b200 import workloads as wl
    ctx = [int(c) for c in wl.randint(seed, n - long_rows, 1024, 8192)] + [32768] * long_rows
    perm = wl.permutation(seed + 1, n)
    return [ctx[i] for i in perm]
