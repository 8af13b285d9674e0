"""The drop-in, proven with the reference's own host: `redline.Engine` - the reference's pybind module
(src/api/pybind.cpp:98-215) over its unmodified engine, scheduler, executor (src/core/engine.cpp:296-373,
src/core/model_executor.cpp:894-961 decode inside graph capture, :1154-1217 prefill), cuBLASLt wrapper and
loader - compiled against this library's kernels.cuh and linked to libredline_b200.so
(oracle/_ref/host_b200, built by `make -C oracle gpuref` where the reference tree is mounted).

It loads a random-init checkpoint of the real architecture written by tests/ref_host.py, is driven
through add_request / step / has_capacity / stats only, and is compared with
 (1) the whole reference engine - the same host over the reference's own CUDA kernels
     (oracle/_ref/host_ref) - teacher-forced onto that engine's tokens, so every position is scored, and
 (2) this repository's Python engine on the same weights,
a disagreement being accepted only where the Python engine's logits at that position show a near-tie
(the reference's margin-audit protocol, docs/DESIGN.md:655-709 of the reference)."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import ref_kernels  # noqa: E402
from redline_llm_b200.engine import Engine, ModelConfig, ModelWeights  # noqa: E402
from tests import ref_host  # noqa: E402

ENGINE_KW = dict(kv_pool_gb=0.5, max_batch=8, enable_cuda_graphs=True, max_seq_len=512, prefill_chunk=128)
NEW = 24
LOGIT_TOL_FRAC = 0.01   # of the largest |logit|: what separates a coin flip from a bug in this suite


def _have(module_dir):
    return os.path.isdir(module_dir) and any(f.startswith("redline.") for f in os.listdir(module_dir))


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not _have(ref_kernels.HOST_B200_DIR):
        pytest.skip("oracle/_ref/host_b200 (the reference's host over this library) was never built")
    cfg = ModelConfig()
    w = ModelWeights(cfg, torch.device("cuda", 0), seed=0x5EED)
    d = ref_host.write_model_dir(str(tmp_path_factory.mktemp("ckpt")), cfg, w)
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, 151000, n).tolist() for n in (5, 33, 130, 64, 17, 200)]
    return cfg, w, d, prompts


def _requests(prompts, forced=None):
    return [{"prompt": p, "max_new_tokens": NEW, "forced_tokens": None if forced is None else forced[i]}
            for i, p in enumerate(prompts)]


def _python_engine_audit(cfg, w, prompts, forced):
    """This repository's engine teacher-forced onto `forced`: per request its own greedy choices and, per
    position, the top-1/runner-up margin and the logit scale."""
    e = Engine(kv_pool_gb=ENGINE_KW["kv_pool_gb"], max_batch=8, max_seq_len=512, prefill_chunk=128, config=cfg, weights=w,
               decode_linear="library")
    ids = [e.add_request(p, NEW, ignore_eos=True, forced_tokens=forced[i]) for i, p in enumerate(prompts)]
    own = {i: [] for i in ids}
    margin = {i: [] for i in ids}
    scale = 0.0
    for _ in range(10000):
        before = e.stats()["decode_tokens"]
        res = e.step()
        if res:
            if e.stats()["decode_tokens"] == before:   # the token of a finished prompt pass
                lg = e.exec.prefill_logits.float()
            else:
                lg = e.exec.logits[:len(res)].float()
            top2 = torch.topk(lg, 2, dim=1).values.cpu().numpy()
            scale = max(scale, float(lg.abs().max()))
            for j, (rid, tok, fin, why) in enumerate(res):
                own[rid].append(tok)
                margin[rid].append(float(top2[j, 0] - top2[j, 1]))
        s = e.stats()
        if s["running"] == 0 and s["waiting"] == 0:
            break
    return [own[i] for i in ids], [margin[i] for i in ids], scale


def test_reference_host_runs_over_this_library(model):
    cfg, w, d, prompts = model
    out = ref_host.run_host(ref_kernels.HOST_B200_DIR, d, _requests(prompts), ENGINE_KW)
    assert out["version"] == "0.1.0"
    assert all(len(t) == NEW for t in out["tokens"]) and out["reasons"] == ["length"] * len(prompts)
    assert all(out["had_capacity"])
    s = out["stats"]
    assert set(s) == {"steps", "prefill_tokens", "decode_tokens", "waiting", "running", "free_blocks",
                      "reserved_blocks", "total_blocks", "graph_replays", "eager_decodes", "aborts",
                      "bucket_histogram"}
    assert s["prefill_tokens"] == sum(len(p) for p in prompts)
    assert s["decode_tokens"] == len(prompts) * (NEW - 1)
    assert s["graph_replays"] > 0 and s["eager_decodes"] == 0          # the decode ran inside CUDA graphs
    assert s["free_blocks"] == s["total_blocks"] - 1 and s["reserved_blocks"] == 0 and s["aborts"] == 0
    assert out["errors"] == {"empty_prompt": "ValueError", "token_outside_vocabulary": "ValueError"}
    # the greedy stream is a real one: not one token repeated, all inside the vocabulary
    flat = [t for ts in out["tokens"] for t in ts]
    assert len(set(flat)) > len(flat) // 4 and all(0 <= t < cfg.vocab for t in flat)

    # (2) against this repository's Python engine on the same weights, teacher-forced onto the host's tokens
    own, margin, scale = _python_engine_audit(cfg, w, prompts, out["tokens"])
    tol = LOGIT_TOL_FRAC * scale
    diff = [(i, k) for i in range(len(prompts)) for k in range(NEW) if own[i][k] != out["tokens"][i][k]]
    assert len(diff) <= 0.08 * len(prompts) * NEW, diff
    assert all(margin[i][k] <= 2 * tol for i, k in diff), [(i, k, margin[i][k]) for i, k in diff]
    print(f"reference host over this library vs the Python engine: {len(prompts) * NEW - len(diff)}/"
          f"{len(prompts) * NEW} positions agree; disagreements at margins "
          f"{[round(margin[i][k], 4) for i, k in diff]} (tolerance {2 * tol:.4f})")


def test_drop_in_agrees_with_the_whole_reference_engine(model):
    cfg, w, d, prompts = model
    if not _have(ref_kernels.HOST_REF_DIR):
        pytest.skip("oracle/_ref/host_ref (the reference's host over its own kernels) was never built")
    ref = ref_host.run_host(ref_kernels.HOST_REF_DIR, d, _requests(prompts), ENGINE_KW)
    assert all(len(t) == NEW for t in ref["tokens"])
    # teacher-forced onto the reference engine's continuation: step() reports the engine's own argmax
    # at every position (src/core/request.hpp:33-41)
    got = ref_host.run_host(ref_kernels.HOST_B200_DIR, d, _requests(prompts, ref["tokens"]), ENGINE_KW)
    _, margin, scale = _python_engine_audit(cfg, w, prompts, ref["tokens"])
    tol = LOGIT_TOL_FRAC * scale
    diff = [(i, k) for i in range(len(prompts)) for k in range(NEW) if got["tokens"][i][k] != ref["tokens"][i][k]]
    first = [next((k for k in range(NEW) if got["tokens"][i][k] != ref["tokens"][i][k]), -1) for i in range(len(prompts))]
    print(f"drop-in vs the reference engine: {len(prompts) * NEW - len(diff)}/{len(prompts) * NEW} positions "
          f"agree, first divergence per request {first}, margins {[round(margin[i][k], 4) for i, k in diff]} "
          f"(tolerance {2 * tol:.4f}); reference engine {ref['step_seconds']} s, drop-in {got['step_seconds']} s")
    assert len(diff) <= 0.08 * len(prompts) * NEW, diff
    assert all(margin[i][k] <= 2 * tol for i, k in diff), [(i, k, margin[i][k]) for i, k in diff]
    assert got["stats"]["decode_tokens"] == ref["stats"]["decode_tokens"]
    assert got["stats"]["bucket_histogram"] == ref["stats"]["bucket_histogram"]
