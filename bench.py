#!/usr/bin/env python
"""Benchmark of the non-GEMM decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0). Workloads (synthetic, seeded; shapes from the benchmark
configurations): `attention` = paged GQA decode attention, batch 64, contexts U[1024,1280],
28 layer pools walked per step so every launch reads KV that is cold in L2; `norm`, `rope_scatter`,
`silu` = the other kernels at their configuration shapes (reported in "kernels" on every run).

`value` is the aggregate over all ranks with inputs resident in HBM; `e2e` is the same metric through
the public host API with pinned host buffers copied in and the result copied out inside the timed
region; `roofline` is for the dominant kernel (attention), timed live with CUDA events.
`--impl reference` times the reference's own CPU implementation (oracle/_ref when it was compiled,
else this repository's CPU restatement) on the host cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from redline_llm_b200 import workloads as wl  # noqa: E402

LAYERS = 28
METRIC = "decode-kernel HBM GB/s"
# dram__bytes_read+write / algorithmic bytes of the attention kernel in the ncu capture at batch 64,
# contexts 4096-8192 (400.5 MB / 397.3 MB); the config-3 capture gives 78.4 / 75.7 = 1.036
ATTENTION_TRAFFIC_RATIO = 1.008


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    """Measured dense bf16 GEMM peak (TFLOP/s, burst) of this pool's B200s; the stated fallback otherwise."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"])
    return 1590.0


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dev(a):
    import torch
    a = np.ascontiguousarray(a)
    return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()


def graphed(fn):
    """Captures one call of fn (launches on the current stream) in a CUDA graph; returns the replay
    callable. The decode path this library serves runs as CUDA-graph replays, and replaying keeps
    the host-side launch cost out of device timings."""
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g.replay


def time_region(fn, steps, stream_sync, finish=None):
    """CUDA-event time (ms) of `steps` calls of fn on the current stream; `finish` (e.g. retiring steps still in
    flight) runs inside the region, after the last call."""
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream_sync()
    start.record()
    for _ in range(steps):
        fn()
    if finish is not None:
        finish()
    end.record()
    stream_sync()
    return start.elapsed_time(end)


# ----------------------------------------------------------------- workloads

class AttentionWorkload:
    """Config 3: batch 64, contexts U[1024,1280], 12 Q / 2 KV heads, d=128, 16-token pages behind a
    random-permuted block table; one step = one attention call per layer pool (28)."""
    name = "paged_attention_b64_ctx1024-1280"

    def __init__(self, rank: int, layers: int = LAYERS, lo: int = 1024, hi: int = 1280):
        import torch
        from redline_llm_b200 import kernels as K
        self.K, self.torch, self.layers = K, torch, layers
        self.name = f"paged_attention_b64_ctx{lo}-{hi}"
        blocks = max(8192, 64 * ((hi + 15) // 16) + 64)
        c = wl.config_attention(seed=wl.SEED_ATTN + 16 * rank, lo=lo, hi=hi, num_blocks=blocks)
        self.c = c
        self.bytes_per_launch = wl.attention_bytes(c["seq_lens"])
        self.tokens = int(np.asarray(c["seq_lens"]).sum())
        base = dev(c["pool"])
        # 28 layer pools: the same page structure, contents rotated so no two layers alias in L2
        self.pools = [base] + [torch.roll(base, 4096 * (i + 1)) for i in range(layers - 1)]
        # live slots must stay NaN-free after the roll: refill every pool's NaN slots is unnecessary for
        # timing, but results are checked on pool 0 only (unrolled).
        self.q = dev(np.pad(c["q"], ((0, 0), (0, 512))))  # rows 2048 apart, as in the fused QKV buffer
        self.tables, self.lens = dev(c["tables"]), dev(c["seq_lens"])
        self.out = torch.zeros(64, 1536, dtype=torch.int16, device="cuda")
        self.mbps = c["tables"].shape[1]
        # pinned host mirrors for the end-to-end leg
        self.h_q = torch.from_numpy(np.pad(c["q"], ((0, 0), (0, 512))).view(np.int16)).pin_memory()
        self.h_tables = torch.from_numpy(c["tables"]).pin_memory()
        self.h_lens = torch.from_numpy(np.asarray(c["seq_lens"], np.int32)).pin_memory()
        self.h_out = torch.empty(64, 1536, dtype=torch.int16).pin_memory()
        self.h2d = self.h_q.numel() * 2 + self.h_tables.numel() * 4 + self.h_lens.numel() * 4
        self.d2h = self.h_out.numel() * 2
        self.launches_per_step = layers  # one kernel per attention call
        K.init()

    def attend(self, pool):
        self.K.launch_paged_attention_decode(self.out, 1536, self.q, 2048, pool, self.tables, self.lens, 64,
                                             self.mbps, 12, 2, 128, self.c["scale"])

    def step(self):
        for pool in self.pools:
            self.attend(pool)

    def step_e2e(self):
        self.q.copy_(self.h_q, non_blocking=True)
        self.tables.copy_(self.h_tables, non_blocking=True)
        self.lens.copy_(self.h_lens, non_blocking=True)
        self.step()
        self.h_out.copy_(self.out, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    def bytes_per_step(self):
        return self.bytes_per_launch * self.layers

    def check(self):
        """Pool 0's result against the CPU checker on 4 sequences (cheap sanity, not the parity suite)."""
        import oracle
        self.attend(self.pools[0])
        got = self.out.cpu().numpy().view(np.uint16)[:4]
        c = self.c
        ref = oracle.own().paged_attention(c["q"][:4], c["pool"], c["tables"][:4], c["seq_lens"][:4], 12, 2, 128,
                                           c["scale"], f64out=True)
        return float(np.abs(oracle.half_bits_to_f64(got) - ref).max())


class DecodeStepWorkload:
    """Config 5: one decode step of a random-init Qwen2.5-1.5B-architecture model (28 layers, hidden 1536,
    FFN 8960, 12 Q / 2 KV heads, d=128, vocab 151936, FP16 ~N(0,0.02)) over 512 sequences - 480 with contexts
    U[1024,8192] and 32 of 32768 tokens - sharded evenly over the ranks and decoded in waves of 64 (the
    engine's largest CUDA-graph bucket). One step = one new token for every sequence of the job. The KV
    cache is filled with seeded ~N(0,1) values in place of a prompt pass (prompt ingestion is not the
    measured path)."""
    name = "decode_step_qwen2.5-1.5b_512seq_ctx1024-8192+32x32768"
    TOTAL, LONG, WAVE, NEW = 512, 32, 64, 256

    def __init__(self, rank: int, world: int, new_tokens: int = 256, total: int = 512, overlap: bool = True,
                 linear: str = "tcgen05", vocab_projection: str = None):
        import torch
        self.TOTAL, self.LONG = total, total // 16
        self.linear = linear
        self.vocab_projection = vocab_projection or linear
        from redline_llm_b200.engine import (Engine, ModelConfig, ModelWeights, balanced_order, blocks_for_tokens,
                                             shard_requests)
        self.torch = torch
        # the host-side router: longest first, snake-dealt over 8 shards, so that at every GPU count each GPU serves
        # the same number of 32 768-token sequences and (within ~1 %) the same number of cached tokens
        ctx = decode_step_contexts(self.TOTAL)
        mine = [int(ctx[i]) for i in shard_requests(self.TOTAL, world, rank)]
        self.cfg = ModelConfig()
        dev = torch.device("cuda", torch.cuda.current_device())
        self.weights = ModelWeights(self.cfg, dev, seed=0x5EED)
        self.engines, self.lens = [], []
        max_seq = 32768 + new_tokens + 16
        for w0 in range(0, len(mine), self.WAVE):
            wave = mine[w0:w0 + self.WAVE]
            blocks = sum(blocks_for_tokens(c + new_tokens) for c in wave) + 8
            gb = blocks * self.cfg.block_bytes() / (1 << 30)
            e = Engine(kv_pool_gb=gb, max_batch=self.WAVE, max_seq_len=max_seq, config=self.cfg, weights=self.weights,
                       device=dev.index, graph_buckets=[64], prologue_overlap=overlap, decode_linear=linear,
                       vocab_projection=self.vocab_projection)
            for j, c in enumerate(wave):
                e.add_synthetic_request(c, new_tokens, seed=wl.SEED_STEP + 1000 * rank + w0 + j)
            self.engines.append(e)
            self.lens.append(wave)
        self.tokens_per_step = len(mine)
        wts = self.weights
        self.weight_bytes = sum(t.numel() * 2 for L in wts.layers for t in L.values()) + wts.final_norm.numel() * 2 \
            + wts.lm_head.numel() * 2  # streamed once per wave per step (the embedding rows gathered are negligible)
        self.kv_bytes_per_token = self.cfg.layers * 2 * self.cfg.kv_heads * self.cfg.head_dim * 2
        # own kernels per layer: 2 norms and attention, plus RoPE+scatter and SiLU beside library GEMMs, or the
        # four linear layers (RoPE+scatter fused into the QKV product, SiLU into gate/up); + embed, final norm, argmax,
        # the device-side input advance
        # and, with the own linear kernel, the vocabulary projection
        self.launches_per_step = len(self.engines) * (self.cfg.layers * (7 if linear == "tcgen05" else 5) + 4
                                                      + (1 if self.vocab_projection == "tcgen05" else 0))
        self.h2d = self.d2h = 0

    def step(self):  # inputs already resident: graph replays only
        for e in self.engines:
            e.exec.run(self.WAVE)

    def step_e2e(self):
        """One step of every wave through the public API: pinned H2D of the step's control block (and of ids /
        positions / seq_lens / changed table rows whenever the host has to rebuild them), graph replay, D2H of
        the sampled tokens. `step_pipelined` launches a wave's next step behind the one in flight - the device
        feeds the sampled tokens back itself - and then retires the older one, so the host's bookkeeping runs
        under the device's work; every step's tokens are still read on the host, one call late."""
        self.h2d = self.d2h = 0
        for e in self.engines:
            e.step_pipelined()
            self.h2d += e.exec.h2d_bytes
            self.d2h += 4 * self.WAVE

    def drain(self):
        for e in self.engines:
            e.drain()

    def resident_inputs(self):
        """Uploads every wave's next inputs once, device-side advance off: `step()` then replays over them."""
        self.drain()
        for e in self.engines:
            assert e.upload_next_inputs() == self.WAVE

    def profile_attention(self, replays: int = 3):
        """The attention kernel's own duration inside this step: for every wave, the step's 28 attention
        launches (same q, tables, seq_lens and the 28 layer pools, 11-12 GB of KV per wave, cold in L2)
        captured alone in a CUDA graph and timed with CUDA events on the launching stream. Returns
        (mean seconds per launch, mean algorithmic bytes per launch)."""
        torch = self.torch
        secs, nbytes = [], []
        for e in self.engines:
            ex, cfg = e.exec, self.cfg
            lens = ex.seq_lens[:self.WAVE].cpu().numpy()

            def sweep(ex=ex, cfg=cfg):
                for li in range(cfg.layers):
                    ex.K.launch_paged_attention_decode(ex.attn[:self.WAVE], cfg.q_width, ex.qkv[:self.WAVE], cfg.qkv_width,
                                                       ex.pool[li], ex.tables, ex.seq_lens, self.WAVE, ex.mbps,
                                                       cfg.q_heads, cfg.kv_heads, cfg.head_dim, ex.scale)
            replay = graphed(sweep)
            replay()
            ms = time_region(replay, replays, torch.cuda.synchronize)
            secs.append(ms * 1e-3 / (replays * cfg.layers))
            nbytes.append(wl.attention_bytes(lens))
        return float(np.mean(secs)), float(np.mean(nbytes))


def sample_rows(w: "DecodeStepWorkload", n: int = 2):
    """The n sequences of wave 0 whose contexts are closest to the job's mean context."""
    mean = float(np.mean([c for wave in w.lens for c in wave]))
    order = np.argsort(np.abs(np.asarray(w.lens[0], np.float64) - mean))
    return sorted(int(i) for i in order[:n])


def cpu_decode_step(w: "DecodeStepWorkload", rows, use_ref: bool):
    """One decode step of the sequences `rows` (indices into wave 0) on the host cores, composed from the
    reference's CPU functions and BLAS FP32 GEMMs (oracle/decode_step.py). Returns (seconds, tokens, logits,
    threads, kind); weight conversion and the cache download are outside the timed part."""
    from oracle.decode_step import CpuDecoder
    if getattr(w, "_cpu_decoder", None) is None:
        w._cpu_decoder = CpuDecoder(w.cfg, w.weights, use_ref)
    dec = w._cpu_decoder
    dt, tokens, logits = dec.step(w.engines[0].exec, rows)
    return dt, tokens, logits, dec.threads, dec.kind


def kernel_table(peak, only=None, eager=False):
    """Achieved GB/s of every kernel at its configuration shape (and a large-T shape where the stated one is
    latency-bound and L2-resident), CUDA-event timed over rotating buffers larger than L2. `only` keeps the
    entries whose name contains it; `eager` launches directly instead of replaying a CUDA graph (profilers)."""
    import torch
    from redline_llm_b200 import kernels as K
    from oracle import ref_kernels as R     # the reference's own CUDA kernels, when oracle/_ref holds them: `ref_us`
    have_ref = R.available()
    out = {}

    def want(name):
        return only is None or only in name

    def timed(fn, nbuf, iters=20):
        def sweep():
            for i in range(nbuf):
                fn(i)
        replay = sweep if eager else graphed(sweep)
        for _ in range(3):
            replay()
        t = time_region(replay, iters, torch.cuda.synchronize)
        return t * 1e-3 / (iters * nbuf)

    def both(fn, nbuf, iters=20):
        """fn(module, i): the same launch through this library and through the reference's kernel library."""
        return timed(lambda i: fn(K, i), nbuf, iters), (timed(lambda i: fn(R, i), nbuf, iters) if have_ref else None)

    def report(name, secs, nbytes, note, ref_secs=None):
        out[name] = {"us": round(secs * 1e6, 3), "GB/s": round(nbytes / secs / 1e9, 1),
                     "frac_of_measured_peak": round(nbytes / secs / 1e9 / peak, 4), "bytes": nbytes, "note": note}
        if ref_secs is not None:
            out[name].update({"ref_us": round(ref_secs * 1e6, 3), "ref_GB/s": round(nbytes / ref_secs / 1e9, 1),
                              "speedup_vs_ref_kernel": round(ref_secs / secs, 2)})

    for t, note in ((64, "config 1; latency-bound, L2-resident"), (16384, "large-T, cold L2")):
        if not want(f"rmsnorm_residual_T{t}"):
            continue
        c = wl.config_rmsnorm(64)
        nbuf = max(2, min(64, int(3e8 // (t * 1536 * 8)) + 1))
        x = [dev(np.tile(c["x"], (t // 64, 1))) for _ in range(nbuf)]
        r = [dev(np.tile(c["residual"], (t // 64, 1))) for _ in range(nbuf)]
        o = [torch.empty(t, 1536, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        w = dev(c["weight"])
        secs, rsecs = both(lambda M, i: M.launch_rms_norm_residual(o[i], r[i], x[i], w, t, 1536, 1e-6), nbuf)
        report(f"rmsnorm_residual_T{t}", secs, 4 * t * 1536 * 2 + 1536 * 2, note, rsecs)
        del x, r, o
    if want("rope_T64") or want("kv_scatter_T64"):
        c = wl.config_rope_scatter(64)
        nbuf = 8
        qkv = [dev(c["qkv"]) for _ in range(nbuf)]
        pos, tab = dev(c["positions"]), dev(c["tables"])
        pool = torch.zeros(8192 * 2 * 2 * 16 * 128, dtype=torch.int16, device="cuda")
        if want("rope_T64"):
            secs, rsecs = both(lambda M, i: M.launch_rope_inplace(qkv[i], qkv[i], 2048, 2048, pos, 64, 12, 2, 128, 1e6,
                                                         k_offset=1536), nbuf)
            report("rope_T64", secs, 2 * 64 * 1792 * 2 + 256, "config 2; latency-bound", rsecs)
        if want("kv_scatter_T64"):
            secs, rsecs = both(lambda M, i: M.launch_kv_scatter(pool, qkv[i], qkv[i], 2048, 2048, tab, tab.shape[1], pos, 64,
                                                       2, 128, k_offset=1536, v_offset=1792), nbuf)
            report("kv_scatter_T64", secs, 64 * 1024 * 2 + 64 * 8, "config 2; latency-bound", rsecs)
        del pool, qkv
    for t, note in ((64, "config 4; L2-resident"), (512, "config 4; L2-resident"), (4096, "config 4; HBM-bound")):
        if not want(f"silu_mul_T{t}"):
            continue
        g = wl.config_silu(64)["gate_up"]
        nbuf = max(2, min(64, int(3e8 // (t * 8960 * 6)) + 1))
        bufs = [dev(np.tile(g, (t // 64, 1))) for _ in range(nbuf)]
        # dense output buffers: writing in place would feed each launch the previous launch's results, which
        # decay towards subnormals over the timed iterations; bytes moved are the same (2 reads + 1 write)
        outs = [torch.empty(t, 8960, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        secs, rsecs = both(lambda M, i: M.launch_silu_mul(outs[i], bufs[i], t, 8960), nbuf)
        report(f"silu_mul_T{t}", secs, 3 * t * 8960 * 2, note + "; dense out", rsecs)
        del bufs, outs
    if want("greedy_argmax_64x151936"):
        nbuf = 8
        lg = [dev(wl.normal_half(0xA46 + i, 64 * 151936).reshape(64, 151936)) for i in range(nbuf)]
        tok = torch.zeros(64, dtype=torch.int32, device="cuda")
        secs, rsecs = both(lambda M, i: M.launch_greedy_argmax(tok, lg[i], 64, 151936), nbuf)
        report("greedy_argmax_64x151936", secs, 64 * 151936 * 2 + 64 * 4, "decode batch of logits; 8-CTA clusters per row", rsecs)
        del lg
    if want("embed_gather_T64"):
        table = dev(wl.normal_half(0xE1, 32768 * 1536).reshape(32768, 1536))
        ids = dev(wl.randint(0xE2, 64, 0, 32767))
        o = [torch.empty(64, 1536, dtype=torch.int16, device="cuda") for _ in range(8)]
        secs, rsecs = both(lambda M, i: M.launch_embed_gather(o[i], 1536, table, ids, 64, 1536), 8)
        report("embed_gather_T64", secs, 2 * 64 * 1536 * 2 + 64 * 4, "latency-bound", rsecs)
        del table, o
    if want("rope_kv_scatter_fused_T64"):
        c = wl.config_rope_scatter(64)
        qkv = [dev(c["qkv"]) for _ in range(8)]
        pos, tab = dev(c["positions"]), dev(c["tables"])
        pool = torch.zeros(8192 * 2 * 2 * 16 * 128, dtype=torch.int16, device="cuda")
        secs = timed(lambda i: K.launch_rope_kv_scatter(qkv[i], 2048, pool, tab, tab.shape[1], pos, 64, 12, 2, 128, 1e6), 8)

        def ref_pair(i):   # what the reference's executor launches for the same work
            R.launch_rope_inplace(qkv[i], qkv[i], 2048, 2048, pos, 64, 12, 2, 128, 1e6, k_offset=1536)
            R.launch_kv_scatter(pool, qkv[i], qkv[i], 2048, 2048, tab, tab.shape[1], pos, 64, 2, 128, k_offset=1536, v_offset=1792)
        report("rope_kv_scatter_fused_T64", secs, 2 * 64 * 1792 * 2 + 64 * 1536 + 64 * 8 + 256,
               "config 2 in one launch; latency-bound; ref_us = the reference's two launches", timed(ref_pair, 8) if have_ref else None)
        del pool, qkv
    # the same three kernels at a prompt chunk's size: 16384 consecutive positions of one sequence (one table
    # row shared by every token, row stride 0, as prompt ingestion calls them), buffers rotated past L2
    big = ("rope_T16384", "kv_scatter_T16384", "rope_kv_scatter_fused_T16384")
    if any(want(n) for n in big):
        t, nbuf = 16384, 10
        src = wl.normal_half(0x2B1, 64 * 2048).reshape(64, 2048)
        qkv = [dev(np.tile(src, (t // 64, 1))) for _ in range(nbuf)]
        pos = torch.arange(t, dtype=torch.int32, device="cuda")
        row = dev((wl.permutation(0x2B2, 2047)[:t // 16] + 1).astype(np.int32).reshape(1, -1))
        pools = [torch.zeros(2048 * 2 * 2 * 16 * 128, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        rope_bytes = 2 * t * 1792 * 2 + t * 4
        if want(big[0]):
            secs, rsecs = both(lambda M, i: M.launch_rope_inplace(qkv[i], qkv[i], 2048, 2048, pos, t, 12, 2, 128, 1e6,
                                                         k_offset=1536), nbuf, iters=5)
            report(big[0], secs, rope_bytes, "prompt chunk, cold L2", rsecs)
        if want(big[1]):
            secs, rsecs = both(lambda M, i: M.launch_kv_scatter(pools[i], qkv[i], qkv[i], 2048, 2048, row, 0, pos, t,
                                                       2, 128, k_offset=1536, v_offset=1792), nbuf, iters=5)
            report(big[1], secs, 2 * t * 1024 + t * 4 + t // 4, "prompt chunk, cold L2; strided 1 KiB reads", rsecs)
        if want(big[2]):
            secs = timed(lambda i: K.launch_rope_kv_scatter(qkv[i], 2048, pools[i], row, 0, pos, t, 12, 2, 128, 1e6),
                         nbuf, iters=5)

            def ref_pair_big(i):
                R.launch_rope_inplace(qkv[i], qkv[i], 2048, 2048, pos, t, 12, 2, 128, 1e6, k_offset=1536)
                R.launch_kv_scatter(pools[i], qkv[i], qkv[i], 2048, 2048, row, 0, pos, t, 2, 128, k_offset=1536, v_offset=1792)
            report(big[2], secs, rope_bytes + t * 1536 + t // 4, "prompt chunk in one launch, cold L2; ref_us = the "
                   "reference's two launches", timed(ref_pair_big, nbuf, iters=5) if have_ref else None)
        del qkv, pools
    # the two prompt-side launchers at one chunk of a long prompt: the gather of a 16384-token context into
    # the dense staging views, and the causal softmax of a 512-row chunk against 8192 keys
    if want("kv_gather_ctx16384"):
        ctx, nbuf = 16384, 10
        row = dev((wl.permutation(0x2B3, 2047)[:ctx // 16] + 1).astype(np.int32))
        pools = [dev(wl.normal_half(0x2B4 + (i & 1), 2048 * 2 * 2 * 16 * 128)) for i in range(nbuf)]
        kh = [torch.empty(2, ctx, 128, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        vh = [torch.empty(2, ctx, 128, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        secs, rsecs = both(lambda M, i: M.launch_kv_gather(kh[i], vh[i], ctx * 128, 128, ctx * 128, 128, pools[i], row, ctx,
                                                  2, 128), nbuf, iters=5)
        report("kv_gather_ctx16384", secs, 2 * ctx * 1024 + ctx // 4, "one sequence's pages into dense K, V; cold L2", rsecs)
        del pools, kh, vh
    if want("prefill_softmax_12x512x8192"):
        h, c, kv, start, nbuf = 12, 512, 8192, 7680, 2
        sc = [torch.randn(h, c, kv, dtype=torch.float32, device="cuda",
                          generator=torch.Generator("cuda").manual_seed(0x2B6 + i)) * 2.5 for i in range(nbuf)]
        pr = [torch.empty(h, c, kv, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        secs, rsecs = both(lambda M, i: M.launch_prefill_softmax(pr[i], sc[i], h, c, kv, start), nbuf, iters=5)
        live = sum(min(start + r + 1, kv) for r in range(c))
        report("prefill_softmax_12x512x8192", secs, h * (live * 4 + c * kv * 2),
               "chunk rows 7680..8191 against 8192 keys: live FP32 scores read once, FP16 probabilities written", rsecs)
        del sc, pr
    # paged attention at the configuration's shape (batch 64, contexts U[1024,1280]) and at long contexts
    # (U[4096,8192]), layer pools rotated past L2; the reference's kernel walks each (sequence, head) serially
    for name, (lo, hi, layers) in (("paged_attention_b64_ctx1024-1280", (1024, 1280, 10)),
                                   ("paged_attention_b64_ctx4096-8192", (4096, 8192, 3))):
        if not want(name):
            continue
        aw = AttentionWorkload(0, layers, lo, hi)
        secs, rsecs = both(lambda M, i: M.launch_paged_attention_decode(aw.out, 1536, aw.q, 2048, aw.pools[i], aw.tables,
                                                                        aw.lens, 64, aw.mbps, 12, 2, 128, aw.c["scale"]),
                           layers, iters=10)
        report(name, secs, aw.bytes_per_launch, f"{layers} layer pools in rotation, cold L2", rsecs)
        del aw
    # fused paged prefill attention: one prompt chunk of 2048 rows at the start of a prompt and deep inside one
    # (context 8192), against the composite it replaces (gather -> FP32 scores -> causal softmax -> P.V, the two
    # products by the library); compute-bound, so the figure of merit is FLOP/s against the measured GEMM peak
    for name, (start, n) in (("paged_prefill_attention_rows2048_ctx2048", (0, 2048)),
                             ("paged_prefill_attention_rows2048_ctx8192", (6144, 2048))):
        if not want(name):
            continue
        end = start + n
        blocks = end // 16
        c = wl.config_attention(lens=[end], num_blocks=blocks + 8, seed=0x9F1 + start, fill="uniform")
        pool, row = dev(c["pool"]), dev(np.ascontiguousarray(c["tables"][0]))
        qkv = [dev(wl.normal_half(0x9F3 + i, n * 2048).reshape(n, 2048)) for i in range(2)]
        outs = [torch.empty(n, 1536, dtype=torch.int16, device="cuda") for _ in range(2)]
        secs = timed(lambda i: K.launch_paged_prefill_attention(outs[i], 1536, qkv[i], 2048, pool, row, blocks, start, n,
                                                                12, 2, 128, c["scale"]), 2, iters=5)
        khat = torch.empty(2, end, 128, dtype=torch.float16, device="cuda")
        vhat = torch.empty_like(khat)
        probs = torch.empty(12, n, end, dtype=torch.float16, device="cuda")

        def composite(i):
            K.launch_kv_gather(khat, vhat, end * 128, 128, end * 128, 128, pool, row, end, 2, 128)
            q = qkv[i].view(torch.float16)[:, :1536].view(n, 12, 128).permute(1, 0, 2)
            sc = torch.bmm(q.float(), khat.repeat_interleave(6, 0).float().transpose(1, 2)) * c["scale"]
            K.launch_prefill_softmax(probs, sc, 12, n, end, start)
            return torch.bmm(probs, vhat.repeat_interleave(6, 0))
        for _ in range(2):
            composite(0)
        csecs = time_region(lambda: composite(0), 3, torch.cuda.synchronize) * 1e-3 / 3
        flops = 12 * 4 * 128 * sum(start + r + 1 for r in range(n))
        tpeak = tensor_peak()
        out[name] = {"us": round(secs * 1e6, 2), "TFLOP/s": round(flops / secs / 1e12, 1),
                     "frac_of_measured_tensor_peak": round(flops / secs / 1e12 / tpeak, 4), "flops": flops,
                     "bytes": 2 * n * 1536 * 2 + end * 1024 + blocks * 4,
                     "composite_us": round(csecs * 1e6, 2), "speedup_vs_composite": round(csecs / secs, 2),
                     "note": "causal flops only (4 * 128 per query-key pair); tensor peak = measured cuBLAS bf16 burst; "
                             "composite = kv_gather + FP32 torch.bmm + causal softmax + FP16 torch.bmm, eager"}
        del pool, qkv, outs, khat, vhat, probs
    # the four linear layers of a decoder block at 64 token rows: weight streams (28 distinct weights, cold L2)
    for name, (n_out, k_in, epi, with_bias) in (("decode_linear_qkv_T64", (2048, 1536, 0, True)),
                                                 ("decode_linear_o_T64", (1536, 1536, 0, False)),
                                                 ("decode_linear_gate_up_silu_T64", (8960, 1536, 1, False)),
                                                 ("decode_linear_down_T64", (1536, 8960, 0, False))):
        if not want(name):
            continue
        nbuf = 28
        rows = 2 * n_out if epi else n_out
        ws = [dev(wl.normal_half(0x11A + i, rows * k_in, 0.0, k_in ** -0.5).reshape(rows, k_in)) for i in range(2)]
        ws += [ws[i % 2].clone() for i in range(nbuf - 2)]
        xs = dev(wl.normal_half(0x11B, 64 * k_in).reshape(64, k_in))
        bias = dev(wl.normal_half(0x11C, n_out)) if with_bias else None
        o = torch.empty(64, n_out, dtype=torch.int16, device="cuda")
        secs = timed(lambda i: K.launch_decode_linear(o, xs, ws[i], bias, num_tokens=64, epilogue=epi), nbuf)
        report(name, secs, rows * k_in * 2 + 64 * k_in * 2 + 64 * n_out * 2 + (n_out * 2 if with_bias else 0),
               "tcgen05 weight stream; bytes = weights + activations in + out"
               + ("; SiLU-mul fused, [T, 2I] never stored" if epi else ""))
        del ws, o
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------ CPU reference

def cpu_attention(sample_seqs: int, use_ref: bool):
    """The CPU implementation of paged attention on `sample_seqs` sequences of config 3; returns
    (GB/s on the algorithmic bytes of that sample, cores, kind, sample description, seconds)."""
    import oracle
    c = wl.config_attention()
    n = sample_seqs
    q, tables, lens = c["q"][:n], c["tables"][:n], np.asarray(c["seq_lens"][:n])
    nbytes = wl.attention_bytes(lens)
    ref = oracle.ref() if use_ref else None
    t0 = time.perf_counter()
    if ref is not None:
        cores = max(1, ref.hardware_threads())
        ref.paged_attention(q, c["pool"], tables, lens, 12, 2, 128, c["scale"], threads=cores)
        kind = "reference"
    else:
        own = oracle.own()
        cores = own.threads()
        own.paged_attention(q, c["pool"], tables, lens, 12, 2, 128, c["scale"])
        kind = "port"
    dt = time.perf_counter() - t0
    return nbytes / dt / 1e9, cores, kind, f"{n} of 64 sequences of config 3, one layer pool, FP64 two-pass softmax", dt


def reference_line(args, metric, unit, value, ms_per_step, config, cpu, dtype, steps, warmup, note):
    """`steps` / `warmup` are the counts that were actually run and timed (the request may be capped)."""
    return {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if unit == "tok/s" else "weak", "vs_baseline": None, "dtype": dtype,
            "data": "synthetic", "config": config, "cpu_baseline": cpu, "note": note,
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


REFERENCE_ARM_BUDGET_S = 90.0   # host seconds the timed steps of the reference arm may take in total


def decode_step_contexts(total: int = 512):
    """Context lengths of the decode-step workload in serving order (host arithmetic only): total - total/16
    uniform in [1024, 8192] plus total/16 of 32768 tokens, shuffled, then ordered by the host-side router."""
    from redline_llm_b200.engine import balanced_order
    long_rows = total // 16
    ctx = np.concatenate([wl.randint(wl.SEED_STEP, total - long_rows, 1024, 8192), np.full(long_rows, 32768, np.int32)])
    ctx = ctx[wl.permutation(wl.SEED_STEP + 1, total)]
    return ctx[balanced_order(ctx, shards=8, seed=wl.SEED_STEP + 2)]


def decode_step_config(total, world, extra=None):
    """The workload description both arms print (static facts only; what was measured goes elsewhere)."""
    c = {"workload": DecodeStepWorkload.name, "sequences": total, "wave": DecodeStepWorkload.WAVE, "new_tokens": 256,
         "contexts": "480 uniform in [1024, 8192] + 32 of 32768 (x sequences/512)", "model": "Qwen2.5-1.5B architecture, "
         "random init FP16 ~N(0,0.02): 28 layers, hidden 1536, FFN 8960, 12 Q / 2 KV heads, d=128, vocab 151936",
         "sharding": "sequences dealt over the GPUs by a host-side router, decoded in waves of 64 per GPU"}
    c.update(extra or {})
    return c


def run_reference_arm(args, rank, world):
    """The reference's own CPU implementation of the path on the host cores (rank 0 only). Inputs are generated
    on the host from the same seeded streams; neither a GPU nor this repository's CUDA library is touched."""
    if rank != 0:
        return
    if args.workload == "attention":
        cores = os.cpu_count() or 1
        n = min(64, max(8, 2 * cores))
        first = cpu_attention(n, True)                                   # also the warm-up
        steps = max(1, min(args.steps, int(REFERENCE_ARM_BUDGET_S / max(first[4], 1e-3))))
        runs = [cpu_attention(n, True) for _ in range(steps)]
        value = float(np.mean([r[0] for r in runs]))
        cpu = {"value": round(value, 4), "unit": "GB/s", "cores": runs[0][1], "kind": runs[0][2], "sample": runs[0][3]}
        print(json.dumps(reference_line(
            args, METRIC, "GB/s", round(value, 4), round(1e3 * float(np.mean([r[4] for r in runs])), 3),
            {"workload": AttentionWorkload.name, "batch_per_gpu": 64}, cpu, "f64", steps, 1,
            f"each step is a bounded sample ({n} of 64 sequences) on the host cores; {steps} of the {args.steps} "
            f"requested steps fit the {REFERENCE_ARM_BUDGET_S:.0f} s budget")), flush=True)
        return
    from oracle.decode_step import CpuDecoder, HostWeights, host_step_inputs
    from redline_llm_b200.engine import ModelConfig
    cfg = ModelConfig()
    ctx = decode_step_contexts(args.sequences)
    wave0 = [int(c) for c in ctx[0::max(1, args.gpus)][:DecodeStepWorkload.WAVE]]
    mean = float(np.mean(ctx))
    rows = sorted(int(i) for i in np.argsort(np.abs(np.asarray(wave0, np.float64) - mean))[:2])
    sample_ctx = [wave0[i] for i in rows]
    dec = CpuDecoder(cfg, HostWeights(cfg, seed=0x5EED), use_ref=True)
    inputs = host_step_inputs(cfg, sample_ctx, wl.SEED_STEP + 77)
    scale = 1.0 / float(np.sqrt(cfg.head_dim))

    def one():
        ids, pos, lens, ctab, pools = inputs
        return dec.step_host(ids, pos, lens, ctab, [p.copy() for p in pools], scale)[0]
    first = one()                                                        # warm-up (page faults, BLAS threads)
    steps = max(1, min(args.steps, int(REFERENCE_ARM_BUDGET_S / max(first, 1e-3))))
    times = [one() for _ in range(steps)]
    dt = float(np.mean(times))
    value = len(rows) / dt
    cpu = {"value": round(value, 4), "unit": "tok/s", "cores": dec.threads, "kind": dec.kind,
           "sample": f"{len(rows)} sequences x 1 decode step, all 28 layers, contexts {sample_ctx} (closest to the "
                     f"job's mean context); tok/s is per {len(rows)}-sequence step as run - the 3.1 GB of weights are "
                     f"amortised over {len(rows)} tokens, not extrapolated to a 64-row batch; BLAS FP32 GEMMs"}
    print(json.dumps(reference_line(
        args, "decode tok/s", "tok/s", round(value, 4), round(1e3 * dt, 3), decode_step_config(args.sequences, world),
        cpu, "f64 kernels / f32 GEMM", steps, 1,
        f"each step is a bounded sample of the workload on the host cores; {steps} of the {args.steps} requested "
        f"steps fit the {REFERENCE_ARM_BUDGET_S:.0f} s budget, after 1 warm-up step")), flush=True)


def run_attention(args, rank, local_rank, world, barrier, dist):
    import torch
    w = AttentionWorkload(rank, args.layers, args.ctx_lo, args.ctx_hi)
    max_abs = w.check()
    peak, peak_kind = measured_peaks()
    step = w.step if args.no_graph else graphed(w.step)
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            step()
        barrier()
        ms = time_region(step, args.steps, barrier)
    for _ in range(2):
        w.step_e2e()
    barrier()
    ms_e2e = time_region(w.step_e2e, args.steps, barrier)
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    health = w.K.attention_health()
    if rank != 0:
        return
    total_bytes = w.bytes_per_step() * world
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    per_launch_s = ms * 1e-3 / (args.steps * args.layers)
    achieved = w.bytes_per_launch / per_launch_s / 1e9
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage / f32 accumulate", "data": "synthetic",
        "config": {"workload": w.name, "batch_per_gpu": 64, "layers_per_step": args.layers,
                   "kv_tokens_per_layer": w.tokens,
                   "cold_l2": f"{args.layers} layer pools walked per step ({args.layers * 0.134:.1f} GB)",
                   "launch": "eager" if args.no_graph else "cuda_graph_replay",
                   "prologue_overlap": not args.no_overlap,
                   "pct_of_8TBps": round(100 * achieved / 8000.0, 2)},
        "roofline": {"bound": "hbm", "kernel": "PagedAttentionSplitKernel",
                     "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "peak_kind": f"of {peak_kind}",
                     "traffic": int(w.bytes_per_launch * (1.036 if args.ctx_hi <= 2048 else ATTENTION_TRAFFIC_RATIO)),
                     "traffic_note": "dram read+write per launch from the ncu capture of this kernel "
                                     "(profiles/paged_attention_split_kernel.txt), scaled by units processed",
                     "algorithmic_bytes_per_launch": w.bytes_per_launch, "us_per_launch": round(per_launch_s * 1e6, 3)},
        "e2e": {"value": round(e2e, 2), "unit": "GB/s", "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h},
        "gpu_launches": w.launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "check": {"attention_max_abs_vs_cpu_checker": max_abs, "attention_health": health},
    }
    if not args.no_kernel_table:
        line["kernels"] = kernel_table(peak)
    if not args.no_cpu_baseline and world == 1:
        cores = os.cpu_count() or 1
        gbs, cores_used, kind, sample, dt = cpu_attention(min(64, max(8, 2 * cores)), True)
        line["cpu_baseline"] = {"value": round(gbs, 4), "unit": "GB/s", "cores": cores_used, "kind": kind,
                                "sample": sample, "seconds": round(dt, 2)}
    print(json.dumps(line), flush=True)


def timed_repeats(fn, steps, repeats, barrier, finish=None):
    """`repeats` timed regions of exactly `steps` calls each (CUDA events, barrier + synchronize on both sides)."""
    return [time_region(fn, steps, barrier, finish) for _ in range(repeats)]


def spread(tokens, steps, ms_list):
    v = sorted(tokens * steps / (m * 1e-3) for m in ms_list)
    return {"median": round(float(np.median(v)), 1), "min": round(v[0], 1), "max": round(v[-1], 1), "repeats": len(v)}


def free_running_check(cfg, weights, quick: bool):
    """The whole greedy decode of one wave of the workload (64 sequences, one of 32768 tokens, 256 new tokens)
    through the shipped path, against the independent path (oracle/free_run.py). Returns the report without
    its per-token arrays."""
    from oracle import free_run
    contexts = free_run.config5_wave_contexts(0xB200C0F5, 64, long_rows=1)
    order = np.argsort(contexts)
    rep = free_run.lockstep_decode(cfg, weights, contexts, 64 if quick else 256, seed=0x5EED0000,
                                   cpu_audit_steps=(0,) if quick else (0, 255), cpu_audit_rows=[int(order[2])],
                                   cpu_audit_divergences=2)
    rep.pop("tokens_free_running")
    listed = rep.pop("disagreement_list")
    rep["audits_ok"] = free_run.audits_ok(rep)
    rep["disagreement_margins"] = sorted(round(d["checker_margin_to_token"], 4) for d in listed)[-8:]
    for au in rep["cpu_audits"]:
        for k in list(au):
            if isinstance(au[k], float):
                au[k] = round(au[k], 5)
    return rep


def run_decode_step(args, rank, local_rank, world, barrier, dist):
    import torch
    from redline_llm_b200 import kernels as K
    need = args.warmup + (2 * args.repeats + 1) * args.steps + 8
    w = DecodeStepWorkload(rank, world, new_tokens=max(256, need), total=args.sequences, overlap=not args.no_overlap,
                           linear=args.linear, vocab_projection=args.vocab_projection)
    peak, peak_kind = measured_peaks()
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            w.step_e2e()
        w.resident_inputs()       # nothing in flight; every wave's next inputs on the device, advance off
        barrier()
        ms_all = timed_repeats(w.step, args.steps, args.repeats, barrier)
        barrier()
        # each region launches exactly `steps` steps per wave and retires them all before its end event
        ms_e2e_all = timed_repeats(w.step_e2e, args.steps, args.repeats, barrier, finish=w.drain)
        w.resident_inputs()       # for the attention profile and the CPU check below
    att_s, att_bytes = w.profile_attention()
    if world > 1:
        t = torch.tensor(ms_all + ms_e2e_all, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)      # every region: the slowest rank's time
        ms_all, ms_e2e_all = t[:args.repeats].tolist(), t[args.repeats:].tolist()
    ms, ms_e2e = float(np.median(ms_all)), float(np.median(ms_e2e_all))
    health = K.attention_health()
    linear_health = K.decode_linear_health()
    tokens = w.TOTAL
    # HBM bytes one step must move on this rank: the weights once per wave, every cached token's K/V once
    # (at the contexts the timed replays saw), the new tokens' K/V written
    ctx_now = sum(int(e.exec.seq_lens[:DecodeStepWorkload.WAVE].sum().item()) for e in w.engines)
    step_bytes = len(w.engines) * w.weight_bytes + (ctx_now + w.tokens_per_step) * w.kv_bytes_per_token
    step_gbs = step_bytes / (ms * 1e-3 / args.steps) / 1e9
    value = tokens * args.steps / (ms * 1e-3)
    e2e = tokens * args.steps / (ms_e2e * 1e-3)
    achieved = att_bytes / att_s / 1e9
    line = None
    if rank == 0:
        line = {
            "metric": "decode tok/s", "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage / f32 accumulate", "data": "synthetic",
            "config": decode_step_config(tokens, world),
            "details": {
                "sequences_per_gpu": w.tokens_per_step, "waves_per_gpu": len(w.engines),
                "launch": "one CUDA-graph replay per wave", "prologue_overlap": not args.no_overlap,
                "router": "host-side: longest first, snake-dealt over 8 shards (every GPU serves 32/N of the "
                          "32768-token sequences and the same number of cached tokens within 1 %)",
                "gemm": ("own tcgen05 weight-streaming kernel for the four linear layers of a block (RoPE + KV scatter "
                         "fused into QKV, SiLU into gate/up) FP16" if args.linear == "tcgen05"
                         else "library (cuBLAS via torch.matmul), FP16"),
                "vocabulary_projection": ("own tcgen05 kernel" if w.vocab_projection == "tcgen05"
                                          else "library GEMM (torch.matmul)"),
                "cold_l2": "every step streams 3.1 GB of weights per wave and the waves' KV, far larger than L2",
                "attention_pct_of_8TBps": round(100 * achieved / 8000.0, 2),
                "step_hbm_bytes_per_gpu": int(step_bytes), "step_GBps_per_gpu": round(step_gbs, 1),
                "step_frac_of_measured_hbm": round(step_gbs / peak, 4),
                "step_pct_of_8TBps": round(100 * step_gbs / 8000.0, 2)},
            "timing": {"repeats": args.repeats, "value": spread(tokens, args.steps, ms_all),
                       "e2e": spread(tokens, args.steps, ms_e2e_all),
                       "note": "value / e2e / ms_per_step are the medians of `repeats` timed regions of `steps` steps each"},
            "roofline": {"bound": "hbm", "kernel": "PagedAttentionSplitKernel", "achieved": round(achieved, 1),
                         "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                         "traffic": int(att_bytes * ATTENTION_TRAFFIC_RATIO),
                         "traffic_note": "dram read+write per launch scaled by units from the ncu capture at batch 64, "
                                         "contexts 4096-8192 (profiles/paged_attention_split_kernel.txt): 1.008 x algorithmic",
                         "algorithmic_bytes_per_launch": int(att_bytes),
                         "us_per_launch": round(att_s * 1e6, 2),
                         "timed": "CUDA events over graph replays of the step's 28 attention launches per wave "
                                  "(same inputs and layer pools as the step, cold L2)"},
            "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h},
            "gpu_launches": w.launches_per_step * args.steps * 2 * args.repeats * world,
            "clocks": clocks.summary(),
            "check": {"attention_health": health, "linear_health": linear_health},
        }
    cfg, weights = w.cfg, w.weights
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        rows = sample_rows(w, 2)
        dt, cpu_tok, cpu_logits, threads, kind = cpu_decode_step(w, rows, True)
        e = w.engines[0]
        e.exec.enqueue_decode(DecodeStepWorkload.WAVE)   # same inputs as the CPU sample saw
        torch.cuda.synchronize()
        gpu_logits = e.exec.logits[rows].float().cpu().numpy()
        gpu_tok = e.exec.tokens[rows].cpu().numpy()
        line["cpu_baseline"] = {"value": round(len(rows) / dt, 4), "unit": "tok/s", "cores": threads, "kind": kind,
                                "sample": f"{len(rows)} sequences of wave 0 (contexts {[w.lens[0][i] for i in rows]}, "
                                          "closest to the job's mean) x 1 decode step, all 28 layers",
                                "seconds": round(dt, 2)}
        line["check"].update({"step_logits_max_abs_vs_cpu": float(np.abs(gpu_logits - cpu_logits).max()),
                              "step_logits_scale": float(np.abs(cpu_logits).max()),
                              "greedy_tokens_equal_cpu": bool((gpu_tok == cpu_tok).all())})
    del w
    torch.cuda.empty_cache()
    # The same step with the library GEMMs left in place (cuBLAS through torch.matmul for the four linear layers of
    # a block and the vocabulary projection; this library's norm / RoPE / scatter / attention / SiLU kernels around
    # them): the configuration in which only the non-GEMM kernels are replaced.
    if args.linear == "tcgen05" and not args.no_library_leg:
        reps = max(1, min(3, args.repeats))
        wl_lib = DecodeStepWorkload(rank, world, new_tokens=max(256, args.warmup + (2 * reps + 1) * args.steps + 8),
                                    total=args.sequences, overlap=not args.no_overlap, linear="library")
        for _ in range(args.warmup):
            wl_lib.step_e2e()
        wl_lib.resident_inputs()
        barrier()
        lib_ms = timed_repeats(wl_lib.step, args.steps, reps, barrier)
        barrier()
        lib_e2e = timed_repeats(wl_lib.step_e2e, args.steps, reps, barrier, finish=wl_lib.drain)
        if world > 1:
            t = torch.tensor(lib_ms + lib_e2e, device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            lib_ms, lib_e2e = t[:reps].tolist(), t[reps:].tolist()
        if rank == 0:
            line["value_library_gemm"] = spread(tokens, args.steps, lib_ms)["median"]
            line["e2e_library_gemm"] = spread(tokens, args.steps, lib_e2e)["median"]
            line["timing"]["value_library_gemm"] = spread(tokens, args.steps, lib_ms)
            line["timing"]["e2e_library_gemm"] = spread(tokens, args.steps, lib_e2e)
            line["gpu_launches"] += wl_lib.launches_per_step * args.steps * 2 * reps * world
        del wl_lib
        torch.cuda.empty_cache()
    if rank != 0:
        return
    if not args.no_free_running and world == 1:
        line["check"]["free_running"] = free_running_check(cfg, weights, args.quick_check)
    del weights
    torch.cuda.empty_cache()
    if not args.no_kernel_table:
        line["kernels"] = kernel_table(peak)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_step", choices=["decode_step", "attention", "kernels"])
    ap.add_argument("--no-kernel-table", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="attention workload: eager launches instead of graph replay")
    ap.add_argument("--layers", type=int, default=LAYERS, help="attention workload: layer pools walked per step")
    ap.add_argument("--ctx-lo", type=int, default=1024, help="attention workload: shortest context")
    ap.add_argument("--ctx-hi", type=int, default=1280, help="attention workload: longest context")
    ap.add_argument("--sequences", type=int, default=512,
                    help="decode_step workload: sequences in the job (512 = the configuration; fewer for profiling)")
    ap.add_argument("--linear", choices=["tcgen05", "library"], default="tcgen05",
                    help="decode_step: linear layers by this library's tcgen05 kernel (default) or by the library GEMM")
    ap.add_argument("--vocab-projection", choices=["tcgen05", "library"], default=None,
                    help="decode_step: the vocabulary projection by this library's kernel or by the library GEMM (default: as --linear)")
    ap.add_argument("--linear-stages", type=int, default=None, help="ring depth of the tcgen05 linear kernel (2..8)")
    ap.add_argument("--linear-splits", type=int, default=None, help="largest K split of the tcgen05 linear kernel (1,2,4,8)")
    ap.add_argument("--no-overlap", action="store_true",
                    help="plain attention launches (no programmatic dependent launch of the prologue)")
    ap.add_argument("--kernel", default=None, help="kernels workload: only entries whose name contains this")
    ap.add_argument("--repeats", type=int, default=5, help="decode_step: timed regions of --steps steps each; the line carries the median")
    ap.add_argument("--no-library-leg", action="store_true", help="decode_step: skip the extra timed pass with the library GEMMs")
    ap.add_argument("--no-free-running", action="store_true", help="decode_step: skip the whole-decode greedy check (N=1 only)")
    ap.add_argument("--quick-check", action="store_true", help="decode_step: 64 instead of 256 tokens in the whole-decode check")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from redline_llm_b200 import kernels as _K
    _K.set_attention_prologue_overlap(not args.no_overlap)
    if args.linear_stages is not None:
        _K.set_decode_linear_stages(args.linear_stages)
    if args.linear_splits is not None:
        _K.set_decode_linear_max_splits(args.linear_splits)
    if args.workload == "kernels":
        peak, kind = measured_peaks()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unit": "GB/s", "peak": peak, "peak_kind": f"of {kind}",
                              "launch": "eager" if args.no_graph else "cuda_graph_replay",
                              "kernels": kernel_table(peak, args.kernel, args.no_graph)}), flush=True)
    elif args.workload == "attention":
        run_attention(args, rank, local_rank, world, barrier, dist)
    else:
        run_decode_step(args, rank, local_rank, world, barrier, dist)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
