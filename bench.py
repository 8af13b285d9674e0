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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def time_region(fn, steps, stream_sync):
    """CUDA-event time (ms) of `steps` calls of fn on the current stream."""
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream_sync()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    stream_sync()
    return start.elapsed_time(end)


# ----------------------------------------------------------------- workloads

class AttentionWorkload:
    """Config 3: batch 64, contexts U[1024,1280], 12 Q / 2 KV heads, d=128, 16-token pages behind a
    random-permuted block table; one step = one attention call per layer pool (28)."""
    name = "paged_attention_b64_ctx1024-1280"

    def __init__(self, rank: int, layers: int = LAYERS):
        import torch
        from redline_llm_b200 import kernels as K
        self.K, self.torch, self.layers = K, torch, layers
        c = wl.config_attention(seed=wl.SEED_ATTN + 16 * rank)
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


def kernel_table(peak):
    """Achieved GB/s of every kernel at its configuration shape (and a large-T shape where the stated one is
    latency-bound and L2-resident), CUDA-event timed, rotating buffers larger than L2."""
    import torch
    from redline_llm_b200 import kernels as K
    out = {}

    def timed(fn, nbuf, iters=20):
        def sweep():
            for i in range(nbuf):
                fn(i)
        replay = graphed(sweep)
        for _ in range(3):
            replay()
        t = time_region(replay, iters, torch.cuda.synchronize)
        return t * 1e-3 / (iters * nbuf)

    def report(name, secs, nbytes, note):
        out[name] = {"us": round(secs * 1e6, 3), "GB/s": round(nbytes / secs / 1e9, 1),
                     "frac_of_measured_peak": round(nbytes / secs / 1e9 / peak, 4), "bytes": nbytes, "note": note}

    for t, note in ((64, "config 1; latency-bound, L2-resident"), (16384, "large-T, cold L2")):
        c = wl.config_rmsnorm(64)
        nbuf = max(2, min(64, int(3e8 // (t * 1536 * 8)) + 1))
        x = [dev(np.tile(c["x"], (t // 64, 1))) for _ in range(nbuf)]
        r = [dev(np.tile(c["residual"], (t // 64, 1))) for _ in range(nbuf)]
        o = [torch.empty(t, 1536, dtype=torch.int16, device="cuda") for _ in range(nbuf)]
        w = dev(c["weight"])
        secs = timed(lambda i: K.launch_rms_norm_residual(o[i], r[i], x[i], w, t, 1536, 1e-6), nbuf)
        report(f"rmsnorm_residual_T{t}", secs, 4 * t * 1536 * 2 + 1536 * 2, note)
        del x, r, o
    c = wl.config_rope_scatter(64)
    nbuf = 8
    qkv = [dev(c["qkv"]) for _ in range(nbuf)]
    pos, tab = dev(c["positions"]), dev(c["tables"])
    pool = torch.zeros(8192 * 2 * 2 * 16 * 128, dtype=torch.int16, device="cuda")
    secs = timed(lambda i: K.launch_rope_inplace(qkv[i], qkv[i], 2048, 2048, pos, 64, 12, 2, 128, 1e6, k_offset=1536), nbuf)
    report("rope_T64", secs, 2 * 64 * 1792 * 2 + 256, "config 2; latency-bound")
    secs = timed(lambda i: K.launch_kv_scatter(pool, qkv[i], qkv[i], 2048, 2048, tab, tab.shape[1], pos, 64, 2, 128,
                                               k_offset=1536, v_offset=1792), nbuf)
    report("kv_scatter_T64", secs, 64 * 1024 * 2 + 64 * 8, "config 2; latency-bound")
    del pool, qkv
    for t, note in ((64, "config 4; L2-resident"), (512, "config 4; L2-resident"), (4096, "config 4; HBM-bound")):
        g = wl.config_silu(64)["gate_up"]
        nbuf = max(2, min(64, int(3e8 // (t * 8960 * 4)) + 1))
        bufs = [dev(np.tile(g, (t // 64, 1))) for _ in range(nbuf)]
        secs = timed(lambda i: K.launch_silu_mul(bufs[i], bufs[i], t, 8960), nbuf)
        report(f"silu_mul_T{t}", secs, 3 * t * 8960 * 2, note)
        del bufs
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


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    n = min(64, max(8, 2 * cores))
    vals = []
    for _ in range(args.warmup):
        cpu_attention(n, True)
    for _ in range(args.steps):
        gbs, cores_used, kind, sample, dt = cpu_attention(n, True)
        vals.append((gbs, dt))
    total_t = sum(d for _, d in vals)
    value = float(np.mean([g for g, _ in vals]))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * total_t / max(1, args.steps), 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": AttentionWorkload.name, "batch": 64, "layers_per_step": LAYERS,
                   "note": "each step is a bounded sample of the workload on the host cores"},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores_used, "kind": kind, "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="attention", choices=["attention"])
    ap.add_argument("--no-kernel-table", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="eager launches instead of CUDA-graph replay")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layer pools walked per step (28 = the model)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

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

    w = AttentionWorkload(rank, args.layers)
    max_abs = w.check()
    peak, peak_kind = measured_peaks()

    step = w.step if args.no_graph else graphed(w.step)
    for _ in range(args.warmup):
        step()
    barrier()
    with ClockSampler(local_rank) as clocks:
        ms = time_region(step, args.steps, barrier)
    for _ in range(2):
        w.step_e2e()
    barrier()
    t0 = time.perf_counter()
    ms_e2e_dev = time_region(w.step_e2e, args.steps, barrier)
    ms_e2e = max(ms_e2e_dev, 0.0)
    _ = time.perf_counter() - t0

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    health = w.K.attention_health()

    if rank == 0:
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
                       "kv_tokens_per_layer": w.tokens, "cold_l2": "28 layer pools (2.1 GB) walked per step, larger than L2",
                       "launch": "eager" if args.no_graph else "cuda_graph_replay",
                       "pct_of_8TBps": round(100 * achieved / 8000.0, 2)},
            "roofline": {"bound": "hbm", "kernel": "PagedAttentionSplitKernel",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "peak_kind": f"of {peak_kind}", "traffic": None,
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
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
