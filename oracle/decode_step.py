"""One decode step of the whole model on the host cores (TEST INFRASTRUCTURE).

The reference has no CPU implementation of a whole decode step; this composes one from its CPU
functions for every non-GEMM stage (tests/reference/*.hpp compiled into oracle/_ref, or this
repository's C restatement where those were never built) in the executor's layer order
(src/core/model_executor.cpp:908-957), with BLAS FP32 GEMMs whose results are rounded to FP16 once
(the FP16-in / FP32-accumulate / FP16-out contract of the library GEMMs). It is the checker of the
engine's logits and tokens and the timed CPU baseline of the decode-step benchmark; the shipped
path never imports it.
"""
from __future__ import annotations

import time

import numpy as np

import oracle


def _u16(t):
    return t.detach().cpu().numpy().view(np.uint16)


def _f32(bits):
    return np.ascontiguousarray(bits).view(np.float16).astype(np.float32)


def _f32_weight(t):
    """A weight tensor (torch, FP16) as a float32 numpy array; torch's vectorised widening, not numpy's."""
    return t.detach().cpu().float().numpy()


def _h16(a):
    with np.errstate(over="ignore"):
        return a.astype(np.float16).view(np.uint16)


class CpuDecoder:
    """Holds FP32 copies of the model's GEMM weights (converted once, outside any timing)."""

    def __init__(self, cfg, weights, use_ref: bool = True):
        self.cfg = cfg
        self.ref = oracle.ref() if use_ref else None
        self.own = oracle.own()
        self.threads = self.ref.hardware_threads() if self.ref is not None else self.own.threads()
        self.kind = "reference" if self.ref is not None else "port"
        self.layers = []
        for L in weights.layers:
            self.layers.append({k: (_f32_weight(v) if k in ("qkv", "o", "gate_up", "down", "qkv_bias") else _u16(v).copy())
                                for k, v in L.items()})
        self.embed = _u16(weights.embed)
        self.head = _f32_weight(weights.embed)
        self.final_norm = _u16(weights.final_norm).copy()

    # the non-GEMM stages, through the reference's CPU code when it is present
    def _norm(self, x, w):
        return self.ref.rmsnorm(x, w, self.cfg.eps, self.threads) if self.ref else self.own.rmsnorm(x, w, self.cfg.eps)

    def _norm_res(self, res, x, w):
        o = (self.ref.rmsnorm_residual(res, x, w, self.cfg.eps, 0.0, self.threads) if self.ref
             else self.own.rmsnorm_residual(res, x, w, self.cfg.eps))
        return o[0], o[1]

    def _rope(self, h, pos, heads):
        c = self.cfg
        return (self.ref.rope(h, pos, heads, c.head_dim, c.rope_theta, self.threads) if self.ref
                else self.own.rope(h, pos, heads, c.head_dim, c.rope_theta))

    def step(self, ex, rows):
        """The decode step the executor `ex` last uploaded from its host mirrors (a step begun with
        Engine.step / step_begin / upload_next_inputs, not one launched on device-fed inputs), for its batch rows
        `rows`, recomputed on the host: takes ids / positions / seq_lens / tables from the mirrors and those
        sequences' pages from the device, then returns (seconds of host compute, tokens int32[len(rows)], logits float32[len(rows), vocab])."""
        import torch
        cfg = self.cfg
        rows = list(rows)
        # The executor's pinned host mirrors hold what was uploaded for the step that has just run; the device
        # copies of ids / positions / seq_lens may already have been advanced to the next step's values by the
        # last kernel of the decode sequence.
        ids = ex.h_ids.numpy()[rows].copy()
        pos = ex.h_pos.numpy()[rows].copy()
        lens = ex.h_lens.numpy()[rows].copy()
        tables = ex.h_tables.numpy()[rows].copy()
        used = np.unique(tables[tables > 0])
        remap = np.zeros(int(tables.max()) + 1, np.int32)
        remap[used] = np.arange(1, len(used) + 1, dtype=np.int32)
        mb = (int(lens.max()) + 15) // 16
        ctab = np.ascontiguousarray(remap[tables][:, :mb])
        idx = torch.as_tensor(np.concatenate([[0], used]), device=ex.pool.device)
        pools = [_u16(ex.pool[li].index_select(0, idx)).reshape(-1).copy() for li in range(cfg.layers)]
        return self.step_host(ids, pos, lens, ctab, pools, ex.scale)

    def step_host(self, ids, pos, lens, ctab, pools, scale):
        """One decode step from host arrays alone: token ids, positions and seq_lens (int32 [n]), block
        tables (int32 [n, mb]) and one flat FP16-bit pool per layer ([blocks, 2, kv_heads, 16, head_dim],
        block 0 the dummy; the step's K/V are scattered into it). Returns (seconds, tokens, logits)."""
        cfg = self.cfg
        mb = ctab.shape[1]
        impl = self.ref or self.own

        t0 = time.perf_counter()
        x = np.ascontiguousarray(self.embed[ids])
        mlp = None
        for li, L in enumerate(self.layers):
            if li == 0:
                normed = self._norm(x, L["in_norm"])
            else:
                normed, x = self._norm_res(x, mlp, L["in_norm"])
            qkv = _h16(_f32(normed) @ L["qkv"].T + L["qkv_bias"])
            q = self._rope(np.ascontiguousarray(qkv[:, :cfg.q_width]), pos, cfg.q_heads)
            k = self._rope(np.ascontiguousarray(qkv[:, cfg.q_width:cfg.q_width + cfg.kv_width]), pos, cfg.kv_heads)
            v = np.ascontiguousarray(qkv[:, cfg.q_width + cfg.kv_width:])
            impl.kv_scatter(pools[li], k.reshape(-1), v.reshape(-1), cfg.kv_width, cfg.kv_width, ctab, mb, pos,
                            cfg.kv_heads, cfg.head_dim)
            if self.ref is not None:
                att = self.ref.paged_attention(q, pools[li], ctab, lens, cfg.q_heads, cfg.kv_heads, cfg.head_dim,
                                               scale, self.threads)
            else:
                att = self.own.paged_attention(q, pools[li], ctab, lens, cfg.q_heads, cfg.kv_heads, cfg.head_dim, scale)
            mlp = _h16(_f32(att) @ L["o"].T)
            normed, x = self._norm_res(x, mlp, L["post_norm"])
            gu = _h16(_f32(normed) @ L["gate_up"].T)
            act = self.ref.silu_mul(gu, self.threads) if self.ref is not None else self.own.silu_mul(gu)
            mlp = _h16(_f32(act) @ L["down"].T)
        normed, x = self._norm_res(x, mlp, self.final_norm)
        logits = _f32(normed) @ self.head.T
        tokens = impl.argmax(_h16(logits))
        return time.perf_counter() - t0, tokens, logits


class HostWeights:
    """Random-init weights of the architecture made on the host cores (FP16 ~N(0, std), norm weights 1;
    torch CPU tensors with the attribute layout of the engine's ModelWeights), for a CPU run that must
    not touch a GPU or the CUDA library. One draw per kind of matrix; layer i holds that draw rotated by
    i * 7919 elements - every layer still has its own copy in memory and the same distribution, which is all a
    timing baseline needs, at a fraction of the set-up time of 1.5 G independent draws."""

    def __init__(self, cfg, seed: int = 0x5EED, std: float = 0.02):
        import torch
        g = torch.Generator()
        g.manual_seed(seed)

        def rnd(*shape):
            return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(torch.float16)

        self.embed = rnd(cfg.vocab, cfg.hidden)
        self.lm_head = self.embed
        self.final_norm = torch.ones(cfg.hidden, dtype=torch.float16)
        base = dict(qkv=rnd(cfg.qkv_width, cfg.hidden), qkv_bias=rnd(cfg.qkv_width), o=rnd(cfg.hidden, cfg.q_width),
                    gate_up=rnd(2 * cfg.inter, cfg.hidden), down=rnd(cfg.hidden, cfg.inter))
        self.layers = []
        for i in range(cfg.layers):
            L = {k: torch.roll(v.reshape(-1), i * 7919).reshape(v.shape) for k, v in base.items()}
            L["in_norm"] = torch.ones(cfg.hidden, dtype=torch.float16)
            L["post_norm"] = torch.ones(cfg.hidden, dtype=torch.float16)
            self.layers.append(L)


def host_step_inputs(cfg, contexts, seed: int):
    """Host arrays for `step_host`: cached sequences of the given context lengths with seeded ~N(0,1) FP16 K/V
    in consecutive blocks 1.. (one pool per layer), each about to decode the token at position `context`."""
    from redline_llm_b200 import workloads as wl
    n = len(contexts)
    lens = np.asarray([c + 1 for c in contexts], np.int32)
    pos = np.asarray(contexts, np.int32)
    ids = wl.randint(seed, n, 0, cfg.vocab - 1)
    nb = (lens + 15) // 16
    mb = int(nb.max())
    ctab = np.zeros((n, mb), np.int32)
    nxt = 1
    for i in range(n):
        ctab[i, :nb[i]] = np.arange(nxt, nxt + nb[i])
        nxt += int(nb[i])
    per_block = 2 * cfg.kv_heads * 16 * cfg.head_dim
    base = wl.normal_half(seed + 1, nxt * per_block)
    pools = [np.roll(base, 8209 * li) for li in range(cfg.layers)]   # one draw, rotated per layer (same distribution)
    return ids, pos, lens, ctab, pools
