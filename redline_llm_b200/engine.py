"""Decode engine around the sm_100a kernels: the caller side of the hot path.

Mirrors the public surface of the reference's Python binding (src/api/pybind.cpp:104-214):
`Engine(...)`, `add_request`, `step`, `has_capacity`, `stats`, plus the pieces of src/core the
hot path needs to run - a reservation block allocator (src/core/block_allocator.hpp:41-57), an
FCFS continuous-batching scheduler with the {1,2,4,8,16,32,48,64} bucket ladder
(src/core/scheduler.cpp:11-34,145-197,248-332) and a model executor that replays one CUDA graph per
bucket (src/core/model_executor.cpp:523-633,721-782). The decode layer sequence is the reference's
(src/core/model_executor.cpp:908-957): every non-GEMM stage is a launcher of this library; the four
linear layers of a block are this library's tcgen05 weight-streaming kernel (SiLU-mul fused into the
gate/up product) or, with decode_linear="library", library GEMMs as in the reference (torch.matmul ->
cuBLAS); the vocabulary projection follows the same switch (vocab_projection= overrides it); the embedding gather and the greedy
argmax at the two ends of the step are this library's too.

One Engine drives one GPU; multi-GPU serving is one Engine per GPU with requests sharded on the
host (`shard_requests`) - sequences and their KV pages never leave their GPU, so no collective exists.

torch is used for device memory, streams, graphs and the GEMMs only.
"""
from __future__ import annotations

import dataclasses
from collections import deque
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

KV_BLOCK = 16       # src/core/types.hpp: kKvBlockSize
DUMMY_BLOCK = 0     # reserved padding target (kDummyBlockId)
BUCKETS = (1, 2, 4, 8, 16, 32, 48, 64)


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Architecture constants (defaults: Qwen2.5-1.5B, docs/MODEL_SPEC.md)."""
    layers: int = 28
    hidden: int = 1536
    inter: int = 8960
    q_heads: int = 12
    kv_heads: int = 2
    head_dim: int = 128
    vocab: int = 151936
    rope_theta: float = 1e6
    eps: float = 1e-6
    eos_token_id: int = 151645                       # <|im_end|>; config.json's scalar
    extra_eos_token_ids: Tuple[int, ...] = (151643,)   # the rest of generation_config.json's stop set (src/core/config.cpp:54-56)

    @property
    def qkv_width(self):
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim

    @property
    def q_width(self):
        return self.q_heads * self.head_dim

    @property
    def kv_width(self):
        return self.kv_heads * self.head_dim

    def block_bytes(self):
        return self.layers * 2 * self.kv_heads * KV_BLOCK * self.head_dim * 2


def blocks_for_tokens(n: int) -> int:
    return (n + KV_BLOCK - 1) // KV_BLOCK


def select_bucket(n: int) -> int:
    """Smallest bucket >= n (src/core/scheduler.cpp:11-34); 0 when none covers it."""
    for b in BUCKETS:
        if b >= n:
            return b
    return 0


def shard_requests(num_requests: int, world: int, rank: int) -> List[int]:
    """Indices of the requests replica `rank` serves: dealt round-robin, so every replica gets the
    same mix of an already shuffled list. Pure host logic; no communication."""
    return list(range(rank, num_requests, world))


def balanced_order(costs: Sequence[int], shards: int = 8, seed: int = 0) -> List[int]:
    """A serving order for requests with the given costs (e.g. context lengths) such that dealing it round-robin
    (`shard_requests`) over `shards` replicas - or over any divisor of `shards` - gives every replica nearly the
    same total cost: requests are taken longest first and dealt to the shards in snake order (0..s-1, s-1..0, ...),
    then the positions inside the shards are shuffled (seeded, the same shuffle for every shard) so that the long
    requests do not all sit at the front. Index i of the result goes to shard i % shards. Host logic only."""
    n = len(costs)
    by_cost = sorted(range(n), key=lambda i: (-int(costs[i]), i))
    lists: List[List[int]] = [[] for _ in range(shards)]
    for k, i in enumerate(by_cost):
        lap, pos = divmod(k, shards)
        lists[pos if lap % 2 == 0 else shards - 1 - pos].append(i)
    depth = max(len(x) for x in lists)
    rng = np.random.default_rng(seed)
    perm = rng.permutation(depth)
    out: List[int] = []
    for j in perm:
        for x in lists:
            if j < len(x):
                out.append(x[int(j)])
    return out


class BlockAllocator:
    """Free-list allocator with reservations: a request reserves the blocks it can ever need at
    admission (`reserve_full`), then turns reservations into real blocks at 16-token boundaries."""

    def __init__(self, total_blocks: int):
        if total_blocks < 2:
            raise ValueError("the pool needs the dummy block and at least one real block")
        self.total = total_blocks
        self.free = list(range(total_blocks - 1, 0, -1))  # block 0 is the dummy
        self.reserved = 0

    def can_reserve(self, n: int) -> bool:
        return len(self.free) - self.reserved >= n

    def reserve(self, n: int) -> None:
        if not self.can_reserve(n):
            raise RuntimeError("reserve beyond capacity")
        self.reserved += n

    def unreserve(self, n: int) -> None:
        assert n <= self.reserved
        self.reserved -= n

    def alloc_reserved(self) -> int:
        assert self.reserved > 0 and self.free
        self.reserved -= 1
        return self.free.pop()

    def free_block(self, b: int) -> None:
        assert 0 < b < self.total
        self.free.append(b)

    @property
    def free_blocks(self) -> int:
        return len(self.free)


@dataclasses.dataclass
class Request:
    req_id: int
    prompt: List[int]
    max_new_tokens: int
    ignore_eos: bool = False
    forced_tokens: Optional[List[int]] = None
    output: List[int] = dataclasses.field(default_factory=list)
    blocks: List[int] = dataclasses.field(default_factory=list)
    reserved_left: int = 0
    prefilled: int = 0          # prompt tokens whose K/V are in the cache
    cached: int = 0             # tokens in the cache (prompt + generated, except the pending one)
    finished: bool = False
    reason: str = ""

    @property
    def seq_len(self) -> int:   # tokens the next decode step attends to, including the new one
        return self.cached + 1


class Scheduler:
    """FCFS admission, prefill-before-decode, bucketed decode batches."""

    def __init__(self, allocator: BlockAllocator, max_batch: int, max_seq_len: int, prefill_chunk: int,
                 eos_token_id=151645):
        self.alloc, self.max_batch, self.max_seq_len, self.chunk = allocator, max_batch, max_seq_len, prefill_chunk
        # one id or the whole stop set; compared as a set (src/core/scheduler.cpp: IsEosToken)
        self.eos = frozenset([eos_token_id] if isinstance(eos_token_id, int) else eos_token_id)
        self.waiting: deque = deque()
        self.running: List[Request] = []
        self.aborts = 0

    def enqueue(self, r: Request) -> None:
        self.waiting.append(r)

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_batch:
            r = self.waiting[0]
            need = blocks_for_tokens(len(r.prompt) + r.max_new_tokens)
            if not self.alloc.can_reserve(need):
                if not self.running:  # can never fit: abort instead of stalling forever
                    self.waiting.popleft()
                    r.finished, r.reason = True, "aborted"
                    self.aborts += 1
                    self.running.append(r)
                return
            self.alloc.reserve(need)
            r.reserved_left = need
            self.running.append(self.waiting.popleft())

    def _grow(self, r: Request, tokens: int) -> None:
        while len(r.blocks) < blocks_for_tokens(tokens):
            r.blocks.append(self.alloc.alloc_reserved())
            r.reserved_left -= 1

    def plan_step(self):
        """Returns ("prefill", request, start, end) | ("decode", [requests]) | ("idle",) | ("flush", [aborted])."""
        self._admit()
        dead = [r for r in self.running if r.finished]
        if dead:
            return ("flush", dead)
        for r in self.running:
            if r.prefilled < len(r.prompt):
                end = min(len(r.prompt), r.prefilled + self.chunk)
                self._grow(r, end)
                return ("prefill", r, r.prefilled, end)
        if not self.running:
            return ("idle",)
        batch = self.running[: BUCKETS[-1]]
        for r in batch:
            self._grow(r, r.seq_len)
        return ("decode", batch)

    def complete(self, r: Request, token: int) -> Tuple[int, int, bool, str]:
        """Appends the sampled token - or, under teacher forcing, the scripted one - applies the stop checks
        to the APPENDED token and frees blocks on finish. The returned tuple still reports the engine's own
        sampled token, so a parity run can score every position along a fixed continuation
        (src/core/scheduler.cpp:284-300, src/core/request.hpp:33-41)."""
        appended = token
        if r.forced_tokens is not None and len(r.output) < len(r.forced_tokens):
            appended = r.forced_tokens[len(r.output)]
        r.output.append(int(appended))
        if not r.ignore_eos and appended in self.eos:
            r.finished, r.reason = True, "eos"     # EOS wins a simultaneous length stop
        elif len(r.output) >= r.max_new_tokens:
            r.finished, r.reason = True, "length"
        if r.finished:
            self.release(r)
        return (r.req_id, int(token), r.finished, r.reason)

    def release(self, r: Request) -> None:
        for b in r.blocks:
            self.alloc.free_block(b)
        r.blocks = []
        self.alloc.unreserve(r.reserved_left)
        r.reserved_left = 0
        if r in self.running:
            self.running.remove(r)


class ModelWeights:
    """Random-init weights of the architecture: FP16 ~N(0, 0.02), norm weights 1 (seeded)."""

    def __init__(self, cfg: ModelConfig, device, seed: int = 0x5EED, std: float = 0.02):
        import torch
        g = torch.Generator(device=device)
        g.manual_seed(seed)

        def rnd(*shape):
            return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.float16)

        self.embed = rnd(cfg.vocab, cfg.hidden)
        self.lm_head = self.embed  # tied, as in the 1.5B checkpoint
        self.final_norm = torch.ones(cfg.hidden, dtype=torch.float16, device=device)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append(dict(
                in_norm=torch.ones(cfg.hidden, dtype=torch.float16, device=device),
                post_norm=torch.ones(cfg.hidden, dtype=torch.float16, device=device),
                qkv=rnd(cfg.qkv_width, cfg.hidden), qkv_bias=rnd(cfg.qkv_width),
                o=rnd(cfg.hidden, cfg.q_width), gate_up=rnd(2 * cfg.inter, cfg.hidden),
                down=rnd(cfg.hidden, cfg.inter)))


class ModelExecutor:
    """Owns the KV pool, the step buffers and one CUDA graph per decode bucket."""

    def __init__(self, cfg: ModelConfig, weights: ModelWeights, num_blocks: int, max_seq_len: int,
                 device, enable_cuda_graphs: bool = True):
        import torch
        from . import kernels as K
        self.torch, self.K, self.cfg, self.w, self.device = torch, K, cfg, weights, device
        self.num_blocks = num_blocks
        self.mbps = blocks_for_tokens(max_seq_len)
        self.graphs_enabled = enable_cuda_graphs
        f16, i32 = torch.float16, torch.int32
        self.pool = torch.zeros(cfg.layers, num_blocks, 2, cfg.kv_heads, KV_BLOCK, cfg.head_dim, dtype=f16, device=device)
        B = BUCKETS[-1]
        # token ids | positions | seq_lens in one buffer: one H2D copy per step instead of three
        self.step_inputs = torch.zeros(3, B, dtype=i32, device=device)
        self.ids, self.positions, self.seq_lens = self.step_inputs[0], self.step_inputs[1], self.step_inputs[2]
        self.tables = torch.zeros(B, self.mbps, dtype=i32, device=device)
        self.x = torch.zeros(B, cfg.hidden, dtype=f16, device=device)          # residual stream
        self.normed = torch.zeros(B, cfg.hidden, dtype=f16, device=device)
        self.qkv = torch.zeros(B, cfg.qkv_width, dtype=f16, device=device)
        self.attn = torch.zeros(B, cfg.q_width, dtype=f16, device=device)
        self.mlp = torch.zeros(B, cfg.hidden, dtype=f16, device=device)
        self.gateup = torch.zeros(B, 2 * cfg.inter, dtype=f16, device=device)
        self.logits = torch.zeros(B, cfg.vocab, dtype=f16, device=device)
        self.tokens = torch.zeros(B, dtype=i32, device=device)
        # pinned mirrors (one H2D each per step, one D2H)
        self.h_step_inputs = torch.zeros(3, B, dtype=i32).pin_memory()
        self.h_ids, self.h_pos, self.h_lens = self.h_step_inputs[0], self.h_step_inputs[1], self.h_step_inputs[2]
        self.h_tables = torch.zeros(B, self.mbps, dtype=i32).pin_memory()
        # Sampled tokens come back through a ring of two pinned buffers, each with its event, so that a second
        # step can be in flight while the host still reads the first one's tokens.
        self.h_tokens = torch.zeros(2, B, dtype=i32).pin_memory()
        # Control block of the device-side input advance (the last kernel of the decode sequence): [0] advance
        # on/off, [1 + i] a scripted token for row i or -1. Uploaded every step from a ring of two pinned copies.
        self.ctrl = torch.zeros(1 + B, dtype=i32, device=device)
        self.h_ctrl = torch.zeros(2, 1 + B, dtype=i32).pin_memory()
        self._np_ctrl = self.h_ctrl.numpy()
        self._np_ids, self._np_pos = self.h_ids.numpy(), self.h_pos.numpy()
        self._np_lens, self._np_tables = self.h_lens.numpy(), self.h_tables.numpy()
        self.row_owner: List[Optional[int]] = [None] * B   # request id whose table sits in row i
        self.row_len = [0] * B
        self.dirty_rows: List[int] = []
        self.h2d_bytes = 0
        self._last_batch_ids: Optional[List[int]] = None   # steady-state detection for fill_mirrors
        self._last_rows = 0
        self._last_tokens = None                            # tokens appended by the previous step (numpy)
        self.graphs: Dict[int, object] = {}
        self.tokens_ready = [torch.cuda.Event(), torch.cuda.Event()]   # recorded behind the D2H copy of the sampled tokens
        self.scale = 1.0 / float(np.sqrt(cfg.head_dim))
        self.attention_events = None  # set by profile runs
        self.prefill_logits = None
        self.prefill_attention = "fused"   # or "composite": gather -> library GEMM -> softmax -> library GEMM
        self.fuse_rope_scatter = True  # one launch for RoPE + scatter; False = the reference's two launches
        # Linear layers of the decode step: "tcgen05" = this library's weight-streaming kernel (with the
        # SiLU-mul fused into the gate/up product), "library" = torch.matmul (cuBLAS), as the reference.
        # The vocabulary projection has its own switch of the same two values and follows decode_linear unless
        # set. This library's kernel streams its 467 MB of weights at normal L2 priority, as the library GEMM
        # does: with evict-first tiles the projection itself was 5 us faster but the step 24 us slower, the
        # sweep through L2 evidently clearing lines that otherwise burden the next wave's launches.
        self.decode_linear = "tcgen05"
        self.vocab_projection = "tcgen05"
        self.fuse_qkv_rope = True      # RoPE + KV scatter in the QKV product's epilogue (tcgen05 path only)
        self.act = torch.zeros(B, cfg.inter, dtype=f16, device=device)         # silu(gate) * up
        K.init(device.index if device.index is not None else -1)

    # ---- the decode layer sequence (src/core/model_executor.cpp:894-961)
    def enqueue_decode(self, rows: int) -> None:
        torch, K, cfg, w = self.torch, self.K, self.cfg, self.w
        x, normed, qkv, attn, mlp, gu = (self.x[:rows], self.normed[:rows], self.qkv[:rows], self.attn[:rows],
                                         self.mlp[:rows], self.gateup[:rows])
        K.launch_embed_gather(x, cfg.hidden, w.embed, self.ids, rows, cfg.hidden)
        for li, L in enumerate(w.layers):
            if li == 0:
                K.launch_rms_norm(normed, x, L["in_norm"], rows, cfg.hidden, cfg.eps)
            else:
                K.launch_rms_norm_residual(normed, x, mlp, L["in_norm"], rows, cfg.hidden, cfg.eps)
            own = self.decode_linear == "tcgen05"
            fused_qkv = own and self.fuse_qkv_rope and cfg.head_dim == 128
            if fused_qkv:
                K.launch_qkv_rope_kv_scatter(qkv, normed, L["qkv"], L["qkv_bias"], self.pool[li], self.tables, self.mbps,
                                             self.positions, rows, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.rope_theta)
            elif own:
                K.launch_decode_linear(qkv, normed, L["qkv"], L["qkv_bias"], num_tokens=rows)
            else:
                torch.addmm(L["qkv_bias"], normed, L["qkv"].t(), out=qkv)
            if fused_qkv:
                pass
            elif self.fuse_rope_scatter:
                K.launch_rope_kv_scatter(qkv, cfg.qkv_width, self.pool[li], self.tables, self.mbps, self.positions,
                                         rows, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.rope_theta)
            else:
                K.launch_rope_inplace(qkv, qkv, cfg.qkv_width, cfg.qkv_width, self.positions, rows, cfg.q_heads,
                                      cfg.kv_heads, cfg.head_dim, cfg.rope_theta, k_offset=cfg.q_width)
                K.launch_kv_scatter(self.pool[li], qkv, qkv, cfg.qkv_width, cfg.qkv_width, self.tables, self.mbps,
                                    self.positions, rows, cfg.kv_heads, cfg.head_dim,
                                    k_offset=cfg.q_width, v_offset=cfg.q_width + cfg.kv_width)
            if self.attention_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            K.launch_paged_attention_decode(attn, cfg.q_width, qkv, cfg.qkv_width, self.pool[li], self.tables,
                                            self.seq_lens, rows, self.mbps, cfg.q_heads, cfg.kv_heads,
                                            cfg.head_dim, self.scale)
            if self.attention_events is not None:
                e1.record()
                self.attention_events.append((e0, e1))
            if own:
                K.launch_decode_linear(mlp, attn, L["o"], num_tokens=rows)
            else:
                torch.matmul(attn, L["o"].t(), out=mlp)
            K.launch_rms_norm_residual(normed, x, mlp, L["post_norm"], rows, cfg.hidden, cfg.eps)
            if own:
                act = self.act[:rows]
                K.launch_decode_linear(act, normed, L["gate_up"], num_tokens=rows, epilogue=K.EPILOGUE_SILU_MUL)
                K.launch_decode_linear(mlp, act, L["down"], num_tokens=rows)
            else:
                torch.matmul(normed, L["gate_up"].t(), out=gu)
                K.launch_silu_mul(gu, gu, rows, cfg.inter)
                torch.matmul(gu[:, :cfg.inter], L["down"].t(), out=mlp)
        K.launch_rms_norm_residual(normed, x, mlp, w.final_norm, rows, cfg.hidden, cfg.eps)
        if self.vocab_projection == "tcgen05":
            K.launch_decode_linear(self.logits[:rows], normed, w.lm_head, num_tokens=rows)
        else:
            torch.matmul(normed, w.lm_head.t(), out=self.logits[:rows])
        K.launch_greedy_argmax(self.tokens, self.logits, rows, cfg.vocab)
        # next step's ids / positions / seq_lens from this step's tokens, on the device (a no-op while
        # control[0] == 0, as during warm-up and capture; the host still uploads all three whenever the batch changed)
        advance = getattr(K, "launch_decode_advance", None)
        if advance is not None:
            advance(self.ids, self.positions, self.seq_lens, self.tokens, self.ctrl, rows)

    def warm_and_capture(self, buckets: Sequence[int]) -> None:
        """Eager warm-up of every bucket (first launches happen outside capture), then one graph each."""
        torch = self.torch
        self.seq_lens.fill_(1)
        for b in buckets:
            self.enqueue_decode(b)
        torch.cuda.synchronize(self.device)
        if not self.graphs_enabled:
            return
        for b in buckets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.enqueue_decode(b)
            self.graphs[b] = g
        self.seq_lens.zero_()

    def fill_mirrors(self, batch: List[Request], rows: int) -> None:
        """token = last output (or last prompt token), position = seq_len - 1, seq_len, table row; padded
        rows get token 0 / position 0 / seq_len 0 / all-dummy row (src/core/model_executor.cpp:784-874).
        A table row is rewritten only when its owner changed or gained a page, and only rewritten rows are
        uploaded: at 33k-token contexts a row is 8 KiB and the whole slab would be 0.5 MB per step."""
        ids, pos, lens, tab = self._np_ids, self._np_pos, self._np_lens, self._np_tables
        self.dirty_rows = []
        n = len(batch)
        batch_ids = [r.req_id for r in batch]
        if batch_ids == self._last_batch_ids and rows == self._last_rows and self._last_tokens is not None:
            # Steady state (same requests in the same rows as the previous step): the new token is last
            # step's result, the new position is last step's seq_len; only rows that crossed a 16-token
            # boundary gained a page.
            ids[:n] = self._last_tokens[:n]
            pos[:n] = lens[:n]
            lens[:n] += 1
            if n and int(lens[:n].max()) > self.mbps * KV_BLOCK:
                raise RuntimeError("a decode row outgrew its block table")
            for i in np.flatnonzero((pos[:n] & (KV_BLOCK - 1)) == 0):
                r = batch[i]
                nb = len(r.blocks)
                if nb < blocks_for_tokens(r.seq_len):
                    raise RuntimeError(f"request {r.req_id}: decode row outside its block table")
                if self.row_len[i] != nb:
                    tab[i, self.row_len[i]:nb] = r.blocks[self.row_len[i]:nb]
                    self.row_len[i] = nb
                    self.dirty_rows.append(int(i))
            return
        self._last_batch_ids, self._last_rows = batch_ids, rows
        ids[:rows] = 0; pos[:rows] = 0; lens[:rows] = 0
        for i in range(rows):
            r = batch[i] if i < len(batch) else None
            if r is None:
                if self.row_owner[i] is not None:
                    tab[i, :self.row_len[i]] = DUMMY_BLOCK
                    self.row_owner[i], self.row_len[i] = None, 0
                    self.dirty_rows.append(i)
                continue
            if r.seq_len > self.mbps * KV_BLOCK or len(r.blocks) < blocks_for_tokens(r.seq_len):
                raise RuntimeError(f"request {r.req_id}: decode row outside its block table")
            ids[i] = r.output[-1] if r.output else r.prompt[-1]
            pos[i] = r.seq_len - 1
            lens[i] = r.seq_len
            nb = len(r.blocks)
            if self.row_owner[i] != r.req_id:
                tab[i, :max(nb, self.row_len[i])] = DUMMY_BLOCK
                tab[i, :nb] = r.blocks
                self.row_owner[i], self.row_len[i] = r.req_id, nb
                self.dirty_rows.append(i)
            elif self.row_len[i] != nb:
                tab[i, self.row_len[i]:nb] = r.blocks[self.row_len[i]:nb]
                self.row_len[i] = nb
                self.dirty_rows.append(i)

    def _grow_rows(self, batch: List[Request]) -> None:
        """Table rows of an unchanged batch: append the pages the requests gained since the last upload."""
        tab = self._np_tables
        self.dirty_rows = []
        for i, r in enumerate(batch):
            nb = len(r.blocks)
            if self.row_len[i] != nb:
                tab[i, self.row_len[i]:nb] = r.blocks[self.row_len[i]:nb]
                self.row_len[i] = nb
                self.dirty_rows.append(i)

    def upload(self, rows: int, slot: int = 0, scripted: Optional[Sequence[int]] = None, advance: bool = False,
               inputs: bool = True) -> None:
        """H2D of one step's inputs from the pinned mirrors: the control block always; ids / positions / seq_lens
        unless the device has advanced them itself (`inputs=False`); the table rows that changed."""
        c = self._np_ctrl[slot]
        c[0] = 1 if advance else 0
        c[1:] = -1
        if scripted is not None:
            c[1:1 + len(scripted)] = scripted
        self.ctrl.copy_(self.h_ctrl[slot], non_blocking=True)
        if inputs:
            self.step_inputs.copy_(self.h_step_inputs, non_blocking=True)
        whole = len(self.dirty_rows) > rows // 2
        if whole:
            self.tables[:rows].copy_(self.h_tables[:rows], non_blocking=True)
        else:
            for i in self.dirty_rows:
                self.tables[i].copy_(self.h_tables[i], non_blocking=True)
        self.h2d_bytes = (self.h_ctrl[slot].numel() * 4 + (self.h_step_inputs.numel() * 4 if inputs else 0)
                          + 4 * self.mbps * (rows if whole else len(self.dirty_rows)))

    def run(self, rows: int) -> None:
        g = self.graphs.get(rows)
        if g is not None:
            g.replay()
        else:
            self.enqueue_decode(rows)

    def download(self, rows: int):
        self.download_begin(rows)
        return self.download_end(rows)

    def download_begin(self, rows: int, slot: int = 0) -> None:
        self.h_tokens[slot, :rows].copy_(self.tokens[:rows], non_blocking=True)
        self.tokens_ready[slot].record()

    def download_end(self, rows: int, slot: int = 0):
        self.tokens_ready[slot].synchronize()
        return self.h_tokens[slot, :rows].tolist()

    # ---- prompt ingestion (not on the hot path): chunked, eager, the reference's gather/GEMM/softmax/GEMM composite
    def prefill_chunk(self, r: Request, start: int, end: int) -> Optional[int]:
        torch, K, cfg, w = self.torch, self.K, self.cfg, self.w
        n = end - start
        dev = self.device
        ids = torch.tensor(r.prompt[start:end], dtype=torch.int32, device=dev)
        pos = torch.arange(start, end, dtype=torch.int32, device=dev)
        row = torch.zeros(1, self.mbps, dtype=torch.int32, device=dev)
        row[0, :len(r.blocks)] = torch.tensor(r.blocks, dtype=torch.int32, device=dev)
        x = torch.empty(n, cfg.hidden, dtype=torch.float16, device=dev)
        K.launch_embed_gather(x, cfg.hidden, w.embed, ids, n, cfg.hidden)
        normed, mlp = torch.empty_like(x), torch.empty_like(x)
        qkv = torch.empty(n, cfg.qkv_width, dtype=torch.float16, device=dev)
        gu = torch.empty(n, 2 * cfg.inter, dtype=torch.float16, device=dev)
        # Attention of the chunk over the sequence's cache: this library's fused paged kernel (TMA page tiles,
        # tcgen05), or - prefill_attention = "composite" - the reference's composite
        # (src/core/model_executor.cpp:1219-1290): kv_gather -> scores GEMMs -> causal softmax -> PV GEMMs, the
        # GEMMs being library calls and the staging below their scratch.
        fused = (self.prefill_attention == "fused" and cfg.head_dim == 128
                 and hasattr(K, "launch_paged_prefill_attention"))
        group = cfg.q_heads // cfg.kv_heads
        if fused:
            attn = torch.empty(n, cfg.q_width, dtype=torch.float16, device=dev)
        else:
            khat = torch.empty(cfg.kv_heads, end, cfg.head_dim, dtype=torch.float16, device=dev)
            vhat = torch.empty_like(khat)
            probs = torch.empty(cfg.q_heads, n, end, dtype=torch.float16, device=dev)
        for li, L in enumerate(w.layers):
            if li == 0:
                K.launch_rms_norm(normed, x, L["in_norm"], n, cfg.hidden, cfg.eps)
            else:
                K.launch_rms_norm_residual(normed, x, mlp, L["in_norm"], n, cfg.hidden, cfg.eps)
            torch.addmm(L["qkv_bias"], normed, L["qkv"].t(), out=qkv)
            K.launch_rope_inplace(qkv, qkv, cfg.qkv_width, cfg.qkv_width, pos, n, cfg.q_heads, cfg.kv_heads,
                                  cfg.head_dim, cfg.rope_theta, k_offset=cfg.q_width)
            K.launch_kv_scatter(self.pool[li], qkv, qkv, cfg.qkv_width, cfg.qkv_width, row, 0, pos, n,
                                cfg.kv_heads, cfg.head_dim, k_offset=cfg.q_width,
                                v_offset=cfg.q_width + cfg.kv_width)
            if fused:
                K.launch_paged_prefill_attention(attn, cfg.q_width, qkv, cfg.qkv_width, self.pool[li], row, self.mbps,
                                                 start, n, cfg.q_heads, cfg.kv_heads, cfg.head_dim, self.scale)
            else:
                K.launch_kv_gather(khat, vhat, end * cfg.head_dim, cfg.head_dim, end * cfg.head_dim, cfg.head_dim,
                                   self.pool[li], row, end, cfg.kv_heads, cfg.head_dim)
                q = qkv[:, :cfg.q_width].view(n, cfg.q_heads, cfg.head_dim).permute(1, 0, 2)      # [q_heads, n, d]
                kx = khat.repeat_interleave(group, dim=0)                                          # [q_heads, end, d]
                scores = torch.bmm(q.float(), kx.float().transpose(1, 2)) * self.scale             # FP32, scaled
                K.launch_prefill_softmax(probs, scores.contiguous(), cfg.q_heads, n, end, start)
                o = torch.bmm(probs, vhat.repeat_interleave(group, dim=0))                         # [q_heads, n, d]
                attn = o.permute(1, 0, 2).reshape(n, cfg.q_width).contiguous()
            torch.matmul(attn, L["o"].t(), out=mlp)
            K.launch_rms_norm_residual(normed, x, mlp, L["post_norm"], n, cfg.hidden, cfg.eps)
            torch.matmul(normed, L["gate_up"].t(), out=gu)
            K.launch_silu_mul(gu, gu, n, cfg.inter)
            torch.matmul(gu[:, :cfg.inter], L["down"].t(), out=mlp)
        r.prefilled = end
        if end < len(r.prompt):
            return None
        K.launch_rms_norm_residual(normed, x, mlp, w.final_norm, n, cfg.hidden, cfg.eps)
        logits = torch.matmul(normed[-1:], w.lm_head.t())
        self.prefill_logits = logits   # kept for parity audits of the first generated token
        tok = torch.zeros(1, dtype=torch.int32, device=dev)
        K.launch_greedy_argmax(tok, logits, 1, cfg.vocab)
        return int(tok.item())


class Engine:
    """`redline.Engine` look-alike (src/api/pybind.cpp:104-214) over one GPU."""

    def __init__(self, model_dir: Optional[str] = None, kv_pool_gb: float = 1.0, max_batch: int = 8,
                 enable_cuda_graphs: bool = True, max_seq_len: int = 2048, prefill_chunk: int = 1024,
                 admission_policy: str = "reserve_full", pad_eager_to_bucket: int = 0,
                 debug_dump_dir: Optional[str] = None, *, config: Optional[ModelConfig] = None,
                 device: int = 0, seed: int = 0x5EED, weights: Optional[ModelWeights] = None,
                 graph_buckets: Optional[Sequence[int]] = None, prologue_overlap: bool = True,
                 decode_linear: str = "tcgen05", vocab_projection: Optional[str] = None,
                 device_feedback: bool = True, prefill_attention: str = "fused"):
        import torch
        if admission_policy != "reserve_full":
            raise ValueError("only the reserve_full admission policy is provided")
        if not 1 <= max_batch <= BUCKETS[-1]:
            raise ValueError(f"max_batch must be in [1, {BUCKETS[-1]}]")
        if model_dir is not None:
            raise ValueError("checkpoint loading is outside this library: pass weights= or use random init")
        if not torch.cuda.is_available():
            raise RuntimeError("the decode kernels need a CUDA device; there is no CPU fallback")
        self.cfg = config or ModelConfig()
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        num_blocks = max(2, int(kv_pool_gb * (1 << 30)) // self.cfg.block_bytes())
        self.allocator = BlockAllocator(num_blocks)
        self.scheduler = Scheduler(self.allocator, max_batch, max_seq_len, prefill_chunk,
                                   (self.cfg.eos_token_id,) + tuple(self.cfg.extra_eos_token_ids))
        from . import kernels as K
        # attention's table walk may overlap the RoPE+scatter kernel before it: seq_lens and the block
        # tables are uploaded at the start of a step, never written by that kernel
        K.set_attention_prologue_overlap(prologue_overlap)
        self.weights = weights or ModelWeights(self.cfg, self.device, seed)
        if decode_linear not in ("tcgen05", "library"):
            raise ValueError("decode_linear must be 'tcgen05' or 'library'")
        self.exec = ModelExecutor(self.cfg, self.weights, num_blocks, max_seq_len, self.device, enable_cuda_graphs)
        self.exec.decode_linear = decode_linear
        self.exec.vocab_projection = vocab_projection or decode_linear
        if prefill_attention not in ("fused", "composite"):
            raise ValueError("prefill_attention must be 'fused' or 'composite'")
        self.exec.prefill_attention = prefill_attention
        self.max_seq_len, self.max_batch = max_seq_len, max_batch
        self.pad_eager_to_bucket = pad_eager_to_bucket
        buckets = [b for b in BUCKETS if b <= select_bucket(max_batch)]
        if graph_buckets is not None:
            buckets = [b for b in buckets if b in set(graph_buckets)]
        self.exec.warm_and_capture(buckets)
        self._next_id = 0
        # Steps begun and not yet ended, oldest first. One, unless `device_feedback` lets a second decode step of
        # the same batch be launched on the tokens the first one leaves on the device (try_step_begin).
        self._queue: deque = deque()
        self.device_feedback = bool(device_feedback)
        self._slot = 0
        self._stats = dict(steps=0, prefill_tokens=0, decode_tokens=0, graph_replays=0, eager_decodes=0)
        self._hist = {b: 0 for b in BUCKETS}

    def add_request(self, token_ids: Sequence[int], max_new_tokens: int, ignore_eos: bool = False,
                    forced_tokens: Optional[Sequence[int]] = None) -> int:
        ids = [int(t) for t in token_ids]
        if not ids or max_new_tokens < 1:
            raise ValueError("a request needs at least one prompt token and max_new_tokens >= 1")
        if any(t < 0 or t >= self.cfg.vocab for t in ids):
            raise ValueError("token id outside the vocabulary")
        if len(ids) + max_new_tokens > self.max_seq_len:
            raise ValueError("prompt + max_new_tokens exceeds max_seq_len")
        r = Request(self._next_id, ids, int(max_new_tokens), bool(ignore_eos),
                    None if forced_tokens is None else [int(t) for t in forced_tokens])
        self._next_id += 1
        self.scheduler.enqueue(r)
        return r.req_id

    def has_capacity(self) -> bool:
        return len(self.scheduler.running) + len(self.scheduler.waiting) < self.max_batch

    def step(self) -> List[Tuple[int, int, bool, str]]:
        self.step_begin()
        return self.step_end()

    # A step in two halves, for a driver that runs several engines (replicas on different GPUs, or admission
    # waves on one): step_begin() plans the step and, for a decode step, uploads the inputs and launches the
    # forward pass without waiting for it; step_end() waits for the sampled tokens and returns what step()
    # returns. Between the two the host is free to begin the steps of other engines. step() is the pair.
    def step_begin(self) -> None:
        if self._queue:
            raise RuntimeError("step_begin: the previous step has not been ended")
        plan = self.scheduler.plan_step()
        self._stats["steps"] += 1
        if plan[0] == "idle":
            self._queue.append(("done", []))
            return
        if plan[0] == "flush":
            out = []
            for r in plan[1]:
                self.scheduler.release(r)
                out.append((r.req_id, -1, True, r.reason))
            self._queue.append(("done", out))
            return
        if plan[0] == "prefill":
            _, r, start, end = plan
            tok = self.exec.prefill_chunk(r, start, end)
            self._stats["prefill_tokens"] += end - start
            if tok is None:
                self._queue.append(("done", []))
                return
            r.cached = len(r.prompt)
            self._queue.append(("done", [self.scheduler.complete(r, tok)]))
            return
        batch = plan[1]
        rows = select_bucket(max(len(batch), self.pad_eager_to_bucket))
        self.exec.fill_mirrors(batch, rows)
        self._slot ^= 1
        self.exec.upload(rows, self._slot, self._scripted(batch, 0), advance=self.device_feedback)
        self.exec.run(rows)
        self.exec.download_begin(rows, self._slot)
        self._queue.append(("decode", list(batch), rows, self._slot))

    @staticmethod
    def _scripted(batch: List[Request], ahead: int) -> List[int]:
        """The teacher-forcing token of each request's output number len(output) + ahead, or -1."""
        out = []
        for r in batch:
            k = len(r.output) + ahead
            out.append(r.forced_tokens[k] if r.forced_tokens is not None and k < len(r.forced_tokens) else -1)
        return out

    def try_step_begin(self) -> bool:
        """step_begin() when nothing is in flight. With one decode step in flight and `device_feedback` on, launches
        the NEXT decode step of the same batch right behind it - its token ids, positions and seq_lens are the
        ones the step in flight leaves on the device (rl_launch_decode_advance), so the host has not had to read
        that step's tokens - provided the batch cannot change in between: nobody waits for admission and no
        request reaches max_new_tokens with the step in flight. A request that stops on an end-of-sequence
        token is noticed one step late; the extra step's token for it is discarded (its K/V went to a page the
        request had reserved). Returns False, launching nothing, when the step in flight must be ended first."""
        if not self._queue:
            self.step_begin()
            return True
        last = self._queue[-1]
        if not self.device_feedback or len(self._queue) >= 2 or last[0] != "decode" or self.scheduler.waiting:
            return False
        _, batch, rows, _ = last
        running = self.scheduler.running[: BUCKETS[-1]]
        if len(running) != len(batch) or any(a is not b for a, b in zip(running, batch)):
            return False
        if any(r.finished or len(r.output) + 2 > r.max_new_tokens for r in batch):
            return False
        for r in batch:
            if r.seq_len + 1 > self.exec.mbps * KV_BLOCK:
                return False
            self.scheduler._grow(r, r.seq_len + 1)      # the step in flight appends one token, this one the next
        self._stats["steps"] += 1
        ex = self.exec
        ex._grow_rows(batch)
        ex._last_batch_ids = None                        # the host mirrors of ids / positions / lens are now stale
        self._slot ^= 1
        ex.upload(rows, self._slot, self._scripted(batch, 1), advance=True, inputs=False)
        ex.run(rows)
        ex.download_begin(rows, self._slot)
        self._queue.append(("decode", batch, rows, self._slot))
        return True

    @property
    def in_flight(self) -> int:
        return len(self._queue)

    def step_pipelined(self) -> List[Tuple[int, int, bool, str]]:
        """One call per step for a driver that keeps the GPU busy: launch the next step if that needs no result
        of the one in flight, then end the oldest step if two are in flight (or nothing could be launched).
        Results therefore arrive one call late while a batch is in its steady state; call drain() at the end."""
        launched = self.try_step_begin()
        if len(self._queue) >= 2 or (not launched and self._queue):
            return self.step_end()
        return []

    def drain(self) -> List[Tuple[int, int, bool, str]]:
        out = []
        while self._queue:
            out.extend(self.step_end())
        return out

    def upload_next_inputs(self) -> int:
        """Plans the next decode batch and uploads its inputs without running it, with the device-side advance
        switched off: afterwards `exec.run(rows)` can be replayed any number of times over the same resident
        inputs (the benchmark's device-only timing). Returns the number of batch rows (0 when no decode step
        is due)."""
        if self._queue:
            raise RuntimeError("upload_next_inputs: a step is in flight")
        plan = self.scheduler.plan_step()
        if plan[0] != "decode":
            return 0
        batch = plan[1]
        rows = select_bucket(max(len(batch), self.pad_eager_to_bucket))
        self.exec.fill_mirrors(batch, rows)
        self.exec._last_batch_ids = None    # no step follows this upload: the next fill starts from the requests
        self.exec.upload(rows, self._slot, None, advance=False)
        return rows

    def step_end(self) -> List[Tuple[int, int, bool, str]]:
        if not self._queue:
            raise RuntimeError("step_end without step_begin")
        pending = self._queue.popleft()
        if pending[0] == "done":
            return pending[1]
        _, batch, rows, slot = pending
        toks = self.exec.download_end(rows, slot)
        self._stats["graph_replays" if rows in self.exec.graphs else "eager_decodes"] += 1
        self._hist[rows] += 1
        out = []
        for r, t in zip(batch, toks):
            if r.finished:      # stopped by the previous step while this one was already in flight
                continue
            r.cached += 1
            self._stats["decode_tokens"] += 1
            out.append(self.scheduler.complete(r, t))
        # what the next step feeds back: the APPENDED tokens (the scripted ones under teacher forcing); any
        # finished request changes the batch, which fill_mirrors notices by itself
        self.exec._last_tokens = np.fromiter((r.output[-1] for r in batch), dtype=np.int32, count=len(batch))
        return out

    def stats(self) -> dict:
        a = self.allocator
        return dict(self._stats, waiting=len(self.scheduler.waiting), running=len(self.scheduler.running),
                    free_blocks=a.free_blocks, reserved_blocks=a.reserved, total_blocks=a.total,
                    aborts=self.scheduler.aborts, bucket_histogram=dict(self._hist))

    def debug_block_table(self, req_id: int) -> List[int]:
        for r in list(self.scheduler.running) + list(self.scheduler.waiting):
            if r.req_id == req_id:
                return list(r.blocks)
        raise ValueError("unknown request id")

    # ---- benchmark support: a request whose cache is filled with seeded synthetic K/V
    def add_synthetic_request(self, context_len: int, max_new_tokens: int, seed: int) -> int:
        """Admits a request as if a prompt of `context_len` tokens had been prefilled: its pages are
        allocated and filled with ~N(0,1) FP16 K/V on the device. No prompt pass runs."""
        torch = self.exec.torch
        if len(self.scheduler.running) >= self.max_batch:
            raise RuntimeError("max_batch sequences are already running")
        if context_len + max_new_tokens > self.max_seq_len:
            raise ValueError("context + max_new_tokens exceeds max_seq_len")
        need = blocks_for_tokens(context_len + max_new_tokens)
        if not self.allocator.can_reserve(need):
            raise RuntimeError("KV pool too small for this request")
        r = Request(self._next_id, [seed % self.cfg.vocab], max_new_tokens, ignore_eos=True)
        self._next_id += 1
        self.allocator.reserve(need)
        r.reserved_left = need
        self.scheduler._grow(r, context_len + 1)
        nb = blocks_for_tokens(context_len)
        if nb:
            g = torch.Generator(device=self.device)
            g.manual_seed(seed)
            idx = torch.tensor(r.blocks[:nb], device=self.device)
            cfg = self.cfg
            for li in range(cfg.layers):
                vals = torch.randn(nb, 2, cfg.kv_heads, KV_BLOCK, cfg.head_dim, generator=g, device=self.device,
                                   dtype=torch.float16)
                self.exec.pool[li].index_copy_(0, idx, vals)
        r.prefilled, r.cached = 1, context_len
        r.prompt = [seed % self.cfg.vocab]
        self.scheduler.running.append(r)
        return r.req_id
