"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no external dataset is involved anywhere).

The generator is the stateful splitmix64 stream the reference's tests use
(tests/reference/fp16_ref.hpp:170-192), vectorised: draw i of a stream seeded
with s is mix(s + (i+1)*gamma). FP16 values are uint16 bit patterns.
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

KV_BLOCK = 16  # tokens per page (src/core/types.hpp: kKvBlockSize)


def splitmix64(seed: int, n: int) -> np.ndarray:
    """The first n outputs of the stream seeded with `seed` (uint64)."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + _GAMMA * np.arange(1, n + 1, dtype=np.uint64)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform01(seed: int, n: int) -> np.ndarray:
    return (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) * 2.0 ** -53


def to_half_bits(x: np.ndarray) -> np.ndarray:
    """float64 -> FP16 bit patterns, one round-to-nearest-even step."""
    with np.errstate(over="ignore"):
        return np.asarray(x, np.float64).astype(np.float16).view(np.uint16)


def uniform_half(seed: int, n: int, lo: float, hi: float) -> np.ndarray:
    return to_half_bits(lo + uniform01(seed, n) * (hi - lo))


def normal_half(seed: int, n: int, mean: float = 0.0, sigma: float = 1.0) -> np.ndarray:
    """N(mean, sigma) by Box-Muller over the uniform stream (pairs share two draws)."""
    m = (n + 1) // 2
    u = uniform01(seed, 2 * m)
    u1 = np.maximum(u[0::2], 2.0 ** -53)
    u2 = u[1::2]
    r = np.sqrt(-2.0 * np.log(u1))
    a = 6.283185307179586476925286766559 * u2
    out = np.empty(2 * m, np.float64)
    out[0::2] = mean + sigma * r * np.cos(a)
    out[1::2] = mean + sigma * r * np.sin(a)
    return to_half_bits(out[:n])


def permutation(seed: int, n: int) -> np.ndarray:
    """Fisher-Yates permutation of 0..n-1 driven by the stream (draw i picks j = draw % (i+1))."""
    draws = splitmix64(seed, n)
    p = np.arange(n, dtype=np.int32)
    for i in range(n - 1, 0, -1):
        j = int(draws[i] % np.uint64(i + 1))
        p[i], p[j] = p[j], p[i]
    return p


def randint(seed: int, n: int, lo: int, hi: int) -> np.ndarray:
    """n integers uniform in [lo, hi] inclusive."""
    return (lo + (splitmix64(seed, n) % np.uint64(hi - lo + 1)).astype(np.int64)).astype(np.int32)


# ---------------------------------------------------------------- configs

SEED_NORM, SEED_ROPE, SEED_ATTN, SEED_SILU, SEED_STEP = (0xB200C001, 0xB200C002, 0xB200C003,
                                                         0xB200C004, 0xB200C005)

HIDDEN, Q_HEADS, KV_HEADS, HEAD_DIM, INTER, QKV_STRIDE = 1536, 12, 2, 128, 8960, 2048
ATTN_SCALE = 0.088388347648318447  # 1/sqrt(128)


def config_rmsnorm(tokens: int = 64, seed: int = SEED_NORM):
    """x, residual [tokens,1536] ~N(0,1); weight [1536] ~N(1,0.1); eps 1e-6."""
    x = normal_half(seed, tokens * HIDDEN).reshape(tokens, HIDDEN)
    r = normal_half(seed + 1, tokens * HIDDEN).reshape(tokens, HIDDEN)
    w = normal_half(seed + 2, HIDDEN, 1.0, 0.1)
    return dict(x=x, residual=r, weight=w, eps=1e-6)


def config_rope_scatter(tokens: int = 64, num_blocks: int = 8192, max_pos: int = 4096,
                        seed: int = SEED_ROPE):
    """qkv [tokens,2048] ~N(0,1), positions U[0,max_pos), block tables drawn from a seeded
    permutation of blocks 1..num_blocks-1 (block 0 is the reserved dummy), distinct per entry."""
    qkv = normal_half(seed, tokens * QKV_STRIDE).reshape(tokens, QKV_STRIDE)
    positions = randint(seed + 1, tokens, 0, max_pos - 1)
    mbps = max_pos // KV_BLOCK
    perm = permutation(seed + 2, num_blocks - 1) + 1
    need = tokens * mbps
    reps = -(-need // len(perm))
    tables = np.tile(perm, reps)[:need].reshape(tokens, mbps).astype(np.int32)
    # the entry each token writes through must be unique across tokens
    tables[np.arange(tokens), positions // KV_BLOCK] = perm[:tokens]
    col = positions // KV_BLOCK
    for t in range(tokens):  # clear accidental duplicates of the live entries elsewhere in that row
        row = tables[t]
        dup = np.isin(row, perm[:tokens])
        dup[col[t]] = False
        row[dup] = 0
    return dict(qkv=qkv, positions=positions, tables=tables, num_blocks=num_blocks, theta=1e6)


def config_attention(batch: int = 64, lo: int = 1024, hi: int = 1280, num_blocks: int = 8192,
                     seed: int = SEED_ATTN, lens=None, kv_heads: int = KV_HEADS,
                     q_heads: int = Q_HEADS, fill: str = "normal"):
    """q [batch, q_heads*128] ~N(0,1); pool [num_blocks,2,kv_heads,16,128] with ~N(0,1) in every
    live slot and NaN patterns elsewhere; pages from a permutation of 1..num_blocks-1."""
    lens = randint(seed, batch, lo, hi) if lens is None else np.asarray(lens, np.int32)
    batch = len(lens)
    blocks = (lens + KV_BLOCK - 1) // KV_BLOCK
    assert int(blocks.sum()) <= num_blocks - 1, "pool too small for these sequence lengths"
    mbps = max(1, int(blocks.max()))
    perm = permutation(seed + 1, num_blocks - 1) + 1
    tables = np.zeros((batch, mbps), np.int32)
    off = 0
    for s in range(batch):
        tables[s, :blocks[s]] = perm[off:off + blocks[s]]
        off += int(blocks[s])
    page = kv_heads * KV_BLOCK * HEAD_DIM
    n = num_blocks * 2 * page
    nanpat = np.array([0x7E00, 0x7C01, 0x7FFF, 0xFE00, 0xFFFF, 0xFDAB], np.uint16)
    pool = nanpat[np.arange(n) % 6].reshape(num_blocks, 2, kv_heads, KV_BLOCK, HEAD_DIM)
    used = perm[:off]
    gen = normal_half if fill == "normal" else (lambda sd, m: uniform_half(sd, m, -1.0, 1.0))
    vals = gen(seed + 2, len(used) * 2 * page).reshape(len(used), 2, kv_heads, KV_BLOCK, HEAD_DIM)
    pool[used] = vals
    # re-poison the slots past each sequence's end
    for s in range(batch):
        tail = int(lens[s]) % KV_BLOCK
        if lens[s] > 0 and tail:
            b = tables[s, blocks[s] - 1]
            pool[b, :, :, tail:, :] = nanpat[np.arange(2 * kv_heads * (KV_BLOCK - tail) * HEAD_DIM) % 6].reshape(
                2, kv_heads, KV_BLOCK - tail, HEAD_DIM)
    q = gen(seed + 3, batch * q_heads * HEAD_DIM).reshape(batch, q_heads * HEAD_DIM)
    return dict(q=q, pool=pool.reshape(-1), tables=tables, seq_lens=lens, q_heads=q_heads,
                kv_heads=kv_heads, scale=ATTN_SCALE, num_blocks=num_blocks)


def config_silu(tokens: int = 64, seed: int = SEED_SILU):
    """gate_up [tokens, 2*8960] ~N(0,1)."""
    return dict(gate_up=normal_half(seed + tokens, tokens * 2 * INTER).reshape(tokens, 2 * INTER))


def attention_bytes(seq_lens, q_heads=Q_HEADS, kv_heads=KV_HEADS) -> int:
    """Algorithmic bytes of one paged-attention launch: K+V of every live token, Q in, out,
    the block-table entries walked and seq_lens."""
    lens = np.asarray(seq_lens, np.int64)
    live = lens[lens > 0]
    return int(live.sum() * kv_heads * HEAD_DIM * 2 * 2 + 2 * len(live) * q_heads * HEAD_DIM * 2
               + ((live + KV_BLOCK - 1) // KV_BLOCK).sum() * 4 + len(lens) * 4)
