"""Generates the committed golden vectors under tests/golden/.

Run where the reference tree is mounted (its location comes from the
REDLINE_REFERENCE_DIR environment variable):
    REDLINE_REFERENCE_DIR=<reference checkout> python tests/golden/make_golden.py

Sources of truth, none of them this repository's code:
  * the reference's committed RoPE capture tests/data/rope_fixture.json
    (HF Qwen2 rotary embedding, 8 tokens x (12+2) heads) - re-encoded as npz;
  * outputs of the reference's own header-only CPU implementation
    (tests/reference/*.hpp, compiled where it lies into oracle/_ref/) on
    seeded splitmix64 inputs.
The goldens let the checker in oracle/ and the CUDA path be verified on
machines where the reference tree does not exist.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

REF_TREE = os.environ.get("REDLINE_REFERENCE_DIR")
if not REF_TREE or not os.path.isdir(REF_TREE):
    raise SystemExit("set REDLINE_REFERENCE_DIR to the reference checkout")


def rope_capture():
    with open(os.path.join(REF_TREE, "tests/data/rope_fixture.json")) as f:
        d = json.load(f)
    m = d["meta"]
    np.savez_compressed(
        os.path.join(HERE, "rope_hf_capture.npz"),
        positions=np.asarray(m["positions"], np.int32),
        theta=np.float64(m["rope_theta"]),
        head_dim=np.int32(m["head_dim"]),
        num_q_heads=np.int32(m["num_q_heads"]),
        num_kv_heads=np.int32(m["num_kv_heads"]),
        q_in=np.asarray(d["q_in"], np.uint16),
        k_in=np.asarray(d["k_in"], np.uint16),
        q_out=np.asarray(d["q_out"], np.uint16),
        k_out=np.asarray(d["k_out"], np.uint16),
    )


def build_decode_case(gen, seed, seq_lens, q_heads, kv_heads, head_dim=128):
    """NaN-poisoned pool, shuffled block tables, live slots filled with U(-1,1)."""
    seq_lens = np.asarray(seq_lens, np.int32)
    blocks = (seq_lens + 15) // 16
    num_blocks = int(blocks.sum()) + 2
    mbps = max(1, int(blocks.max()))
    draws = gen.u64(seed, num_blocks)
    live = np.arange(1, num_blocks, dtype=np.int32)
    for i in range(len(live) - 1, 0, -1):  # Fisher-Yates over block ids 1..
        j = int(draws[i] % np.uint64(i + 1))
        live[i], live[j] = live[j], live[i]
    nan_patterns = np.array([0x7E00, 0x7C01, 0x7FFF, 0xFE00, 0xFFFF, 0xFDAB], np.uint16)
    pool = nan_patterns[np.arange(num_blocks * 2 * kv_heads * 16 * head_dim) % 6].copy()
    tables = np.zeros((len(seq_lens), mbps), np.int32)
    nxt = 0
    w = kv_heads * head_dim
    for s, ln in enumerate(seq_lens):
        if ln <= 0:
            continue
        nb = int(blocks[s])
        tables[s, :nb] = live[nxt:nxt + nb]
        nxt += nb
        k = gen.uniform_half(seed * 1000 + 2 * s + 1, int(ln) * w, -1.0, 1.0)
        v = gen.uniform_half(seed * 1000 + 2 * s + 2, int(ln) * w, -1.0, 1.0)
        gen.kv_scatter(pool, k, v, w, w, tables[s], 0, np.arange(ln, dtype=np.int32), kv_heads, head_dim)
    q = gen.uniform_half(seed * 1000 + 999, len(seq_lens) * q_heads * head_dim, -1.0, 1.0)
    return q.reshape(len(seq_lens), -1), pool, tables, seq_lens


def main():
    ref = oracle.ref()
    if ref is None:
        raise SystemExit("oracle/_ref is not built: mount the reference tree and run make -C oracle")
    gen = oracle.own()  # only its splitmix64 generators and bit-move scatter build the inputs
    rope_capture()
    out = {}

    # FP16 helpers: every pattern widened, and quantisation at crafted doubles.
    probes = np.array([0.0, -0.0, 1.0, 1.00048828125, 1.000244140625, 65504.0, 65519.99, 65520.0,
                       -65520.0, 5.9604644775390625e-08, 2.9802322387695312e-08,
                       2.98023223876953e-08, 6.103515625e-05, 6.097555160522461e-05, 1e-10,
                       0.333333333333, 1234.5678, -0.1, 3.0e-8], np.float64)
    out["quant_probe_in"] = probes
    out["quant_probe_out"] = np.array([ref.quantize(float(x)) for x in probes], np.uint16)
    out["widen_all"] = np.array([ref.half_to_double(i) for i in range(65536)], np.float64)

    # RMSNorm boundary fixture (seed 1) through the reference and both mutants.
    res, inp, w, isb = ref.boundary_fixture(1)
    o, r2, inv, exc = ref.rmsnorm_residual(res, inp, w, 1e-6, rel_floor=1e-5)
    out.update(bf_out=o, bf_residual=r2, bf_excluded=exc, bf_is_boundary=isb,
               bf_mut_unrounded=ref.rmsnorm_mutant("unrounded", res, inp, w, 1e-6),
               bf_mut_single=ref.rmsnorm_mutant("single", res, inp, w, 1e-6))

    # Seeded small cases.
    x = gen.uniform_half(0x51C + 17, 17 * 1536, -1.0, 1.0).reshape(17, 1536)
    r = gen.uniform_half(0x51D + 17, 17 * 1536, -1.0, 1.0).reshape(17, 1536)
    wt = gen.uniform_half(0x51E, 1536, 0.5, 1.5)
    out.update(rn_x=x, rn_r=r, rn_w=wt, rn_plain=ref.rmsnorm(x, wt, 1e-6))
    o, r2, _, _ = ref.rmsnorm_residual(r, x, wt, 1e-6)
    out.update(rn_fused_out=o, rn_fused_res=r2)

    heads = gen.uniform_half(0x40FE, 9 * 14 * 128, -1.0, 1.0).reshape(9, 14 * 128)
    pos = np.array([0, 1, 15, 16, 17, 255, 2047, 4095, 32767], np.int32)
    out.update(rope_in=heads, rope_pos=pos, rope_out=ref.rope(heads, pos, 14, 128, 1e6))

    gu = gen.uniform_half(0x5111, 5 * 2 * 896, -3.0, 3.0).reshape(5, 2 * 896)
    out.update(silu_in=gu, silu_out=ref.silu_mul(gu))

    q, pool, tables, lens = build_decode_case(gen, 0xA77E, [257, 0, 64, 1, 17, 15, 63, 65], 12, 2)
    out.update(att_q=q, att_pool=pool, att_tables=tables, att_lens=lens,
               att_out=ref.paged_attention(q, pool, tables, lens, 12, 2, 128, 0.088388347648318447))

    np.savez_compressed(os.path.join(HERE, "reference_cpu_vectors.npz"), **out)
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
