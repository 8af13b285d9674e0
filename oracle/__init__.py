"""ctypes/numpy doorway onto the CPU checker (TEST INFRASTRUCTURE).

Only the test-suite, the smoke check and the benchmark's CPU-baseline /
reference legs import this package. The shipped CUDA path never does.

`own`  : libredline_oracle.so  - this repository's restatement (plain C).
`ref`  : _ref/libredline_ref.so - the reference's header-only CPU code compiled
         where it lies; present only where it was built (it travels as a
         prebuilt file). `ref` is None when absent.

All FP16 data are numpy uint16 arrays of bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_OWN_PATH = os.path.join(_HERE, "libredline_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libredline_ref.so")

u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def _reference_dir() -> str:
    """Where the reference tree is mounted: $REDLINE_REFERENCE_DIR, else the `reference_path` recorded in the
    repository's BASELINE.json; '' when neither names an existing directory."""
    ref = os.environ.get("REDLINE_REFERENCE_DIR", "")
    if not ref:
        try:
            import json
            with open(os.path.join(os.path.dirname(_HERE), "BASELINE.json")) as f:
                ref = str(json.load(f).get("reference_path", ""))
        except (OSError, ValueError):
            ref = ""
    return ref if ref and os.path.isdir(ref) else ""


def _make(*targets: str) -> None:
    env = dict(os.environ)
    env["REDLINE_REFERENCE_DIR"] = _reference_dir()
    subprocess.run(["make", "-C", _HERE, "-j8", *targets], check=True, capture_output=True, env=env)


def build(force: bool = False, gpu_ref: bool = False) -> None:
    """Compile the CPU checker and, where the reference tree is mounted (the environment variable REDLINE_REFERENCE_DIR, else
    the `reference_path` of BASELINE.json), the reference's own CPU code into _ref/. With
    `gpu_ref` also the GPU-side comparators of the Makefile's `gpuref` target (the reference's CUDA
    kernels behind a C ABI, and the reference's C++ host over either kernel library); those link
    against this repository's built CUDA library, so it must exist. Where the tree is absent the
    prebuilt files under _ref/ are used as they are."""
    src = os.path.join(_HERE, "redline_oracle.c")
    if force or not os.path.exists(_OWN_PATH) or os.path.getmtime(_OWN_PATH) < os.path.getmtime(src):
        _make("all")
    elif not os.path.exists(_REF_PATH):
        _make("ref")
    if gpu_ref:
        _make("gpuref")


def _sig(fn, res, *args):
    fn.restype = res
    fn.argtypes = list(args)
    return fn


class _Own:
    """This repository's restatement."""

    def __init__(self):
        L = C.CDLL(_OWN_PATH)
        self.L = L
        _sig(L.rlo_half_to_double, C.c_double, C.c_uint16)
        _sig(L.rlo_quantize, C.c_uint16, C.c_double)
        _sig(L.rlo_half_add, C.c_uint16, C.c_uint16, C.c_uint16)
        _sig(L.rlo_rel_distance_to_boundary, C.c_double, C.c_double)
        _sig(L.rlo_fill_uniform_half, C.c_uint64, C.c_uint64, u16p, C.c_int64, C.c_double, C.c_double)
        _sig(L.rlo_fill_normal_half, C.c_uint64, C.c_uint64, u16p, C.c_int64, C.c_double, C.c_double)
        _sig(L.rlo_fill_u64, C.c_uint64, C.c_uint64, u64p, C.c_int64)
        _sig(L.rlo_rmsnorm, None, u16p, u16p, u16p, C.c_int32, C.c_int32, C.c_float)
        _sig(L.rlo_rmsnorm_residual, None, u16p, u16p, u16p, u16p, C.c_int32, C.c_int32, C.c_float,
             C.c_void_p, C.c_void_p, C.c_double)
        for name in ("rlo_rmsnorm_residual_mutant_unrounded", "rlo_rmsnorm_residual_mutant_single_round"):
            _sig(getattr(L, name), None, u16p, u16p, u16p, u16p, C.c_int32, C.c_int32, C.c_float)
        _sig(L.rlo_build_rmsnorm_boundary_fixture, None, C.c_uint64, u16p, u16p, u16p, u8p)
        _sig(L.rlo_rmsnorm_f32, None, u16p, C.c_void_p, u16p, u16p, C.c_int32, C.c_int32, C.c_float)
        _sig(L.rlo_rope, None, u16p, C.c_int64, i32p, C.c_int32, C.c_int32, C.c_int32, C.c_double)
        _sig(L.rlo_rope_f32, None, u16p, C.c_int64, i32p, C.c_int32, C.c_int32, C.c_int32, C.c_float)
        _sig(L.rlo_rope_inv_freq_f32, None, f32p, C.c_int32, C.c_float)
        _sig(L.rlo_kv_scatter, None, u16p, u16p, u16p, C.c_int64, C.c_int64, i32p, C.c_int64, i32p,
             C.c_int32, C.c_int32, C.c_int32)
        _sig(L.rlo_paged_attention, None, u16p, u16p, u16p, i32p, i32p, C.c_int32, C.c_int32,
             C.c_int32, C.c_int32, C.c_int32, C.c_double)
        _sig(L.rlo_paged_attention_f64out, None, f64p, u16p, u16p, i32p, i32p, C.c_int32, C.c_int32,
             C.c_int32, C.c_int32, C.c_int32, C.c_double)
        _sig(L.rlo_silu_mul, None, u16p, C.c_int64, u16p, C.c_int32, C.c_int32)
        _sig(L.rlo_silu_mul_f32, None, u16p, C.c_int64, u16p, C.c_int32, C.c_int32)
        _sig(L.rlo_argmax, None, i32p, u16p, C.c_int32, C.c_int32)
        _sig(L.rlo_kv_gather, None, u16p, u16p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, u16p, i32p,
             C.c_int32, C.c_int32, C.c_int32)
        _sig(L.rlo_prefill_softmax, None, u16p, f32p, C.c_int32, C.c_int32, C.c_int32, C.c_int32)
        _sig(L.rlo_omp_threads, C.c_int)
        _sig(L.rlo_set_threads, None, C.c_int)

    # ---- scalar helpers
    def half_to_double(self, bits: int) -> float:
        return self.L.rlo_half_to_double(bits)

    def quantize(self, x: float) -> int:
        return self.L.rlo_quantize(x)

    def threads(self) -> int:
        return self.L.rlo_omp_threads()

    def set_threads(self, n: int) -> None:
        self.L.rlo_set_threads(n)

    # ---- generators (splitmix64 streams)
    def uniform_half(self, seed: int, n: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, np.uint16)
        self.L.rlo_fill_uniform_half(seed, out, n, lo, hi)
        return out

    def normal_half(self, seed: int, n: int, mean: float = 0.0, sigma: float = 1.0) -> np.ndarray:
        out = np.empty(n, np.uint16)
        self.L.rlo_fill_normal_half(seed, out, n, mean, sigma)
        return out

    def u64(self, seed: int, n: int) -> np.ndarray:
        out = np.empty(n, np.uint64)
        self.L.rlo_fill_u64(seed, out, n)
        return out

    # ---- kernels
    def rmsnorm(self, x, w, eps):
        rows, hidden = x.shape
        out = np.empty_like(x)
        self.L.rlo_rmsnorm(out, np.ascontiguousarray(x), np.ascontiguousarray(w), rows, hidden, eps)
        return out

    def rmsnorm_residual(self, residual, x, w, eps, rel_floor: float = 0.0):
        """Returns (out, new_residual, inv_rms, excluded)."""
        rows, hidden = x.shape
        res = np.ascontiguousarray(residual).copy()
        out = np.empty_like(res)
        inv = np.empty(rows, np.float64)
        exc = np.zeros((rows, hidden), np.uint8)
        self.L.rlo_rmsnorm_residual(out, res, np.ascontiguousarray(x), np.ascontiguousarray(w), rows,
                                    hidden, eps, inv.ctypes.data, exc.ctypes.data, rel_floor)
        return out, res, inv, exc

    def rmsnorm_mutant(self, which, residual, x, w, eps):
        rows, hidden = x.shape
        out = np.empty_like(x)
        fn = (self.L.rlo_rmsnorm_residual_mutant_unrounded if which == "unrounded"
              else self.L.rlo_rmsnorm_residual_mutant_single_round)
        fn(out, np.ascontiguousarray(residual), np.ascontiguousarray(x), np.ascontiguousarray(w),
           rows, hidden, eps)
        return out

    def boundary_fixture(self, seed: int):
        res = np.empty((8, 1536), np.uint16)
        inp = np.empty((8, 1536), np.uint16)
        w = np.empty(1536, np.uint16)
        isb = np.empty((8, 1536), np.uint8)
        self.L.rlo_build_rmsnorm_boundary_fixture(seed, res, inp, w, isb)
        return res, inp, w, isb

    def rmsnorm_f32(self, residual, x, w, eps):
        """FP32-order variant. residual None -> plain. Returns (out, new_residual|None)."""
        rows, hidden = x.shape
        out = np.empty_like(x)
        res = None if residual is None else np.ascontiguousarray(residual).copy()
        self.L.rlo_rmsnorm_f32(out, None if res is None else res.ctypes.data,
                               np.ascontiguousarray(x), np.ascontiguousarray(w), rows, hidden, eps)
        return out, res

    def rope(self, heads, positions, num_heads, head_dim, theta, f32=False):
        """heads: [T, num_heads*head_dim] dense; returns the rotated copy."""
        h = np.ascontiguousarray(heads).copy()
        t = h.shape[0]
        pos = np.ascontiguousarray(positions, np.int32)
        if f32:
            self.L.rlo_rope_f32(h, h.shape[1], pos, t, num_heads, head_dim, theta)
        else:
            self.L.rlo_rope(h, h.shape[1], pos, t, num_heads, head_dim, theta)
        return h

    def rope_inv_freq_f32(self, head_dim, theta):
        out = np.empty(head_dim // 2, np.float32)
        self.L.rlo_rope_inv_freq_f32(out, head_dim, theta)
        return out

    def kv_scatter(self, pool, k, v, k_stride, v_stride, tables, table_stride, positions, kv_heads,
                   head_dim):
        """Scatters into `pool` (flat uint16 array) in place."""
        self.L.rlo_kv_scatter(pool, k, v, k_stride, v_stride, np.ascontiguousarray(tables, np.int32),
                              table_stride, np.ascontiguousarray(positions, np.int32),
                              len(positions), kv_heads, head_dim)

    def paged_attention(self, q, pool, tables, seq_lens, q_heads, kv_heads, head_dim, scale,
                        f64out=False):
        """q dense [S, q_heads*head_dim]. Rows with seq_len<=0 are left 0 / 0.0."""
        s = q.shape[0]
        tables = np.ascontiguousarray(tables, np.int32)
        mbps = tables.shape[1]
        lens = np.ascontiguousarray(seq_lens, np.int32)
        if f64out:
            out = np.zeros(q.shape, np.float64)
            self.L.rlo_paged_attention_f64out(out, np.ascontiguousarray(q), pool, tables, lens, s,
                                              mbps, q_heads, kv_heads, head_dim, scale)
        else:
            out = np.zeros(q.shape, np.uint16)
            self.L.rlo_paged_attention(out, np.ascontiguousarray(q), pool, tables, lens, s, mbps,
                                       q_heads, kv_heads, head_dim, scale)
        return out

    def silu_mul(self, gate_up, f32=False):
        rows, two_i = gate_up.shape
        out = np.empty((rows, two_i // 2), np.uint16)
        fn = self.L.rlo_silu_mul_f32 if f32 else self.L.rlo_silu_mul
        fn(out, two_i // 2, np.ascontiguousarray(gate_up), rows, two_i // 2)
        return out

    def argmax(self, logits):
        rows, vocab = logits.shape
        out = np.empty(rows, np.int32)
        self.L.rlo_argmax(out, np.ascontiguousarray(logits), rows, vocab)
        return out


    def kv_gather(self, khat, vhat, head_stride, row_stride, pool, table_row, ctx_len, kv_heads, head_dim):
        """Gathers into the flat uint16 arrays khat / vhat in place."""
        self.L.rlo_kv_gather(khat, vhat, head_stride, row_stride, head_stride, row_stride, pool,
                             np.ascontiguousarray(table_row, np.int32), ctx_len, kv_heads, head_dim)

    def prefill_softmax(self, scores, chunk_start):
        heads, chunk_len, kv_len = scores.shape
        out = np.empty(scores.shape, np.uint16)
        self.L.rlo_prefill_softmax(out, np.ascontiguousarray(scores, np.float32), heads, chunk_len, kv_len, chunk_start)
        return out


class _Ref:
    """The reference's own CPU code (tests/reference/*.hpp), when built."""

    def __init__(self):
        L = C.CDLL(_REF_PATH)
        self.L = L
        _sig(L.rlr_half_to_double, C.c_double, C.c_uint16)
        _sig(L.rlr_quantize, C.c_uint16, C.c_double)
        _sig(L.rlr_half_add, C.c_uint16, C.c_uint16, C.c_uint16)
        _sig(L.rlr_rel_distance_to_boundary, C.c_double, C.c_double)
        _sig(L.rlr_fill_uniform_half, C.c_uint64, C.c_uint64, u16p, C.c_int64, C.c_double, C.c_double)
        _sig(L.rlr_rmsnorm, None, u16p, u16p, u16p, C.c_int32, C.c_int32, C.c_float, C.c_int)
        _sig(L.rlr_rmsnorm_residual, None, u16p, u16p, u16p, u16p, C.c_int32, C.c_int32, C.c_float,
             C.c_void_p, C.c_void_p, C.c_double, C.c_int)
        for name in ("rlr_rmsnorm_residual_mutant_unrounded", "rlr_rmsnorm_residual_mutant_single_round"):
            _sig(getattr(L, name), None, u16p, u16p, u16p, u16p, C.c_int32, C.c_int32, C.c_float)
        _sig(L.rlr_build_rmsnorm_boundary_fixture, None, C.c_uint64, u16p, u16p, u16p, u8p)
        _sig(L.rlr_rope, None, u16p, i32p, C.c_int32, C.c_int32, C.c_int32, C.c_double, C.c_int)
        _sig(L.rlr_kv_scatter, None, u16p, C.c_int64, u16p, u16p, C.c_int64, C.c_int64, i32p,
             C.c_int64, i32p, C.c_int32, C.c_int32, C.c_int32)
        _sig(L.rlr_paged_attention, None, u16p, u16p, u16p, C.c_int64, i32p, i32p, C.c_int32,
             C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_double, C.c_int)
        _sig(L.rlr_silu_mul, None, u16p, u16p, C.c_int32, C.c_int32, C.c_int)
        _sig(L.rlr_argmax, None, i32p, u16p, C.c_int32, C.c_int32)
        _sig(L.rlr_kv_gather, None, u16p, u16p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, u16p, C.c_int64, i32p,
             C.c_int32, C.c_int32, C.c_int32)
        _sig(L.rlr_prefill_softmax, None, u16p, f32p, C.c_int32, C.c_int32, C.c_int32, C.c_int32)
        _sig(L.rlr_hardware_threads, C.c_int)

    def half_to_double(self, bits):
        return self.L.rlr_half_to_double(bits)

    def quantize(self, x):
        return self.L.rlr_quantize(x)

    def hardware_threads(self):
        return self.L.rlr_hardware_threads()

    def uniform_half(self, seed, n, lo, hi):
        out = np.empty(n, np.uint16)
        self.L.rlr_fill_uniform_half(seed, out, n, lo, hi)
        return out

    def rmsnorm(self, x, w, eps, threads=1):
        rows, hidden = x.shape
        out = np.empty_like(x)
        self.L.rlr_rmsnorm(out, np.ascontiguousarray(x), np.ascontiguousarray(w), rows, hidden, eps, threads)
        return out

    def rmsnorm_residual(self, residual, x, w, eps, rel_floor=0.0, threads=1):
        rows, hidden = x.shape
        res = np.ascontiguousarray(residual).copy()
        out = np.empty_like(res)
        inv = np.empty(rows, np.float64)
        exc = np.zeros((rows, hidden), np.uint8)
        self.L.rlr_rmsnorm_residual(out, res, np.ascontiguousarray(x), np.ascontiguousarray(w), rows,
                                    hidden, eps, inv.ctypes.data, exc.ctypes.data, rel_floor, threads)
        return out, res, inv, exc

    def rmsnorm_mutant(self, which, residual, x, w, eps):
        rows, hidden = x.shape
        out = np.empty_like(x)
        fn = (self.L.rlr_rmsnorm_residual_mutant_unrounded if which == "unrounded"
              else self.L.rlr_rmsnorm_residual_mutant_single_round)
        fn(out, np.ascontiguousarray(residual), np.ascontiguousarray(x), np.ascontiguousarray(w),
           rows, hidden, eps)
        return out

    def boundary_fixture(self, seed):
        res = np.empty((8, 1536), np.uint16)
        inp = np.empty((8, 1536), np.uint16)
        w = np.empty(1536, np.uint16)
        isb = np.empty((8, 1536), np.uint8)
        self.L.rlr_build_rmsnorm_boundary_fixture(seed, res, inp, w, isb)
        return res, inp, w, isb

    def rope(self, heads, positions, num_heads, head_dim, theta, threads=1):
        h = np.ascontiguousarray(heads).copy()
        self.L.rlr_rope(h, np.ascontiguousarray(positions, np.int32), h.shape[0], num_heads,
                        head_dim, theta, threads)
        return h

    def kv_scatter(self, pool, k, v, k_stride, v_stride, tables, table_stride, positions, kv_heads,
                   head_dim):
        self.L.rlr_kv_scatter(pool, pool.size, k, v, k_stride, v_stride,
                              np.ascontiguousarray(tables, np.int32), table_stride,
                              np.ascontiguousarray(positions, np.int32), len(positions), kv_heads,
                              head_dim)

    def paged_attention(self, q, pool, tables, seq_lens, q_heads, kv_heads, head_dim, scale, threads=1):
        s = q.shape[0]
        tables = np.ascontiguousarray(tables, np.int32)
        out = np.zeros(q.shape, np.uint16)
        self.L.rlr_paged_attention(out, np.ascontiguousarray(q), pool, pool.size, tables,
                                   np.ascontiguousarray(seq_lens, np.int32), s, tables.shape[1],
                                   q_heads, kv_heads, head_dim, scale, threads)
        return out

    def silu_mul(self, gate_up, threads=1):
        rows, two_i = gate_up.shape
        out = np.empty((rows, two_i // 2), np.uint16)
        self.L.rlr_silu_mul(out, np.ascontiguousarray(gate_up), rows, two_i // 2, threads)
        return out

    def argmax(self, logits):
        rows, vocab = logits.shape
        out = np.empty(rows, np.int32)
        self.L.rlr_argmax(out, np.ascontiguousarray(logits), rows, vocab)
        return out


    def kv_gather(self, khat, vhat, head_stride, row_stride, pool, table_row, ctx_len, kv_heads, head_dim):
        self.L.rlr_kv_gather(khat, vhat, head_stride, row_stride, head_stride, row_stride, pool, pool.size,
                             np.ascontiguousarray(table_row, np.int32), ctx_len, kv_heads, head_dim)

    def prefill_softmax(self, scores, chunk_start):
        heads, chunk_len, kv_len = scores.shape
        out = np.empty(scores.shape, np.uint16)
        self.L.rlr_prefill_softmax(out, np.ascontiguousarray(scores, np.float32), heads, chunk_len, kv_len, chunk_start)
        return out


_own = None
_ref = None


def own() -> _Own:
    global _own
    if _own is None:
        build()
        _own = _Own()
    return _own


def ref():
    """The compiled reference CPU code, or None where it was never built."""
    global _ref
    if _ref is None:
        build()
        if not os.path.exists(_REF_PATH):
            return None
        _ref = _Ref()
    return _ref


# ---- numpy helpers shared by tests and the benchmark ------------------------

def half_bits_to_f64(bits: np.ndarray) -> np.ndarray:
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float64)


def ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in FP16 lattice steps (sign-magnitude order); NaN pairs count 0."""
    a = np.asarray(a_bits, np.uint16).astype(np.int32)
    b = np.asarray(b_bits, np.uint16).astype(np.int32)
    ka = np.where(a & 0x8000, -(a & 0x7FFF), a & 0x7FFF)
    kb = np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    d = np.abs(ka - kb)
    both_nan = ((a & 0x7FFF) > 0x7C00) & ((b & 0x7FFF) > 0x7C00)
    return np.where(both_nan, 0, d)


def _step(bits: np.ndarray, delta: int) -> np.ndarray:
    """The FP16 pattern `delta` lattice steps away (sign-magnitude order, clamped at +-max finite)."""
    a = np.asarray(bits, np.uint16).astype(np.int32)
    k = np.where(a & 0x8000, -(a & 0x7FFF), a & 0x7FFF) + delta
    k = np.clip(k, -0x7BFF, 0x7BFF)
    return np.where(k < 0, (-k) | 0x8000, k).astype(np.uint16)


def rmsnorm_gate(got_bits, h_bits, inv_rms, w_bits):
    """Gate for a two-rounding op: the kernel's intermediate fp16(h * inv_rms) may sit one FP16 step
    from the FP64 one when the unrounded value is next to a rounding midpoint (FP32 vs FP64 inv_rms);
    given that intermediate, the weight product must be exact. Returns (ok mask, exact mask)."""
    h = half_bits_to_f64(h_bits)
    w = half_bits_to_f64(w_bits)
    with np.errstate(over="ignore"):
        n0 = (h * np.asarray(inv_rms)[:, None]).astype(np.float16).view(np.uint16)
        ok = np.zeros(n0.shape, bool)
        exact = None
        for delta in (0, -1, 1):
            cand = (half_bits_to_f64(_step(n0, delta)) * w[None, :]).astype(np.float16).view(np.uint16)
            hit = cand == np.asarray(got_bits, np.uint16)
            ok |= hit
            if delta == 0:
                exact = hit
    return ok, exact
