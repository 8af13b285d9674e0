"""Helpers for the GPU parity tests: numpy bit patterns <-> device buffers."""
import numpy as np
import torch

import oracle


def dev(arr: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns / int32 arrays -> CUDA tensor holding the same bytes."""
    a = np.ascontiguousarray(arr)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    a = t.cpu().numpy()
    return a.view(np.uint16) if a.dtype == np.int16 else a


def is_nan_bits(bits):
    return (np.asarray(bits) & 0x7FFF) > 0x7C00


def ulp_of(values_f64):
    """Size of one FP16 step at |value| (2^-24 in the subnormal band)."""
    a = np.maximum(np.abs(values_f64), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(a)) - 10)


def assert_within_one_ulp(got_bits, ref_bits, what, min_exact=0.0):
    d = oracle.ulp_distance(got_bits, ref_bits)
    assert d.max() <= 1, f"{what}: {int((d > 1).sum())} elements differ by more than 1 FP16 ulp (max {d.max()})"
    exact = float((d == 0).mean())
    assert exact >= min_exact, f"{what}: only {exact:.5f} bit-exact"
    return exact
