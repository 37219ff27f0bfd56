"""Helpers shared by the tests: the reference test-suite's input streams and
the reference's tolerance for tensor-core results."""
from __future__ import annotations

import numpy as np


def lcg_values(count: int, state: int = 1):
    """`count` raw draws of the LCG in the reference's GPU test
    (tests/gpu.rs:58-63) and the state afterwards."""
    out = np.empty(count, np.uint64)
    mul, inc, mask = 6364136223846793005, 1442695040888963407, (1 << 64) - 1
    for i in range(count):
        state = (state * mul + inc) & mask
        out[i] = state >> 40
    return out, state


def lcg_buffers(lengths, small: bool):
    """One f32 buffer per length, drawn in order from one stream: small
    integers in [-8, 8] or values in [-1, 1) (tests/gpu.rs:64-83)."""
    state, bufs = 1, []
    for n in lengths:
        raw, state = lcg_values(n, state)
        if small:
            bufs.append((raw % 17).astype(np.float32) - np.float32(8.0))
        else:
            bufs.append(raw.astype(np.float32) / np.float32(1 << 23) - np.float32(1.0))
    return bufs


def tensor_core_bound(k: int, magnitude: np.ndarray) -> np.ndarray:
    """Allowed |new - oracle| per element: 2 * k * 2^-23 * sum|a*b|, the bound
    of check_tensor_core in the reference (tests/gpu.rs:146-176)."""
    return 2.0 * k * 2.0 ** -23 * magnitude.astype(np.float64)


def bf16_ulp(x_f32: np.ndarray) -> np.ndarray:
    """Size of one bf16 unit in the last place at |x| (8 significand bits)."""
    ax = np.maximum(np.abs(x_f32.astype(np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(ax)) - 7)
