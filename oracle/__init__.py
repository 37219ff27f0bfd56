"""ctypes front end of the CPU oracle (``oracle.c``).

Test infrastructure only: the parity tests, the smoke check and the CPU
baseline leg of the benchmark import this module.  Nothing in the product
package may.  The functions take and return numpy arrays; f16/bf16 values
travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F16, BF16, F32 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` into ``liboracle.so`` (gcc + OpenMP) if needed."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "-B", "liboracle.so"], check=True)
    return _LIB_PATH


_REF_PATH = os.path.join(_HERE, "libref_sm80.so")


def build_ref_kernel(force: bool = False) -> str:
    """Compile the restated reference GPU kernel (needs nvcc)."""
    src = os.path.join(_HERE, "ref_kernel_sm80.cu")
    if force or not os.path.exists(_REF_PATH) or os.path.getmtime(_REF_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "-B", "libref_sm80.so"], check=True)
    return _REF_PATH


_ref = None


def ref_tensorop_gemm(bf16: bool, m: int, n: int, k: int, dA: int, dB: int, dC: int, stream: int = 0) -> None:
    """Launch the restated reference kernel (mma.sync, cp.async ring) on device
    pointers: C f32 (m, n) = A (m, k) * B (n, k)^T."""
    global _ref
    if _ref is None:
        build_ref_kernel()
        _ref = ctypes.CDLL(_REF_PATH)
        _ref.ref_tensorop_gemm.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 4
        _ref.ref_tensorop_gemm.restype = ctypes.c_int
    rc = _ref.ref_tensorop_gemm(int(bf16), m, n, k, dA, dB, dC, stream)
    if rc != 0:
        raise RuntimeError(f"ref_tensorop_gemm: cudaError {rc}")


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        sz, vp, f, i = ctypes.c_size_t, ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        for name in ("oracle_f32_to_f16", "oracle_f16_to_f32", "oracle_f32_to_bf16", "oracle_bf16_to_f32"):
            getattr(L, name).argtypes = [vp, vp, sz]
            getattr(L, name).restype = None
        L.oracle_num_threads.restype = i
        L.oracle_set_num_threads.argtypes = [i]
        L.oracle_set_num_threads.restype = None
        L.oracle_elementwise_add_f32.argtypes = [vp, vp, vp, sz]
        L.oracle_elementwise_add_f32.restype = None
        L.oracle_gemm_tn.argtypes = [i, i, sz, sz, sz, vp, vp, vp, f, f, sz, sz]
        L.oracle_gemm_tn.restype = i
        L.oracle_gemm_tn_abs.argtypes = [i, sz, sz, sz, vp, vp, vp, sz, sz]
        L.oracle_gemm_tn_abs.restype = i
        L.oracle_sgemm_nt.argtypes = [sz, sz, sz, f, f, vp, vp, vp]
        L.oracle_sgemm_nt.restype = i
        L.oracle_gemm_tn_naive_elem.argtypes = [i, sz, vp, vp, sz, sz]
        L.oracle_gemm_tn_naive_elem.restype = f
        L.oracle_sgemm_nt_naive_elem.argtypes = [sz, sz, sz, f, f, vp, vp, f, sz, sz]
        L.oracle_sgemm_nt_naive_elem.restype = f
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Let OpenMP use every core this process may run on (overrides an
    inherited OMP_NUM_THREADS); returns the thread count now in effect."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(n)
    return num_threads()


def f32_to_f16_bits(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_f16(_p(x), _p(out), x.size)
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().oracle_f16_to_f32(_p(h), _p(out), h.size)
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_bf16(_p(x), _p(out), x.size)
    return out


def bf16_bits_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().oracle_bf16_to_f32(_p(h), _p(out), h.size)
    return out


def elementwise_add(x, y) -> np.ndarray:
    x, y = _c(x, np.float32), _c(y, np.float32)
    assert x.shape == y.shape
    out = np.empty(x.shape, np.float32)
    lib().oracle_elementwise_add_f32(_p(x), _p(y), _p(out), x.size)
    return out


def gemm_tn(a_bits, b_bits, ab_dtype: int, c_dtype: int = F32, alpha: float = 1.0, beta: float = 0.0,
            c_init=None, rows=None) -> np.ndarray:
    """C (M,N) from A (M,K) and B (N,K) given as uint16 bit patterns.

    ``c_init`` (f32 values or bf16 bits, by ``c_dtype``) is the prior C that a
    non-trivial beta reads.  ``rows=(lo, hi)`` limits the rows computed; the
    others keep their ``c_init`` (or zero) contents.
    """
    a, b = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    (M, K), (N, K2) = a.shape, b.shape
    assert K == K2
    cdt = np.float32 if c_dtype == F32 else np.uint16
    c = np.zeros((M, N), cdt) if c_init is None else _c(c_init, cdt).copy().reshape(M, N)
    lo, hi = (0, M) if rows is None else rows
    rc = lib().oracle_gemm_tn(ab_dtype, c_dtype, M, N, K, _p(a), _p(b), _p(c), alpha, beta, lo, hi)
    assert rc == 0, rc
    return c


def gemm_tn_abs(a_bits, b_bits, ab_dtype: int, rows=None) -> np.ndarray:
    """sum_k |a||b| per output (f32), the scale of the reference's tolerance."""
    a, b = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    (M, K), (N, _) = a.shape, b.shape
    mag = np.zeros((M, N), np.float32)
    lo, hi = (0, M) if rows is None else rows
    rc = lib().oracle_gemm_tn_abs(ab_dtype, M, N, K, _p(a), _p(b), _p(mag), lo, hi)
    assert rc == 0, rc
    return mag


def sgemm_nt(a, b, c, alpha: float, beta: float, M: int, N: int, K: int) -> np.ndarray:
    """Column-major f32 sgemm on flat arrays; returns the new flat C."""
    a, b = _c(a, np.float32).reshape(-1), _c(b, np.float32).reshape(-1)
    out = _c(c, np.float32).reshape(-1).copy()
    assert a.size == M * K and b.size == N * K and out.size == M * N
    rc = lib().oracle_sgemm_nt(M, N, K, alpha, beta, _p(a), _p(b), _p(out))
    assert rc == 0, rc
    return out


def gemm_tn_naive_elem(a_bits, b_bits, ab_dtype: int, i: int, j: int) -> float:
    a, b = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    return float(lib().oracle_gemm_tn_naive_elem(ab_dtype, a.shape[1], _p(a), _p(b), i, j))


def sgemm_nt_naive_elem(a, b, c_old: float, alpha, beta, M, N, K, i, j) -> float:
    a, b = _c(a, np.float32).reshape(-1), _c(b, np.float32).reshape(-1)
    return float(lib().oracle_sgemm_nt_naive_elem(M, N, K, alpha, beta, _p(a), _p(b), c_old, i, j))
