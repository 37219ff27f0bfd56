"""Generates tests/golden/golden.npz.

The reference crate is Rust and cannot be run in the build image, so these
vectors are derived from the inputs and rules its own tests state, with
arithmetic that shares no code with the oracle or the CUDA kernels:

* integer-valued example inputs (examples/tensorop_gemm.rs:170-171,
  examples/sgemm.rs:87-90, examples/elementwise_add.rs:83-84): the expected
  outputs are computed in int64 / exact halves, which is what the examples'
  own host checks assert;
* the LCG streams of the reference's GPU test (tests/gpu.rs:55-83): sampled
  outputs are computed with exact rational arithmetic and an explicit
  round-to-nearest-even to binary32 after every step, in the order the
  simulator uses (k ascending; fma for sgemm, exact product then add for the
  tensor-core GEMM; mul, mul, add for the alpha/beta epilogue);
* f32 -> f16 / bf16 conversions of edge values, rounded from exact rationals
  (rules of src/value.rs:88-158).

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import struct
from fractions import Fraction

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


# ---- exact rounding helpers --------------------------------------------------
def f32_to_frac(x: np.float32) -> Fraction:
    return Fraction(float(x))  # f32 -> f64 is exact, f64 -> Fraction is exact


def round_to_float(fr: Fraction, mant_bits: int, emin: int, emax: int) -> float:
    """Round an exact rational to a binary float with `mant_bits` significand
    bits (incl. the hidden one), minimum normal exponent emin, maximum emax,
    ties to even, gradual underflow, overflow to infinity.  Returned as a
    Python float (exact for every format narrower than binary64)."""
    if fr == 0:
        return 0.0
    sign = -1 if fr < 0 else 1
    fr = abs(fr)
    # exponent e with 2^e <= fr < 2^(e+1)
    e = fr.numerator.bit_length() - fr.denominator.bit_length()
    if Fraction(2) ** e > fr:
        e -= 1
    e = max(e, emin)
    quantum = Fraction(2) ** (e - (mant_bits - 1))
    q = fr / quantum
    n = q.numerator // q.denominator
    rem = q - n
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and n % 2 == 1):
        n += 1
    val = n * quantum
    if val >= Fraction(2) ** (emax + 1):
        return sign * float("inf")
    return sign * float(val)


def rn32(fr: Fraction) -> np.float32:
    return np.float32(round_to_float(fr, 24, -126, 127))


def rn16(fr: Fraction) -> float:
    return round_to_float(fr, 11, -14, 15)


def rnbf16(fr: Fraction) -> float:
    return round_to_float(fr, 8, -126, 127)


def f16_bits_of(value: float) -> int:
    return int(np.float16(value).view(np.uint16))  # value is exactly representable here


def bf16_bits_of(value: float) -> int:
    return struct.unpack("<I", struct.pack("<f", value))[0] >> 16  # exactly representable: low half is zero


# ---- the reference test's input streams (tests/gpu.rs:55-83) ------------------
class Lcg:
    def __init__(self):
        self.state = 1

    def next(self) -> int:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        return self.state >> 40


def lcg_buffers(lengths, small: bool):
    g = Lcg()
    out = []
    for n in lengths:
        v = np.empty(n, np.float32)
        for i in range(n):
            r = g.next()
            v[i] = np.float32(r % 17) - np.float32(8.0) if small else np.float32(r) / np.float32(1 << 23) - np.float32(1.0)
        out.append(v)
    return out


def main() -> None:
    g = {}

    # -- conversions ---------------------------------------------------------------
    edge = [0.0, 1.0, -1.0, 0.5, 1.0 + 2.0 ** -11, 1.0 + 2.0 ** -10 + 2.0 ** -11, 1.0 + 2.0 ** -11 + 2.0 ** -20,
            65504.0, 65519.99, 65520.0, 70000.0, 2.0 ** -14, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 + 2.0 ** -40,
            3.0 * 2.0 ** -25, 2.0 ** -26, 6.1e-5, 1e-8, 0.1, -0.3, 3.14159274, 1.0 + 2.0 ** -8, 1.0 + 2.0 ** -7 + 2.0 ** -8,
            1.0 + 2.0 ** -8 + 2.0 ** -23, 255.5, 256.5, 3.3895314e38, 1e-40, -2.5e-39, 1234.5678, -0.02, 0.02]
    edge32 = np.array(edge, np.float32)
    g["conv_in"] = edge32
    def bits16(x, rnd, to_bits):
        mag = rnd(abs(f32_to_frac(x)))  # round the magnitude, then attach the sign (RNE is symmetric)
        return to_bits(mag) | (0x8000 if np.signbit(x) else 0)

    g["conv_f16_bits"] = np.array([bits16(x, rn16, f16_bits_of) for x in edge32], np.uint16)
    g["conv_bf16_bits"] = np.array([bits16(x, rnbf16, bf16_bits_of) for x in edge32], np.uint16)

    # -- integer example inputs: exact expected outputs --------------------------------
    for (m, n, k) in [(128, 128, 64), (256, 128, 96), (128, 256, 160)]:
        a = ((np.arange(m * k, dtype=np.int64) * 7 + 3) % 7 - 3).reshape(m, k)
        b = ((np.arange(n * k, dtype=np.int64) * 5 + 1) % 5 - 2).reshape(n, k)
        g[f"tensorop_int_{m}x{n}x{k}"] = (a @ b.T).astype(np.int32)
    m, n, k = 256, 256, 64
    a = ((np.arange(m * k, dtype=np.int64) * 7) % 11 - 5)
    b = ((np.arange(n * k, dtype=np.int64) * 3) % 13 - 6)
    c0 = (np.arange(m * n, dtype=np.int64) % 5)
    dot = a.reshape(k, m).T @ b.reshape(k, n)  # column-major (m,k): a[i + l*m]
    # alpha = 1.5, beta = -0.5: every term is a multiple of 0.5, exact in f32
    g["sgemm_int_256x256x64"] = (1.5 * dot - 0.5 * c0.reshape(n, m).T).T.reshape(-1).astype(np.float32)
    i = np.arange(300 * 512, dtype=np.int64)
    g["add_int_300x512"] = ((i % 97) * 0.5 + ((i % 13) - 6.0)).astype(np.float32)

    # -- LCG random data: sampled outputs with exact-rational step rounding ----------------
    # sgemm 256 x 128 x 32 (tests/gpu.rs:249-253), scalars alpha = 1.5, beta = -0.5
    m, n, k = 256, 128, 32
    a, b, c0 = lcg_buffers([m * k, n * k, m * n], small=False)
    samples = [(0, 0), (1, 0), (255, 127), (128, 64), (37, 29), (200, 5), (13, 99), (64, 127)]
    exp = []
    alpha, beta = np.float32(1.5), np.float32(-0.5)
    for (i_, j_) in samples:
        acc = np.float32(0.0)
        for l in range(k):
            acc = rn32(f32_to_frac(a[i_ + l * m]) * f32_to_frac(b[j_ + l * n]) + f32_to_frac(acc))
        p = rn32(f32_to_frac(alpha) * f32_to_frac(acc))
        q = rn32(f32_to_frac(beta) * f32_to_frac(c0[i_ + j_ * m]))
        exp.append(rn32(f32_to_frac(p) + f32_to_frac(q)))
    g["sgemm_lcg_samples"] = np.array(samples, np.int32)
    g["sgemm_lcg_expected"] = np.array(exp, np.float32)

    # tensorop_gemm 256 x 128 x 96, f16 and bf16 (tests/gpu.rs:260-262, 281-284)
    m, n, k = 256, 128, 96
    a, b, _ = lcg_buffers([m * k, n * k, m * n], small=False)
    samples = [(0, 0), (255, 127), (17, 3), (128, 64), (77, 100), (200, 31)]
    for tag, rnd in (("f16", rn16), ("bf16", rnbf16)):
        exp = []
        for (i_, j_) in samples:
            acc = np.float32(0.0)
            for l in range(k):
                av = Fraction(rnd(f32_to_frac(a[i_ * k + l])))
                bv = Fraction(rnd(f32_to_frac(b[j_ * k + l])))
                acc = rn32(f32_to_frac(acc) + av * bv)  # the product is exact, the add rounds
            exp.append(acc)
        g[f"tensorop_lcg_{tag}_expected"] = np.array(exp, np.float32)
    g["tensorop_lcg_samples"] = np.array(samples, np.int32)

    # elementwise add on LCG random data: first 64 and last 64 elements of 300 x 512
    a, b, _ = lcg_buffers([300 * 512, 300 * 512, 0], small=False)
    idx = np.concatenate([np.arange(64), np.arange(300 * 512 - 64, 300 * 512)])
    g["add_lcg_index"] = idx.astype(np.int32)
    g["add_lcg_expected"] = np.array([rn32(f32_to_frac(a[t]) + f32_to_frac(b[t])) for t in idx], np.float32)

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **g)
    print("wrote", os.path.join(HERE, "golden.npz"), {k_: v.shape for k_, v in g.items()})


if __name__ == "__main__":
    main()
