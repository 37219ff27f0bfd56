"""The CPU oracle against the committed golden vectors and against its own
naive forms.  No GPU involved."""
import numpy as np
import pytest

import oracle
from tests.util import lcg_buffers


def test_conversions_match_golden(golden):
    x = golden["conv_in"]
    assert np.array_equal(oracle.f32_to_f16_bits(x), golden["conv_f16_bits"])
    assert np.array_equal(oracle.f32_to_bf16_bits(x), golden["conv_bf16_bits"])


def test_conversions_exhaustive_round_trip():
    h = np.arange(1 << 16, dtype=np.uint32).astype(np.uint16)
    f = oracle.f16_bits_to_f32(h)
    finite = np.isfinite(f)
    assert np.array_equal(f[finite], h.view(np.float16).astype(np.float32)[finite])
    assert np.array_equal(oracle.f32_to_f16_bits(f[finite]), h[finite])
    b = oracle.bf16_bits_to_f32(h)
    fin = np.isfinite(b)
    assert np.array_equal(oracle.f32_to_bf16_bits(b[fin]), h[fin])


def test_f16_conversion_matches_ieee_on_random_values():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.uniform(-70000, 70000, 20000), rng.normal(0, 1e-4, 20000),
                        rng.normal(0, 1e-7, 20000)]).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))


def test_nan_conversion_rules():
    nan = np.array([np.float32("nan")], np.float32)
    # bf16: high half with the quiet bit (src/value.rs:95-97)
    assert oracle.f32_to_bf16_bits(nan)[0] == (nan.view(np.uint32)[0] >> 16) | 0x40
    assert oracle.f32_to_f16_bits(nan)[0] & 0x7c00 == 0x7c00 and oracle.f32_to_f16_bits(nan)[0] & 0x3ff


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 128, 96), (128, 256, 160)])
@pytest.mark.parametrize("ab", [oracle.F16, oracle.BF16])
def test_tensorop_integer_inputs(golden, shape, ab):
    m, n, k = shape
    a = ((np.arange(m * k, dtype=np.int64) * 7 + 3) % 7 - 3).astype(np.float32).reshape(m, k)
    b = ((np.arange(n * k, dtype=np.int64) * 5 + 1) % 5 - 2).astype(np.float32).reshape(n, k)
    conv = oracle.f32_to_f16_bits if ab == oracle.F16 else oracle.f32_to_bf16_bits
    c = oracle.gemm_tn(conv(a), conv(b), ab)
    assert np.array_equal(c, golden[f"tensorop_int_{m}x{n}x{k}"].astype(np.float32))


@pytest.mark.parametrize("tag,ab", [("f16", oracle.F16), ("bf16", oracle.BF16)])
def test_tensorop_lcg_samples(golden, tag, ab):
    m, n, k = 256, 128, 96
    a, b, _ = lcg_buffers([m * k, n * k, m * n], small=False)
    conv = oracle.f32_to_f16_bits if ab == oracle.F16 else oracle.f32_to_bf16_bits
    c = oracle.gemm_tn(conv(a.reshape(m, k)), conv(b.reshape(n, k)), ab)
    for (i, j), want in zip(golden["tensorop_lcg_samples"], golden[f"tensorop_lcg_{tag}_expected"]):
        assert c[i, j].view(np.uint32) == want.view(np.uint32), (i, j)


def test_gemm_blocked_equals_naive_and_handles_ragged_shapes():
    rng = np.random.default_rng(11)
    m, n, k = 37, 70, 200
    a = oracle.f32_to_f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = oracle.f32_to_f16_bits(rng.uniform(-1, 1, (n, k)).astype(np.float32))
    c = oracle.gemm_tn(a, b, oracle.F16)
    for i, j in [(0, 0), (36, 69), (5, 64), (6, 63), (35, 1)]:
        assert c[i, j] == np.float32(oracle.gemm_tn_naive_elem(a, b, oracle.F16, i, j))
    # rows outside the requested block are left alone
    part = oracle.gemm_tn(a, b, oracle.F16, rows=(6, 12))
    assert np.array_equal(part[6:12], c[6:12]) and not part[:6].any() and not part[12:].any()


def test_gemm_epilogue_and_bf16_output():
    rng = np.random.default_rng(12)
    m, n, k = 16, 72, 64
    a = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (m, k)).astype(np.float32))
    b = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    acc = oracle.gemm_tn(a, b, oracle.BF16)
    out = oracle.gemm_tn(a, b, oracle.BF16, oracle.BF16)
    assert np.array_equal(out, oracle.f32_to_bf16_bits(acc))
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    got = oracle.gemm_tn(a, b, oracle.BF16, oracle.F32, alpha=1.5, beta=0.5, c_init=c0)
    want = (np.float32(1.5) * acc).astype(np.float32) + (np.float32(0.5) * c0).astype(np.float32)
    assert np.array_equal(got, want.astype(np.float32))
    # k == 0: only the beta term
    z = oracle.gemm_tn(np.zeros((m, 0), np.uint16), np.zeros((n, 0), np.uint16), oracle.BF16, alpha=2.0, beta=0.5, c_init=c0)
    assert np.array_equal(z, (np.float32(0.5) * c0).astype(np.float32))


def test_sgemm_integer_inputs(golden):
    m, n, k = 256, 256, 64
    a = ((np.arange(m * k, dtype=np.int64) * 7) % 11 - 5).astype(np.float32)
    b = ((np.arange(n * k, dtype=np.int64) * 3) % 13 - 6).astype(np.float32)
    c0 = (np.arange(m * n, dtype=np.int64) % 5).astype(np.float32)
    assert np.array_equal(oracle.sgemm_nt(a, b, c0, 1.5, -0.5, m, n, k), golden["sgemm_int_256x256x64"])


def test_sgemm_lcg_samples(golden):
    m, n, k = 256, 128, 32
    a, b, c0 = lcg_buffers([m * k, n * k, m * n], small=False)
    c = oracle.sgemm_nt(a, b, c0, 1.5, -0.5, m, n, k)
    for (i, j), want in zip(golden["sgemm_lcg_samples"], golden["sgemm_lcg_expected"]):
        assert c[i + j * m].view(np.uint32) == want.view(np.uint32), (i, j)
        assert c[i + j * m] == np.float32(oracle.sgemm_nt_naive_elem(a, b, float(c0[i + j * m]), 1.5, -0.5, m, n, k, i, j))


def test_elementwise_add(golden):
    i = np.arange(300 * 512, dtype=np.int64)
    a = (i % 97).astype(np.float32) * np.float32(0.5)
    b = (i % 13).astype(np.float32) - np.float32(6.0)
    assert np.array_equal(oracle.elementwise_add(a, b), golden["add_int_300x512"])
    a, b, _ = lcg_buffers([300 * 512, 300 * 512, 0], small=False)
    got = oracle.elementwise_add(a, b)
    assert np.array_equal(got[golden["add_lcg_index"]].view(np.uint32), golden["add_lcg_expected"].view(np.uint32))
    # subnormals are kept, empty input is fine
    tiny = np.array([1e-45, 2e-45], np.float32)
    assert np.array_equal(oracle.elementwise_add(tiny, tiny), tiny + tiny) and (tiny + tiny)[0] != 0
    assert oracle.elementwise_add(np.zeros(0, np.float32), np.zeros(0, np.float32)).size == 0


def test_nan_results_are_the_canonical_ptx_nan():
    # inf + -inf, and NaN operands of any payload or sign (src/sim/float.rs:416-428)
    x = np.array([np.inf, -np.inf, 1.0], np.float32)
    y = np.array([-np.inf, np.inf, 0.0], np.float32)
    y[2:] = np.array([0xFFC12345], np.uint32).view(np.float32)
    assert list(oracle.elementwise_add(x, y).view(np.uint32)) == [0x7FFFFFFF] * 3
    m = n = 64
    k = 4
    a = np.ones(m * k, np.float32)
    b = np.ones(n * k, np.float32)
    a[5] = np.array([0xFFC00001], np.uint32).view(np.float32)[0]  # a NaN operand in row 5, k = 0
    c = oracle.sgemm_nt(a, b, np.zeros(m * n, np.float32), 1.0, 1.0, m, n, k)
    assert (c.reshape(n, m)[:, 5].view(np.uint32) == 0x7FFFFFFF).all()
    # a kernel-side narrowing to bf16 maps NaN to 0x7fff (src/sim/exec.rs:430-449)
    z = np.zeros((8, 8), np.uint16)
    c0 = np.full((8, 8), np.float32(np.nan))
    out = oracle.gemm_tn(z, z, oracle.BF16, oracle.BF16, alpha=1.0, beta=1.0, c_init=oracle.f32_to_bf16_bits(c0))
    assert (out == 0x7FFF).all()
