"""Parity of the CUDA kernels with the CPU oracle, through the C ABI.

Criteria are the reference's own (tests/gpu.rs): elementwise_add and sgemm
bit-exact on any data; tensor-core GEMMs bit-exact on small-integer data and
within 2*k*2^-23*sum|a*b| per element on data that has to round (plus one bf16
unit in the last place when C is bf16).
"""
import numpy as np
import pytest

import oracle
from tests.util import bf16_ulp, lcg_buffers, tensor_core_bound

pytestmark = pytest.mark.gpu


def dev(arr):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int16) if arr.dtype == np.uint16 else np.ascontiguousarray(arr))
    return t.cuda()


def host(t, dtype):
    a = t.cpu().numpy()
    return a.view(np.uint16) if dtype == np.uint16 else a


def run_gemm(lib, a_bits, b_bits, ab, cdt, alpha=1.0, beta=0.0, c0=None, tile_n=0, cta_group=0, tile_m=0, split_k=0):
    import torch
    (m, k), n = a_bits.shape, b_bits.shape[0]
    if c0 is None:
        c0 = np.zeros((m, n), np.float32 if cdt == lib.F32 else np.uint16)
    dA, dB, dC = dev(a_bits), dev(b_bits), dev(c0)
    a_ptr = dA.data_ptr() if k else 0
    b_ptr = dB.data_ptr() if k else 0
    lib.gemm_tn(lib.gemm_desc(m, n, k, ab, cdt, alpha, beta, tile_n, cta_group, tile_m, split_k), a_ptr, b_ptr, dC.data_ptr(), 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    return host(dC, c0.dtype).reshape(m, n)


def conv(lib, ab):
    return oracle.f32_to_bf16_bits if ab == lib.BF16 else oracle.f32_to_f16_bits


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("n,offset", [(0, 0), (1, 0), (3, 1), (4095, 0), (4096, 0), (4097, 0), (4096, 1), (4096, 3),
                                      (300 * 512, 0), (1 << 22, 2), ((1 << 22) + 5, 0)])
def test_elementwise_add_bit_exact_with_ragged_ends(lib, gpu, n, offset):
    import torch
    rng = np.random.default_rng(n + offset)
    x = rng.uniform(-1, 1, n + 8).astype(np.float32)
    y = rng.uniform(-1, 1, n + 8).astype(np.float32)
    if n > 16:
        x[offset + 3], y[offset + 3] = np.float32(1e-45), np.float32(2e-45)  # subnormals must survive
        x[offset + 5], y[offset + 5] = np.float32(np.inf), np.float32(-np.inf)
    dx, dy = dev(x), dev(y)
    out = torch.full((n + 8,), 7.0, device="cuda")
    lib.elementwise_add_f32(dx.data_ptr() + 4 * offset, dy.data_ptr() + 4 * offset, out.data_ptr() + 4 * offset, n, 0)
    torch.cuda.synchronize()
    want = np.full(n + 8, 7.0, np.float32)
    want[offset:offset + n] = oracle.elementwise_add(x[offset:offset + n], y[offset:offset + n])
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_elementwise_add_mixed_alignment_uses_scalar_kernel(lib, gpu):
    import torch
    n = 10007
    rng = np.random.default_rng(3)
    x, y = rng.uniform(-1, 1, n + 4).astype(np.float32), rng.uniform(-1, 1, n + 4).astype(np.float32)
    dx, dy, out = dev(x), dev(y), torch.zeros(n + 4, device="cuda")
    lib.elementwise_add_f32(dx.data_ptr() + 4, dy.data_ptr() + 8, out.data_ptr(), n, 0)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy()[:n], oracle.elementwise_add(x[1:n + 1], y[2:n + 2]))
    assert not out.cpu().numpy()[n:].any()
    with pytest.raises(lib.CuteB200Error) as e:
        lib.elementwise_add_f32(dx.data_ptr() + 2, dy.data_ptr(), out.data_ptr(), 4, 0)
    assert e.value.status == lib.ERR_MISALIGNED


def test_elementwise_add_random_lengths_and_alignments(lib, gpu):
    """A seeded sweep over lengths and independent 4-byte offsets of the three buffers: every
    combination of the 256-bit, 128-bit and scalar kernels with ragged heads and tails."""
    import torch
    rng = np.random.default_rng(77)
    big = 1 << 16
    x = rng.uniform(-1, 1, big + 64).astype(np.float32)
    y = rng.uniform(-1, 1, big + 64).astype(np.float32)
    dx, dy = dev(x), dev(y)
    for _ in range(40):
        n = int(rng.choice([0, 1, 2, 7, 8, 9, 31, 33, 255, 2049, 4096, 5000, big]))
        ox, oy, oo = (int(v) for v in rng.integers(0, 16, 3))
        if rng.integers(2):
            oy = ox + 8 * int(rng.integers(0, 2))  # often the same phase, so the vector kernels are reached
            oo = ox + 4 * int(rng.integers(0, 3))
        out = torch.full((big + 64,), 9.0, device="cuda")
        lib.elementwise_add_f32(dx.data_ptr() + 4 * ox, dy.data_ptr() + 4 * oy, out.data_ptr() + 4 * oo, n, 0)
        torch.cuda.synchronize()
        want = np.full(big + 64, 9.0, np.float32)
        want[oo:oo + n] = oracle.elementwise_add(x[ox:ox + n], y[oy:oy + n])
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), (n, ox, oy, oo)


def test_elementwise_add_golden_and_lcg(lib, gpu, golden):
    import torch
    for small in (True, False):
        a, b, _ = lcg_buffers([300 * 512, 300 * 512, 0], small=small)
        da, db, out = dev(a), dev(b), torch.empty(300 * 512, device="cuda")
        lib.elementwise_add_f32(da.data_ptr(), db.data_ptr(), out.data_ptr(), a.size, 0)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), oracle.elementwise_add(a, b).view(np.uint32))
        if not small:
            assert np.array_equal(got[golden["add_lcg_index"]].view(np.uint32), golden["add_lcg_expected"].view(np.uint32))


def test_elementwise_add_full_size_properties(lib, gpu):
    """2^28 elements: too large to compare everywhere cheaply, so check
    commutativity, x + 0 == x, sampled slices against the oracle, and that
    the guard elements after the end stay untouched."""
    import torch
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand(n + 4, device="cuda", generator=g) * 2 - 1
    y = torch.rand(n + 4, device="cuda", generator=g) * 2 - 1
    out = torch.full((n + 4,), 3.0, device="cuda")
    lib.elementwise_add_f32(x.data_ptr(), y.data_ptr(), out.data_ptr(), n, 0)
    out2 = torch.empty(n, device="cuda")
    lib.elementwise_add_f32(y.data_ptr(), x.data_ptr(), out2.data_ptr(), n, 0)
    torch.cuda.synchronize()
    assert torch.equal(out[:n].view(torch.int32), out2.view(torch.int32))
    assert bool((out[n:] == 3.0).all())
    for lo in (0, 4096 * 1000 + 1, n - 4096):
        got = out[lo:lo + 4096].cpu().numpy()
        want = oracle.elementwise_add(x[lo:lo + 4096].cpu().numpy(), y[lo:lo + 4096].cpu().numpy())
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    zero = torch.zeros(n, device="cuda")
    lib.elementwise_add_f32(x.data_ptr(), zero.data_ptr(), out2.data_ptr(), n, 0)
    torch.cuda.synchronize()
    assert torch.equal(out2, x[:n])


# ------------------------------------------------------------------------ sgemm
@pytest.mark.parametrize("m,n,k", [(128, 128, 8), (256, 128, 32), (128, 256, 16), (256, 256, 64), (384, 128, 100), (128, 128, 0)])
@pytest.mark.parametrize("small", [True, False])
def test_sgemm_bit_exact(lib, gpu, m, n, k, small):
    import torch
    a, b, c0 = lcg_buffers([m * k, n * k, m * n], small=small)
    dA, dB, dC = dev(a if k else np.zeros(4, np.float32)), dev(b if k else np.zeros(4, np.float32)), dev(c0)
    lib.sgemm_nt(m, n, k, 1.5, -0.5, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    torch.cuda.synchronize()
    want = oracle.sgemm_nt(a, b, c0, 1.5, -0.5, m, n, k)
    assert np.array_equal(dC.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_sgemm_random_shapes(lib, gpu):
    """Seeded sweep over the shapes the kernel takes (multiples of 128 x 128 x 8) and epilogue scalars."""
    import torch
    rng = np.random.default_rng(9)
    for _ in range(8):
        m, n, k = 128 * int(rng.integers(1, 6)), 128 * int(rng.integers(1, 6)), 8 * int(rng.integers(0, 40))
        alpha, beta = [(1.5, -0.5), (1.0, 0.0), (0.0, 1.0), (-2.0, 3.0)][int(rng.integers(4))]
        a, b, c0 = (rng.uniform(-1, 1, s).astype(np.float32) for s in (max(m * k, 4), max(n * k, 4), m * n))
        dA, dB, dC = dev(a), dev(b), dev(c0)
        lib.sgemm_nt(m, n, k, alpha, beta, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
        torch.cuda.synchronize()
        want = oracle.sgemm_nt(a[:m * k], b[:n * k], c0, alpha, beta, m, n, k)
        assert np.array_equal(dC.cpu().numpy().view(np.uint32), want.view(np.uint32)), (m, n, k, alpha, beta)


def test_sgemm_golden(lib, gpu, golden):
    import torch
    m, n, k = 256, 256, 64
    a = ((np.arange(m * k, dtype=np.int64) * 7) % 11 - 5).astype(np.float32)
    b = ((np.arange(n * k, dtype=np.int64) * 3) % 13 - 6).astype(np.float32)
    c0 = (np.arange(m * n, dtype=np.int64) % 5).astype(np.float32)
    dA, dB, dC = dev(a), dev(b), dev(c0)
    lib.sgemm_nt(m, n, k, 1.5, -0.5, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    torch.cuda.synchronize()
    assert np.array_equal(dC.cpu().numpy(), golden["sgemm_int_256x256x64"])
    m, n, k = 256, 128, 32
    a, b, c0 = lcg_buffers([m * k, n * k, m * n], small=False)
    dA, dB, dC = dev(a), dev(b), dev(c0)
    lib.sgemm_nt(m, n, k, 1.5, -0.5, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    torch.cuda.synchronize()
    got = dC.cpu().numpy()
    for (i, j), want in zip(golden["sgemm_lcg_samples"], golden["sgemm_lcg_expected"]):
        assert got[i + j * m].view(np.uint32) == want.view(np.uint32)


def test_sgemm_rejects_bad_shapes(lib, gpu):
    with pytest.raises(lib.CuteB200Error) as e:
        lib.sgemm_nt(100, 128, 8, 1.0, 0.0, 256, 256, 256, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "multiple of the tile size" in e.value.message


def test_sgemm_full_size_bands(lib, gpu):
    """4096^3 (the sgemm config): full-size run, checked bit for bit on whole bands
    of 128 columns and of 128 rows (first, interior and last tiles), each band
    computed by the oracle as a GEMM of its own, plus single elements elsewhere."""
    import torch
    n = 4096
    rng = np.random.default_rng(2)
    a, b, c0 = (rng.uniform(-1, 1, n * n).astype(np.float32) for _ in range(3))
    dA, dB, dC = dev(a), dev(b), dev(c0)
    lib.sgemm_nt(n, n, n, 1.5, 0.5, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    torch.cuda.synchronize()
    got = dC.cpu().numpy()
    a2, b2, c2, g2 = a.reshape(n, n), b.reshape(n, n), c0.reshape(n, n), got.reshape(n, n)  # [l or j, i or j]
    for j0 in (0, 1920, n - 128):  # columns j0 .. j0 + 128 of C: contiguous in column-major storage
        want = oracle.sgemm_nt(a, np.ascontiguousarray(b2[:, j0:j0 + 128]), c2[j0:j0 + 128], 1.5, 0.5, n, 128, n)
        assert np.array_equal(g2[j0:j0 + 128].reshape(-1).view(np.uint32), want.view(np.uint32)), j0
    for i0 in (0, 2176, n - 128):  # rows i0 .. i0 + 128 of C
        want = oracle.sgemm_nt(np.ascontiguousarray(a2[:, i0:i0 + 128]), b, np.ascontiguousarray(c2[:, i0:i0 + 128]), 1.5, 0.5,
                               128, n, n)
        assert np.array_equal(np.ascontiguousarray(g2[:, i0:i0 + 128]).reshape(-1).view(np.uint32), want.view(np.uint32)), i0
    for i, j in [(127, 128), (128, 127), (1000, 3001), (2048, 64), (63, 4032)]:
        want = np.float32(oracle.sgemm_nt_naive_elem(a, b, float(c0[i + j * n]), 1.5, 0.5, n, n, n, i, j))
        assert got[i + j * n].view(np.uint32) == want.view(np.uint32), (i, j)


# ------------------------------------------------------------------------- gemm
GEMM_SHAPES = [(128, 128, 64), (256, 128, 96), (128, 256, 160), (256, 256, 256), (512, 512, 512), (128, 128, 32),
               (384, 640, 1088)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("ab_name", ["f16", "bf16"])
@pytest.mark.parametrize("cta_group,tile_n,tile_m", [(1, 128, 128), (1, 256, 128), (2, 128, 128), (2, 256, 128), (1, 128, 256),
                                                      (1, 256, 256), (2, 128, 256), (2, 256, 256), (0, 0, 0),
                                                      (2, 128, 64), (2, 256, 64), (0, 0, 64)])
def test_gemm_small_integers_bit_exact(lib, gpu, m, n, k, ab_name, cta_group, tile_n, tile_m):
    ab = lib.F16 if ab_name == "f16" else lib.BF16
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = conv(lib, ab)(a.reshape(m, k)), conv(lib, ab)(b.reshape(n, k))
    got = run_gemm(lib, a_bits, b_bits, ab, lib.F32, tile_n=tile_n, cta_group=cta_group, tile_m=tile_m)
    want = oracle.gemm_tn(a_bits, b_bits, ab)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 128, 96), (128, 256, 160)])
@pytest.mark.parametrize("ab_name", ["f16", "bf16"])
def test_gemm_example_inputs_match_golden(lib, gpu, golden, shape, ab_name):
    m, n, k = shape
    ab = lib.F16 if ab_name == "f16" else lib.BF16
    a = ((np.arange(m * k, dtype=np.int64) * 7 + 3) % 7 - 3).astype(np.float32).reshape(m, k)
    b = ((np.arange(n * k, dtype=np.int64) * 5 + 1) % 5 - 2).astype(np.float32).reshape(n, k)
    got = run_gemm(lib, conv(lib, ab)(a), conv(lib, ab)(b), ab, lib.F32)
    assert np.array_equal(got, golden[f"tensorop_int_{m}x{n}x{k}"].astype(np.float32))


@pytest.mark.parametrize("m,n,k", [(256, 128, 96), (256, 256, 256), (512, 384, 2048)])
@pytest.mark.parametrize("ab_name", ["f16", "bf16"])
@pytest.mark.parametrize("cta_group,tile_m", [(1, 128), (2, 128), (2, 256), (2, 64)])
def test_gemm_random_within_reference_bound(lib, gpu, m, n, k, ab_name, cta_group, tile_m):
    ab = lib.F16 if ab_name == "f16" else lib.BF16
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=False)
    a_bits, b_bits = conv(lib, ab)(a.reshape(m, k)), conv(lib, ab)(b.reshape(n, k))
    got = run_gemm(lib, a_bits, b_bits, ab, lib.F32, cta_group=cta_group, tile_m=tile_m)
    want = oracle.gemm_tn(a_bits, b_bits, ab)
    allowed = tensor_core_bound(k, oracle.gemm_tn_abs(a_bits, b_bits, ab))
    assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= allowed).all()


def test_gemm_config0_256_cubed_uniform_seed0(lib, gpu):
    """tensorop_gemm 256^3, f16 uniform[-1, 1) seed 0, C zeros, alpha 1, beta 0."""
    rng = np.random.default_rng(0)
    a = oracle.f32_to_f16_bits(rng.uniform(-1, 1, (256, 256)).astype(np.float32))
    b = oracle.f32_to_f16_bits(rng.uniform(-1, 1, (256, 256)).astype(np.float32))
    got = run_gemm(lib, a, b, lib.F16, lib.F32)
    want = oracle.gemm_tn(a, b, lib.F16)
    assert (np.abs(got.astype(np.float64) - want) <= tensor_core_bound(256, oracle.gemm_tn_abs(a, b, lib.F16))).all()


@pytest.mark.parametrize("m,n,k", [(1, 1, 8), (100, 200, 72), (200, 136, 8), (129, 257, 520), (300, 520, 200), (128, 130, 64)])
@pytest.mark.parametrize("cdt_name", ["f32", "bf16"])
@pytest.mark.parametrize("cta_group,tile_m", [(1, 128), (2, 128), (2, 256), (1, 256), (2, 64), (0, 64)])
def test_gemm_ragged_shapes(lib, gpu, m, n, k, cdt_name, cta_group, tile_m):
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a.reshape(m, k)), oracle.f32_to_bf16_bits(b.reshape(n, k))
    got = run_gemm(lib, a_bits, b_bits, lib.BF16, cdt, cta_group=cta_group, tile_m=tile_m)
    want = oracle.gemm_tn(a_bits, b_bits, lib.BF16, cdt)
    if cdt == lib.F32:
        assert np.array_equal(got, want)
    else:  # integer sums can exceed 8 significand bits: compare after the same rounding
        assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (100, 200, 72), (200, 136, 8), (129, 257, 520), (300, 520, 200), (128, 130, 64),
                                   (512, 384, 1088), (64, 64, 0)])
@pytest.mark.parametrize("cdt_name", ["f32", "bf16"])
@pytest.mark.parametrize("cta_group,tile_m", [(0, 0), (1, 128), (2, 128), (2, 256), (2, 64)])
@pytest.mark.parametrize("register_stores", [False, True])
def test_gemm_several_destinations(lib, gpu, m, n, k, cdt_name, cta_group, tile_m, register_stores):
    """gemm_tn_multi writes the same C to every destination, by TMA stores where the
    row pitch allows them (a multiple of 16 bytes) and from registers otherwise."""
    import torch
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    a, b, _ = lcg_buffers([m * max(k, 1), n * max(k, 1), 0], small=True)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a[:m * k].reshape(m, k)), oracle.f32_to_bf16_bits(b[:n * k].reshape(n, k))
    want = oracle.gemm_tn(a_bits, b_bits, lib.BF16, cdt)
    np_c = np.float32 if cdt == lib.F32 else np.uint16
    # a guard row after each destination shows stores that run past the end
    dests = [dev(np.full((m + 1, n), 7, np_c)) for _ in range(3)]
    dA, dB = dev(a_bits if k else np.zeros((1, 8), np.uint16)), dev(b_bits if k else np.zeros((1, 8), np.uint16))
    d = lib.gemm_desc(m, n, k, lib.BF16, cdt, 1.0, 0.0, 0, cta_group, tile_m, 0)
    if register_stores:
        d.tuning[0] |= 16
    lib.gemm_tn_multi(d, dA.data_ptr() if k else 0, dB.data_ptr() if k else 0, [t.data_ptr() for t in dests], 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    for t in dests:
        got = host(t, np_c).reshape(m + 1, n)
        assert np.array_equal(got[:m], want)
        assert np.all(got[m] == 7)


@pytest.mark.parametrize("cdt_name", ["f32", "bf16"])
def test_gemm_eight_destinations(lib, gpu, cdt_name):
    """The largest fan-out the entry point takes (one own C and seven peers)."""
    import torch
    m, n, k = 1024, 768, 512
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a.reshape(m, k)), oracle.f32_to_bf16_bits(b.reshape(n, k))
    want = oracle.gemm_tn(a_bits, b_bits, lib.BF16, cdt)
    np_c = np.float32 if cdt == lib.F32 else np.uint16
    dests = [dev(np.full((m, n), 3, np_c)) for _ in range(8)]
    dA, dB = dev(a_bits), dev(b_bits)
    lib.gemm_tn_multi(lib.gemm_desc(m, n, k, lib.BF16, cdt), dA.data_ptr(), dB.data_ptr(), [t.data_ptr() for t in dests], 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    for t in dests:
        assert np.array_equal(host(t, np_c).reshape(m, n), want)


@pytest.mark.parametrize("seed", range(3))
def test_gemm_several_destinations_random(lib, gpu, seed):
    """Seeded sweep of the several-destination form: ragged sizes, both output types, every tiling,
    two to five copies; small-integer data, bit-exact, guard rows untouched."""
    import torch
    rng = np.random.default_rng(500 + seed)
    for _ in range(8):
        m, n = int(rng.integers(1, 900)), int(rng.integers(1, 900))
        if rng.integers(3):
            n = (n + 7) // 8 * 8  # mostly pitches the pusher can take; the rest go the register way
        k = 8 * int(rng.integers(1, 120))
        cdt = lib.F32 if rng.integers(2) else lib.BF16
        cta_group, tile_n, tile_m = int(rng.integers(0, 3)), int(rng.choice([0, 128, 256])), int(rng.choice([0, 128, 256]))
        copies = int(rng.integers(2, 6))
        a_bits = oracle.f32_to_bf16_bits(rng.integers(-4, 5, (m, k)).astype(np.float32))
        b_bits = oracle.f32_to_bf16_bits(rng.integers(-4, 5, (n, k)).astype(np.float32))
        want = oracle.gemm_tn(a_bits, b_bits, lib.BF16, cdt)
        np_c = np.float32 if cdt == lib.F32 else np.uint16
        dests = [dev(np.full((m + 1, n), 7, np_c)) for _ in range(copies)]
        dA, dB = dev(a_bits), dev(b_bits)
        d = lib.gemm_desc(m, n, k, lib.BF16, cdt, 1.0, 0.0, tile_n, cta_group, tile_m, 0)
        lib.gemm_tn_multi(d, dA.data_ptr(), dB.data_ptr(), [x.data_ptr() for x in dests], 0)
        torch.cuda.synchronize()
        assert lib.device_status() == (0, 0, 0, 0)
        for x in dests:
            got = host(x, np_c).reshape(m + 1, n)
            assert np.array_equal(got[:m], want) and np.all(got[m] == 7), (m, n, k, cdt, cta_group, tile_n, tile_m, copies)


def test_gemm_several_destinations_rejects_bad_arguments(lib, gpu):
    import torch
    c = torch.zeros(128 * 128 + 8, dtype=torch.float32, device="cuda")
    ab = torch.zeros(128 * 64, dtype=torch.int16, device="cuda")
    d = lib.gemm_desc(128, 128, 64, lib.BF16, lib.F32)
    with pytest.raises(lib.CuteB200Error):
        lib.gemm_tn_multi(d, ab.data_ptr(), ab.data_ptr(), [], 0)
    with pytest.raises(lib.CuteB200Error):
        lib.gemm_tn_multi(d, ab.data_ptr(), ab.data_ptr(), [c.data_ptr()] * 9, 0)
    with pytest.raises(lib.CuteB200Error):  # second destination in another 32-byte phase
        lib.gemm_tn_multi(d, ab.data_ptr(), ab.data_ptr(), [c.data_ptr(), c.data_ptr() + 4], 0)
    with pytest.raises(lib.CuteB200Error):
        lib.gemm_tn_multi(lib.gemm_desc(128, 128, 64, lib.BF16, lib.F32, 2.0, 0.0), ab.data_ptr(), ab.data_ptr(),
                          [c.data_ptr(), c.data_ptr()], 0)
    torch.cuda.synchronize()


@pytest.mark.parametrize("seed", range(6))
def test_gemm_random_shapes_and_tilings(lib, gpu, seed):
    """A seeded sweep: ten problems per seed with random ragged sizes, input and output types,
    tilings, k splits and epilogues, small-integer data, bit-exact against the oracle.  (With a k
    split the partial sums are exact integers below 2^24, so the order of the sums cannot show.)"""
    rng = np.random.default_rng(1000 + seed)
    for _ in range(10):
        m, n = int(rng.integers(1, 700)), int(rng.integers(1, 700))
        k = 8 * int(rng.integers(1, 160))
        ab = lib.F16 if rng.integers(2) else lib.BF16
        cdt = lib.F32 if rng.integers(2) else lib.BF16
        cta_group, tile_n, tile_m = int(rng.integers(0, 3)), int(rng.choice([0, 128, 256])), int(rng.choice([0, 128, 256]))
        split_k = int(rng.choice([0, 1, 1, 2, 3, 5]))
        alpha, beta = [(1.0, 0.0), (1.0, 0.0), (2.0, 0.0), (1.0, 1.0), (0.5, -1.0)][int(rng.integers(5))]
        a = rng.integers(-4, 5, (m, k)).astype(np.float32)
        b = rng.integers(-4, 5, (n, k)).astype(np.float32)
        c0f = rng.integers(-8, 9, (m, n)).astype(np.float32)
        a_bits, b_bits = conv(lib, ab)(a), conv(lib, ab)(b)
        c0 = c0f if cdt == lib.F32 else oracle.f32_to_bf16_bits(c0f)
        got = run_gemm(lib, a_bits, b_bits, ab, cdt, alpha, beta, c0=c0.copy(), tile_n=tile_n, cta_group=cta_group,
                       tile_m=tile_m, split_k=split_k)
        want = oracle.gemm_tn(a_bits, b_bits, ab, cdt, alpha, beta, c_init=c0)
        assert np.array_equal(got, want), (m, n, k, ab, cdt, cta_group, tile_n, tile_m, split_k, alpha, beta)


@pytest.mark.parametrize("cdt_name", ["f32", "bf16"])
@pytest.mark.parametrize("alpha,beta", [(1.5, -0.5), (0.0, 1.0), (2.0, 0.0), (1.0, 1.0)])
@pytest.mark.parametrize("tile_m", [64, 128, 256])
def test_gemm_alpha_beta_epilogue(lib, gpu, cdt_name, alpha, beta, tile_m):
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    m, n, k = 256, 384, 128
    a, b, c = lcg_buffers([m * k, n * k, m * n], small=True)
    a_bits, b_bits = oracle.f32_to_f16_bits(a.reshape(m, k)), oracle.f32_to_f16_bits(b.reshape(n, k))
    c0 = c.reshape(m, n) if cdt == lib.F32 else oracle.f32_to_bf16_bits(c.reshape(m, n))
    got = run_gemm(lib, a_bits, b_bits, lib.F16, cdt, alpha, beta, c0=c0, tile_m=tile_m)
    want = oracle.gemm_tn(a_bits, b_bits, lib.F16, cdt, alpha, beta, c_init=c0)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k", [(256, 128, 512), (200, 136, 328), (512, 256, 1088), (128, 128, 64), (143, 365, 1080), (9, 7, 512),
                                   (256, 136, 1600)])
@pytest.mark.parametrize("split_k", [2, 3, 5, 6, 16])
@pytest.mark.parametrize("cdt_name,alpha,beta", [("f32", 1.0, 0.0), ("bf16", 1.0, 0.0), ("f32", 1.5, -0.5), ("bf16", 2.0, 1.0)])
def test_gemm_split_k(lib, gpu, m, n, k, split_k, cdt_name, alpha, beta):
    """k cut into ranges summed by the second kernel (or, where the chosen tiling is a single-CTA
    128-row tile cut in two in one wave, inside the kernel by a cluster): exact on integer data.  The
    library takes the asked number of ranges as it is, cut down to the number of
    64-wide k blocks (k = 64 therefore runs unsplit); where the blocks do not
    divide evenly the last ranges stay empty and contribute zeros (k = 1600 in 6
    ranges: 25 blocks, five ranges of five and an empty one; k = 328 in 5: six
    blocks, three ranges of two and two empty ones)."""
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    a, b, c = lcg_buffers([m * k, n * k, m * n], small=True)
    a_bits, b_bits = oracle.f32_to_f16_bits(a.reshape(m, k)), oracle.f32_to_f16_bits(b.reshape(n, k))
    c0 = c.reshape(m, n) if cdt == lib.F32 else oracle.f32_to_bf16_bits(c.reshape(m, n))
    got = run_gemm(lib, a_bits, b_bits, lib.F16, cdt, alpha, beta, c0=c0, split_k=split_k)
    want = oracle.gemm_tn(a_bits, b_bits, lib.F16, cdt, alpha, beta, c_init=c0)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k,tile_n,split_k", [(128, 128, 256, 128, 2), (256, 128, 512, 128, 2), (1000, 200, 1024, 128, 4),
                                                  (384, 256, 512, 256, 2), (300, 520, 2048, 256, 4), (128, 136, 192, 128, 2),
                                                  (143, 365, 1080, 0, 2), (520, 264, 4160, 0, 4), (9, 7, 512, 128, 4)])
@pytest.mark.parametrize("cdt_name,alpha,beta", [("f32", 1.0, 0.0), ("bf16", 1.0, 0.0), ("f32", 1.5, -0.5), ("bf16", 2.0, 1.0)])
def test_gemm_split_k_summed_in_the_cluster(lib, gpu, m, n, k, tile_n, split_k, cdt_name, alpha, beta):
    """Single-CTA 128-row tiles cut in two or four ranges that fit one wave: the CTAs of a cluster
    take a tile's ranges, add their partial sums through each other's shared memory (ascending, like
    the second kernel of the two-pass form) and write C - one launch.  Exact on integer data; and on
    random data the same bits as the two-pass form (tuning bit 7), whose sums it restates."""
    import torch
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    a, b, c = lcg_buffers([m * k, n * k, m * n], small=True)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a.reshape(m, k)), oracle.f32_to_bf16_bits(b.reshape(n, k))
    c0 = c.reshape(m, n) if cdt == lib.F32 else oracle.f32_to_bf16_bits(c.reshape(m, n))
    want = oracle.gemm_tn(a_bits, b_bits, oracle.BF16, cdt, alpha, beta, c_init=c0)

    def run(a_bits, b_bits, tuning):
        dA, dB, dC = dev(a_bits), dev(b_bits), dev(c0)
        desc = lib.gemm_desc(m, n, k, lib.BF16, cdt, alpha, beta, tile_n, 1, 128, split_k)
        desc.tuning[0] = tuning
        before = lib.launch_count()
        lib.gemm_tn(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
        torch.cuda.synchronize()
        assert lib.device_status() == (0, 0, 0, 0)
        return host(dC, c0.dtype).reshape(m, n), lib.launch_count() - before

    got, launches = run(a_bits, b_bits, 0)
    assert launches == 1 and np.array_equal(got, want)
    ra, rb, _ = lcg_buffers([m * k, n * k, 0], small=False)
    ra_bits, rb_bits = oracle.f32_to_bf16_bits(ra.reshape(m, k)), oracle.f32_to_bf16_bits(rb.reshape(n, k))
    in_cluster, one = run(ra_bits, rb_bits, 0)
    two_pass, two = run(ra_bits, rb_bits, 128)
    assert (one, two) == (1, 2) and np.array_equal(in_cluster, two_pass)


def test_gemm_launches_of_every_form_back_to_back(lib, gpu):
    """GEMM launches are programmatic dependents of the kernel before them, so a launch is set up while
    its predecessor drains.  Queue the forms one behind the other without a host wait in between - pair
    tiles, single CTAs, the 64-row tile, a k split in two kernels, a k split summed inside clusters,
    a launch whose C is the next one's A - and check every result at the end."""
    import torch
    rng = np.random.default_rng(11)
    m, n, k = 384, 256, 1024
    a_bits = oracle.f32_to_bf16_bits(rng.integers(-4, 5, (m, k)).astype(np.float32))
    b_bits = oracle.f32_to_bf16_bits(rng.integers(-4, 5, (n, k)).astype(np.float32))
    b2_bits = oracle.f32_to_bf16_bits(rng.integers(-1, 2, (128, n)).astype(np.float32))  # (n2, k2 = n) for the chained product
    want = oracle.gemm_tn(a_bits, b_bits, oracle.BF16, oracle.BF16)
    want_chain = oracle.gemm_tn(want, b2_bits, oracle.BF16, oracle.F32)
    dA, dB, dB2 = dev(a_bits), dev(b_bits), dev(b2_bits)
    forms = [dict(cta_group=2, tile_m=256), dict(cta_group=1, tile_m=128, split_k=1), dict(cta_group=2, tile_m=64),
             dict(cta_group=2, tile_m=128, split_k=2), dict(cta_group=1, tile_m=128, tile_n=128, split_k=2),
             dict(cta_group=1, tile_m=128, split_k=4), dict()]
    outs = [torch.zeros(m, n, dtype=torch.int16, device="cuda") for _ in forms]
    chains = [torch.zeros(m, 128, device="cuda") for _ in forms]
    for _ in range(4):
        for kw, c, chain in zip(forms, outs, chains):
            lib.gemm_tn(lib.gemm_desc(m, n, k, lib.BF16, lib.BF16, **kw), dA.data_ptr(), dB.data_ptr(), c.data_ptr(), 0)
            # the next launch reads what this one wrote
            lib.gemm_tn(lib.gemm_desc(m, 128, n, lib.BF16, lib.F32), c.data_ptr(), dB2.data_ptr(), chain.data_ptr(), 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    for kw, c, chain in zip(forms, outs, chains):
        assert np.array_equal(host(c, np.uint16).reshape(m, n), want), kw
        assert np.array_equal(chain.cpu().numpy(), want_chain), kw


@pytest.mark.parametrize("seed", range(3))
def test_gemm_64_row_tile_random_shapes(lib, gpu, seed):
    """The 64-rows-per-CTA pair tile (tile_m = 64) over random ragged sizes, both column
    widths, input and output types, k splits and epilogues; integer data, bit-exact."""
    rng = np.random.default_rng(6400 + seed)
    for _ in range(10):
        m, n = int(rng.integers(1, 700)), int(rng.integers(1, 700))
        k = 8 * int(rng.integers(1, 260))
        ab = lib.F16 if rng.integers(2) else lib.BF16
        cdt = lib.F32 if rng.integers(2) else lib.BF16
        tile_n, cta_group = int(rng.choice([0, 128, 256])), int(rng.choice([0, 2]))
        split_k = int(rng.choice([0, 1, 1, 2, 3]))
        alpha, beta = [(1.0, 0.0), (1.0, 0.0), (2.0, 0.0), (1.0, 1.0), (0.5, -1.0)][int(rng.integers(5))]
        a_bits = conv(lib, ab)(rng.integers(-4, 5, (m, k)).astype(np.float32))
        b_bits = conv(lib, ab)(rng.integers(-4, 5, (n, k)).astype(np.float32))
        c0f = rng.integers(-8, 9, (m, n)).astype(np.float32)
        c0 = c0f if cdt == lib.F32 else oracle.f32_to_bf16_bits(c0f)
        got = run_gemm(lib, a_bits, b_bits, ab, cdt, alpha, beta, c0=c0.copy(), tile_n=tile_n, cta_group=cta_group, tile_m=64,
                       split_k=split_k)
        want = oracle.gemm_tn(a_bits, b_bits, ab, cdt, alpha, beta, c_init=c0)
        assert np.array_equal(got, want), (m, n, k, ab, cdt, cta_group, tile_n, split_k, alpha, beta)


def test_gemm_64_row_tile_needs_a_pair(lib, gpu):
    with pytest.raises(lib.CuteB200Error) as e:
        lib.gemm_tn(lib.gemm_desc(128, 128, 64, lib.F16, lib.F32, cta_group=1, tile_m=64), 256, 256, 256, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "CTA pair" in e.value.message


def test_gemm_split_k_random_within_bound(lib, gpu):
    m, n, k = 256, 128, 4096
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=False)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a.reshape(m, k)), oracle.f32_to_bf16_bits(b.reshape(n, k))
    want = oracle.gemm_tn(a_bits, b_bits, lib.BF16)
    allowed = tensor_core_bound(k, oracle.gemm_tn_abs(a_bits, b_bits, lib.BF16))
    for split_k in (0, 4, 8):  # 0: the library splits this shape on its own
        got = run_gemm(lib, a_bits, b_bits, lib.BF16, lib.F32, split_k=split_k)
        assert (np.abs(got.astype(np.float64) - want) <= allowed).all()


def test_gemm_split_k_on_two_streams_takes_turns(lib, gpu):
    """Split GEMMs share one scratch buffer per device.  Two of them queued on
    different streams (a skinny shape the library splits by itself, and a forced
    split of another size) must not mix their partial sums: the library orders
    them with an event.  Integer data, so any mixing shows as wrong bits."""
    import torch
    shapes = [(8192, 128, 2048, 0), (1024, 256, 4096, 8)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    cases = []
    for (m, n, k, split_k), seed in zip(shapes, (1, 2)):
        rng = np.random.default_rng(seed)
        a_bits = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (m, k)).astype(np.float32))
        b_bits = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (n, k)).astype(np.float32))
        cases.append((m, n, k, split_k, a_bits, b_bits, dev(a_bits.view(np.int16)), dev(b_bits.view(np.int16)),
                      torch.zeros(m, n, device="cuda"), oracle.gemm_tn(a_bits, b_bits, oracle.BF16)))
    torch.cuda.synchronize()
    for _ in range(6):
        for (m, n, k, split_k, _, _, dA, dB, dC, _), stream in zip(cases, streams):
            lib.gemm_tn(lib.gemm_desc(m, n, k, lib.BF16, lib.F32, split_k=split_k), dA.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                        stream.cuda_stream)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    for case in cases:
        assert np.array_equal(case[8].cpu().numpy(), case[9])


def test_gemm_k_zero_and_write_only_c(lib, gpu):
    m, n = 130, 70
    c0 = np.full((m, n), np.float32(np.nan))
    z = np.zeros((m, 0), np.uint16), np.zeros((n, 0), np.uint16)
    got = run_gemm(lib, z[0], z[1], lib.F16, lib.F32, c0=c0)
    assert not got.any()  # alpha 1, beta 0: C is never read, NaNs do not leak
    c1 = np.arange(m * n, dtype=np.float32).reshape(m, n)
    got = run_gemm(lib, z[0], z[1], lib.F16, lib.F32, 2.0, 0.5, c0=c1)
    assert np.array_equal(got, np.float32(0.5) * c1)
    # beta == 0 with prior NaNs in C and k > 0
    a, b, _ = lcg_buffers([128 * 64, 128 * 64, 0], small=True)
    a_bits, b_bits = oracle.f32_to_f16_bits(a.reshape(128, 64)), oracle.f32_to_f16_bits(b.reshape(128, 64))
    got = run_gemm(lib, a_bits, b_bits, lib.F16, lib.F32, c0=np.full((128, 128), np.float32(np.nan)))
    assert np.array_equal(got, oracle.gemm_tn(a_bits, b_bits, lib.F16))


def test_gemm_rejects_bad_arguments(lib, gpu):
    d = lib.gemm_desc(128, 128, 20, lib.F16, lib.F32)
    with pytest.raises(lib.CuteB200Error) as e:
        lib.gemm_tn(d, 256, 256, 256, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "multiple of 8" in e.value.message
    with pytest.raises(lib.CuteB200Error) as e:
        lib.gemm_tn(lib.gemm_desc(128, 128, 64, lib.F16, lib.F32), 256 + 2, 256, 256, 0)
    assert e.value.status == lib.ERR_MISALIGNED
    with pytest.raises(lib.CuteB200Error) as e:
        lib.gemm_tn(lib.gemm_desc(128, 128, 64, lib.F32, lib.F32), 256, 256, 256, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
                                   (8192, 128, 8192), (16384, 1024, 8192)])
def test_runtime_gemm_bf16_normal_inputs(lib, gpu, m, n, k):
    """The runtime_gemm sweep: bf16 in, bf16 out, normal(0, 0.02) seed 3.
    Large shapes are checked on a band of rows (the oracle computes only those)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.randn(m, k, device="cuda", generator=g) * 0.02).bfloat16()
    B = (torch.randn(n, k, device="cuda", generator=g) * 0.02).bfloat16()
    C = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    lib.gemm_tn(lib.gemm_desc(m, n, k, lib.BF16, lib.BF16), A.data_ptr(), B.data_ptr(), C.data_ptr(), 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    a_bits = A.view(torch.int16).cpu().numpy().view(np.uint16)
    b_bits = B.view(torch.int16).cpu().numpy().view(np.uint16)
    got = C.view(torch.int16).cpu().numpy().view(np.uint16)
    bands = [(0, min(m, 256))] if m <= 1024 else [(0, 128), (m // 2 - 64, m // 2 + 64), (m - 128, m)]
    for lo, hi in bands:
        acc = oracle.gemm_tn(a_bits, b_bits, lib.BF16, rows=(lo, hi))[lo:hi]
        mag = oracle.gemm_tn_abs(a_bits, b_bits, lib.BF16, rows=(lo, hi))[lo:hi]
        diff = np.abs(oracle.bf16_bits_to_f32(got[lo:hi]).astype(np.float64) - acc.astype(np.float64))
        # rounding the f32 result to bf16 costs half a unit; a result that lands
        # on the other side of a tie costs a whole one
        assert (diff <= tensor_core_bound(k, mag) + bf16_ulp(acc)).all()


@pytest.mark.parametrize("rank", [0, 5])
def test_row_sharded_gemm_config_on_one_gpu(lib, gpu, rank):
    """The 8-GPU workload, 32768 x 32768 x 8192 bf16 with normal(0, 0.02) inputs, as one rank
    of eight sees it (cute_b200_gemm_tn_shard: 4096 rows of A, all of B, its rows of a full-size
    C are not allocated here, so the shard goes to a C of its own).  Checked on bands of rows
    against the oracle, and the two placements of C (own block / offset into a full C) agree."""
    import torch
    M = N = 32768
    K = 8192
    world = 8
    begin, rows = lib.shard_rows(M, world, rank)
    assert (begin, rows) == (rank * 4096, 4096)
    g = torch.Generator(device="cuda").manual_seed(4 + rank)
    A = (torch.randn(rows, K, device="cuda", generator=g) * 0.02).bfloat16()
    B = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    C = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    desc = lib.gemm_desc(M, N, K, lib.BF16, lib.BF16)
    lib.gemm_tn_shard(desc, world, rank, A.data_ptr(), B.data_ptr(), C.data_ptr(), False, 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    # c_is_full: given the base of a full C the call writes at the rank's row offset; the base passed
    # here is chosen so that those rows are exactly a second buffer (nothing else is touched)
    C2 = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    lib.gemm_tn_shard(desc, world, rank, A.data_ptr(), B.data_ptr(), C2.data_ptr() - begin * N * 2, True, 0)
    torch.cuda.synchronize()
    assert torch.equal(C.view(torch.int16), C2.view(torch.int16))
    a_bits = A.view(torch.int16).cpu().numpy().view(np.uint16)
    b_bits = B.view(torch.int16).cpu().numpy().view(np.uint16)
    got = C.view(torch.int16).cpu().numpy().view(np.uint16)
    for lo, hi in [(0, 32), (2048 - 16, 2048 + 16), (rows - 32, rows)]:
        acc = oracle.gemm_tn(a_bits, b_bits, lib.BF16, rows=(lo, hi))[lo:hi]
        mag = oracle.gemm_tn_abs(a_bits, b_bits, lib.BF16, rows=(lo, hi))[lo:hi]
        diff = np.abs(oracle.bf16_bits_to_f32(got[lo:hi]).astype(np.float64) - acc.astype(np.float64))
        assert (diff <= tensor_core_bound(K, mag) + bf16_ulp(acc)).all()


def test_gemm_c_beyond_2_31_elements(lib, gpu):
    """A C of 65536 x 33000 = 2.16e9 elements (the reference stops at 2^31: 32-bit element offsets):
    rows at both ends and around the 2^31st element are checked against the oracle."""
    import torch
    m, n, k = 65536, 33000, 64
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randint(-3, 4, (m, k), device="cuda", generator=g).to(torch.bfloat16)
    B = torch.randint(-3, 4, (n, k), device="cuda", generator=g).to(torch.bfloat16)
    C = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    lib.gemm_tn(lib.gemm_desc(m, n, k, lib.BF16, lib.BF16), A.data_ptr(), B.data_ptr(), C.data_ptr(), 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (0, 0, 0, 0)
    b_bits = B.view(torch.int16).cpu().numpy().view(np.uint16)
    edge = (1 << 31) // n  # the row that holds element 2^31
    for lo in (0, edge - 2, m - 4):
        a_bits = A[lo:lo + 4].view(torch.int16).cpu().numpy().view(np.uint16)
        want = oracle.gemm_tn(a_bits, b_bits, lib.BF16, lib.BF16)
        got = C[lo:lo + 4].view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got, want), lo


def test_elementwise_add_beyond_2_31_elements(lib, gpu):
    """2^31 + 5 elements: 64-bit indexing in the kernel; the ends and the neighbourhood of 2^31 are compared."""
    import torch
    n = (1 << 31) + 5
    x = torch.empty(n, device="cuda").uniform_(-1, 1)
    y = torch.empty(n, device="cuda").uniform_(-1, 1)
    out = torch.full((n + 3,), 2.0, device="cuda")
    lib.elementwise_add_f32(x.data_ptr(), y.data_ptr(), out.data_ptr(), n, 0)
    torch.cuda.synchronize()
    for lo in (0, (1 << 31) - 4096, n - 4096):
        want = oracle.elementwise_add(x[lo:lo + 4096].cpu().numpy(), y[lo:lo + 4096].cpu().numpy())
        assert np.array_equal(out[lo:lo + 4096].cpu().numpy().view(np.uint32), want.view(np.uint32)), lo
    assert bool((out[n:] == 2.0).all())
    del x, y, out
    torch.cuda.empty_cache()


def test_gemm_full_size_properties(lib, gpu):
    """8192^3 bf16: linearity in A (exact for a power-of-two scale) and
    agreement of the two tilings on sampled rows."""
    import torch
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.randn(n, n, device="cuda", generator=g) * 0.02).bfloat16()
    B = (torch.randn(n, n, device="cuda", generator=g) * 0.02).bfloat16()
    C1 = torch.empty(n, n, device="cuda", dtype=torch.float32)
    C2 = torch.empty_like(C1)
    lib.gemm_tn(lib.gemm_desc(n, n, n, lib.BF16, lib.F32), A.data_ptr(), B.data_ptr(), C1.data_ptr(), 0)
    A2 = (A.float() * 2).bfloat16()
    lib.gemm_tn(lib.gemm_desc(n, n, n, lib.BF16, lib.F32), A2.data_ptr(), B.data_ptr(), C2.data_ptr(), 0)
    torch.cuda.synchronize()
    assert torch.equal(C2, C1 * 2)  # scaling by two is exact at every step
    lib.gemm_tn(lib.gemm_desc(n, n, n, lib.BF16, lib.F32, tile_n=128, cta_group=1, tile_m=128), A.data_ptr(), B.data_ptr(), C2.data_ptr(), 0)
    torch.cuda.synchronize()
    assert torch.equal(C2, C1)  # same k order per output in every tiling
    a_bits = A[4000:4016].view(torch.int16).cpu().numpy().view(np.uint16)
    b_bits = B.view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.gemm_tn(a_bits, b_bits, lib.BF16)
    mag = oracle.gemm_tn_abs(a_bits, b_bits, lib.BF16)
    diff = np.abs(C1[4000:4016].cpu().numpy().astype(np.float64) - want)
    assert (diff <= tensor_core_bound(n, mag)).all()


@pytest.mark.parametrize("m,n,k,cdt_name,alpha,beta", [(4096, 512, 256, "f32", 1.0, 0.0), (2600, 264, 136, "bf16", 1.0, 0.0),
                                                        (3000, 128, 64, "f32", 1.5, -0.5), (100, 72, 0, "f32", 2.0, 0.5),
                                                        (4096, 2304, 1024, "bf16", 1.0, 0.0), (3000, 1304, 1024, "f32", 1.5, -0.5),
                                                        (520, 4104, 2048, "bf16", 2.0, 1.0)])
def test_gemm_host_buffers_pipelined(lib, gpu, m, n, k, cdt_name, alpha, beta):
    """cute_b200_gemm_tn_host: host buffers in and out.  The larger cases are cut
    into panels of A and B that go up alternately; every panel unlocks a block of
    C that is multiplied (into a strided block of the device C) and comes down
    while the next panels go up."""
    cdt = lib.F32 if cdt_name == "f32" else lib.BF16
    a, b, c = lcg_buffers([m * k, n * k, m * n], small=True)
    a_bits = oracle.f32_to_f16_bits(a.reshape(m, k))
    b_bits = oracle.f32_to_f16_bits(b.reshape(n, k))
    c0 = c.reshape(m, n).copy() if cdt == lib.F32 else oracle.f32_to_bf16_bits(c.reshape(m, n))
    want = oracle.gemm_tn(a_bits, b_bits, lib.F16, cdt, alpha, beta, c_init=c0)
    a_in, b_in = a_bits.copy(), b_bits.copy()
    for _ in range(2):  # the second call reuses the staging buffers
        hc = c0.copy()
        sec = lib.gemm_tn_host(lib.gemm_desc(m, n, k, lib.F16, cdt, alpha, beta), a_bits.ctypes.data if k else 0,
                               b_bits.ctypes.data if k else 0, hc.ctypes.data)
        assert np.array_equal(hc, want) and sec >= 0.0
    assert np.array_equal(a_bits, a_in) and np.array_equal(b_bits, b_in)  # inputs untouched
    lib.release_workspace()


def test_gemm_host_buffers_random_shapes(lib, gpu):
    """Seeded ragged problems through the host-buffer call: sizes large enough for several panels of
    A and B, so the blocks of C are strided pieces of the device C and come down as pitched copies."""
    rng = np.random.default_rng(31)
    for _ in range(6):
        m, n = int(rng.integers(300, 2400)), int(rng.integers(300, 2400))
        k = 8 * int(rng.integers(64, 300))
        cdt = lib.F32 if rng.integers(2) else lib.BF16
        alpha, beta = [(1.0, 0.0), (1.0, 0.0), (2.0, -1.0)][int(rng.integers(3))]
        a_bits = oracle.f32_to_bf16_bits(rng.integers(-3, 4, (m, k)).astype(np.float32))
        b_bits = oracle.f32_to_bf16_bits(rng.integers(-3, 4, (n, k)).astype(np.float32))
        c0f = rng.integers(-8, 9, (m, n)).astype(np.float32)
        c0 = c0f if cdt == lib.F32 else oracle.f32_to_bf16_bits(c0f)
        want = oracle.gemm_tn(a_bits, b_bits, lib.BF16, cdt, alpha, beta, c_init=c0)
        hc = c0.copy()
        lib.gemm_tn_host(lib.gemm_desc(m, n, k, lib.BF16, cdt, alpha, beta), a_bits.ctypes.data, b_bits.ctypes.data, hc.ctypes.data)
        assert np.array_equal(hc, want), (m, n, k, cdt, alpha, beta)
    lib.release_workspace()


def test_alloc_upload_copy_download_round_trip(lib, gpu):
    """The memory entry points a multi-process caller builds on: allocate, upload, device-to-device copy,
    export a handle, download, free; null and zero-size arguments answer with status codes."""
    rng = np.random.default_rng(5)
    src = rng.integers(0, 255, 1 << 20, dtype=np.uint8)
    d0 = lib.upload(src.ctypes.data, src.nbytes)
    d1 = lib.alloc(src.nbytes)
    lib.copy_async(d1, d0, src.nbytes, 0)
    lib.synchronize()
    back = np.zeros_like(src)
    lib.download(d1, back.ctypes.data, back.nbytes)
    assert np.array_equal(back, src)
    handle = lib.ipc_export(d1)
    assert isinstance(handle, bytes) and len(handle) == 64 and any(handle)
    lib.copy_async(d1, d0, 0, 0)  # nothing to copy is not an error
    with pytest.raises(lib.CuteB200Error):
        lib.copy_async(0, d0, 16, 0)
    with pytest.raises(lib.CuteB200Error):
        lib.ipc_export(0)
    lib.free(d0)
    lib.free(d1)


# -------------------------------------------------------- launch by kernel name
def test_launch_by_name_mirrors_the_reference_examples(lib, gpu, golden):
    from cute_rs_b200 import CudaContext, DeviceArg, DType
    from cute_rs_b200 import examples as ex
    ctx = CudaContext.new(0)
    # tensorop_gemm, f16 and bf16 (examples/tensorop_gemm.rs:167-186)
    for ab in (DType.F16, DType.BF16):
        cfg = ex.GemmConfig(256, 128, 96, ab=ab)
        kernel = ex.tensorop_gemm(cfg)
        launch, args, a, b = ex.tensorop_gemm_problem(cfg)
        stats = kernel.run_cuda(ctx, launch, args)
        assert stats.kernel_seconds > 0.0
        assert np.array_equal(args[2].as_f32().reshape(256, 128), golden["tensorop_int_256x128x96"].astype(np.float32))
    # runtime_gemm: one kernel, several sizes, then device-resident relaunch
    # (tests/gpu.rs:212-241)
    kernel = ex.runtime_gemm()
    for m, n, k in [(128, 128, 32), (256, 128, 96), (128, 256, 160), (512, 512, 512)]:
        launch, args, a, b = ex.runtime_gemm_problem(m, n, k)
        ctx.launch(kernel, launch, args)
        want = a.reshape(m, k).astype(np.int64) @ b.reshape(n, k).astype(np.int64).T
        assert np.array_equal(args[2].as_f32().reshape(m, n), want.astype(np.float32))
    launch, args, a, b = ex.runtime_gemm_problem(256, 256, 64)
    ua, ub, uc = ctx.upload(args[0]), ctx.upload(args[1]), ctx.upload(args[2])
    dargs = [DeviceArg.Buffer(ua), DeviceArg.Buffer(ub), DeviceArg.Buffer(uc), DeviceArg.Scalar(args[3]), DeviceArg.Scalar(args[4])]
    for _ in range(3):
        ctx.launch_async(kernel, launch, dargs)
    ctx.synchronize()
    ctx.download(uc, args[2])
    want = a.reshape(256, 64).astype(np.int64) @ b.reshape(256, 64).astype(np.int64).T
    assert np.array_equal(args[2].as_f32().reshape(256, 256), want.astype(np.float32))
    # sgemm (examples/sgemm.rs:84-112) and elementwise add (examples/elementwise_add.rs:82-91)
    launch, args, *_ = ex.sgemm_problem(256, 256, 64)
    ex.sgemm(256, 256, 64).run_cuda(ctx, launch, args)
    assert np.array_equal(args[2].as_f32(), golden["sgemm_int_256x256x64"])
    from cute_rs_b200 import LaunchConfig
    for kernel, grid, block in [(ex.elementwise_add_naive(), ex.naive_grid(), [256, 1, 1]),
                                (ex.elementwise_add_tiled(), ex.tiled_grid(), [128, 1, 1])]:
        args, a, b = ex.elementwise_add_problem()
        kernel.run_cuda(ctx, LaunchConfig.new(grid, block), args)
        assert np.array_equal(args[2].as_f32(), golden["add_int_300x512"])
        assert np.array_equal(args[0].as_f32(), a) and np.array_equal(args[1].as_f32(), b)  # inputs untouched


def test_launch_by_name_errors(lib, gpu):
    from cute_rs_b200 import CudaContext, CudaError, KernelArg, LaunchConfig
    from cute_rs_b200 import examples as ex
    ctx = CudaContext.new(0)
    kernel = ex.runtime_gemm()
    launch, args, *_ = ex.runtime_gemm_problem(128, 128, 32)
    args[4] = KernelArg.ScalarI32(40)
    with pytest.raises(CudaError, match=r"argument 4 \(`k`\) must be a multiple of 32, got 40"):
        ctx.launch(kernel, launch, args)
    launch, args, *_ = ex.runtime_gemm_problem(128, 128, 32)
    with pytest.raises(CudaError, match="needs at least"):
        ctx.launch(kernel, LaunchConfig.new([2, 1, 1], [128, 1, 1]), args)
    t = ex.tensorop_gemm(ex.GemmConfig.new(128, 128, 64))
    launch, args, *_ = ex.tensorop_gemm_problem(ex.GemmConfig.new(128, 128, 32))
    with pytest.raises(CudaError, match=r"argument 0 \(`a`\) needs at least 8192 elements, got 4096"):
        ctx.launch(t, launch, args)
