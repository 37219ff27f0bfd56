"""cute_b200_gemm_tn_static: the split-k GEMM that allocates no device memory.

Some users of the library cannot call cudaMalloc at the moment they need a
GEMM: their GPU memory belongs to a pool with a fixed budget, or they sit in a
latency-critical loop where cudaMalloc's device-wide synchronisation is not
acceptable.  For them the library offers this variant, whose scratch is a
32 MiB array built into the library image.  The checks here go through the C
ABI and compare it with the ordinary entry point on two calls in a row; the
second call is smaller than the first, so the stale partial sums the first one
left in the shared array would show up if the kernel ever read them.

The file sorts last on purpose: a run that stops at the first failure has then
already covered everything else.  It does not use the fixture that calls
cute_b200_init, so run alone it also exercises the entry point's own first-call
set-up.
"""
import numpy as np
import pytest

import oracle
from tests.util import lcg_buffers

pytestmark = pytest.mark.gpu


def _dev(bits):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def _both(lib, m, n, k, split_k, small, cdt, alpha=1.0, beta=0.0):
    """(static entry point, ordinary entry point) outputs for one problem."""
    import torch
    a, b, c = lcg_buffers([m * k, n * k, m * n], small=small)
    a_bits = oracle.f32_to_bf16_bits(a.reshape(m, k))
    b_bits = oracle.f32_to_bf16_bits(b.reshape(n, k))
    c0 = c.reshape(m, n).astype(np.float32) if cdt == lib.F32 else oracle.f32_to_bf16_bits(c.reshape(m, n))
    dA, dB = _dev(a_bits), _dev(b_bits)
    outs = []
    for fn in (lib.gemm_tn_static, lib.gemm_tn):
        dC = torch.from_numpy(c0.copy() if cdt == lib.F32 else c0.view(np.int16).copy()).cuda()
        fn(lib.gemm_desc(m, n, k, lib.BF16, cdt, alpha, beta, split_k=split_k), dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
        torch.cuda.synchronize()
        outs.append(dC.cpu().numpy())
    return outs[0], outs[1], a_bits, b_bits, c0


def test_static_scratch_gemm_matches_the_allocating_one_twice_in_a_row(lib):
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    # first call: 1024 x 512, 4 ranges = 8 MiB of the array; random data, bf16 out, alpha/beta
    got, ref, a_bits, b_bits, c0 = _both(lib, 1024, 512, 2048, 4, small=False, cdt=lib.BF16, alpha=1.5, beta=-0.5)
    assert np.array_equal(got, ref)  # same ranges added in the same order: identical bits
    # second call straight after: smaller, ragged, integer data, f32 out; checked against the oracle too
    got, ref, a_bits, b_bits, c0 = _both(lib, 200, 136, 328, 3, small=True, cdt=lib.F32)
    assert np.array_equal(got, ref)
    assert np.array_equal(got, oracle.gemm_tn(a_bits, b_bits, oracle.BF16))
    # and once more with the library choosing the split
    got, ref, a_bits, b_bits, c0 = _both(lib, 8192, 128, 1024, 0, small=True, cdt=lib.F32)
    want = oracle.gemm_tn(a_bits, b_bits, oracle.BF16)
    assert np.array_equal(got, want) and np.array_equal(ref, want)
    # five k blocks in four ranges: 2 + 2 + 1 and one range without a block, which must contribute zeros
    # over whatever the calls above left in the array; random data, so the order of the additions counts
    got, ref, a_bits, b_bits, c0 = _both(lib, 384, 256, 320, 4, small=False, cdt=lib.F32, alpha=0.75, beta=2.0)
    assert np.array_equal(got, ref)


def test_static_scratch_gemm_allocates_no_device_memory(lib):
    """What the entry point exists for: with its inputs and output in place, a call
    leaves the device's free memory exactly as it found it, and launches exactly two
    kernels (the k ranges, then their sum)."""
    import torch
    torch.cuda.set_device(0)
    m, n, k = 1024, 512, 2048
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    dA, dB = _dev(oracle.f32_to_bf16_bits(a.reshape(m, k))), _dev(oracle.f32_to_bf16_bits(b.reshape(n, k)))
    dC = torch.zeros(m, n, device="cuda")
    desc = lib.gemm_desc(m, n, k, lib.BF16, lib.F32, split_k=4)
    lib.gemm_tn_static(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)  # first call on the device: set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    launches_before = lib.launch_count()
    lib.gemm_tn_static(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert lib.launch_count() - launches_before == 2
    assert np.array_equal(dC.cpu().numpy(), oracle.gemm_tn(oracle.f32_to_bf16_bits(a.reshape(m, k)),
                                                           oracle.f32_to_bf16_bits(b.reshape(n, k)), oracle.BF16))


_NO_INIT_TIMEOUT = r"""
import sys
import numpy as np
import torch
sys.path.insert(0, sys.argv[1])
from cute_rs_b200 import _lib as lib
torch.cuda.set_device(0)
m, n, k = 256, 256, 512
dA = torch.ones(m, k, device="cuda", dtype=torch.bfloat16)
dB = torch.ones(n, k, device="cuda", dtype=torch.bfloat16)
dC = torch.zeros(m, n, device="cuda")
desc = lib.gemm_desc(m, n, k, lib.BF16, lib.F32, split_k=2)
lib.gemm_tn_static(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)  # set-up call, cute_b200_init never runs
torch.cuda.synchronize()
free_before, _ = torch.cuda.mem_get_info()
desc.tuning[0] = 4 | 8  # the producer withholds every load; waits give up after 20 ms
lib.gemm_tn_static(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
try:
    lib.synchronize()
    print("NO ERROR")
except lib.CuteB200Error as e:
    print("STATUS", e.status, e.message)
print("FREE_UNCHANGED", torch.cuda.mem_get_info()[0] == free_before)
print("CLEARED", lib.device_status())
desc.tuning[0] = 0
lib.gemm_tn_static(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
lib.synchronize()
print("RESULT_OK", bool((dC == float(k)).all()))
"""


def test_static_scratch_gemm_reports_a_timeout_without_init(lib):
    """In a fresh process that never calls cute_b200_init, a bounded wait that runs
    out inside the static entry point's kernel still reaches the host:
    cute_b200_synchronize returns CUTE_B200_ERR_DEVICE_TIMEOUT (read from the words
    the entry point owns, without allocating), the report is cleared, and the
    next call computes the right result.  The wait is made to run out by the
    test knob that keeps the producer from issuing anything; nothing faults."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _NO_INIT_TIMEOUT, root], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert f"STATUS {lib.ERR_DEVICE_TIMEOUT}" in out.stdout and "bounded wait gave up" in out.stdout, out.stdout
    assert "FREE_UNCHANGED True" in out.stdout, out.stdout
    assert "CLEARED (0, 0, 0, 0)" in out.stdout, out.stdout
    assert "RESULT_OK True" in out.stdout, out.stdout


def test_static_scratch_gemm_rejects_what_does_not_fit(lib):
    import torch
    torch.cuda.set_device(0)
    buf = torch.zeros(1 << 20, dtype=torch.int16, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(lib.CuteB200Error) as e:  # 4096 x 4096 x 4 B x 2 ranges = 128 MiB > 32 MiB
        lib.gemm_tn_static(lib.gemm_desc(4096, 4096, 4096, lib.BF16, lib.BF16, split_k=2), p, p, p, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "33554432" in e.value.message
    with pytest.raises(lib.CuteB200Error) as e:  # fits with 2 ranges, not with 16
        lib.gemm_tn_static(lib.gemm_desc(1024, 1024, 4096, lib.BF16, lib.BF16, split_k=16), p, p, p, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "built-in buffer" in e.value.message
    with pytest.raises(lib.CuteB200Error) as e:
        lib.gemm_tn_static(lib.gemm_desc(256, 256, 1024, lib.BF16, lib.BF16, split_k=1), p, p, p, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "split_k" in e.value.message
