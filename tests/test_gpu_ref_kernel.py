"""The restated reference GPU kernel (oracle/ref_kernel_sm80.cu: mma.sync,
cp.async ring, ldmatrix, the reference's swizzle) against the CPU oracle, with
the reference's own acceptance rule (tests/gpu.rs:146-176).  It is the GPU
baseline the sm_100a kernel is timed against, so it has to be right too."""
import numpy as np
import pytest

import oracle
from tests.util import lcg_buffers, tensor_core_bound

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 128, 96), (256, 256, 256), (128, 128, 32), (384, 256, 1024)])
@pytest.mark.parametrize("bf16", [False, True])
def test_restated_reference_kernel_matches_oracle(gpu, m, n, k, bf16):
    import torch
    conv = oracle.f32_to_bf16_bits if bf16 else oracle.f32_to_f16_bits
    dt = oracle.BF16 if bf16 else oracle.F16
    for small in (True, False):
        a, b, _ = lcg_buffers([m * k, n * k, 0], small=small)
        a_bits, b_bits = conv(a.reshape(m, k)), conv(b.reshape(n, k))
        dA = torch.from_numpy(a_bits.view(np.int16)).cuda()
        dB = torch.from_numpy(b_bits.view(np.int16)).cuda()
        dC = torch.full((m, n), float("nan"), device="cuda")
        oracle.ref_tensorop_gemm(bf16, m, n, k, dA.data_ptr(), dB.data_ptr(), dC.data_ptr())
        torch.cuda.synchronize()
        got, want = dC.cpu().numpy(), oracle.gemm_tn(a_bits, b_bits, dt)
        if small:
            assert np.array_equal(got, want)
        else:
            assert (np.abs(got.astype(np.float64) - want) <= tensor_core_bound(k, oracle.gemm_tn_abs(a_bits, b_bits, dt))).all()
