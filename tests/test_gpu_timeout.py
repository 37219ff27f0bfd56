"""Failure detection without a GPU fault: the producer of the GEMM kernel is
told to issue nothing, so every consumer wait inside the kernel runs out (after
a 20 ms limit), the kernel drains and returns, the host reads the report as
CUTE_B200_ERR_DEVICE_TIMEOUT, and the context stays usable."""
import numpy as np
import pytest

import oracle
from tests.util import lcg_buffers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cta_group,tile_m", [(1, 128), (2, 256)])
def test_wait_that_runs_out_is_reported_and_the_device_stays_usable(lib, gpu, cta_group, tile_m):
    import torch
    m, n, k = 512, 256, 256
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = oracle.f32_to_f16_bits(a.reshape(m, k)), oracle.f32_to_f16_bits(b.reshape(n, k))
    dA = torch.from_numpy(a_bits.view(np.int16)).cuda()
    dB = torch.from_numpy(b_bits.view(np.int16)).cuda()
    dC = torch.zeros(m, n, device="cuda")
    desc = lib.gemm_desc(m, n, k, lib.F16, lib.F32, cta_group=cta_group, tile_m=tile_m, split_k=1)
    desc.tuning[0] = 4 | 8  # the producer withholds every load; waits give up after 20 ms
    lib.gemm_tn(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    with pytest.raises(lib.CuteB200Error) as e:
        lib.synchronize()
    assert e.value.status == lib.ERR_DEVICE_TIMEOUT and "bounded wait gave up" in e.value.message
    assert lib.device_status() == (0, 0, 0, 0)  # the report was consumed
    # the same problem without the knob: correct result, no report
    desc.tuning[0] = 0
    lib.gemm_tn(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    lib.synchronize()
    assert np.array_equal(dC.cpu().numpy(), oracle.gemm_tn(a_bits, b_bits, oracle.F16))


def test_pusher_gives_up_with_the_other_roles(lib, gpu):
    """The several-destination form under the same knob: the pusher warp waits for
    tiles that never come, sees the CTA give up, and returns with everything else;
    afterwards the same call delivers C to every destination."""
    import torch
    m, n, k = 512, 512, 256
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a.reshape(m, k)), oracle.f32_to_bf16_bits(b.reshape(n, k))
    dA = torch.from_numpy(a_bits.view(np.int16)).cuda()
    dB = torch.from_numpy(b_bits.view(np.int16)).cuda()
    dests = [torch.zeros(m, n, device="cuda") for _ in range(3)]
    desc = lib.gemm_desc(m, n, k, lib.BF16, lib.F32)
    desc.tuning[0] = 4 | 8
    lib.gemm_tn_multi(desc, dA.data_ptr(), dB.data_ptr(), [t.data_ptr() for t in dests], 0)
    with pytest.raises(lib.CuteB200Error) as e:
        lib.synchronize()
    assert e.value.status == lib.ERR_DEVICE_TIMEOUT
    desc.tuning[0] = 0
    lib.gemm_tn_multi(desc, dA.data_ptr(), dB.data_ptr(), [t.data_ptr() for t in dests], 0)
    lib.synchronize()
    want = oracle.gemm_tn(a_bits, b_bits, oracle.BF16)
    for t in dests:
        assert np.array_equal(t.cpu().numpy(), want)
