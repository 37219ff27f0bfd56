"""Failure detection without a GPU fault: the producer of the GEMM kernel is
told to issue nothing, so every consumer wait inside the kernel runs out (after
a 20 ms limit), the kernel drains and returns, the host reads the report as
CUTE_B200_ERR_DEVICE_TIMEOUT, and the context stays usable."""
import numpy as np
import pytest

import oracle
from tests.util import lcg_buffers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cta_group,tile_m", [(1, 128), (2, 256), (2, 64)])
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


def test_split_summed_in_the_cluster_gives_up_cleanly(lib, gpu):
    """The k split whose ranges are added inside a cluster (single-CTA 128-row tiles, split in two):
    with the producer silent every CTA's waits run out, all CTAs still meet at the cluster barriers
    around the exchange, nothing is stored, and the report comes back as usual."""
    import torch
    m, n, k = 512, 256, 512
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = oracle.f32_to_f16_bits(a.reshape(m, k)), oracle.f32_to_f16_bits(b.reshape(n, k))
    dA = torch.from_numpy(a_bits.view(np.int16)).cuda()
    dB = torch.from_numpy(b_bits.view(np.int16)).cuda()
    dC = torch.full((m, n), 7.0, device="cuda")
    desc = lib.gemm_desc(m, n, k, lib.F16, lib.F32, cta_group=1, tile_m=128, split_k=2)
    assert lib.gemm_plan(desc) == (1, 256, 128, 2) or lib.gemm_plan(desc)[3] == 2
    desc.tuning[0] = 4 | 8
    before = lib.launch_count()
    lib.gemm_tn(desc, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0)
    assert lib.launch_count() - before == 1  # one kernel: the in-cluster form
    with pytest.raises(lib.CuteB200Error) as e:
        lib.synchronize()
    assert e.value.status == lib.ERR_DEVICE_TIMEOUT and "bounded wait gave up" in e.value.message
    assert (dC == 7.0).all().item()  # a CTA that gave up stores nothing
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


def test_completion_signal_and_its_bounded_wait(lib, gpu):
    """The several-destination GEMM with completion counters (what replaces a barrier among
    processes): the last CTA of a launch adds 1 to the counter of every further destination;
    cute_b200_wait_signal returns once the counters have reached the step.  A wait for a count
    that nobody sends runs out after its limit and is reported like every other bounded wait,
    a launch that gives up signals nothing, and the device stays usable throughout.  All
    destinations are on this one GPU and the wait kernel runs behind the GEMM on the same
    stream, so no kernel ever waits for a concurrent one here."""
    import torch
    m, n, k = 640, 512, 256
    a, b, _ = lcg_buffers([m * k, n * k, 0], small=True)
    a_bits, b_bits = oracle.f32_to_bf16_bits(a.reshape(m, k)), oracle.f32_to_bf16_bits(b.reshape(n, k))
    want = oracle.gemm_tn(a_bits, b_bits, oracle.BF16)
    dA = torch.from_numpy(a_bits.view(np.int16)).cuda()
    dB = torch.from_numpy(b_bits.view(np.int16)).cuda()
    dests = [torch.zeros(m, n, device="cuda") for _ in range(3)]
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    ptrs = [t.data_ptr() for t in dests]
    sig = [0, flags.data_ptr() + 4, flags.data_ptr() + 8]
    desc = lib.gemm_desc(m, n, k, lib.BF16, lib.F32)
    for step in (1, 2):
        for t in dests:
            t.zero_()
        lib.gemm_tn_multi_signal(desc, dA.data_ptr(), dB.data_ptr(), ptrs, sig, 0)
        lib.wait_signal(flags.data_ptr(), 0b110, step, 2000, 0)
        lib.synchronize()
        assert flags.cpu().tolist() == [0, step, step, 0, 0, 0, 0, 0]
        for t in dests:
            assert np.array_equal(t.cpu().numpy(), want)
    # a count that never comes: counter 3 stays at zero
    lib.wait_signal(flags.data_ptr(), 0b1110, 2, 20, 0)
    with pytest.raises(lib.CuteB200Error) as e:
        lib.synchronize()
    assert e.value.status == lib.ERR_DEVICE_TIMEOUT
    lib.wait_signal(flags.data_ptr(), 0b1000, 1, 20, 0)
    torch.cuda.synchronize()
    assert lib.device_status() == (7, 1, 3, 0)  # where, expected, which counter, what it held
    assert lib.device_status() == (0, 0, 0, 0)
    # a launch that gives up (the producer withholds every load) signals nothing ...
    desc.tuning[0] = 4 | 8
    lib.gemm_tn_multi_signal(desc, dA.data_ptr(), dB.data_ptr(), ptrs, sig, 0)
    with pytest.raises(lib.CuteB200Error):
        lib.synchronize()
    assert flags.cpu().tolist()[:3] == [0, 2, 2]
    # ... and the next one counts its CTAs from zero again and signals once
    desc.tuning[0] = 0
    lib.gemm_tn_multi_signal(desc, dA.data_ptr(), dB.data_ptr(), ptrs, sig, 0)
    lib.wait_signal(flags.data_ptr(), 0b110, 3, 2000, 0)
    lib.synchronize()
    assert flags.cpu().tolist()[:3] == [0, 3, 3]
    with pytest.raises(lib.CuteB200Error) as e:
        lib.wait_signal(flags.data_ptr(), 1, 1, 0, 0)
    assert e.value.status == lib.ERR_INVALID_ARGUMENT
