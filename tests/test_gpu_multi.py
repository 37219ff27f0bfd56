"""Two ranks on two GPUs: the row-sharded GEMM with C replicated by peer copies
and by panel-wise NCCL exchange.  Skipped on a box with a single GPU."""
import os
import socket

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cute_rs_b200 import _lib
        from cute_rs_b200.sharded import PeerBuffer, RowShardedGemm, launch_replicated_fused, launch_replicated_p2p
        _lib.init(rank)
        rng = np.random.default_rng(4)
        a = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (m, k)).astype(np.float32))
        b = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (n, k)).astype(np.float32))
        want = oracle.gemm_tn(a, b, oracle.BF16)
        plan = RowShardedGemm(m, n, k, _lib.BF16, _lib.F32, world, rank)
        lo, hi = plan.row_begin, plan.row_begin + plan.rows
        dA = torch.from_numpy(a[lo:hi].view(np.int16).copy()).cuda()
        dB = torch.from_numpy(b.view(np.int16)).cuda()
        # peer copies
        peer_c = PeerBuffer(m * n * 4, world, rank)
        full = peer_c.tensor((m, n), torch.float32)
        full.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):
            launch_replicated_p2p(plan, dA.data_ptr(), dB.data_ptr(), peer_c, 4, panels=3)
        assert np.array_equal(full.cpu().numpy(), want)
        # the GEMM kernel's own epilogue stores into every peer's C
        for tile_m, regs, how in ((0, False, "signal"), (128, False, "signal"), (0, True, "signal"), (64, False, "signal"),
                                  (0, False, "all_reduce"), (0, False, "signal")):
            full.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            launch_replicated_fused(plan, dA.data_ptr(), dB.data_ptr(), peer_c, 4, tile_m=tile_m, register_stores=regs, barrier=how)
            assert np.array_equal(full.cpu().numpy(), want), (tile_m, regs, how)
        peer_c.close()
        # NCCL send/recv per panel
        full2 = torch.zeros(m, n, device="cuda")
        plan.launch_replicated(dA.data_ptr(), dB.data_ptr(), full2, panels=3)
        torch.cuda.synchronize()
        assert np.array_equal(full2.cpu().numpy(), want)
        assert _lib.device_status() == (0, 0, 0, 0)
    finally:
        dist.destroy_process_group()


def _worker_ragged(rank, world, port):
    """Uneven row blocks (1000 rows: 512 + 488), a bf16 C whose pitch only the register stores can
    take (260 columns), and a problem with fewer 128-row tiles than ranks (100 rows: rank 1 has none)."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cute_rs_b200 import _lib
        from cute_rs_b200.sharded import PeerBuffer, RowShardedGemm, launch_replicated_fused, launch_replicated_p2p
        _lib.init(rank)
        for m, n, k, cdt, tdt, npdt in ((1000, 264, 136, _lib.F32, torch.float32, np.float32),
                                        (1000, 260, 72, _lib.BF16, torch.bfloat16, np.uint16),
                                        (100, 136, 64, _lib.F32, torch.float32, np.float32)):
            rng = np.random.default_rng(m + n)
            a = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (m, k)).astype(np.float32))
            b = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (n, k)).astype(np.float32))
            want = oracle.gemm_tn(a, b, oracle.BF16, cdt)
            plan = RowShardedGemm(m, n, k, _lib.BF16, cdt, world, rank)
            lo, hi = plan.row_begin, plan.row_begin + plan.rows
            dA = torch.from_numpy(np.ascontiguousarray(a[lo:hi]).view(np.int16).copy()).cuda() if plan.rows else torch.zeros(8, dtype=torch.int16, device="cuda")
            dB = torch.from_numpy(b.view(np.int16)).cuda()
            c_elem = 4 if cdt == _lib.F32 else 2
            peer_c = PeerBuffer(m * n * c_elem, world, rank)
            full = peer_c.tensor((m, n), tdt)
            for launch in (lambda: launch_replicated_fused(plan, dA.data_ptr(), dB.data_ptr(), peer_c, c_elem),
                           lambda: launch_replicated_p2p(plan, dA.data_ptr(), dB.data_ptr(), peer_c, c_elem, panels=3)):
                full.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                launch()
                got = full.view(torch.int16).cpu().numpy().view(np.uint16) if cdt == _lib.BF16 else full.cpu().numpy()
                assert np.array_equal(got, want), (m, n, k, cdt)
            peer_c.close()
        assert _lib.device_status() == (0, 0, 0, 0)
    finally:
        dist.destroy_process_group()


def _worker_missing_signal(rank, world, port):
    """A peer whose completion count never arrives: in the second step rank 1 launches nothing, so
    rank 0's wait for rank 1's counter runs out after its (short) limit; the wait kernel returns,
    the host reads the report, nothing hangs or faults, and after the counters are reset the next
    step delivers the right C to both ranks.  NVLS is off and the kernels use plain peer stores."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cute_rs_b200 import _lib
        from cute_rs_b200.sharded import PeerBuffer, RowShardedGemm, launch_replicated_fused
        _lib.init(rank)
        m, n, k = 1024, 384, 256
        rng = np.random.default_rng(9)
        a = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (m, k)).astype(np.float32))
        b = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (n, k)).astype(np.float32))
        want = oracle.gemm_tn(a, b, oracle.BF16)
        plan = RowShardedGemm(m, n, k, _lib.BF16, _lib.F32, world, rank)
        dA = torch.from_numpy(a[plan.row_begin:plan.row_begin + plan.rows].view(np.int16).copy()).cuda()
        dB = torch.from_numpy(b.view(np.int16)).cuda()
        peer_c = PeerBuffer(m * n * 4, world, rank)
        full = peer_c.tensor((m, n), torch.float32)
        full.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        launch_replicated_fused(plan, dA.data_ptr(), dB.data_ptr(), peer_c, 4, timeout_ms=5000)
        assert _lib.device_status() == (0, 0, 0, 0) and np.array_equal(full.cpu().numpy(), want)
        dist.barrier()
        # step 2: rank 1 stays silent
        if rank == 0:
            launch_replicated_fused(plan, dA.data_ptr(), dB.data_ptr(), peer_c, 4, timeout_ms=300)
            assert _lib.device_status() == (7, 2, 1, 1)  # waited for count 2 of counter 1 (rank 1's), which held 1
            assert _lib.device_status() == (0, 0, 0, 0)
        dist.barrier()
        peer_c.reset_signals()
        full.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        launch_replicated_fused(plan, dA.data_ptr(), dB.data_ptr(), peer_c, 4, timeout_ms=5000)
        assert _lib.device_status() == (0, 0, 0, 0) and np.array_equal(full.cpu().numpy(), want)
        peer_c.close()
    finally:
        dist.destroy_process_group()


def test_two_gpus_missing_signal_times_out_and_recovers(lib):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker_missing_signal, args=(2, _free_port()), nprocs=2, join=True)


def test_two_gpus_replicated_c(lib):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), 1024, 384, 256), nprocs=2, join=True)


def test_two_gpus_ragged_blocks(lib):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker_ragged, args=(2, _free_port()), nprocs=2, join=True)
