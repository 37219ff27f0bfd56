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
        for tile_m, regs in ((0, False), (128, False), (0, True)):
            full.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            launch_replicated_fused(plan, dA.data_ptr(), dB.data_ptr(), peer_c, 4, tile_m=tile_m, register_stores=regs)
            assert np.array_equal(full.cpu().numpy(), want)
        peer_c.close()
        # NCCL send/recv per panel
        full2 = torch.zeros(m, n, device="cuda")
        plan.launch_replicated(dA.data_ptr(), dB.data_ptr(), full2, panels=3)
        torch.cuda.synchronize()
        assert np.array_equal(full2.cpu().numpy(), want)
        assert _lib.device_status() == (0, 0, 0, 0)
    finally:
        dist.destroy_process_group()


def test_two_gpus_replicated_c(lib):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), 1024, 384, 256), nprocs=2, join=True)
