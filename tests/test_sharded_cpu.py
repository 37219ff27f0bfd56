"""The N > 1 host logic on CPU: two gloo ranks partition the rows with the
library's own rule, each produces its block (with the oracle standing in for
the GPU kernel, which cannot run here) and the gather reassembles C."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cute_rs_b200 import _lib
        from cute_rs_b200.sharded import RowShardedGemm
        rng = np.random.default_rng(4)
        a = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (m, k)).astype(np.float32))
        b = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32))
        plan = RowShardedGemm(m, n, k, _lib.BF16, _lib.F32, world, rank)
        lo, hi = plan.row_begin, plan.row_begin + plan.rows
        block = oracle.gemm_tn(a[lo:hi], b, oracle.BF16) if plan.rows else np.zeros((0, n), np.float32)
        full = torch.zeros(m, n)
        plan.all_gather(torch.from_numpy(block), full)
        want = oracle.gemm_tn(a, b, oracle.BF16)
        assert np.array_equal(full.numpy(), want)
        np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([lo, hi]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [512, 640, 100])
def test_two_ranks_partition_and_gather(tmp_path, m):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), m, 96, 64, str(tmp_path)), nprocs=world, join=True)
    spans = [np.load(tmp_path / f"ok{r}.npy") for r in range(world)]
    assert spans[0][0] == 0 and spans[0][1] == spans[1][0] and spans[1][1] == m


def _worker_overlap(rank, world, port, m, n, k, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cute_rs_b200 import _lib
        from cute_rs_b200.sharded import RowShardedGemm
        rng = np.random.default_rng(4)
        a = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (m, k)).astype(np.float32))
        b = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32))
        plan = RowShardedGemm(m, n, k, _lib.BF16, _lib.F32, world, rank)
        full = torch.zeros(m, n)

        def compute_panel(r0, rows):  # the oracle stands in for the GPU kernel
            lo = plan.row_begin + r0
            full[lo:lo + rows] = torch.from_numpy(oracle.gemm_tn(a[lo:lo + rows], b, oracle.BF16))

        plan.launch_replicated(0, 0, full, panels=3, compute_panel=compute_panel)
        assert np.array_equal(full.numpy(), oracle.gemm_tn(a, b, oracle.BF16))
        assert sum(r for _, r in plan.panels(3)) == plan.rows
        np.save(os.path.join(out_dir, f"ov{rank}.npy"), np.array([1]))
    finally:
        dist.destroy_process_group()


def test_panels_of_a_rank_without_rows():
    from cute_rs_b200 import _lib
    from cute_rs_b200.sharded import RowShardedGemm
    assert RowShardedGemm(100, 96, 64, _lib.BF16, _lib.F32, 2, 1).panels(8) == []
    assert RowShardedGemm(100, 96, 64, _lib.BF16, _lib.F32, 2, 0).panels(8) == [(0, 100)]
    assert RowShardedGemm(1024, 96, 64, _lib.BF16, _lib.F32, 2, 1).panels(3) == [(0, 256), (256, 256)]


@pytest.mark.parametrize("m", [1024, 640, 100])
def test_two_ranks_replicate_with_overlapped_panels(tmp_path, m):
    """Even split (1024): panel-by-panel exchange; ragged split (640) and a rank without rows (100): one gather."""
    mp.spawn(_worker_overlap, args=(2, _free_port(), m, 96, 64, str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"ov{r}.npy").exists() for r in range(2))
