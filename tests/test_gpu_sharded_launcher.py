"""The single-process launcher for several GPUs (cute_b200_comm_create /
cute_b200_gemm_tn_sharded / cute_b200_gemm_tn_sharded_host) against the oracle.

A device may be named more than once in a communicator, so the partition, the
fused replication (the GEMM kernel's pusher stores into the other blocks' C),
the copy fallback and the host-buffer pipeline are all exercised on a box with a
single GPU; with two or more GPUs the same cases also run over real peers and
through the collective library.
"""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _device_sets():
    import torch
    sets = [[0], [0, 0], [0, 0, 0]]
    if torch.cuda.device_count() >= 2:
        sets += [[0, 1], [1, 0, 1]]
    return sets


def _upload(arr, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.int16 if arr.dtype == np.uint16 else arr.dtype)).to(f"cuda:{device}")


def _case(m, n, k, seed, cdt_bf16):
    rng = np.random.default_rng(seed)
    a = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (m, k)).astype(np.float32))
    b = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (n, k)).astype(np.float32))
    want = oracle.gemm_tn(a, b, oracle.BF16, oracle.BF16 if cdt_bf16 else oracle.F32)
    return a, b, want


@pytest.mark.parametrize("m,n,k,cdt_bf16", [(1024, 384, 256, False), (1000, 264, 136, False), (1000, 260, 72, True), (100, 136, 64, False),
                                            (2048, 512, 512, True)])
def test_sharded_gemm_on_device_buffers(lib, gpu, m, n, k, cdt_bf16):
    import torch
    a, b, want = _case(m, n, k, m + n, cdt_bf16)
    cdt, tdt = (lib.BF16, torch.bfloat16) if cdt_bf16 else (lib.F32, torch.float32)
    desc = lib.gemm_desc(m, n, k, lib.BF16, cdt)
    for devices in _device_sets():
        world = len(devices)
        comm = lib.comm_create(devices)
        try:
            info = lib.comm_info(comm)
            assert info["ngpus"] == world and info["distinct"] == (len(set(devices)) == world)
            spans = [lib.shard_rows(m, world, g) for g in range(world)]
            dA = [_upload(a[lo:lo + rows] if rows else a[:1], dev) for (lo, rows), dev in zip(spans, devices)]
            dB = [_upload(b, dev) for dev in devices]
            # every GPU keeps its own block
            blocks = [torch.zeros(max(rows, 1), n, dtype=tdt, device=f"cuda:{dev}") for (_, rows), dev in zip(spans, devices)]
            lib.gemm_tn_sharded(comm, desc, [t.data_ptr() for t in dA], [t.data_ptr() for t in dB], [t.data_ptr() for t in blocks],
                                lib.REPLICATE_NONE)
            for (lo, rows), blk in zip(spans, blocks):
                got = blk[:rows].cpu().view(torch.int16).numpy().view(np.uint16) if cdt_bf16 else blk[:rows].cpu().numpy()
                assert np.array_equal(got, want[lo:lo + rows]), (devices, "blocks")
            # every GPU ends up with all of C, each way the launcher knows
            modes = [lib.REPLICATE_AUTO, lib.REPLICATE_FUSED, lib.REPLICATE_COPIES]
            if info["collective_library"] and world > 1:
                modes.append(lib.REPLICATE_COLLECTIVE)
            for mode in modes:
                fulls = [torch.zeros(m, n, dtype=tdt, device=f"cuda:{dev}") for dev in devices]
                lib.gemm_tn_sharded(comm, desc, [t.data_ptr() for t in dA], [t.data_ptr() for t in dB], [t.data_ptr() for t in fulls], mode)
                for full in fulls:
                    got = full.cpu().view(torch.int16).numpy().view(np.uint16) if cdt_bf16 else full.cpu().numpy()
                    assert np.array_equal(got, want), (devices, mode)
            for dev in set(devices):
                torch.cuda.set_device(dev)
                assert lib.device_status() == (0, 0, 0, 0)
        finally:
            torch.cuda.set_device(0)
            lib.comm_destroy(comm)


@pytest.mark.parametrize("m,n,k,cdt_bf16,alpha,beta", [(1024, 640, 256, True, 1.0, 0.0), (1000, 264, 136, False, 1.0, 0.0),
                                                       (100, 136, 64, False, 1.5, -0.5), (4096, 1024, 512, True, 1.0, 0.0),
                                                       (300, 200, 0, False, 2.0, 0.5),
                                                       # 8192 columns and more: C goes in blocks of columns, B up block by block
                                                       (700, 8448, 128, True, 1.0, 0.0), (520, 8200, 72, False, 1.5, -0.5),
                                                       (256, 16640, 64, True, 1.0, 0.0)])
def test_sharded_gemm_on_host_buffers(lib, gpu, m, n, k, cdt_bf16, alpha, beta):
    """Whole matrices in host memory: every GPU uploads its rows of A and its share of B,
    the shares are passed around, C comes back block by block (panels of rows, and from 8192 columns on
    also blocks of columns)."""
    import torch
    rng = np.random.default_rng(m * 3 + n)
    a = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (m, k)).astype(np.float32))
    b = oracle.f32_to_bf16_bits(rng.integers(-8, 9, (n, k)).astype(np.float32))
    c0f = rng.integers(-8, 9, (m, n)).astype(np.float32)
    c0 = oracle.f32_to_bf16_bits(c0f) if cdt_bf16 else c0f
    ocdt = oracle.BF16 if cdt_bf16 else oracle.F32
    want = oracle.gemm_tn(a, b, oracle.BF16, ocdt, alpha, beta, c_init=c0)
    desc = lib.gemm_desc(m, n, k, lib.BF16, lib.BF16 if cdt_bf16 else lib.F32, alpha, beta)
    for devices in _device_sets():
        comm = lib.comm_create(devices)
        try:
            for _ in range(2):  # the second call reuses the communicator's staging memory
                hc = c0.copy()
                sec = lib.gemm_tn_sharded_host(comm, desc, a.ctypes.data if k else 0, b.ctypes.data if k else 0, hc.ctypes.data)
                assert sec > 0 and np.array_equal(hc, want), devices
        finally:
            torch.cuda.set_device(0)
            lib.comm_destroy(comm)


def test_sharded_launcher_rejects_bad_arguments(lib, gpu):
    import torch
    with pytest.raises(lib.CuteB200Error) as e:
        lib.comm_create([])
    assert e.value.status == lib.ERR_INVALID_ARGUMENT
    with pytest.raises(lib.CuteB200Error) as e:
        lib.comm_create([torch.cuda.device_count()])
    assert e.value.status == lib.ERR_NO_DEVICE and "requested" in e.value.message
    comm = lib.comm_create([0, 0])
    try:
        d = lib.gemm_desc(256, 128, 64, lib.BF16, lib.F32, 2.0, 0.0)
        buf = torch.zeros(1 << 16, device="cuda")
        p = [buf.data_ptr()] * 2
        with pytest.raises(lib.CuteB200Error) as e:  # the fused form needs the plain epilogue
            lib.gemm_tn_sharded(comm, d, p, p, p, lib.REPLICATE_FUSED)
        assert e.value.status == lib.ERR_INVALID_ARGUMENT and "alpha = 1" in e.value.message
        with pytest.raises(lib.CuteB200Error) as e:
            lib.gemm_tn_sharded(comm, lib.gemm_desc(256, 128, 64, lib.BF16, lib.F32), p, p, [buf.data_ptr(), 0], lib.REPLICATE_NONE)
        assert e.value.status == lib.ERR_NULL_POINTER and "GPU 1" in e.value.message
        with pytest.raises(lib.CuteB200Error) as e:
            lib.gemm_tn_sharded(comm, lib.gemm_desc(256, 128, 64, lib.BF16, lib.F32), p, p, p, 9)
        assert e.value.status == lib.ERR_INVALID_ARGUMENT
        with pytest.raises(lib.CuteB200Error) as e:  # a failure on one GPU names it: k not a multiple of 8
            lib.gemm_tn_sharded(comm, lib.gemm_desc(256, 128, 20, lib.BF16, lib.F32), p, p, p, lib.REPLICATE_NONE)
        assert e.value.status == lib.ERR_INVALID_ARGUMENT and "GPU 0 (device 0)" in e.value.message and "multiple of 8" in e.value.message
    finally:
        lib.comm_destroy(comm)
    with pytest.raises(lib.CuteB200Error):
        lib.gemm_tn_sharded(ctypes.addressof(ctypes.create_string_buffer(256)), lib.gemm_desc(256, 128, 64, lib.BF16, lib.F32), [1], [1], [1])
