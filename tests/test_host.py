"""Host-side logic that needs no GPU: the C ABI loads and exports every symbol
the header declares, the mirrored builder / argument types behave like the
reference's, and compute entry points fail loudly without a device."""
import os
import re

import numpy as np
import pytest

from cute_rs_b200 import examples as ex
from cute_rs_b200.host import (CudaContext, CudaError, DType, Kernel, KernelArg, LaunchConfig, Layout, bf16_bits_to_f32,
                               f32_to_bf16_bits, f32_to_f16_bits, param_tensor)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "cute_b200.h")).read()
    declared = set(re.findall(r"\b(cute_b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(lib.EXPORTS)
    L = lib.load()
    for name in declared:
        assert hasattr(L, name), name


def test_status_strings(lib):
    assert lib.status_string(0) == "CUTE_B200_OK"
    assert lib.status_string(lib.ERR_DEVICE_TIMEOUT) == "CUTE_B200_ERR_DEVICE_TIMEOUT"
    assert lib.status_string(12345) == "CUTE_B200_ERR_UNKNOWN"


def test_shard_rows_partitions_whole_tiles(lib):
    for m, world in [(32768, 8), (32768, 1), (8192, 4), (1000, 3), (128, 4), (0, 2), (129, 2)]:
        spans = [lib.shard_rows(m, world, r) for r in range(world)]
        pos = 0
        for begin, rows in spans:
            assert begin == pos and rows >= 0
            pos += rows
        assert pos == m
        for begin, rows in spans[:-1]:
            assert rows % 128 == 0 or begin + rows == m
    with pytest.raises(lib.CuteB200Error):
        lib.shard_rows(128, 2, 2)


def test_no_cpu_fallback_without_a_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(lib.CuteB200Error) as e:
        lib.elementwise_add_f32(16, 16, 16, 4)
    assert e.value.status == lib.ERR_NO_DEVICE
    with pytest.raises(CudaError):
        CudaContext.new(0)


def test_sharded_launcher_checks_its_arguments_without_a_device(lib):
    import ctypes
    with pytest.raises(lib.CuteB200Error) as e:
        lib.comm_create([])
    assert e.value.status == lib.ERR_INVALID_ARGUMENT and "1 to 8 GPUs" in e.value.message
    with pytest.raises(lib.CuteB200Error) as e:
        lib.comm_create(list(range(9)))
    assert e.value.status == lib.ERR_INVALID_ARGUMENT
    assert lib.load().cute_b200_comm_create(1, None, None) == lib.ERR_NULL_POINTER
    lib.comm_destroy(None)  # destroying nothing is fine
    junk = ctypes.create_string_buffer(512)
    d = lib.gemm_desc(256, 128, 64, lib.BF16, lib.F32)
    for call in (lambda: lib.comm_destroy(ctypes.addressof(junk)), lambda: lib.comm_info(ctypes.addressof(junk)),
                 lambda: lib.gemm_tn_sharded(ctypes.addressof(junk), d, [1], [1], [1]),
                 lambda: lib.gemm_tn_sharded_host(ctypes.addressof(junk), d, 1, 1, 1)):
        with pytest.raises(lib.CuteB200Error) as e:
            call()
        assert e.value.status == lib.ERR_INVALID_ARGUMENT and "not a communicator" in e.value.message
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(lib.CuteB200Error) as e:
            lib.comm_create([0])
        assert e.value.status == lib.ERR_NO_DEVICE


def test_tiling_choices_for_the_benchmark_shapes(lib):
    """The cost model's picks for the configurations of the runtime_gemm sweep, pinned: each was
    measured to be the fastest tiling for its shape (a change of the model that moves one of them has
    to be deliberate)."""
    plan = lambda m, n, k, **kw: lib.gemm_plan(lib.gemm_desc(m, n, k, lib.BF16, lib.BF16, **kw))
    assert plan(8192, 8192, 8192) == (2, 256, 256, 1)          # the 512 x 256 pair tile
    assert plan(32768, 32768, 8192) == (2, 256, 256, 1)
    assert plan(4096, 32768, 8192) == (2, 256, 256, 1)         # one rank's block of the sharded workload
    assert plan(4096, 4096, 4096) == (2, 256, 256, 1)
    assert plan(16384, 1024, 8192) == (2, 256, 256, 1)
    assert plan(2048, 2048, 2048) == (1, 256, 128, 1)          # one wave of single CTAs
    assert plan(1024, 1024, 1024) == (1, 128, 128, 1)
    assert plan(8192, 128, 8192) == (1, 128, 128, 2)           # few row tiles, long k: k cut in two, summed inside a cluster
    assert plan(8192, 256, 8192) == (1, 256, 128, 2)
    assert plan(1536, 1536, 2048) == (1, 128, 128, 1)          # short k: the exchange would cost more than it saves
    desc = lib.gemm_desc(8192, 128, 8192, lib.BF16, lib.BF16)
    desc.tuning[0] = 128                                       # without the in-cluster form: the 64-row pair tile, one kernel
    assert lib.gemm_plan(desc) == (2, 128, 64, 1)
    assert plan(8192, 128, 8192, split_k=4)[3] == 4 and plan(8192, 128, 64, split_k=4)[3] == 1  # honoured, cut to the k blocks
    assert plan(256, 256, 256, tile_m=64)[:3] == (2, 128, 64) or plan(256, 256, 256, tile_m=64)[0] == 2


def test_argument_checks_come_before_the_device(lib):
    # check_launch runs before any CUDA call (src/cuda.rs:452), so its
    # messages can be compared without a GPU.
    a = lib.Arg(0, lib.F32, 0, 16)
    cases = [
        (("elementwise_add_tiled", [1, 1, 1], [128, 1, 1], [a, a]), "kernel `elementwise_add_tiled` takes 3 arguments, 2 were given"),
        (("elementwise_add_tiled", [1, 1, 1], [2048, 1, 1], [a, a, a]), "invalid block size [2048, 1, 1]"),
        (("elementwise_add_tiled", [0, 1, 1], [128, 1, 1], [a, a, a]), "invalid grid size [0, 1, 1]"),
        (("elementwise_add_tiled", [3, 1, 1], [128, 1, 1], [a, a, a], (2, 1, 1)),
         "grid [3, 1, 1] is not a whole number of clusters of [2, 1, 1]"),
        (("elementwise_add_tiled", [1, 1, 1], [256, 1, 1], [a, a, a]),
         "kernel `elementwise_add_tiled` was built for blocks of [128, 1, 1], launched with [256, 1, 1]"),
        (("sgemm_nt", [1, 1, 1], [256, 1, 1], [a, a, lib.Arg(0, lib.F16, 0, 16), a, a]),
         "argument 2 (`c`) must be a f32 buffer, got an f16 buffer of 16"),
        (("runtime_gemm", [1, 1, 1], [128, 1, 1],
          [lib.Arg(0, lib.F16, 0, 1), lib.Arg(0, lib.F16, 0, 1), a, lib.Arg(1, lib.I32, 128, 0), lib.Arg(1, lib.I32, 40, 0)]),
         "argument 4 (`k`) must be a multiple of 32, got 40"),
        (("runtime_gemm", [1, 1, 1], [128, 1, 1],
          [lib.Arg(0, lib.F16, 0, 1), lib.Arg(0, lib.F16, 0, 1), a, lib.Arg(1, lib.F32, 128, 0), lib.Arg(1, lib.I32, 32, 0)]),
         "argument 3 (`n`) must be a i32 scalar, got an f32 scalar"),
    ]
    for call, message in cases:
        with pytest.raises(lib.CuteB200Error) as e:
            lib.launch(*call)
        assert e.value.status == lib.ERR_INVALID_ARGUMENT and e.value.message == message
    with pytest.raises(lib.CuteB200Error) as e:
        lib.launch("single_warp_pipeline", [1, 1, 1], [32, 1, 1], [])
    assert e.value.status == lib.ERR_UNSUPPORTED


def test_builder_records_parameters_in_order():
    k = ex.tensorop_gemm(ex.GemmConfig.new(256, 128, 96))
    assert k.name() == "tensorop_gemm" and k.block_dim == (128, 1, 1)
    assert [(p.name, p.dtype, p.length) for p in k.params] == [("a", DType.F16, 256 * 96), ("b", DType.F16, 128 * 96),
                                                                 ("c", DType.F32, 256 * 128)]
    assert ex.tensorop_gemm(ex.GemmConfig(256, 128, 96, ab=DType.BF16, swizzle=False)).name() == "tensorop_gemm_bf16_unswizzled"
    r = ex.runtime_gemm()
    assert [(p.name, p.is_scalar, p.multiple_of) for p in r.params][3:] == [("n", True, 128), ("k", True, 32)]
    assert [p.name for p in ex.sgemm(128, 128, 8).params] == ["a", "b", "c", "alpha", "beta"]
    with pytest.raises(ValueError, match="multiple of the tile size"):
        ex.tensorop_gemm(ex.GemmConfig.new(100, 128, 32))
    with pytest.raises(RuntimeError):
        param_tensor(DType.F32, "x", Layout.row_major((4, 4)))  # outside a build
    with pytest.raises(ValueError, match="duplicate"):
        Kernel.builder("k").build(lambda: [param_tensor(DType.F32, "x", Layout.row_major((4,))) for _ in range(2)])


def test_layout_cosize():
    assert Layout.row_major((300, 512)).cosize() == 300 * 512
    assert Layout.col_major((128, 8)).stride == (1, 128)
    assert Layout((4, 4), (1, 8)).cosize() == 1 + 3 + 24


def test_kernel_arg_types_and_conversions(golden):
    x = golden["conv_in"]
    assert np.array_equal(f32_to_f16_bits(x), golden["conv_f16_bits"])
    assert np.array_equal(f32_to_bf16_bits(x), golden["conv_bf16_bits"])
    nan = np.array([np.nan], np.float32)
    assert f32_to_bf16_bits(nan)[0] == (nan.view(np.uint32)[0] >> 16) | 0x40
    a = KernelArg.f16_from_f32([1.0, 2.5])
    assert a.describe() == "an f16 buffer of 2" and np.array_equal(a.to_f32(), [1.0, 2.5])
    assert KernelArg.ScalarI32(7).describe() == "an i32 scalar" and KernelArg.ScalarF32(1.5).scalar_bits() == 0x3FC00000
    with pytest.raises(TypeError, match="not an f32 buffer"):
        a.as_f32()
    assert np.array_equal(bf16_bits_to_f32(KernelArg.bf16_from_f32([0.02]).data), [np.float32(0.02001953125)])
    cfg = LaunchConfig.new([4, 2, 1], [128, 1, 1]).with_cluster([2, 1, 1])
    assert cfg.cluster == (2, 1, 1) and cfg.threads_per_block() == 128


def test_example_problems_use_the_reference_formulas(golden):
    launch, args, a, b = ex.tensorop_gemm_problem(ex.GemmConfig.new(128, 128, 64))
    assert launch.grid == (1, 1, 1) and launch.block == (128, 1, 1)
    want = (a.reshape(128, 64).astype(np.int64) @ b.reshape(128, 64).astype(np.int64).T)
    assert np.array_equal(want, golden["tensorop_int_128x128x64"])
    assert ex.naive_grid() == [600, 1, 1] and ex.tiled_grid() == [19, 4, 1]
