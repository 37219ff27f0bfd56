"""The reference's example kernels, declared through the mirrored builder.

Each function returns a ``Kernel`` with the name, block size and parameter
list of the reference example of the same name; the body that runs is the
sm_100a kernel of that name inside libcute_b200.so.  The ``problem``/``inputs``
helpers reproduce the examples' own integer-valued test inputs, whose results
are exact in f32.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .host import (DType, Kernel, KernelArg, LaunchConfig, Layout, param_extent, param_ptr, param_scalar,
                   param_tensor)


@dataclass
class GemmConfig:
    """examples/tensorop_gemm.rs:22-40.  bm/bn/bk/stages/swizzle describe the
    reference's mma.sync kernel and only select the kernel NAME here; the
    sm_100a kernel picks its own tiling."""
    m: int
    n: int
    k: int
    bm: int = 128
    bn: int = 128
    bk: int = 32
    stages: int = 3
    swizzle: bool = True
    ab: DType = DType.F16

    @staticmethod
    def new(m: int, n: int, k: int) -> "GemmConfig":
        return GemmConfig(m, n, k)


def tensorop_gemm(cfg: GemmConfig) -> Kernel:
    """tensorop_gemm::build (examples/tensorop_gemm.rs:42-164)."""
    if cfg.ab not in (DType.F16, DType.BF16):
        raise ValueError(f"tensorop_gemm takes f16 or bf16 inputs, not {cfg.ab}")
    if cfg.m % cfg.bm or cfg.n % cfg.bn or cfg.k % cfg.bk:
        raise ValueError("problem size must be a multiple of the tile size")
    if cfg.bk != 32:
        raise ValueError("the shared-memory swizzle atom below assumes BK = 32")
    name = {(True, DType.F16): "tensorop_gemm", (False, DType.F16): "tensorop_gemm_unswizzled",
            (True, DType.BF16): "tensorop_gemm_bf16", (False, DType.BF16): "tensorop_gemm_bf16_unswizzled"}[
        (cfg.swizzle, cfg.ab)]

    def body():
        param_tensor(cfg.ab, "a", Layout.row_major((cfg.m, cfg.k)))
        param_tensor(cfg.ab, "b", Layout.row_major((cfg.n, cfg.k)))
        param_tensor(DType.F32, "c", Layout.row_major((cfg.m, cfg.n)))

    return Kernel.builder(name).block_dim([128, 1, 1]).build(body)


def tensorop_gemm_problem(cfg: GemmConfig):
    """Inputs and launch of tensorop_gemm::run (examples/tensorop_gemm.rs:167-178)."""
    a = ((np.arange(cfg.m * cfg.k, dtype=np.int64) * 7 + 3) % 7 - 3).astype(np.float32)
    b = ((np.arange(cfg.n * cfg.k, dtype=np.int64) * 5 + 1) % 5 - 2).astype(np.float32)
    conv = KernelArg.bf16_from_f32 if cfg.ab == DType.BF16 else KernelArg.f16_from_f32
    args = [conv(a), conv(b), KernelArg.f32(np.zeros(cfg.m * cfg.n, np.float32))]
    launch = LaunchConfig.new([cfg.m // cfg.bm, cfg.n // cfg.bn, 1], [128, 1, 1])
    return launch, args, a, b


def runtime_gemm() -> Kernel:
    """runtime_gemm::build (examples/runtime_gemm.rs:22-33): sizes at launch."""
    def body():
        param_ptr(DType.F16, "a")
        param_ptr(DType.F16, "b")
        param_ptr(DType.F32, "c")
        param_extent("n", 128)
        param_extent("k", 32)

    return Kernel.builder("runtime_gemm").block_dim([128, 1, 1]).build(body)


def runtime_gemm_problem(m: int, n: int, k: int):
    """runtime_gemm::problem (examples/runtime_gemm.rs:107-121)."""
    if m % 128 or n % 128 or k % 32:
        raise ValueError("size must be a tile multiple")
    a = ((np.arange(m * k, dtype=np.int64) * 7 + 3) % 7 - 3).astype(np.float32)
    b = ((np.arange(n * k, dtype=np.int64) * 5 + 1) % 5 - 2).astype(np.float32)
    args = [KernelArg.f16_from_f32(a), KernelArg.f16_from_f32(b), KernelArg.f32(np.zeros(m * n, np.float32)),
            KernelArg.ScalarI32(n), KernelArg.ScalarI32(k)]
    return LaunchConfig.new([m // 128, n // 128, 1], [128, 1, 1]), args, a, b


def sgemm(m: int, n: int, k: int) -> Kernel:
    """sgemm::build (examples/sgemm.rs:23-33)."""
    if m % 128 or n % 128 or k % 8:
        raise ValueError("problem size must be a multiple of the tile size")

    def body():
        param_tensor(DType.F32, "a", Layout.col_major((m, k)))
        param_tensor(DType.F32, "b", Layout.col_major((n, k)))
        param_tensor(DType.F32, "c", Layout.col_major((m, n)))
        param_scalar(DType.F32, "alpha")
        param_scalar(DType.F32, "beta")

    return Kernel.builder("sgemm_nt").block_dim([256, 1, 1]).build(body)


def sgemm_problem(m: int, n: int, k: int):
    """Inputs and launch of sgemm::run (examples/sgemm.rs:84-99)."""
    a = ((np.arange(m * k, dtype=np.int64) * 7) % 11 - 5).astype(np.float32)
    b = ((np.arange(n * k, dtype=np.int64) * 3) % 13 - 6).astype(np.float32)
    c0 = (np.arange(m * n, dtype=np.int64) % 5).astype(np.float32)
    alpha, beta = 1.5, -0.5
    args = [KernelArg.f32(a), KernelArg.f32(b), KernelArg.f32(c0), KernelArg.ScalarF32(alpha),
            KernelArg.ScalarF32(beta)]
    return LaunchConfig.new([m // 128, n // 128, 1], [256, 1, 1]), args, a, b, c0, alpha, beta


def elementwise_add_naive(m: int = 300, n: int = 512) -> Kernel:
    """elementwise_add::naive (examples/elementwise_add.rs:23-35)."""
    def body():
        for name in ("a", "b", "c"):
            param_tensor(DType.F32, name, Layout.row_major((m, n)))

    return Kernel.builder("elementwise_add_naive").block_dim([256, 1, 1]).build(body)


def elementwise_add_tiled(m: int = 300, n: int = 512) -> Kernel:
    """elementwise_add::tiled (examples/elementwise_add.rs:37-80)."""
    def body():
        for name in ("a", "b", "c"):
            param_tensor(DType.F32, name, Layout.row_major((m, n)))

    return Kernel.builder("elementwise_add_tiled").block_dim([128, 1, 1]).build(body)


def elementwise_add_problem(m: int = 300, n: int = 512):
    """Inputs of elementwise_add::run (examples/elementwise_add.rs:82-86)."""
    i = np.arange(m * n, dtype=np.int64)
    a = ((i % 97).astype(np.float32) * np.float32(0.5))
    b = ((i % 13).astype(np.float32) - np.float32(6.0))
    return [KernelArg.f32(a), KernelArg.f32(b), KernelArg.f32(np.zeros(m * n, np.float32))], a, b


def naive_grid(m: int = 300, n: int = 512):
    return [-(-(m * n) // 256), 1, 1]


def tiled_grid(m: int = 300, n: int = 512):
    return [-(-m // 16), -(-n // 128), 1]
