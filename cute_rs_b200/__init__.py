"""cute_rs_b200: the cute-rs GEMM / elementwise hot path on B200 (sm_100a).

``_lib`` binds the C ABI of libcute_b200.so (include/cute_b200.h), ``host``
mirrors the reference crate's launch surface (Kernel.builder, param_tensor,
KernelArg, LaunchConfig, CudaContext) and ``examples`` declares the reference's
example kernels through it.  All arithmetic happens in the CUDA library.
"""
from . import _lib  # noqa: F401
from .host import (CudaContext, CudaError, DeviceArg, DeviceBuffer, DType, Kernel, KernelArg, LaunchConfig,  # noqa: F401
                   LaunchStats, Layout, param_extent, param_ptr, param_scalar, param_tensor)

__all__ = ["CudaContext", "CudaError", "DeviceArg", "DeviceBuffer", "DType", "Kernel", "KernelArg", "LaunchConfig",
           "LaunchStats", "Layout", "param_extent", "param_ptr", "param_scalar", "param_tensor"]
