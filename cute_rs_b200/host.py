"""Host-side mirror of the cute-rs launch surface for the hot-path kernels.

Same names, argument meaning and error behaviour as the reference crate:

* ``Kernel.builder(name).block_dim([..]).build(closure)`` with ``param_tensor``,
  ``param_ptr``, ``param_extent`` and ``param_scalar`` called inside the closure
  in declaration order (src/builder.rs:747-824, src/tensor.rs:401-431, 526-539);
* ``KernelArg`` / ``LaunchConfig`` (src/sim/mod.rs:41-216);
* ``CudaContext`` with ``upload`` / ``download`` / ``launch`` /
  ``launch_on_device`` / ``synchronize`` and ``Kernel.run_cuda``
  (src/cuda.rs:204-488, 570-593).

Only the launch path is mirrored.  The closure declares the kernel's
parameters; the kernel body is the hand-written sm_100a code behind
libcute_b200.so, selected by the kernel's name.  There is no CPU path here:
``Kernel.simulate`` is the reference's CPU interpreter and has no counterpart
in this package.
"""
from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Optional, Sequence

import numpy as np

from . import _lib


class DType(Enum):
    F16 = _lib.F16
    BF16 = _lib.BF16
    F32 = _lib.F32
    I32 = _lib.I32

    def bytes(self) -> int:
        return 2 if self in (DType.F16, DType.BF16) else 4

    def __str__(self) -> str:
        return self.name.lower()


_NP = {DType.F16: np.uint16, DType.BF16: np.uint16, DType.F32: np.float32, DType.I32: np.int32}


def f32_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns; a NaN keeps its high
    half and gains the quiet bit (BF16::from_f32, src/value.rs:92-99)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    high = (bits >> 16).astype(np.uint32)
    low = bits & np.uint32(0xFFFF)
    up = (low > 0x8000) | ((low == 0x8000) & ((high & 1) == 1))
    out = np.where(np.isnan(np.asarray(x, dtype=np.float32)), high | 0x40, high + up.astype(np.uint32))
    return out.astype(np.uint16)


def bf16_bits_to_f32(h) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> f16 bit patterns (F16::from_f32,
    src/value.rs:101-134); numpy's conversion implements the same IEEE rule."""
    with np.errstate(over="ignore"):
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(h) -> np.ndarray:
    return np.ascontiguousarray(h, dtype=np.uint16).view(np.float16).astype(np.float32)


# --------------------------------------------------------------------------- #
# Layouts: only what param_tensor needs (shape, strides, cosize).              #
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class Layout:
    shape: tuple
    stride: tuple

    @staticmethod
    def row_major(shape: Sequence[int]) -> "Layout":
        shape = tuple(int(s) for s in shape)
        stride, acc = [], 1
        for s in reversed(shape):
            stride.append(acc)
            acc *= s
        return Layout(shape, tuple(reversed(stride)))

    @staticmethod
    def col_major(shape: Sequence[int]) -> "Layout":
        shape = tuple(int(s) for s in shape)
        stride, acc = [], 1
        for s in shape:
            stride.append(acc)
            acc *= s
        return Layout(shape, tuple(stride))

    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64))

    def cosize(self) -> int:
        """One past the largest offset the layout produces."""
        if self.size() == 0:
            return 0
        return 1 + sum((s - 1) * d for s, d in zip(self.shape, self.stride))


# --------------------------------------------------------------------------- #
# Launch configuration and arguments                                           #
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class LaunchConfig:
    """Grid and block dimensions of a launch (src/sim/mod.rs:41-66)."""
    grid: tuple
    block: tuple
    cluster: tuple = (1, 1, 1)

    @staticmethod
    def new(grid, block) -> "LaunchConfig":
        return LaunchConfig(tuple(grid), tuple(block))

    def with_cluster(self, cluster) -> "LaunchConfig":
        return LaunchConfig(self.grid, self.block, tuple(cluster))

    def threads_per_block(self) -> int:
        return int(self.block[0]) * int(self.block[1]) * int(self.block[2])


class KernelArg:
    """A kernel argument: a host buffer per tensor parameter, a scalar per
    scalar parameter, in declaration order (src/sim/mod.rs:68-216)."""

    def __init__(self, dtype: DType, data: Optional[np.ndarray] = None, scalar=None):
        self.dtype = dtype
        self.data = data
        self.scalar = scalar

    # -- constructors named after the reference's ---------------------------------
    @staticmethod
    def f32(v) -> "KernelArg":
        return KernelArg(DType.F32, np.array(v, dtype=np.float32).reshape(-1))

    @staticmethod
    def f16_from_f32(v) -> "KernelArg":
        return KernelArg(DType.F16, f32_to_f16_bits(np.asarray(v, dtype=np.float32).reshape(-1)))

    @staticmethod
    def bf16_from_f32(v) -> "KernelArg":
        """KernelArg::buffer(&[BF16::from_f32(x)..]) in the reference."""
        return KernelArg(DType.BF16, f32_to_bf16_bits(np.asarray(v, dtype=np.float32).reshape(-1)))

    @staticmethod
    def i32(v) -> "KernelArg":
        return KernelArg(DType.I32, np.array(v, dtype=np.int32).reshape(-1))

    @staticmethod
    def buffer(dtype: DType, bits) -> "KernelArg":
        return KernelArg(dtype, np.array(bits, dtype=_NP[dtype]).reshape(-1))

    @staticmethod
    def ScalarF32(x: float) -> "KernelArg":
        return KernelArg(DType.F32, scalar=np.float32(x))

    @staticmethod
    def ScalarI32(x: int) -> "KernelArg":
        return KernelArg(DType.I32, scalar=np.int32(x))

    # -- accessors ---------------------------------------------------------------------
    def is_scalar(self) -> bool:
        return self.data is None

    def as_f32(self) -> np.ndarray:
        if self.is_scalar() or self.dtype != DType.F32:
            raise TypeError(f"argument is {self.describe()}, not an f32 buffer")
        return self.data

    def to_f32(self) -> np.ndarray:
        """Buffer contents widened to f32 (exact for f16 and bf16)."""
        if self.dtype == DType.F16:
            return f16_bits_to_f32(self.data)
        if self.dtype == DType.BF16:
            return bf16_bits_to_f32(self.data)
        return self.data.astype(np.float32)

    def describe(self) -> str:
        article = "an" if self.dtype in (DType.F32, DType.F16, DType.I32) else "a"
        if self.is_scalar():
            return f"{article} {self.dtype} scalar"
        return f"{article} {self.dtype} buffer of {self.data.size}"

    def scalar_bits(self) -> int:
        if self.dtype == DType.F32:
            return int(np.float32(self.scalar).view(np.uint32))
        return int(np.int32(self.scalar).view(np.uint32))

    def clone(self) -> "KernelArg":
        return KernelArg(self.dtype, None if self.data is None else self.data.copy(), self.scalar)


# --------------------------------------------------------------------------- #
# Kernel builder                                                               #
# --------------------------------------------------------------------------- #
@dataclass
class Param:
    name: str
    dtype: DType
    is_scalar: bool
    length: Optional[int] = None  # buffers: minimum element count; None for param_ptr
    multiple_of: int = 1          # scalars


_builder = threading.local()


def _declare(p: Param) -> Param:
    params = getattr(_builder, "params", None)
    if params is None:
        raise RuntimeError("kernel parameters can only be declared inside Kernel.builder(..).build(closure)")
    if any(q.name == p.name for q in params):
        raise ValueError(f"duplicate kernel parameter `{p.name}`")
    params.append(p)
    return p


def param_tensor(dtype: DType, name: str, layout: Layout) -> Param:
    """A global tensor of `layout.cosize()` elements, 16-byte aligned
    (src/tensor.rs:401-416)."""
    return _declare(Param(name, dtype, False, layout.cosize()))


def param_ptr(dtype: DType, name: str) -> Param:
    """A global pointer whose extent is only known at launch (src/tensor.rs:418-431)."""
    return _declare(Param(name, dtype, False, None))


def param_extent(name: str, multiple_of: int = 1) -> Param:
    """An i32 size passed at launch, checked to be a multiple (src/tensor.rs:526-533)."""
    return _declare(Param(name, DType.I32, True, None, int(multiple_of)))


def param_scalar(dtype: DType, name: str) -> Param:
    return _declare(Param(name, dtype, True))


class KernelOptions:
    def __init__(self, name: str):
        self._name = name
        self._block_dim = None

    def block_dim(self, dims) -> "KernelOptions":
        self._block_dim = tuple(int(d) for d in dims)
        return self

    def build(self, closure: Callable[[], None]) -> "Kernel":
        if getattr(_builder, "params", None) is not None:
            raise RuntimeError("Kernel builds cannot be nested")
        _builder.params = []
        try:
            closure()
            params = _builder.params
        finally:
            _builder.params = None
        return Kernel(self._name, self._block_dim, params)


@dataclass
class LaunchStats:
    """What the device reports about one launch (src/cuda.rs:65-69)."""
    kernel_seconds: float


class Kernel:
    def __init__(self, name: str, block_dim, params):
        self._name = name
        self.block_dim = block_dim
        self.params = params

    @staticmethod
    def builder(name: str) -> KernelOptions:
        return KernelOptions(name)

    def name(self) -> str:
        return self._name

    def run_cuda(self, ctx: "CudaContext", cfg: LaunchConfig, args: list) -> LaunchStats:
        """Upload, run, wait, download (Kernel::run_cuda, src/cuda.rs:574-592)."""
        return ctx.launch(self, cfg, args)


# --------------------------------------------------------------------------- #
# Launcher                                                                     #
# --------------------------------------------------------------------------- #
class CudaError(RuntimeError):
    def __init__(self, message: str, status: int = _lib.ERR_CUDA):
        super().__init__(f"CUDA: {message}")
        self.message = message
        self.status = status


def _wrap(fn, *a, **kw):
    try:
        return fn(*a, **kw)
    except _lib.CuteB200Error as e:
        raise CudaError(e.message, e.status) from None


class DeviceBuffer:
    """Device memory owned by the object and freed with it (src/cuda.rs:491-502)."""

    def __init__(self, ptr: int, nbytes: int, dtype: DType, length: int):
        self.ptr, self.bytes, self.dtype, self.len = ptr, nbytes, dtype, length

    def __del__(self):
        try:
            if self.ptr:
                _lib.free(self.ptr)
        except Exception:
            pass
        self.ptr = 0


@dataclass
class DeviceArg:
    """A launch argument already on the device (src/cuda.rs:505-509)."""
    buffer: Optional[DeviceBuffer] = None
    scalar: Optional[KernelArg] = None

    @staticmethod
    def Buffer(b: DeviceBuffer) -> "DeviceArg":
        return DeviceArg(buffer=b)

    @staticmethod
    def Scalar(s: KernelArg) -> "DeviceArg":
        return DeviceArg(scalar=s)


class CudaContext:
    """A CUDA device's primary context (src/cuda.rs:204-488)."""

    def __init__(self, ordinal: int = 0):
        self.ordinal = ordinal
        _wrap(_lib.init, ordinal)

    @staticmethod
    def new(ordinal: int = 0) -> "CudaContext":
        return CudaContext(ordinal)

    def upload(self, arg: KernelArg) -> DeviceBuffer:
        if arg.is_scalar():
            raise TypeError("only buffers can be uploaded")
        data = np.ascontiguousarray(arg.data)
        ptr = _wrap(_lib.upload, data.ctypes.data, data.nbytes)
        return DeviceBuffer(ptr, data.nbytes, arg.dtype, data.size)

    def download(self, buffer: DeviceBuffer, arg: KernelArg) -> None:
        if arg.data.nbytes != buffer.bytes:
            raise CudaError(f"downloading {buffer.bytes} bytes into {arg.data.nbytes}")
        _wrap(_lib.download, buffer.ptr, arg.data.ctypes.data, buffer.bytes)

    def synchronize(self) -> None:
        _wrap(_lib.synchronize)

    @staticmethod
    def _check_static(kernel: Kernel, nargs: int) -> None:
        if nargs != len(kernel.params):
            raise CudaError(f"kernel `{kernel.name()}` takes {len(kernel.params)} arguments, {nargs} were given",
                            _lib.ERR_INVALID_ARGUMENT)

    @staticmethod
    def _check_lengths(kernel: Kernel, lens_dtypes) -> None:
        # The statically declared sizes of param_tensor (src/sim/mod.rs:350-357).
        for i, (p, (length, _)) in enumerate(zip(kernel.params, lens_dtypes)):
            if not p.is_scalar and p.length is not None and length is not None and length < p.length:
                raise CudaError(f"argument {i} (`{p.name}`) needs at least {p.length} elements, got {length}",
                                _lib.ERR_INVALID_ARGUMENT)

    def launch(self, kernel: Kernel, cfg: LaunchConfig, args: list) -> LaunchStats:
        """CudaContext::launch: host buffers in, results copied back in place."""
        self._check_static(kernel, len(args))
        cargs = []
        for a in args:
            if a.is_scalar():
                cargs.append(_lib.Arg(1, a.dtype.value, a.scalar_bits(), 0))
            else:
                if not a.data.flags["C_CONTIGUOUS"]:
                    a.data = np.ascontiguousarray(a.data)
                cargs.append(_lib.Arg(0, a.dtype.value, a.data.ctypes.data, a.data.size))
        self._check_lengths(kernel, [(None if a.is_scalar() else a.data.size, a.dtype) for a in args])
        sec = _wrap(_lib.launch_host, kernel.name(), cfg.grid, cfg.block, cargs, cfg.cluster)
        return LaunchStats(sec)

    def launch_async(self, kernel: Kernel, cfg: LaunchConfig, args: list, stream: int = 0) -> None:
        """Submit without waiting, arguments already on the device
        (CudaContext::launch_async, src/cuda.rs:428-439)."""
        self._check_static(kernel, len(args))
        cargs = []
        for a in args:
            if a.scalar is not None:
                cargs.append(_lib.Arg(1, a.scalar.dtype.value, a.scalar.scalar_bits(), 0))
            else:
                cargs.append(_lib.Arg(0, a.buffer.dtype.value, a.buffer.ptr, a.buffer.len))
        self._check_lengths(kernel, [(None if a.scalar is not None else a.buffer.len, None) for a in args])
        _wrap(_lib.launch, kernel.name(), cfg.grid, cfg.block, cargs, cfg.cluster, stream)

    def launch_on_device(self, kernel: Kernel, cfg: LaunchConfig, args: list) -> None:
        """Submit and wait (CudaContext::launch_on_device, src/cuda.rs:414-426)."""
        self.launch_async(kernel, cfg, args)
        self.synchronize()
