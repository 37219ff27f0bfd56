"""ctypes binding of libcute_b200.so: one Python function per C entry point.

The signatures are those of include/cute_b200.h: plain integers, floats and
device addresses.  Nothing here computes anything; without the shared library
(or without a B200) every call fails loudly.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcute_b200.so")

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_MISALIGNED = -2
ERR_UNSUPPORTED = -3
ERR_NO_DEVICE = -4
ERR_DEVICE_TIMEOUT = -5
ERR_CUDA = -6
ERR_NULL_POINTER = -7

F16, BF16, F32, I32 = 0, 1, 2, 3

EXPORTS = (
    "cute_b200_status_string", "cute_b200_last_error", "cute_b200_init", "cute_b200_gemm_tn", "cute_b200_sgemm_nt",
    "cute_b200_gemm_tn_host", "cute_b200_release_workspace", "cute_b200_gemm_tn_static",
    "cute_b200_elementwise_add_f32", "cute_b200_launch", "cute_b200_launch_host", "cute_b200_upload",
    "cute_b200_download", "cute_b200_free", "cute_b200_synchronize", "cute_b200_shard_rows",
    "cute_b200_gemm_tn_shard", "cute_b200_device_status", "cute_b200_launch_count", "cute_b200_alloc",
    "cute_b200_ipc_export", "cute_b200_ipc_open", "cute_b200_ipc_close", "cute_b200_copy_async", "cute_b200_gemm_tn_multi",
    "cute_b200_gemm_layout_info", "cute_b200_gemm_plan", "cute_b200_comm_create", "cute_b200_comm_destroy", "cute_b200_comm_info",
    "cute_b200_gemm_tn_sharded", "cute_b200_gemm_tn_sharded_host", "cute_b200_gemm_tn_multi_signal", "cute_b200_wait_signal",
)

REPLICATE_NONE, REPLICATE_AUTO, REPLICATE_FUSED, REPLICATE_COLLECTIVE, REPLICATE_COPIES = range(5)


class GemmDesc(ctypes.Structure):
    _fields_ = [("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32), ("ab_dtype", ctypes.c_int32),
                ("c_dtype", ctypes.c_int32), ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
                ("tile_n", ctypes.c_int32), ("cta_group", ctypes.c_int32), ("tile_m", ctypes.c_int32),
                ("split_k", ctypes.c_int32), ("tuning", ctypes.c_int32 * 2)]


class GemmLayout(ctypes.Structure):
    """cute_b200_gemm_layout: the constants one GEMM tiling is compiled from."""
    _fields_ = [(name, ctypes.c_uint32) for name in (
        "instruction_descriptor", "umma_m", "umma_n", "umma_k", "block_k", "cta_rows", "a_block_bytes", "b_block_bytes",
        "k_blocks_per_stage", "stage_bytes", "stages", "accumulator_halves", "half_columns", "accumulator_buffers", "tmem_columns", "threads",
        "epilogue_warps", "full_arrivals", "empty_arrivals", "tmem_full_arrivals", "tmem_empty_arrivals",
        "full_expect_tx_bytes_per_k_block", "push_chunk_bytes", "push_chunk_rows", "push_chunks_per_tile", "shared_memory_bytes",
        "descriptor_k_step")] + [("smem_descriptor", ctypes.c_uint64)]


class Arg(ctypes.Structure):
    _fields_ = [("is_scalar", ctypes.c_int32), ("dtype", ctypes.c_int32), ("value", ctypes.c_uint64),
                ("len", ctypes.c_uint64)]


class LaunchCfg(ctypes.Structure):
    _fields_ = [("grid", ctypes.c_uint32 * 3), ("block", ctypes.c_uint32 * 3), ("cluster", ctypes.c_uint32 * 3)]


class CuteB200Error(RuntimeError):
    """A non-zero status from the library; carries the code and its message."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{status_string(status)}: {message}")
        self.status = status
        self.message = message


_lib = None


def load() -> ctypes.CDLL:
    """dlopen the library (no implicit build: see cute_rs_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m cute_rs_b200.build` (needs nvcc)")
    L = ctypes.CDLL(LIB_PATH)
    i32, u64, f32, vp, cp = ctypes.c_int32, ctypes.c_uint64, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p
    L.cute_b200_status_string.argtypes = [i32]
    L.cute_b200_status_string.restype = cp
    L.cute_b200_last_error.argtypes = []
    L.cute_b200_last_error.restype = cp
    L.cute_b200_init.argtypes = [i32]
    L.cute_b200_gemm_tn.argtypes = [ctypes.POINTER(GemmDesc), u64, u64, u64, vp]
    L.cute_b200_gemm_tn_static.argtypes = [ctypes.POINTER(GemmDesc), u64, u64, u64, vp]
    L.cute_b200_gemm_tn_host.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, ctypes.POINTER(ctypes.c_double)]
    L.cute_b200_release_workspace.argtypes = []
    L.cute_b200_sgemm_nt.argtypes = [i32, i32, i32, f32, f32, u64, u64, u64, vp]
    L.cute_b200_elementwise_add_f32.argtypes = [u64, u64, u64, u64, vp]
    L.cute_b200_launch.argtypes = [cp, ctypes.POINTER(LaunchCfg), ctypes.POINTER(Arg), i32, vp]
    L.cute_b200_launch_host.argtypes = [cp, ctypes.POINTER(LaunchCfg), ctypes.POINTER(Arg), i32,
                                        ctypes.POINTER(ctypes.c_double)]
    L.cute_b200_upload.argtypes = [vp, u64, ctypes.POINTER(u64)]
    L.cute_b200_download.argtypes = [u64, vp, u64]
    L.cute_b200_free.argtypes = [u64]
    L.cute_b200_synchronize.argtypes = []
    L.cute_b200_alloc.argtypes = [u64, ctypes.POINTER(u64)]
    L.cute_b200_ipc_export.argtypes = [u64, ctypes.c_char_p]
    L.cute_b200_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(u64)]
    L.cute_b200_ipc_close.argtypes = [u64]
    L.cute_b200_copy_async.argtypes = [u64, u64, u64, vp]
    L.cute_b200_gemm_tn_multi.argtypes = [ctypes.POINTER(GemmDesc), u64, u64, ctypes.POINTER(u64), i32, vp]
    L.cute_b200_gemm_tn_multi_signal.argtypes = [ctypes.POINTER(GemmDesc), u64, u64, ctypes.POINTER(u64), ctypes.POINTER(u64), i32, vp]
    L.cute_b200_wait_signal.argtypes = [u64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, vp]
    L.cute_b200_shard_rows.argtypes = [i32, i32, i32, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    L.cute_b200_gemm_tn_shard.argtypes = [ctypes.POINTER(GemmDesc), i32, i32, u64, u64, u64, i32, vp]
    L.cute_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint32 * 4)]
    L.cute_b200_gemm_layout_info.argtypes = [i32, i32, i32, i32, i32, ctypes.c_uint32, ctypes.POINTER(GemmLayout)]
    L.cute_b200_comm_create.argtypes = [i32, ctypes.POINTER(i32), ctypes.POINTER(vp)]
    L.cute_b200_comm_destroy.argtypes = [vp]
    L.cute_b200_comm_info.argtypes = [vp, ctypes.POINTER(i32 * 4)]
    L.cute_b200_gemm_tn_sharded.argtypes = [vp, ctypes.POINTER(GemmDesc), ctypes.POINTER(u64), ctypes.POINTER(u64),
                                            ctypes.POINTER(u64), i32]
    L.cute_b200_gemm_tn_sharded_host.argtypes = [vp, ctypes.POINTER(GemmDesc), vp, vp, vp, ctypes.POINTER(ctypes.c_double)]
    L.cute_b200_gemm_plan.argtypes = [ctypes.POINTER(GemmDesc), i32, ctypes.POINTER(i32 * 4)]
    L.cute_b200_launch_count.argtypes = []
    L.cute_b200_launch_count.restype = u64
    for name in EXPORTS:
        if name not in ("cute_b200_status_string", "cute_b200_last_error", "cute_b200_launch_count"):
            getattr(L, name).restype = i32
    _lib = L
    return L


def status_string(status: int) -> str:
    return load().cute_b200_status_string(status).decode()


def last_error() -> str:
    return load().cute_b200_last_error().decode()


def check(status: int) -> None:
    if status != OK:
        raise CuteB200Error(status, last_error())


def init(device: int = 0) -> None:
    check(load().cute_b200_init(device))


def gemm_desc(m, n, k, ab_dtype, c_dtype, alpha=1.0, beta=0.0, tile_n=0, cta_group=0, tile_m=0,
              split_k=0) -> GemmDesc:
    return GemmDesc(m, n, k, ab_dtype, c_dtype, alpha, beta, tile_n, cta_group, tile_m, split_k,
                    (ctypes.c_int32 * 2)(0, 0))


def gemm_tn(desc: GemmDesc, dA: int, dB: int, dC: int, stream: int = 0) -> None:
    check(load().cute_b200_gemm_tn(ctypes.byref(desc), dA, dB, dC, stream))


def gemm_tn_multi(desc: GemmDesc, dA: int, dB: int, dC_list, stream: int = 0) -> None:
    """GEMM whose epilogue writes the result to every address in dC_list (own C and peers')."""
    arr = (ctypes.c_uint64 * len(dC_list))(*dC_list)
    check(load().cute_b200_gemm_tn_multi(ctypes.byref(desc), dA, dB, arr, len(dC_list), stream))


def gemm_tn_multi_signal(desc: GemmDesc, dA: int, dB: int, dC_list, dSignal_list, stream: int = 0) -> None:
    """gemm_tn_multi that adds 1 to the counter of every further destination's owner once the launch is complete."""
    n = len(dC_list)
    assert len(dSignal_list) == n
    check(load().cute_b200_gemm_tn_multi_signal(ctypes.byref(desc), dA, dB, (ctypes.c_uint64 * n)(*dC_list),
                                                (ctypes.c_uint64 * n)(*dSignal_list), n, stream))


def wait_signal(dSignals: int, mask: int, at_least: int, timeout_ms: int = 30000, stream: int = 0) -> None:
    """Queue the bounded wait for the counters dSignals[i], i in `mask`, on `stream`."""
    check(load().cute_b200_wait_signal(dSignals, mask, at_least & 0xFFFFFFFF, timeout_ms, stream))


def gemm_tn_static(desc: GemmDesc, dA: int, dB: int, dC: int, stream: int = 0) -> None:
    """Split-k GEMM on the library's built-in scratch array: allocates nothing."""
    check(load().cute_b200_gemm_tn_static(ctypes.byref(desc), dA, dB, dC, stream))


def gemm_tn_host(desc: GemmDesc, hA: int, hB: int, hC: int) -> float:
    """GEMM on host buffers (addresses); returns the kernel's device seconds."""
    sec = ctypes.c_double(0.0)
    check(load().cute_b200_gemm_tn_host(ctypes.byref(desc), hA, hB, hC, ctypes.byref(sec)))
    return sec.value


def release_workspace() -> None:
    check(load().cute_b200_release_workspace())


def gemm_tn_shard(desc: GemmDesc, world: int, rank: int, dA_shard: int, dB: int, dC_base: int, c_is_full: bool,
                  stream: int = 0) -> None:
    check(load().cute_b200_gemm_tn_shard(ctypes.byref(desc), world, rank, dA_shard, dB, dC_base, int(c_is_full),
                                         stream))


def shard_rows(m: int, world: int, rank: int) -> tuple[int, int]:
    b, r = ctypes.c_int32(), ctypes.c_int32()
    check(load().cute_b200_shard_rows(m, world, rank, ctypes.byref(b), ctypes.byref(r)))
    return b.value, r.value


def sgemm_nt(m, n, k, alpha, beta, dA: int, dB: int, dC: int, stream: int = 0) -> None:
    check(load().cute_b200_sgemm_nt(m, n, k, alpha, beta, dA, dB, dC, stream))


def elementwise_add_f32(dX: int, dY: int, dOut: int, n: int, stream: int = 0) -> None:
    check(load().cute_b200_elementwise_add_f32(dX, dY, dOut, n, stream))


def _cfg(grid, block, cluster=(1, 1, 1)) -> LaunchCfg:
    return LaunchCfg((ctypes.c_uint32 * 3)(*grid), (ctypes.c_uint32 * 3)(*block), (ctypes.c_uint32 * 3)(*cluster))


def launch(name: str, grid, block, args: list[Arg], cluster=(1, 1, 1), stream: int = 0) -> None:
    arr = (Arg * len(args))(*args)
    check(load().cute_b200_launch(name.encode(), ctypes.byref(_cfg(grid, block, cluster)), arr, len(args), stream))


def launch_host(name: str, grid, block, args: list[Arg], cluster=(1, 1, 1)) -> float:
    arr = (Arg * len(args))(*args)
    sec = ctypes.c_double(0.0)
    check(load().cute_b200_launch_host(name.encode(), ctypes.byref(_cfg(grid, block, cluster)), arr, len(args),
                                       ctypes.byref(sec)))
    return sec.value


def upload(host_ptr: int, nbytes: int) -> int:
    out = ctypes.c_uint64()
    check(load().cute_b200_upload(host_ptr, nbytes, ctypes.byref(out)))
    return out.value


def download(device: int, host_ptr: int, nbytes: int) -> None:
    check(load().cute_b200_download(device, host_ptr, nbytes))


def free(device: int) -> None:
    check(load().cute_b200_free(device))


def alloc(nbytes: int) -> int:
    out = ctypes.c_uint64()
    check(load().cute_b200_alloc(nbytes, ctypes.byref(out)))
    return out.value


def ipc_export(device: int) -> bytes:
    buf = ctypes.create_string_buffer(64)
    check(load().cute_b200_ipc_export(device, buf))
    return buf.raw


def ipc_open(handle: bytes) -> int:
    out = ctypes.c_uint64()
    check(load().cute_b200_ipc_open(handle, ctypes.byref(out)))
    return out.value


def ipc_close(device: int) -> None:
    check(load().cute_b200_ipc_close(device))


def copy_async(dst: int, src: int, nbytes: int, stream: int = 0) -> None:
    check(load().cute_b200_copy_async(dst, src, nbytes, stream))


def synchronize() -> None:
    check(load().cute_b200_synchronize())


def device_status() -> tuple[int, int, int, int]:
    out = (ctypes.c_uint32 * 4)()
    check(load().cute_b200_device_status(ctypes.byref(out)))
    return tuple(out)


def comm_create(ordinals) -> int:
    """One communicator over the listed devices of this process (an int n means devices 0 .. n-1)."""
    if isinstance(ordinals, int):
        ordinals = list(range(ordinals))
    arr = (ctypes.c_int32 * len(ordinals))(*ordinals)
    out = ctypes.c_void_p()
    check(load().cute_b200_comm_create(len(ordinals), arr, ctypes.byref(out)))
    return out.value


def comm_destroy(comm: int) -> None:
    check(load().cute_b200_comm_destroy(comm))


def comm_info(comm: int) -> dict:
    out = (ctypes.c_int32 * 4)()
    check(load().cute_b200_comm_info(comm, ctypes.byref(out)))
    return {"ngpus": out[0], "distinct": bool(out[1]), "peer_access": bool(out[2]), "collective_library": bool(out[3])}


def gemm_tn_sharded(comm: int, desc: GemmDesc, dA_shards, dB, dC, replicate_c: int = REPLICATE_NONE) -> None:
    """The row-sharded GEMM on every GPU of `comm`: one device pointer per GPU in each list; returns when all are done."""
    n = len(dA_shards)
    mk = lambda xs: (ctypes.c_uint64 * n)(*xs)
    check(load().cute_b200_gemm_tn_sharded(comm, ctypes.byref(desc), mk(dA_shards), mk(dB), mk(dC), replicate_c))


def gemm_tn_sharded_host(comm: int, desc: GemmDesc, hA: int, hB: int, hC: int) -> float:
    """The same on whole host matrices (addresses); returns the duration of the call in seconds."""
    sec = ctypes.c_double(0.0)
    check(load().cute_b200_gemm_tn_sharded_host(comm, ctypes.byref(desc), hA, hB, hC, ctypes.byref(sec)))
    return sec.value


def gemm_layout_info(cta_group: int, tile_n: int, tile_m: int, ab_dtype: int = BF16, c_dtype: int = BF16,
                     smem_addr: int = 0) -> GemmLayout:
    """The constants the compiled kernel of this tiling uses (host arithmetic, no GPU needed)."""
    out = GemmLayout()
    check(load().cute_b200_gemm_layout_info(cta_group, tile_n, tile_m, ab_dtype, c_dtype, smem_addr, ctypes.byref(out)))
    return out


def gemm_plan(desc: GemmDesc, sm_count: int = 0) -> tuple:
    """(cta_group, tile_n, tile_m, split_k) the library would run `desc` with."""
    out = (ctypes.c_int32 * 4)()
    check(load().cute_b200_gemm_plan(ctypes.byref(desc), sm_count, ctypes.byref(out)))
    return tuple(out)


# Every (cta_group, tile_n, tile_m) the library instantiates.
GEMM_TILINGS = [(g, n, m) for g in (1, 2) for n in (128, 256) for m in (128, 256)] + [(2, 128, 64), (2, 256, 64)]


def launch_count() -> int:
    return int(load().cute_b200_launch_count())
