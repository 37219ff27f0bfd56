"""The reference's atom API for the hot-path kernels, plus Sm100 atoms.

Mirrors `src/atom/mma.rs` and `src/atom/copy.rs` of cute-rs as far as the
example kernels use them: `MmaOp`, `MmaF16BF16Op`, `make_mma_atom`,
`make_tiled_mma` / `TiledMma`, `CopyOp`, `make_copy_atom`,
`make_tiled_copy_tv`, `make_tiled_copy_a/b`.  Layouts are CuTe layouts
(hierarchical shape:stride, colexicographic index) evaluated on the host; only
evaluation is implemented, not the layout algebra.

New here (the reference stops at sm_80 `mma.sync`): the atoms of the sm_100a
GEMM in `csrc/gemm_sm100.cu` - `Sm100UmmaOp` (tcgen05.mma: operands through
shared-memory descriptors, accumulator in TMEM), `CopyOp.TmaLoad` (a
128-byte-swizzled box) and `CopyOp.TmemLoad` (tcgen05.ld 32x32b) - with the
exact shared-memory, TMEM and descriptor layouts the kernel relies on, so that
tests and the protocol checker can hold the hand-written kernel against them.
Nothing here runs on the GPU or computes results.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .host import DType


# --------------------------------------------------------------------------- #
# CuTe layouts: evaluation only                                                #
# --------------------------------------------------------------------------- #
def _flatten(t):
    if isinstance(t, int):
        return [t]
    out = []
    for x in t:
        out += _flatten(x)
    return out


class Layout:
    """shape:stride with nested tuples; `layout(i)` is the offset of the i-th
    element in colexicographic order (first mode fastest)."""

    def __init__(self, shape, stride):
        self.shape, self.stride = shape, stride
        self._s, self._d = _flatten(shape), _flatten(stride)
        assert len(self._s) == len(self._d), "shape and stride are not congruent"

    @staticmethod
    def row_major(shape):
        shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        stride, acc = [], 1
        for s in reversed(shape):
            stride.append(acc)
            acc *= s
        return Layout(shape, tuple(reversed(stride)))

    @staticmethod
    def col_major(shape):
        shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        stride, acc = [], 1
        for s in shape:
            stride.append(acc)
            acc *= s
        return Layout(shape, tuple(stride))

    def size(self) -> int:
        n = 1
        for s in self._s:
            n *= s
        return n

    def cosize(self) -> int:
        return 0 if self.size() == 0 else 1 + sum((s - 1) * d for s, d in zip(self._s, self._d))

    def __call__(self, index: int) -> int:
        off = 0
        for s, d in zip(self._s, self._d):
            off += (index % s) * d
            index //= s
        return off

    def values(self):
        return [self(i) for i in range(self.size())]

    def __eq__(self, other):
        return isinstance(other, Layout) and self.shape == other.shape and self.stride == other.stride

    def __repr__(self):
        return f"{self.shape}:{self.stride}"


def make_layout_tv(thr_layout: Layout, val_layout: Layout):
    """CuTe's make_layout_tv for rank-2 thread and value layouts: returns
    ((tile_m, tile_n), f) where f(thread, value) is the colexicographic index
    into the (tile_m, tile_n) tile that the thread's value covers: the value
    layout is repeated over the thread layout (a raked product)."""
    (tm, tn), (vm, vn) = thr_layout.shape, val_layout.shape
    tile = (tm * vm, tn * vn)

    def coord(l: Layout, idx: int, shape):
        # position (i, j) whose layout value equals idx (layouts here are bijections onto 0..size)
        for j in range(shape[1]):
            for i in range(shape[0]):
                if l(i + shape[0] * j) == idx:
                    return i, j
        raise ValueError("layout is not a bijection onto its index range")

    def f(thread: int, value: int) -> int:
        ti, tj = coord(thr_layout, thread, (tm, tn))
        vi, vj = coord(val_layout, value, (vm, vn))
        return (ti * vm + vi) + tile[0] * (tj * vn + vj)

    return tile, f


# --------------------------------------------------------------------------- #
# MMA atoms                                                                    #
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class MmaF16BF16Op:
    """cute.nvgpu.warp.MmaF16BF16Op (src/atom/mma.rs:37-91): warp-level mma.sync."""
    ab_dtype: DType
    acc_dtype: DType
    shape_mnk: tuple

    def __post_init__(self):
        if self.ab_dtype not in (DType.F16, DType.BF16):
            raise ValueError(f"cute: MmaF16BF16Op expects the 'ab_dtype' Op parameter to be one of Float16 or BFloat16, not {self.ab_dtype}")
        if self.acc_dtype not in (DType.F16, DType.F32):
            raise ValueError(f"cute: MmaF16BF16Op expects the 'acc_dtype' Op parameter to be one of Float16 or Float32, not {self.acc_dtype}")
        if self.ab_dtype == DType.BF16 and self.acc_dtype != DType.F32:
            raise ValueError("cute: MmaF16BF16Op expects the 'acc_dtype' Op parameter to be Float32 when 'ab_dtype' is BFloat16")
        if tuple(self.shape_mnk) not in ((16, 8, 8), (16, 8, 16)):
            raise ValueError(f"cute: MmaF16BF16Op expects the 'shape_mnk' Op parameter to be one of (16,8,8) or (16,8,16), not {self.shape_mnk}")


@dataclass(frozen=True)
class UniversalFma:
    """MmaOp::UniversalFma: one thread, d = a * b + c on scalars (src/atom/mma.rs:19-27)."""
    dtype: DType


@dataclass(frozen=True)
class Sm100UmmaOp:
    """tcgen05.mma.cta_group::{1,2}.kind::f16: one thread issues an
    (m x n x 16) MMA whose A and B come from shared memory through matrix
    descriptors and whose f32 accumulator lives in TMEM.  m counts the rows of
    the whole CTA group (128 per CTA)."""
    ab_dtype: DType
    m: int
    n: int
    cta_group: int = 1

    def __post_init__(self):
        if self.ab_dtype not in (DType.F16, DType.BF16):
            raise ValueError("Sm100UmmaOp takes f16 or bf16 operands")
        if self.cta_group not in (1, 2) or self.m != 128 * self.cta_group:
            raise ValueError("Sm100UmmaOp: m must be 128 per CTA of the group")
        if self.n % 16 or not 16 <= self.n <= 256:
            raise ValueError("Sm100UmmaOp: n must be a multiple of 16 in [16, 256]")

    shape_k = 16

    def instruction_descriptor(self) -> int:
        """The 32-bit descriptor: f32 accumulator (bits 4-5 = 1), A/B format
        (0 = f16, 1 = bf16) at bits 7 and 10, both operands K-major (bits 15, 16 =
        0), n >> 3 at bit 17, m >> 4 at bit 24."""
        fmt = 1 if self.ab_dtype == DType.BF16 else 0
        return (1 << 4) | (fmt << 7) | (fmt << 10) | ((self.n >> 3) << 17) | ((self.m >> 4) << 24)

    def tmem_coord(self, m: int, n: int, column0: int = 0):
        """(CTA of the group, TMEM lane, TMEM column) holding accumulator element (m, n)."""
        return m // 128, m % 128, column0 + n


class MmaAtom:
    """Thread/value layouts of one MMA instruction (src/atom/mma.rs:148-198):
    each maps (thread, value) to the colexicographic index into the M x K,
    N x K or M x N operand."""

    def __init__(self, op):
        self.op = op
        if isinstance(op, UniversalFma):
            self.shape_mnk, self.thr_id = (1, 1, 1), Layout(1, 0)
            self.a = self.b = self.c = Layout((1, 1), (0, 0))
        elif isinstance(op, MmaF16BF16Op):
            self.shape_mnk, self.thr_id = tuple(op.shape_mnk), Layout(32, 1)
            if op.shape_mnk[2] == 16:  # CuTe's SM80_16x8x16 traits
                self.a = Layout(((4, 8), (2, 2, 2)), ((32, 1), (16, 8, 128)))
                self.b = Layout(((4, 8), (2, 2)), ((16, 1), (8, 64)))
            else:
                self.a = Layout(((4, 8), (2, 2)), ((32, 1), (16, 8)))
                self.b = Layout(((4, 8), 2), ((16, 1), 8))
            self.c = Layout(((4, 8), (2, 2)), ((32, 1), (16, 8)))
        elif isinstance(op, Sm100UmmaOp):
            # A single thread issues it; operands are not register fragments.
            self.shape_mnk, self.thr_id = (op.m, op.n, 16), Layout(1, 0)
            self.a = self.b = self.c = None
        else:
            raise TypeError(f"not an MMA op: {op!r}")


def make_mma_atom(op) -> MmaAtom:
    return MmaAtom(op)


class TiledMma:
    """make_tiled_mma(op, atom_layout_mnk): atoms repeated over a layout of
    warps (src/atom/mma.rs:278-301).  `thr_layout_vmnk` is
    (threads per atom, atoms in m, n, k)."""

    def __init__(self, op, atom_layout: Layout):
        self.atom = op if isinstance(op, MmaAtom) else MmaAtom(op)
        shape = tuple(_flatten(atom_layout.shape)) + (1, 1, 1)
        self.atoms_mnk = shape[:3]
        threads = self.atom.thr_id.size()
        self.thr_layout_vmnk = Layout((threads,) + self.atoms_mnk,
                                      (1, threads, threads * shape[0], threads * shape[0] * shape[1]))
        m, n, k = self.atom.shape_mnk
        self.tile_shape = (m * shape[0], n * shape[1], k * shape[2])

    def size(self) -> int:
        return self.thr_layout_vmnk.size()

    def _atom_of(self, tid: int):
        t = self.atom.thr_id.size()
        w = tid // t
        return tid % t, w % self.atoms_mnk[0], (w // self.atoms_mnk[0]) % self.atoms_mnk[1]

    def c_coords(self, tid: int, tile_mn=None):
        """(m, n) of every accumulator value of thread `tid` over a CTA tile
        `tile_mn` (default: one tiled-MMA step), in value order, the atom tile
        repeating with the tiled-MMA's extent (interleaved, as partition_C does)."""
        lane, am, an = self._atom_of(tid)
        m, n, _ = self.atom.shape_mnk
        step_m, step_n = self.tile_shape[0], self.tile_shape[1]
        tile_mn = tile_mn or (step_m, step_n)
        out = []
        for rn in range(tile_mn[1] // step_n):
            for rm in range(tile_mn[0] // step_m):
                for v in range(self.atom.c.size() // 32):
                    idx = self.atom.c(lane + 32 * v)
                    out.append((rm * step_m + am * m + idx % m, rn * step_n + an * n + idx // m))
        return out

    def layout_a_tv(self) -> Layout:
        return self.atom.a

    def layout_b_tv(self) -> Layout:
        return self.atom.b

    def layout_c_tv(self) -> Layout:
        return self.atom.c


def make_tiled_mma(op, atom_layout: Layout = None) -> TiledMma:
    return TiledMma(op, atom_layout or Layout.col_major((1, 1, 1)))


# --------------------------------------------------------------------------- #
# Copy atoms                                                                   #
# --------------------------------------------------------------------------- #
class CopyOp:
    """The copy instructions (src/atom/copy.rs:21-33), plus the sm_100a ones."""

    @dataclass(frozen=True)
    class Universal:
        bits: int

    @dataclass(frozen=True)
    class CpAsync:
        bytes: int
        bypass_l1: bool = True

    @dataclass(frozen=True)
    class LdMatrix:
        num: int
        trans: bool = False

    @dataclass(frozen=True)
    class TmaLoad:
        """cp.async.bulk.tensor.2d of a (rows x 64 element) box of a K-major
        16-bit matrix into 128-byte-swizzled shared memory, completion counted in
        bytes on an mbarrier."""
        rows: int
        elem_bytes: int = 2
        swizzle_bytes: int = 128

        @property
        def box_bytes(self) -> int:
            return self.rows * 64 * self.elem_bytes

    @dataclass(frozen=True)
    class TmaStore:
        """cp.async.bulk.tensor.2d.global.shared::cta.bulk_group of a (rows x cols
        element) box of a row-major matrix from unswizzled shared memory; rows and
        columns past the end of the matrix are clipped; completion by bulk group.
        The pusher warp's copy of a finished tile into another GPU's C."""
        rows: int
        cols: int
        elem_bytes: int = 2

        @property
        def box_bytes(self) -> int:
            return self.rows * self.cols * self.elem_bytes

        def __post_init__(self):
            if self.cols > 256 or (self.cols * self.elem_bytes) % 16:
                raise ValueError("TmaStore: at most 256 elements per box row, a multiple of 16 bytes")

    @dataclass(frozen=True)
    class TmemLoad:
        """tcgen05.ld.32x32b.xN: a warp reads N consecutive 32-bit columns of its
        32 TMEM lanes; lane l of warp w addresses TMEM lane 32 * (w % 4) + l."""
        columns: int = 32


def sw128_offset(row: int, k: int, elem_bytes: int = 2) -> int:
    """Byte offset of element (row, k) of a K-major tile of 64 16-bit elements per
    row as TMA writes it with the 128-byte swizzle and tcgen05.mma reads it: rows
    are 128 bytes apart and the 16-byte chunk index is XORed with row % 8
    (Swizzle<3,4,3> on byte addresses; the pattern repeats every 1024 bytes, which
    is why tile bases are 1024-byte aligned)."""
    byte = k * elem_bytes
    assert 0 <= byte < 128
    return row * 128 + ((((byte >> 4) ^ (row & 7)) << 4) | (byte & 15))


def sw128_descriptor(smem_addr: int) -> int:
    """The 64-bit shared-memory matrix descriptor of such a tile at `smem_addr`:
    (addr & 0x3ffff) >> 4 at bit 0, leading byte offset 1 at bit 16 (unused for
    swizzled K-major), stride byte offset 1024 >> 4 at bit 32 (eight rows),
    descriptor version 1 at bit 46, layout type 2 (SWIZZLE_128B) at bit 61.
    Advancing k by 16 elements adds 32 bytes = 2 to the address field."""
    return ((smem_addr & 0x3FFFF) >> 4) | (1 << 16) | ((1024 >> 4) << 32) | (1 << 46) | (2 << 61)


class CopyAtom:
    """make_copy_atom::<T>(op) (src/atom/copy.rs:46-90): source and destination
    thread/value layouts in elements of `dtype`."""

    def __init__(self, dtype: DType, op):
        self.dtype, self.op = dtype, op
        ebits = dtype.bytes() * 8
        if isinstance(op, (CopyOp.Universal, CopyOp.CpAsync)):
            bits = op.bits if isinstance(op, CopyOp.Universal) else op.bytes * 8
            if bits % ebits:
                raise ValueError(f"a {bits}-bit copy does not hold whole {dtype} values")
            n = bits // ebits
            self.thr_id = Layout(1, 0)
            self.layout_src_tv = self.layout_dst_tv = Layout((1, n), (0, 1))
        elif isinstance(op, CopyOp.LdMatrix):
            if ebits != 16:
                raise ValueError("ldmatrix moves 16-bit values")
            self.thr_id = Layout(32, 1)
            # CuTe's SM75_U32x{1,2,4}_LDSM_N traits in 16-bit values
            self.layout_src_tv = Layout((32, 8), (8, 1))
            self.layout_dst_tv = Layout((32, (2, op.num)), (2, (1, 64)))
        elif isinstance(op, CopyOp.TmaLoad):
            self.thr_id = Layout(1, 0)  # one elected thread issues it
            self.layout_src_tv = self.layout_dst_tv = None
        elif isinstance(op, CopyOp.TmemLoad):
            self.thr_id = Layout(32, 1)
            self.layout_src_tv = self.layout_dst_tv = Layout((32, op.columns), (1, 32))
        else:
            raise TypeError(f"not a copy op: {op!r}")

    def value_type(self) -> DType:
        return self.dtype

    def num_threads(self) -> int:
        return self.thr_id.size()


def make_copy_atom(dtype: DType, op) -> CopyAtom:
    return CopyAtom(dtype, op)


class TiledCopy:
    def __init__(self, atom: CopyAtom, tile_shape, threads: int, values: int, tv: Callable[[int, int], int],
                 src_tv: Callable[[int, int], int] = None):
        self.atom, self.tile_shape_, self.threads, self.values, self._tv = atom, tile_shape, threads, values, tv
        self._src_tv = src_tv or tv

    def size(self) -> int:
        return self.threads

    def tile_shape(self):
        return self.tile_shape_

    def layout_tv_tiled(self, thread: int, value: int) -> int:
        """Colexicographic index into the tile of the value a thread receives."""
        return self._tv(thread, value)

    def layout_src_tv_tiled(self, thread: int, value: int) -> int:
        """... and of the value it supplies the address for."""
        return self._src_tv(thread, value)


def make_tiled_copy_tv(atom: CopyAtom, thr_layout: Layout, val_layout: Layout) -> TiledCopy:
    """make_tiled_copy_tv (src/atom/copy.rs:210-214): `thr_layout` threads each
    moving `val_layout` values; the values of one instruction must be contiguous
    in the value layout's fastest mode."""
    tile, f = make_layout_tv(thr_layout, val_layout)
    return TiledCopy(atom, tile, thr_layout.size(), val_layout.size(), f)


def make_tiled_copy_a(atom: CopyAtom, mma: TiledMma) -> TiledCopy:
    """ldmatrix.x4 laid out like the MMA's A fragment (src/atom/copy.rs:178-232):
    thread l receives the values layout_a_tv gives it and addresses row
    l % 8 + 8 * ((l / 8) % 2), k chunk l / 16 of the 16 x 16 tile."""
    a = mma.layout_a_tv()
    m, _, k = mma.atom.shape_mnk
    return TiledCopy(atom, (m, k), 32, a.size() // 32, lambda t, v: a(t + 32 * v),
                     lambda t, v: (t % 8 + 8 * ((t // 8) % 2)) + m * (8 * (t // 16) + v))


def make_tiled_copy_b(atom: CopyAtom, mma: TiledMma) -> TiledCopy:
    """ldmatrix.x2 for the B fragment: thread l < 16 addresses row l % 8 of the
    8 x 16 (N x K) tile, k chunk (l / 8) % 2."""
    b = mma.layout_b_tv()
    _, n, k = mma.atom.shape_mnk
    return TiledCopy(atom, (n, k), 32, b.size() // 32, lambda t, v: b(t + 32 * v),
                     lambda t, v: (t % 8) + n * (8 * ((t // 8) % 2) + v))
