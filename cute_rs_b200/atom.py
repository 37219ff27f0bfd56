"""The reference's atom API for the hot-path kernels, plus Sm100 atoms.

Mirrors `src/atom/mma.rs` and `src/atom/copy.rs` of cute-rs as far as the
example kernels use them: `MmaOp`, `MmaF16BF16Op`, `make_mma_atom`,
`make_tiled_mma` / `TiledMma`, `CopyOp`, `make_copy_atom`, `make_tiled_copy`,
`make_tiled_copy_tv`, `make_tiled_copy_a/b/c`, `make_tiled_copy_s/d`,
`make_tiled_copy_c_atom`, `TiledCopy.retile`, and `copy` / `copy_if` /
`autovec_copy` as planners that return the instructions a copy breaks into
(the reference emits them into its IR).  Layouts are CuTe layouts
(hierarchical shape:stride, colexicographic index) evaluated on the host:
results that the reference derives with its layout algebra are derived here by
evaluating the maps and reading the strides back (`Layout.with_strides_of`,
`Layout.from_values`, `Layout.filter`).

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

    def rank(self) -> int:
        return len(self.shape) if isinstance(self.shape, tuple) else 1

    def mode(self, i: int) -> "Layout":
        if not isinstance(self.shape, tuple):
            assert i == 0
            return self
        return Layout(self.shape[i], self.stride[i])

    @staticmethod
    def from_values(vals) -> "Layout":
        """The coalesced layout whose values, in colexicographic order, are `vals`
        (vals[0] must be 0): the first mode is the longest arithmetic run from the
        start, the next mode steps over whole runs, and so on.  Raises if the
        sequence is not a layout."""
        vals = list(vals)
        n = len(vals)
        if n == 0 or vals[0] != 0:
            raise ValueError("not the values of a layout")
        shape, stride, step = [], [], 1
        while step < n:
            d = vals[step]
            e = 1
            while (e + 1) * step <= n and vals[e * step] == e * d:
                e += 1
            if n % (e * step):
                raise ValueError("not the values of a layout")
            shape.append(e)
            stride.append(d)
            step *= e
        if not shape:
            shape, stride = [1], [0]
        out = Layout(shape[0], stride[0]) if len(shape) == 1 else Layout(tuple(shape), tuple(stride))
        if out.values() != vals:
            raise ValueError("not the values of a layout")
        return out

    @staticmethod
    def with_strides_of(shape, fn) -> "Layout":
        """The layout of hierarchical `shape` that agrees with `fn` (a function of
        the colexicographic index): every stride is read off at the unit step of
        its mode; raises if `fn` is not linear in the coordinates."""
        flat = _flatten(shape)
        strides, step = [], 1
        for e in flat:
            strides.append(fn(step) - fn(0) if e > 1 else 0)
            step *= e
        it = iter(strides)

        def rebuild(t):
            return next(it) if isinstance(t, int) else tuple(rebuild(x) for x in t)

        out = Layout(shape, rebuild(shape))
        if fn(0) != 0 or any(out(i) != fn(i) for i in range(out.size())):
            raise ValueError("the function is not a layout over this shape")
        return out

    def filter(self) -> "Layout":
        """CuTe's filter: modes of stride 0 or extent 1 dropped, the rest coalesced."""
        modes = [(e, d) for e, d in zip(self._s, self._d) if e > 1 and d != 0]
        merged = []
        for e, d in modes:
            if merged and merged[-1][1] * merged[-1][0] == d:
                merged[-1] = (merged[-1][0] * e, merged[-1][1])
            else:
                merged.append((e, d))
        if not merged:
            return Layout(1, 0)
        if len(merged) == 1:
            return Layout(merged[0][0], merged[0][1])
        return Layout(tuple(e for e, _ in merged), tuple(d for _, d in merged))

    def __eq__(self, other):
        return isinstance(other, Layout) and self.shape == other.shape and self.stride == other.stride

    def __repr__(self):
        return f"{self.shape}:{self.stride}"


def make_layout_tv(thr_layout: Layout, val_layout: Layout):
    """CuTe's make_layout_tv for rank-2 thread and value layouts: returns
    ((tile_m, tile_n), f) where f(thread, value) is the colexicographic index
    into the (tile_m, tile_n) tile that the thread's value covers: the value
    layout is repeated over the thread layout (a raked product)."""
    def two(l: Layout):  # a rank-1 layout counts as (n, 1)
        sh = l.shape if isinstance(l.shape, tuple) else (l.shape,)
        return (sh[0], 1) if len(sh) == 1 else sh

    (tm, tn), (vm, vn) = two(thr_layout), two(val_layout)
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
    the whole CTA group: 128 per CTA, or 64 per CTA of a pair (m = 128,
    cta_group = 2), whose accumulator still fills all 128 TMEM lanes of each
    CTA: lanes 0-63 hold its 64 rows for columns [0, n/2), lanes 64-127 the
    same rows for columns [n/2, n)."""
    ab_dtype: DType
    m: int
    n: int
    cta_group: int = 1

    def __post_init__(self):
        if self.ab_dtype not in (DType.F16, DType.BF16):
            raise ValueError("Sm100UmmaOp takes f16 or bf16 operands")
        if self.cta_group not in (1, 2) or self.m not in ((128,) if self.cta_group == 1 else (128, 256)):
            raise ValueError("Sm100UmmaOp: m must be 128 per CTA of the group, or 64 per CTA of a pair")
        if self.n % 16 or not 16 <= self.n <= 256:
            raise ValueError("Sm100UmmaOp: n must be a multiple of 16 in [16, 256]")

    shape_k = 16

    def instruction_descriptor(self) -> int:
        """The 32-bit descriptor: f32 accumulator (bits 4-5 = 1), A/B format
        (0 = f16, 1 = bf16) at bits 7 and 10, both operands K-major (bits 15, 16 =
        0), n >> 3 at bit 17, m >> 4 at bit 24."""
        fmt = 1 if self.ab_dtype == DType.BF16 else 0
        return (1 << 4) | (fmt << 7) | (fmt << 10) | ((self.n >> 3) << 17) | ((self.m >> 4) << 24)

    @property
    def rows_per_cta(self) -> int:
        return self.m // self.cta_group

    @property
    def tmem_columns(self) -> int:
        """TMEM columns one accumulator takes in each CTA."""
        return self.n // 2 if self.rows_per_cta == 64 else self.n

    def tmem_coord(self, m: int, n: int, column0: int = 0):
        """(CTA of the group, TMEM lane, TMEM column) holding accumulator element (m, n)."""
        if self.rows_per_cta == 64:
            half = self.n // 2
            return m // 64, m % 64 + 64 * (n // half), column0 + n % half
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

    def num_val_src(self) -> int:
        return self.layout_src_tv.mode(1).size()

    def num_val_dst(self) -> int:
        return self.layout_dst_tv.mode(1).size()

    def num_val_ref(self) -> int:
        """Values per thread of the atom's reference layout (the source side for every op here)."""
        return self.num_val_src()


def make_copy_atom(dtype: DType, op) -> CopyAtom:
    return CopyAtom(dtype, op)


def _tiler_size(t) -> int:
    if isinstance(t, Layout):
        return t.size()
    if isinstance(t, int):
        return t
    n = 1
    for x in t:
        n *= _tiler_size(x)
    return n


def _tiler_shape(t):
    if isinstance(t, Layout):
        return t.shape
    if isinstance(t, int):
        return t
    return tuple(_tiler_shape(x) for x in t)


class TiledCopy:
    """A copy atom tiled across threads and values (src/atom/copy.rs:150-232).
    `tiler_mn` is the tile one application covers: an extent per mode, or a
    layout per mode that selects scattered coordinates (make_tiled_copy_c_atom)."""

    def __init__(self, atom: CopyAtom, tile_shape, threads: int, values: int, tv: Callable[[int, int], int],
                 src_tv: Callable[[int, int], int] = None, tiler_mn=None):
        self.atom, self.tile_shape_, self.threads, self.values, self._tv = atom, tile_shape, threads, values, tv
        self._src_tv = src_tv or tv
        self.tiler_mn_ = tiler_mn if tiler_mn is not None else tile_shape

    def size(self) -> int:
        return self.threads

    def tile_shape(self):
        return self.tile_shape_

    def tiler_mn(self):
        return self.tiler_mn_

    def value_type(self) -> DType:
        return self.atom.dtype

    def thr_id(self) -> Layout:
        return Layout(self.threads, 1)

    def layout_tv_tiled(self, thread: int, value: int) -> int:
        """Colexicographic index into the tile of the value a thread receives."""
        return self._tv(thread, value)

    layout_dst_tv_tiled = layout_tv_tiled

    def layout_src_tv_tiled(self, thread: int, value: int) -> int:
        """... and of the value it supplies the address for."""
        return self._src_tv(thread, value)

    def layout_tv(self, shape=None) -> Layout:
        """(thread, value) -> tile index as a layout; `shape` gives the hierarchy
        of the two modes (default: each mode coalesced on its own)."""
        if shape is not None:
            return Layout.with_strides_of(shape, lambda i: self._tv(i % self.threads, i // self.threads))
        t = Layout.from_values([self._tv(i, 0) for i in range(self.threads)])
        v = Layout.from_values([self._tv(0, j) for j in range(self.values)])
        out = Layout((t.shape, v.shape), (t.stride, v.stride))
        if any(out(i) != self._tv(i % self.threads, i // self.threads) for i in range(out.size())):
            raise ValueError("the (thread, value) map is not a layout")
        return out

    def retile(self, frag: Layout) -> Layout:
        """View a thread's fragment as a source or destination of this copy
        (src/atom/copy.rs:355-391, CuTe's retile).  Mode 0 of `frag` holds a run of
        the thread's values in the order of this copy's value layout; its other
        modes count, fastest first, the runs the thread owns along each mode of the
        tile and then the repeats of the whole tile.  The result is
        ((values of one tile in the copy's order), repeats along m, n, ...) ->
        offset in the fragment."""
        modes = [frag.mode(i) for i in range(frag.rank())]
        v = modes[0].size()
        if self.values % v:
            raise ValueError(f"cute: a fragment run of {v} values does not divide the copy's {self.values} values per thread")
        shape = self.tile_shape_ if isinstance(self.tile_shape_, tuple) else (self.tile_shape_,)
        extents = [_tiler_size(x) for x in shape]
        runs = self.values // v
        # where each run of thread 0 starts, as a coordinate per tile mode, ranked among the runs
        coords = []
        for r in range(runs):
            idx, c = self._tv(0, r * v), []
            for e in extents:
                c.append(idx % e)
                idx //= e
            coords.append(c)
        ranks = [sorted({c[i] for c in coords}) for i in range(len(extents))]
        per_mode = [len(x) for x in ranks]
        rest = [m.size() for m in modes[1:]]
        if len(rest) > len(per_mode) or any(n != 1 for n in per_mode[len(rest):]):
            if len(rest) < len(per_mode) and any(n != 1 for n in per_mode[len(rest):]):
                raise ValueError(f"cute: cannot retile a rank-{len(modes)} tensor for a copy over {len(per_mode)} modes")
        while len(rest) < len(per_mode):
            rest.append(1)
            modes.append(Layout(1, 0))
        for got, need in zip(rest, per_mode):
            if got % need:
                raise ValueError("cute: the fragment's modes do not hold whole tiles of this copy")
        repeats = [got // need for got, need in zip(rest, per_mode)] + rest[len(per_mode):]

        def slot(w: int, rep) -> int:
            off = modes[0](w % v)
            c = coords[w // v]
            for i, m in enumerate(modes[1:]):
                inner = ranks[i].index(c[i]) if i < len(per_mode) else 0
                need = per_mode[i] if i < len(per_mode) else 1
                off += m(inner + need * rep[i])
            return off

        zero = [0] * len(repeats)
        mode0 = Layout.from_values([slot(w, zero) for w in range(self.values)])
        shapes, strides = [mode0.shape], [mode0.stride]
        for i, n in enumerate(repeats):
            unit = list(zero)
            unit[i] = 1
            shapes.append(n)
            strides.append(slot(0, unit) if n > 1 else 0)
        return Layout(tuple(shapes), tuple(strides))


def make_fragment(shape) -> Layout:
    """A register fragment of `shape`, first mode fastest (the reference's make_fragment)."""
    return Layout.col_major(shape)


def make_tiled_copy(atom: CopyAtom, layout_tv: Layout, tiler_mn) -> TiledCopy:
    """make_tiled_copy(atom, layout_tv, tiler_mn) (src/atom/copy.rs:178-207), with
    its three checks and their wording."""
    if layout_tv.rank() != 2:
        raise ValueError(f"cute: make_tiled_copy needs a (thread, value) layout, not {layout_tv}")
    threads, values = layout_tv.mode(0).size(), layout_tv.mode(1).size()
    if threads % atom.num_threads():
        raise ValueError(f"cute: a tiled copy of {threads} threads cannot be built from a {atom.op!r} atom of "
                         f"{atom.num_threads()} threads")
    if values % atom.num_val_ref():
        raise ValueError(f"cute: each thread's {values} values must be a multiple of the {atom.op!r} atom's {atom.num_val_ref()}")
    tile = _tiler_size(tiler_mn)
    if layout_tv.cosize() > tile:
        raise ValueError(f"cute: layout_tv {layout_tv} reaches index {layout_tv.cosize() - 1} outside the {tile}-element tile")
    return TiledCopy(atom, _tiler_shape(tiler_mn), threads, values, lambda t, v: layout_tv(t + threads * v), tiler_mn=tiler_mn)


def make_tiled_copy_tv(atom: CopyAtom, thr_layout: Layout, val_layout: Layout) -> TiledCopy:
    """make_tiled_copy_tv (src/atom/copy.rs:210-214): `thr_layout` threads each
    moving `val_layout` values; the values of one instruction must be contiguous
    in the value layout's fastest mode."""
    tile, f = make_layout_tv(thr_layout, val_layout)
    threads, values = thr_layout.size(), val_layout.size()
    if threads % atom.num_threads():
        raise ValueError(f"cute: a tiled copy of {threads} threads cannot be built from a {atom.op!r} atom of "
                         f"{atom.num_threads()} threads")
    if values % atom.num_val_ref():
        raise ValueError(f"cute: each thread's {values} values must be a multiple of the {atom.op!r} atom's {atom.num_val_ref()}")
    return TiledCopy(atom, tile, threads, values, f)


def make_tiled_copy_c(atom: CopyAtom, mma: TiledMma) -> TiledCopy:
    """A tiled copy matching the accumulator fragments of `mma` (src/atom/copy.rs:229-232)."""
    c = mma.layout_c_tv()
    m, n, _ = mma.atom.shape_mnk
    return make_tiled_copy(atom, c, (m, n))


def make_tiled_copy_s(atom: CopyAtom, tiled: TiledCopy) -> TiledCopy:
    """`atom` partitioned like the source side of `tiled` (src/atom/copy.rs:234-239)."""
    return TiledCopy(atom, tiled.tile_shape_, tiled.threads, tiled.values, tiled._src_tv, tiler_mn=tiled.tiler_mn_)


def make_tiled_copy_d(atom: CopyAtom, tiled: TiledCopy) -> TiledCopy:
    """`atom` partitioned like the destination side of `tiled` (src/atom/copy.rs:241-246)."""
    return TiledCopy(atom, tiled.tile_shape_, tiled.threads, tiled.values, tiled._tv, tiler_mn=tiled.tiler_mn_)


def make_tiled_copy_c_atom(atom: CopyAtom, mma: TiledMma) -> TiledCopy:
    """The smallest tiled copy that retiles `mma`'s accumulators at `atom`'s
    granularity (src/atom/copy.rs:248-273): each thread keeps the first
    `atom` values of its accumulator fragment, in the fragment's order; the
    tiler is, per mode, the layout of the C coordinates those values touch, and
    the (thread, value) layout indexes the tile the tiler selects."""
    c_tv = mma.layout_c_tv()
    threads, mma_v, copy_v = c_tv.mode(0).size(), c_tv.mode(1).size(), atom.num_val_src()
    if copy_v > mma_v:
        raise ValueError(f"cute: the copy atom's {copy_v} source values are more than the {mma_v} accumulators per thread of the MMA")
    m_ext, n_ext, _ = mma.atom.shape_mnk
    # the truncated (thread, value) domain keeps the hierarchy of the thread mode; the value mode becomes flat
    dom = (c_tv.shape[0], copy_v)
    f = lambda i: c_tv((i % threads) + threads * (i // threads))  # i < threads * copy_v
    tiler_m = Layout.with_strides_of(dom, lambda i: f(i) % m_ext).filter()
    tiler_n = Layout.with_strides_of(dom, lambda i: f(i) // m_ext).filter()
    # tile coordinate -> index into the MMA's C tile, inverted
    back = {}
    for j in range(tiler_n.size()):
        for i in range(tiler_m.size()):
            back[tiler_m(i) + m_ext * tiler_n(j)] = i + tiler_m.size() * j
    layout_tv = Layout.with_strides_of(dom, lambda i: back[f(i)])
    return make_tiled_copy(atom, layout_tv, (tiler_m, tiler_n))


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


# --------------------------------------------------------------------------- #
# copy / copy_if / autovec_copy: which instructions a copy breaks into          #
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class TensorView:
    """What `copy` needs to know about a tensor: its layout (mode 0 holds the
    values one thread moves), the element offset of its first element, and whether
    it lives in registers (register tensors take any vector width)."""
    layout: Layout
    base_offset: int = 0
    register: bool = False

    def size(self) -> int:
        return self.layout.size()


@dataclass(frozen=True)
class CopyChunk:
    """One instruction of a copy: `values` elements from `src` to `dst` (element
    offsets including the tensors' bases); `pred` is the offset of the flag that
    guards it (copy_if), or None."""
    op: object
    values: int
    src: int
    dst: int
    pred: int = None


def _chunks(layout: Layout, v: int, what: str):
    m0 = layout.mode(0) if layout.rank() > 1 or isinstance(layout.shape, tuple) else layout
    if m0.size() % v:
        raise ValueError(f"copy: {what} mode 0 ({m0}) is not a multiple of the atom's {v} values")
    per_row = m0.size()
    starts = []
    for i in range(0, layout.size(), v):
        starts.append(layout(i))
    atom_offsets = [m0(i) for i in range(v)]
    return atom_offsets, starts, per_row


def _check_vector_access(t: TensorView, atom_offsets, start: int, what: str, op) -> None:
    v = len(atom_offsets)
    if v == 1:
        return
    if atom_offsets != list(range(v)):
        raise ValueError(f"copy: {op!r} needs {v} contiguous {what} elements per thread, but they are laid out as "
                         f"{Layout.from_values(atom_offsets) if atom_offsets[0] == 0 else atom_offsets}")
    if not t.register and (t.base_offset + start) % v:
        raise ValueError(f"copy: cannot prove that the {what} offset {t.base_offset + start} is aligned to {v} elements for {op!r}")


def _copy_impl(atom: CopyAtom, src: TensorView, dst: TensorView, pred: TensorView = None):
    sv, dv = atom.num_val_src(), atom.num_val_dst()
    s_atom, s_starts, _ = _chunks(src.layout, sv, "source")
    d_atom, d_starts, _ = _chunks(dst.layout, dv, "destination")
    if len(s_starts) != len(d_starts):
        raise ValueError(f"copy: source {src.layout} and destination {dst.layout} split into different numbers of {atom.op!r} chunks")
    p_starts = _chunks(pred.layout, sv, "predicate")[1] if pred is not None else None
    out = []
    for c, (so, do) in enumerate(zip(s_starts, d_starts)):
        _check_vector_access(src, s_atom, so, "source", atom.op)
        _check_vector_access(dst, d_atom, do, "destination", atom.op)
        out.append(CopyChunk(atom.op, sv, src.base_offset + so, dst.base_offset + do,
                             None if p_starts is None else pred.base_offset + p_starts[c]))
    return out


def copy(atom, src: TensorView, dst: TensorView):
    """cute.copy (src/atom/copy.rs:482-488): both tensors are split into atom-sized
    chunks along mode 0 and the remaining modes are iterated.  Returns the
    instructions in issue order; raises with the reference's messages when a chunk is
    not contiguous or its alignment cannot be shown."""
    return _copy_impl(atom.atom if isinstance(atom, TiledCopy) else atom, src, dst)


def copy_if(atom, pred: TensorView, src: TensorView, dst: TensorView):
    """cute.copy with one flag per source element, of which the first of every
    chunk is consulted (src/atom/copy.rs:490-498)."""
    if pred.size() != src.size():
        raise ValueError("copy_if: predicate tensor must have one flag per source element")
    return _copy_impl(atom.atom if isinstance(atom, TiledCopy) else atom, src, dst, pred)


def _vectorizable(t: TensorView, v: int) -> bool:
    if t.register:
        return True
    n = t.layout.size()
    m0 = t.layout.mode(0).size() if isinstance(t.layout.shape, tuple) else n
    if m0 % v:
        return False
    for start in range(0, n, v):
        base = t.layout(start)
        if any(t.layout(start + i) != base + i for i in range(v)) or (t.base_offset + base) % v:
            return False
    return True


def autovec_copy(dtype: DType, src: TensorView, dst: TensorView):
    """Element-wise copy with the widest vectors both tensors allow, at most 128
    bits (src/atom/copy.rs:500-513): the width halves until every chunk of both
    tensors is contiguous and aligned."""
    if src.size() != dst.size():
        raise ValueError("autovec_copy: tensors have different sizes")
    bits = max(dtype.bytes() * 8, 8)
    flat = lambda t: TensorView(Layout((t.size(),), (1,)) if t.register else _flat_view(t.layout), t.base_offset, t.register)
    s1, d1 = flat(src), flat(dst)
    v = 128 // bits
    while v > 1 and not (_vectorizable(s1, v) and _vectorizable(d1, v)):
        v //= 2
    return _copy_impl(CopyAtom(dtype, CopyOp.Universal(v * bits)), s1, d1)


class _flat_view(Layout):
    """A layout seen as one mode of its size (as_1d, src/atom/copy.rs:524-527)."""

    def __init__(self, inner: Layout):
        self._inner = inner
        self.shape, self.stride = (inner.size(),), (None,)

    def size(self) -> int:
        return self._inner.size()

    def __call__(self, index: int) -> int:
        return self._inner(index)

    def mode(self, i: int):
        return self

    def rank(self) -> int:
        return 1

    def __repr__(self):
        return f"flat({self._inner})"
