"""The atom API: the facts the reference's own tests pin (tests/atoms.rs,
src/layout/tests.rs) and the sm_100a atoms against the hand-written kernels."""
import pytest

from cute_rs_b200.atom import (CopyOp, Layout, MmaF16BF16Op, Sm100UmmaOp, UniversalFma, make_copy_atom, make_layout_tv,
                               make_mma_atom, make_tiled_copy_a, make_tiled_copy_b, make_tiled_copy_tv, make_tiled_mma,
                               sw128_descriptor, sw128_offset)
from cute_rs_b200.host import DType


def single_warp_mma():
    return make_tiled_mma(MmaF16BF16Op(DType.F16, DType.F32, (16, 8, 16)), Layout.col_major((1,)))


def test_layout_evaluation():
    # CuTe documentation examples (src/layout/tests.rs:51-91)
    assert Layout((2, 3), (1, 2)).values() == [0, 1, 2, 3, 4, 5]
    assert Layout((2, 3), (3, 1)).values() == [0, 3, 1, 4, 2, 5]
    assert Layout((2, (2, 2)), (4, (2, 1))).values() == [0, 4, 2, 6, 1, 5, 3, 7]
    assert Layout.row_major((300, 512)).cosize() == 300 * 512 and Layout((4, 4), (1, 8)).cosize() == 28


def test_elementwise_tutorial_tv_layout():
    # thr (4,32) row-major x val (4,4) row-major -> ((32,4),(4,4)):((64,4),(16,1)) over a 16 x 128 tile
    # (src/layout/tests.rs:93-101, examples/elementwise_add.rs:40-42)
    tile, f = make_layout_tv(Layout.row_major((4, 32)), Layout.row_major((4, 4)))
    want = Layout(((32, 4), (4, 4)), ((64, 4), (16, 1)))
    assert tile == (16, 128)
    assert all(f(t, v) == want(t + 128 * v) for t in range(128) for v in range(16))
    copy = make_tiled_copy_tv(make_copy_atom(DType.F32, CopyOp.Universal(128)), Layout.row_major((4, 32)), Layout.row_major((4, 4)))
    assert (copy.size(), copy.tile_shape()) == (128, (16, 128))
    # the four values of one 128-bit access are contiguous along n (row-major memory)
    assert [copy.layout_tv_tiled(5, v) // 16 for v in range(4)] == [20, 21, 22, 23]


def test_copy_atom_introspection():
    ldsm = make_copy_atom(DType.F16, CopyOp.LdMatrix(4))
    assert ldsm.value_type() == DType.F16 and ldsm.thr_id == Layout(32, 1)
    assert ldsm.layout_src_tv == Layout((32, 8), (8, 1)) and ldsm.layout_dst_tv == Layout((32, (2, 4)), (2, (1, 64)))
    u = make_copy_atom(DType.F32, CopyOp.Universal(128))
    assert (u.value_type(), u.num_threads(), u.layout_src_tv.size()) == (DType.F32, 1, 4) and u.thr_id == Layout(1, 0)
    assert make_copy_atom(DType.F16, CopyOp.CpAsync(16)).layout_src_tv.size() == 8
    with pytest.raises(ValueError):
        make_copy_atom(DType.F32, CopyOp.LdMatrix(4))


def test_mma_atom_layouts_and_parameter_checks():
    atom = make_mma_atom(MmaF16BF16Op(DType.BF16, DType.F32, (16, 8, 16)))
    assert atom.a == Layout(((4, 8), (2, 2, 2)), ((32, 1), (16, 8, 128)))
    assert atom.b == Layout(((4, 8), (2, 2)), ((16, 1), (8, 64))) and atom.c == Layout(((4, 8), (2, 2)), ((32, 1), (16, 8)))
    assert make_mma_atom(UniversalFma(DType.F32)).shape_mnk == (1, 1, 1)
    with pytest.raises(ValueError, match="Float32 when 'ab_dtype' is BFloat16"):
        MmaF16BF16Op(DType.BF16, DType.F16, (16, 8, 16))
    with pytest.raises(ValueError, match=r"one of \(16,8,8\) or \(16,8,16\)"):
        MmaF16BF16Op(DType.F16, DType.F32, (16, 16, 16))


def test_tiled_copy_from_an_mma():
    # tests/atoms.rs:28-52
    mma = single_warp_mma()
    ldsm = make_tiled_copy_a(make_copy_atom(DType.F16, CopyOp.LdMatrix(4)), mma)
    assert (ldsm.size(), ldsm.tile_shape()) == (32, (16, 16))
    a = mma.layout_a_tv()
    for lane in range(32):
        for v in range(8):
            assert ldsm.layout_tv_tiled(lane, v) == a(lane + 32 * v)
            m, k = lane % 8 + 8 * ((lane // 8) % 2), 8 * (lane // 16) + v
            assert ldsm.layout_src_tv_tiled(lane, v) == m + 16 * k
    ldsb = make_tiled_copy_b(make_copy_atom(DType.F16, CopyOp.LdMatrix(2)), mma)
    assert ldsb.tile_shape() == (8, 16) and ldsb.layout_src_tv_tiled(9, 3) == 1 + 8 * 11


def test_tiled_mma_matches_the_restated_reference_kernel():
    """The 2 x 2 warp tiling of tensorop_gemm (examples/tensorop_gemm.rs:107) gives every thread the
    accumulator coordinates that oracle/ref_kernel_sm80.cu's epilogue writes."""
    mma = make_tiled_mma(MmaF16BF16Op(DType.F16, DType.F32, (16, 8, 16)), Layout.col_major((2, 2, 1)))
    assert mma.thr_layout_vmnk == Layout((32, 2, 2, 1), (1, 32, 64, 128)) and mma.size() == 128
    assert mma.tile_shape == (32, 16, 16)
    for tid in (0, 5, 37, 70, 127):
        lane, warp = tid % 32, tid // 32
        wm, wn = warp % 2, warp // 2
        want = []
        for j in range(8):
            for i in range(4):
                row, col = 32 * i + 16 * wm + lane // 4, 16 * j + 8 * wn + 2 * (lane % 4)
                want += [(row, col), (row, col + 1), (row + 8, col), (row + 8, col + 1)]
        assert mma.c_coords(tid, (128, 128)) == want
    # every element of the 128 x 128 tile is owned exactly once
    owned = [c for t in range(128) for c in mma.c_coords(t, (128, 128))]
    assert len(owned) == len(set(owned)) == 128 * 128


def test_sm100_umma_atom():
    op = Sm100UmmaOp(DType.BF16, 256, 256, cta_group=2)
    assert op.instruction_descriptor() == 0x10400490
    assert Sm100UmmaOp(DType.F16, 128, 128).instruction_descriptor() == (1 << 4) | (16 << 17) | (8 << 24)
    assert op.tmem_coord(130, 17, column0=256) == (1, 2, 273)
    assert make_mma_atom(op).shape_mnk == (256, 256, 16)
    with pytest.raises(ValueError):
        Sm100UmmaOp(DType.BF16, 128, 256, cta_group=2)
    with pytest.raises(ValueError):
        Sm100UmmaOp(DType.BF16, 128, 264)


def test_sm100_shared_memory_layout():
    # the 128-byte swizzle: 16-byte chunk c of row r is stored at chunk c ^ (r % 8)
    for r in (0, 1, 7, 8, 13, 127):
        for k in range(0, 64, 8):
            assert sw128_offset(r, k) == r * 128 + (((k // 8) ^ (r % 8)) * 16)
            assert sw128_offset(r, k + 3) == sw128_offset(r, k) + 6
    # a tile is a bijection onto its bytes and its pattern repeats every 8 rows (1024 bytes)
    offs = {sw128_offset(r, k) for r in range(128) for k in range(64)}
    assert len(offs) == 128 * 64 and max(offs) == 128 * 128 - 2
    assert all(sw128_offset(r + 8, k) == sw128_offset(r, k) + 1024 for r in range(8) for k in range(0, 64, 8))
    # descriptor fields; k advances by 16 elements = +2 in the address field
    d = sw128_descriptor(0x4400)
    assert d & 0x3FFF == 0x440 and (d >> 16) & 0x3FFF == 1 and (d >> 32) & 0x3FFF == 64 and (d >> 46) & 3 == 1 and d >> 61 == 2
    assert sw128_descriptor(0x4400 + 32) - d == 2
    tma = CopyOp.TmaLoad(rows=256)
    assert tma.box_bytes == 32768 and CopyOp.TmaLoad(rows=128).box_bytes + tma.box_bytes == 48 * 1024  # one 512x256 stage
    # the pusher's chunk: BN columns of whole tile rows, 16 KiB per staging buffer, for bf16 and f32 C
    assert CopyOp.TmaStore(rows=32, cols=256, elem_bytes=2).box_bytes == 16384
    assert CopyOp.TmaStore(rows=16, cols=256, elem_bytes=4).box_bytes == 16384
    assert CopyOp.TmaStore(rows=64, cols=128, elem_bytes=2).box_bytes == 16384
    with pytest.raises(ValueError):
        CopyOp.TmaStore(rows=8, cols=260)
