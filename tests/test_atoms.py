"""The atom API: the facts the reference's own tests pin (tests/atoms.rs,
src/layout/tests.rs) and the sm_100a atoms against the hand-written kernels."""
import pytest

from cute_rs_b200.atom import (CopyOp, Layout, MmaF16BF16Op, Sm100UmmaOp, UniversalFma, make_copy_atom, make_fragment,
                               make_layout_tv, make_mma_atom, make_tiled_copy, make_tiled_copy_a, make_tiled_copy_b,
                               make_tiled_copy_c, make_tiled_copy_c_atom, make_tiled_copy_d, make_tiled_copy_s,
                               make_tiled_copy_tv, make_tiled_mma, sw128_descriptor, sw128_offset, TensorView, autovec_copy, copy,
                               copy_if)
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


def test_tiled_copy_s_and_d_reuse_the_layouts_with_another_atom():
    # tests/atoms.rs:47-52
    mma = single_warp_mma()
    ldsm = make_tiled_copy_a(make_copy_atom(DType.F16, CopyOp.LdMatrix(4)), mma)
    s = make_tiled_copy_s(make_copy_atom(DType.F16, CopyOp.Universal(128)), ldsm)
    d = make_tiled_copy_d(make_copy_atom(DType.F16, CopyOp.Universal(32)), ldsm)
    a = mma.layout_a_tv()
    for lane in range(32):
        for v in range(8):
            assert s.layout_tv_tiled(lane, v) == ldsm.layout_src_tv_tiled(lane, v)
            assert d.layout_tv_tiled(lane, v) == a(lane + 32 * v)
    assert s.tiler_mn() == ldsm.tiler_mn() == (16, 16) and s.atom.op == CopyOp.Universal(128)
    c = make_tiled_copy_c(make_copy_atom(DType.F32, CopyOp.Universal(64)), mma)
    assert (c.size(), c.tile_shape()) == (32, (16, 8))
    assert all(c.layout_tv_tiled(t, v) == mma.layout_c_tv()(t + 32 * v) for t in range(32) for v in range(4))


def test_tiled_copy_c_atom_is_the_smallest_c_copy():
    # tests/atoms.rs:54-66: an m16n8 accumulator and a two-value atom: each thread keeps c0 and c1 (row g,
    # columns 2t and 2t + 1), so the tile is rows 0..8 and all 8 columns, in the order (t, c0/c1)
    c = make_tiled_copy_c_atom(make_copy_atom(DType.F32, CopyOp.Universal(64)), single_warp_mma())
    assert c.layout_tv(((4, 8), 2)) == Layout(((4, 8), 2), ((8, 1), 32))
    assert c.layout_tv() == Layout(((4, 8), 2), ((8, 1), 32))
    assert c.tiler_mn() == (Layout(8, 1), Layout((4, 2), (2, 1)))
    assert c.tile_shape() == (8, (4, 2))
    # the values a thread keeps are its first accumulators: coordinates (lane / 4, 2 * (lane % 4) + v)
    tm, tn = c.tiler_mn()
    for lane in range(32):
        for v in range(2):
            idx = c.layout_tv_tiled(lane, v)
            assert (tm(idx % 8), tn(idx // 8)) == (lane // 4, 2 * (lane % 4) + v)
    with pytest.raises(ValueError, match="more than the 4 accumulators"):
        make_tiled_copy_c_atom(make_copy_atom(DType.F32, CopyOp.Universal(256)), single_warp_mma())


def test_retile_follows_the_copy_value_order():
    # tests/atoms.rs:68-92
    atom = make_copy_atom(DType.F16, CopyOp.LdMatrix(4))
    # threads 8 x 4, each with a 4 x 2 block (columns fastest): copy value w is row w / 2, column w % 2
    tiled = make_tiled_copy_tv(atom, Layout.row_major((8, 4)), Layout.row_major((4, 2)))
    r = tiled.retile(make_fragment((2, 4)))
    assert r.size() == 8 and r.values() == list(range(8))
    # the same fragment stored row by row: value w is slot 4 * (w % 2) + w / 2
    assert tiled.retile(Layout((2, 4), (4, 1))).values() == [0, 4, 1, 5, 2, 6, 3, 7]
    # an MMA fragment retiled for the ldmatrix copy built from the same MMA keeps its value order and
    # its (MMA_M, MMA_K) modes
    ldsm = make_tiled_copy_a(atom, single_warp_mma())
    view = ldsm.retile(make_fragment((8, 4, 2)))
    assert view.rank() == 3 and (view.mode(1).size(), view.mode(2).size()) == (4, 2)
    assert view.values() == list(range(64))


def test_tiled_copy_misuse_is_rejected():
    # tests/atoms.rs:94-108
    atom = make_copy_atom(DType.F16, CopyOp.LdMatrix(4))
    with pytest.raises(ValueError) as e:
        make_tiled_copy_tv(atom, Layout.row_major((4, 4)), Layout.col_major(8))
    assert "16 threads" in str(e.value) and "32 threads" in str(e.value)
    with pytest.raises(ValueError, match="multiple of"):
        make_tiled_copy_tv(atom, Layout.row_major((8, 4)), Layout.col_major(4))
    with pytest.raises(ValueError, match="outside the 64-element tile"):
        make_tiled_copy(make_copy_atom(DType.F32, CopyOp.Universal(32)), Layout((32, 4), (1, 32)), (8, 8))


def test_copy_breaks_into_the_instructions_of_the_elementwise_example():
    """examples/elementwise_add.rs:60-79: a thread's 4 x 4 values of a row-major (M, 512) tensor move as
    four 128-bit accesses, one per row; copy_if consults the first flag of each; autovec_copy finds
    the same width by itself and narrows it when the base is less aligned (src/atom/copy.rs:500-588)."""
    n = 512
    g = TensorView(Layout((4, 4), (1, n)), base_offset=3 * n + 8)
    r = TensorView(Layout.col_major((4, 4)), register=True)
    atom = make_copy_atom(DType.F32, CopyOp.Universal(128))
    plan = copy(atom, g, r)
    assert [(c.src, c.dst, c.values) for c in plan] == [(3 * n + 8 + i * n, 4 * i, 4) for i in range(4)]
    flags = TensorView(Layout.col_major((4, 4)), register=True)
    assert [c.pred for c in copy_if(atom, flags, g, r)] == [0, 4, 8, 12]
    assert [(c.values, c.dst) for c in autovec_copy(DType.F32, r, g)] == [(4, 3 * n + 8 + i * n) for i in range(4)]
    narrow = autovec_copy(DType.F32, r, TensorView(Layout((4, 4), (1, n)), base_offset=2))
    assert len(narrow) == 8 and narrow[0].values == 2 and narrow[0].op == CopyOp.Universal(64)
    with pytest.raises(ValueError, match="needs 4 contiguous source elements"):
        copy(atom, TensorView(Layout((4, 4), (n, 1))), r)
    with pytest.raises(ValueError, match="cannot prove that the source offset 2 is aligned to 4 elements"):
        copy(atom, TensorView(Layout((4, 4), (1, n)), base_offset=2), r)
    with pytest.raises(ValueError, match="is not a multiple of the atom's 4 values"):
        copy(atom, TensorView(Layout((2, 4), (1, n))), TensorView(Layout.col_major((2, 4)), register=True))
    with pytest.raises(ValueError, match="one flag per source element"):
        copy_if(atom, TensorView(Layout(4, 1), register=True), g, r)


def test_layout_recovered_from_values():
    for l in (Layout((4, 8, 2), (8, 1, 32)), Layout((2, 4), (4, 1)), Layout(8, 3), Layout((2, 2, 2), (1, 16, 4))):
        assert Layout.from_values(l.values()).values() == l.values()
    assert Layout.from_values([0, 4, 1, 5, 2, 6, 3, 7]) == Layout((2, 4), (4, 1))
    assert Layout(((4, 8), 2), ((0, 1), 0)).filter() == Layout(8, 1)
    assert Layout(((4, 8), 2), ((2, 0), 1)).filter() == Layout((4, 2), (2, 1))
    with pytest.raises(ValueError):
        Layout.from_values([0, 1, 3, 4, 5])


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


def test_sm100_atoms_match_the_compiled_kernel(lib):
    """The atoms against the library's own account of every tiling it instantiates
    (cute_b200_gemm_layout_info evaluates the expressions the kernel is compiled from):
    instruction descriptor, shared-memory descriptor and its k step, TMA box bytes, the
    ring that fits, TMEM columns, the pusher's chunk."""
    for g, tile_n, tile_m in lib.GEMM_TILINGS:
        for ab, dt in ((lib.F16, DType.F16), (lib.BF16, DType.BF16)):
            for cdt, c_bytes in ((lib.F32, 4), (lib.BF16, 2)):
                info = lib.gemm_layout_info(g, tile_n, tile_m, ab, cdt, smem_addr=0x4400)
                op = Sm100UmmaOp(dt, min(tile_m, 128) * g, tile_n, cta_group=g)
                assert info.instruction_descriptor == op.instruction_descriptor(), (g, tile_n, tile_m)
                assert (info.umma_m, info.umma_n, info.umma_k) == (op.m, op.n, op.shape_k)
                assert info.smem_descriptor == sw128_descriptor(0x4400)
                assert sw128_descriptor(0x4400 + 2 * info.umma_k) - sw128_descriptor(0x4400) == info.descriptor_k_step
                # one stage = the A box and this CTA's share of the B box, 64 k each (one 128-byte swizzle row)
                assert info.block_k * 2 == CopyOp.TmaLoad(rows=1).swizzle_bytes
                assert info.a_block_bytes == CopyOp.TmaLoad(rows=info.cta_rows).box_bytes
                assert info.b_block_bytes == CopyOp.TmaLoad(rows=tile_n // g).box_bytes
                assert info.stage_bytes == info.k_blocks_per_stage * (info.a_block_bytes + info.b_block_bytes)
                assert info.full_expect_tx_bytes_per_k_block == g * (info.a_block_bytes + info.b_block_bytes)
                assert info.k_blocks_per_stage in (1, 2, 4) and 16 * 1024 <= info.stage_bytes <= 64 * 1024
                assert info.stages == min(192 * 1024 // info.stage_bytes, 12) and info.stages * info.stage_bytes <= 192 * 1024
                assert info.cta_rows == tile_m and info.accumulator_halves == max(tile_m // 128, 1)
                assert info.half_columns == op.tmem_columns
                cols = info.accumulator_halves * info.half_columns * info.accumulator_buffers
                assert cols <= info.tmem_columns <= 512 and info.tmem_columns in (128, 256, 512)
                assert info.accumulator_buffers == (2 if 2 * info.accumulator_halves * info.half_columns <= 512 else 1)
                # the last accumulator element sits inside the allocation
                cta, lane, col = op.tmem_coord(op.m - 1, op.n - 1, column0=(info.accumulator_halves - 1) * info.half_columns)
                assert cta == g - 1 and lane == 127 and col < info.tmem_columns
                # the epilogue warps cover the 128 lanes; one TMEM read is 32 lanes x 32 columns
                assert info.epilogue_warps % 4 == 0 and info.threads == 32 * (2 + info.epilogue_warps + 1)
                assert info.half_columns % (CopyOp.TmemLoad().columns * (info.epilogue_warps // 4)) == 0
                store = CopyOp.TmaStore(rows=info.push_chunk_rows, cols=tile_n, elem_bytes=c_bytes)
                assert store.box_bytes == info.push_chunk_bytes == 16384
                assert info.push_chunks_per_tile * info.push_chunk_rows == info.cta_rows
                assert info.shared_memory_bytes <= 227 * 1024
    with pytest.raises(lib.CuteB200Error):
        lib.gemm_layout_info(1, 128, 64)  # the 64-row tile is a pair tile


def test_sm100_umma_atom():
    op = Sm100UmmaOp(DType.BF16, 256, 256, cta_group=2)
    assert op.instruction_descriptor() == 0x10400490
    half = Sm100UmmaOp(DType.BF16, 128, 128, cta_group=2)  # 64 rows per CTA
    assert (half.rows_per_cta, half.tmem_columns) == (64, 64)
    assert half.tmem_coord(70, 5) == (1, 6, 5) and half.tmem_coord(70, 64 + 5, column0=64) == (1, 64 + 6, 64 + 5)
    assert Sm100UmmaOp(DType.F16, 128, 128).instruction_descriptor() == (1 << 4) | (16 << 17) | (8 << 24)
    assert op.tmem_coord(130, 17, column0=256) == (1, 2, 273)
    assert make_mma_atom(op).shape_mnk == (256, 256, 16)
    with pytest.raises(ValueError):
        Sm100UmmaOp(DType.BF16, 256, 256, cta_group=1)
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
    assert tma.box_bytes == 32768 and CopyOp.TmaLoad(rows=128).box_bytes + tma.box_bytes == 48 * 1024  # one k block of the 512x256 tile
    # the pusher's chunk: BN columns of whole tile rows, 16 KiB per staging buffer, for bf16 and f32 C
    assert CopyOp.TmaStore(rows=32, cols=256, elem_bytes=2).box_bytes == 16384
    assert CopyOp.TmaStore(rows=16, cols=256, elem_bytes=4).box_bytes == 16384
    assert CopyOp.TmaStore(rows=64, cols=128, elem_bytes=2).box_bytes == 16384
    with pytest.raises(ValueError):
        CopyOp.TmaStore(rows=8, cols=260)
