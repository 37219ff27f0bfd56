"""The protocol checker on the GEMM kernel's schedule: every tiling the library
instantiates is clean, and each deliberate protocol bug is reported as the kind
of error the reference's simulator reports for it (tests/diagnostics.rs)."""
import pytest

from cute_rs_b200.check import ProtocolError, check_cluster_sum, check_gemm, check_signal, tiling_from_library

TILINGS = [dict(cta_group=g, stages=s, mh=mh, acc_bufs=ab, kps=kps) for g, s, mh, ab, kps in
           [(2, 4, 2, 1, 1), (1, 3, 2, 1, 1), (2, 7, 1, 2, 1), (1, 4, 1, 2, 1), (2, 9, 1, 2, 1), (2, 5, 2, 2, 1), (1, 7, 1, 2, 1),
            (2, 3, 1, 2, 4), (1, 3, 1, 2, 2), (2, 4, 1, 2, 2)]]


@pytest.mark.parametrize("tiling", TILINGS)
@pytest.mark.parametrize("units", [(1,), (8, 8, 8), (3, 5, 2, 7, 1), (13,) * 5, (4, 0, 4), (0, 0), (2, 2, 2, 2, 2, 2, 2)])
def test_kernel_protocol_is_clean(tiling, units):
    check_gemm(units=units, **tiling)


@pytest.mark.parametrize("units,chunks", [((8, 8, 8), 0), ((3, 5, 2, 7, 1), 0), ((13,) * 5, 0), ((4, 0, 4), 0), ((26, 1, 30), 0),
                                          ((8, 8, 8), None), ((4, 0, 4), None)])
def test_every_compiled_tiling_is_clean(lib, units, chunks):
    """The schedule run with the ring depth, stage bytes, accumulator buffering,
    barrier arrival counts and transaction bytes that the compiled kernel uses
    (cute_b200_gemm_layout_info), for every tiling the library instantiates; with
    chunks None the pusher runs too, with the kernel's chunks per tile."""
    for g, tile_n, tile_m in lib.GEMM_TILINGS:
        info = lib.gemm_layout_info(g, tile_n, tile_m)
        push = info.push_chunks_per_tile if chunks is None else chunks
        check_gemm(units=units, push_chunks=push, seeds=range(2), **tiling_from_library(info, g))


def test_wrong_barrier_constants_would_be_seen(lib):
    """What the tie to the library buys: were the kernel built with an arrival count
    that forgets the second CTA of a pair, or with a transaction count of one CTA's
    bytes, the schedule run with those constants fails."""
    info = lib.gemm_layout_info(2, 256, 256)
    good = tiling_from_library(info, 2)
    check_gemm(units=(8, 8, 8), **good)
    with pytest.raises(ProtocolError):
        check_gemm(units=(8, 8, 8), **dict(good, tmem_empty_arrivals=info.tmem_empty_arrivals // 2))
    with pytest.raises(ProtocolError):
        check_gemm(units=(8, 8, 8), **dict(good, expect_tx=info.full_expect_tx_bytes_per_k_block // 2))
    with pytest.raises(ProtocolError):
        check_gemm(units=(8, 8, 8), **dict(good, tmem_empty_arrivals=info.tmem_empty_arrivals + 1))


@pytest.mark.parametrize("mutation,kind", [
    ("producer_skips_empty_wait", ("race", "arrive")),  # write-after-read on a ring stage, or an arrival into a full phase
    ("mma_skips_full_wait", ("race", "uninitialised")),  # read before the copy is known to have landed
    ("mma_skips_tmem_wait", "race"),         # accumulator overwritten while the epilogue reads it
    ("epilogue_arrives_early", "race"),
    ("expect_tx_short", ("tx", "race", "uninitialised")),  # the phase completes before the peer's bytes: early read, or surplus bytes
    ("wrong_empty_parity", ("parity", "deadlock")),
    ("no_peer_commit", "deadlock"),          # the peer CTA's producer never sees its stages released
])
def test_protocol_bugs_are_reported(mutation, kind):
    kinds = (kind,) if isinstance(kind, str) else kind
    with pytest.raises(ProtocolError) as e:
        check_gemm(cta_group=2, stages=4, mh=2, acc_bufs=1, units=(8, 8, 8), mutations=(mutation,))
    assert e.value.kind in kinds, str(e.value)


def test_single_cta_mutations():
    for mutation in ("producer_skips_empty_wait", "mma_skips_tmem_wait", "epilogue_arrives_early"):
        with pytest.raises(ProtocolError):
            check_gemm(cta_group=1, stages=4, mh=1, acc_bufs=2, units=(6,) * 6, mutations=(mutation,))


# ---- the pusher of the several-destination form ------------------------------------------
@pytest.mark.parametrize("tiling", TILINGS)
@pytest.mark.parametrize("units,chunks", [((8, 8, 8), 8), ((1,), 4), ((3, 5, 2, 7, 1), 2), ((4, 0, 4), 8), ((2,) * 7, 4)])
def test_pusher_protocol_is_clean(tiling, units, chunks):
    check_gemm(units=units, push_chunks=chunks, **tiling)


@pytest.mark.parametrize("mutation,kind", [
    ("epilogue_signals_early", "race"),                 # the TMA load reads a part of C that is still being stored
    ("pusher_skips_tile_wait", ("race", "uninitialised")),
    ("pusher_skips_load_wait", "race"),                 # the store reads the staging buffer while the load fills it
    ("pusher_skips_read_wait", "race"),                 # the next load overwrites a buffer a store still reads
    ("pusher_wrong_parity", ("parity", "deadlock")),
])
def test_pusher_bugs_are_reported(mutation, kind):
    kinds = (kind,) if isinstance(kind, str) else kind
    with pytest.raises(ProtocolError) as e:
        check_gemm(cta_group=2, stages=4, mh=2, acc_bufs=1, units=(4, 4, 4, 4), push_chunks=4, mutations=(mutation,))
    assert e.value.kind in kinds, str(e.value)


def test_one_shared_tile_count_is_a_race_when_a_warp_falls_behind():
    """The kernel publishes one tile count per epilogue warp.  With a single shared
    count a warp that has handed its accumulator back but not yet stored its part
    is covered by a faster warp's count for the next tile: the checker shows it
    once that warp is held back, and shows the per-warp slots to be safe."""
    from cute_rs_b200.check import gemm_schedule, run

    def held_back(mutations):
        programs, barriers = gemm_schedule(push_chunks=2, units=(2, 2, 2), mutations=mutations)
        slow = "epilogue0.3"
        pc = next(i for i, op in enumerate(programs[slow]) if op[0] == "st")
        for seed in range(8):
            run(programs, barriers, seed=seed, stalls={slow: (pc, 100)})

    held_back(())
    with pytest.raises(ProtocolError) as e:
        held_back(("shared_tile_counter",))
    assert e.value.kind in ("uninitialised", "race")


# ---- completion counters of the several-destination form ----------------------------------
@pytest.mark.parametrize("ctas,chunks", [(1, 1), (4, 3), (8, 2)])
def test_completion_signal_protocol_is_clean(ctas, chunks):
    check_signal(ctas=ctas, chunks=chunks)


@pytest.mark.parametrize("mutation,kind", [
    ("signal_without_store_wait", ("race", "uninitialised")),   # the owner reads rows whose bulk store may not have landed
    ("signal_before_all_ctas", ("race", "uninitialised")),      # ... rows of the CTA that was not waited for
    ("peer_reads_without_waiting", ("race", "uninitialised")),
    ("peer_expects_another_sender", "deadlock"),                # what the bounded wait turns into a reported timeout
])
def test_completion_signal_bugs_are_reported(mutation, kind):
    kinds = (kind,) if isinstance(kind, str) else kind
    with pytest.raises(ProtocolError) as e:
        check_signal(ctas=4, chunks=3, mutations=(mutation,), seeds=range(12))
    assert e.value.kind in kinds, str(e.value)


# ---- the k split summed inside a cluster ---------------------------------------------------
@pytest.mark.parametrize("kc,warps", [(2, 8), (4, 8), (2, 1)])
def test_cluster_sum_protocol_is_clean(kc, warps):
    check_cluster_sum(kc=kc, warps=warps)


@pytest.mark.parametrize("mutation,kind", [
    ("sum_before_barrier", ("race", "uninitialised")),    # partial sums of another CTA read before they are written
    ("barrier_of_one_cta", ("race", "uninitialised")),
    ("exit_without_barrier", ("race", "uninitialised")),  # a CTA's shared memory reused while a peer still reads it
    ("a_warp_skips_barrier", "deadlock"),
])
def test_cluster_sum_bugs_are_reported(mutation, kind):
    kinds = (kind,) if isinstance(kind, str) else kind
    with pytest.raises(ProtocolError) as e:
        check_cluster_sum(kc=2, warps=4, mutations=(mutation,), seeds=range(12))
    assert e.value.kind in kinds, str(e.value)
