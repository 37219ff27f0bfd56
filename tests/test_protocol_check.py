"""The protocol checker on the GEMM kernel's schedule: every tiling the library
instantiates is clean, and each deliberate protocol bug is reported as the kind
of error the reference's simulator reports for it (tests/diagnostics.rs)."""
import pytest

from cute_rs_b200.check import ProtocolError, check_gemm

TILINGS = [dict(cta_group=g, stages=s, mh=mh, acc_bufs=ab) for g, s, mh, ab in
           [(2, 4, 2, 1), (1, 3, 2, 1), (2, 7, 1, 2), (1, 4, 1, 2), (2, 9, 1, 2), (2, 5, 2, 2), (1, 7, 1, 2)]]


@pytest.mark.parametrize("tiling", TILINGS)
@pytest.mark.parametrize("units", [(1,), (8, 8, 8), (3, 5, 2, 7, 1), (13,) * 5, (4, 0, 4), (0, 0), (2, 2, 2, 2, 2, 2, 2)])
def test_kernel_protocol_is_clean(tiling, units):
    check_gemm(units=units, **tiling)


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
