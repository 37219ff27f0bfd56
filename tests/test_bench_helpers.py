"""bench.py's own checker: the band comparison against the oracle accepts a correct
result (computed here in float64 and rounded to bf16) and rejects a wrong one."""
import importlib.util
import os

import numpy as np

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_band_check_accepts_right_and_rejects_wrong_results():
    bench = _bench()
    rng = np.random.default_rng(5)
    m, n, k = 96, 80, 256
    a = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (m, k)).astype(np.float32))
    b = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    exact = oracle.bf16_bits_to_f32(a).astype(np.float64) @ oracle.bf16_bits_to_f32(b).astype(np.float64).T
    c = oracle.f32_to_bf16_bits(exact.astype(np.float32))
    bands = bench.three_bands(m, height=16)
    assert bands == [(0, 16), (48, 64), (80, 96)]
    chk = bench.BandCheck(a, b, bands, k)
    good = chk.check(c, 0)
    assert good["ok"] and good["rows_checked"] == 48 and good["max_excess"] <= 0
    sub = bench.BandCheck(a, b, [(48, 64)], k)
    assert sub.check(c[40:70], 40)["ok"]
    bad = c.copy()
    bad[50, 7] ^= 0x0100  # one element, a few units of the last place off
    res = chk.check(bad, 0)
    assert not res["ok"] and res["max_excess"] > 0
    assert bench.three_bands(40) == [(0, 40)]
