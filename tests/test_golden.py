"""The CPU oracle against outputs of pocket-engine's own kernels (tests/golden/reference_kernels.npz, made on
a B200 by tests/golden/make_golden.py). No GPU needed here."""
import os
import sys

import numpy as np
import pytest

import harness

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURE = os.path.join(HERE, "golden", "reference_kernels.npz")


@pytest.mark.skipif(not os.path.exists(FIXTURE), reason="fixture not generated yet")
def test_oracle_matches_the_reference_kernels_outputs(pe, oracle):
    sys.path.insert(0, os.path.join(HERE, "golden"))
    import make_golden
    from pocket_engine_b200 import workloads
    gold = np.load(FIXTURE)
    for name, wl in make_golden.cases(pe, workloads).items():
        table, _ = harness.oracle_registry(wl)
        tiles = oracle.fill_tiles(wl.row_n, wl.row_slot, wl.tokens // 16 + wl.n_seqs)
        y64 = harness.oracle_f64(wl, table, tiles)
        emul32 = harness.oracle_rounded(wl, table, tiles, True, pe, mode="emul")
        emul16 = harness.oracle_rounded(wl, table, tiles, False, pe, mode="emul")
        for si in range(len(wl.sites)):
            ref32 = gold[f"{name}.site{si}.f32"]
            # the reference's own kernels sit inside the stated tolerance of the fp64 oracle ...
            mx, mn = harness.tolerance(ref32, y64[si])
            assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, (name, si, mx, mn)
            # ... and within rounding of the oracle's emulation of their rounding points
            mx, mn = harness.tolerance(ref32, emul32[si].astype(np.float64))
            assert mx <= 1e-3 and mn <= 5e-5, (name, si, mx, mn)
            ref16 = pe.bf16_to_f32(gold[f"{name}.site{si}.bf16"]).reshape(emul16[si].shape)
            ulp = harness.bf16_ulp_diff(ref16, emul16[si], pe, floor=5e-4)
            assert ulp.max() <= 1 and (ulp > 0).mean() < 5e-3, (name, si, int(ulp.max()))
            # rows no tile covers are untouched, bit for bit
            base = wl.y_base(si)
            tslot = wl.token_slot()
            assert np.array_equal(ref32[tslot == 0], base[tslot == 0])
