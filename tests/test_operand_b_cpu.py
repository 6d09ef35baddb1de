"""The second-operand layout (the fork's InitSparseMatrixA_bitmap_v6_B) on the CPU: the oracle's restatement against the
fixtures produced by the compiled reference (tests/golden/operand_b), against the compiled reference itself where
it is built, and the decode round trip."""
import glob
import os

import numpy as np
import pytest

import oracle
from conftest import make_sparse

GOLDEN_B = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "operand_b", "*.npz")))
FIELDS = ("vals", "tile_nnz", "mtile", "gtile", "bitmap")


def test_fixtures_present():
    assert len(GOLDEN_B) >= 7


@pytest.mark.parametrize("path", GOLDEN_B, ids=[os.path.basename(p) for p in GOLDEN_B])
def test_restatement_matches_the_reference_fixtures(path):
    d = np.load(path)
    e = oracle.encode_b(d["A"])
    for f in FIELDS:
        assert np.array_equal(getattr(e, f), d[f]), f
    assert e.max_nnz == int(d["max_nnz"])
    assert np.array_equal(oracle.decode_b(e), np.where((d["A"] & 0x7FFF) == 0, 0, d["A"]))   # -0 comes back as +0


@pytest.mark.skipif(not oracle.have_ref_b(), reason="compiled reference encoder absent")
@pytest.mark.parametrize("M,K,s,seed", [(64, 64, 0.5, 1), (256, 128, 0.6, 2), (128, 512, 0.95, 3), (320, 192, 0.3, 4)])
def test_restatement_matches_the_compiled_reference(M, K, s, seed):
    A = make_sparse(M, K, s, seed)
    a, b = oracle.encode_b(A), oracle.ref_encode_b(A)
    for f in FIELDS:
        assert np.array_equal(getattr(a, f), getattr(b, f)), f
    assert a.max_nnz == b.max_nnz


def test_layout_differs_from_the_weight_layout_only_in_tile_order():
    A = make_sparse(128, 128, 0.6, 9)
    w, b = oracle.encode(A), oracle.encode_b(A)
    assert np.array_equal(w.gtile, b.gtile) and w.max_nnz == b.max_nnz        # same counts per global tile
    assert sorted(w.bitmap.tolist()) == sorted(b.bitmap.tolist())              # same tiles, another order
    assert not np.array_equal(w.bitmap, b.bitmap)
    assert b.mtile.size == 4 * w.mtile.size
