"""Loader of the on-disk weight format (spb_load_bin_files) against files written by the reference's own writer.

CPU only: the reference's Our_GenSparseMatrixBinFile (compiled unmodified into oracle/_ref) writes the six files,
the library reads them back, and the result must equal the oracle's encoding bit for bit.
"""
import os

import numpy as np
import pytest

import oracle
from conftest import make_sparse


@pytest.fixture(scope="module")
def sp(lib_built):
    import spmspm_b200
    return spmspm_b200


def _write_with_reference(tmp_path, A, name="w"):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference encoder) is not built")
    dense = tmp_path / f"{name}.bin"
    A.tofile(dense)
    prefix = str(tmp_path / name)
    oracle.ref_gen_bin_files(str(dense), A.shape[0], A.shape[1], prefix)
    return prefix


@pytest.mark.parametrize("M,K,s", [(64, 64, 0.5), (128, 192, 0.6), (192, 64, 0.9), (64, 128, 1.0), (64, 64, 0.0)])
def test_load_of_reference_files_equals_oracle_encoding(sp, tmp_path, M, K, s):
    A = make_sparse(M, K, s, seed=M + K)
    prefix = _write_with_reference(tmp_path, A)
    h = sp.load_bin_files(prefix, M, K)
    e = oracle.encode(A)
    assert np.array_equal(h.vals, e.vals)
    assert np.array_equal(h.gtile, e.gtile)
    assert np.array_equal(h.mtile, e.mtile)
    assert np.array_equal(h.bitmap, e.bitmap)
    assert np.array_equal(h.tile_nnz, e.tile_nnz)          # rebuilt from the bitmaps
    mx = e.max_nnz if e.max_nnz % 64 == 0 else (e.max_nnz // 64 + 1) * 64   # the writer rounds (csrc/SpMM_API.cuh:284-286)
    assert h.max_nnz == mx
    # and the loaded arrays decode to the matrix
    back = oracle.decode(oracle.Encoded(M, K, h.vals, h.tile_nnz, h.mtile, h.gtile, h.bitmap, h.max_nnz))
    assert np.array_equal(back, A.view(np.uint16))


def test_load_rejects_wrong_shape_and_missing_files(sp, tmp_path):
    A = make_sparse(128, 128, 0.6, seed=5)
    prefix = _write_with_reference(tmp_path, A)
    with pytest.raises(sp.SpmmError):
        sp.load_bin_files(prefix, 128, 192)                 # OutputSizes does not match the shape
    with pytest.raises(sp.SpmmError):
        sp.load_bin_files(prefix, 100, 128)                 # not a multiple of 64
    os.remove(prefix + ".mtile.bin")
    with pytest.raises(sp.SpmmError):
        sp.load_bin_files(prefix, 128, 128)
    with pytest.raises(sp.SpmmError):
        sp.load_bin_files(str(tmp_path / "nothing"), 128, 128)


def test_load_rejects_truncated_values(sp, tmp_path):
    A = make_sparse(128, 128, 0.5, seed=6)
    prefix = _write_with_reference(tmp_path, A)
    v = np.fromfile(prefix + ".NZWeights.bin", np.uint16)
    v[:-8].tofile(prefix + ".NZWeights.bin")
    with pytest.raises(sp.SpmmError):
        sp.load_bin_files(prefix, 128, 128)


def test_rank_lists_round_trip(sp, tmp_path):
    """The five per-rank list files: one int32 per matrix from its OutputSizes file, zeros for a matrix left dense."""
    prefixes, shapes = [], [(128, 64), (64, 128), (64, 64)]
    for i, (M, K) in enumerate(shapes):
        A = make_sparse(M, K, 0.6, seed=40 + i)
        prefixes.append(_write_with_reference(tmp_path, A, name=f"layer0.m{i}"))
    prefixes.append(str(tmp_path / "layer0.dense_one"))      # never converted: no OutputSizes file
    sp.write_rank_lists(str(tmp_path), 3, prefixes, [2, 1, 4, 7])
    lists = sp.read_rank_lists(str(tmp_path), 3)
    for i, (M, K) in enumerate(shapes):
        G = (M // 64) * (K // 64)
        e = oracle.encode(make_sparse(M, K, 0.6, seed=40 + i))
        assert lists["val_count_List"][i] == e.vals.size
        assert lists["num_gtiles_List"][i] == G + 1
        assert lists["num_mtiles_List"][i] == 4 * G
        assert lists["num_ltiles_List"][i] == 64 * G
    assert list(lists["SplitK_List"]) == [2, 1, 4, 0]
    assert all(lists[k][3] == 0 for k in lists)
    assert all(v.dtype == np.int32 and v.size == 4 for v in lists.values())
