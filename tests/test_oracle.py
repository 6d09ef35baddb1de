"""CPU tests of the oracle: golden fixtures, the compiled reference encoder, round trips, fp16 helpers."""
import glob
import os

import numpy as np
import pytest

import oracle
from conftest import make_dense, make_sparse

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _golden(path):
    z = np.load(path)
    return z["A"], oracle.Encoded(z["A"].shape[0], z["A"].shape[1], z["vals"], z["tile_nnz"], z["mtile"], z["gtile"],
                                  z["bitmap"], int(z["max_nnz"]))


def test_golden_present():
    assert len(GOLDEN) >= 7


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_encoder_matches_golden(path):
    A, want = _golden(path)
    got = oracle.encode(A)
    assert got.same_as(want)
    assert np.array_equal(oracle.decode(got), np.where((A & 0x7FFF) == 0, 0, A))


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (reference sources absent)")
@pytest.mark.parametrize("M,K,s", [(64, 64, 0.5), (128, 256, 0.6), (320, 192, 0.4), (64, 64, 1.0), (256, 64, 0.0),
                                   (1024, 1024, 0.7)])
def test_oracle_encoder_matches_compiled_reference(M, K, s):
    A = make_sparse(M, K, s, seed=M + K)
    assert oracle.encode(A).same_as(oracle.ref_encode(A))


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (reference sources absent)")
def test_golden_is_what_the_reference_produces():
    for path in GOLDEN:
        A, want = _golden(path)
        assert oracle.ref_encode(A).same_as(want)


def test_row_shard_is_a_slice_of_the_full_encoding():
    M, K, P = 512, 256, 4
    A = make_sparse(M, K, 0.6, seed=5)
    full = oracle.encode(A)
    gk = K // 64
    for r in range(P):
        sub = oracle.encode(A[r * M // P:(r + 1) * M // P])
        g0, g1 = r * (M // P // 64) * gk, (r + 1) * (M // P // 64) * gk
        o0, o1 = full.gtile[g0], full.gtile[g1]
        assert np.array_equal(sub.vals, full.vals[o0:o1])
        assert np.array_equal(sub.bitmap, full.bitmap[64 * g0:64 * g1])
        assert np.array_equal(sub.mtile, full.mtile[4 * g0:4 * g1])
        assert np.array_equal(sub.gtile, full.gtile[g0:g1 + 1] - o0)
        assert sub.max_nnz == int(np.diff(full.gtile[g0:g1 + 1]).max())


def test_fp16_helpers_exhaustive():
    lib = oracle.lib()
    bits = np.arange(1 << 16, dtype=np.uint16)
    f = bits.view(np.float16).astype(np.float32)
    for b in range(0, 1 << 16, 7):
        if np.isnan(f[b]):
            continue
        assert lib.oracle_h2f(int(b)) == float(f[b])
        assert lib.oracle_f2h(float(f[b])) == b
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(20000) * np.exp(rng.uniform(-18, 10, 20000))).astype(np.float32)
    want = x.astype(np.float16).view(np.uint16)
    for v, w in zip(x[:5000], want[:5000]):
        assert lib.oracle_f2h(float(v)) == w


def test_gemm_against_numpy():
    A = make_sparse(256, 320, 0.5, 1)
    B = make_dense(24, 320, 2)
    C = oracle.gemm_f32(A, B)
    want = B.astype(np.float64) @ A.astype(np.float64).T
    assert np.abs(C - want).max() <= 1e-5 * np.abs(want).max()


def test_splitk_chain_and_reduction():
    A = make_sparse(128, 1024, 0.5, 11)
    B = make_dense(16, 1024, 12)
    ref = oracle.gemm_f32(A, B)
    for sk in (1, 2, 3, 7, 16):
        C = oracle.spmm_splitk_f16(A, B, sk).view(np.float16).astype(np.float32)
        assert np.abs(C - ref).max() <= 2e-3 * np.abs(ref).max()
    # reduction alone: fixed-order fp32 sum of fp16 partials
    rng = np.random.default_rng(0)
    parts = rng.standard_normal((5, 16, 128)).astype(np.float16)
    got = oracle.splitk_reduce(parts, 128, 16, 5).view(np.float16)
    acc = np.zeros((16, 128), np.float32)
    for s in range(5):
        acc = acc + parts[s].astype(np.float32)
    assert np.array_equal(got, acc.astype(np.float16))


def test_total_error_metric():
    a = np.array([1.0, 2.0, -3.0], np.float16)
    b = np.array([1.5, 2.0, -1.0], np.float16)
    assert oracle.total_error(a, b) == pytest.approx(2.5)
