"""GPU encoder parity (bit-exact) against the oracle and the committed reference fixtures, through the C ABI."""
import glob
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_sparse  # noqa: E402

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200
    return spmspm_b200


def _same_device(W, e):
    return (np.array_equal(W.vals.cpu().numpy().view(np.uint16)[:e.vals.size], e.vals) and W.val_count == e.vals.size
            and np.array_equal(W.bitmap.cpu().numpy().view(np.uint64), e.bitmap)
            and np.array_equal(W.gtile.cpu().numpy(), e.gtile) and np.array_equal(W.mtile.cpu().numpy(), e.mtile)
            and np.array_equal(W.tile_nnz.cpu().numpy(), e.tile_nnz) and int(W.max_nnz.item()) == e.max_nnz)


def _same_host(h, e):
    return (np.array_equal(h.vals, e.vals) and np.array_equal(h.bitmap, e.bitmap) and np.array_equal(h.gtile, e.gtile)
            and np.array_equal(h.mtile, e.mtile) and np.array_equal(h.tile_nnz, e.tile_nnz) and h.max_nnz == e.max_nnz)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_encoder_matches_reference_fixtures(sp, path):
    z = np.load(path)
    A = z["A"]
    want = oracle.Encoded(A.shape[0], A.shape[1], z["vals"], z["tile_nnz"], z["mtile"], z["gtile"], z["bitmap"],
                          int(z["max_nnz"]))
    assert _same_host(sp.init_sparse_matrix_a_bitmap(A), want)
    W = sp.encode_device(torch.from_numpy(A.view(np.float16)).cuda())
    assert _same_device(W, want)


@pytest.mark.parametrize("M,K,s", [(64, 64, 0.5), (128, 128, 0.5), (256, 192, 0.9), (192, 320, 0.4), (64, 128, 0.0),
                                   (128, 64, 1.0), (1024, 2048, 0.6), (4096, 4096, 0.5), (5120, 5120, 0.6)])
def test_encoder_matches_oracle(sp, M, K, s):
    A = make_sparse(M, K, s, seed=M * 7 + K)
    e = oracle.encode(A)
    assert _same_device(sp.encode_device(torch.from_numpy(A).cuda()), e)
    if M * K <= 1024 * 2048:
        assert _same_host(sp.init_sparse_matrix_a_bitmap(A), e)


def test_encoder_per_shard_is_bit_exact(sp):
    """Every M-shard's encoding equals the reference encoding of that sub-matrix (and a slice of the full one)."""
    M, K, P = 1024, 512, 8
    A = make_sparse(M, K, 0.6, seed=9)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    for r in range(P):
        sub = oracle.encode(A[r * M // P:(r + 1) * M // P])
        Wr = W.shard_rows(r, P)
        assert _same_device(Wr, sub)


def test_decode_of_gpu_encoding_round_trips(sp):
    A = make_sparse(512, 768, 0.55, seed=21)
    h = sp.init_sparse_matrix_a_bitmap(A)
    e = oracle.Encoded(512, 768, h.vals, h.tile_nnz, h.mtile, h.gtile, h.bitmap, h.max_nnz)
    assert np.array_equal(oracle.decode(e), A.view(np.uint16))


def test_full_size_round_trip_property(sp):
    """OPT-30B FC1 shape: popcount(bitmaps) == nnz(A) and the packed values are exactly A's non-zeros in tile order."""
    M, K = 28672, 7168
    g = torch.Generator(device="cuda").manual_seed(0x5EED0003)
    A = (torch.randn((M, K), device="cuda", generator=g) * 0.02).half()
    A[torch.rand((M, K), device="cuda", generator=g) < 0.6] = 0
    W = sp.encode_device(A)
    nnz = int((A != 0).sum().item())
    assert int(W.tile_nnz.sum().item()) == nnz
    pads = int(W.gtile[-1].item()) - nnz
    assert 0 <= pads <= 7 * W.G
    # checksum of checksums: sum of packed values equals the sum of the matrix (zero pads add nothing)
    assert abs(float(W.vals.double().sum().item()) - float(A.double().sum().item())) < 1e-6 * max(1.0, nnz)
    # spot-check 6 global tiles bit-exactly against the oracle
    gt = W.gtile.cpu().numpy()
    for (gm, gk) in [(0, 0), (1, 5), (17, 111), (200, 3), (447, 111), (300, 57)]:
        sub = A[gm * 64:(gm + 1) * 64, gk * 64:(gk + 1) * 64].contiguous().cpu().numpy()
        e = oracle.encode(sub)
        gidx = gm * (K // 64) + gk
        got = W.vals[gt[gidx]:gt[gidx + 1]].cpu().numpy().view(np.uint16)
        assert np.array_equal(got, e.vals)
        assert np.array_equal(W.bitmap[gidx * 64:(gidx + 1) * 64].cpu().numpy().view(np.uint64), e.bitmap)


def test_encoder_rejects_bad_shapes(sp):
    with pytest.raises(sp.SpmmError):
        sp.encode_device(torch.zeros((65, 64), dtype=torch.float16, device="cuda"))
    with pytest.raises(sp.SpmmError):
        sp.init_sparse_matrix_a_bitmap(np.zeros((64, 100), np.float16))


def test_file_encoder_writes_reference_files(sp, tmp_path):
    M, K = 128, 192
    A = make_sparse(M, K, 0.6, seed=33)
    dense = tmp_path / "w.bin"
    A.tofile(dense)
    names = {k: str(tmp_path / f"w.{k}") for k in ("NZWeights", "gtile", "mtile", "ltile", "intile", "OutputSizes")}
    sp.our_gen_sparse_matrix_bin_file(str(dense), M, K, names["NZWeights"], names["gtile"], names["mtile"],
                                      names["ltile"], names["intile"], names["OutputSizes"])
    e = oracle.encode(A)
    G = e.G
    assert np.array_equal(np.fromfile(names["OutputSizes"], np.int32), [e.vals.size, G + 1, 4 * G, 64 * G])
    assert np.array_equal(np.fromfile(names["NZWeights"], np.uint16), e.vals)
    assert np.array_equal(np.fromfile(names["gtile"], np.int32), e.gtile)
    assert np.array_equal(np.fromfile(names["mtile"], np.int32), e.mtile)
    assert np.array_equal(np.fromfile(names["ltile"], np.uint64), e.bitmap)
    mx = e.max_nnz if e.max_nnz % 64 == 0 else (e.max_nnz // 64 + 1) * 64
    assert np.fromfile(names["intile"], np.int32)[0] == mx
    with pytest.raises(sp.SpmmError):
        sp.our_gen_sparse_matrix_bin_file(str(tmp_path / "missing.bin"), M, K, *[names[k] for k in
                                          ("NZWeights", "gtile", "mtile", "ltile", "intile", "OutputSizes")])
