"""The fork's extension on the GPU: encoder for a compressed second operand (bit-exact with the reference's), its
expansion, and the SpMM with both operands compressed (the bits of the SpMM on the dense activations)."""
import glob
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402

GOLDEN_B = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "operand_b", "*.npz")))
FIELDS = ("vals", "tile_nnz", "mtile", "gtile", "bitmap")


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200
    spmspm_b200.reset_device_status()
    return spmspm_b200


@pytest.mark.parametrize("path", GOLDEN_B, ids=[os.path.basename(p) for p in GOLDEN_B])
def test_gpu_encoder_matches_the_reference_fixtures(sp, path):
    d = np.load(path)
    e = sp.init_sparse_matrix_a_bitmap_v6_b(d["A"])
    for f in FIELDS:
        assert np.array_equal(getattr(e, f), d[f]), f
    assert e.max_nnz == int(d["max_nnz"])


@pytest.mark.parametrize("M,K,s,seed", [(1024, 2048, 0.6, 1), (64, 4096, 0.0, 2), (4096, 64, 0.97, 3), (1536, 1536, 0.5, 4)])
def test_gpu_encoder_and_expansion_against_the_oracle(sp, M, K, s, seed):
    A = make_sparse(M, K, s, seed)
    e, want = sp.init_sparse_matrix_a_bitmap_v6_b(A), oracle.encode_b(A)
    for f in FIELDS:
        assert np.array_equal(getattr(e, f), getattr(want, f)), f
    assert e.max_nnz == want.max_nnz
    dense = sp.decode_operand_b(sp.to_device(e))
    torch.cuda.synchronize()
    assert np.array_equal(dense.cpu().numpy().view(np.uint16), A.view(np.uint16))
    assert sp.device_status() == 0


@pytest.mark.parametrize("M,K,N,sa,sb,sk", [(512, 1024, 64, 0.6, 0.5, 1), (1024, 1024, 128, 0.5, 0.5, 2), (256, 2048, 320, 0.6, 0.7, 1),
                                            (1024, 1024, 1024, 0.5, 0.5, 1)])
def test_spmspm_has_the_bits_of_spmm_on_the_dense_operand(sp, M, K, N, sa, sb, sk):
    A = make_sparse(M, K, sa, seed=M + N)
    B = make_dense(N, K, seed=K + N)
    B[np.random.default_rng(N).random((N, K)) < sb] = 0          # prune the activations too
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bc = sp.to_device(sp.init_sparse_matrix_a_bitmap_v6_b(B))
    got = sp.spmspm(W, Bc, split_k=sk)
    want = sp.spmm(W, torch.from_numpy(B).cuda(), split_k=sk)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
    ref = oracle.gemm_f32(A, B)
    assert float(np.abs(got.cpu().numpy().astype(np.float32) - ref).max()) <= 1e-2 * float(np.abs(ref).max())
    assert sp.device_status() == 0


def test_spmspm_inside_a_cuda_graph(sp):
    """The expansion buffer comes from the stream's memory pool, so the call can be captured and replayed."""
    M, K, N = 512, 1024, 128
    A = make_sparse(M, K, 0.6, seed=21)
    B = make_sparse(N, K, 0.5, seed=22)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bc = sp.to_device(sp.init_sparse_matrix_a_bitmap_v6_b(B))
    want = sp.spmm(W, torch.from_numpy(B).cuda(), split_k=1)
    out = torch.zeros((N, M), dtype=torch.float16, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        sp.spmspm(W, Bc, split_k=1, out=out)
        st.synchronize()
        out.zero_()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            sp.spmspm(W, Bc, split_k=1, out=out)
    for _ in range(3):
        out.zero_()
        gr.replay()
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
    assert sp.device_status() == 0


def test_spmspm_rejects_bad_shapes_and_reports_corrupt_offsets(sp):
    A = make_sparse(256, 512, 0.6, 5)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    B = make_dense(64, 512, seed=6)
    e = sp.init_sparse_matrix_a_bitmap_v6_b(B)
    Bc = sp.to_device(e)
    Bc48 = sp.BitmapMatrix(48, 512, Bc.vals, Bc.gtile, Bc.mtile, Bc.bitmap, Bc.max_nnz)
    with pytest.raises(sp.SpmmError):
        sp.spmspm(W, Bc48)                                          # N not a multiple of 64: nothing is launched
    # offsets that run backwards: the expansion writes zeros and sets the status word; nothing faults
    bad = sp.BitmapMatrix(64, 512, Bc.vals, torch.flip(Bc.gtile, dims=[0]).contiguous(), Bc.mtile, Bc.bitmap, Bc.max_nnz)
    dense = sp.decode_operand_b(bad)
    torch.cuda.synchronize()
    assert sp.device_status() != 0
    sp.reset_device_status()
    assert float(dense[:, 64:448].abs().max()) == 0.0
