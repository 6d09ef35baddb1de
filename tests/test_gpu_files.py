"""File-level parity on the GPU: the six weight files against the reference's own writer, a load -> SpMM round
trip, and the C++ symbols FasterTransformer binds, executed from a compiled caller."""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import ROOT, make_dense, make_sparse  # noqa: E402

REL = 1e-2   # fp16 output, fp32 accumulation: max |c - ref| <= REL * max |ref|


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200
    spmspm_b200.reset_device_status()
    return spmspm_b200


@pytest.mark.parametrize("M,K,s", [(128, 192, 0.6), (256, 512, 0.5), (64, 64, 1.0)])
def test_six_files_equal_the_reference_writers(sp, tmp_path, M, K, s):
    """Our_GenSparseMatrixBinFile of this library and of the reference (oracle/_ref) on the same dense file."""
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference) is not built")
    A = make_sparse(M, K, s, seed=3 * M + K)
    dense = tmp_path / "w.bin"
    A.tofile(dense)
    ref_names = oracle.ref_gen_bin_files(str(dense), M, K, str(tmp_path / "ref"))
    our_names = sp.bin_file_names(str(tmp_path / "ours"))
    sp.our_gen_sparse_matrix_bin_file(str(dense), M, K, *our_names)
    for a, b in zip(our_names, ref_names):
        assert open(a, "rb").read() == open(b, "rb").read(), os.path.basename(a)


@pytest.mark.parametrize("M,K,N,s,sk", [(256, 512, 16, 0.6, 1), (512, 1024, 32, 0.5, 2)])
def test_write_load_spmm_round_trip(sp, tmp_path, M, K, N, s, sk):
    """Files written by the reference's writer, read by spb_load_bin_files, uploaded, multiplied."""
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference) is not built")
    A = make_sparse(M, K, s, seed=M + N)
    B = make_dense(N, K, seed=K + N, dist="normal")
    dense = tmp_path / "w.bin"
    A.tofile(dense)
    oracle.ref_gen_bin_files(str(dense), M, K, str(tmp_path / "w"))
    W = sp.to_device(sp.load_bin_files(str(tmp_path / "w"), M, K))
    C = sp.spmm(W, torch.from_numpy(B).cuda(), split_k=sk)
    torch.cuda.synchronize()
    ref = oracle.gemm_f32(A, B)
    err = np.abs(C.cpu().numpy().astype(np.float32) - ref).max() / max(np.abs(ref).max(), 1e-12)
    assert err <= REL
    assert sp.device_status() == 0


@pytest.fixture(scope="module")
def caller(lib_built, tmp_path_factory):
    """tests/cxx/ref_api_caller.cu compiled against include/SpMM_API.cuh and linked with -lSpMM_API."""
    from spmspm_b200 import _lib
    out = tmp_path_factory.mktemp("cxx") / "ref_api_caller"
    libdir = os.path.dirname(_lib.LIB_PATH)
    cmd = ["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared",
           "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cxx", "ref_api_caller.cu"),
           "-L", libdir, "-lSpMM_API", "-Xlinker", f"-rpath={libdir}", "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return str(out)


@pytest.mark.parametrize("M,K,N,s,sk", [(128, 256, 16, 0.6, 1), (256, 512, 8, 0.5, 3), (192, 384, 32, 0.7, 2)])
def test_mangled_cxx_entry_points_execute(sp, caller, tmp_path, M, K, N, s, sk):
    """InitSparseMatrixA_bitmap and SpMM_SplitK_API_bitmap_v3 called as C++ functions from a separate program."""
    A = make_sparse(M, K, s, seed=7 * M + N)
    B = make_dense(N, K, seed=K - N, dist="normal")
    A.tofile(tmp_path / "A.bin")
    B.tofile(tmp_path / "B.bin")
    prefix = str(tmp_path / "out")
    r = subprocess.run([caller, str(tmp_path / "A.bin"), str(tmp_path / "B.bin"), prefix, str(M), str(K), str(N), str(sk)],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    e = oracle.encode(A)
    assert np.array_equal(np.fromfile(prefix + ".vals.bin", np.uint16), e.vals)
    assert np.array_equal(np.fromfile(prefix + ".gtile.bin", np.int32), e.gtile)
    assert np.array_equal(np.fromfile(prefix + ".mtile.bin", np.int32), e.mtile)
    assert np.array_equal(np.fromfile(prefix + ".bitmap.bin", np.uint64), e.bitmap)
    assert np.array_equal(np.fromfile(prefix + ".tile_nnz.bin", np.int32), e.tile_nnz)
    assert int(np.fromfile(prefix + ".max_nnz.bin", np.int32)[0]) == e.max_nnz
    C = np.fromfile(prefix + ".C.bin", np.float16).reshape(N, M).astype(np.float32)
    ref = oracle.gemm_f32(A, B)
    assert np.abs(C - ref).max() <= REL * max(np.abs(ref).max(), 1e-12)
    if sk > 1:   # split-K: same ranges and rounding points as the reference; only the order of the fp32 additions
        # inside a range differs from the oracle's, which moves a partial sum by at most one fp16 unit
        want = oracle.spmm_splitk_f16(A, B, sk).view(np.float16).astype(np.float32)
        assert np.abs(C - want).max() <= 4e-3 * np.abs(want).max()
