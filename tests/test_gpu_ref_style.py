"""Second numerics pin: the reference-style mma.sync / cp.async SpMM (oracle/ref_style_spmm.cu, put together from the
reference's own device functions, compiled for sm_100a into oracle/_ref) on the same inputs as the library.

Tolerance: both results within 1e-2 * max|ref| of the fp32 host GEMM, and within 4e-3 * max|ref| of each other
(both accumulate in fp32 and round once to fp16; only the order of the additions differs)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    if not oracle.have_ref_style():
        pytest.skip("oracle/_ref/libref_style_spmm.so is not built")
    import spmspm_b200
    spmspm_b200.reset_device_status()
    return spmspm_b200


def ref_style(W, B, split_k):
    """C [N, M] of the reference-style kernel; B [N, K] on the device."""
    N = B.shape[0]
    Bp = B
    if N == 8:   # that kernel copies a 16-row activation tile
        Bp = torch.zeros((16, B.shape[1]), dtype=B.dtype, device=B.device)
        Bp[:8] = B
    C = torch.empty((N, W.M), dtype=torch.float16, device=B.device)
    ws = torch.empty(max(split_k, 1) * N * W.M, dtype=torch.float16, device=B.device)
    oracle.ref_style_spmm(torch.cuda.current_stream().cuda_stream, W.vals.data_ptr(), W.gtile.data_ptr(),
                          W.mtile.data_ptr(), W.bitmap.data_ptr(), Bp.data_ptr(), C.data_ptr(), W.M, N, W.K,
                          ws.data_ptr(), split_k, int(W.max_nnz.item()))
    torch.cuda.synchronize()
    return C


@pytest.mark.parametrize("M,K,N,s,sk", [
    (64, 64, 16, 0.5, 1),
    (256, 512, 8, 0.6, 1),
    (256, 512, 16, 0.6, 3),
    (512, 1024, 32, 0.5, 2),
    (512, 1024, 64, 0.7, 1),
    (256, 1024, 128, 0.4, 1),
    (1024, 4096, 16, 0.6, 4),
    (5120, 5120, 16, 0.6, 1),      # OPT-13B out-proj
])
def test_library_and_reference_style_kernel_agree(sp, M, K, N, s, sk):
    A = make_sparse(M, K, s, seed=11 * M + N)
    B = make_dense(N, K, seed=3 * K + N, dist="normal")
    ref = oracle.gemm_f32(A, B)
    scale = max(float(np.abs(ref).max()), 1e-12)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bd = torch.from_numpy(B).cuda()
    ours = sp.spmm(W, Bd, split_k=sk)
    torch.cuda.synchronize()
    theirs = ref_style(W, Bd, sk)
    o, t = ours.cpu().numpy().astype(np.float32), theirs.cpu().numpy().astype(np.float32)
    assert np.abs(t - ref).max() <= 1e-2 * scale, "reference-style kernel off the fp32 GEMM"
    assert np.abs(o - ref).max() <= 1e-2 * scale
    assert np.abs(o - t).max() <= 4e-3 * scale
    # the reference's own figure of merit (csrc/spmm_test_utils.h:110-115): sum of absolute differences
    assert oracle.total_error(ours.cpu().numpy(), theirs.cpu().numpy()) <= 4e-3 * scale * o.size
    assert sp.device_status() == 0
