"""The allocation-free SpMM entry point against the regular one, through the C ABI.

Collected last (file name) so that a run stopping at the first failure has already run everything else.
The entry point serves callers that cannot allocate device memory (fixed memory plans, plug-ins that only
see framework buffers, stream capture): its split-K partials live in an array inside the library, shared
by all calls, so the test makes two different calls back to back and checks that the second is not
disturbed by what the first left behind.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402

REL = 1e-2  # the tolerance of tests/test_gpu_spmm.py


def _close(a, b):
    a, b = a.astype(np.float32), b.astype(np.float32)
    scale = max(float(np.abs(b).max()), 1e-12)
    return float(np.abs(a - b).max()) <= REL * scale


def test_noalloc_entry_point_matches_regular_entry_point(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200 as sp
    from spmspm_b200 import _lib

    lib = _lib.load()
    # M, K, N, sparsity, split_k, seed; the last two leave split-K ranges empty (10 and 8 k-tiles in 7 ranges of 2):
    # their partials must come out as zeros although the shared scratch still holds the previous call's sums
    cases = [(1024, 2048, 16, 0.6, 4, 11), (512, 1024, 32, 0.5, 3, 12), (128, 640, 16, 0.5, 7, 13), (128, 512, 16, 0.5, 7, 14)]
    for M, K, N, s, sk, seed in cases:  # two calls in a row on the shared scratch
        A = make_sparse(M, K, s, seed)
        B = torch.from_numpy(make_dense(N, K, seed + 100)).cuda()
        W = sp.encode_device(torch.from_numpy(A).cuda())
        balanced = sp.spmm(W, B, split_k=sk)                  # regular entry point, caller-owned workspace
        prev = sp.set_schedule(sp.SCHEDULE_STATIC)            # the schedule the allocation-free entry point uses
        try:
            want = sp.spmm(W, B, split_k=sk)
        finally:
            sp.set_schedule(prev)
        got = torch.full((N, M), float("nan"), dtype=torch.float16, device="cuda")
        code = lib.spb_spmm_bitmap_v3_noalloc(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                              ctypes.c_void_p(W.vals.data_ptr()), ctypes.c_void_p(W.gtile.data_ptr()),
                                              ctypes.c_void_p(W.mtile.data_ptr()), ctypes.c_void_p(W.bitmap.data_ptr()),
                                              ctypes.c_void_p(W.max_nnz.data_ptr()), ctypes.c_void_p(B.data_ptr()),
                                              ctypes.c_void_p(got.data_ptr()), M, N, K, sk)
        assert code == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert _close(got.cpu().numpy(), want.cpu().numpy())
        assert _close(got.cpu().numpy(), balanced.cpu().numpy())
        assert _close(got.cpu().numpy(), oracle.gemm_f32(A, B.cpu().numpy()))   # and against the fp32 host GEMM
        # same kernels, same split, same schedule: the two paths are in fact bit-identical
        assert np.array_equal(got.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
    assert sp.device_status() == 0


def test_noalloc_entry_point_rejects_oversized_requests(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200 as sp
    from spmspm_b200 import _lib

    M, K, N = 8192, 2048, 64
    sk = 32  # 32 * 8192 * 64 * 2 bytes = 32 MiB > the 16 MiB built-in scratch
    assert 2 * sk * M * N > _lib.NOALLOC_MAX_SCRATCH_BYTES
    W = sp.encode_device(torch.from_numpy(make_sparse(M, K, 0.7, 5)).cuda())
    B = torch.zeros((N, K), dtype=torch.float16, device="cuda")
    out = torch.full((N, M), 3.0, dtype=torch.float16, device="cuda")
    with pytest.raises(sp.SpmmError, match="exceed the built-in scratch"):
        sp.spmm_noalloc(W, B, sk, out)
    torch.cuda.synchronize()
    assert float(out.min()) == 3.0 and float(out.max()) == 3.0   # nothing was launched
    sp.spmm_noalloc(W, B, 1, out)                                # Split_K == 1 needs no scratch
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
