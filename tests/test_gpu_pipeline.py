"""The host-buffer front end (spmspm_b200.pipeline.HostBatch): results in pinned host memory equal the resident SpMM's
bits, for both staging sets, also when a set is resubmitted with new inputs while the other is in flight."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402


def test_host_batch_matches_resident_spmm(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200 as sp
    from spmspm_b200.pipeline import HostBatch
    sp.reset_device_status()
    shapes = [(512, 1024, 16), (1024, 512, 8), (256, 2048, 40)]
    As = [make_sparse(M, K, 0.6, seed=M + K) for (M, K, N) in shapes]
    Ws = [sp.encode_device(torch.from_numpy(A).cuda()) for A in As]
    hb = HostBatch([(W, N) for W, (M, K, N) in zip(Ws, shapes)], "cuda")
    for rnd in range(3):
        Bs = {s: [make_dense(N, K, seed=100 * rnd + 10 * s + i) for i, (M, K, N) in enumerate(shapes)] for s in (0, 1)}
        for s in (0, 1):
            for view, B in zip(hb.inputs(s), Bs[s]):
                view.copy_(torch.from_numpy(B))
            hb.submit(s)                                   # set 1 is submitted while set 0 is in flight
        for s in (0, 1):
            hb.wait(s)
            for out, W, A, B, sk in zip(hb.outputs(s), Ws, As, Bs[s], hb.split_k):
                want = sp.spmm(W, torch.from_numpy(B).cuda(), split_k=sk)
                torch.cuda.synchronize()
                assert np.array_equal(out.numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
                ref = oracle.gemm_f32(A, B)
                assert float(np.abs(out.numpy().astype(np.float32) - ref).max()) <= 1e-2 * float(np.abs(ref).max())
    hb.close()
    h2d, d2h = hb.bytes_per_batch()
    assert h2d == 2 * sum(N * K for (M, K, N) in shapes) and d2h == 2 * sum(N * M for (M, K, N) in shapes)
    assert sp.device_status() == 0


def test_host_batch_with_a_custom_body(lib_built):
    """The batch's work can be any sequence enqueued on the compute stream (here: linear layers with bias and ReLU)."""
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200 as sp
    from spmspm_b200.pipeline import HostBatch
    shapes = [(512, 1024, 16), (256, 1024, 16)]
    As = [make_sparse(M, K, 0.6, seed=7 * M) for (M, K, N) in shapes]
    Ws = [sp.encode_device(torch.from_numpy(A).cuda()) for A in As]
    biases = [torch.randn(M, device="cuda").half() for (M, K, N) in shapes]
    called = []

    def body(s, ins, outs):
        called.append(s)
        for W, b, x, y in zip(Ws, biases, ins, outs):
            sp.linear(W, x, bias=b, activation=sp.ACT_RELU, split_k=1, out=y)

    hb = HostBatch([(W, N) for W, (M, K, N) in zip(Ws, shapes)], "cuda", body=body, ready=lambda: None)
    assert sorted(set(called)) == [0, 1]
    Bs = [make_dense(N, K, seed=50 + i) for i, (M, K, N) in enumerate(shapes)]
    for view, B in zip(hb.inputs(1), Bs):
        view.copy_(torch.from_numpy(B))
    hb.submit(1)
    hb.wait(1)
    for out, W, b, B in zip(hb.outputs(1), Ws, biases, Bs):
        want = torch.relu(sp.spmm(W, torch.from_numpy(B).cuda(), split_k=1) + b)
        torch.cuda.synchronize()
        assert np.array_equal(out.numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
    hb.close()
    assert sp.device_status() == 0
