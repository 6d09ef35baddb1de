"""The linear-layer entry point (SpMM with bias / ReLU / residual folded into its launches) and its PyTorch operator.

Every element-wise step rounds to fp16 like the separate kernel it replaces, so the fused result is compared BIT FOR
BIT with spmm followed by the torch fp16 operations, on every path that writes final rows: the kernel's epilogue
(Split_K 1, static and balanced schedule), the reduction fused into the kernel (static, Split_K > 1), the reduction
launch (balanced, Split_K > 1) and the all-reduce's second half."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200
    spmspm_b200.reset_device_status()
    return spmspm_b200


def _tail(y, bias, residual, relu):
    if bias is not None:
        y = y + bias
    if relu:
        y = torch.relu(y)
    if residual is not None:
        y = residual + y
    return y


def _bits(t):
    return t.cpu().numpy().view(np.uint16)


CASES = [  # M, K, N, split_k, schedule
    (512, 1024, 16, 1, "static"), (512, 1024, 16, 1, "balanced"), (1024, 2048, 8, 4, "static"),
    (1024, 2048, 32, 3, "balanced"), (256, 512, 5, 1, "balanced"), (256, 1024, 40, 2, "static"),
    (384, 512, 200, 1, "static"), (128, 640, 16, 7, "static"),      # the last: empty split-K ranges
]


@pytest.mark.parametrize("M,K,N,sk,sched", CASES)
def test_linear_has_the_bits_of_spmm_plus_elementwise_kernels(sp, M, K, N, sk, sched):
    A = make_sparse(M, K, 0.6, seed=M + N)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    B = torch.from_numpy(make_dense(N, K, seed=7)).cuda()
    g = torch.Generator(device="cuda").manual_seed(5)
    bias = torch.randn(M, device="cuda", generator=g).half()
    res = torch.randn((N, M), device="cuda", generator=g).half()
    prev = sp.set_schedule({"static": sp.SCHEDULE_STATIC, "balanced": sp.SCHEDULE_BALANCED}[sched])
    try:
        y = sp.spmm(W, B, split_k=sk)
        ref32 = oracle.gemm_f32(A, B.cpu().numpy())
        assert float(np.abs(y.cpu().numpy().astype(np.float32) - ref32).max()) <= 1e-2 * float(np.abs(ref32).max())
        for b, r, relu in ((bias, None, False), (bias, None, True), (bias, res, False), (None, res, True), (None, None, True)):
            got = sp.linear(W, B, bias=b, residual=r, activation=sp.ACT_RELU if relu else sp.ACT_NONE, split_k=sk)
            torch.cuda.synchronize()
            want = _tail(y, b, r, relu)
            assert np.array_equal(_bits(got), _bits(want)), (b is not None, r is not None, relu)
        # the residual may be the destination itself
        buf = res.clone()
        sp.linear(W, B, bias=bias, residual=buf, split_k=sk, out=buf)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(buf), _bits(_tail(y, bias, res, False)))
    finally:
        sp.set_schedule(prev)
    assert sp.device_status() == 0


def test_relu_keeps_nan_and_maps_negative_zero_to_zero(sp):
    M, K, N = 128, 128, 16
    A = np.zeros((M, K), dtype=np.float16)
    A[0, 0] = 1.0
    W = sp.encode_device(torch.from_numpy(A).cuda())
    B = torch.zeros((N, K), dtype=torch.float16, device="cuda")
    B[0, 0] = float("nan")
    B[1, 0] = -0.0
    B[2, 0] = -3.0
    B[3, 0] = 2.5
    got = sp.linear(W, B, activation=sp.ACT_RELU, split_k=1)
    want = torch.relu(sp.spmm(W, B, split_k=1))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(got), _bits(want))
    assert bool(torch.isnan(got[0, 0])) and float(got[2, 0]) == 0.0 and float(got[3, 0]) == 2.5
    assert _bits(got[1:2, 0:1])[0, 0] == 0   # +0, like torch.relu


def test_operator_and_module(sp):
    from spmspm_b200.ops import SparseLinear, ACT_RELU
    M, K, N = 512, 1024, 24
    A = make_sparse(M, K, 0.6, seed=3)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    x = torch.from_numpy(make_dense(N, K, seed=4)).cuda()
    bias = torch.randn(M, device="cuda").half()
    res = torch.randn((N, M), device="cuda").half()
    y = torch.ops.spmspm_b200.sparse_linear(x, W.vals, W.gtile, W.mtile, W.bitmap, W.max_nnz, M, bias, res, ACT_RELU, 0)
    want = _tail(sp.spmm(W, x), bias, res, True)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(y), _bits(want))
    mod = SparseLinear(W, bias, activation=ACT_RELU)
    y3 = mod(x.reshape(2, 12, K), residual=res.reshape(2, 12, M))
    assert y3.shape == (2, 12, M) and np.array_equal(_bits(y3.reshape(N, M)), _bits(want))
    assert set(mod.state_dict()) == {"vals", "gtile", "mtile", "bitmap", "max_nnz", "bias"}
    # shape function: the operator can be traced without running
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode(allow_non_fake_inputs=True) as mode:
        fx = mode.from_tensor(x)
        fy = torch.ops.spmspm_b200.sparse_linear(fx, W.vals, W.gtile, W.mtile, W.bitmap, W.max_nnz, M, None, None, 0, 0)
        assert tuple(fy.shape) == (N, M) and fy.dtype == torch.float16
    # and captured into a CUDA graph
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        mod(x)
        st.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            yg = mod(x, residual=res)
    gr.replay()
    torch.cuda.synchronize()
    assert np.array_equal(_bits(yg), _bits(want))
    with pytest.raises(sp.SpmmError):
        sp.linear(W, x, bias=bias[:-1].contiguous())
    with pytest.raises(sp.SpmmError):
        sp.linear(W, x, activation=5)
    assert sp.device_status() == 0


def test_layer_with_fused_tails_has_the_bits_of_the_unfused_layer(sp):
    from spmspm_b200.layer import SparseOptDecoderLayer, _gen
    dev = torch.device("cuda", 0)
    B, T, hidden, heads, ffn = 2, 8, 256, 4, 1024
    fused = SparseOptDecoderLayer(hidden, heads, ffn, 0.6, dev, batch=B, max_len=32, fused=True)
    plain = SparseOptDecoderLayer(hidden, heads, ffn, 0.6, dev, batch=B, max_len=32, fused=False)
    x = _gen((B * T, hidden), 3, dev, 1.0)
    xt = _gen((B, hidden), 4, dev, 1.0)
    a, b = fused.forward(x, T), plain.forward(x, T)
    a1, b1 = fused.forward(xt, 1), plain.forward(xt, 1)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(a), _bits(b)) and np.array_equal(_bits(a1), _bits(b1))


def test_single_rank_allreduce_finish_with_tail(sp):
    import ctypes
    M, K, N = 512, 1024, 16
    A = make_sparse(M, K, 0.6, seed=9)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    B = torch.from_numpy(make_dense(N, K, seed=10)).cuda()
    bias = torch.randn(M, device="cuda").half()
    res = torch.randn((N, M), device="cuda").half()
    parts = torch.zeros((1, N, M), dtype=torch.float16, device="cuda")
    flags = torch.zeros(3, dtype=torch.int32, device="cuda")
    pp = (ctypes.c_void_p * 1)(parts.data_ptr())
    fp = (ctypes.c_void_p * 1)(flags.data_ptr())
    out = torch.empty((N, M), dtype=torch.float16, device="cuda")
    for turn, sk in enumerate((1, 2, 1)):
        sp.spmm_allreduce(W, B, pp, fp, 1, 0, split_k=sk)
        sp.allreduce_finish(out, parts, flags, 1, bias=bias, residual=res, activation=sp.ACT_RELU)
        torch.cuda.synchronize()
        want = _tail(sp.spmm(W, B, split_k=sk), bias, res, True)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(out), _bits(want))
        assert flags.cpu().tolist() == [turn + 1, turn + 1, turn + 1]
    assert sp.device_status() == 0
