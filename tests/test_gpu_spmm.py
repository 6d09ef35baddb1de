"""SpMM parity through the C ABI: CUDA kernel vs the CPU oracle on the same seeded inputs.

Tolerance (fp16 output, fp32 accumulation): max |c - ref| <= 1e-2 * max|ref| and element-wise
|c - ref| <= 1e-2 * |ref| + 1e-2 * rms(ref), ref = fp32 host GEMM.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402

REL = 1e-2


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200
    spmspm_b200.reset_device_status()
    return spmspm_b200


def _assert_close(C, ref):
    C = C.astype(np.float32)
    scale = max(float(np.abs(ref).max()), 1e-12)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    err = np.abs(C - ref)
    assert float(err.max()) <= REL * scale, f"max err {err.max()} vs scale {scale}"
    assert np.all(err <= REL * np.abs(ref) + REL * rms + 1e-12)


def _run(sp, A, B, split_k):
    W = sp.encode_device(torch.from_numpy(A).cuda())
    C = sp.spmm(W, torch.from_numpy(B).cuda(), split_k=split_k)
    torch.cuda.synchronize()
    return C.cpu().numpy()


@pytest.mark.parametrize("M,K,N,s,sk", [
    (64, 64, 16, 0.5, 1),        # smallest legal shape: half-filled 128-row block
    (128, 64, 8, 0.5, 1),        # N = 8 (padded activation tile)
    (128, 128, 16, 0.5, 2),
    (192, 512, 16, 0.6, 1),      # odd number of 64-row tiles
    (256, 512, 32, 0.6, 3),      # split-K not dividing the 8 k-tiles
    (1024, 1024, 64, 0.4, 4),
    (512, 1024, 128, 0.5, 1),
    (512, 1024, 256, 0.5, 2),    # one 256-column activation tile (stages of two k-tiles, 8 operand blocks)
    (256, 1024, 100, 0.6, 1),    # 128-column tile, partly filled
    (384, 2048, 129, 0.6, 3),    # 256-column tile, barely more than 128
    (512, 1024, 512, 0.6, 1),    # two 256-column tiles (prefill: batch x sequence)
    (256, 512, 600, 0.5, 2),     # three tiles, the last partly filled
    (128, 4096, 256, 0.0, 1),    # dense tiles with the widest activation tile: a single stage fits
    (512, 1024, 24, 0.7, 1),     # N the reference rejects
    (256, 2048, 1, 0.6, 1),
    (128, 4096, 16, 0.0, 1),     # fully dense tiles (4096 values per global tile)
    (128, 4096, 16, 1.0, 1),     # all-zero matrix
    (256, 2048, 128, 0.0, 2),    # dense tiles with the widest activation tile: shallowest stage ring
    (256, 1024, 64, 0.05, 1),
    (4096, 4096, 16, 0.5, 1),    # BASELINE config 1
    (4096, 4096, 16, 0.5, 6),
    (5120, 5120, 16, 0.6, 6),    # OPT-13B out-proj
    (5120, 20480, 8, 0.6, 8),    # OPT-13B FC2
    (128, 640, 16, 0.5, 7),      # 10 k-tiles in 7 ranges of 2: the last two ranges are empty and must come out as zeros
    (128, 512, 16, 0.5, 7),      # 8 k-tiles in 7 ranges of 2: three empty ranges
])
def test_spmm_matches_fp32_oracle(sp, M, K, N, s, sk):
    A = make_sparse(M, K, s, seed=M + 3 * K + N)
    B = make_dense(N, K, seed=N + K, dist="uniform" if M == 4096 else "normal")
    ref = oracle.gemm_f32(A, B)
    for schedule in (sp.SCHEDULE_BALANCED, sp.SCHEDULE_STATIC):
        prev = sp.set_schedule(schedule)
        try:
            C = _run(sp, A, B, sk)
        finally:
            sp.set_schedule(prev)
        _assert_close(C, ref)
    assert sp.device_status() == 0


@pytest.mark.parametrize("M,K,N,s,sk", [
    (5120, 5120, 16, 0.6, 1),     # 3200 k-tiles over the SMs: every range is cut between several SMs
    (4096, 4096, 32, 0.5, 6),     # ranges of 11 k-tiles, shares of 13.8
    (192, 64 * 40, 16, 0.5, 1),   # fewer k-tiles than SMs, half-filled last row block
    (1024, 1024, 128, 0.5, 3),    # 128-column tile
    (2048, 2048, 512, 0.6, 1),    # two 256-column tiles, ranges shared between SMs
    (1024, 4096, 320, 0.6, 2),
    (15360, 5120, 8, 0.6, 1),     # OPT-13B QKV
])
def test_balanced_schedule_repeatable_and_close_to_static(sp, M, K, N, s, sk):
    """Equal k-tile shares per SM with the fp32 fix-up: the same bits on every call (the sums are taken in k
    order whoever finishes last, and the arrival counters return to zero), and the static schedule's result
    up to the order of the fp32 additions."""
    A = make_sparse(M, K, s, seed=M + K + N + 5)
    B = torch.from_numpy(make_dense(N, K, seed=N + K + 5)).cuda()
    W = sp.encode_device(torch.from_numpy(A).cuda())
    assert sp.set_schedule(sp.SCHEDULE_BALANCED) == sp.SCHEDULE_AUTO
    try:
        runs = [sp.spmm(W, B, split_k=sk).cpu().numpy() for _ in range(3)]
        sp.set_schedule(sp.SCHEDULE_STATIC)
        static = sp.spmm(W, B, split_k=sk).cpu().numpy()
    finally:
        sp.set_schedule(sp.SCHEDULE_AUTO)
    assert np.array_equal(runs[0].view(np.uint16), runs[1].view(np.uint16))
    assert np.array_equal(runs[0].view(np.uint16), runs[2].view(np.uint16))
    scale = float(np.abs(static.astype(np.float32)).max())
    assert float(np.abs(runs[0].astype(np.float32) - static.astype(np.float32)).max()) <= 2e-3 * scale
    if M <= 5120:
        _assert_close(runs[0], oracle.gemm_f32(A, B.cpu().numpy()))
    assert sp.device_status() == 0


def test_captured_calls_replay(sp):
    """Calls captured into a CUDA graph after a warm-up call on the capturing stream (balanced schedule, the
    stream's scratch exists) and on a stream that never ran one (static schedule): replays give the eager result."""
    A = make_sparse(2048, 2048, 0.6, seed=21)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    B = torch.from_numpy(make_dense(16, 2048, seed=22)).cuda()
    eager = sp.spmm(W, B, split_k=1)
    torch.cuda.synchronize()
    sp.set_schedule(sp.SCHEDULE_BALANCED)
    for warm in (True, False):
        st = torch.cuda.Stream()
        out = torch.zeros((16, 2048), dtype=torch.float16, device="cuda")
        ws = torch.empty(2 * 16 * 2048, dtype=torch.float16, device="cuda")
        if warm:
            with torch.cuda.stream(st):
                sp.spmm(W, B, split_k=1, out=out, stream=st)
            st.synchronize()
            out.zero_()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            sp.spmm(W, B, split_k=1, out=out, stream=st)
            sp.spmm(W, B, split_k=2, out=out, workspace=ws, stream=st)
            sp.spmm(W, B, split_k=1, out=out, stream=st)
        for _ in range(3):
            out.zero_()
            g.replay()
            torch.cuda.synchronize()
            got, want = out.float(), eager.float()
            assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())
    sp.set_schedule(sp.SCHEDULE_AUTO)
    assert sp.device_status() == 0


def test_many_short_work_items_per_sm(sp):
    """300 row blocks of 5 k-tiles: every SM runs several work items whose last pipeline stage is partly empty."""
    M, K, N = 128 * 300, 64 * 5, 16
    A = make_sparse(M, K, 0.5, seed=31)
    B = make_dense(N, K, seed=32)
    for sk in (1, 2):
        _assert_close(_run(sp, A, B, sk), oracle.gemm_f32(A, B))
    assert sp.device_status() == 0


def test_spmm_from_reference_format_host_arrays(sp):
    """Arrays produced by the reference-format host encoder, uploaded as FT's loader would, max_nnz rounded to 64."""
    A = make_sparse(384, 640, 0.6, seed=77)
    B = make_dense(16, 640, seed=78)
    h = sp.init_sparse_matrix_a_bitmap(A)
    if h.max_nnz % 64:
        h.max_nnz = (h.max_nnz // 64 + 1) * 64   # reference csrc/SpMM_API.cuh:284-286
    W = sp.to_device(h)
    C = sp.spmm(W, torch.from_numpy(B).cuda(), split_k=2)
    torch.cuda.synchronize()
    _assert_close(C.cpu().numpy(), oracle.gemm_f32(A, B))


def test_split_k_chain_close_to_reference_rounding(sp):
    """Same split ranges and rounding points as the reference; accumulation order inside a range may differ."""
    A = make_sparse(256, 2048, 0.5, seed=5)
    B = make_dense(16, 2048, seed=6)
    for sk in (2, 5):
        C = _run(sp, A, B, sk).astype(np.float32)
        want = oracle.spmm_splitk_f16(A, B, sk).view(np.float16).astype(np.float32)
        assert np.abs(C - want).max() <= 4e-3 * np.abs(want).max()


def test_reduction_kernel_bit_exact(sp):
    rng = np.random.default_rng(4)
    M, N, sk = 256, 24, 7
    parts = rng.standard_normal((sk, N, M)).astype(np.float16)
    ws = torch.from_numpy(parts).cuda()
    C = torch.empty((N, M), dtype=torch.float16, device="cuda")
    sp.splitk_reduce(C, ws, M, N, sk)
    torch.cuda.synchronize()
    assert np.array_equal(C.cpu().numpy().view(np.uint16), oracle.splitk_reduce(parts, M, N, sk))


def test_special_values_propagate(sp):
    """inf in the weights reaches the output; NaN payloads are kept by the encoder and poison only their row."""
    A = make_sparse(128, 256, 0.5, seed=8)
    A[3, 10] = np.float16(np.inf)
    A[70, 200] = np.float16(np.nan)
    B = np.abs(make_dense(16, 256, seed=9)) + np.float16(0.5)
    C = _run(sp, A, B, 1).astype(np.float32)
    assert np.all(np.isinf(C[:, 3])) and np.all(np.isnan(C[:, 70]))
    ok_rows = [r for r in range(128) if r not in (3, 70)]
    ref = oracle.gemm_f32(A, B)
    assert np.abs(C[:, ok_rows] - ref[:, ok_rows]).max() <= REL * np.abs(ref[:, ok_rows]).max()


def test_linearity_at_full_size(sp):
    """OPT-30B FC1 shape (28672 x 7168, 60 %): S(B1 + B2) == S(B1) + S(B2) within fp16 rounding, and the result
    matches an fp32 product of the decoded weight on sampled rows."""
    M, K, N = 28672, 7168, 16
    g = torch.Generator(device="cuda").manual_seed(0x5EED0002)
    A = (torch.randn((M, K), device="cuda", generator=g) * 0.02).half()
    A[torch.rand((M, K), device="cuda", generator=g) < 0.6] = 0
    W = sp.encode_device(A)
    B1 = torch.randn((N, K), device="cuda", generator=g).half()
    B2 = torch.randn((N, K), device="cuda", generator=g).half()
    Bs = (B1.float() + B2.float()).half()
    C1 = sp.spmm(W, B1, split_k=1).float()
    C2 = sp.spmm(W, B2, split_k=1).float()
    Cs = sp.spmm(W, Bs, split_k=2).float()
    scale = float(Cs.abs().max())
    assert float((Cs - (C1 + C2)).abs().max()) <= 1e-2 * scale
    rows = torch.randint(0, M, (512,), device="cuda", generator=g)
    ref = Bs.float() @ A[rows].float().T
    assert float((Cs[:, rows] - ref).abs().max()) <= REL * float(ref.abs().max())
    # CPU oracle on a 256-row slab of the same matrix
    slab = A[1024:1280].cpu().numpy()
    want = oracle.gemm_f32(slab, Bs.cpu().numpy())
    assert np.abs(Cs[:, 1024:1280].cpu().numpy() - want).max() <= REL * np.abs(want).max()
    assert sp.device_status() == 0


def test_errors_launch_nothing(sp):
    A = make_sparse(128, 128, 0.5, seed=1)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    B = torch.zeros((16, 128), dtype=torch.float16, device="cuda")
    C = torch.full((16, 128), 7.0, dtype=torch.float16, device="cuda")
    with pytest.raises(sp.SpmmError):   # M not a multiple of 64
        sp.spmm_splitk_api_bitmap_v3(None, None, W.vals, W.gtile, W.mtile, W.bitmap, W.max_nnz, B, C, 100, 16, 128, None, 1)
    with pytest.raises(sp.SpmmError):   # split-K without a workspace
        sp.spmm_splitk_api_bitmap_v3(None, None, W.vals, W.gtile, W.mtile, W.bitmap, W.max_nnz, B, C, 128, 16, 128, None, 2)
    with pytest.raises(sp.SpmmError):   # more ranges than k-tiles
        sp.spmm(W, B, split_k=3)
    with pytest.raises(sp.SpmmError):   # misaligned activation pointer
        Bm = torch.zeros(16 * 128 + 8, dtype=torch.float16, device="cuda")[1:16 * 128 + 1].view(16, 128)
        sp.spmm_splitk_api_bitmap_v3(None, None, W.vals, W.gtile, W.mtile, W.bitmap, W.max_nnz, Bm, C, 128, 16, 128, None, 1)
    torch.cuda.synchronize()
    assert float(C.min()) == 7.0 and float(C.max()) == 7.0


def test_stream_and_repeat_calls(sp):
    A = make_sparse(512, 1024, 0.6, seed=2)
    B = make_dense(16, 1024, seed=3)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bd = torch.from_numpy(B).cuda()
    ref = oracle.gemm_f32(A, B)
    s = torch.cuda.Stream()
    outs = []
    with torch.cuda.stream(s):
        for sk in (1, 2, 4, 1, 2):
            outs.append(sp.spmm(W, Bd, split_k=sk, stream=s))
    s.synchronize()
    for C in outs:
        _assert_close(C.cpu().numpy(), ref)


def test_entry_point_allocates_nothing_until_spb_init(sp):
    """spb_spmm_bitmap_v3 on a stream spb_init was never called for: no device memory is taken (the balanced
    schedule's scratch is created by spb_init only) and the result is right; after spb_init the scratch exists."""
    import ctypes
    from spmspm_b200 import _lib
    lib = _lib.load()
    A = make_sparse(5120, 1024, 0.6, seed=91)
    B = torch.from_numpy(make_dense(16, 1024, seed=92)).cuda()
    W = sp.encode_device(torch.from_numpy(A).cuda())
    ref = oracle.gemm_f32(A, B.cpu().numpy())
    out = torch.zeros((16, 5120), dtype=torch.float16, device="cuda")
    st = torch.cuda.Stream()
    sp.set_schedule(sp.SCHEDULE_BALANCED)
    try:
        def call():
            code = lib.spb_spmm_bitmap_v3(ctypes.c_void_p(st.cuda_stream), None, ctypes.c_void_p(W.vals.data_ptr()),
                                          ctypes.c_void_p(W.gtile.data_ptr()), ctypes.c_void_p(W.mtile.data_ptr()),
                                          ctypes.c_void_p(W.bitmap.data_ptr()), ctypes.c_void_p(W.max_nnz.data_ptr()),
                                          ctypes.c_void_p(B.data_ptr()), ctypes.c_void_p(out.data_ptr()), 5120, 16, 1024,
                                          None, 1)
            assert code == 0, _lib.last_error()
            st.synchronize()
        torch.cuda.synchronize()
        call()                                   # first call on the device may load the module
        free0 = torch.cuda.mem_get_info()[0]
        call()
        assert torch.cuda.mem_get_info()[0] == free0
        _assert_close(out.cpu().numpy(), ref)
        sp.init(st)
        assert torch.cuda.mem_get_info()[0] < free0
        out.zero_()
        call()                                   # now under the balanced schedule
        _assert_close(out.cpu().numpy(), ref)
    finally:
        sp.set_schedule(sp.SCHEDULE_AUTO)
    assert sp.device_status() == 0


def test_more_streams_than_scratch_sets_and_release(sp):
    """A process that keeps creating streams: once the device's scratch sets are taken, calls on further streams run
    the static schedule (no error, same tolerance); spb_release gives a set back."""
    from spmspm_b200 import _lib
    A = make_sparse(512, 1024, 0.6, seed=301)
    B = torch.from_numpy(make_dense(16, 1024, seed=302)).cuda()
    W = sp.encode_device(torch.from_numpy(A).cuda())
    ref = oracle.gemm_f32(A, B.cpu().numpy())
    scale = float(np.abs(ref).max())
    streams = [torch.cuda.Stream(priority=p) for p in (0, -1) for _ in range(20)]   # torch hands out pooled streams
    seen = set()
    for st in streams:
        with torch.cuda.stream(st):
            got = sp.spmm(W, B, split_k=2)
        st.synchronize()
        seen.add(st.cuda_stream)
        assert float(np.abs(got.cpu().numpy().astype(np.float32) - ref).max()) <= 1e-2 * scale
    lib = _lib.load()
    for st in streams:                                       # give back whatever these streams took
        sp.release(st)
    sp.release(torch.cuda.current_stream())                  # at least one set is free now
    try:
        cudart = ctypes.CDLL("libcudart.so.12")
    except OSError:
        cudart = ctypes.CDLL("libcudart.so")
    extra, refused = [], None
    for _ in range(40):                                      # raw streams until spb_init refuses
        h = ctypes.c_void_p()
        assert cudart.cudaStreamCreate(ctypes.byref(h)) == 0
        if lib.spb_init(h) != 0:
            refused = h
            break
        extra.append(h)
    assert refused is not None and len(extra) >= 1 and b"no scratch set left" in lib.spb_last_error()
    assert lib.spb_release(extra[0]) == 0
    assert lib.spb_init(refused) == 0                        # the freed set goes to the stream that was refused
    for h in extra + [refused]:
        assert lib.spb_release(h) == 0
        assert cudart.cudaStreamDestroy(h) == 0
    got = sp.spmm(W, B, split_k=2)                           # the default stream gets a set again on its next call
    torch.cuda.synchronize()
    assert float(np.abs(got.cpu().numpy().astype(np.float32) - ref).max()) <= 1e-2 * scale
    assert sp.device_status() == 0
