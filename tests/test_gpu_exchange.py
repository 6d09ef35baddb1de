"""SpMM fused with the all-gather of its output rows (spb_spmm_bitmap_v3_allgather, spb_wait_flags).

On one GPU the exchange runs with a single rank (the kernel stores into its own buffer, numbers the launch,
writes its own flag; the consumer waits on it), which covers every device-side step.  With two or more GPUs
the same sequence runs as two ranks over symmetric memory in child processes.
"""
import ctypes
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import oracle  # noqa: E402
from conftest import make_dense, make_sparse  # noqa: E402


def test_single_rank_exchange_and_chained_wait(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200 as sp
    sp.reset_device_status()
    M_full, K, N, lo = 1024, 1024, 16, 256          # a 512-row shard written at rows 256..767 of a 1024-row buffer
    A = make_sparse(512, K, 0.6, seed=41)
    B = make_dense(N, K, seed=42)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bd = torch.from_numpy(B).cuda()
    ref = oracle.gemm_f32(A, B)
    bufs = [torch.full((N, M_full), 7.0, dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(3, dtype=torch.int32, device="cuda") for _ in range(2)]
    cptr = [(ctypes.c_void_p * 1)(b.data_ptr()) for b in bufs]
    fptr = [(ctypes.c_void_p * 1)(f.data_ptr()) for f in flags]
    # exchange 1 into buffer 0, consumed by a wait kernel
    sp.spmm_allgather(W, Bd, cptr[0], fptr[0], 1, 0, M_full, lo)
    sp.wait_flags(flags[0], 1)
    # a chain: buffer 1, then buffer 0 again by a launch that itself waits for buffer 1's exchange, then a wait kernel
    sp.spmm_allgather(W, Bd, cptr[1], fptr[1], 1, 0, M_full, lo)
    sp.spmm_allgather(W, Bd, cptr[0], fptr[0], 1, 0, M_full, lo, B_flags=flags[1])
    sp.wait_flags(flags[0], 1)
    torch.cuda.synchronize()
    first = bufs[0].clone()
    # the same with Split_K = 3: the reduction kernel stores the rows and writes the flag
    sp.spmm_allgather(W, Bd, cptr[1], fptr[1], 1, 0, M_full, lo, split_k=3)
    sp.spmm_allgather(W, Bd, cptr[0], fptr[0], 1, 0, M_full, lo, B_flags=flags[1], split_k=3)
    sp.wait_flags(flags[0], 1)
    torch.cuda.synchronize()
    assert float((bufs[0].float() - first.float()).abs().max()) <= 4e-3 * float(first.float().abs().max())
    for b in bufs:
        out = b.cpu().numpy().astype(np.float32)
        got = out[:, lo:lo + 512]
        assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()
        assert np.all(out[:, :lo] == 7.0) and np.all(out[:, lo + 512:] == 7.0)   # only the shard's rows were written
    f0, f1 = flags[0].cpu().tolist(), flags[1].cpu().tolist()
    assert f0 == [3, 3, 3]      # three launches numbered 1..3; three exchanges consumed
    assert f1 == [2, 2, 2]      # two launches, each consumed by the chained launch after it
    assert sp.device_status() == 0


def test_single_rank_allreduce_path(lib_built):
    """K-split entry points with one rank: the partial goes to slot 0 of the local buffer, the finish kernel waits for
    the flag and sums one slot, which must reproduce the plain SpMM bit for bit (same kernel, one rounding each)."""
    import spmspm_b200 as sp
    sp.reset_device_status()
    M, K, N = 512, 1024, 16
    A = make_sparse(M, K, 0.6, seed=61)
    B = make_dense(N, K, seed=62)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bd = torch.from_numpy(B).cuda()
    want = sp.spmm(W, Bd, split_k=1)
    parts = torch.full((1, N, M), 5.0, dtype=torch.float16, device="cuda")
    flags = torch.zeros(3, dtype=torch.int32, device="cuda")
    out = torch.zeros((N, M), dtype=torch.float16, device="cuda")
    pp, fp = (ctypes.c_void_p * 1)(parts.data_ptr()), (ctypes.c_void_p * 1)(flags.data_ptr())
    for sk in (1, 3):
        sp.spmm_allreduce(W, Bd, pp, fp, 1, 0, split_k=sk)
        sp.allreduce_finish(out, parts, flags, 1)
        torch.cuda.synchronize()
        got = out.cpu().numpy().astype(np.float32)
        ref = oracle.gemm_f32(A, B)
        assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()
        if sk == 1:
            assert np.array_equal(out.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
    assert flags.cpu().tolist() == [2, 2, 2]
    assert sp.device_status() == 0


def test_exchange_argument_checks(lib_built):
    import spmspm_b200 as sp
    A = make_sparse(128, 128, 0.5, seed=1)
    W = sp.encode_device(torch.from_numpy(A).cuda())
    Bd = torch.zeros((16, 128), dtype=torch.float16, device="cuda")
    buf = torch.full((16, 256), 3.0, dtype=torch.float16, device="cuda")
    flg = torch.zeros(3, dtype=torch.int32, device="cuda")
    c, f = (ctypes.c_void_p * 1)(buf.data_ptr()), (ctypes.c_void_p * 1)(flg.data_ptr())
    with pytest.raises(sp.SpmmError):      # shard does not fit below M_full
        sp.spmm_allgather(W, Bd, c, f, 1, 0, 256, 192)
    with pytest.raises(sp.SpmmError):      # rank outside the peers
        sp.spmm_allgather(W, Bd, c, f, 1, 1, 256, 0)
    torch.cuda.synchronize()
    assert float(buf.min()) == 3.0 and float(buf.max()) == 3.0 and flg.cpu().tolist() == [0, 0, 0]


_CHILD = r"""
import os, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import numpy as np, torch, torch.distributed as dist
import spmspm_b200 as sp
from spmspm_b200 import dist as spd
from conftest import make_dense, make_sparse
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
M, K, N = 2048, 1024, 16
A = make_sparse(M, K, 0.6, seed=51); B = torch.from_numpy(make_dense(N, K, seed=52)).to(dev)
lo, hi = spd.row_shard_bounds(M, world, rank)
W = sp.encode_device(torch.from_numpy(A[lo:hi].copy()).to(dev))
ref = sp.spmm(sp.encode_device(torch.from_numpy(A).to(dev)), B, split_k=1).float()
pg = spd.PeerGather(N, M, dev)
bad = 0
def check(out):
    torch.cuda.synchronize()
    return int(float((out.float() - ref).abs().max()) > 2e-3 * float(ref.abs().max()))
pg.spmm(W, B, lo)                               # consumed by a wait kernel
bad += check(pg.wait())
dist.barrier()
pg.spmm(W, B, lo, split_k=2)                    # a chain: each launch waits for the exchange before it
pg.spmm(W, B, lo, after=pg)
pg.spmm(W, B, lo, after=pg, split_k=2)
bad += check(pg.wait())
dist.barrier()
# K-split: every rank multiplies its column slice, the partials are summed over the ranks (one-shot all-reduce)
klo, khi = spd.col_shard_bounds(K, world, rank)
Wk = sp.encode_device(torch.from_numpy(np.ascontiguousarray(A[:, klo:khi])).to(dev))
Bk = B[:, klo:khi].contiguous()
pr = spd.PeerReduce(N, M, dev)
for sk in (1, 2, 1):
    pr.spmm(Wk, Bk, split_k=sk)
    out = pr.reduce()
    torch.cuda.synchronize()
    bad += int(float((out.float() - ref).abs().max()) > 4e-3 * float(ref.abs().max()))
dist.barrier()
bad += int(sp.device_status() != 0)
open(os.path.join(sys.argv[2], f"result_{rank}"), "w").write(str(bad))   # the ranks' prints would interleave
dist.barrier(); os._exit(0 if bad == 0 else 1)
"""


def test_two_ranks_over_symmetric_memory(lib_built, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script), root, str(tmp_path)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    for rank in (0, 1):
        assert (tmp_path / f"result_{rank}").read_text() == "0"


def test_wait_that_runs_out_sets_the_status_word_and_leaves_the_context_usable(lib_built):
    """A rank that never sends: the flag wait gives up after its bounded number of polls (about half a second),
    reports through the device status word, and the next call works.  Nothing faults or hangs."""
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200 as sp
    sp.reset_device_status()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")      # two ranks: nobody ever writes entries 0 and 1
    sp.wait_flags(flags, 2)
    torch.cuda.synchronize()
    assert sp.device_status() == 1                                 # kStatusWaitTimeout
    assert flags.cpu().tolist() == [0, 0, 0, 1]                    # the wait was counted, nothing arrived
    sp.reset_device_status()
    assert sp.device_status() == 0
    A = make_sparse(256, 512, 0.6, seed=77)
    B = torch.from_numpy(make_dense(16, 512, seed=78)).cuda()
    got = sp.spmm(sp.encode_device(torch.from_numpy(A).cuda()), B, split_k=1).cpu().numpy().astype(np.float32)
    ref = oracle.gemm_f32(A, B.cpu().numpy())
    assert float(np.abs(got - ref).max()) <= 1e-2 * float(np.abs(ref).max())
    assert sp.device_status() == 0
