"""world_size-2 gloo test of the tensor-parallel host logic (M-split + all-gather, K-split + all-reduce).

The local product is computed with the CPU oracle here: this test covers sharding and the
collectives, not the CUDA kernel.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, make_dense, make_sparse


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from spmspm_b200 import dist as spd
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = 256, 512, 8
        A = make_sparse(M, K, 0.6, 42)
        B = make_dense(N, K, 43)
        full = oracle.gemm_f32(A, B)

        def compute(W, Bt):  # W: dense fp16 shard (numpy), Bt: torch [N,K']
            return torch.from_numpy(oracle.gemm_f32(W, Bt.numpy()))

        lo, hi = spd.row_shard_bounds(M, world, rank)
        C = spd.spmm_m_sharded(A[lo:hi], torch.from_numpy(B), compute)
        ok_m = np.allclose(C.numpy(), full, rtol=0, atol=1e-6)
        klo, khi = spd.col_shard_bounds(K, world, rank)
        C2 = spd.spmm_k_sharded(np.ascontiguousarray(A[:, klo:khi]), torch.from_numpy(np.ascontiguousarray(B[:, klo:khi])),
                                compute)
        ok_k = np.allclose(C2.numpy(), full, rtol=0, atol=1e-4)
        q.put((rank, ok_m, ok_k))
    except Exception as e:  # report instead of leaving the parent waiting
        q.put((rank, False, repr(e)))
    finally:
        dist.destroy_process_group()


def test_m_split_and_k_split_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(60)
    assert all(ok_m is True and ok_k is True for _, ok_m, ok_k in res), res


def test_shard_bounds_reject_ragged_splits():
    from spmspm_b200 import dist as spd
    import pytest
    assert spd.row_shard_bounds(512, 4, 1) == (128, 256)
    with pytest.raises(ValueError):
        spd.row_shard_bounds(320, 4, 0)
