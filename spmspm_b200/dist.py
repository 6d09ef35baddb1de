"""Tensor-parallel use of the SpMM, one process per GPU (torch.distributed).

The reference library is single-GPU; its caller (FasterTransformer) splits QKV and FC1 by
output rows (M-split, every rank sees the whole activation) and out-proj / FC2 by input
columns (K-split, followed by an all-reduce); see the per-rank shapes in
end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:284-285.  These helpers do the
same two splits around the local SpMM.  The collectives work on whatever device the tensors
live on, so the host logic is exercised on CPU ranks with the gloo backend.
"""
import torch
import torch.distributed as dist


def row_shard_bounds(M, world, rank):
    """Rows [lo, hi) owned by `rank` under an even M-split; M/world must be a multiple of 64."""
    if M % (64 * world):
        raise ValueError(f"M={M} cannot be split into {world} shards of whole 64-row tiles")
    per = M // world
    return rank * per, (rank + 1) * per


def col_shard_bounds(K, world, rank):
    if K % (64 * world):
        raise ValueError(f"K={K} cannot be split into {world} shards of whole 64-column tiles")
    per = K // world
    return rank * per, (rank + 1) * per


def all_gather_rows(local_C, group=None):
    """local_C [N, M/P] on every rank -> [N, M] (rank r's rows at columns r*M/P ...)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_C
    N, Ms = local_C.shape
    buf = torch.empty((world, N, Ms), dtype=local_C.dtype, device=local_C.device)
    if local_C.is_cuda:
        dist.all_gather_into_tensor(buf, local_C.contiguous(), group=group)
    else:  # gloo has no flat-tensor variant
        dist.all_gather(list(buf.unbind(0)), local_C.contiguous(), group=group)
    return buf.permute(1, 0, 2).reshape(N, world * Ms)


def all_reduce_partial(local_C, group=None):
    """Sum of the ranks' partial [N, M] outputs, in place (fp16 on the wire, like FasterTransformer)."""
    if dist.get_world_size(group) > 1:
        dist.all_reduce(local_C, op=dist.ReduceOp.SUM, group=group)
    return local_C


def spmm_m_sharded(W_local, B, compute, group=None, **kw):
    """QKV / FC1 style: W_local holds this rank's rows; returns the gathered [N, M]."""
    return all_gather_rows(compute(W_local, B, **kw), group)


def spmm_k_sharded(W_local, B_local, compute, group=None, **kw):
    """out-proj / FC2 style: W_local holds this rank's columns, B_local the matching slice of the activations."""
    return all_reduce_partial(compute(W_local, B_local, **kw), group)
