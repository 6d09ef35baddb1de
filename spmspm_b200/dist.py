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


class PeerGather:
    """Output buffers for the SpMM fused with the all-gather of its output rows (spb_spmm_bitmap_v3_allgather).

    Every rank allocates `slots` output buffers [N, M_full] and a flag array per buffer in symmetric memory
    (torch.distributed._symmetric_memory: the peers' copies are mapped into this process).  `spmm(W_local, B)`
    makes this rank's SpMM store its rows into every rank's current buffer; `wait()` enqueues the bounded wait for
    all ranks' rows and returns the gathered [N, M_full] tensor of this rank.  Calls alternate between the
    buffers, so a buffer is rewritten only after `slots - 1` further exchanges; every rank must make the same
    sequence of calls.
    """

    def __init__(self, N, M_full, device, group=None, slots=2):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("PeerGather serves up to 8 ranks")
        self.N, self.M_full = N, M_full
        self.bufs, self.flags, self._cptrs, self._fptrs = [], [], [], []
        for _ in range(slots):
            buf = symm_mem.empty((N, M_full), dtype=torch.float16, device=device)
            flg = symm_mem.empty((self.world + 2,), dtype=torch.int32, device=device)
            buf.zero_()
            flg.zero_()
            hb = symm_mem.rendezvous(buf, self.group.group_name)
            hf = symm_mem.rendezvous(flg, self.group.group_name)
            self.bufs.append(buf)
            self.flags.append(flg)
            self._cptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hb.buffer_ptrs]))
            self._fptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hf.buffer_ptrs]))
        torch.cuda.synchronize(device)
        dist.barrier(self.group)   # every rank's buffers and flags are zero before anybody writes
        self._turn = 0

    def spmm(self, W_local, B, row_offset, after=None, split_k=1, workspace=None, stream=None):
        """Enqueue this rank's SpMM; its rows [row_offset, row_offset + W_local.M) go to every rank's buffer.

        `after`: a PeerGather whose current exchange produced B (its `gathered()` buffer): the kernel itself waits
        for that exchange before it reads B, and that exchange counts as consumed."""
        from . import api
        flags = None
        if after is not None:   # before this call's own buffer is chosen: `after` may be this object
            flags = after.flags[after._turn % len(after.bufs)]
            after._turn += 1
        slot = self._turn % len(self.bufs)
        api.spmm_allgather(W_local, B, self._cptrs[slot], self._fptrs[slot], self.world, self.rank, self.M_full,
                           row_offset, B_flags=flags, split_k=split_k, workspace=workspace, stream=stream)
        return slot

    def gathered(self):
        """This rank's buffer of the current exchange (complete only after `wait()` or a consuming `spmm(after=)`)."""
        return self.bufs[self._turn % len(self.bufs)]

    def wait(self, stream=None):
        """Enqueue the wait for all ranks' rows of the current exchange; returns this rank's gathered tensor."""
        from . import api
        slot = self._turn % len(self.bufs)
        api.wait_flags(self.flags[slot], self.world, stream=stream)
        self._turn += 1
        return self.bufs[slot]


class PeerReduce:
    """Partial-result buffers for the K-split SpMM with the one-shot all-reduce over peer stores
    (spb_spmm_bitmap_v3_allreduce / spb_allreduce_finish).

    Every rank allocates `slots` buffers [world, N, M] and a flag array per buffer in symmetric memory.
    `spmm(W_local, B_local)` makes this rank's SpMM (its column shard of the weight times its slice of the
    activations) store its fp16 partial into slot `rank` of every rank's current buffer; `reduce()` enqueues the
    bounded wait for all ranks' partials and their sum (fp32, rank order, one rounding) and returns the [N, M]
    result.  Calls alternate between the buffers; every rank must make the same sequence of calls.
    """

    def __init__(self, N, M, device, group=None, slots=2):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("PeerReduce serves up to 8 ranks")
        self.N, self.M = N, M
        self.bufs, self.flags, self._pptrs, self._fptrs, self.outs = [], [], [], [], []
        for _ in range(slots):
            buf = symm_mem.empty((self.world, N, M), dtype=torch.float16, device=device)
            flg = symm_mem.empty((self.world + 2,), dtype=torch.int32, device=device)
            buf.zero_()
            flg.zero_()
            hb = symm_mem.rendezvous(buf, self.group.group_name)
            hf = symm_mem.rendezvous(flg, self.group.group_name)
            self.bufs.append(buf)
            self.flags.append(flg)
            self._pptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hb.buffer_ptrs]))
            self._fptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hf.buffer_ptrs]))
            self.outs.append(torch.empty((N, M), dtype=torch.float16, device=device))
        torch.cuda.synchronize(device)
        dist.barrier(self.group)   # every rank's buffers and flags are zero before anybody writes
        self._turn = 0

    def spmm(self, W_local, B_local, split_k=1, workspace=None, stream=None):
        """Enqueue this rank's SpMM; its partial [N, M] goes to slot `rank` of every rank's current buffer."""
        from . import api
        slot = self._turn % len(self.bufs)
        api.spmm_allreduce(W_local, B_local, self._pptrs[slot], self._fptrs[slot], self.world, self.rank,
                           split_k=split_k, workspace=workspace, stream=stream)
        return slot

    def reduce(self, out=None, stream=None, bias=None, residual=None, activation=0):
        """Enqueue the wait for all ranks' partials of the current exchange and their sum (then the linear layer's
        tail: bias, activation, residual, see spmspm_b200.linear); returns the [N, M] result."""
        from . import api
        slot = self._turn % len(self.bufs)
        out = self.outs[slot] if out is None else out
        api.allreduce_finish(out, self.bufs[slot], self.flags[slot], self.world, stream=stream, bias=bias,
                             residual=residual, activation=activation)
        self._turn += 1
        return out
