"""Host-buffer front end for a fixed batch of SpMMs: the caller keeps activations and results in (pinned) host memory,
as a serving process does that receives requests from the network and the reference's FasterTransformer host code does
with its input ids and output logits; the library moves them.

A `HostBatch` is built once for a list of (weight, N) pairs.  It owns two sets of staging buffers (one packed pinned
host buffer and one packed device buffer for all activations, the same for all results) and, per set, the batch's
SpMMs captured into one CUDA graph.  `submit(s)` enqueues, for set `s`: one host-to-device copy of the packed
activations on a copy stream, the graph on the compute stream, one device-to-host copy of the packed results on a
second copy stream, chained by events; it returns at once.  `wait(s)` blocks the host until set `s`'s results are in
host memory.  Submitting set 1 while set 0 is in flight overlaps the copies of one batch with the SpMMs of the other.
There is no CPU path: the SpMMs are spmspm_b200.spmm."""
import torch

from . import api


class HostBatch:
    def __init__(self, items, device, split_k=None, sets=2, streams=None, body=None, out_cols=None, ready=None):
        """items: list of (BitmapMatrix W, N); split_k: optional list of Split_K values (default: the library's);
        streams: (copy-in, compute, copy-out) streams to share with other batches (default: three new ones; every
        compute stream takes one of the library's per-stream scratch sets).
        body(s, ins, outs): replaces the plain loop of SpMMs for staging set s (ins / outs: the device views of the
        packed buffers), e.g. SpMMs of row shards followed by an exchange between GPUs; it is captured into the set's
        graph.  out_cols: result columns per item when they differ from W.M (gathered rows of a sharded weight).
        ready(): called after the buffers exist and before each set's first (uncaptured) run, e.g. a barrier between
        the processes of a body that exchanges data, whose device-side waits are bounded."""
        self.device = torch.device(device)
        self.items = list(items)
        self.split_k = [sk if sk else api.suggest_split_k(W.M, N, W.K)
                        for (W, N), sk in zip(self.items, split_k or [None] * len(self.items))]
        n_in = sum(N * W.K for W, N in self.items)
        self.out_cols = list(out_cols) if out_cols is not None else [W.M for W, N in self.items]
        self.body = body
        n_out = sum(N * m for (W, N), m in zip(self.items, self.out_cols))
        ws_elems = max([sk * N * W.M for (W, N), sk in zip(self.items, self.split_k) if sk > 1] or [8])
        self.h_in = [torch.empty(n_in, dtype=torch.float16).pin_memory() for _ in range(sets)]
        self.h_out = [torch.empty(n_out, dtype=torch.float16).pin_memory() for _ in range(sets)]
        self.d_in = [torch.empty(n_in, dtype=torch.float16, device=self.device) for _ in range(sets)]
        self.d_out = [torch.empty(n_out, dtype=torch.float16, device=self.device) for _ in range(sets)]
        self.ws = torch.empty(ws_elems, dtype=torch.float16, device=self.device)
        self.s_in, self.s_run, self.s_out = streams or tuple(torch.cuda.Stream(self.device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(sets)]
        self.ev_run = [torch.cuda.Event() for _ in range(sets)]
        self.ev_out = [torch.cuda.Event() for _ in range(sets)]
        self._busy = [False] * sets
        self.graphs = []
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.s_run):
                api._init_if_possible(self.s_run)   # without a free scratch set the batch runs the static schedule
            for s in range(sets):
                if ready is not None:
                    ready()
                with torch.cuda.stream(self.s_run):
                    self._enqueue(s)                      # warm-up outside capture
                self.s_run.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.s_run):
                    self._enqueue(s)
                self.graphs.append(g)

    def _views(self, flat, cols):
        out, at = [], 0
        for (W, N), c in zip(self.items, cols):
            out.append(flat[at:at + N * c].view(N, c))
            at += N * c
        return out

    def inputs(self, s):
        """Host views [N, K] of set s's packed activation buffer, one per item: the caller writes them."""
        return self._views(self.h_in[s], [W.K for W, N in self.items])

    def outputs(self, s):
        """Host views [N, M] of set s's packed result buffer, valid after wait(s)."""
        return self._views(self.h_out[s], self.out_cols)

    def _enqueue(self, s):
        ins, outs = self._views(self.d_in[s], [W.K for W, N in self.items]), self._views(self.d_out[s], self.out_cols)
        if self.body is not None:
            self.body(s, ins, outs)
            return
        for (W, N), sk, x, y in zip(self.items, self.split_k, ins, outs):
            api.spmm(W, x, split_k=sk, out=y, workspace=self.ws)

    def submit(self, s):
        if self._busy[s]:
            self.wait(s)
        with torch.cuda.stream(self.s_in):
            self.d_in[s].copy_(self.h_in[s], non_blocking=True)
            self.ev_in[s].record()
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[s])
            self.graphs[s].replay()
            self.ev_run[s].record()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[s])
            self.h_out[s].copy_(self.d_out[s], non_blocking=True)
            self.ev_out[s].record()
        self._busy[s] = True

    def wait(self, s):
        if self._busy[s]:
            self.ev_out[s].synchronize()
            self._busy[s] = False

    def join(self, stream=None):
        """Make `stream` (default: the current one) wait for everything submitted so far, without blocking the host."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s, busy in enumerate(self._busy):
            if busy:
                stream.wait_event(self.ev_out[s])

    def close(self):
        """Wait for everything submitted and give the compute stream's scratch back to the library."""
        for s in range(len(self._busy)):
            self.wait(s)
        with torch.cuda.device(self.device):
            api.release(self.s_run)

    def bytes_per_batch(self):
        return 2 * self.h_in[0].numel(), 2 * self.h_out[0].numel()
