"""A tensor-parallel OPT decoder layer whose four linear layers run through the bitmap SpMM.

The reference library is the GEMM of FasterTransformer's OPT decoder: its patch routes the fused QKV projection,
the attention output projection and the two FFN matrices through SpMM_SplitK_API_bitmap_v3
(third_party/ft_spinfer.patch:681-696, 811-826 FFN; 1459-1474, 1558-1573 decode attention; 1704-1718, 1796-1811
context attention) and splits them over the tensor-parallel ranks as the converter lays the files out
(end2end_inference/ft_tools/huggingface_opt_convert_Phase1.py:67-99, per-rank shapes
huggingface_opt_convert_Phase2.py:284-285):

    QKV  [3h/P, h]   by output rows (each rank its heads' q, k and v rows)      no communication
    out  [h, h/P]    by input columns                                           all-reduce of the [N, h] partials
    FC1  [4h/P, h]   by output rows, ReLU                                       no communication
    FC2  [h, 4h/P]   by input columns                                           all-reduce

This module is the harness for that call sequence: layer norms, attention (torch's scaled_dot_product_attention on a
static key/value cache) and residuals are stock PyTorch; the linear layers are spmspm_b200.spmm, and the two
all-reduces are either the one-shot exchange over peer stores (spmspm_b200.dist.PeerReduce) or NCCL.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import api
from . import dist as spd


def _gen(shape, seed, device, scale):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g) * scale).half()


def gen_pruned(shape, seed, device, sparsity, scale=0.02):
    """fp16 N(0, scale^2) weights under a seeded Bernoulli(keep = 1 - sparsity) mask; kept values are never zero."""
    g = torch.Generator(device=device).manual_seed(seed)
    A = (torch.randn(shape, device=device, generator=g) * scale).half()
    A = torch.where(A == 0, torch.full_like(A, 6.1035e-05), A)
    keep = torch.rand(shape, device=device, generator=g) >= sparsity
    return A * keep


class SparseOptDecoderLayer:
    """One OPT decoder layer (pre-layer-norm, ReLU FFN), tensor-parallel over `group`.

    hidden % (64 * world) == 0 and heads % world == 0.  `reduce`: "peer" (one-shot all-reduce over peer stores),
    "nccl", or "none" for a single rank.  The key/value cache is static ([batch, heads/P, max_len, head_dim]) and the
    position is a device counter, so that a decode step has fixed shapes and can be captured into a CUDA graph.
    """

    def __init__(self, hidden, heads, ffn, sparsity, device, batch, max_len, group=None, reduce="peer", seed=0x5EED0005,
                 keep_dense=False, fused=True):
        self.fused = fused   # bias / ReLU / residual inside the SpMM's launches (spb_linear_bitmap_v3) or as torch ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        P, r = self.world, self.rank
        if hidden % (64 * P) or heads % P or ffn % (64 * P) or hidden % heads:
            raise ValueError("hidden, ffn must be multiples of 64 * world and heads a multiple of world")
        self.h, self.heads, self.ffn, self.d = hidden, heads, ffn, hidden // heads
        self.hp, self.fp_, self.heads_p = hidden // P, ffn // P, heads // P
        self.batch, self.max_len, self.device = batch, max_len, device
        self.reduce_kind = reduce if P > 1 else "none"
        dev = device
        # full weights are generated on every rank from the same seeds and sharded; only the shards are kept
        lo, hi = r * self.hp, (r + 1) * self.hp
        Wq, Wk, Wv = (gen_pruned((hidden, hidden), seed + i, dev, sparsity) for i in range(3))
        qkv = torch.cat([Wq[lo:hi], Wk[lo:hi], Wv[lo:hi]], 0).contiguous()          # [3h/P, h]
        Wo = gen_pruned((hidden, hidden), seed + 3, dev, sparsity)[:, lo:hi].contiguous()         # [h, h/P]
        W1 = gen_pruned((ffn, hidden), seed + 4, dev, sparsity)[r * self.fp_:(r + 1) * self.fp_].contiguous()
        W2 = gen_pruned((hidden, ffn), seed + 5, dev, sparsity)[:, r * self.fp_:(r + 1) * self.fp_].contiguous()
        del Wq, Wk, Wv
        self.dense = {"qkv": qkv, "out": Wo, "fc1": W1, "fc2": W2} if keep_dense else None
        self.W = {k: api.encode_device(v) for k, v in (("qkv", qkv), ("out", Wo), ("fc1", W1), ("fc2", W2))}
        bq = _gen((3, hidden), seed + 6, dev, 0.02)
        self.b_qkv = bq[:, lo:hi].reshape(-1).contiguous()
        self.b_out = _gen((hidden,), seed + 7, dev, 0.02)
        self.b_fc1 = _gen((ffn,), seed + 8, dev, 0.02)[r * self.fp_:(r + 1) * self.fp_].contiguous()
        self.b_fc2 = _gen((hidden,), seed + 9, dev, 0.02)
        self.ln1_w, self.ln1_b = torch.ones(hidden, dtype=torch.float16, device=dev), torch.zeros(hidden, dtype=torch.float16, device=dev)
        self.ln2_w, self.ln2_b = self.ln1_w.clone(), self.ln1_b.clone()
        self.k_cache = torch.zeros((batch, self.heads_p, max_len, self.d), dtype=torch.float16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.pos = torch.zeros(1, dtype=torch.int64, device=dev)            # tokens in the cache
        self.arange = torch.arange(max_len, device=dev)
        self.split = {}
        self._peer = {}
        # split-K workspace: up to 4 partial results at 512 activation rows (more partials at decode batch sizes)
        self.ws = torch.empty(4 * 512 * max(hidden, 3 * self.hp, self.fp_), dtype=torch.float16, device=dev)

    # ---- linear layers -------------------------------------------------------------------------------------
    def _split_k(self, name, N):
        key = (name, N)
        if key not in self.split:
            W = self.W[name]
            sk = api.suggest_split_k(W.M, N, W.K)
            while sk > 1 and sk * N * W.M > self.ws.numel():
                sk -= 1
            self.split[key] = sk
        return self.split[key]

    def _linear(self, name, x, bias=None, residual=None, relu=False):
        """x [N, K_local] -> residual + act(x W^T + bias) [N, M_local]; with `fused` in the SpMM's own launches."""
        sk = self._split_k(name, x.shape[0])
        if self.fused:
            return api.linear(self.W[name], x, bias=bias, residual=residual, activation=api.ACT_RELU if relu else api.ACT_NONE,
                              split_k=sk, workspace=self.ws)
        return self._tail(api.spmm(self.W[name], x, split_k=sk, workspace=self.ws), bias, residual, relu)

    @staticmethod
    def _tail(y, bias, residual, relu):
        if bias is not None:
            y = y + bias
        if relu:
            y = torch.relu(y)
        if residual is not None:
            y = residual + y
        return y

    def _linear_reduced(self, name, x, bias, residual):
        """K-split linear layer: x [N, K/P] -> residual + (all-reduced x W^T + bias) [N, M]."""
        N = x.shape[0]
        if self.reduce_kind == "none":
            return self._linear(name, x, bias, residual)
        if self.reduce_kind == "peer":
            key = (name, N)
            if key not in self._peer:
                self._peer[key] = spd.PeerReduce(N, self.W[name].M, self.device, self.group, slots=1)
            pr = self._peer[key]
            pr.spmm(self.W[name], x, split_k=self._split_k(name, N), workspace=self.ws)
            if self.fused:
                return pr.reduce(bias=bias, residual=residual)
            return self._tail(pr.reduce(), bias, residual, False)
        y = self._linear(name, x)
        dist.all_reduce(y, group=self.group)
        return self._tail(y, bias, residual, False)

    def prepare(self, Ns):
        """Create the exchange buffers for the activation widths that will be used (symmetric-memory allocation is a
        collective and cannot happen inside a captured graph)."""
        if self.reduce_kind == "peer":
            for N in Ns:
                for name in ("out", "fc2"):
                    # one buffer each: the two reductions of a layer alternate, so a buffer is rewritten only after
                    # every rank has passed the other reduction, i.e. has consumed it; and a captured step then
                    # names the same buffers on every replay
                    if (name, N) not in self._peer:
                        self._peer[(name, N)] = spd.PeerReduce(N, self.W[name].M, self.device, self.group, slots=1)

    # ---- forward -------------------------------------------------------------------------------------------
    def reset(self):
        self.pos.zero_()

    def forward(self, x, T):
        """x [batch * T, h] (token-major within a sequence: row b * T + t), T new tokens per sequence appended at the
        cache position.  Returns [batch * T, h]."""
        Bn, hp, d = self.batch, self.hp, self.d
        h1 = F.layer_norm(x, (self.h,), self.ln1_w, self.ln1_b)
        qkv = self._linear("qkv", h1, self.b_qkv)                                    # [N, 3h/P]
        q, k, v = (t.reshape(Bn, T, self.heads_p, d).transpose(1, 2) for t in qkv.split(hp, dim=1))   # [B, H/P, T, d]
        idx = self.pos + self.arange[:T]                                             # device-side positions
        self.k_cache.index_copy_(2, idx, k.contiguous())
        self.v_cache.index_copy_(2, idx, v.contiguous())
        # key j is visible to query t when j <= pos + t
        mask = self.arange[None, :] <= (self.pos + self.arange[:T])[:, None]         # [T, max_len]
        attn = F.scaled_dot_product_attention(q, self.k_cache, self.v_cache, attn_mask=mask[None, None])
        attn = attn.transpose(1, 2).reshape(Bn * T, hp).contiguous()
        x = self._linear_reduced("out", attn, self.b_out, x)
        h2 = F.layer_norm(x, (self.h,), self.ln2_w, self.ln2_b)
        f1 = self._linear("fc1", h2, self.b_fc1, relu=True)
        x = self._linear_reduced("fc2", f1, self.b_fc2, x)
        self.pos += T
        return x

    def forward_dense_reference(self, x, T):
        """The same layer with fp32 torch matmuls on the dense shards (keep_dense=True, single rank): the numerics
        reference of the tests."""
        assert self.dense is not None and self.world == 1
        Bn, d = self.batch, self.d
        xf = x.float()
        h1 = F.layer_norm(xf, (self.h,), self.ln1_w.float(), self.ln1_b.float())
        qkv = (h1.half().float() @ self.dense["qkv"].float().t()).half().float() + self.b_qkv.float()
        q, k, v = (t.reshape(Bn, T, self.heads, d).transpose(1, 2) for t in qkv.split(self.h, dim=1))
        mask = torch.ones((T, T), dtype=torch.bool, device=x.device).tril()
        attn = F.scaled_dot_product_attention(q, k, v, attn_mask=mask[None, None])
        attn = attn.transpose(1, 2).reshape(Bn * T, self.h)
        xf = xf + (attn.half().float() @ self.dense["out"].float().t()) + self.b_out.float()
        h2 = F.layer_norm(xf, (self.h,), self.ln2_w.float(), self.ln2_b.float())
        f1 = torch.relu(h2.half().float() @ self.dense["fc1"].float().t() + self.b_fc1.float())
        return xf + (f1.half().float() @ self.dense["fc2"].float().t()) + self.b_fc2.float()


def generate_timed(layer, prompt_len, new_tokens, steps=1, warmup=1, use_graph=True):
    """Times `steps` generations of `new_tokens` tokens after a prompt of `prompt_len` tokens per sequence through one
    layer: one prefill pass (N = batch * prompt_len) and new_tokens decode passes (N = batch).  Returns
    (seconds per generation, seconds of the prefill, seconds per decode step).  The decode step is captured into a
    CUDA graph when use_graph is set (fixed shapes: static cache, device-side position)."""
    dev, B, h = layer.device, layer.batch, layer.h
    xp = _gen((B * prompt_len, h), 11, dev, 1.0)
    xd = _gen((B, h), 12, dev, 1.0)
    layer.prepare([B * prompt_len, B])
    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        for _ in range(max(warmup, 1)):
            layer.reset()
            n0 = api.launch_count()
            layer.forward(xp, prompt_len)
            n1 = api.launch_count()
            layer.forward(xd, 1)
            # kernels of the SpMM library in one prefill pass and in one decode step (torch's and NCCL's not counted)
            layer.launches = (n1 - n0, api.launch_count() - n1)
    stream.synchronize()
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = layer.forward(xd, 1)
        except Exception:
            graph = None
    world = layer.world

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(layer.group)
            torch.cuda.synchronize()

    t_total = t_pre = 0.0
    for _ in range(steps):
        sync()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        with torch.cuda.stream(stream):
            layer.reset()
            e[0].record()
            layer.forward(xp, prompt_len)
            e[1].record()
            for _ in range(new_tokens):
                if graph is not None:
                    graph.replay()
                else:
                    layer.forward(xd, 1)
            e[2].record()
        torch.cuda.synchronize()
        pre, tot = e[0].elapsed_time(e[1]), e[0].elapsed_time(e[2])
        if world > 1:
            t = torch.tensor([pre, tot], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=layer.group)
            pre, tot = float(t[0]), float(t[1])
        t_total += tot * 1e-3
        t_pre += pre * 1e-3
    t_total /= steps
    t_pre /= steps
    return t_total, t_pre, (t_total - t_pre) / new_tokens, graph is not None
