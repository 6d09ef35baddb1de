#!/usr/bin/env python
"""Benchmark of the bitmap-v3 SpMM path.

A step is one pass over a set of layer-shaped SpMMs.  The default workload is the OPT-13B layer set (four weight
matrices at 60 % uniform-random sparsity, each multiplied at N = 8, 16 and 32: twelve SpMMs), the configuration
the headline metric is quoted on; `--workload opt66b_tp` is the OPT-66B set at N = 16 (four SpMMs) whose row shards
are checked bit for bit against the CPU encoder inside the run; `--workload opt66b_layer` runs one synthetic OPT-66B
decoder layer (batch 8, 64 prompt tokens, 128 generated tokens) and reports tokens/s.  Inputs are synthetic and
seeded.  With more than one GPU each weight matrix is split by rows across the ranks (tensor-parallel M-split) and
the output rows are gathered on every rank (the layer workload splits as FasterTransformer does: QKV and FC1 by rows,
out-proj and FC2 by columns with an all-reduce), so the total work is fixed ("strong" scaling).

The JSON line carries: value (device-resident, CUDA events, graph replay over rotating weight copies), e2e (host
buffers through spmspm_b200.pipeline.HostBatch), roofline (algorithmic bytes / time against the measured HBM copy
bandwidth; traffic from the committed profiler capture), parity (sampled rows against the fp32 host GEMM; a failure
exits 1), comparators (dense cuBLAS fp16 and the reference-style mma.sync kernel), cpu_baseline, encoder, clocks.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME | --case M,K,N[,s[,sk]]]

Prints one JSON line (rank 0).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    # QKV, out-proj, FC1, FC2
    "opt13b_layer_set_s60": {"shapes": [(15360, 5120), (5120, 5120), (20480, 5120), (5120, 20480)], "ns": [8, 16, 32],
                             "sparsity": 0.6},
    "opt66b_tp": {"shapes": [(27648, 9216), (9216, 9216), (36864, 9216), (9216, 36864)], "ns": [16], "sparsity": 0.6},
    # one synthetic OPT-66B decoder layer, tensor-parallel as FasterTransformer splits it (see spmspm_b200/layer.py);
    # handled by run_layer, the shapes here are only what the JSON line reports
    "opt66b_layer": {"shapes": [(27648, 9216), (9216, 9216), (36864, 9216), (9216, 36864)], "ns": [8, 512], "sparsity": 0.6},
}
WORKLOAD = "opt13b_layer_set_s60"
SHAPES = WORKLOADS[WORKLOAD]["shapes"]
NS = WORKLOADS[WORKLOAD]["ns"]
SPARSITY = WORKLOADS[WORKLOAD]["sparsity"]
SEED = 0x5EED0001
REL_TOL = 1e-2   # max |c - ref| / max |ref| against the fp32 host GEMM
# Split_K the reference's converter assigns by M (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:23);
# used for the reference-style comparator kernel
REF_SPLIT_K = {4096: 6, 12288: 2, 16384: 2, 5120: 6, 15360: 2, 20480: 3, 7680: 4, 10240: 2, 7168: 4, 21504: 3, 28672: 1}


def gen_weight(M, K, idx, device):
    """fp16 N(0, 0.02^2) weights with a seeded Bernoulli(keep = 1 - sparsity) mask; kept values are never zero."""
    g = torch.Generator(device=device).manual_seed(SEED + 16 * idx)
    A = (torch.randn((M, K), device=device, generator=g) * 0.02).half()
    A = torch.where(A == 0, torch.full_like(A, 6.1035e-05), A)
    keep = torch.rand((M, K), device=device, generator=g) >= SPARSITY
    return A * keep


def gen_act(N, K, idx, device):
    g = torch.Generator(device=device).manual_seed(SEED + 1000 + 16 * idx + N)
    return torch.randn((N, K), device=device, generator=g).half()


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        try:
            p = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                  "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
        except OSError:
            return
        try:
            while not self._stop.is_set():
                line = p.stdout.readline()
                if not line:
                    break
                self.rows.append([c.strip() for c in line.split(",")])
        finally:
            p.terminate()

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        time.sleep(0.15)
        self._stop.set()
        self._t.join(2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def traffic_ratio():
    """dram bytes / algorithmic bytes of the SpMM kernel in the committed profiler capture (profiles/)."""
    path = os.path.join(ROOT, "profiles", "spmm_dram_traffic.json")
    try:
        d = json.load(open(path))
        return float(d["dram_bytes"]) / float(d["algorithmic_bytes"]), d.get("capture", "profiles/spmm_dram_traffic.json")
    except Exception:
        return None, None


def flops_per_step():
    return sum(2.0 * M * K * N for (M, K) in SHAPES for N in NS)


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------- reference arm

def run_reference(args, rank):
    """The path on the host cores: decode of the bitmap format + fp32 GEMM (OpenMP, every core of the box), the CPU
    restatement of the reference's algorithm (the reference ships no CPU SpMM; its own CPU code on this path is the
    encoder).  A step is the whole set when that fits the time budget, else the same set on a slab of rows of
    every matrix (the rate does not depend on the number of rows)."""
    if rank != 0:
        return
    import oracle
    cores = oracle.set_num_threads(host_threads())   # a launcher may have exported OMP_NUM_THREADS=1
    budget_s = 120.0
    total_steps = max(args.warmup, 1) + args.steps
    # calibrate on 512 rows of the first matrix
    M0, K0 = SHAPES[0]
    A0 = gen_weight(min(M0, 512), K0, 0, "cpu").numpy()
    e0 = oracle.encode(A0)
    B0 = gen_act(NS[0], K0, 0, "cpu").numpy()
    oracle.spmm_f32(e0, B0)
    t0 = time.perf_counter()
    oracle.spmm_f32(e0, B0)
    rate = 2.0 * A0.shape[0] * K0 * NS[0] / max(time.perf_counter() - t0, 1e-6)
    frac = min(1.0, budget_s * rate / (flops_per_step() * total_steps))
    mats, flops = [], 0.0
    for i, (M, K) in enumerate(SHAPES):
        rows = M if frac >= 1.0 else max(64, int(M * frac) // 64 * 64)
        A = gen_weight(rows, K, i, "cpu").numpy()
        mats.append((oracle.encode(A), [gen_act(N, K, i, "cpu").numpy() for N in NS]))
        flops += sum(2.0 * rows * K * N for N in NS)

    def step():
        for enc, Bs in mats:
            for B in Bs:
                oracle.spmm_f32(enc, B)

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e12
    sample = ("the whole set per step" if frac >= 1.0 else
              f"the first {frac * 100:.1f} % of the rows of every matrix of the set per step "
              f"({flops / 1e9:.1f} of {flops_per_step() / 1e9:.1f} GFLOP)")
    line = {"impl": "reference", "metric": "spmm_dense_equiv_tflops", "value": val, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": {"workload": WORKLOAD, "sparsity": SPARSITY, "N": NS, "shapes": SHAPES},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="opt13b_layer_set_s60", choices=sorted(WORKLOADS),
                    help="opt13b_layer_set_s60: the headline set; opt66b_tp: the OPT-66B shapes at N = 16 with every "
                         "row shard's encoding checked against the CPU encoder inside the run; opt66b_layer: one "
                         "synthetic OPT-66B decoder layer, batch 8, 64 prompt tokens, 128 generated tokens, tokens/s")
    ap.add_argument("--case", default=None,
                    help="M,K,N[,sparsity[,split_k]]: time one SpMM shape instead of a set "
                         "(used for per-shape tables and for small profiler captures)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="several GPUs: how the output rows are gathered. peer = the SpMM kernel stores its rows into "
                         "every GPU's buffer over NVLink and the next SpMM waits for the flags itself "
                         "(spb_spmm_bitmap_v3_allgather); nccl = local SpMM, then an NCCL all-gather; auto = both are "
                         "timed for a few steps and the faster one is used")
    ap.add_argument("--schedule", default="auto", choices=["auto", "static", "balanced"],
                    help="work schedule of the SpMM kernel (spb_set_schedule); auto lets the library choose per call")
    ap.add_argument("--no-extras", action="store_true", help="skip comparators, CPU baseline and encoder timing")
    ap.add_argument("--spmspm", action="store_true",
                    help="with --case on one GPU: the activations are pruned (50 %%) and passed bitmap-compressed in the "
                         "second-operand layout (spb_spmspm_bitmap_v3, the fork's 19-argument form); N a multiple of 64")
    args = ap.parse_args()
    global SHAPES, NS, SPARSITY, WORKLOAD
    WORKLOAD = args.workload
    SHAPES, NS, SPARSITY = (WORKLOADS[WORKLOAD][k] for k in ("shapes", "ns", "sparsity"))
    forced_split = None
    if args.case:
        f = args.case.split(",")
        SHAPES, NS = [(int(f[0]), int(f[1]))], [int(f[2])]
        if len(f) > 3:
            SPARSITY = float(f[3])
        if len(f) > 4:
            forced_split = int(f[4])
        WORKLOAD = "case_" + args.case.replace(",", "_")
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    import spmspm_b200 as sp
    sp.set_schedule({"auto": sp.SCHEDULE_AUTO, "static": sp.SCHEDULE_STATIC, "balanced": sp.SCHEDULE_BALANCED}[args.schedule])
    from spmspm_b200 import dist as spd

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    l2_bytes = int(torch.cuda.get_device_properties(dev).L2_cache_size)
    if args.workload == "opt66b_layer" and not args.case:
        run_layer(args, sp, dist, dev, rank, world, local_rank)
        return

    # ---- weights: generate, encode on the GPU, keep only this rank's row shard
    mats = []
    shard_check = None
    for i, (M, K) in enumerate(SHAPES):
        A = gen_weight(M, K, i, dev)
        lo, hi = spd.row_shard_bounds(M, world, rank)
        shard = A[lo:hi].contiguous()
        del A
        W = sp.encode_device(shard)
        if args.workload == "opt66b_tp" and not args.case:
            # the shard's encoding against the CPU restatement of the reference encoder on the same sub-matrix
            import oracle
            e = oracle.encode(shard.cpu().numpy())
            same = (np.array_equal(W.vals.cpu().numpy().view(np.uint16), e.vals)
                    and np.array_equal(W.gtile.cpu().numpy(), e.gtile) and np.array_equal(W.mtile.cpu().numpy(), e.mtile)
                    and np.array_equal(W.bitmap.cpu().numpy().view(np.uint64), e.bitmap)
                    and np.array_equal(W.tile_nnz.cpu().numpy(), e.tile_nnz) and int(W.max_nnz.item()) == e.max_nnz)
            shard_check = (shard_check if shard_check is not None else True) and bool(same)
        del shard
        mats.append(W)
    torch.cuda.empty_cache()
    if shard_check is not None and world > 1:
        t = torch.tensor([1 if shard_check else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        shard_check = bool(t.item())
    weight_bytes = sum(2 * W.val_count + 8 * (W.M * W.K // 64) + 20 * W.G for W in mats)
    # Rotation: enough copies of this rank's weights that the bytes streamed between two uses of the same copy exceed
    # twice the L2 capacity at every world size (one copy is enough when the set itself is that large).
    copies = 1 if args.case else max(1, math.ceil(2.0 * l2_bytes / max(weight_bytes, 1)))
    copies = min(copies, 16)

    def clone(W):
        return sp.BitmapMatrix(W.M, W.K, W.vals.clone(), W.gtile.clone(), W.mtile.clone(), W.bitmap.clone(),
                               W.max_nnz.clone(), None, W.val_count)

    mat_sets = [mats] + [[clone(W) for W in mats] for _ in range(copies - 1)]
    rotating = copies * weight_bytes > 2 * l2_bytes
    acts = {(i, N): gen_act(N, K, i, dev) for i, (M, K) in enumerate(SHAPES) for N in NS}
    acts_c = None
    if args.spmspm:
        if world > 1 or not args.case or any(N % 64 for N in NS):
            print("[bench] --spmspm needs --case on one GPU with N a multiple of 64", file=sys.stderr)
            sys.exit(2)
        g = torch.Generator(device=dev).manual_seed(SEED + 77)
        for k in acts:   # prune the activations (seeded Bernoulli, 50 %) and encode them in the second-operand layout
            acts[k] = acts[k] * (torch.rand(acts[k].shape, device=dev, generator=g) >= 0.5)
        acts_c = {k: sp.to_device(sp.init_sparse_matrix_a_bitmap_v6_b(v.cpu().numpy()), dev) for k, v in acts.items()}
    splits = {(i, N): forced_split or sp.suggest_split_k(mats[i].M, N, mats[i].K)
              for i in range(len(SHAPES)) for N in NS}
    outs = {(i, N): torch.empty((N, mats[i].M), dtype=torch.float16, device=dev) for (i, N) in acts}
    ws = torch.empty(max(splits[k] * k[1] * mats[k[0]].M for k in acts), dtype=torch.float16, device=dev)
    gathered = {(i, N): torch.empty((world, N, mats[i].M), dtype=torch.float16, device=dev) for (i, N) in acts} \
        if world > 1 else None
    order = [(i, N) for N in NS for i in range(len(SHAPES))]
    launches_per_step = None   # counted by the library while a step is issued (spb_launch_count)
    alg_bytes_step = sum(mats[i].algorithmic_bytes(N) for (i, N) in order)

    # Several GPUs, peer exchange: one symmetric output buffer per SpMM of the step; every SpMM waits (inside its
    # kernel) for the exchange of the SpMM before it, as a chain of layers would, the first one of a step for the
    # last one of the step before.
    peer = None
    if world > 1 and args.exchange in ("auto", "peer"):
        try:
            # one buffer each: in this chain a buffer is rewritten a whole step after every rank consumed it,
            # and a captured step then names the same buffers on every replay
            peer = {k: spd.PeerGather(k[1], SHAPES[k[0]][0], dev, slots=1) for k in order}
        except Exception as exc:
            print(f"[bench] symmetric memory unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
    row_lo = {i: spd.row_shard_bounds(SHAPES[i][0], world, rank)[0] for i in range(len(SHAPES))}
    chain = {"prev": None}

    def step_peer(c=0):
        for k in order:
            i, N = k
            peer[k].spmm(mat_sets[c][i], acts[k], row_lo[i], after=chain["prev"], split_k=splits[k], workspace=ws)
            chain["prev"] = peer[k]

    def step_local(c=0):
        for k in order:
            i, N = k
            if acts_c is not None:
                sp.spmspm(mat_sets[c][i], acts_c[k], split_k=splits[k], out=outs[k], workspace=ws)
                continue
            sp.spmm(mat_sets[c][i], acts[k], split_k=splits[k], out=outs[k], workspace=ws)
            if world > 1:
                dist.all_gather_into_tensor(gathered[k], outs[k])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        """Event time of `steps` calls of fn(i), max over the ranks, in ms."""
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    work = torch.cuda.Stream()
    exchange = "none"
    step = step_local
    exchange_probe = None
    if world > 1:
        exchange = "nccl"
        if peer is not None:
            exchange = "peer"
            if args.exchange == "auto":
                # both ways of gathering are timed for a few steps; the faster one (max over ranks) is used
                probe = {}
                for name, fn in (("nccl", step_local), ("peer", step_peer)):
                    with torch.cuda.stream(work):
                        for _ in range(3):
                            fn(0)
                        probe[name] = timed(lambda i, fn=fn: fn(i % copies), 6) / 6
                    work.synchronize()
                exchange = min(probe, key=probe.get)
                exchange_probe = probe
        step = step_peer if exchange == "peer" else step_local

    # The step (its SpMM calls and, on several GPUs, their exchanges) is captured once per weight copy into a CUDA
    # graph and replayed in rotation, so that the host's call overhead is not part of the device-resident number; the
    # eager figure is reported beside it.
    with torch.cuda.stream(work):
        for w_ in range(args.warmup):
            n0 = sp.launch_count()
            step(w_ % copies)
            launches_per_step = sp.launch_count() - n0   # the library's own kernels only (no NCCL, no torch)
    work.synchronize()
    with torch.cuda.stream(work):
        eager_ms = timed(lambda i: step(i % copies), args.steps) / args.steps
    timed_as = "cuda_graph_replay"
    try:
        graphs = []
        for c in range(copies):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=work):
                step(c)
            graphs.append(g)
        for w_ in range(args.warmup):
            graphs[w_ % copies].replay()

        def run(i):
            graphs[i % copies].replay()
    except Exception as exc:  # a collective that cannot be captured on this stack: time the eager loop
        print(f"[bench] graph capture failed ({type(exc).__name__}: {exc}); timing the eager loop", file=sys.stderr)
        timed_as = "eager"

        def run(i):
            step(i % copies)
    with ClockSampler(local_rank) as clocks:
        ms_total = timed(run, args.steps)
    ms_step = ms_total / args.steps
    value = flops_per_step() / (ms_step * 1e-3) / 1e12

    # ---- parity of what the timed loop produced: every SpMM's gathered output against the fp32 host GEMM on
    # sampled rows of the full (unsharded) weight, at every world size
    def full_output(k):
        if world == 1:
            return outs[k]
        if exchange == "peer":
            return peer[k].bufs[0]
        return gathered[k].permute(1, 0, 2).reshape(k[1], -1)

    torch.cuda.synchronize()
    parity = None
    if rank == 0:
        import oracle
        oracle.set_num_threads(host_threads())
        worst, rows_checked = 0.0, 0
        for i, (M, K) in enumerate(SHAPES):
            rows = np.unique(np.linspace(0, M - 1, num=min(M, 768)).astype(np.int64))
            A_rows = gen_weight(M, K, i, dev)[torch.from_numpy(rows).to(dev)].cpu().numpy()
            for N in NS:
                ref = oracle.gemm_f32(A_rows, acts[(i, N)].cpu().numpy())            # [N, rows]
                got = full_output((i, N))[:, torch.from_numpy(rows).to(dev)].float().cpu().numpy()
                worst = max(worst, float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-12)))
            rows_checked += len(rows)
        parity = {"max_rel_err": worst, "ok": bool(worst <= REL_TOL), "tolerance": REL_TOL,
                  "rows_checked_per_step": rows_checked, "against": "fp32 host GEMM (oracle) on sampled rows of every SpMM"}

    # ---- end to end through the C ABI with host buffers: activations in, outputs back, every SpMM
    h_acts = {k: v.cpu().pin_memory() for k, v in acts.items()}
    # The package's host-buffer front end (spmspm_b200.pipeline.HostBatch): per step one packed copy of the step's
    # activations from pinned host memory, the step's SpMMs (several GPUs: row shards + exchange, every rank ends up
    # with all rows), one packed copy of the results back to pinned host memory; two staging sets, so the copies of one
    # step overlap the SpMMs of the next.  Every step's inputs are written into the pinned buffer and every step's
    # results are waited for on the host.
    from spmspm_b200.pipeline import HostBatch
    streams = tuple(torch.cuda.Stream(dev) for _ in range(3))
    full_cols = [SHAPES[i][0] for (i, N) in order]
    e2e_copies = copies if world == 1 else 1     # several GPUs: one weight copy (buffers of the exchange per staging set)
    bodies = [None] * e2e_copies
    if world > 1:
        e2e_peer = None
        if exchange == "peer":
            # buffers of their own per staging set: a set is resubmitted only after every rank has been seen to finish
            # the set between, whose SpMMs run after this rank's copies out of the first
            e2e_peer = [{k: spd.PeerGather(k[1], SHAPES[k[0]][0], dev, slots=1) for k in order} for _ in range(2)]
        e2e_gathered = {k: torch.empty((world, k[1], mats[k[0]].M), dtype=torch.float16, device=dev) for k in order}

        def body(s, ins, outs_v):
            if e2e_peer is not None:
                for k, x in zip(order, ins):
                    e2e_peer[s][k].spmm(mat_sets[0][k[0]], x, row_lo[k[0]], split_k=splits[k], workspace=ws)
                for k, y in zip(order, outs_v):
                    y.copy_(e2e_peer[s][k].wait())
            else:
                for k, x, y in zip(order, ins, outs_v):
                    sp.spmm(mat_sets[0][k[0]], x, split_k=splits[k], out=outs[k], workspace=ws)
                    dist.all_gather_into_tensor(e2e_gathered[k], outs[k])
                    y.copy_(e2e_gathered[k].permute(1, 0, 2).reshape(k[1], -1))
        bodies = [body]
    batches = [HostBatch([(mat_sets[c][i], N) for (i, N) in order], dev, split_k=[splits[k] for k in order],
                         streams=streams, body=bodies[c], out_cols=full_cols, ready=sync_all if world > 1 else None)
               for c in range(e2e_copies)]
    for hb in batches:
        for s_ in range(2):
            for view, k in zip(hb.inputs(s_), order):
                view.copy_(h_acts[k])
    state = {"prev": None}

    def e2e_step(it):
        hb, s_ = batches[it % e2e_copies], (it // e2e_copies) % 2
        hb.submit(s_)
        if state["prev"] is not None:
            state["prev"][0].wait(state["prev"][1])      # the host reads the previous step's results
        state["prev"] = (hb, s_)

    def e2e_timed(steps):
        sync_all()
        t0 = time.perf_counter()
        for i_ in range(steps):
            e2e_step(i_)
        state["prev"][0].wait(state["prev"][1])
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    e2e_timed(3)
    e2e_ms = e2e_timed(args.steps) / args.steps
    got = batches[0].outputs(0)[0].float()
    want = full_output(order[0]).float().cpu()
    if not torch.allclose(got, want, atol=1e-2 * float(want.abs().max())):
        print("[bench] host-buffer pipeline result differs from the resident result", file=sys.stderr)
        sys.exit(1)
    for hb in batches:
        hb.close()
    e2e_how = ("HostBatch: packed copy in, graph of the step's SpMMs" + (" and their exchange" if world > 1 else "") +
               ", packed copy out, double-buffered; wall clock over the steps (max over ranks), host waits for every "
               "step's results")
    h2d = sum(N * SHAPES[i][1] * 2 for (i, N) in order)
    d2h = sum(N * SHAPES[i][0] * 2 for (i, N) in order)

    status = sp.device_status()
    if rank != 0:
        if world > 1:
            finish_ranks(dist)
        return

    peak, peak_kind = measured_peak_gbs()
    achieved = alg_bytes_step / (ms_step * 1e-3) / 1e9
    if rotating:
        l2_note = (f"rotating: {copies} cop{'y' if copies == 1 else 'ies'} of {weight_bytes / 1e6:.0f} MB of compressed weights "
                   f"per rank are streamed between two uses of the same bytes (L2: {l2_bytes / 1e6:.0f} MB)")
    else:
        l2_note = (f"L2-warm: {copies * weight_bytes / 1e6:.0f} MB of compressed weights per rank against an L2 of "
                   f"{l2_bytes / 1e6:.0f} MB")
    ratio, capture = traffic_ratio()
    line = {
        "metric": "spmm_dense_equiv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "shapes": SHAPES, "N": NS, "sparsity": SPARSITY, "spmm_per_step": len(order),
                   "split_k": {f"{SHAPES[i][0]}x{SHAPES[i][1]}xN{N}": splits[(i, N)] for (i, N) in order},
                   "schedule": args.schedule,
                   "parallelism": f"tp{world}_m_split_allgather_{exchange}" if world > 1 else "single_gpu",
                   "l2": l2_note, "weight_copies": copies, "algorithmic_bytes_per_step": alg_bytes_step,
                   "second_operand": "bitmap-compressed, 50 % pruned (spb_spmspm_bitmap_v3)" if acts_c is not None else "dense",
                   "launches_per_step": launches_per_step},
        "hbm_gbs": achieved * world if world > 1 else achieved,
        "e2e": {"value": flops_per_step() / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "how": e2e_how},
        "timed_as": timed_as,
        "eager_ms_per_step": eager_ms,
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "device_status": status,
        "parity": parity,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": ratio * alg_bytes_step / len(order) if ratio else None,
                     "note": "algorithmic bytes of this rank's SpMMs / event time of the step (SpMM kernel plus "
                             "its split-K reduction launch); traffic = average algorithmic bytes of a launch x the "
                             "dram-bytes / algorithmic-bytes ratio of the capture named in traffic_from",
                     "traffic_from": capture},
    }
    if shard_check is not None:
        line["shard_encoding_bit_exact"] = shard_check
    if exchange_probe:
        line["exchange_probe_ms_per_step"] = exchange_probe
    if world == 1 and not args.no_extras:
        line["comparators"] = {"cublas_dense_fp16": cublas_dense(dev, acts, order, args, ours=outs)}
        rs = ref_style(dev, sp, mats, acts, order, args)
        if rs is not None:
            line["comparators"]["reference_style_mma_sync"] = rs
        line["l2_hot"] = l2_hot(dev, sp, mats, acts, outs, ws, splits, order, ms_step)
    if world == 1 and not args.case and not args.no_extras:
        line["cpu_baseline"] = cpu_baseline()
        line["encoder"] = encoder_timing(dev)
    print(json.dumps(line), flush=True)
    failed = (parity is not None and not parity["ok"]) or shard_check is False or status != 0
    if world > 1:
        finish_ranks(dist, 1 if failed else 0)
    if failed:
        sys.exit(1)


def run_layer(args, sp, dist, dev, rank, world, local_rank):
    """One synthetic OPT-66B decoder layer (hidden 9216, 72 heads, FFN 36864, 60 % pruned), batch 8: a prompt of 64
    tokens per sequence, then 128 generated tokens; QKV and FC1 split by rows, out-proj and FC2 by columns with an
    all-reduce (one-shot over peer stores, or NCCL).  A step is one whole generation.  tokens/s as the reference's
    plots compute it (end2end_inference/draw_plot.py:120-123): batch * generated tokens / latency, per layer."""
    from spmspm_b200.layer import SparseOptDecoderLayer, generate_timed
    hidden, heads, ffn, batch, prompt, new = 9216, 72, 36864, 8, 64, 128
    results = {}
    kinds = ["none"] if world == 1 else (["peer", "nccl"] if args.exchange == "auto" else [args.exchange])
    for kind in kinds:
        try:
            layer = SparseOptDecoderLayer(hidden, heads, ffn, SPARSITY, dev, batch=batch, max_len=prompt + new, reduce=kind)
        except Exception as exc:
            if rank == 0:
                print(f"[bench] layer with reduce={kind} unavailable ({type(exc).__name__}: {exc})", file=sys.stderr)
            continue
        with ClockSampler(local_rank) as clocks:
            total, pre, per_step, graphed = generate_timed(layer, prompt, new, steps=max(args.steps // 4, 2), warmup=2)
        results[kind] = {"s_per_generation": total, "prefill_ms": pre * 1e3, "decode_step_us": per_step * 1e6,
                         "decode_graph": graphed, "tokens_per_s": batch * new / total, "clocks": clocks.summary(),
                         "library_launches": {"prefill": layer.launches[0], "decode_step": layer.launches[1]},
                         "device_status": sp.device_status()}
        del layer
        torch.cuda.empty_cache()
    if rank == 0:
        best = max(results, key=lambda k: results[k]["tokens_per_s"])
        r = results[best]
        line = {"metric": "decoder_layer_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s (one layer)",
                "n_gpus": world, "steps": max(args.steps // 4, 2), "warmup": 2, "ms_per_step": r["s_per_generation"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": "opt66b_layer", "hidden": hidden, "heads": heads, "ffn": ffn, "sparsity": SPARSITY,
                           "batch": batch, "prompt_tokens": prompt, "generated_tokens": new,
                           "parallelism": f"tp{world}_ft_split_allreduce_{best}" if world > 1 else "single_gpu"},
                "tokens_per_s_per_gpu": r["tokens_per_s"] / world,
                "tokens_per_s_64_layers": r["tokens_per_s"] / 64.0,
                "gpu_launches": (r["library_launches"]["prefill"] + new * r["library_launches"]["decode_step"]) * max(args.steps // 4, 2),
                "by_reduce": results, "clocks": r["clocks"], "device_status": r["device_status"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        finish_ranks(dist, 0)


def finish_ranks(dist, code=0):
    """All ranks meet, then leave without tearing the communicator down: destroying a process group while a
    captured graph still holds its collectives did not return on this stack."""
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


def graph_time(fn, args):
    """fn() captured into a CUDA graph on a side stream, replayed: ms per replay."""
    work = torch.cuda.Stream()
    with torch.cuda.stream(work):
        for _ in range(args.warmup):
            fn()
    work.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=work):
        fn()
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / args.steps


def cublas_dense(dev, acts, order, args, ours=None):
    """Dense fp16 GEMM (cuBLAS through torch.mm, fp32 accumulate) on the un-compressed pruned weights, same shapes,
    same rotation over the matrices; the comparator the reference's drivers use (csrc/spmm_test.cu:101-102).  With
    `ours` (this library's outputs of the same SpMMs) also the figure those drivers print: TotalError, the sum over
    all outputs of |cuBLAS - other| (csrc/spmm_test_utils.h:110-115), here summed over the SpMMs of the step."""
    dense = [gen_weight(M, K, i, dev) for i, (M, K) in enumerate(SHAPES)]
    outs = {k: torch.empty((k[1], SHAPES[k[0]][0]), dtype=torch.float16, device=dev) for k in order}

    def step():
        for k in order:
            torch.mm(acts[k], dense[k[0]].t(), out=outs[k])

    ms = graph_time(step, args)
    dense_bytes = sum(2 * SHAPES[i][0] * SHAPES[i][1] for (i, N) in order)
    res = {"value": flops_per_step() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
           "dense_weight_gbs": dense_bytes / (ms * 1e-3) / 1e9}
    if ours is not None:
        step()
        torch.cuda.synchronize()
        total = sum(float((outs[k].float() - ours[k].float()).abs().sum()) for k in order)
        count = sum(outs[k].numel() for k in order)
        res["total_error_vs_this_library"] = total
        res["mean_abs_error_vs_this_library"] = total / count
    return res


def ref_style(dev, sp, mats, acts, order, args):
    """The reference's mma.sync / cp.async kernel (oracle/_ref/libref_style_spmm.so, put together from the reference's
    own device functions and compiled for sm_100a) on the same encoded weights, same rotation, timed the same way.
    Split_K from the reference's per-M table where it has an entry, else 1."""
    import oracle
    if not oracle.have_ref_style():
        return None
    ok_ns = [N for N in NS if N in (8, 16, 32, 64) or N % 128 == 0]
    if len(ok_ns) != len(NS):
        return {"unavailable": "the reference kernel only takes N in {8, 16, 32, 64, k*128}"}
    bufs = {}
    for (i, N) in order:
        W = mats[i]
        sk = REF_SPLIT_K.get(W.M, 1)
        if sk > 1 and (W.M * N) % 256:
            sk = 1
        B = acts[(i, N)]
        if N == 8:   # that kernel copies a 16-row activation tile
            Bp = torch.zeros((16, B.shape[1]), dtype=B.dtype, device=dev)
            Bp[:8] = B
            B = Bp
        bufs[(i, N)] = (B, torch.empty((N, W.M), dtype=torch.float16, device=dev),
                        torch.empty(max(sk, 1) * N * W.M, dtype=torch.float16, device=dev), sk, int(W.max_nnz.item()))

    def step():
        s = torch.cuda.current_stream().cuda_stream
        for (i, N) in order:
            W = mats[i]
            B, C, w, sk, mx = bufs[(i, N)]
            oracle.ref_style_spmm(s, W.vals.data_ptr(), W.gtile.data_ptr(), W.mtile.data_ptr(), W.bitmap.data_ptr(),
                                  B.data_ptr(), C.data_ptr(), W.M, N, W.K, w.data_ptr(), sk, mx)

    try:
        ms = graph_time(step, args)
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"}
    alg = sum(mats[i].algorithmic_bytes(N) for (i, N) in order)
    return {"value": flops_per_step() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "hbm_gbs": alg / (ms * 1e-3) / 1e9,
            "split_k": {f"{SHAPES[i][0]}x{SHAPES[i][1]}xN{N}": bufs[(i, N)][3] for (i, N) in order}}


def l2_hot(dev, sp, mats, acts, outs, ws, splits, order, cold_ms):
    """The same SpMMs with each one launched five times in a row: the four repeats find what fits of their weight
    in L2.  Reported as the time of a step made of such repeats, beside the rotating (cold) figure."""
    class A:
        warmup, steps = 3, 10

    def once(rep):
        def fn():
            for k in order:
                for _ in range(rep):
                    sp.spmm(mats[k[0]], acts[k], split_k=splits[k], out=outs[k], workspace=ws)
        return fn

    t1, t5 = graph_time(once(1), A), graph_time(once(5), A)
    hot = (t5 - t1) / 4.0
    return {"ms_per_step": hot, "value": flops_per_step() / (hot * 1e-3) / 1e12, "unit": "TFLOP/s",
            "cold_ms_per_step": cold_ms}


def cpu_baseline():
    """fp32 host GEMM over the decoded weight (the CPU restatement of the path), all host threads, bounded sample."""
    import oracle
    cores = oracle.set_num_threads(host_threads())
    M, K = SHAPES[1]
    A = gen_weight(M, K, 1, "cpu").numpy()
    enc = oracle.encode(A)
    Bs = [gen_act(N, K, 1, "cpu").numpy() for N in NS]
    oracle.spmm_f32(enc, Bs[0])
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0 and reps < 50:
        for B in Bs:
            oracle.spmm_f32(enc, B)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    flops = sum(2.0 * M * K * N for N in NS)
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"out-proj matrix {M}x{K} at N={NS}, {reps} passes in {dt * reps:.1f} s"}


def encoder_timing(dev):
    """GPU encoder vs the reference's own CPU encoder (compiled, unmodified, 1 thread) on the out-proj matrix."""
    import oracle
    import spmspm_b200 as sp
    M, K = SHAPES[1]
    A = gen_weight(M, K, 1, dev)
    sp.encode_device(A)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(5):
        sp.encode_device(A)
    torch.cuda.synchronize()
    gpu_ms = (time.perf_counter() - t0) / 5 * 1e3
    Ah = A.cpu().numpy()
    out = {"matrix": f"{M}x{K}", "gpu_ms": gpu_ms}
    t0 = time.perf_counter()
    if oracle.have_ref():
        oracle.ref_encode(Ah)
        out["cpu_kind"] = "reference"
    else:
        oracle.encode(Ah)
        out["cpu_kind"] = "port"
    out["cpu_ms"] = (time.perf_counter() - t0) * 1e3
    out["cpu_cores"] = 1
    return out


if __name__ == "__main__":
    main()
