#!/usr/bin/env python
"""Benchmark of the bitmap-v3 SpMM path.

A step is one pass over the OPT-13B layer-shaped SpMM set (four weight matrices at 60 %
uniform-random sparsity, each multiplied at N = 8, 16 and 32: twelve SpMMs), the configuration
the headline metric is quoted on.  Inputs are synthetic and seeded.  With more than one GPU each
weight matrix is split by rows across the ranks (tensor-parallel M-split) and the output rows
are all-gathered over NCCL, so the total work is fixed ("strong" scaling).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line (rank 0).
"""
import argparse
import json
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

WORKLOAD = "opt13b_layer_set_s60"
SHAPES = [(15360, 5120), (5120, 5120), (20480, 5120), (5120, 20480)]  # QKV, out-proj, FC1, FC2
NS = [8, 16, 32]
SPARSITY = 0.6
SEED = 0x5EED0001


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


def flops_per_step():
    return sum(2.0 * M * K * N for (M, K) in SHAPES for N in NS)


# ------------------------------------------------------------------------------------- reference arm

def run_reference(args, rank):
    """The path on the host cores: decode of the bitmap format + fp32 GEMM (OpenMP), the CPU restatement of the
    reference's algorithm (the reference ships no CPU SpMM; its own CPU code on this path is the encoder)."""
    if rank != 0:
        return
    import oracle
    M, K = SHAPES[1]
    A = gen_weight(M, K, 1, "cpu").numpy()
    enc = oracle.encode(A)
    Bs = [gen_act(N, K, 1, "cpu").numpy() for N in NS]
    flops = sum(2.0 * M * K * N for N in NS)

    def step():
        for B in Bs:
            oracle.spmm_f32(enc, B)

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e12
    sample = f"out-proj matrix {M}x{K} at N={NS} per step (1 of the 4 matrices of the set)"
    line = {"impl": "reference", "metric": "spmm_dense_equiv_tflops", "value": val, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": {"workload": WORKLOAD, "sparsity": SPARSITY, "N": NS, "shapes": SHAPES},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None,
                    help="M,K,N[,sparsity[,split_k]]: time one SpMM shape instead of the OPT-13B set "
                         "(used for per-shape tables and for small profiler captures)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="several GPUs: how the output rows are gathered. peer = the SpMM kernel stores its rows into "
                         "every GPU's buffer over NVLink and the next SpMM waits for the flags itself "
                         "(spb_spmm_bitmap_v3_allgather); nccl = local SpMM, then an NCCL all-gather; auto = peer on "
                         "2 GPUs, where it was measured faster, nccl on more (the fused exchange of this build "
                         "has not been measured there)")
    ap.add_argument("--schedule", default="auto", choices=["auto", "static", "balanced"],
                    help="work schedule of the SpMM kernel (spb_set_schedule); auto lets the library choose per call")
    args = ap.parse_args()
    global SHAPES, NS, SPARSITY, WORKLOAD
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

    # ---- weights: generate, encode on the GPU, keep only this rank's row shard
    mats = []
    for i, (M, K) in enumerate(SHAPES):
        A = gen_weight(M, K, i, dev)
        lo, hi = spd.row_shard_bounds(M, world, rank)
        W = sp.encode_device(A[lo:hi].contiguous())
        del A
        mats.append(W)
    torch.cuda.empty_cache()
    acts = {(i, N): gen_act(N, K, i, dev) for i, (M, K) in enumerate(SHAPES) for N in NS}
    splits = {(i, N): forced_split or sp.suggest_split_k(mats[i].M, N, mats[i].K)
              for i in range(len(SHAPES)) for N in NS}
    outs = {(i, N): torch.empty((N, mats[i].M), dtype=torch.float16, device=dev) for (i, N) in acts}
    ws = torch.empty(max(splits[k] * k[1] * mats[k[0]].M for k in acts), dtype=torch.float16, device=dev)
    gathered = {(i, N): torch.empty((world, N, mats[i].M), dtype=torch.float16, device=dev) for (i, N) in acts} \
        if world > 1 else None
    order = [(i, N) for N in NS for i in range(len(SHAPES))]
    launches_per_step = sum(1 + (1 if splits[k] > 1 else 0) for k in order)
    alg_bytes_step = sum(mats[i].algorithmic_bytes(N) for (i, N) in order)
    weight_bytes = sum(2 * W.val_count + 8 * (W.M * W.K // 64) + 20 * W.G for W in mats)

    # Several GPUs, peer exchange: one pair of symmetric output buffers per SpMM of the step; every SpMM waits
    # (inside its kernel) for the exchange of the SpMM before it, as a chain of layers would, the first one of a
    # step for the last one of the step before.
    peer = None
    exchange = "none"
    if world > 1:
        exchange = args.exchange
        if exchange == "auto":
            exchange = "peer" if world == 2 else "nccl"
        if exchange == "peer":
            try:
                # one buffer each: in this chain a buffer is rewritten a whole step after every rank consumed it,
                # and a captured step then names the same buffers on every replay
                peer = {k: spd.PeerGather(k[1], SHAPES[k[0]][0], dev, slots=1) for k in order}
            except Exception as exc:
                print(f"[bench] symmetric memory unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
                exchange = "nccl"
    row_lo = {i: spd.row_shard_bounds(SHAPES[i][0], world, rank)[0] for i in range(len(SHAPES))}
    chain = {"prev": None}

    def step():
        for k in order:
            i, N = k
            if peer is not None:
                peer[k].spmm(mats[i], acts[k], row_lo[i], after=chain["prev"], split_k=splits[k], workspace=ws)
                chain["prev"] = peer[k]
                continue
            sp.spmm(mats[i], acts[k], split_k=splits[k], out=outs[k], workspace=ws)
            if world > 1:
                dist.all_gather_into_tensor(gathered[k], outs[k])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # The step (its 12 SpMM calls and, on several GPUs, their all-gathers) is captured once into a CUDA graph and
    # replayed, so that the host's call overhead is not part of the device-resident number; the eager figure
    # is reported beside it.
    work = torch.cuda.Stream()
    with torch.cuda.stream(work):
        for _ in range(args.warmup):
            step()
    work.synchronize()
    with torch.cuda.stream(work):
        eager_ms = timed(step, args.steps) / args.steps
    timed_as = "cuda_graph_replay"
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=work):
            step()
        for _ in range(args.warmup):
            graph.replay()
        run = graph.replay
    except Exception as exc:  # a collective that cannot be captured on this stack: time the eager loop
        print(f"[bench] graph capture failed ({type(exc).__name__}: {exc}); timing the eager loop", file=sys.stderr)
        timed_as = "eager"
        run = step
    with ClockSampler(local_rank) as clocks:
        ms_total = timed(run, args.steps)
    ms_step = ms_total / args.steps
    value = flops_per_step() / (ms_step * 1e-3) / 1e12

    # ---- end to end through the C ABI with host buffers: activations in, outputs back, every SpMM
    h_acts = {k: v.cpu().pin_memory() for k, v in acts.items()}
    h_outs = {k: torch.empty((k[1], SHAPES[k[0]][0]), dtype=torch.float16).pin_memory() for k in acts}
    d_full = {k: torch.empty((k[1], SHAPES[k[0]][0]), dtype=torch.float16, device=dev) for k in acts}

    def e2e_step():
        for k in order:
            i, N = k
            acts[k].copy_(h_acts[k], non_blocking=True)
            sp.spmm(mats[i], acts[k], split_k=splits[k], out=outs[k], workspace=ws)
            if world > 1:
                dist.all_gather_into_tensor(gathered[k], outs[k])
                d_full[k].copy_(gathered[k].permute(1, 0, 2).reshape(N, -1))
                h_outs[k].copy_(d_full[k], non_blocking=True)
            else:
                h_outs[k].copy_(outs[k], non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps) / args.steps
    h2d = sum(N * SHAPES[i][1] * 2 for (i, N) in order)
    d2h = sum(N * SHAPES[i][0] * 2 for (i, N) in order)

    status = sp.device_status()
    if rank != 0:
        if world > 1:
            finish_ranks(dist)
        return

    peak, peak_kind = measured_peak_gbs()
    achieved = alg_bytes_step / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "spmm_dense_equiv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "shapes": SHAPES, "N": NS, "sparsity": SPARSITY, "spmm_per_step": len(order),
                   "split_k": {f"{SHAPES[i][0]}x{SHAPES[i][1]}xN{N}": splits[(i, N)] for (i, N) in order},
                   "schedule": args.schedule,
                   "parallelism": f"tp{world}_m_split_allgather_{exchange}" if world > 1 else "single_gpu",
                   "l2": f"inputs larger than L2: {weight_bytes / 1e6:.0f} MB of compressed weights per rank "
                         "rotate between reuses"},
        "hbm_gbs": achieved * world if world > 1 else achieved,
        "e2e": {"value": flops_per_step() / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
        "timed_as": timed_as,
        "eager_ms_per_step": eager_ms,
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "device_status": status,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": None,
                     "note": "algorithmic bytes of this rank's SpMMs / event time of the step (SpMM kernel plus "
                             "its split-K reduction launch)"},
    }
    # DRAM traffic of one SpMM launch: the ncu capture of the kernel (profiles/) shows
    # dram__bytes_read + dram__bytes_write = 1.024 x the algorithmic bytes (191.98 + 5.37 MB against 192.7 MB);
    # traffic grows with the bytes streamed, so the average launch of this workload is scaled by that ratio.
    line["roofline"]["traffic"] = 1.024 * alg_bytes_step / len(order)
    if world == 1:
        line["comparators"] = {"cublas_dense_fp16": cublas_dense(dev, acts, order, args)}
    if world == 1 and not args.case:
        line["cpu_baseline"] = cpu_baseline(mats)
        line["encoder"] = encoder_timing(dev)
    print(json.dumps(line), flush=True)
    if world > 1:
        finish_ranks(dist)


def finish_ranks(dist):
    """All ranks meet, then leave without tearing the communicator down: destroying a process group while a
    captured graph still holds its collectives did not return on this stack."""
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def cublas_dense(dev, acts, order, args):
    """Dense fp16 GEMM (cuBLAS through torch.mm, fp32 accumulate) on the un-compressed pruned weights, same shapes,
    same rotation over the matrices; the comparator the reference's drivers use (csrc/spmm_test.cu:101-102)."""
    dense = [gen_weight(M, K, i, dev) for i, (M, K) in enumerate(SHAPES)]
    outs = {k: torch.empty((k[1], SHAPES[k[0]][0]), dtype=torch.float16, device=dev) for k in order}

    def step():
        for k in order:
            torch.mm(acts[k], dense[k[0]].t(), out=outs[k])

    work = torch.cuda.Stream()
    with torch.cuda.stream(work):
        for _ in range(args.warmup):
            step()
    work.synchronize()
    graph = torch.cuda.CUDAGraph()   # timed like the SpMM loop: one captured step, replayed
    with torch.cuda.graph(graph, stream=work):
        step()
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    dense_bytes = sum(2 * SHAPES[i][0] * SHAPES[i][1] for (i, N) in order)
    return {"value": flops_per_step() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "dense_weight_gbs": dense_bytes / (ms * 1e-3) / 1e9}


def cpu_baseline(mats):
    """fp32 host GEMM over the decoded weight (the CPU restatement of the path), all host threads, bounded sample."""
    import oracle
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
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
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
