"""The tensor-parallel decoder-layer harness on one GPU against a dense fp32 torch reference of the same layer.

Tolerance: the four linear layers each carry the SpMM tolerance (1e-2 of the output scale); the layer output is
compared at 2e-2 * max|ref|, and the decode step (one new token on the cache) against a prefill one token longer."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def sp(lib_built):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import spmspm_b200
    spmspm_b200.reset_device_status()
    return spmspm_b200


def test_layer_matches_dense_reference_and_decode_matches_prefill(sp):
    from spmspm_b200.layer import SparseOptDecoderLayer, _gen
    dev = torch.device("cuda", 0)
    B, T, hidden, heads, ffn = 2, 8, 256, 4, 1024
    layer = SparseOptDecoderLayer(hidden, heads, ffn, 0.6, dev, batch=B, max_len=32, keep_dense=True)
    x = _gen((B * (T + 1), hidden), 3, dev, 1.0).reshape(B, T + 1, hidden)
    # prefill of T + 1 tokens at once
    layer.reset()
    full = layer.forward(x.reshape(B * (T + 1), hidden).contiguous(), T + 1).reshape(B, T + 1, hidden)
    ref = layer.forward_dense_reference(x.reshape(B * (T + 1), hidden).contiguous(), T + 1).reshape(B, T + 1, hidden)
    scale = float(ref.abs().max())
    assert float((full.float() - ref).abs().max()) <= 2e-2 * scale
    # prefill of T tokens, then one decode step: the last token's output must agree with the long prefill
    layer.reset()
    layer.forward(x[:, :T].reshape(B * T, hidden).contiguous(), T)
    last = layer.forward(x[:, T].contiguous(), 1)
    assert int(layer.pos.item()) == T + 1
    assert float((last.float() - full[:, T].float()).abs().max()) <= 1e-2 * scale
    assert sp.device_status() == 0


def test_generation_timer_runs_with_and_without_graph(sp):
    from spmspm_b200.layer import SparseOptDecoderLayer, generate_timed
    dev = torch.device("cuda", 0)
    layer = SparseOptDecoderLayer(256, 4, 1024, 0.6, dev, batch=2, max_len=24)
    for use_graph in (False, True):
        total, pre, per_step, graphed = generate_timed(layer, 8, 12, steps=1, warmup=1, use_graph=use_graph)
        assert total > 0 and pre > 0 and per_step > 0 and (graphed or not use_graph)
        assert int(layer.pos.item()) == 20
    assert sp.device_status() == 0


_CHILD = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import spmspm_b200 as sp
from spmspm_b200.layer import SparseOptDecoderLayer, generate_timed, _gen
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
alone = [dist.new_group([r]) for r in range(world)][rank]        # a group of this rank only: the unsplit layer
B, T, hidden, heads, ffn = 2, 8, 512, 8, 2048
x = _gen((B * T, hidden), 3, dev, 1.0)
xt = _gen((B, hidden), 4, dev, 1.0)
whole = SparseOptDecoderLayer(hidden, heads, ffn, 0.6, dev, batch=B, max_len=32, group=alone, reduce="none")
want = whole.forward(x, T).float(); want1 = whole.forward(xt, 1).float()
scale = float(want.abs().max())
bad = 0
for kind in ("peer", "nccl"):
    layer = SparseOptDecoderLayer(hidden, heads, ffn, 0.6, dev, batch=B, max_len=32, reduce=kind)
    layer.prepare([B * T, B])
    for _ in range(2):                                           # twice: the exchange buffers are reused
        layer.reset()
        got = layer.forward(x, T).float(); got1 = layer.forward(xt, 1).float()
        torch.cuda.synchronize()
        bad += int(float((got - want).abs().max()) > 1e-2 * scale)
        bad += int(float((got1 - want1).abs().max()) > 1e-2 * scale)
    total, pre, step, graphed = generate_timed(layer, 8, 12, steps=1, warmup=1)
    bad += int(not (total > 0 and step > 0))
    dist.barrier()
bad += int(sp.device_status() != 0)
open(os.path.join(sys.argv[2], f"result_{rank}"), "w").write(str(bad))
dist.barrier(); os._exit(0 if bad == 0 else 1)
"""


def test_two_rank_layer_matches_the_unsplit_layer(lib_built, tmp_path):
    """Tensor-parallel over two GPUs, with the one-shot all-reduce over peer stores and with NCCL, against the same
    layer on one rank (tolerance 1e-2 of the output scale: the K-split changes the order of the fp32 sums)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", str(script), root, str(tmp_path)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    for rank in (0, 1):
        assert (tmp_path / f"result_{rank}").read_text() == "0"
