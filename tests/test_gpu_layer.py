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
