"""Activation offload: same gradients with and without it; on the GPU the kept tensors really leave the
device (bytes counted) and come back layer by layer."""
import pytest
import torch

from axon_b200.models.config import tiny_gpu, tiny_qwen3
from axon_b200.models.dense import DenseModel, PackedBatch
from axon_b200.utils.activation_offload import ActivationOffloader


def _grads(dev, dtype, cfg, offload, recompute):
    m = DenseModel(cfg, device=dev, dtype=dtype)
    m.params.init_random(std=0.05, seed=3)
    m.recompute = recompute
    if offload:
        m.offloader = ActivationOffloader(dev, min_bytes=1024)
    g = torch.Generator().manual_seed(0)
    b = PackedBatch.from_sequences([torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (200, 312)], dev)
    m.params.alloc_grads()
    for _ in range(2):                      # two steps: the pinned pool is reused
        lp, _ = m.forward(b, 1.0, save_for_backward=True)
        m.backward(torch.ones_like(lp) / lp.numel(), None)
    return m.params.grad_flat.clone(), (m.offloader.stats if offload else None)


@pytest.mark.parametrize("recompute", ["full", "none"])
def test_offload_is_transparent_cpu(recompute):
    a, _ = _grads("cpu", torch.float32, tiny_qwen3(), False, recompute)
    b, st = _grads("cpu", torch.float32, tiny_qwen3(), True, recompute)
    assert torch.equal(a, b) and st["offloaded_bytes"] == 0      # CPU tensors pass through


@pytest.mark.gpu
@pytest.mark.parametrize("recompute", ["full", "selective", "none"])
def test_offload_matches_and_moves_bytes_gpu(recompute):
    a, _ = _grads("cuda", torch.bfloat16, tiny_gpu(), False, recompute)
    b, st = _grads("cuda", torch.bfloat16, tiny_gpu(), True, recompute)
    assert torch.equal(a, b)
    assert st["offloaded_bytes"] > 0 and st["fetched_bytes"] == st["offloaded_bytes"]
