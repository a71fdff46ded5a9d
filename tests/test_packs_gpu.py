"""The pack writers run on the GPU too (27B-shape packs are quantised where they stay).  Their bytes
may differ from the CPU's in the last bit of an f16 scale (torch divides by a constant differently on
the two devices), so the check is that the GPU-written blocks are valid: the oracle decodes them to
exactly what the torch decoder gives, and they are as close to the weights as the CPU-written ones."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ty", ["Q8_0", "Q4_K", "Q5_K", "Q6_K"])
def test_quantisers_cpu_equals_gpu(packs, oracle, llb, ty):
    rng = np.random.default_rng(4)
    w = torch.from_numpy(rng.standard_normal((96, 2560), dtype=np.float32) * 0.02)
    raw_cpu = packs.QUANT[ty](w)
    raw_gpu = packs.QUANT[ty](w.cuda())
    assert raw_gpu.shape == raw_cpu.shape
    assert (raw_gpu.cpu() != raw_cpu).float().mean().item() < 1e-3
    deq_gpu = packs.dequant(ty, raw_gpu, 96, 2560).cpu().numpy()
    ref = oracle.Oracle.deq_rows(packs.FMT[ty], raw_gpu.cpu().numpy(), 96, 2560)
    assert np.array_equal(deq_gpu.view(np.uint32), ref.view(np.uint32))
    err_cpu = float((packs.dequant(ty, raw_cpu, 96, 2560) - w).abs().max())
    assert float(np.abs(deq_gpu - w.numpy()).max()) <= 1.01 * err_cpu + 1e-7
    idx = torch.tensor([5, 90, 17], device="cuda")
    sub = packs.dequant(ty, raw_gpu.reshape(96, -1)[idx].contiguous(), 3, 2560).cpu().numpy()
    assert np.array_equal(sub.view(np.uint32), ref[[5, 90, 17]].view(np.uint32))
