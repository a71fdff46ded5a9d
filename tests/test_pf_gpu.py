"""The prompt path's dense GEMM (tcgen05, both operands as two fp16 planes) against float64 dot products of the oracle's
dequantised weights,
through the C ABI: every weight format, ragged row counts (tiles of 128 with a partial last tile), partial chunks,
chunks of one and of two units of 128 rows (the second unit partial), several K-slices, and enough tiles that a CTA
takes more than two."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(llb, packs, oracle, dev, ty, rows, K, R, ksplit, seed):
    L = llb.lib()
    fmt = packs.FMT[ty]
    rng = np.random.default_rng(seed)
    raw = packs.QUANT[ty](torch.from_numpy(rng.standard_normal((rows, K), dtype=np.float32) * 0.05)).numpy()
    w = dev(L.llb_b200_weight_bytes(fmt, rows, K))
    llb.check(L.llb_b200_weight_upload(fmt, rows, K, raw.ctypes.data, 0, w.ptr), "weight_upload")
    x = rng.standard_normal((R, K), dtype=np.float32)
    xd = dev(x.nbytes).write(x)
    out = dev(R * rows * 4)
    llb.check(L.llb_b200_pf_gemm(fmt, w.ptr, rows, K, xd.ptr, R, out.ptr, ksplit), "llb_b200_pf_gemm")
    got = out.read((R, rows), np.float32)
    deq = oracle.Oracle.deq_rows(fmt, raw, rows, K)
    ref = x.astype(np.float64) @ deq.astype(np.float64).T
    mass = np.abs(x) @ np.abs(deq).T
    err = np.abs(got - ref)
    # both operands carry about 22 bits and the sums are fp32: the bar of the T-row GEMM tests
    assert np.all(err <= 1.0e-5 * mass + 1e-6), (ty, rows, K, R, ksplit, float((err / (mass + 1e-9)).max()))
    assert float(np.sqrt((err ** 2).mean()) / np.sqrt((ref ** 2).mean())) < 1e-5
    assert L.llb_b200_wait_errors() == 0


@pytest.mark.parametrize("ty", ["Q4_K", "Q5_K", "Q6_K", "Q8_0"])
def test_dense_gemm_formats(llb, packs, oracle, dev, ty):
    _case(llb, packs, oracle, dev, ty, 200, 512, 128, 0, seed=1)        # a partial second tile
    _case(llb, packs, oracle, dev, ty, 128, 1024, 37, 2, seed=2)        # a partial chunk, two K-slices
    _case(llb, packs, oracle, dev, ty, 300, 768, 256, 0, seed=6)        # two whole units of 128 rows
    _case(llb, packs, oracle, dev, ty, 130, 512, 191, 2, seed=7)        # the second unit partial


def test_dense_gemm_many_tiles_and_slices(llb, packs, oracle, dev):
    sms = llb.lib().llb_b200_sm_count()
    rows = 128 * (2 * sms + 40)                                          # every CTA takes at least two tiles, some three
    _case(llb, packs, oracle, dev, "Q4_K", rows, 256, 128, 1, seed=3)
    _case(llb, packs, oracle, dev, "Q4_K", 640, 2048, 100, 4, seed=4)
    _case(llb, packs, oracle, dev, "Q6_K", 48, 1536, 128, 3, seed=5)    # fewer rows than a tile
    _case(llb, packs, oracle, dev, "Q4_K", 128 * (sms + 9), 512, 256, 1, seed=8)   # two units, more than one tile per CTA
