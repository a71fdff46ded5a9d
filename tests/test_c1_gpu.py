"""The isolated verify-step GEMM sweep at the 27B shapes (weights as Q4_K super-blocks built directly from seed 2,
bf16 activations, N = k+1 in {1, 2, 4, 8}) at FULL size on the GPU: dequantised rows bit-exact and GEMM outputs
within tolerance against the oracle on a sample of rows, and two size-independent properties over all rows --
a row of an N-row launch equals the N = 1 launch bit for bit, and the tcgen05 kernel agrees with the mma.sync one."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(17408, 5120), (5120, 17408), (6144, 5120)]


def _planes(llb, K, x_bf16):
    L = llb.lib()
    n = x_bf16.shape[0]
    xp = llb.handle(L.llb_b200_xp_new(K, n, 1), "xp_new")
    llb.check(L.llb_b200_xp_set_bf16(xp, x_bf16.data_ptr()), "xp_set")
    return xp


@pytest.mark.parametrize("rows,K", SHAPES)
def test_gemm_sweep_full_size(llb, packs, oracle, rows, K):
    L = llb.lib()
    dev = torch.device("cuda:0")
    fmt = packs.FMT["Q4_K"]
    raw = packs.q4k_random_blocks(rows, K, seed=2, device=dev)
    w = llb.alloc(L.llb_b200_weight_bytes(fmt, rows, K))
    llb.check(L.llb_b200_weight_upload(fmt, rows, K, raw.data_ptr(), 1, w), "weight_upload")
    rng = np.random.default_rng(2)
    sample = np.sort(rng.choice(rows, 48, replace=False)).astype(np.int32)
    raw_s = raw[torch.from_numpy(sample).to(dev).long()].cpu().numpy()
    # dequantised rows: bit-exact
    ids = torch.from_numpy(sample).to(dev)
    out = torch.zeros(len(sample), K, device=dev)
    llb.check(L.llb_b200_dequant(fmt, rows, K, w, ids.data_ptr(), len(sample), out.data_ptr()), "dequant")
    ref = oracle.Oracle.deq_rows(fmt, raw_s, len(sample), K)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    x8 = torch.randn(8, K, device=dev, generator=torch.Generator(device=dev).manual_seed(3)).to(torch.bfloat16)
    xf = x8.float().cpu().numpy()
    mass = np.abs(xf) @ np.abs(ref).T                       # [8][sample]
    ys = {}
    for n in (1, 2, 4, 8):
        xp = _planes(llb, K, x8[:n].contiguous())
        y = torch.zeros(n, rows, device=dev)
        llb.gemm(fmt, [w], [rows], [y.data_ptr()], K, xp, 0)
        L.llb_b200_sync()
        L.llb_b200_xp_free(xp)
        ys[n] = y.cpu().numpy()
        for t in range(n):
            want = oracle.Oracle.gemv(fmt, raw_s, len(sample), K, xf[t])
            assert np.all(np.abs(ys[n][t, sample] - want) <= 1e-5 * mass[t] + 1e-6), (rows, K, n, t)
    # row 0 of every N-row launch is the N = 1 launch, bit for bit, over ALL rows (what makes greedy speculation lossless)
    for n in (2, 4, 8):
        assert np.array_equal(ys[n][0].view(np.uint32), ys[1][0].view(np.uint32)), n
    # the tcgen05 kernel (N <= 4 here: 8 bf16 rows in 8 plane columns) against the mma.sync one, all rows
    was = L.llb_b200_use_tcgen05(1)
    try:
        xp = _planes(llb, K, x8[:4].contiguous())
        y = torch.zeros(4, rows, device=dev)
        llb.gemm(fmt, [w], [rows], [y.data_ptr()], K, xp, 0)
        L.llb_b200_sync()
        L.llb_b200_xp_free(xp)
        assert L.llb_b200_wait_errors() == 0
        d = np.abs(y.cpu().numpy() - ys[4])
        full_mass = float(np.abs(ys[4]).max())
        assert float(d.max()) <= 2e-5 * full_mass + 1e-5, float(d.max())
    finally:
        L.llb_b200_use_tcgen05(was)
    L.llb_b200_free(w)
