"""The allocation-free GEMM entry point (llb_b200_gemm_noalloc) against the ordinary one.

It exists for hosts that hand a library its memory once and then forbid driver allocations (serving
processes that cannot take cudaMalloc's device-wide stall, sandboxes that deny the call): its scratch is a
fixed array inside the library image, shared by all calls and never cleared between them.  So the check is
two calls in a row with different shapes -- the second must not see the first's leftovers -- each compared
with llb_b200_gemm on the same inputs and, so that a fault shared by both entry points cannot hide, with the CPU
oracle's row-by-row dot products.  This file sorts last on purpose: a run that stops at the first
failure has then already run every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(llb, packs, oracle, dev, ty, rows, K, T, seed):
    L = llb.lib()
    fmt = packs.FMT[ty]
    rng = np.random.default_rng(seed)
    raw = packs.QUANT[ty](torch.from_numpy(rng.standard_normal((rows, K), dtype=np.float32) * 0.05)).numpy()
    w = dev(L.llb_b200_weight_bytes(fmt, rows, K))
    llb.check(L.llb_b200_weight_upload(fmt, rows, K, raw.ctypes.data, 0, w.ptr), "weight_upload")
    x = rng.standard_normal((T, K), dtype=np.float32)
    xd = dev(x.nbytes).write(x)
    # the ordinary entry point (allocates its planes and scratch)
    xp = llb.handle(L.llb_b200_xp_new(K, T, 2), "xp_new")
    llb.check(L.llb_b200_xp_set_f32(xp, xd.ptr), "xp_set")
    o1 = dev(T * rows * 4)
    llb.gemm(fmt, [w.ptr], [rows], [o1.ptr], K, xp, 0)
    ref = o1.read((T, rows), np.float32)
    L.llb_b200_xp_free(xp)
    # the allocation-free one
    o2 = dev(T * rows * 4)
    llb.check(L.llb_b200_gemm_noalloc(fmt, w.ptr, rows, K, xd.ptr, T, o2.ptr), "llb_b200_gemm_noalloc")
    got = o2.read((T, rows), np.float32)
    deq = np.abs(packs.dequant(ty, torch.from_numpy(raw), rows, K).numpy())
    mass = np.abs(x) @ deq.T
    assert np.all(np.abs(got - ref) <= 1e-5 * mass + 1e-6), (ty, rows, K, T, float(np.abs(got - ref).max()))
    cpu = np.stack([oracle.Oracle.gemv(fmt, raw, rows, K, x[t]) for t in range(T)])
    assert np.all(np.abs(got - cpu) <= 1e-5 * mass + 1e-6), (ty, rows, K, T, float(np.abs(got - cpu).max()))
    return got


def test_noalloc_matches_ordinary_entry_point_twice(llb, packs, oracle, dev):
    # first a wide, K-split case with all four rows, then a narrower one with fewer rows and another format:
    # stale planes or partial sums from the first call would show in the second
    _both(llb, packs, oracle, dev, "Q4_K", 320, 8192, 4, seed=1)
    _both(llb, packs, oracle, dev, "Q6_K", 96, 1024, 2, seed=2)
    _both(llb, packs, oracle, dev, "Q4_K", 320, 8192, 4, seed=3)


def test_noalloc_rejects_what_does_not_fit(llb, packs, dev):
    L = llb.lib()
    w = dev(1 << 20)
    x = dev(1 << 20)
    o = dev(1 << 20)
    for args, word in (((packs.FMT["Q4_K"], w.ptr, 64, 8192 + 256, x.ptr, 4, o.ptr), b"8192"),
                       ((packs.FMT["Q4_K"], w.ptr, 64, 1024, x.ptr, 5, o.ptr), b"1..4"),
                       ((packs.FMT["Q4_K"], w.ptr, 64, 1000, x.ptr, 4, o.ptr), b"256"),
                       ((packs.FMT["Q4_K"], w.ptr, 3000000, 256, x.ptr, 4, o.ptr), b"scratch")):
        assert L.llb_b200_gemm_noalloc(*args) == -1
        assert word in L.llb_b200_last_error(), L.llb_b200_last_error()
