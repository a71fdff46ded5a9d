"""GPU parity of the dequant-fused skinny GEMM and of row dequantisation, through the C ABI,
against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FMTS = ["Q4_K", "Q5_K", "Q6_K", "Q8_0"]


def _upload(llb, packs, dev, ty, raw, rows, cols):
    L = llb.lib()
    fmt = packs.FMT[ty]
    w = dev(L.llb_b200_weight_bytes(fmt, rows, cols))
    raw = np.ascontiguousarray(raw)
    llb.check(L.llb_b200_weight_upload(fmt, rows, cols, raw.ctypes.data, 0, w.ptr), "weight_upload")
    return w


def _random_raw(packs, ty, rows, cols, seed):
    """Valid blocks with every field exercised: quantised Gaussians, then the scale fields
    overwritten with random bytes (negative int8 scales, all 64 six-bit values, subnormal f16 d)."""
    rng = np.random.default_rng(seed)
    w = torch.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32) * 0.05)
    raw = packs.QUANT[ty](w).numpy().copy()
    if ty in ("Q4_K", "Q5_K"):
        bb = 144 if ty == "Q4_K" else 176
        blk = raw.reshape(rows, cols // 256, bb)
        blk[:, :, 4:16] = rng.integers(0, 256, blk[:, :, 4:16].shape, dtype=np.uint8)
    elif ty == "Q6_K":
        blk = raw.reshape(rows, cols // 256, 210)
        blk[:, :, 192:208] = rng.integers(0, 256, blk[:, :, 192:208].shape, dtype=np.uint8)
    return raw


@pytest.mark.parametrize("ty", FMTS)
def test_dequant_bit_exact(llb, packs, oracle, dev, ty):
    rows, cols = 48, 1280
    raw = _random_raw(packs, ty, rows, cols, 3)
    w = _upload(llb, packs, dev, ty, raw, rows, cols)
    out = dev(rows * cols * 4)
    llb.check(llb.lib().llb_b200_dequant(packs.FMT[ty], rows, cols, w.ptr, 0, rows, out.ptr), "dequant")
    got = out.read((rows, cols), np.float32)
    ref = oracle.Oracle.deq_rows(packs.FMT[ty], raw, rows, cols)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # gathered rows (the embedding lookup)
    ids = np.array([7, 0, 47, 7], np.int32)
    idb = dev(ids.nbytes).write(ids)
    llb.check(llb.lib().llb_b200_dequant(packs.FMT[ty], rows, cols, w.ptr, idb.ptr, 4, out.ptr), "dequant")
    got = out.read((4, cols), np.float32)
    assert np.array_equal(got.view(np.uint32), ref[ids].view(np.uint32))


def _gemm_case(llb, packs, oracle, dev, ty, rows_list, K, T, planes, ksplit, seed):
    L = llb.lib()
    fmt = packs.FMT[ty]
    rng = np.random.default_rng(seed)
    raws = [_random_raw(packs, ty, r, K, seed + 10 * i) for i, r in enumerate(rows_list)]
    ws = [_upload(llb, packs, dev, ty, raw, r, K) for raw, r in zip(raws, rows_list)]
    x = rng.standard_normal((T, K), dtype=np.float32)
    if planes == 1:
        xb = torch.from_numpy(x).to(torch.bfloat16)
        x = xb.float().numpy()
        xd = dev(T * K * 2).write(xb.view(torch.int16).numpy())
    else:
        xd = dev(T * K * 4).write(x)
    xp = llb.handle(L.llb_b200_xp_new(K, T, planes), "xp_new")
    try:
        llb.check((L.llb_b200_xp_set_bf16 if planes == 1 else L.llb_b200_xp_set_f32)(xp, xd.ptr), "xp_set")
        outs = [dev(T * r * 4) for r in rows_list]
        llb.gemm(fmt, [w.ptr for w in ws], rows_list, [o.ptr for o in outs], K, xp, ksplit)
        for raw, r, o in zip(raws, rows_list, outs):
            got = o.read((T, r), np.float32)
            ref = np.stack([oracle.Oracle.gemv(fmt, raw, r, K, x[t]) for t in range(T)])
            # f32 accumulation in a different order than the oracle's serial dot: 1e-5 of the row's
            # absolute dot mass is far inside the path's 2e-2 / 1e-2 logit tolerance
            deq = np.abs(oracle.Oracle.deq_rows(fmt, raw, r, K))
            mass = np.abs(x) @ deq.T
            assert np.all(np.abs(got - ref) <= 1e-5 * mass + 1e-6), (ty, rows_list, K, T, planes, ksplit,
                                                                    float(np.abs(got - ref).max()))
    finally:
        L.llb_b200_xp_free(xp)


@pytest.mark.parametrize("ty", FMTS)
@pytest.mark.parametrize("K,ksplit", [(256, 1), (768, 1), (1280, 0), (2560, 3), (5120, 0)])
def test_gemm_vs_oracle(llb, packs, oracle, dev, ty, K, ksplit):
    _gemm_case(llb, packs, oracle, dev, ty, [80], K, 4, 2, ksplit, seed=K)


@pytest.mark.parametrize("ty", FMTS)
def test_gemm_ragged_rows_and_cat(llb, packs, oracle, dev, ty):
    # four matrices sharing x, row counts that are not multiples of 16 (8-row beta/alpha of the 0.8B shape)
    _gemm_case(llb, packs, oracle, dev, ty, [40, 8, 16, 3], 1024, 4, 2, 0, seed=5)
    _gemm_case(llb, packs, oracle, dev, ty, [40, 8, 16, 3], 1024, 4, 2, 2, seed=6)


@pytest.mark.parametrize("ty", FMTS)
@pytest.mark.parametrize("T,planes", [(1, 2), (2, 2), (3, 2), (6, 2), (8, 2), (9, 2), (12, 2), (16, 2), (1, 1), (8, 1), (16, 1), (32, 1)])
def test_gemm_row_counts(llb, packs, oracle, dev, ty, T, planes):
    _gemm_case(llb, packs, oracle, dev, ty, [64], 1536, T, planes, 0, seed=T + planes)


@pytest.mark.parametrize("ty", FMTS)
def test_gemm_sixteen_rows_long_k(llb, packs, oracle, dev, ty):
    """Sixteen rows (the rows of several streams in one pass, 32 plane columns) at the 27B shape's widest K: the
    activation slice a CTA can stage is small there, so K splits 12 to 16 ways (Q6_K on a two-stage ring)."""
    _gemm_case(llb, packs, oracle, dev, ty, [48, 16], 17408, 16, 2, 0, seed=21)
    _gemm_case(llb, packs, oracle, dev, ty, [33], 5120, 13, 2, 0, seed=22)


def test_gemm_many_tiles(llb, packs, oracle, dev):
    # more tiles than resident warps: every warp walks several units and prefetches across them
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [20000], 512, 4, 2, 0, seed=9)
    _gemm_case(llb, packs, oracle, dev, "Q6_K", [20000], 512, 4, 2, 2, seed=9)


def test_column_independence(llb, packs, dev):
    """Row t of a T-row launch equals the T = 1 launch bit for bit (the property that makes greedy
    speculative decoding lossless; the reference checks the same for its T-row leaves,
    tools/payload-spec.patch:41-44)."""
    _column_independence(llb, packs, dev)


def _column_independence(llb, packs, dev):
    L = llb.lib()
    rows, K = 256, 2048
    rng = np.random.default_rng(1)
    raw = packs.QUANT["Q4_K"](torch.from_numpy(rng.standard_normal((rows, K), dtype=np.float32) * 0.02)).numpy()
    w = _upload(llb, packs, dev, "Q4_K", raw, rows, K)
    x = rng.standard_normal((4, K), dtype=np.float32)
    ys = []
    for T, xs in ((4, x), (1, x[2:3])):
        xd = dev(T * K * 4).write(xs)
        xp = llb.handle(L.llb_b200_xp_new(K, T, 2), "xp_new")
        llb.check(L.llb_b200_xp_set_f32(xp, xd.ptr), "xp_set")
        o = dev(T * rows * 4)
        llb.gemm(packs.FMT["Q4_K"], [w.ptr], [rows], [o.ptr], K, xp, 2)
        ys.append(o.read((T, rows), np.float32))
        L.llb_b200_xp_free(xp)
    assert np.array_equal(ys[0][2].view(np.uint32), ys[1][0].view(np.uint32))


@pytest.mark.parametrize("ty", FMTS)
def test_row_independence_at_sixteen_rows(llb, packs, dev, ty):
    """A row's result does not depend on which other rows share the launch nor on its place among them: what lets
    several streams be verified in one pass with each stream's tokens bit-identical to the stream run alone."""
    L = llb.lib()
    rows, K = 96, 2560
    raw = _random_raw(packs, ty, rows, K, 31)
    w = _upload(llb, packs, dev, ty, raw, rows, K)
    rng = np.random.default_rng(2)
    xa, xb = rng.standard_normal((16, K), dtype=np.float32), rng.standard_normal((16, K), dtype=np.float32)
    xb[3] = xa[9]
    ys = []
    for xs in (xa, xb):
        xd = dev(16 * K * 4).write(xs)
        xp = llb.handle(L.llb_b200_xp_new(K, 16, 2), "xp_new")
        llb.check(L.llb_b200_xp_set_f32(xp, xd.ptr), "xp_set")
        o = dev(16 * rows * 4)
        llb.gemm(packs.FMT[ty], [w.ptr], [rows], [o.ptr], K, xp, 0)
        ys.append(o.read((16, rows), np.float32))
        L.llb_b200_xp_free(xp)
    assert np.array_equal(ys[0][9].view(np.uint32), ys[1][3].view(np.uint32))


@pytest.fixture
def tcgen05(llb):
    """Q4_K, T <= 4 GEMMs of this test run on the tcgen05 kernel (weights in tensor memory)."""
    L = llb.lib()
    was = L.llb_b200_use_tcgen05(1)
    yield
    L.llb_b200_use_tcgen05(was)
    assert L.llb_b200_wait_errors() == 0      # no bounded wait on an mbarrier ran out


@pytest.mark.parametrize("K,ksplit", [(256, 1), (768, 1), (1280, 0), (2560, 3), (5120, 0)])
def test_tcgen05_gemm_vs_oracle(llb, packs, oracle, dev, tcgen05, K, ksplit):
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [80], K, 4, 2, ksplit, seed=K)
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [300], K, 3, 2, ksplit, seed=K + 1)


def test_tcgen05_column_independence(llb, packs, dev, tcgen05):
    _column_independence(llb, packs, dev)


def test_tcgen05_gemm_ragged_cat_and_planes(llb, packs, oracle, dev, tcgen05):
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [40, 8, 16, 3], 1024, 4, 2, 0, seed=5)
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [200, 130, 128], 1024, 4, 2, 2, seed=6)
    for T, planes in ((1, 2), (2, 2), (1, 1), (8, 1)):
        _gemm_case(llb, packs, oracle, dev, "Q4_K", [64], 1536, T, planes, 0, seed=T + planes)


def test_tcgen05_gemm_many_tiles(llb, packs, oracle, dev, tcgen05):
    # more 128-row tiles than CTAs: a CTA walks several tiles and prefetches across them
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [40000], 512, 4, 2, 0, seed=9)
    _gemm_case(llb, packs, oracle, dev, "Q4_K", [20000], 1024, 4, 2, 2, seed=10)
