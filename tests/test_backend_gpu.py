"""The backend half of the boundary on the GPU: kernels fetched by name and launched with the reference's LLB_LAUNCH
argument convention (host/llb_backend.h:9-24), the launch recorder (host/llb_backend_cuda.h:125-184), and the
one-device-per-process rule of llb_b200_init."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _launch(L, k, gx, gy, bx, sm, *vals):
    """LLB_LAUNCH's convention: every argument is the address of a host variable copied at the call."""
    holders = list(vals)
    argv = (C.c_void_p * len(holders))(*[C.addressof(h) for h in holders])
    return L.llb_b200_launch(k, gx, gy, bx, sm, argv, len(holders))


def test_kernel_by_name_and_launch(llb, packs, oracle, dev):
    L = llb.lib()
    assert not L.llb_b200_kernel_by_name(b"llb_spec_gu3")                 # a reference kernel: not exported
    assert b"llb_spec_gu3" in L.llb_b200_last_error()
    assert _launch(L, None, 1, 1, 256, 0, C.c_int(0)) == -1               # a NULL handle queues nothing and says so
    k = L.llb_b200_kernel_by_name(b"llb_b200_k_dequant_rows")
    assert k
    rows, cols, ty = 24, 512, "Q4_K"
    fmt = packs.FMT[ty]
    rng = np.random.default_rng(3)
    raw = packs.QUANT[ty](torch.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32) * 0.05)).numpy()
    w = dev(L.llb_b200_weight_bytes(fmt, rows, cols))
    llb.check(L.llb_b200_weight_upload(fmt, rows, cols, raw.ctypes.data, 0, w.ptr), "upload")
    out = dev(rows * cols * 4)
    assert _launch(L, k, 2, rows, 256, 0, C.c_int(fmt), C.c_uint64(w.ptr), C.c_int(cols)) == -1      # wrong argument count
    assert b"arguments" in L.llb_b200_last_error()
    assert _launch(L, k, 2, rows, 256, 0, C.c_int(fmt), C.c_uint64(w.ptr), C.c_int(cols), C.c_uint64(0), C.c_uint64(out.ptr)) == 0
    got = out.read((rows, cols), np.float32)
    ref = oracle.Oracle.deq_rows(fmt, raw, rows, cols)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))      # dequantisation is bit-exact


def test_graph_recorder_replays_and_bails(llb, dev):
    L = llb.lib()
    k = L.llb_b200_kernel_by_name(b"llb_b200_k_sum_parts")
    n, ns = 1000, 3
    parts = np.arange(ns * n, dtype=np.float32).reshape(ns, n)
    p, o = dev(parts.nbytes).write(parts), dev(n * 4)
    st0 = (C.c_ulonglong * 4)()
    L.llb_b200_graph_stats(st0)
    for it in range(3):
        assert L.llb_b200_graph_begin() == 0
        # two launches a step; the second step re-uses the first one's graph with new arguments
        assert _launch(L, k, 4, 1, 256, 0, C.c_uint64(p.ptr), C.c_int(ns - (it == 1)), C.c_longlong(n), C.c_int(n), C.c_uint64(o.ptr)) == 0
        assert _launch(L, k, 4, 1, 256, 0, C.c_uint64(p.ptr), C.c_int(ns - (it == 1)), C.c_longlong(n), C.c_int(n), C.c_uint64(o.ptr)) == 0
        assert L.llb_b200_graph_end() == 0
        got = o.read((n,), np.float32)                      # llb_b200_read synchronises
        assert np.array_equal(got, parts[: ns - (it == 1)].sum(0))
    st = (C.c_ulonglong * 4)()
    L.llb_b200_graph_stats(st)
    assert st[0] - st0[0] == 1 and st[1] - st0[1] == 3 and st[2] - st0[2] == 2
    # a memory primitive while recording runs what was recorded first
    o.write(np.zeros(n, np.float32))
    assert L.llb_b200_graph_begin() == 0
    assert _launch(L, k, 4, 1, 256, 0, C.c_uint64(p.ptr), C.c_int(ns), C.c_longlong(n), C.c_int(n), C.c_uint64(o.ptr)) == 0
    got = o.read((n,), np.float32)                          # bails: the launch has run
    assert np.array_equal(got, parts.sum(0))
    L.llb_b200_graph_stats(st)
    assert st[3] - st0[3] >= 1
    assert L.llb_b200_graph_end() == 0                      # nothing is being recorded any more


def test_one_device_per_process(llb):
    L = llb.lib()
    assert L.llb_b200_init(0) == 0                          # the same device again: a no-op
    assert L.llb_b200_init(1) == -1
    assert b"already bound" in L.llb_b200_last_error()


@pytest.mark.parametrize("which", [0, 1], ids=["mbarrier", "grid-barrier"])
def test_a_bounded_wait_that_runs_out(llb, packs, oracle, dev, which):
    """Failure detection without a fault: a launch whose only wait nothing can satisfy (an mbarrier nobody arrives on,
    waited for with the tcgen05 kernels' bounded wait; the fused FFN's grid barrier told to expect a block that does
    not exist) gives up after 2000 tries, sets the status word and returns.  The host reads 1, clears it, and the
    device still computes: a dequantisation afterwards is bit-exact."""
    L = llb.lib()
    assert L.llb_b200_wait_errors() == 0
    assert L.llb_b200_wait_selftest(which, 0) == -1 and b"limit" in L.llb_b200_last_error()
    assert L.llb_b200_wait_selftest(which, 2000) == 0
    assert L.llb_b200_wait_errors() == 1
    assert L.llb_b200_wait_errors_clear() == 0
    assert L.llb_b200_wait_errors() == 0
    rows, cols, ty = 16, 512, "Q6_K"
    fmt = packs.FMT[ty]
    rng = np.random.default_rng(5)
    raw = packs.QUANT[ty](torch.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32) * 0.05)).numpy()
    w = dev(L.llb_b200_weight_bytes(fmt, rows, cols))
    llb.check(L.llb_b200_weight_upload(fmt, rows, cols, raw.ctypes.data, 0, w.ptr), "upload")
    out = dev(rows * cols * 4)
    llb.check(L.llb_b200_dequant(fmt, rows, cols, w.ptr, 0, rows, out.ptr), "dequant")
    ref = oracle.Oracle.deq_rows(fmt, raw, rows, cols)
    assert np.array_equal(out.read((rows, cols), np.float32).view(np.uint32), ref.view(np.uint32))
    assert L.llb_b200_wait_errors() == 0
