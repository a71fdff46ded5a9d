"""ctypes binding of libllb_b200.so (the C ABI declared in include/llb_b200.h).

The library is the product; this module only loads it and turns error codes into exceptions.
There is no CPU fallback: importing works anywhere, but every call needs a B200 and raises if the
shared library is missing or the device is not sm_100.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.environ.get("LLB_SO") or os.path.join(HERE, "libllb_b200.so")   # LLB_SO: another build of the library

F32, Q8_0, Q4_K, Q6_K, Q5_K = 0, 1, 3, 4, 9
FMT_ID = {"F32": F32, "Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K, "Q5_K": Q5_K}

_lib = None


class LlbError(RuntimeError):
    pass


def build(verbose: bool = False) -> str:
    """Compile libllb_b200.so for sm_100a (nvcc cross-compiles without a GPU)."""
    r = subprocess.run(["make", "-C", os.path.join(HERE, "csrc"), "-j8"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode:
        raise LlbError("building libllb_b200.so failed")
    return SO_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise LlbError(f"{SO_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` first; "
                           "there is no fallback path")
        L = C.CDLL(SO_PATH)
        vp, i32, u64, sz = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t
        sig = {
            "llb_b200_init": (i32, [i32]), "llb_b200_last_error": (C.c_char_p, []), "llb_b200_sm_count": (i32, []),
            "llb_b200_alloc_zero": (u64, [sz]), "llb_b200_free": (i32, [u64]), "llb_b200_zero": (i32, [u64, sz]),
            "llb_b200_copy": (i32, [u64, u64, sz]), "llb_b200_write": (i32, [u64, vp, sz]), "llb_b200_read": (i32, [vp, u64, sz]),
            "llb_b200_sync": (i32, []), "llb_b200_stream": (u64, []),
            "llb_b200_weight_bytes": (sz, [i32, i32, i32]),
            "llb_b200_weight_upload": (i32, [i32, i32, i32, vp, i32, u64]),
            "llb_b200_dequant": (i32, [i32, i32, i32, u64, u64, i32, u64]),
            "llb_b200_xp_new": (vp, [i32, i32, i32]), "llb_b200_xp_free": (None, [vp]),
            "llb_b200_xp_set_f32": (i32, [vp, u64]), "llb_b200_xp_set_bf16": (i32, [vp, u64]),
            "llb_b200_gemm": (i32, [i32, i32, C.POINTER(u64), C.POINTER(i32), C.POINTER(u64), i32, vp, i32]),
            "llb_b200_wait_errors": (i32, []), "llb_b200_wait_errors_clear": (i32, []), "llb_b200_wait_selftest": (i32, [i32, i32]), "llb_b200_use_tcgen05": (i32, [i32]), "llb_b200_use_fused_ffn": (i32, [i32]),
            "llb_b200_gemm_host": (i32, [i32, u64, i32, i32, vp, i32, vp, vp, u64, u64]),
            "llb_b200_gemm_noalloc": (i32, [i32, u64, i32, i32, u64, i32, u64]),
            "llb_spec_open": (vp, [C.c_char_p, vp, sz, i32, vp, sz, i32, i32, i32, i32]),
            "llb_spec_close": (None, [vp]), "llb_spec_reset": (i32, [vp]),
            "llb_spec_prefill": (i32, [vp, vp, i32]), "llb_spec_cycle": (i32, [vp, vp, vp, vp]),
            "llb_spec_generate": (i32, [vp, i32, vp, vp]), "llb_spec_pass": (i32, [vp, i32, i32, vp]),
            "llb_spec_position": (i32, [vp]), "llb_spec_stats": (i32, [vp, vp]),
            "llb_spec_read_state": (i32, [vp, i32, i32, i32, vp, sz]), "llb_spec_read_logits": (i32, [vp, i32, vp]),
            "llb_spec_moe_ffn": (i32, [vp, i32, i32, vp, vp, vp, vp]),
            "llb_spec_open_gguf": (vp, [C.c_char_p, vp, sz, i32, i32, i32, i32]), "llb_b200_gguf_index": (i32, [C.c_char_p, vp, i32]),
            "llb_spec_run_cycles": (i32, [vp, i32, vp, i32]), "llb_spec_time_verify": (i32, [vp, i32, vp]),
            "llb_spec_time_verify_rows": (i32, [vp, i32, i32, vp]),
            "llb_spec_time_gemm": (i32, [vp, i32, vp, vp]), "llb_spec_graph_nodes": (i32, [vp, i32]),
            "llb_spec_profile_verify": (i32, [vp, C.c_char_p, i32]),
            "llb_spec_check_index": (i32, [C.c_char_p, sz]),
            "llb_b200_tp_unique_id": (i32, [C.c_char_p, vp]), "llb_b200_tp_init": (i32, [C.c_char_p, i32, i32, vp]),
            "llb_b200_tp_finalize": (None, []), "llb_b200_tp_plan": (i32, [i32, i32, i32, i32, i32, i32, i32, C.POINTER(i32)]),
            "llb_spec_open_tp": (vp, [C.c_char_p, vp, sz, i32, vp, sz, i32, i32, i32, i32, i32]),
            "llb_b200_tp_peer_alloc": (i32, [vp]), "llb_b200_tp_peer_open": (i32, [vp, i32]), "llb_b200_tp_peer_active": (i32, []),
            "llb_spec_last_record": (i32, [vp, i32, vp]),
            "llb_spec_set_sampler": (i32, [vp, vp]), "llb_spec_sampler_errors": (i32, [vp]),
            "llb_b200_smp_rows": (i32, [vp, u64, i32, i32, vp, vp, vp, vp, vp, vp, vp]),
            "llb_spec_open_streams": (vp, [C.c_char_p, vp, sz, i32, vp, sz, i32, i32, i32, i32, i32]),
            "llb_spec_streams": (i32, [vp]), "llb_spec_prefill_stream": (i32, [vp, i32, vp, i32]),
            "llb_spec_prefill_streams": (i32, [vp, i32, vp, vp, vp]),
            "llb_spec_open_sibling": (vp, [vp, i32, i32, i32]), "llb_spec_weight_bytes": (sz, [vp]),
            "llb_spec_cycle_streams": (i32, [vp, vp, vp, vp]), "llb_spec_run_cycles_streams": (i32, [vp, i32, vp]),
            "llb_spec_position_stream": (i32, [vp, i32]), "llb_spec_stats_stream": (i32, [vp, i32, vp]),
            "llb_spec_read_state_stream": (i32, [vp, i32, i32, i32, i32, vp, sz]),
            "llb_spec_set_prefill": (i32, [vp, i32]), "llb_spec_fast_rows": (C.c_double, [vp]),
            "llb_b200_pf_gemm": (i32, [i32, u64, i32, i32, u64, i32, u64, i32]),
            "llb_b200_gemm_ksplit": (i32, [i32, i32, i32, i32, i32]), "llb_b200_ring_ksplit": (i32, [i32, i32, i32, i32, i32, i32]),
            "llb_b200_kernel_by_name": (vp, [C.c_char_p]),
            "llb_b200_launch": (i32, [vp, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.POINTER(vp), C.c_uint]),
            "llb_b200_graph_begin": (i32, []), "llb_b200_graph_end": (i32, []), "llb_b200_graph_bail": (i32, []),
            "llb_b200_graph_stats": (None, [C.POINTER(C.c_ulonglong)]),
        }
        for name, (res, args) in sig.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def check(rc, what: str = "call"):
    """Raise with the library's own message when a call returned a negative status."""
    if isinstance(rc, int) and rc < 0:
        raise LlbError(f"{what} failed: {lib().llb_b200_last_error().decode()}")
    return rc


def handle(h, what: str):
    """Raise when a call that returns a handle / device address returned 0."""
    if not h:
        raise LlbError(f"{what} failed: {lib().llb_b200_last_error().decode()}")
    return h


def init(device: int = 0):
    check(lib().llb_b200_init(device), "llb_b200_init")


def tp_plan(rank: int, size: int, H: int, KV: int, f: int, GK: int, TR: int):
    """Rank `rank` of `size`'s share of a model (no GPU needed): dict of H_l, h0, KV_l, kv0, f_l, f0, GK_l, g0, TR_l, reps."""
    out = (C.c_int * 10)()
    check(lib().llb_b200_tp_plan(rank, size, H, KV, f, GK, TR, out), "llb_b200_tp_plan")
    return dict(zip(("H_l", "h0", "KV_l", "kv0", "f_l", "f0", "GK_l", "g0", "TR_l", "reps"), list(out)))


def exchange_unique_id(make_id, rank: int, device=None):
    """Rank 0's 128-byte communicator id on every rank of the initialised torch.distributed group (gloo or nccl)."""
    import torch
    import torch.distributed as dist
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = torch.frombuffer(bytearray(make_id()), dtype=torch.uint8).clone()
    t = buf.to(device) if device is not None else buf
    dist.broadcast(t, 0)
    return bytes(t.cpu().numpy().tobytes())


def tp_init(device=None, peer: bool = True):
    """Join the tensor-parallel communicator of the torch.distributed group this process belongs to (after init(device)):
    rank 0 makes the NCCL id, torch.distributed carries it to the others.  peer: also open the ranks' peer buffers, so
    that the engines' all-reduces are the library's own one-shot kernel over peer memory instead of NCCL calls.
    Returns (rank, size)."""
    import torch.distributed as dist
    L = lib()
    rank, size = dist.get_rank(), dist.get_world_size()

    def make():
        b = C.create_string_buffer(128)
        check(L.llb_b200_tp_unique_id(None, b), "llb_b200_tp_unique_id")
        return b.raw
    uid = exchange_unique_id(make, rank, device)
    keep = C.create_string_buffer(uid, 128)
    check(L.llb_b200_tp_init(None, rank, size, keep), "llb_b200_tp_init")
    if peer and size > 1:
        import torch
        h = C.create_string_buffer(64)
        check(L.llb_b200_tp_peer_alloc(h), "llb_b200_tp_peer_alloc")
        mine = torch.frombuffer(bytearray(h.raw), dtype=torch.uint8).clone()
        if device is not None:
            mine = mine.to(device)
        every = [torch.zeros_like(mine) for _ in range(size)]
        dist.all_gather(every, mine)
        blob = b"".join(bytes(t.cpu().numpy().tobytes()) for t in every)
        check(L.llb_b200_tp_peer_open(C.create_string_buffer(blob, len(blob)), size), "llb_b200_tp_peer_open")
    return rank, size


def alloc(nbytes: int) -> int:
    p = lib().llb_b200_alloc_zero(nbytes)
    if not p:
        raise LlbError(f"llb_b200_alloc_zero({nbytes}) failed: {lib().llb_b200_last_error().decode()}")
    return p


def arr(ty, vals):
    return (ty * len(vals))(*vals)


def gemm(fmt: int, ws, rows, outs, K: int, xp, ksplit: int = 0):
    n = len(ws)
    check(lib().llb_b200_gemm(fmt, n, arr(C.c_uint64, ws), arr(C.c_int, rows), arr(C.c_uint64, outs), K, xp, ksplit),
          "llb_b200_gemm")


class SmpParams(C.Structure):
    """llb_smp_params (include/llb_b200.h): the reference's LlbSmpParams without the two fields the path does not use."""
    _fields_ = [("temp", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("top_k", C.c_int), ("repeat_penalty", C.c_float),
                ("repeat_last_n", C.c_int), ("presence", C.c_float), ("frequency", C.c_float), ("seed", C.c_uint64), ("min_keep", C.c_int),
                ("n_bias", C.c_int), ("bias_ids", C.c_int * 64), ("bias_vals", C.c_float * 64)]

    @classmethod
    def make(cls, temp=0.0, top_p=1.0, min_p=0.0, top_k=0, repeat_penalty=1.0, repeat_last_n=64, presence=0.0, frequency=0.0, seed=0,
             min_keep=0, bias=()):
        p = cls()
        p.temp, p.top_p, p.min_p, p.top_k = temp, top_p, min_p, top_k
        p.repeat_penalty, p.repeat_last_n, p.presence, p.frequency = repeat_penalty, repeat_last_n, presence, frequency
        p.seed, p.min_keep, p.n_bias = seed, min_keep, len(bias)
        for j, (t, v) in enumerate(bias):
            p.bias_ids[j], p.bias_vals[j] = t, v
        return p


def smp_rows(params: "SmpParams", logits_ptr: int, T: int, V: int, drafts, pos, windows):
    """The device sampler on T rows of logits on the device: (tokens, accepted, raw logit of each token)."""
    import numpy as np
    d = np.ascontiguousarray(drafts, dtype=np.int32)
    ps = np.ascontiguousarray(pos, dtype=np.int64)
    win = np.zeros((T, 256), np.int32)
    nwin = np.zeros(T, np.int32)
    for t, w in enumerate(windows):
        w = np.asarray(w, dtype=np.int32)[-256:]
        win[t, : len(w)] = w
        nwin[t] = len(w)
    tok, acc, val = np.zeros(T, np.int32), np.zeros(T, np.int32), np.zeros(T, np.float32)
    check(lib().llb_b200_smp_rows(C.byref(params), logits_ptr, T, V, d.ctypes.data, ps.ctypes.data, win.ctypes.data, nwin.ctypes.data,
                                  tok.ctypes.data, acc.ctypes.data, val.ctypes.data), "llb_b200_smp_rows")
    return tok, acc, val


class SpecEngine:
    """The speculative-decoding engine behind llb_spec_* (one sequence, greedy, MTP drafter).

    `pack` is a packs.Pack whose bytes live on the host (numpy / CPU tensor) or on the GPU (CUDA
    tensor); `mtp` the drafter image as bytes (host) or a CUDA uint8 tensor.
    """

    def __init__(self, pack, mtp=None, k: int = 3, max_ctx: int = 4096, layers: int = 0, tp: int = 1, streams: int = 1):
        import numpy as np
        import torch
        L = lib()
        self.L = L
        data = pack.data
        on_dev = bool(isinstance(data, torch.Tensor) and data.is_cuda)
        ptr = data.data_ptr() if isinstance(data, torch.Tensor) else data.ctypes.data
        nbytes = data.numel() if isinstance(data, torch.Tensor) else data.size
        if mtp is None:
            mptr, mbytes, mdev = None, 0, 0
        elif isinstance(mtp, (bytes, bytearray)):
            self._mtp_keep = np.frombuffer(mtp, dtype=np.uint8)
            mptr, mbytes, mdev = self._mtp_keep.ctypes.data, len(mtp), 0
        else:
            self._mtp_keep = mtp
            mptr, mbytes, mdev = mtp.data_ptr(), mtp.numel(), int(mtp.is_cuda)
        if streams > 1:
            assert tp == 1
            self.h = handle(L.llb_spec_open_streams(pack.index_text().encode(), ptr, nbytes, int(on_dev), mptr, mbytes, mdev, k,
                                                    max_ctx, layers, streams), "llb_spec_open_streams")
        else:
            self.h = handle(L.llb_spec_open_tp(pack.index_text().encode(), ptr, nbytes, int(on_dev), mptr, mbytes, mdev, k, max_ctx,
                                               layers, tp), "llb_spec_open")
        self.streams = streams
        self.k, self.vocab, self.d = k, pack.cfg.vocab_size, pack.cfg.d_model
        self.cfg = pack.cfg

    @classmethod
    def from_gguf(cls, path: str, cfg, mtp=None, k: int = 3, max_ctx: int = 4096, layers: int = 0):
        """The engine opened straight from a GGUF file (llb_spec_open_gguf); cfg only names vocabulary and widths
        for the Python-side helpers."""
        import numpy as np
        self = cls.__new__(cls)
        self.L = lib()
        if mtp is None:
            mptr, mbytes = None, 0
        else:
            self._mtp_keep = np.frombuffer(mtp, dtype=np.uint8)
            mptr, mbytes = self._mtp_keep.ctypes.data, len(mtp)
        self.h = handle(self.L.llb_spec_open_gguf(path.encode(), mptr, mbytes, 0, k, max_ctx, layers), "llb_spec_open_gguf")
        self.k, self.vocab, self.d, self.cfg = k, cfg.vocab_size, cfg.d_model, cfg
        return self

    def sibling(self, k: int = None, max_ctx: int = 4096, streams: int = None) -> "SpecEngine":
        """Another engine on this one's weights (llb_spec_open_sibling): its own k, context, streams and sequence state."""
        o = SpecEngine.__new__(SpecEngine)
        o.L = self.L
        o.k = self.k if k is None else k
        o.streams = getattr(self, "streams", 1) if streams is None else streams
        o.h = handle(self.L.llb_spec_open_sibling(self.h, o.k, max_ctx, o.streams), "llb_spec_open_sibling")
        o.vocab, o.d, o.cfg = self.vocab, self.d, self.cfg
        return o

    def weight_bytes(self) -> int:
        return int(self.L.llb_spec_weight_bytes(self.h))

    def close(self):
        if getattr(self, "h", None):
            self.L.llb_spec_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prefill(self, ids):
        import numpy as np
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        check(self.L.llb_spec_prefill(self.h, ids.ctypes.data, len(ids)), "llb_spec_prefill")

    def last_record(self, b: int = 0):
        import numpy as np
        o = np.zeros(51, np.uint32)
        check(self.L.llb_spec_last_record(self.h, b, o.ctypes.data), "llb_spec_last_record")
        T = int(o[1])
        return {"p0": int(o[0]), "T": T, "served": int(o[2]), "tin": [int(v) for v in o[3:3 + T].view(np.int32)],
                "ids": [int(v) for v in o[11:11 + T].view(np.int32)], "top2": o[19:19 + 4 * T].reshape(T, 4).copy()}

    def set_sampler(self, params: "SmpParams"):
        check(self.L.llb_spec_set_sampler(self.h, C.byref(params)), "llb_spec_set_sampler")

    def sampler_errors(self) -> int:
        return self.L.llb_spec_sampler_errors(self.h)

    def prefill_stream(self, b: int, ids):
        import numpy as np
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        check(self.L.llb_spec_prefill_stream(self.h, b, ids.ctypes.data, len(ids)), "llb_spec_prefill_stream")

    def prefill_streams(self, prompts, streams=None):
        """{stream: ids}, or a list of prompts for `streams` (default: stream i gets prompts[i]), through shared prompt passes."""
        import numpy as np
        items = sorted(prompts.items()) if isinstance(prompts, dict) else list(zip(streams if streams is not None else range(len(prompts)), prompts))
        arrs = [np.ascontiguousarray(p, dtype=np.int32) for _, p in items]
        n = len(items)
        bs = (C.c_int * n)(*[int(b) for b, _ in items])
        ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
        ns = (C.c_int * n)(*[len(a) for a in arrs])
        check(self.L.llb_spec_prefill_streams(self.h, n, bs, ptrs, ns), "llb_spec_prefill_streams")

    def cycle_streams(self):
        """One cycle of every stream with a prompt: [(ids, top2) per stream] (empty arrays for an idle stream)."""
        import numpy as np
        B = self.streams
        ids = np.zeros((B, 8), np.int32)
        n = np.zeros(B, np.int32)
        t2 = np.zeros((B, 8, 4), np.uint32)
        check(self.L.llb_spec_cycle_streams(self.h, ids.ctypes.data, n.ctypes.data, t2.ctypes.data), "llb_spec_cycle_streams")
        return [(ids[b, : n[b]].copy(), t2[b, : n[b]].copy()) for b in range(B)]

    def run_cycles_streams(self, n: int):
        import numpy as np
        tok = np.zeros(self.streams, np.int32)
        check(self.L.llb_spec_run_cycles_streams(self.h, n, tok.ctypes.data), "llb_spec_run_cycles_streams")
        return tok

    def stats_stream(self, b: int):
        import numpy as np
        out = np.zeros(19, np.uint64)
        check(self.L.llb_spec_stats_stream(self.h, b, out.ctypes.data), "llb_spec_stats_stream")
        return {"cycles": int(out[0]), "rows": int(out[1]), "served": int(out[2]),
                "drafted": [int(v) for v in out[3:11]], "accepted": [int(v) for v in out[11:19]]}

    def position_stream(self, b: int) -> int:
        return self.L.llb_spec_position_stream(self.h, b)

    def read_state_stream(self, b: int, what: int, il: int = 0, pos: int = 0):
        import numpy as np
        c = self.cfg
        n = max(c.ssm_heads * c.ssm_state * c.ssm_state, c.convd, c.d_model, c.n_kv_heads * c.head_dim)
        out = np.zeros(n, np.float32)
        got = check(self.L.llb_spec_read_state_stream(self.h, b, what, il, pos, out.ctypes.data, n), "llb_spec_read_state_stream")
        return out[:got].copy()

    def cycle(self):
        import numpy as np
        ids = np.zeros(8, np.int32)
        n = C.c_int(0)
        t2 = np.zeros((8, 4), np.uint32)
        check(self.L.llb_spec_cycle(self.h, ids.ctypes.data, C.addressof(n), t2.ctypes.data), "llb_spec_cycle")
        return ids[: n.value].copy(), t2[: n.value].copy()

    def generate(self, steps: int):
        import numpy as np
        ids = np.zeros(steps, np.int32)
        t2 = np.zeros((steps, 4), np.uint32)
        n = check(self.L.llb_spec_generate(self.h, steps, ids.ctypes.data, t2.ctypes.data), "llb_spec_generate")
        assert n == steps
        return ids, t2

    def stats(self):
        import numpy as np
        out = np.zeros(19, np.uint64)
        check(self.L.llb_spec_stats(self.h, out.ctypes.data), "llb_spec_stats")
        return {"cycles": int(out[0]), "rows": int(out[1]), "served": int(out[2]),
                "drafted": [int(v) for v in out[3:11]], "accepted": [int(v) for v in out[11:19]]}

    def set_prefill(self, fast: bool) -> int:
        """True: prompts go through the dense tcgen05 path in chunks of 128 rows; returns the previous mode."""
        return self.L.llb_spec_set_prefill(self.h, 1 if fast else 0)

    def fast_rows(self) -> float:
        return self.L.llb_spec_fast_rows(self.h)

    def position(self) -> int:
        return self.L.llb_spec_position(self.h)

    def run_cycles(self, n: int, cap: int = 4096):
        import numpy as np
        ids = np.zeros(cap, np.int32)
        got = check(self.L.llb_spec_run_cycles(self.h, n, ids.ctypes.data, cap), "llb_spec_run_cycles")
        return ids[: min(got, cap)].copy(), got

    def step(self, pos: int, tok: int):
        """The reference's per-token operator: (pos, tok) in, [v1, id1, v2, id2] out."""
        import numpy as np
        y = np.zeros(4, np.float32)
        check(self.L.llb_spec_pass(self.h, int(pos), int(tok), y.ctypes.data), "llb_spec_pass")
        return y

    def time_verify(self, iters: int) -> float:
        ms = C.c_float(0)
        check(self.L.llb_spec_time_verify(self.h, iters, C.addressof(ms)), "llb_spec_time_verify")
        return ms.value

    def time_verify_rows(self, iters: int, rows: int) -> float:
        ms = C.c_float(0)
        check(self.L.llb_spec_time_verify_rows(self.h, iters, rows, C.addressof(ms)), "llb_spec_time_verify_rows")
        return ms.value

    def time_gemm(self, iters: int):
        us, nb = C.c_float(0), C.c_double(0)
        check(self.L.llb_spec_time_gemm(self.h, iters, C.addressof(us), C.addressof(nb)), "llb_spec_time_gemm")
        return us.value, nb.value

    def profile_verify(self):
        """Per-op device time of one eager verify pass: {name: (count, total_us)}."""
        buf = C.create_string_buffer(1 << 16)
        check(self.L.llb_spec_profile_verify(self.h, buf, len(buf)), "llb_spec_profile_verify")
        out = {}
        for line in buf.value.decode().splitlines():
            n, c, t = line.split("\t")
            out[n] = (int(c), float(t))
        return out

    def graph_nodes(self, which: int = 0) -> int:
        return self.L.llb_spec_graph_nodes(self.h, which)

    def read_state(self, what: int, il: int = 0, pos: int = 0):
        import numpy as np
        c = self.cfg
        n = max(c.ssm_heads * c.ssm_state * c.ssm_state, c.convd, c.d_model, c.n_kv_heads * c.head_dim)
        out = np.zeros(n, np.float32)
        got = check(self.L.llb_spec_read_state(self.h, what, il, pos, out.ctypes.data, n), "llb_spec_read_state")
        return out[:got].copy()

    def read_logits(self, r: int):
        import numpy as np
        out = np.zeros(self.vocab, np.float32)
        check(self.L.llb_spec_read_logits(self.h, r, out.ctypes.data), "llb_spec_read_logits")
        return out

    def moe_ffn(self, il: int, h2):
        """Layer il's routed-expert FFN alone on normed rows h2[T][d]: (out[T][d], ids[T][k+1], wt[T][k+1])."""
        import numpy as np
        h2 = np.ascontiguousarray(h2, np.float32)
        T, d = h2.shape
        ns = self.cfg.n_experts_used + 1
        out = np.zeros((T, d), np.float32)
        ids = np.zeros((T, ns), np.int32)
        wt = np.zeros((T, ns), np.float32)
        check(self.L.llb_spec_moe_ffn(self.h, il, T, h2.ctypes.data, out.ctypes.data, ids.ctypes.data, wt.ctypes.data), "llb_spec_moe_ffn")
        return out, ids, wt


def gguf_index(path: str) -> str:
    """The index text the library derives from a GGUF header (no GPU needed)."""
    L = lib()
    n = L.llb_b200_gguf_index(path.encode(), None, 0)
    if n < 0:
        raise LlbError("llb_b200_gguf_index failed: " + L.llb_b200_last_error().decode())
    buf = C.create_string_buffer(n + 1)
    L.llb_b200_gguf_index(path.encode(), buf, n + 1)
    return buf.value.decode()
