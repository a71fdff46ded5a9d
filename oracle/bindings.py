"""ctypes bindings of the two CPU checkers.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the
package smoke check and by the benchmark's CPU-baseline leg, never by the product path.

  Oracle   oracle/_build/libq35_oracle.so  this repository's C restatement (oracle/q35_oracle.c)
  RefTwin  oracle/_ref/libq35ref.so        the reference CPU engine built from its own sources
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "_build", "libq35_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libq35ref.so")
REF_CLI = os.path.join(HERE, "_ref", "qwen35_ref")
REF_SMP_SO = os.path.join(HERE, "_ref", "libllbsmp.so")

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float


def build_port() -> str:
    subprocess.run(["make", "-s", "-C", HERE, "port"], check=True)
    return PORT_SO


def build_ref(ref_root: str) -> str:
    subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={ref_root}"], check=True)
    return REF_SO


def _p(a: np.ndarray):
    return a.ctypes.data_as(_vp)


class Cfg(C.Structure):
    _fields_ = [(n, _i) for n in ("n_layers d_model n_heads n_kv_heads head_dim d_ff vocab interval conv_kernel "
                                  "ssm_state ssm_groups ssm_heads vhd kdc vdc convd rope_dim").split()] + \
               [("rope_base", _f), ("eps", _f)] + \
               [(n, _i) for n in "n_experts n_used d_expert d_shared".split()]


class SpecStats(C.Structure):
    _fields_ = [("cycles", C.c_uint64), ("rows", C.c_uint64), ("served", C.c_uint64),
                ("drafted", C.c_uint64 * 8), ("accepted", C.c_uint64 * 8)]


class SmpParams(C.Structure):
    """Sampler parameters, in the oracle's layout (oracle/q35_sampler.c: Q35Smp)."""
    _fields_ = [("temp", _f), ("top_p", _f), ("min_p", _f), ("top_k", _i), ("repeat_penalty", _f), ("repeat_last_n", _i),
                ("presence", _f), ("frequency", _f), ("seed", C.c_uint64), ("min_keep", _i), ("n_bias", _i),
                ("bias_ids", _i * 64), ("bias_vals", _f * 64)]

    @classmethod
    def make(cls, temp=0.0, top_p=1.0, min_p=0.0, top_k=0, repeat_penalty=1.0, repeat_last_n=64, presence=0.0, frequency=0.0,
             seed=0, min_keep=0, bias=()):
        p = cls()
        p.temp, p.top_p, p.min_p, p.top_k = temp, top_p, min_p, top_k
        p.repeat_penalty, p.repeat_last_n, p.presence, p.frequency = repeat_penalty, repeat_last_n, presence, frequency
        p.seed, p.min_keep, p.n_bias = seed, min_keep, len(bias)
        for j, (t, v) in enumerate(bias):
            p.bias_ids[j], p.bias_vals[j] = t, v
        return p


class RefSmpParams(C.Structure):
    """LlbSmpParams of the reference (host/llb_sampler.h:38-52), for oracle/_ref/libllbsmp.so."""
    _fields_ = [("temp", _f), ("top_p", _f), ("min_p", _f), ("top_k", _i), ("repeat_penalty", _f), ("repeat_last_n", _i),
                ("presence", _f), ("frequency", _f), ("seed", C.c_uint64), ("min_keep", _i), ("n_logprobs", _i), ("max_tokens", _i),
                ("n_bias", _i), ("bias_ids", _i * 64), ("bias_vals", _f * 64)]


def smp_row(params: SmpParams, logits: np.ndarray, hist, draft: int, pos: int):
    """The oracle's sampler on one row: (token, accepted, margin)."""
    L = Oracle.lib()
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    h = np.ascontiguousarray(hist if hist is not None else [], dtype=np.int32)
    acc, mg = _i(0), C.c_double(0)
    t = L.q35_smp_row(C.byref(params), _p(logits), len(logits), _p(h) if len(h) else None, len(h), draft, C.c_uint64(pos), C.byref(acc), C.byref(mg))
    return t, acc.value, mg.value


def ref_smp_row(params: SmpParams, logits: np.ndarray, hist, draft: int, pos: int):
    """The reference's own sampler (oracle/_ref/libllbsmp.so: llb_smp_new / _history / _verify / _sample) on one row."""
    L = C.CDLL(REF_SMP_SO)
    L.llb_smp_new.restype = _vp
    L.llb_smp_new.argtypes = [_vp, _i]
    L.llb_smp_free.argtypes = [_vp]
    L.llb_smp_history.argtypes = [_vp, _vp, _i]
    L.llb_smp_sample.argtypes = [_vp, _vp, C.c_uint64]
    L.llb_smp_verify.argtypes = [_vp, _vp, _i, _vp, C.c_uint64, _vp]
    rp = RefSmpParams()
    for n in ("temp", "top_p", "min_p", "top_k", "repeat_penalty", "repeat_last_n", "presence", "frequency", "seed", "min_keep", "n_bias"):
        setattr(rp, n, getattr(params, n))
    for j in range(params.n_bias):
        rp.bias_ids[j], rp.bias_vals[j] = params.bias_ids[j], params.bias_vals[j]
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    s = L.llb_smp_new(C.byref(rp), len(logits))
    try:
        if hist is not None and len(hist):
            h = np.ascontiguousarray(hist, dtype=np.int32)
            L.llb_smp_history(s, _p(h), len(h))
        acc = _i(0)
        if draft >= 0:
            t = L.llb_smp_verify(s, _p(logits), draft, None, C.c_uint64(pos), C.byref(acc))
        else:
            t = L.llb_smp_sample(s, _p(logits), C.c_uint64(pos))
    finally:
        L.llb_smp_free(s)
    return t, acc.value


class Oracle:
    """The C restatement.  Leaves are static; a model is an instance."""
    _lib = None

    @classmethod
    def lib(cls):
        if cls._lib is None:
            if not os.path.exists(PORT_SO):
                build_port()
            L = C.CDLL(PORT_SO)
            L.q35_half.restype = _f
            L.q35_half.argtypes = [C.c_uint16]
            L.q35_dot.restype = _f
            L.q35_dot.argtypes = [_i, _vp, _i, _vp]
            L.q35_deq_row.argtypes = [_i, _vp, _i, _vp]
            L.q35_gemv.argtypes = [_i, _vp, _i, _i, _i, _vp, _vp]
            for n in ("q35_silu", "q35_sigmoid", "q35_softplus", "q35_exp"):
                getattr(L, n).restype = _f
                getattr(L, n).argtypes = [_f]
            L.q35_rope.argtypes = [_vp, _i, _i, _f]
            L.q35_open_dir.restype = _vp
            L.q35_open_dir.argtypes = [C.c_char_p, _i, _i]
            L.q35_open_mem.restype = _vp
            L.q35_open_mem.argtypes = [C.c_char_p, _vp, C.c_size_t, _i, _i]
            L.q35_close.argtypes = [_vp]
            L.q35_cfg.argtypes = [_vp, C.POINTER(Cfg)]
            L.q35_reset.argtypes = [_vp]
            L.q35_forward.argtypes = [_vp, _i, _i]
            for n in ("q35_logits", "q35_residual", "q35_hnorm"):
                getattr(L, n).restype = C.POINTER(_f)
                getattr(L, n).argtypes = [_vp]
            for n in ("q35_state_S", "q35_state_conv"):
                getattr(L, n).restype = C.POINTER(_f)
                getattr(L, n).argtypes = [_vp, _i]
            for n in ("q35_state_k", "q35_state_v"):
                getattr(L, n).restype = C.POINTER(_f)
                getattr(L, n).argtypes = [_vp, _i, _i]
            L.q35_top2.argtypes = [_vp, _i, _vp, _vp]
            L.q35_greedy.restype = _i
            L.q35_greedy.argtypes = [_vp, _vp, _i, _i, _vp, _vp]
            L.q35_mtp_load.restype = _i
            L.q35_mtp_load.argtypes = [_vp, C.c_char_p, C.c_size_t]
            L.q35_spec_greedy.restype = _i
            L.q35_spec_greedy.argtypes = [_vp, _vp, _i, _i, _i, _vp, _vp, C.POINTER(SpecStats)]
            L.q35_spec_lookup.restype = _i
            L.q35_spec_lookup.argtypes = [_vp, _vp, _i, _i, _i, _vp, _vp, C.POINTER(SpecStats)]
            L.q35_lookup_draft.restype = _i
            L.q35_lookup_draft.argtypes = [_vp, _i, _i, _vp]
            L.q35_moe_ffn.restype = _i
            L.q35_moe_ffn.argtypes = [_vp, _i, _vp, _vp, _vp, _vp]
            L.q35_mtp_rows.restype = _i
            L.q35_mtp_rows.argtypes = [_vp, _i, _i, _vp, _vp, _vp]
            L.q35_threads.argtypes = [_i]
            L.q35_smp_row.restype = _i
            L.q35_smp_row.argtypes = [_vp, _vp, _i, _vp, _i, _i, C.c_uint64, _vp, _vp]
            cls._lib = L
        return cls._lib

    # ---- leaves -------------------------------------------------------------------------
    @classmethod
    def deq_rows(cls, fmt: int, raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, -1)
        out = np.empty((rows, cols), np.float32)
        for r in range(rows):
            cls.lib().q35_deq_row(fmt, _p(raw[r]), cols, _p(out[r]))
        return out

    @classmethod
    def gemv(cls, fmt: int, raw: np.ndarray, rows: int, cols: int, x: np.ndarray) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, -1)
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(rows, np.float32)
        cls.lib().q35_gemv(fmt, _p(raw), raw.shape[1], rows, cols, _p(x), _p(y))
        return y

    # ---- model --------------------------------------------------------------------------
    def __init__(self, index_text: str, pack: np.ndarray, cap: int, layers: int = 0):
        self.L = self.lib()
        self._pack = np.ascontiguousarray(pack, dtype=np.uint8)   # borrowed by the C side: keep alive
        self.h = self.L.q35_open_mem(index_text.encode(), _p(self._pack), self._pack.size, layers, cap)
        if not self.h:
            raise RuntimeError("q35_open_mem failed")
        self.cfg = Cfg()
        self.L.q35_cfg(self.h, C.byref(self.cfg))
        self.cap = cap

    def close(self):
        if self.h:
            self.L.q35_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        self.L.q35_reset(self.h)

    def moe_ffn(self, il: int, h2: np.ndarray):
        """The routed-expert FFN of layer il on one normed row: (out[d], ids[k], wts[k + 1])."""
        c = self.cfg
        h2 = np.ascontiguousarray(h2, np.float32)
        out = np.zeros(c.d_model, np.float32)
        ids = np.zeros(c.n_used, np.int32)
        wts = np.zeros(c.n_used + 1, np.float32)
        if self.L.q35_moe_ffn(self.h, int(il), _p(h2), _p(out), _p(ids), _p(wts)):
            raise RuntimeError("q35_moe_ffn: layer %d has no routed experts" % il)
        return out, ids, wts

    def forward(self, tok: int, pos: int):
        self.L.q35_forward(self.h, int(tok), int(pos))

    def _arr(self, ptr, n):
        return np.ctypeslib.as_array(ptr, shape=(n,)).copy()

    def logits(self) -> np.ndarray:
        return self._arr(self.L.q35_logits(self.h), self.cfg.vocab)

    def residual(self) -> np.ndarray:
        return self._arr(self.L.q35_residual(self.h), self.cfg.d_model)

    def hnorm(self) -> np.ndarray:
        return self._arr(self.L.q35_hnorm(self.h), self.cfg.d_model)

    def state_S(self, il: int) -> np.ndarray:
        c = self.cfg
        return self._arr(self.L.q35_state_S(self.h, il), c.ssm_heads * c.ssm_state * c.ssm_state)

    def state_conv(self, il: int) -> np.ndarray:
        c = self.cfg
        return self._arr(self.L.q35_state_conv(self.h, il), (c.conv_kernel - 1) * c.convd)

    def state_kv(self, il: int, pos: int):
        n = self.cfg.n_kv_heads * self.cfg.head_dim
        return self._arr(self.L.q35_state_k(self.h, il, pos), n), self._arr(self.L.q35_state_v(self.h, il, pos), n)

    def greedy(self, prompt, steps: int):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        ids = np.zeros(steps, np.int32)
        top2 = np.zeros((steps, 4), np.uint32)
        n = self.L.q35_greedy(self.h, _p(prompt), len(prompt), steps, _p(ids), _p(top2))
        if n != steps:
            raise RuntimeError(f"q35_greedy returned {n}")
        return ids, top2

    def mtp_load(self, img: bytes):
        rc = self.L.q35_mtp_load(self.h, img, len(img))
        if rc:
            raise RuntimeError(f"q35_mtp_load failed: {rc}")

    def mtp_rows(self, pa: int, toks, hs: np.ndarray):
        toks = np.ascontiguousarray(toks, dtype=np.int32)
        hs = np.ascontiguousarray(hs, dtype=np.float32).reshape(len(toks), -1)
        hn = np.zeros_like(hs)
        d = self.L.q35_mtp_rows(self.h, len(toks), pa, _p(toks), _p(hs), _p(hn))
        return d, hn

    def spec_greedy(self, prompt, steps: int, k: int):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        ids = np.zeros(steps, np.int32)
        top2 = np.zeros((steps, 4), np.uint32)
        st = SpecStats()
        n = self.L.q35_spec_greedy(self.h, _p(prompt), len(prompt), steps, k, _p(ids), _p(top2), C.byref(st))
        if n != steps:
            raise RuntimeError(f"q35_spec_greedy returned {n}")
        return ids, top2, st

    def spec_lookup(self, prompt, steps: int, k: int):
        """Greedy generation with the prompt-lookup drafter (no MTP head)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        ids = np.zeros(steps, np.int32)
        top2 = np.zeros((steps, 4), np.uint32)
        st = SpecStats()
        n = self.L.q35_spec_lookup(self.h, _p(prompt), len(prompt), steps, k, _p(ids), _p(top2), C.byref(st))
        if n != steps:
            raise RuntimeError(f"q35_spec_lookup returned {n}")
        return ids, top2, st


def lookup_draft(hist, pos: int, k: int):
    """Drafts of the prompt-lookup drafter for the history hist[0..pos]."""
    hist = np.ascontiguousarray(hist, dtype=np.int32)
    out = np.zeros(8, np.int32)
    n = Oracle.lib().q35_lookup_draft(_p(hist), pos, k, _p(out))
    return out[:n].copy()


class RefTwin:
    """The reference CPU engine (one model per process: it keeps its state in globals)."""

    def __init__(self, pack_dir: str, cap: int, layers: int = 0, pack: "np.ndarray | None" = None, threads: int = 0):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.L = L = C.CDLL(REF_SO)
        L.q35ref_open.argtypes = [C.c_char_p, _i, _i]
        for n in ("q35ref_logits", "q35ref_x", "q35ref_hnorm"):
            getattr(L, n).restype = C.POINTER(_f)
        for n in ("q35ref_state_S", "q35ref_state_conv"):
            getattr(L, n).restype = C.POINTER(_f)
            getattr(L, n).argtypes = [_i]
        for n in ("q35ref_state_k", "q35ref_state_v"):
            getattr(L, n).restype = C.POINTER(_f)
            getattr(L, n).argtypes = [_i, _i]
        L.q35ref_deq_row.argtypes = [_i, _vp, _i, _vp]
        L.q35ref_dot.restype = _f
        L.q35ref_dot.argtypes = [_i, _vp, _i, _vp]
        L.q35ref_gemv.argtypes = [_i, _vp, _i, _i, _i, _vp, _vp]
        L.q35ref_half.restype = _f
        L.q35ref_half.argtypes = [C.c_uint16]
        for n in ("q35ref_silu", "q35ref_sigmoid", "q35ref_softplus"):
            getattr(L, n).restype = _f
            getattr(L, n).argtypes = [_f]
        L.q35ref_open_mem.argtypes = [C.c_char_p, _vp, _i, _i]
        L.q35ref_threads(threads)
        if pack is not None:
            self._pack = np.ascontiguousarray(pack, dtype=np.uint8)
            rc = L.q35ref_open_mem(pack_dir.encode(), _p(self._pack), layers, cap)
        else:
            rc = L.q35ref_open(pack_dir.encode(), layers, cap)
        if rc:
            raise RuntimeError("q35ref_open failed")
        cfg = (C.c_int * 19)()
        L.q35ref_cfg(cfg)
        self.c = list(cfg)
        (self.n_layers, self.d_model, self.n_heads, self.n_kv, self.head_dim, self.d_ff, self.vocab, self.interval,
         self.kc, self.sz, self.gk, self.tr, self.vhd, self.kdc, self.vdc, self.convd, self.rope_dim) = self.c[:17]

    def forward(self, tok, pos):
        self.L.q35ref_forward(int(tok), int(pos))

    def logits(self):
        return np.ctypeslib.as_array(self.L.q35ref_logits(), shape=(self.vocab,)).copy()

    def top2(self):
        """ids, values of the top two logits of the last q35ref_logits call"""
        ids = (C.c_int * 2)()
        vals = (C.c_float * 2)()
        self.L.q35ref_top2(ids, vals)
        return [ids[0], ids[1]], [vals[0], vals[1]]

    def greedy(self, prompt, steps):
        """Plain greedy decoding as the reference CLI does it (tools/qwen35_engine.c:981-1007):
        ids[steps], top2[steps][4] = id1, bits1, id2, bits2."""
        ids = np.zeros(steps, np.int32)
        t2 = np.zeros((steps, 4), np.uint32)
        for t, tok in enumerate(prompt):
            self.forward(tok, t)
        for s in range(steps):
            self.logits()
            (i1, i2), (v1, v2) = self.top2()
            ids[s] = i1
            t2[s] = [i1, np.float32(v1).view(np.uint32), i2, np.float32(v2).view(np.uint32)]
            if s + 1 < steps:
                self.forward(i1, len(prompt) + s)
        return ids, t2

    def residual(self):
        return np.ctypeslib.as_array(self.L.q35ref_x(), shape=(self.d_model,)).copy()

    def hnorm(self):
        return np.ctypeslib.as_array(self.L.q35ref_hnorm(), shape=(self.d_model,)).copy()

    def state_S(self, il):
        return np.ctypeslib.as_array(self.L.q35ref_state_S(il), shape=(self.tr * self.sz * self.sz,)).copy()

    def state_conv(self, il):
        return np.ctypeslib.as_array(self.L.q35ref_state_conv(il), shape=((self.kc - 1) * self.convd,)).copy()

    def deq_rows(self, fmt, raw, rows, cols):
        raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, -1)
        out = np.empty((rows, cols), np.float32)
        for r in range(rows):
            self.L.q35ref_deq_row(fmt, _p(raw[r]), cols, _p(out[r]))
        return out

    def gemv(self, fmt, raw, rows, cols, x):
        raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, -1)
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(rows, np.float32)
        self.L.q35ref_gemv(fmt, _p(raw), raw.shape[1], rows, cols, _p(x), _p(y))
        return y
