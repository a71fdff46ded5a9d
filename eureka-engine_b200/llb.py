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
SO_PATH = os.path.join(HERE, "libllb_b200.so")

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
            "llb_alloc_zero": (u64, [sz]), "llb_free": (i32, [u64]), "llb_zero": (i32, [u64, sz]),
            "llb_copy": (i32, [u64, u64, sz]), "llb_write": (i32, [u64, vp, sz]), "llb_read": (i32, [vp, u64, sz]),
            "llb_sync": (i32, []), "llb_stream": (u64, []),
            "llb_b200_weight_bytes": (sz, [i32, i32, i32]),
            "llb_b200_weight_upload": (i32, [i32, i32, i32, vp, i32, u64]),
            "llb_b200_dequant": (i32, [i32, i32, i32, u64, u64, i32, u64]),
            "llb_b200_xp_new": (vp, [i32, i32, i32]), "llb_b200_xp_free": (None, [vp]),
            "llb_b200_xp_set_f32": (i32, [vp, u64]), "llb_b200_xp_set_bf16": (i32, [vp, u64]),
            "llb_b200_gemm": (i32, [i32, i32, C.POINTER(u64), C.POINTER(i32), C.POINTER(u64), i32, vp, i32]),
            "llb_b200_gemm_host": (i32, [i32, u64, i32, i32, vp, i32, vp, vp, u64, u64]),
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


def alloc(nbytes: int) -> int:
    p = lib().llb_alloc_zero(nbytes)
    if not p:
        raise LlbError(f"llb_alloc_zero({nbytes}) failed: {lib().llb_b200_last_error().decode()}")
    return p


def arr(ty, vals):
    return (ty * len(vals))(*vals)


def gemm(fmt: int, ws, rows, outs, K: int, xp, ksplit: int = 0):
    n = len(ws)
    check(lib().llb_b200_gemm(fmt, n, arr(C.c_uint64, ws), arr(C.c_int, rows), arr(C.c_uint64, outs), K, xp, ksplit),
          "llb_b200_gemm")
