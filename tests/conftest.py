import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    return graft.load_package()


@pytest.fixture(scope="session")
def packs(pkg):
    return pkg.packs


@pytest.fixture(scope="session")
def oracle():
    """The CPU restatement (oracle/q35_oracle.c), built on demand."""
    from oracle import bindings
    if not os.path.exists(bindings.PORT_SO):
        bindings.build_port()
    return bindings


@pytest.fixture(scope="session")
def llb(pkg):
    """The CUDA library, initialised on cuda:0.  Fails loudly when it is missing."""
    import torch
    assert torch.cuda.is_available(), "a test marked gpu ran without a GPU"
    pkg.llb.init(0)
    return pkg.llb


class DevBuf:
    """A device allocation of the library, freed with the test."""

    def __init__(self, llb, nbytes):
        self.llb, self.nbytes = llb, nbytes
        self.ptr = llb.alloc(nbytes)

    def write(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        self.llb.check(self.llb.lib().llb_b200_write(self.ptr, a.ctypes.data, a.nbytes), "llb_b200_write")
        return self

    def read(self, shape, dtype):
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        self.llb.check(self.llb.lib().llb_b200_read(out.ctypes.data, self.ptr, out.nbytes), "llb_b200_read")
        return out

    def free(self):
        if self.ptr:
            self.llb.lib().llb_b200_free(self.ptr)
            self.ptr = 0


@pytest.fixture()
def dev(llb):
    bufs = []

    def make(nbytes):
        b = DevBuf(llb, nbytes)
        bufs.append(b)
        return b

    yield make
    for b in bufs:
        b.free()
