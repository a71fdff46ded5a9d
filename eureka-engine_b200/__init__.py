"""B200-native speculative-decoding path for the eureka-engine Qwen3.5 hybrid model.

  csrc/    CUDA kernels (sm_100a) and the C ABI of include/llb_b200.h -> libllb_b200.so
  llb.py   ctypes binding of that ABI
  packs.py synthetic weight packs in the reference's on-disk formats

The directory name is not a Python identifier; load it with `__graft_entry__.load_package()`.
"""
from . import dp, llb, packs  # noqa: F401
