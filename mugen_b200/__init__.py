"""B200 (sm_100a) implementation of Mugen's MLA absorbed-attention decode path.

Only what that path needs: `csrc/` (CUDA kernels and the C ABI of include/mugen_mla.h),
`host/` (C++ bookkeeping shared with the library, and the C++23 wrapper), `capi` / `mla`
(ctypes binding and the Python mirror of the reference interface used by tests and bench.py),
`synth` (seeded synthetic inputs).  There is no CPU implementation in this package.
"""
from .capi import MlaError  # noqa: F401


def __getattr__(name):
    if name == "MlaContext":
        from .mla import MlaContext
        return MlaContext
    raise AttributeError(name)
