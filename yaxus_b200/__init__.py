"""yaxus_b200: attention over yaxus's paged, prefix-shared KV cache, hand-written for B200.

The product is `libyaxus_cuda.so` (C ABI, include/yaxus_cuda.h).  This package holds its
sources (csrc/), its build script and a thin Python mirror of the reference's backend
interface used by the tests and the benchmark.
"""
from ._lib import BF16, F16, F32, HEAD_DIM, PAGE  # noqa: F401
from .kvcache import KvCache, PassMeta, slot  # noqa: F401


def __getattr__(name):
    # CudaBackend needs torch; import it lazily so that the host-side pieces work without it.
    if name in ("CudaBackend", "LayerMeta", "Rope", "Kv", "BackendError"):
        from . import backend
        return getattr(backend, name)
    raise AttributeError(name)
