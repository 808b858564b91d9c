"""mechta_b200: the KV-cache / attention hot path of ssomenzi/mechta on B200 (sm_100a).

The product is libmechta_kv.so (CUDA kernels behind the C ABI of include/mechta_kv.h); this package is the
host-side mirror of the reference's operator interface for that path plus the multi-GPU plumbing.
"""
from . import _lib
from ._lib import MkvError

__all__ = ["_lib", "MkvError"]
