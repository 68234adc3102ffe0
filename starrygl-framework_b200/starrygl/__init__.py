"""Drop-in replacement of the reference's per-mini-batch data path (``starrygl.graph``, ``starrygl.cache``,
``starrygl.route``) backed by libsgl_b200.so -- hand-written sm_100a CUDA kernels behind a C ABI.

Module paths, class names and call signatures follow the reference package so that existing callers keep
working; everything that moves data runs in the CUDA library (there is no CPU or PyTorch fallback).
"""
from .utils.context import DistributedContext  # noqa: F401  (same re-export as the reference's utils/__init__.py)

__all__ = ["DistributedContext"]
