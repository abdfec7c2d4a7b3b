"""Alias of the reference's backend module path (tests/benchmark.py:6 imports
``loopfuse.torch_backend.interface.loopfuse_backend``)."""
from loopfuse_b200.backend import loopfuse_backend, loopfuse_compiler

__all__ = ["loopfuse_backend", "loopfuse_compiler"]
