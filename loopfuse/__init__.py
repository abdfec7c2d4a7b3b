"""Import alias so that code written for the reference keeps working unchanged:
``from loopfuse import loopfuse_backend`` resolves to the sm_100a implementation in
``loopfuse_b200`` (reference: loopfuse/__init__.py:1-3)."""
from loopfuse_b200 import loopfuse_backend

__all__ = ["loopfuse_backend"]
