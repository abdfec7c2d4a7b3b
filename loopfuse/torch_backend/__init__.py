"""Alias of the reference's op-registration module (loopfuse/torch_backend/__init__.py:4-63):
importing it registers ``torch.ops.loopfuse.*`` through ``loopfuse_b200.ops``."""
from loopfuse_b200.ops import causal_mask, paged_load, scan_max, sliding_mask

__all__ = ["causal_mask", "sliding_mask", "scan_max", "paged_load"]
