"""loopfuse_b200: B200-native (sm_100a) implementation of loopfuse's fused-attention hot path.

``loopfuse_backend`` is the ``torch.compile`` backend; importing the package registers the
``torch.ops.loopfuse.*`` custom ops. The kernels live in ``liblf_sm100.so`` (C ABI, see
``include/lf_sm100.h``), built in-tree by ``python -m loopfuse_b200.build``.
"""
from . import ops  # noqa: F401  registers torch.ops.loopfuse.{causal_mask,sliding_mask,scan_max,paged_load}
from .backend import AttentionPlan, loopfuse_backend
from .spec import AttentionSpec, skip_range, skip_table

__all__ = ["loopfuse_backend", "AttentionPlan", "AttentionSpec", "skip_range", "skip_table"]
