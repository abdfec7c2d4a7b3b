"""The four ``torch.ops.loopfuse.*`` custom ops, with eager and fake implementations.

Schemas match the reference (loopfuse/torch_backend/__init__.py:4-63) so that user code written
against it runs unchanged:

* ``loopfuse::causal_mask(Tensor a) -> Tensor``
* ``loopfuse::sliding_mask(Tensor a, int window_size) -> Tensor``
* ``loopfuse::scan_max(Tensor a) -> (Tensor, Tensor)``
* ``loopfuse::paged_load(Tensor buffer, Tensor block_table) -> Tensor``

The eager implementations are what runs when a function is *not* compiled; under
``torch.compile(backend=loopfuse_backend)`` the ops only mark the mask kind / the paged gather in
the captured graph and the CUDA kernels implement them.

Two deliberate differences from the reference's eager code, both documented where they occur:

* ``causal_mask`` aligns the diagonal to the top-left corner for non-square scores instead of
  failing (the reference builds an ``[S_kv, S_kv]`` mask, loopfuse/torch_backend/__init__.py:6-8,
  which only broadcasts for square scores); square scores give identical results.
* ``sliding_mask`` keeps ``0 <= i - j < window`` - the mask the reference's *compiled* kernel
  applies (loopfuse/torch_backend/ops.py:733-741) and its benchmark checks against
  (tests/benchmark.py:236). The reference's eager op keeps ``j > i - window`` only, i.e. it also
  keeps future keys (loopfuse/torch_backend/__init__.py:21-22), so its eager and compiled results
  disagree; wherever a function also applies ``causal_mask`` the two readings coincide.

The namespace is the reference's, so the reference package and this one cannot be imported into
one process.
"""
from __future__ import annotations

import torch

_NEG_INF = float("-inf")


@torch.library.custom_op("loopfuse::causal_mask", mutates_args=())
def causal_mask(a: torch.Tensor) -> torch.Tensor:
    s_q, s_kv = a.shape[-2], a.shape[-1]
    rows = torch.arange(s_q, device=a.device)[:, None]
    cols = torch.arange(s_kv, device=a.device)[None, :]
    return a.masked_fill(cols > rows, _NEG_INF)


@torch.library.register_fake("loopfuse::causal_mask")
def _(a: torch.Tensor) -> torch.Tensor:
    return torch.empty_like(a)


@torch.library.custom_op("loopfuse::sliding_mask", mutates_args=())
def sliding_mask(a: torch.Tensor, window_size: int) -> torch.Tensor:
    s_q, s_kv = a.shape[-2], a.shape[-1]
    rows = torch.arange(s_q, device=a.device)[:, None]
    cols = torch.arange(s_kv, device=a.device)[None, :]
    keep = (cols <= rows) & (cols > rows - window_size)
    return a.masked_fill(~keep, _NEG_INF)


@torch.library.register_fake("loopfuse::sliding_mask")
def _(a: torch.Tensor, window_size: int) -> torch.Tensor:
    return torch.empty_like(a)


@torch.library.custom_op("loopfuse::scan_max", mutates_args=())
def scan_max(a: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    running = torch.cummax(a, dim=-1).values
    final = torch.max(a, dim=-1, keepdim=True).values
    return running, final


@torch.library.register_fake("loopfuse::scan_max")
def _(a: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return torch.empty_like(a), a.new_empty((*a.shape[:-1], 1))


@torch.library.custom_op("loopfuse::paged_load", mutates_args=())
def paged_load(buffer: torch.Tensor, block_table: torch.Tensor) -> torch.Tensor:
    """``out[*s, *t] = buffer[block_table[*s], *t]`` for ``buffer [N, *T]``, ``block_table [*S]``."""
    return buffer[block_table.long()]


@torch.library.register_fake("loopfuse::paged_load")
def _(buffer: torch.Tensor, block_table: torch.Tensor) -> torch.Tensor:
    return buffer.new_empty((*block_table.shape, *buffer.shape[1:]))
