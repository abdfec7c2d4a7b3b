"""Multi-GPU layout of the attention path: independent (batch x kv-head) units, one process per
GPU, no collective inside the data path, a single all-gather of the output slabs at the end.

The reference is single-GPU (no communication layer at all), so nothing here replaces reference
code; the partition follows from the kernels' unit of work: every (batch, kv head) pair - with
the g query heads that share the kv head - is computed independently.

* ``unit_range`` gives rank r a contiguous range of the flattened (b, kv-head) units.
* ``shard_units`` re-views Q/K/V so that a rank's units look like a batch of single-kv-head
  problems ([n_local, g, S, D] queries, [n_local, 1, S, D] keys/values): the same kernels run
  unchanged, and the rank's output rows are contiguous in the full [B, Hq, S, D] output.
* ``gather_output`` is the one collective: ``all_gather_into_tensor`` of equal-sized slabs
  (NCCL over NVLink/NVSwitch on GPUs, gloo on CPU for the tests).
* Paged caches shard by sequence instead (``batch_range``): a page holds all kv heads of 16
  tokens, so whole pages stay with the rank that owns the sequence.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def unit_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, equal-sized ranges (n_units must divide evenly, so that the final gather is
    a plain all_gather_into_tensor)."""
    if n_units % world:
        raise ValueError(f"{n_units} (batch x kv-head) units do not divide over {world} ranks")
    per = n_units // world
    return rank * per, (rank + 1) * per


def batch_range(batch: int, rank: int, world: int) -> tuple[int, int]:
    return unit_range(batch, rank, world)


def shard_units(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int):
    """Rank-local views of contiguous q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D].

    Returns (q_loc [n, g, Sq, D], k_loc [n, 1, Skv, D], v_loc [n, 1, Skv, D]) - no copies.
    """
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    u0, u1 = unit_range(B * Hkv, rank, world)
    q_units = q.contiguous().view(B * Hkv, g, Sq, D)
    k_units = k.contiguous().view(B * Hkv, 1, Skv, D)
    v_units = v.contiguous().view(B * Hkv, 1, Skv, D)
    return q_units[u0:u1], k_units[u0:u1], v_units[u0:u1]


def gather_output(local_out: torch.Tensor, full_shape: tuple,
                  group: Optional[dist.ProcessGroup] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The single collective of the path: concatenate every rank's contiguous output slab.

    ``local_out`` is this rank's [n_local, g, Sq, D] (or any contiguous slab of the output);
    the result has ``full_shape`` (e.g. [B, Hq, Sq, D]) on every rank.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    local_out = local_out.contiguous()
    if out is None:
        out = torch.empty(full_shape, dtype=local_out.dtype, device=local_out.device)
    if out.numel() != local_out.numel() * world:
        raise ValueError("slabs must have equal size on every rank")
    if world == 1:
        out.view(-1).copy_(local_out.view(-1))
        return out
    dist.all_gather_into_tensor(out.view(-1), local_out.view(-1), group=group)
    return out
