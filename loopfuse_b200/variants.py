"""The benchmark's attention variants as a user writes them for ``torch.compile``, their seeded
synthetic inputs, and the algorithmic FLOP / byte counts used to report throughput.

The functions follow the reference's benchmark (tests/benchmark.py:79-83 causal, :142-147
softcap, :221-230 sliding window + GQA + softcap, :481-484 decode, :438-443 + :421-426 paged GQA
decode with the ``[B, Hkv, g, D]`` query convention). Shapes and parameters are those of the
five benchmark configurations; the data is synthetic (seeded N(0,1)), no dataset is involved.
"""
from __future__ import annotations

import dataclasses
from typing import Callable

import torch

from . import ops as _ops  # noqa: F401


def causal_attention(q, k, v):
    qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
    masked = torch.ops.loopfuse.causal_mask(qk)
    return torch.softmax(masked, dim=-1) @ v


def make_softcap_causal_attention(softcap: float) -> Callable:
    def softcap_causal_attention(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        qk = torch.tanh(qk / softcap) * softcap
        masked = torch.ops.loopfuse.causal_mask(qk)
        return torch.softmax(masked, dim=-1) @ v
    return softcap_causal_attention


def make_window_gqa_softcap_attention(softcap: float, window: int) -> Callable:
    def window_gqa_softcap_attention(q, k, v):
        hq, hk = q.shape[1], k.shape[1]
        k = k.repeat_interleave(hq // hk, dim=1)
        v = v.repeat_interleave(hq // hk, dim=1)
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        qk = torch.tanh(qk / softcap) * softcap
        # causal_mask(sliding_mask(.)) keeps i - window < j <= i under either reading of
        # sliding_mask (see ops.py).
        masked = torch.ops.loopfuse.causal_mask(torch.ops.loopfuse.sliding_mask(qk, window))
        return torch.softmax(masked, dim=-1) @ v
    return window_gqa_softcap_attention


def decode_attention(q, k, v):
    qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
    return torch.softmax(qk, dim=-1) @ v


def paged_gqa_decode_attention(q, k_pool, v_pool, block_table):
    """q is [B, Hkv, g, D]; pools are [pages, page_size, Hkv, D]; block_table [B, blocks]."""
    b = q.shape[0]
    k = torch.ops.loopfuse.paged_load(k_pool, block_table)
    v = torch.ops.loopfuse.paged_load(v_pool, block_table)
    k = k.reshape(b, -1, k.shape[-2], k.shape[-1]).transpose(1, 2)
    v = v.reshape(b, -1, v.shape[-2], v.shape[-1]).transpose(1, 2)
    qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
    return torch.softmax(qk, dim=-1) @ v


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    kind: str           # "prefill" | "decode" | "paged_decode"
    B: int
    Hq: int
    Hkv: int
    S: int              # query length for prefill, KV length for decode
    D: int
    softcap: float = 0.0
    window: int = 0
    page_size: int = 0
    pages_per_seq: int = 0

    @property
    def group(self) -> int:
        return self.Hq // self.Hkv

    def fn(self) -> Callable:
        if self.kind == "prefill":
            if self.window:
                return make_window_gqa_softcap_attention(self.softcap, self.window)
            if self.softcap:
                return make_softcap_causal_attention(self.softcap)
            return causal_attention
        if self.kind == "decode":
            return decode_attention
        return paged_gqa_decode_attention

    # -- work accounting (reference formulas: tests/benchmark.py:110,186 causal,
    #    :280-284 sliding window, :369,452,501 decode bytes) ---------------------------
    def flops(self, batch: int | None = None) -> int:
        b = self.B if batch is None else batch
        if self.kind != "prefill":
            return 4 * b * self.Hq * self.S * self.D
        if self.window:
            return 2 * b * self.Hq * (2 * self.S * self.window - self.window ** 2) * self.D
        return 2 * b * self.Hq * self.S ** 2 * self.D

    def kv_bytes(self, batch: int | None = None) -> int:
        b = self.B if batch is None else batch
        return 2 * 2 * b * self.Hkv * self.S * self.D

    def io_bytes(self, batch: int | None = None) -> int:
        """Minimum HBM traffic of a prefill launch: Q, K, V read once, O written once."""
        b = self.B if batch is None else batch
        return 2 * b * self.S * self.D * (2 * self.Hq + 2 * self.Hkv)

    def with_batch(self, batch: int) -> "Workload":
        return dataclasses.replace(self, B=batch)


WORKLOADS = {
    "causal_tiny": Workload("causal_tiny", "prefill", 2, 4, 4, 512, 64),
    "causal_softcap": Workload("causal_softcap", "prefill", 8, 32, 32, 2048, 128, softcap=50.0),
    "window_gqa_softcap": Workload("window_gqa_softcap", "prefill", 8, 32, 8, 2048, 128,
                                   softcap=50.0, window=256),
    "decode": Workload("decode", "decode", 64, 32, 32, 2048, 128),
    "paged_decode_gqa": Workload("paged_decode_gqa", "paged_decode", 64, 32, 8, 2048, 128,
                                 page_size=16, pages_per_seq=128),
}


def make_inputs(w: Workload, seed: int = 0, device="cpu", dtype=torch.bfloat16,
                batch_offset: int = 0, batch: int | None = None) -> tuple:
    """Seeded inputs for a workload, as the tuple its function takes.

    Values are drawn in fp32 on the CPU from ``torch.Generator(seed + 1000 * b)`` per batch
    element b (so a shard of the batch sees exactly the rows the full run sees), rounded to
    ``dtype`` and moved to ``device``.
    """
    nb = w.B if batch is None else batch
    qs, ks, vs, tables = [], [], [], []
    for b in range(batch_offset, batch_offset + nb):
        g = torch.Generator().manual_seed(seed + 1000 * b)
        if w.kind == "prefill":
            qs.append(torch.randn(w.Hq, w.S, w.D, generator=g))
            ks.append(torch.randn(w.Hkv, w.S, w.D, generator=g))
            vs.append(torch.randn(w.Hkv, w.S, w.D, generator=g))
        elif w.kind == "decode":
            qs.append(torch.randn(w.Hq, 1, w.D, generator=g))
            ks.append(torch.randn(w.Hkv, w.S, w.D, generator=g))
            vs.append(torch.randn(w.Hkv, w.S, w.D, generator=g))
        else:
            # Each sequence owns pages_per_seq physical pages of the pool; the block table is
            # a seeded permutation of the pool's page ids (of this shard's pool).
            qs.append(torch.randn(w.Hkv, w.group, w.D, generator=g))
            ks.append(torch.randn(w.pages_per_seq, w.page_size, w.Hkv, w.D, generator=g))
            vs.append(torch.randn(w.pages_per_seq, w.page_size, w.Hkv, w.D, generator=g))
    q = torch.stack(qs).to(dtype).to(device)
    if w.kind == "paged_decode":
        k_pool = torch.cat(ks).to(dtype).to(device)
        v_pool = torch.cat(vs).to(dtype).to(device)
        g = torch.Generator().manual_seed(seed + 7 + 1000 * batch_offset)
        table = torch.randperm(nb * w.pages_per_seq, generator=g).view(nb, w.pages_per_seq)
        return q, k_pool, v_pool, table.to(torch.int32).to(device)
    k = torch.stack(ks).to(dtype).to(device)
    v = torch.stack(vs).to(dtype).to(device)
    return q, k, v
