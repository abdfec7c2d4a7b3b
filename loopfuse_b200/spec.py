"""What the analysis layer hands to the kernel binder: an ``AttentionSpec`` per captured graph.

The reference compiler lowers a graph to loop IR, fuses it and prints Triton
(loopfuse/optimize.py:34-60, loopfuse/codegen.py:100-126). Here the same information - score-mod
chain, mask kind, GQA mapping, paged gather, block-skip ranges - is kept as a small declarative
record that selects and parameterises one of the hand-written CUDA kernels.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional

# Mask kinds and score-mod opcodes: numeric values are the C ABI's (include/lf_sm100.h).
MASK_NONE = 0
MASK_CAUSAL = 1
MASK_CAUSAL_WINDOW = 2

MOD_MUL = 1
MOD_ADD = 2
MOD_TANH = 3
MOD_EXP = 4
MOD_EXP2 = 5
MOD_SIN = 6
MOD_COS = 7
MOD_RELU = 8
MOD_SQUARE = 9
MOD_DIV = 10
MAX_MODS = 8

MOD_NAMES = {
    MOD_MUL: "mul", MOD_ADD: "add", MOD_TANH: "tanh", MOD_EXP: "exp", MOD_EXP2: "exp2",
    MOD_SIN: "sin", MOD_COS: "cos", MOD_RELU: "relu", MOD_SQUARE: "square", MOD_DIV: "div",
}

TILE_Q = 128
TILE_K = 64


@dataclasses.dataclass(frozen=True)
class ScalarExpr:
    """A scalar that is only known at call time (e.g. ``Q.shape[-1] ** -0.5`` with a dynamic
    head dim): ``node`` is the FX node to evaluate from the call's integer arguments."""
    node: Any

    def __repr__(self) -> str:  # keep spec dumps short
        return f"ScalarExpr({getattr(self.node, 'name', self.node)})"


@dataclasses.dataclass(frozen=True)
class ScoreMod:
    op: int
    arg: Any = 0.0  # float, or ScalarExpr resolved per call

    def __repr__(self) -> str:
        name = MOD_NAMES.get(self.op, str(self.op))
        return f"{name}({self.arg})" if self.op in (MOD_MUL, MOD_ADD, MOD_DIV) else name


@dataclasses.dataclass(frozen=True)
class KVSource:
    """Where a K or V operand comes from: a dense ``[B, Hkv, S, D]`` graph input, or a paged
    gather ``paged_load(cache, block_table)`` of a ``[n_pages, (page_size,) Hkv, D]`` pool."""
    placeholder: int                 # flat argument index of the tensor (dense) or of the pool
    block_table: Optional[int] = None  # flat argument index of the block table when paged
    repeated: bool = False           # went through repeat_interleave (GQA expansion)

    @property
    def paged(self) -> bool:
        return self.block_table is not None


@dataclasses.dataclass(frozen=True)
class AttentionSpec:
    q: int                    # flat argument index of Q
    k: KVSource
    v: KVSource
    mods: tuple               # tuple[ScoreMod, ...] applied to q.k before the mask, in order
    mask_kind: int = MASK_NONE
    windows: tuple = ()       # window of every sliding_mask met (int or ScalarExpr); min applies
    n_args: int = 0           # number of flat arguments of the compiled callable
    # Additive tensors of the reference's modified attention (tests/test_accuracy.py:176-194):
    q_bias: Optional[int] = None      # flat argument index of a [B,Hq,Sq,D] tensor added to Q
    out_bias: Optional[int] = None    # ... added to the output
    score_bias: Optional[int] = None  # ... of a [B,Hq,Sq,Skv] tensor added to the scores
    bias_pos: int = 0                 # the score bias is added after this many ops of ``mods``
    # Second score product of the MLA-style graph (tests/test_attention.py:126-151):
    # scores = Q K^T + Q_pe K_pe^T; flat argument indices of Q_pe and K_pe
    q_pe: Optional[int] = None
    k_pe: Optional[int] = None

    @property
    def window(self) -> int:
        """Effective window when every window is a compile-time constant (else 0)."""
        if self.windows and all(isinstance(w, int) for w in self.windows):
            return min(self.windows)
        return 0

    def describe(self) -> str:
        mask = {MASK_NONE: "none", MASK_CAUSAL: "causal",
                MASK_CAUSAL_WINDOW: f"causal_window({list(self.windows)})"}[self.mask_kind]
        bias = "".join(f", {n}=arg{i}" for n, i in (("q_bias", self.q_bias),
                                                    ("score_bias", self.score_bias),
                                                    ("out_bias", self.out_bias)) if i is not None)
        if self.score_bias is not None:
            bias += f"@{self.bias_pos}"
        return (f"AttentionSpec(q=arg{self.q}, k={self.k}, v={self.v}, "
                f"mods={list(self.mods)}, mask={mask}{bias})")


def skip_range(mask_kind: int, window: int, causal_offset: int, s_q: int, s_kv: int,
               tile_q: int, tile_k: int, iq: int) -> tuple[int, int]:
    """KV-tile range ``[lo, hi)`` that q-tile ``iq`` visits; integer-for-integer the same
    arithmetic as ``lf::skip_range`` in csrc/lf_skip_range.h (and ``lf_skip_range`` in the C
    ABI). Replaces the reference's symbolic derivation
    (loopfuse/compiler/passes/skip_loop_iterations.py:287-378)."""
    n_kt = -(-s_kv // tile_k)
    row_first = iq * tile_q
    row_last = min(row_first + tile_q - 1, s_q - 1)
    if row_first > row_last:
        return 0, 0
    lo, hi = 0, n_kt
    if mask_kind in (MASK_CAUSAL, MASK_CAUSAL_WINDOW):
        last_col = row_last + causal_offset
        hi = 0 if last_col < 0 else min(hi, last_col // tile_k + 1)
    if mask_kind == MASK_CAUSAL_WINDOW:
        first_col = row_first + causal_offset - (window - 1)
        if first_col > 0:
            lo = max(lo, first_col // tile_k)
    if hi <= lo:
        return 0, 0
    return lo, hi


def skip_table(mask_kind: int, window: int, causal_offset: int, s_q: int, s_kv: int,
               tile_q: int = TILE_Q, tile_k: int = TILE_K) -> list[tuple[int, int]]:
    n_qt = -(-s_q // tile_q)
    return [skip_range(mask_kind, window, causal_offset, s_q, s_kv, tile_q, tile_k, iq)
            for iq in range(n_qt)]
