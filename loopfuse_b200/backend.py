"""``loopfuse_backend``: the ``torch.compile`` backend, drop-in for the reference's.

Same entry point and call convention as loopfuse/torch_backend/interface.py:77-86:
``torch.compile(fn, backend=loopfuse_backend, dynamic=True[, mode=...])``. The dynamo graph goes
through ``aot_module_simplified``; the forward compiler analyses the aten graph
(``capture.analyse_graph``) and returns a callable that binds the call's tensors to one of the
sm_100a kernels - where the reference printed and launched a Triton kernel
(loopfuse/codegen.py:100-126, interface.py:624-644).

Environment flags (reference: interface.py:23-29):
  ``CODEGEN_ONLY=1``  analysis only - the compiled callable returns the ``AttentionPlan`` instead
                      of launching (works on hosts without a GPU);
  ``DEBUG=1``         print the spec, the chosen kernel and the skip table at compile/call time.
One flag of this package's own:
  ``LF_CHECK_STATUS=1``  (also implied by ``DEBUG=1``) pass a device status word to every launch
                      and read it back after the call (a synchronisation): a bounded device-side
                      wait that ran out, or a block-table entry outside the pool, raises instead
                      of returning a plausible tensor. Without the flag the word is not read.
"""
from __future__ import annotations

import dataclasses
import os
from functools import partial
from typing import Any, Callable, Optional

import torch
from torch._functorch.aot_autograd import aot_module_simplified

from . import functional as F
from .capture import analyse_graph, evaluate_scalar
from .spec import (AttentionSpec, MASK_CAUSAL, MASK_CAUSAL_WINDOW, MASK_NONE, MOD_MUL, ScalarExpr,
                   ScoreMod, TILE_K, TILE_Q, skip_table)


def _flag(name: str) -> bool:
    return os.environ.get(name, "0") == "1"


_DECODE_GROUPS = (1, 2, 4, 8)


@dataclasses.dataclass
class AttentionPlan:
    """A spec bound to concrete sizes: which kernel runs, with which parameters."""
    spec: AttentionSpec
    kernel: str                 # "prefill" | "paged_prefill" | "decode" | "paged_decode"
    B: int
    Hq: int
    Hkv: int
    Sq: int
    Skv: int
    D: int
    scale: float
    mods: tuple
    window: int = 0
    page_size: int = 0
    mask_kind: int = MASK_NONE

    @property
    def skip_ranges(self) -> Optional[list]:
        """Per q-tile (lo, hi) in KV tiles of TILE_K (prefill kernels only); built on demand -
        the kernels derive the same integers themselves."""
        if self.kernel in ("decode", "paged_decode"):
            return None
        return skip_table(self.mask_kind, self.window, 0, self.Sq, self.Skv)

    def describe(self) -> str:
        s = (f"{self.kernel}: B={self.B} Hq={self.Hq} Hkv={self.Hkv} Sq={self.Sq} "
             f"Skv={self.Skv} D={self.D} scale={self.scale:.6g} mods={list(self.mods)}")
        if self.window:
            s += f" window={self.window}"
        if self.page_size:
            s += f" page_size={self.page_size}"
        if self.skip_ranges is not None:
            s += f" skip_ranges[{TILE_Q}x{TILE_K}]={self.skip_ranges}"
        return s


class CompiledAttention:
    """The callable handed back to AOT autograd for one captured graph."""

    def __init__(self, gm: torch.fx.GraphModule, spec: AttentionSpec, mode: Optional[str]):
        self.spec = spec
        self.mode = mode
        self.placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
        self.workspace = F.DecodeWorkspace()
        self.analysis_only = _flag("CODEGEN_ONLY")
        self.debug = _flag("DEBUG")
        self.check_status = self.debug or _flag("LF_CHECK_STATUS")
        self._plans: dict = {}
        self._prepared: dict = {}
        self._status: dict = {}

    # -- binding -------------------------------------------------------------------------
    def _resolve_mods(self, flat_args: list) -> tuple[float, tuple]:
        mods = []
        for m in self.spec.mods:
            arg = m.arg
            if isinstance(arg, ScalarExpr):
                arg = evaluate_scalar(arg, self.placeholders, flat_args)
            mods.append(ScoreMod(m.op, arg))
        scale = 1.0
        bias_first = self.spec.score_bias is not None and self.spec.bias_pos == 0
        if mods and mods[0].op == MOD_MUL and not bias_first:   # the usual `* D ** -0.5`
            scale = mods[0].arg
            mods = mods[1:]
        return scale, tuple(mods)

    def _bias_pos(self, plan: "AttentionPlan") -> int:
        """Position of the score bias in ``plan.mods`` (one less than in the captured chain when
        its leading multiplier became the kernel's ``scale``)."""
        return self.spec.bias_pos - (len(self.spec.mods) - len(plan.mods))

    def plan(self, flat_args: list) -> AttentionPlan:
        """The plan for this call's sizes; cached per (shapes, integer arguments)."""
        key = tuple(a.shape if isinstance(a, torch.Tensor) else a for a in flat_args)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._make_plan(flat_args)
            if len(self._plans) >= 64:
                self._plans.clear()
            self._plans[key] = plan
        return plan

    def _make_plan(self, flat_args: list) -> AttentionPlan:
        spec = self.spec
        q = flat_args[spec.q]
        if q.dim() != 4:
            raise ValueError("Q must be [B, H, S, D]")
        B, Hq, Sq, D = q.shape
        if spec.k.paged:
            pool = flat_args[spec.k.placeholder]
            table = flat_args[spec.k.block_table]
            page_size = pool.shape[1] if pool.dim() == 4 else 1
            Hkv = pool.shape[-2]
            Skv = table.shape[1] * page_size
        else:
            k = flat_args[spec.k.placeholder]
            page_size = 0
            Hkv, Skv = k.shape[1], k.shape[2]
        if spec.v.paged and not spec.k.paged:
            vpool = flat_args[spec.v.placeholder]
            page_size = vpool.shape[1] if vpool.dim() == 4 else 1
        if spec.k.repeated:
            if Hq % Hkv:
                raise ValueError(f"repeat_interleave: Hq={Hq} is not a multiple of Hkv={Hkv}")
        elif Hq != Hkv:
            raise ValueError(f"Q has {Hq} heads but K has {Hkv}; use repeat_interleave for GQA")
        scale, mods = self._resolve_mods(flat_args)
        window = 0
        if spec.mask_kind == MASK_CAUSAL_WINDOW:
            window = min(int(evaluate_scalar(w, self.placeholders, flat_args))
                         if isinstance(w, ScalarExpr) else w for w in spec.windows)
            if window <= 0:
                raise ValueError("sliding_mask window must be positive")

        group = Hq // Hkv
        decode_rows = Sq * group
        both_paged = spec.k.paged and spec.v.paged
        is_decode = (spec.mask_kind == MASK_NONE and decode_rows in _DECODE_GROUPS
                     and (Sq == 1 or group == 1) and (both_paged or not
                                                      (spec.k.paged or spec.v.paged)))
        if (spec.q_bias is not None or spec.out_bias is not None or spec.score_bias is not None
                or spec.q_pe is not None):
            is_decode = False   # bias tensors / a second score product: prefill kernel only
        if is_decode:
            kernel = "paged_decode" if both_paged else "decode"
        else:
            kernel = "paged_prefill" if (spec.k.paged or spec.v.paged) else "prefill"
        return AttentionPlan(spec, kernel, B, Hq, Hkv, Sq, Skv, D, scale, mods, window, page_size,
                             spec.mask_kind)

    # -- launch --------------------------------------------------------------------------
    def _status_for(self, device) -> Optional[torch.Tensor]:
        if not self.check_status:
            return None
        st = self._status.get(device)
        if st is None:
            st = self._status[device] = F.new_status(device)
        return st

    def _prepared_prefill(self, plan: AttentionPlan, q, k, v, status) -> "F.PreparedPrefill":
        """Prefill launches bound to (buffers, plan): a loop that calls the compiled function on
        the same buffers pays the argument marshalling once."""
        key = (q.data_ptr(), k.data_ptr(), v.data_ptr(), q.shape, k.shape, q.stride(),
               k.stride(), v.stride(), id(plan))
        prep = self._prepared.get(key)
        if prep is None:
            if len(self._prepared) >= 16:
                self._prepared.clear()
            prep = F.PreparedPrefill(q, k, v, scale=plan.scale, mods=plan.mods,
                                     mask_kind=plan.mask_kind, window=plan.window,
                                     status=status)
            self._prepared[key] = prep
        return prep

    def __call__(self, *flat_args: Any):
        args = list(flat_args)
        plan = self.plan(args)
        if self.debug:
            print(f"[loopfuse_b200] {self.spec.describe()}\n[loopfuse_b200] {plan.describe()}")
        if self.analysis_only:
            return (plan,)
        spec = self.spec
        q = args[spec.q]
        status = self._status_for(q.device)
        if plan.kernel in ("decode", "paged_decode"):
            # G query rows per kv head: either Sq rows of one head (the reference's
            # [B, Hkv, g, D] convention, tests/benchmark.py:438-443) or the g heads that
            # repeat_interleave maps onto one kv head, each with a single row.
            if plan.Sq == 1 and plan.Hq != plan.Hkv:
                g = plan.Hq // plan.Hkv
                q4 = q.as_strided((plan.B, plan.Hkv, g, plan.D),
                                  (q.stride(0), q.stride(1) * g, q.stride(1), 1))
                out = torch.empty((plan.B, plan.Hq, 1, plan.D), dtype=q.dtype, device=q.device)
                o4 = out.view(plan.B, plan.Hkv, g, plan.D)
            else:
                q4 = q
                out = torch.empty((plan.B, plan.Hq, plan.Sq, plan.D), dtype=q.dtype,
                                  device=q.device)
                o4 = out
            if plan.kernel == "decode":
                F.decode_attention(q4, args[spec.k.placeholder], args[spec.v.placeholder],
                                   scale=plan.scale, mods=plan.mods, out=o4,
                                   workspace=self.workspace, status=status)
            else:
                kt, vt = args[spec.k.block_table], args[spec.v.block_table]
                F.paged_decode_attention(
                    q4, args[spec.k.placeholder], args[spec.v.placeholder], kt,
                    block_table_v=None if spec.v.block_table == spec.k.block_table else vt,
                    scale=plan.scale, mods=plan.mods, out=o4, workspace=self.workspace,
                    status=status)
            self._check(status, plan)
            return (out,)
        # Prefill. K and V may be paged independently, as in the reference's own paged-attention
        # tests (tests/test_accuracy.py:253-311: K through paged_load, V dense); the gather of a
        # paged operand is fused into the kernel's tile loads.
        if spec.k.paged or spec.v.paged:
            out = F.prefill_attention(
                q, args[spec.k.placeholder], args[spec.v.placeholder], scale=plan.scale,
                mods=plan.mods, mask_kind=spec.mask_kind, window=plan.window, status=status,
                k_block_table=args[spec.k.block_table] if spec.k.paged else None,
                v_block_table=args[spec.v.block_table] if spec.v.paged else None)
        elif spec.q_pe is not None:
            # Two-matmul (MLA-style) scores, tests/test_attention.py:126-151 of the reference.
            out = F.prefill_attention(
                q, args[spec.k.placeholder], args[spec.v.placeholder], scale=plan.scale,
                mods=plan.mods, mask_kind=spec.mask_kind, window=plan.window, status=status,
                q_pe=args[spec.q_pe], k_pe=args[spec.k_pe])
            if spec.out_bias is not None:
                F.add_bf16(out, args[spec.out_bias], out=out)
        elif spec.q_bias is not None or spec.out_bias is not None or spec.score_bias is not None:
            # Modified attention of the reference's tests (tests/test_accuracy.py:176-194): the
            # query bias is added first (one bf16 rounding, as in the eager graph), the score
            # bias is read inside the attention kernel, the output bias is added in place.
            k, v = args[spec.k.placeholder], args[spec.v.placeholder]
            if spec.q_bias is not None:
                q = F.add_bf16(q, args[spec.q_bias])
            out = F.prefill_attention(
                q, k, v, scale=plan.scale, mods=plan.mods, mask_kind=spec.mask_kind,
                window=plan.window, status=status,
                score_bias=args[spec.score_bias] if spec.score_bias is not None else None,
                bias_pos=self._bias_pos(plan))
            if spec.out_bias is not None:
                F.add_bf16(out, args[spec.out_bias], out=out)
        else:
            k, v = args[spec.k.placeholder], args[spec.v.placeholder]
            out = torch.empty((plan.B, plan.Hq, plan.Sq, plan.D), dtype=q.dtype, device=q.device)
            self._prepared_prefill(plan, q, k, v, status).run(out)
        self._check(status, plan)
        return (out,)

    def _check(self, status: Optional[torch.Tensor], plan: AttentionPlan) -> None:
        if status is not None:
            try:
                F.check_status(status, plan.kernel)
            finally:
                status.zero_()


def loopfuse_compiler(gm: torch.fx.GraphModule, sample_inputs, mode: Optional[str] = None,
                      **kwargs) -> Callable:
    """Forward compiler for AOT autograd: aten graph -> CompiledAttention."""
    spec = analyse_graph(gm)
    if _flag("DEBUG"):
        print(gm.code)
        print(f"[loopfuse_b200] {spec.describe()}")
    return CompiledAttention(gm, spec, mode)


def loopfuse_backend(gm, sample_inputs, mode="max-autotune", **kwargs):
    """Main entry point for the loopfuse torch.compile backend (sm_100a kernels).

    ``mode`` is accepted for compatibility; the kernels are hand-tuned, nothing is autotuned.
    """
    compiler = partial(loopfuse_compiler, mode=mode, **kwargs)
    return aot_module_simplified(gm, sample_inputs, fw_compiler=compiler)
