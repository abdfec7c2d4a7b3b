"""Graph capture and analysis: aten FX graph -> ``AttentionSpec``.

The reference parses the aten graph into loop IR (loopfuse/torch_backend/interface.py:357-527)
and lets its fusion passes discover the attention structure. This layer recognises the same
graphs directly, walking back from the graph output:

    out   = view(bmm(view(expand(P)), view(expand(V'))))
    P     = _softmax(M, -1, False)
    M     = [causal_mask | sliding_mask]* ( score-mod chain ( view(bmm(Q', K'^T)) ) )
    optionally with the additive tensors of the reference's modified attention
    (tests/test_accuracy.py:176-194): out + out_bias, (Q + q_bias), and one `+ scores_bias`
    ([B,H,S,S]) anywhere in the score-mod chain; and with the two-matmul scores of its MLA test
    (tests/test_attention.py:126-151): view(bmm(Q, K^T)) + view(bmm(Q_pe, K_pe^T)) at the start
    of the chain
    K',V' = dense input, optionally through repeat_interleave (unsqueeze -> expand -> clone -> view)
            or a paged gather  paged_load(pool, table) [-> view merging page dims] -> transpose(1, 2)

Anything else raises ``NotImplementedError`` (surfacing as ``BackendCompilerFailed``), as the
reference does for unsupported ops (loopfuse/torch_backend/interface.py:157-161); there is no
fallback path.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import fx

from . import ops as _ops  # noqa: F401  (registers torch.ops.loopfuse.*)
from .spec import (AttentionSpec, KVSource, ScalarExpr, ScoreMod, MASK_CAUSAL,
                   MASK_CAUSAL_WINDOW, MASK_NONE, MAX_MODS, MOD_ADD, MOD_COS, MOD_DIV, MOD_EXP,
                   MOD_EXP2, MOD_MUL, MOD_RELU, MOD_SIN, MOD_SQUARE, MOD_TANH)

aten = torch.ops.aten

_VIEW_LIKE = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)
_CASTS = (torch.ops.prims.convert_element_type.default, aten._to_copy.default)
_UNARY_MODS = {
    aten.tanh.default: MOD_TANH,
    aten.exp.default: MOD_EXP,
    aten.exp2.default: MOD_EXP2,
    aten.sin.default: MOD_SIN,
    aten.cos.default: MOD_COS,
    aten.relu.default: MOD_RELU,
}


def _is(node: Any, *targets) -> bool:
    return isinstance(node, fx.Node) and node.op == "call_function" and node.target in targets


def _rank(node: fx.Node) -> int:
    val = node.meta.get("val")
    if val is None:
        raise NotImplementedError(f"no shape metadata on {node.name}")
    return val.dim()


def _norm_dim(node: fx.Node, dim: int) -> int:
    r = _rank(node)
    return dim + r if dim < 0 else dim


def _is_transpose(node: Any, d0: int, d1: int) -> bool:
    """transpose/permute that swaps exactly (d0, d1) of its input (dims given non-negative)."""
    if _is(node, aten.transpose.int):
        a, b = _norm_dim(node.args[0], node.args[1]), _norm_dim(node.args[0], node.args[2])
        return {a, b} == {d0, d1}
    if _is(node, aten.permute.default):
        perm = [p + len(node.args[1]) if p < 0 else p for p in node.args[1]]
        want = list(range(len(perm)))
        want[d0], want[d1] = want[d1], want[d0]
        return perm == want
    return False


class _Matcher:
    def __init__(self, gm: fx.GraphModule):
        self.gm = gm
        self.placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
        self.ph_index = {n: i for i, n in enumerate(self.placeholders)}

    # -- helpers -------------------------------------------------------------------------
    def _tensor_placeholder(self, node: Any, what: str) -> int:
        if isinstance(node, fx.Node) and node.op == "placeholder" and isinstance(
                node.meta.get("val"), torch.Tensor):
            return self.ph_index[node]
        raise NotImplementedError(f"{what}: expected a graph input, found {_describe(node)}")

    def _is_tensor_input(self, node: Any, rank: int) -> bool:
        return (isinstance(node, fx.Node) and node.op == "placeholder"
                and isinstance(node.meta.get("val"), torch.Tensor)
                and node.meta["val"].dim() == rank)

    def _strip_bmm_operand(self, node: fx.Node) -> fx.Node:
        """Undo the batch flattening around bmm: [expand ->] [clone ->] view(3-D)."""
        if not _is(node, *_VIEW_LIKE):
            raise NotImplementedError(f"bmm operand is not a flattened 4-D tensor: {_describe(node)}")
        node = node.args[0]
        if _is(node, aten.clone.default):
            node = node.args[0]
        if _is(node, aten.expand.default):
            node = node.args[0]
        if _rank(node) != 4:
            raise NotImplementedError(f"attention operands must be 4-D, got rank {_rank(node)}")
        return node

    def _kv_source(self, node: fx.Node, what: str) -> KVSource:
        repeated = False
        # repeat_interleave(n, dim=1): unsqueeze(x, 2) -> expand -> clone -> view
        if _is(node, *_VIEW_LIKE) and _is(node.args[0], aten.clone.default):
            exp = node.args[0].args[0]
            if _is(exp, aten.expand.default) and _is(exp.args[0], aten.unsqueeze.default):
                unsq = exp.args[0]
                if _norm_dim(unsq, unsq.args[1]) == 2 and _rank(unsq.args[0]) == 4:
                    repeated = True
                    node = unsq.args[0]
        # paged gather: paged_load(pool, table) [-> view] -> transpose(1, 2)
        if _is_transpose(node, 1, 2) and _rank(node) == 4:
            inner = node.args[0]
            if _is(inner, *_VIEW_LIKE):
                inner = inner.args[0]
            if _is(inner, torch.ops.loopfuse.paged_load.default):
                pool = self._tensor_placeholder(inner.args[0], f"{what} pool")
                table = self._tensor_placeholder(inner.args[1], f"{what} block table")
                if _rank(inner.args[1]) != 2:
                    raise NotImplementedError("block table must be [batch, blocks]")
                if _rank(inner.args[0]) not in (3, 4):
                    raise NotImplementedError(
                        "paged pool must be [pages, heads, D] or [pages, page_size, heads, D]")
                return KVSource(pool, table, repeated)
        return KVSource(self._tensor_placeholder(node, what), None, repeated)

    def _scalar_arg(self, arg: Any, what: str):
        if isinstance(arg, (int, float)):
            return float(arg)
        if isinstance(arg, fx.Node) and self._scalar_only(arg):
            val = arg.meta.get("val")
            if not isinstance(val, torch.Tensor) or val.numel() == 1:
                return ScalarExpr(arg)
        raise NotImplementedError(f"{what}: only constant operands are supported, found "
                                  f"{_describe(arg)}")

    def _scalar_only(self, node: fx.Node) -> bool:
        """True when the node is computed from scalar graph inputs and constants alone."""
        seen = set()
        stack = [node]
        while stack:
            n = stack.pop()
            if n in seen:
                continue
            seen.add(n)
            if n.op == "placeholder":
                # integers, floats (dynamo passes float closure constants as 0-dim CPU
                # tensors) - but never a real tensor operand
                val = n.meta.get("val")
                if isinstance(val, torch.Tensor) and val.dim() != 0:
                    return False
                continue
            if n.op != "call_function":
                return False
            stack.extend(a for a in n.all_input_nodes)
        return True

    # -- main ----------------------------------------------------------------------------
    def match(self) -> AttentionSpec:
        out_node = next(n for n in self.gm.graph.nodes if n.op == "output")
        outs = out_node.args[0]
        if not isinstance(outs, (tuple, list)) or len(outs) != 1:
            raise NotImplementedError("expected a graph with exactly one output")
        node = outs[0]
        out_bias = None
        if _is(node, aten.add.Tensor):
            a, b = node.args[0], node.args[1]
            if _is(b, *_VIEW_LIKE) and not _is(a, *_VIEW_LIKE):
                a, b = b, a
            out_bias = self._tensor_placeholder(b, "output bias")
            node = a
        if not _is(node, *_VIEW_LIKE) or not _is(node.args[0], aten.bmm.default):
            raise NotImplementedError(
                f"graph output is not `probabilities @ V`: {_describe(node)}")
        pv = node.args[0]
        probs = self._strip_bmm_operand(pv.args[0])
        v_src = self._kv_source(self._strip_bmm_operand(pv.args[1]), "V")

        if not _is(probs, aten._softmax.default):
            raise NotImplementedError(f"left operand of the last matmul is not a softmax: "
                                      f"{_describe(probs)}")
        if _norm_dim(probs, probs.args[1]) != 3 or probs.args[2]:
            raise NotImplementedError("softmax must be over the last dim, without half_to_float")
        node = probs.args[0]

        # masks (any order, any number)
        mask_kind = MASK_NONE
        windows: list = []
        while _is(node, torch.ops.loopfuse.causal_mask.default,
                  torch.ops.loopfuse.sliding_mask.default):
            if node.target is torch.ops.loopfuse.sliding_mask.default:
                w = node.args[1]
                if isinstance(w, fx.Node):
                    # a closure variable under dynamic=True arrives as an integer graph input
                    if not self._scalar_only(w):
                        raise NotImplementedError("sliding_mask window must be an integer")
                    w = ScalarExpr(w)
                elif not isinstance(w, int):
                    raise NotImplementedError("sliding_mask window must be an integer")
                elif w <= 0:
                    raise ValueError("sliding_mask window must be positive")
                windows.append(w)
                mask_kind = MASK_CAUSAL_WINDOW
            elif mask_kind == MASK_NONE:
                mask_kind = MASK_CAUSAL
            node = node.args[0]

        # score-mod chain, collected back to front
        mods: list[ScoreMod] = []
        score_bias = None
        ops_after_bias = 0
        def is_qk(n):
            return _is(n, *_VIEW_LIKE) and _is(n.args[0], aten.bmm.default)

        pe_qk = None
        while not is_qk(node):
            if (_is(node, aten.add.Tensor) and is_qk(node.args[0]) and is_qk(node.args[1])):
                # Q K^T + Q_pe K_pe^T: the main product is the one whose width V shares
                node, pe_qk = node.args[0], node.args[1]
                v_width = self.placeholders[v_src.placeholder].meta["val"].shape[-1]
                width = lambda n: self._strip_bmm_operand(n.args[0].args[0]).meta["val"].shape[-1]
                if width(node) != v_width and width(pe_qk) == v_width:
                    node, pe_qk = pe_qk, node
                break
            if _is(node, *_CASTS):
                # dtype round trips of the eager bf16 graph; the kernels keep scores in fp32
                # (the reference strips them too: cleanup_passes.py:211-271)
                node = node.args[0]
            elif _is(node, *_UNARY_MODS.keys()):
                mods.append(ScoreMod(_UNARY_MODS[node.target]))
                node = node.args[0]
            elif _is(node, aten.neg.default):
                mods.append(ScoreMod(MOD_MUL, -1.0))
                node = node.args[0]
            elif _is(node, aten.pow.Tensor_Scalar):
                if node.args[1] != 2:
                    raise NotImplementedError("pow is only supported with exponent 2")
                mods.append(ScoreMod(MOD_SQUARE))
                node = node.args[0]
            elif _is(node, aten.add.Tensor) and any(self._is_tensor_input(x, 4)
                                                    for x in node.args[:2]):
                # + scores_bias: a full [B, H, Sq, Skv] graph input
                a, b = node.args[0], node.args[1]
                if self._is_tensor_input(a, 4):
                    a, b = b, a
                if score_bias is not None:
                    raise NotImplementedError("only one additive score tensor is supported")
                if len(node.args) > 2 or node.kwargs.get("alpha", 1) != 1:
                    raise NotImplementedError("add with alpha is not supported")
                score_bias = self.ph_index[b]
                ops_after_bias = len(mods)
                node = a
            elif _is(node, aten.mul.Tensor, aten.add.Tensor):
                a, b = node.args[0], node.args[1]
                tensor_side, scalar_side = (a, b)
                if not (isinstance(a, fx.Node) and isinstance(a.meta.get("val"), torch.Tensor)
                        and a.meta["val"].dim() == 4):
                    tensor_side, scalar_side = (b, a)
                op = MOD_MUL if node.target is aten.mul.Tensor else MOD_ADD
                mods.append(ScoreMod(op, self._scalar_arg(scalar_side, node.name)))
                node = tensor_side
            elif _is(node, aten.div.Tensor, aten.sub.Tensor):
                arg = self._scalar_arg(node.args[1], node.name)
                if node.target is aten.div.Tensor:
                    mods.append(ScoreMod(MOD_DIV, arg))
                else:
                    if isinstance(arg, ScalarExpr):
                        raise NotImplementedError("sub with a run-time scalar is not supported")
                    mods.append(ScoreMod(MOD_ADD, -arg))
                node = node.args[0]
            else:
                raise NotImplementedError(
                    f"unsupported op between QK^T and softmax: {_describe(node)}")
            if not isinstance(node, fx.Node):
                raise NotImplementedError("score chain does not start at QK^T")
        mods.reverse()
        if len(mods) > MAX_MODS:
            raise NotImplementedError(f"score-mod chain longer than {MAX_MODS} ops")

        qk = node.args[0]
        q_node = self._strip_bmm_operand(qk.args[0])
        q_bias = None
        if _is(q_node, aten.add.Tensor):
            a, b = q_node.args[0], q_node.args[1]
            q_bias = self._tensor_placeholder(b, "query bias")
            q_node = a
        kt_node = self._strip_bmm_operand(qk.args[1])
        if not _is_transpose(kt_node, 2, 3):
            raise NotImplementedError(
                f"right operand of QK^T is not K.transpose(-2, -1): {_describe(kt_node)}")
        k_src = self._kv_source(kt_node.args[0], "K")
        q_idx = self._tensor_placeholder(q_node, "Q")
        if k_src.repeated != v_src.repeated:
            raise NotImplementedError("K and V must both (or neither) be repeat_interleave'd")

        for idx, what in ((q_idx, "Q"), (k_src.placeholder, "K"), (v_src.placeholder, "V")):
            dt = self.placeholders[idx].meta["val"].dtype
            if dt != torch.bfloat16:
                raise NotImplementedError(
                    f"{what} has dtype {dt}; the sm_100a kernels take bfloat16 inputs")
        q_pe = k_pe = None
        if pe_qk is not None:
            pq = self._strip_bmm_operand(pe_qk.args[0].args[0])
            pkt = self._strip_bmm_operand(pe_qk.args[0].args[1])
            if not _is_transpose(pkt, 2, 3):
                raise NotImplementedError("second score product is not Q_pe @ K_pe.transpose(-2, -1)")
            q_pe = self._tensor_placeholder(pq, "Q_pe")
            k_pe = self._tensor_placeholder(pkt.args[0], "K_pe")
            for idx in (q_pe, k_pe):
                if self.placeholders[idx].meta["val"].dtype != torch.bfloat16:
                    raise NotImplementedError("Q_pe / K_pe must be bfloat16")
            if (k_src.paged or v_src.paged or k_src.repeated or q_bias is not None
                    or score_bias is not None):
                raise NotImplementedError(
                    "two-product scores are supported with dense, ungrouped K/V and no bias")
            if any(m.op not in (MOD_MUL, MOD_DIV) for m in mods):
                raise NotImplementedError(
                    "two-product scores take constant multipliers only between QK^T and the mask")
        biases = [i for i in (q_bias, out_bias, score_bias) if i is not None]
        for idx in biases:
            if self.placeholders[idx].meta["val"].dtype != torch.bfloat16:
                raise NotImplementedError("bias tensors must be bfloat16")
        if biases and (k_src.paged or v_src.paged or k_src.repeated):
            raise NotImplementedError("bias tensors are supported with dense, ungrouped K/V only")
        return AttentionSpec(q=q_idx, k=k_src, v=v_src, mods=tuple(mods), mask_kind=mask_kind,
                             windows=tuple(windows), n_args=len(self.placeholders),
                             q_bias=q_bias, out_bias=out_bias, score_bias=score_bias,
                             bias_pos=len(mods) - ops_after_bias, q_pe=q_pe, k_pe=k_pe)


def _describe(node: Any) -> str:
    if isinstance(node, fx.Node):
        return f"{node.op}:{node.target} ({node.name})"
    return repr(node)


def analyse_graph(gm: fx.GraphModule) -> AttentionSpec:
    """aten-level FX graph (as handed to an AOT forward compiler) -> AttentionSpec."""
    return _Matcher(gm).match()


def evaluate_scalar(expr: ScalarExpr, placeholders: list, flat_args: list) -> float:
    """Evaluate a call-time scalar from the integer arguments of this call."""
    env: dict[fx.Node, Any] = {ph: flat_args[i] for i, ph in enumerate(placeholders)}

    def ev(x: Any) -> Any:
        if isinstance(x, fx.Node):
            if x not in env:
                args = fx.node.map_arg(x.args, ev)
                kwargs = fx.node.map_arg(x.kwargs, ev)
                if x.target in _CASTS and not isinstance(args[0], torch.Tensor):
                    env[x] = args[0]  # dtype cast of a Python scalar: value unchanged
                else:
                    env[x] = x.target(*args, **kwargs)
            return env[x]
        return x

    val = ev(expr.node)
    return float(val.item() if isinstance(val, torch.Tensor) else val)
