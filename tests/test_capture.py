"""Graph capture and analysis on the CPU (analysis-only mode): the five benchmark variants and
the shapes the reference's tests use map to the expected AttentionSpec / plan; unsupported
graphs raise instead of falling back."""
import dataclasses

import pytest
import torch

from loopfuse_b200 import loopfuse_backend, spec as S
from loopfuse_b200.variants import WORKLOADS, make_inputs


@pytest.fixture(autouse=True)
def analysis_only(monkeypatch):
    monkeypatch.setenv("CODEGEN_ONLY", "1")
    torch._dynamo.reset()
    yield
    torch._dynamo.reset()


def compile_plan(fn, inputs, mark=True, **kw):
    if mark:
        torch._dynamo.mark_static(inputs[0], 3)
        torch._dynamo.mark_dynamic(inputs[0], 2)
    return torch.compile(fn, backend=loopfuse_backend, dynamic=True, **kw)(*inputs)


def small(name, **kw):
    w = WORKLOADS[name]
    return dataclasses.replace(w, B=2, S=min(w.S, 256),
                               pages_per_seq=16 if w.page_size else 0, **kw)


def mod_names(plan):
    return [(S.MOD_NAMES[m.op], m.arg) for m in plan.mods]


def test_causal_tiny():
    w = small("causal_tiny")
    plan = compile_plan(w.fn(), make_inputs(w))
    assert plan.kernel == "prefill"
    assert (plan.B, plan.Hq, plan.Hkv, plan.Sq, plan.Skv, plan.D) == (2, 4, 4, 256, 256, 64)
    assert plan.scale == pytest.approx(64 ** -0.5)
    assert plan.mods == () and plan.spec.mask_kind == S.MASK_CAUSAL
    assert plan.skip_ranges == [(0, 2), (0, 4)]


def test_causal_softcap():
    w = small("causal_softcap")
    plan = compile_plan(w.fn(), make_inputs(w))
    assert plan.kernel == "prefill" and plan.spec.mask_kind == S.MASK_CAUSAL
    assert plan.scale == pytest.approx(128 ** -0.5)
    assert mod_names(plan) == [("div", 50.0), ("tanh", 0.0), ("mul", 50.0)]


def test_window_gqa_softcap_with_duck_shaped_dims():
    # B == Hkv makes dynamo alias the two sizes into one symbol
    w = small("window_gqa_softcap", Hq=8, Hkv=2)
    plan = compile_plan(w.fn(), make_inputs(w))
    assert plan.kernel == "prefill"
    assert (plan.Hq, plan.Hkv) == (8, 2) and plan.spec.k.repeated and plan.spec.v.repeated
    assert plan.spec.mask_kind == S.MASK_CAUSAL_WINDOW and plan.window == 256
    assert mod_names(plan) == [("div", 50.0), ("tanh", 0.0), ("mul", 50.0)]


def test_window_ranges_at_benchmark_length():
    w = dataclasses.replace(WORKLOADS["window_gqa_softcap"], B=1, Hq=4, Hkv=1, D=64)
    plan = compile_plan(w.fn(), make_inputs(w))
    assert plan.skip_ranges == S.skip_table(S.MASK_CAUSAL_WINDOW, 256, 0, 2048, 2048)
    assert sum(hi - lo for lo, hi in plan.skip_ranges) == 90


def test_decode():
    w = small("decode")
    plan = compile_plan(w.fn(), make_inputs(w))
    assert plan.kernel == "decode" and plan.Sq == 1 and plan.Skv == 256
    assert plan.spec.mask_kind == S.MASK_NONE and plan.skip_ranges is None


def test_paged_gqa_decode_page16():
    w = small("paged_decode_gqa")
    plan = compile_plan(w.fn(), make_inputs(w))
    assert plan.kernel == "paged_decode"
    assert plan.page_size == 16 and plan.Skv == 256 and plan.Sq == 4 and plan.Hkv == 8
    assert plan.spec.k.paged and plan.spec.k.block_table == plan.spec.v.block_table


def test_paged_one_token_pages_separate_tables():
    # the reference's own paged benchmark layout: cache [N, H, D], one token per page,
    # independent K and V tables (tests/benchmark.py:308-334)
    def fn(q, kc, kt, vc, vt):
        k = torch.ops.loopfuse.paged_load(kc, kt).transpose(-3, -2)
        v = torch.ops.loopfuse.paged_load(vc, vt).transpose(-3, -2)
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(qk, dim=-1) @ v

    q = torch.randn(2, 4, 1, 64, dtype=torch.bfloat16)
    kc = torch.randn(300, 4, 64, dtype=torch.bfloat16)
    vc = torch.randn(300, 4, 64, dtype=torch.bfloat16)
    kt = torch.randint(0, 300, (2, 96), dtype=torch.int32)
    vt = torch.randint(0, 300, (2, 96), dtype=torch.int32)
    plan = compile_plan(fn, (q, kc, kt, vc, vt))
    assert plan.kernel == "paged_decode" and plan.page_size == 1 and plan.Skv == 96
    assert plan.spec.k.block_table != plan.spec.v.block_table


def test_repeat_interleave_decode_maps_to_grouped_decode():
    def fn(q, k, v):
        g = q.shape[1] // k.shape[1]
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(qk, dim=-1) @ v

    q = torch.randn(3, 8, 1, 128, dtype=torch.bfloat16)
    k = torch.randn(3, 2, 200, 128, dtype=torch.bfloat16)
    plan = compile_plan(fn, (q, k, k.clone()))
    assert plan.kernel == "decode" and (plan.Hq, plan.Hkv, plan.Sq) == (8, 2, 1)


def test_paged_prefill_goes_through_gather():
    # tests/test_accuracy.py:253-278 - paged K with a causal mask over a full prefill
    def fn(q, kc, kt, vc):
        k = torch.ops.loopfuse.paged_load(kc, kt).transpose(1, 2)
        v = torch.ops.loopfuse.paged_load(vc, kt).transpose(1, 2)
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(torch.ops.loopfuse.causal_mask(qk), dim=-1) @ v

    q = torch.randn(2, 4, 160, 64, dtype=torch.bfloat16)
    kc = torch.randn(500, 4, 64, dtype=torch.bfloat16)
    kt = torch.randint(0, 500, (2, 160), dtype=torch.int32)
    plan = compile_plan(fn, (q, kc, kt, kc.clone()))
    assert plan.kernel == "paged_prefill" and plan.spec.mask_kind == S.MASK_CAUSAL


def test_generic_score_mods_are_captured_in_order():
    def fn(q, k, v):
        s = q @ k.transpose(-2, -1) * 0.25
        s = torch.relu(s * 3.5 + 1.0) - 2.0
        return torch.softmax(s, dim=-1) @ v

    q = torch.randn(1, 2, 64, 64, dtype=torch.bfloat16)
    plan = compile_plan(fn, (q, q.clone(), q.clone()))
    assert plan.scale == pytest.approx(0.25)
    assert mod_names(plan) == [("mul", 3.5), ("add", 1.0), ("relu", 0.0), ("add", -2.0)]


def test_modified_attention_of_the_reference_tests_is_captured():
    """The graph of the reference's tests/test_accuracy.py:176-181: query bias, score multiplier
    and score bias, causal mask, output bias."""
    def fn(Q, K, V, q_bias, scores_bias, out_bias):
        QK = (Q + q_bias) @ K.transpose(-2, -1) * (Q.shape[-1] ** -0.5)
        QK = QK * 3.5 + scores_bias
        masked = torch.ops.loopfuse.causal_mask(QK)
        return torch.softmax(masked, dim=-1) @ V + out_bias

    q = torch.randn(2, 2, 128, 64, dtype=torch.bfloat16)
    sb = torch.randn(2, 2, 128, 128, dtype=torch.bfloat16)
    plan = compile_plan(fn, (q, q.clone(), q.clone(), q.clone(), sb, q.clone()))
    spec = plan.spec
    assert plan.kernel == "prefill" and plan.mask_kind == 1
    # (flat argument indices: symbolic sizes sit between the tensors)
    idx = (spec.q, spec.k.placeholder, spec.v.placeholder, spec.q_bias, spec.score_bias,
           spec.out_bias)
    assert None not in idx and len(set(idx)) == 6
    assert plan.scale == pytest.approx(0.125)
    assert mod_names(plan) == [("mul", 3.5)]
    assert spec.bias_pos == 2          # after `* D ** -0.5` and `* 3.5` of the captured chain


def test_two_matmul_scores_of_the_reference_mla_test_are_captured():
    """The graph of the reference's tests/test_attention.py:126-134."""
    def fn(Q_nope, Q_pe, K_nope, K_pe, V):
        qk_nope = Q_nope @ K_nope.transpose(-2, -1)
        qk_pe = Q_pe @ K_pe.transpose(-2, -1)
        qk = qk_nope + qk_pe
        qk *= (Q_nope.shape[-1] + Q_pe.shape[-1]) ** (-0.5)
        masked_qk = torch.ops.loopfuse.causal_mask(qk)
        return torch.softmax(masked_qk, dim=-1) @ V

    qn = torch.randn(1, 2, 128, 64, dtype=torch.bfloat16)
    qp = torch.randn(1, 2, 128, 8, dtype=torch.bfloat16)
    plan = compile_plan(fn, (qn, qp, qn.clone(), qp.clone(), qn.clone()))
    spec = plan.spec
    assert plan.kernel == "prefill" and plan.mask_kind == 1 and plan.D == 64
    assert spec.q_pe is not None and spec.k_pe is not None
    assert len({spec.q, spec.q_pe, spec.k.placeholder, spec.k_pe, spec.v.placeholder}) == 5
    assert plan.scale == pytest.approx(72 ** -0.5) and mod_names(plan) == []


def test_mode_kwarg_is_accepted():
    w = small("causal_tiny")
    plan = compile_plan(w.fn(), make_inputs(w), mode=None)
    assert plan.kernel == "prefill"


def test_import_aliases_of_the_reference_paths():
    from loopfuse import loopfuse_backend as a
    from loopfuse.torch_backend.interface import loopfuse_backend as b
    assert a is loopfuse_backend and b is loopfuse_backend


@pytest.mark.parametrize("case", ["bias_tensor", "fp32", "not_attention", "softmax_dim"])
def test_unsupported_graphs_raise(case):
    from torch._dynamo.exc import BackendCompilerFailed
    q = torch.randn(1, 2, 64, 64, dtype=torch.bfloat16)
    if case == "bias_tensor":   # a broadcast bias (only a full [B, H, S, S] one is supported)
        bias = torch.randn(64, 64, dtype=torch.bfloat16)

        def fn(q, k, v):
            return torch.softmax(q @ k.transpose(-2, -1) + bias, dim=-1) @ v
        args = (q, q.clone(), q.clone())
    elif case == "fp32":
        def fn(q, k, v):
            return torch.softmax(q @ k.transpose(-2, -1), dim=-1) @ v
        args = (q.float(), q.float(), q.float())
    elif case == "not_attention":
        def fn(q, k, v):
            return q + k * v
        args = (q, q.clone(), q.clone())
    else:
        def fn(q, k, v):
            return torch.softmax(q @ k.transpose(-2, -1), dim=-2) @ v
        args = (q, q.clone(), q.clone())
    with pytest.raises(BackendCompilerFailed):
        compile_plan(fn, args)
