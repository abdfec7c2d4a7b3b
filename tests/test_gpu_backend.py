"""End to end on the GPU through the drop-in front door: torch.compile(fn,
backend=loopfuse_backend) versus the same function run eagerly in fp32 on the CPU - the way the
reference's tests/test_accuracy.py:13-26 checks itself, with the 2e-2 bf16 tolerance."""
import dataclasses

import pytest
import torch

from loopfuse_b200 import loopfuse_backend
from loopfuse_b200.variants import WORKLOADS, make_inputs
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2


def compile_and_run(fn, inputs):
    torch._dynamo.reset()
    dev_inputs = tuple(t.to("cuda") for t in inputs)
    torch._dynamo.mark_static(dev_inputs[0], 3)
    torch._dynamo.mark_dynamic(dev_inputs[0], 2)
    out = torch.compile(fn, backend=loopfuse_backend, dynamic=True)(*dev_inputs)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("name,batch,seq", [
    ("causal_tiny", 2, 512), ("causal_softcap", 1, 1024), ("window_gqa_softcap", 1, 1024),
    ("decode", 4, 2048), ("paged_decode_gqa", 4, 2048),
])
def test_compiled_variant_matches_eager_fp32(name, batch, seq):
    w = dataclasses.replace(WORKLOADS[name], B=batch, S=seq)
    inputs = make_inputs(w)
    out = compile_and_run(w.fn(), inputs)
    want = O.workload_ref(w, inputs)
    assert out.dtype == torch.bfloat16 and out.shape == want.shape
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_compiled_function_equals_own_eager_ops_on_gpu():
    """The package's eager custom ops (what runs without torch.compile) against the compiled
    kernels, both on the GPU, ragged length as in the reference's S=593 case."""
    w = dataclasses.replace(WORKLOADS["causal_tiny"], B=4, Hq=8, Hkv=8, S=593)
    inputs = make_inputs(w)
    out = compile_and_run(w.fn(), inputs)
    eager = w.fn()(*(t.to("cuda").float() for t in inputs))
    assert (out.float() - eager).abs().max().item() <= TOL


def test_reference_style_gqa_test_shape():
    # tests/test_accuracy.py:146-169: B4 Hq8 Hk4 S1024 D64, causal GQA via repeat_interleave
    def fn(Q, K, V):
        Hq, Hk = Q.shape[1], K.shape[1]
        K = K.repeat_interleave(Hq // Hk, dim=1)
        V = V.repeat_interleave(Hq // Hk, dim=1)
        QK = Q @ K.transpose(-2, -1) * (Q.shape[-1] ** -0.5)
        return torch.softmax(torch.ops.loopfuse.causal_mask(QK), dim=-1) @ V

    g = torch.Generator().manual_seed(5)
    Q = torch.randn(4, 8, 1024, 64, generator=g).bfloat16()
    K = torch.randn(4, 4, 1024, 64, generator=g).bfloat16()
    V = torch.randn(4, 4, 1024, 64, generator=g).bfloat16()
    out = compile_and_run(fn, (Q, K, V))
    want = O.attention_ref(Q, K, V, mask="causal", batch_chunk=4)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_reference_style_paged_prefill():
    # tests/test_accuracy.py:253-278: K through paged_load (one token per page, random table
    # with repeats), V dense, causal prefill
    def fn(Q, K_cache, K_block_table, V):
        K = torch.ops.loopfuse.paged_load(K_cache, K_block_table).transpose(1, 2)
        QK = Q @ K.transpose(-2, -1) * (Q.shape[-1] ** -0.5)
        return torch.softmax(torch.ops.loopfuse.causal_mask(QK), dim=-1) @ V

    g = torch.Generator().manual_seed(6)
    B, H, S_, D = 4, 8, 1024, 64
    Kc = torch.randn(B * S_ * 2, H, D, generator=g).bfloat16()
    bt = torch.randint(0, B * S_ * 2, (B, S_), generator=g, dtype=torch.int32)
    Q = torch.randn(B, H, S_, D, generator=g).bfloat16()
    V = torch.randn(B, H, S_, D, generator=g).bfloat16()
    out = compile_and_run(fn, (Q, Kc, bt, V))
    K = O.paged_load_ref(Kc, bt.long()).transpose(1, 2)          # [B, H, S, D]
    want = O.attention_ref(Q, K, V, mask="causal", batch_chunk=B)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_reference_style_paged_prefill_gqa():
    # tests/test_accuracy.py:281-311: the same with grouped heads (repeat_interleave of the
    # paged K and of the dense V)
    def fn(Q, K_cache, K_block_table, V):
        K = torch.ops.loopfuse.paged_load(K_cache, K_block_table).transpose(1, 2)
        Hq_, Hk_ = Q.shape[1], K.shape[1]
        K = K.repeat_interleave(Hq_ // Hk_, dim=1)
        V = V.repeat_interleave(Hq_ // Hk_, dim=1)
        QK = Q @ K.transpose(-2, -1) * (Q.shape[-1] ** -0.5)
        return torch.softmax(torch.ops.loopfuse.causal_mask(QK), dim=-1) @ V

    g = torch.Generator().manual_seed(7)
    B, Hq, Hk, S_, D = 4, 8, 4, 256, 64
    Kc = torch.randn(B * S_ * 2, Hk, D, generator=g).bfloat16()
    bt = torch.randint(0, B * S_ * 2, (B, S_), generator=g, dtype=torch.int32)
    Q = torch.randn(B, Hq, S_, D, generator=g).bfloat16()
    V = torch.randn(B, Hk, S_, D, generator=g).bfloat16()
    out = compile_and_run(fn, (Q, Kc, bt, V))
    K = O.paged_load_ref(Kc, bt.long()).transpose(1, 2)
    want = O.attention_ref(Q, K, V, mask="causal", batch_chunk=B)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("S_", [1024, 200])
def test_reference_style_modified_attention(S_):
    # tests/test_accuracy.py:172-194: B4 H8 S1024 D64 with a query bias, a score multiplier and
    # a full [B, H, S, S] score bias, causal mask, output bias (S = 200: ragged tiles)
    def fn(Q, K, V, q_bias, scores_bias, out_bias):
        QK = (Q + q_bias) @ K.transpose(-2, -1) * (Q.shape[-1] ** -0.5)
        QK = QK * 3.5 + scores_bias
        masked_attn = torch.ops.loopfuse.causal_mask(QK)
        scores = torch.softmax(masked_attn, dim=-1)
        return scores @ V + out_bias

    g = torch.Generator().manual_seed(8)
    B, H, D = 4, 8, 64
    mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
    Q, K, V, qb, ob = (mk(B, H, S_, D) for _ in range(5))
    sb = mk(B, H, S_, S_)
    out = compile_and_run(fn, (Q, K, V, qb, sb, ob))
    want = O.modified_attention_ref(Q, K, V, qb, sb, ob, batch_chunk=B)
    # 2e-2 on the attention part, plus one bf16 step of the biased output (its last rounding
    # can fall the other way when the attention part differs within its tolerance)
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2 ** -7)


@pytest.mark.parametrize("D,S_", [(128, 1024), (64, 593)])
def test_reference_style_mla_two_matmul_scores(D, S_):
    # tests/test_attention.py:126-151: scores = Q_nope K_nope^T + Q_pe K_pe^T with D_pe = D / 8,
    # scaled by (D + D_pe)^-0.5, causal (the reference only prints the generated code for this
    # graph; parity here is against the eager fp32 function)
    def fn(Q_nope, Q_pe, K_nope, K_pe, V):
        qk_nope = Q_nope @ K_nope.transpose(-2, -1)
        qk_pe = Q_pe @ K_pe.transpose(-2, -1)
        qk = qk_nope + qk_pe
        qk *= (Q_nope.shape[-1] + Q_pe.shape[-1]) ** (-0.5)
        masked_qk = torch.ops.loopfuse.causal_mask(qk)
        scores = torch.softmax(masked_qk, dim=-1)
        return scores @ V

    g = torch.Generator().manual_seed(11)
    B, H = 2, 4
    mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
    Qn, Kn, V = (mk(B, H, S_, D) for _ in range(3))
    Qp, Kp = mk(B, H, S_, D // 8), mk(B, H, S_, D // 8)
    out = compile_and_run(fn, (Qn, Qp, Kn, Kp, V))
    want = O.mla_attention_ref(Qn, Qp, Kn, Kp, V, batch_chunk=B)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_second_score_product_with_a_wide_rotary_part():
    """C-ABI level: D_pe = 48 (three k-steps of the extra block), no mask, Sq != Skv."""
    from loopfuse_b200 import functional as F
    g = torch.Generator().manual_seed(12)
    mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
    q, qp = mk(1, 2, 130, 128), mk(1, 2, 130, 48)
    k, kp, v = mk(1, 2, 300, 128), mk(1, 2, 300, 48), mk(1, 2, 300, 128)
    out = F.prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=176 ** -0.5, q_pe=qp.cuda(),
                              k_pe=kp.cuda())
    want = O.mla_attention_ref(q, qp, k, kp, v, mask="none")
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_score_bias_position_in_the_chain():
    """C-ABI level: the bias is added after `bias_pos` ops of the chain (here between a tanh and
    a multiplier), not at its end."""
    from loopfuse_b200 import functional as F, spec as SP
    g = torch.Generator().manual_seed(9)
    B, H, S_, D = 1, 2, 192, 128
    mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
    q, k, v = (mk(B, H, S_, D) for _ in range(3))
    sb = mk(B, H, S_, S_)
    mods = [SP.ScoreMod(SP.MOD_TANH), SP.ScoreMod(SP.MOD_MUL, 2.0)]
    out = F.prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5, mods=mods,
                              mask_kind=SP.MASK_CAUSAL, score_bias=sb.cuda(), bias_pos=1)
    s = torch.tanh(q.float() @ k.float().transpose(-2, -1) * D ** -0.5) + sb.float()
    s = O.causal_mask_general(s * 2.0)
    want = torch.softmax(s, dim=-1) @ v.float()
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_add_bf16_is_bit_exact():
    from loopfuse_b200 import functional as F
    g = torch.Generator().manual_seed(10)
    a = torch.randn(2, 3, 70, 128, generator=g).bfloat16().cuda()
    b = torch.randn(2, 70, 3, 128, generator=g).bfloat16().cuda().transpose(1, 2)   # strided
    assert torch.equal(F.add_bf16(a, b), a + b)
    c = a.clone()
    F.add_bf16(c, b, out=c)
    assert torch.equal(c, a + b)


def test_status_word_is_checked_when_asked(monkeypatch):
    """LF_CHECK_STATUS=1: an out-of-range block-table entry raises through the compiled
    function (the reference's eager gather would raise an index error); the kernel itself
    clamps the address, nothing faults."""
    monkeypatch.setenv("LF_CHECK_STATUS", "1")
    w = dataclasses.replace(WORKLOADS["paged_decode_gqa"], B=2, S=512, pages_per_seq=32)
    q, kp, vp, table = make_inputs(w)
    bad = table.clone()
    bad[1, 3] = kp.shape[0] + 7
    with pytest.raises(Exception, match="page id"):
        compile_and_run(w.fn(), (q, kp, vp, bad))
    out = compile_and_run(w.fn(), (q, kp, vp, table))         # the next call is clean again
    want = O.workload_ref(w, (q, kp, vp, table))
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_cpu_tensors_fail_loudly():
    w = dataclasses.replace(WORKLOADS["causal_tiny"], B=1, S=128)
    inputs = make_inputs(w)
    torch._dynamo.reset()
    fn = torch.compile(w.fn(), backend=loopfuse_backend, dynamic=True)
    with pytest.raises(Exception, match="CUDA"):
        fn(*inputs)
