"""GPU parity at the launch geometries the benchmark times, the KV-cache append kernel, the
generic score-mod interpreter and the sharded layout on a real device. Everything calls through
the C ABI; the CPU oracle is the checker. Tolerance for bf16 outputs: max-abs error <= 2e-2;
pure data movement (append, gather) is bit-exact."""
import dataclasses

import pytest
import torch

from loopfuse_b200 import functional as F
from loopfuse_b200 import sharding
from loopfuse_b200 import spec as S
from loopfuse_b200.spec import ScoreMod
from loopfuse_b200.variants import WORKLOADS, make_inputs
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-2
DEV = "cuda"
SOFTCAP = [ScoreMod(S.MOD_DIV, 50.0), ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_MUL, 50.0)]


def randn_bf16(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def max_err(got, want) -> float:
    return (got.float().cpu() - want.float()).abs().max().item()


# ------------------------------------------------------------------------------------------
# decode / paged decode at the benchmark's batch (the split count depends on the batch)
# ------------------------------------------------------------------------------------------
def test_decode_config4_at_the_benchmark_batch():
    """cfg 4 with B = 64 and splits = 0, exactly the launch bench.py times; the oracle is
    per-sequence, so it checks the first and the last eight sequences."""
    w = WORKLOADS["decode"]
    q, k, v = make_inputs(w)
    st = F.new_status(DEV)
    out = F.decode_attention(q.to(DEV).view(w.B, w.Hkv, w.group, w.D), k.to(DEV), v.to(DEV),
                             scale=w.D ** -0.5, splits=0, status=st)
    F.check_status(st)
    out = out.view(w.B, w.Hq, 1, w.D)
    for sl in (slice(0, 8), slice(w.B - 8, w.B)):
        want = O.attention_ref(q[sl], k[sl], v[sl], batch_chunk=8)
        assert max_err(out[sl], want) <= TOL


def test_paged_decode_config5_at_the_benchmark_batch():
    """cfg 5 with B = 64 and splits = 0 (the benchmark's launch geometry), first and last eight
    sequences against the oracle; and bit for bit against the dense decode on the gathered K/V
    at the same split count."""
    w = WORKLOADS["paged_decode_gqa"]
    q, kp, vp, table = make_inputs(w)
    qd, kpd, vpd, td = q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV)
    st = F.new_status(DEV)
    out = F.paged_decode_attention(qd, kpd, vpd, td, scale=w.D ** -0.5, splits=0, status=st)
    F.check_status(st)
    for sl in (slice(0, 8), slice(w.B - 8, w.B)):
        k = O.paged_kv_ref(kp, table[sl])
        v = O.paged_kv_ref(vp, table[sl])
        want = O.attention_ref(q[sl], k, v, batch_chunk=8)
        assert max_err(out[sl], want) <= TOL
    from loopfuse_b200 import _native
    splits = _native.load().lf_decode_auto_splits(w.B, w.Hkv, w.group, w.S, w.D, w.page_size)
    dense = F.decode_attention(qd, F.paged_gather(kpd, td), F.paged_gather(vpd, td),
                               scale=w.D ** -0.5, splits=splits)
    assert torch.equal(out, dense)


def test_paged_decode_one_token_pages_long_context():
    """The reference's own paged layout (one token per page, [n_pages, Hkv, D] pools, separate
    K and V tables; tests/benchmark.py:305-330) at a context where the block-table slice of a
    whole sequence does not fit next to the K/V rings: the library splits the KV range until
    it does."""
    B, Hkv, G, D, Skv = 40, 8, 1, 128, 8192          # B * Hkv = 320 >= 2 x SM count
    g = torch.Generator().manual_seed(3)
    n_pages = B * Skv
    q = randn_bf16(B, Hkv, G, D, seed=1)
    kp = randn_bf16(n_pages, Hkv, D, seed=2)
    vp = randn_bf16(n_pages, Hkv, D, seed=3)
    kt = torch.randint(0, n_pages, (B, Skv), generator=g, dtype=torch.int32)
    vt = torch.randint(0, n_pages, (B, Skv), generator=g, dtype=torch.int32)
    st = F.new_status(DEV)
    out = F.paged_decode_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), kt.to(DEV),
                                   block_table_v=vt.to(DEV), scale=D ** -0.5, status=st)
    F.check_status(st)
    for b in (0, B - 1):
        k = kp[kt[b].long()].transpose(0, 1)[None]       # [1, Hkv, Skv, D]
        v = vp[vt[b].long()].transpose(0, 1)[None]
        want = O.attention_ref(q[b:b + 1], k, v)
        assert max_err(out[b:b + 1], want) <= TOL


# ------------------------------------------------------------------------------------------
# KV-cache append (the producer of the paged format)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,D,T", [(16, 128, 37), (1, 128, 5), (12, 64, 30), (16, 128, 1)])
def test_kv_append_is_bit_exact_and_round_trips(P, D, T):
    B, Hkv, blocks = 3, 4, 8
    g = torch.Generator().manual_seed(11)
    n_pages = B * blocks + 7
    table = torch.randperm(n_pages, generator=g)[:B * blocks].view(B, blocks).to(torch.int32)
    kp = randn_bf16(n_pages, P, Hkv, D, seed=1)
    vp = randn_bf16(n_pages, P, Hkv, D, seed=2)
    kn = randn_bf16(B, Hkv, T, D, seed=3)
    vn = randn_bf16(B, Hkv, T, D, seed=4)
    cap = P * blocks                                   # tokens a sequence's table can hold
    pos = torch.tensor([0, min(5, cap - T), min(cap - T, 17)], dtype=torch.int32)
    kpd, vpd, td = kp.to(DEV), vp.to(DEV), table.to(DEV)
    st = F.new_status(DEV)
    F.kv_append(kn.to(DEV), vn.to(DEV), kpd, vpd, td, seq_pos=pos.to(DEV), status=st)
    F.check_status(st)
    assert torch.equal(kpd.cpu(), O.kv_append_ref(kp, kn, table, pos.tolist()))
    assert torch.equal(vpd.cpu(), O.kv_append_ref(vp, vn, table, pos.tolist()))
    # round trip through the gather kernel: the appended rows come back where they were put
    gathered = F.paged_gather(kpd, td).cpu()                 # [B, Hkv, blocks * P, D]
    for b in range(B):
        p0 = int(pos[b])
        assert torch.equal(gathered[b, :, p0:p0 + T], kn[b])


def test_kv_append_then_paged_decode_equals_dense_decode():
    """Prefill-sized append (strided new rows, scalar start position) followed by one-token
    appends; the paged decode over the produced cache equals the dense decode bit for bit."""
    B, Hkv, G, D, P, S0 = 4, 8, 4, 128, 16, 480
    blocks = 32
    g = torch.Generator().manual_seed(2)
    n_pages = B * blocks
    table = torch.randperm(n_pages, generator=g).view(B, blocks).to(torch.int32).to(DEV)
    kpool = torch.zeros(n_pages, P, Hkv, D, dtype=torch.bfloat16, device=DEV)
    vpool = torch.zeros_like(kpool)
    kv = randn_bf16(B, S0 + 3, 2, Hkv, D, seed=5).to(DEV)     # packed [B, S, 2, Hkv, D]
    k_all, v_all = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
    F.kv_append(k_all[:, :, :S0], v_all[:, :, :S0], kpool, vpool, table, start_pos=0)
    for t in range(S0, S0 + 3):
        F.kv_append(k_all[:, :, t:t + 1], v_all[:, :, t:t + 1], kpool, vpool, table, start_pos=t)
    q = randn_bf16(B, Hkv, G, D, seed=6).to(DEV)
    for splits in (1, 2):
        paged = F.paged_decode_attention(q, kpool, vpool, table, seq_len=S0 + 3, scale=0.09,
                                         splits=splits)
        dense = F.decode_attention(q, k_all.contiguous(), v_all.contiguous(), scale=0.09,
                                   splits=splits)
        assert torch.equal(paged, dense)


def test_kv_append_bad_positions_set_status_and_write_nothing():
    B, Hkv, D, P, blocks = 2, 2, 128, 16, 2
    table = torch.tensor([[0, 1], [2, 99]], dtype=torch.int32, device=DEV)   # 99: outside pool
    kpool = torch.zeros(4, P, Hkv, D, dtype=torch.bfloat16, device=DEV)
    vpool = torch.zeros_like(kpool)
    new = torch.ones(B, Hkv, 4, D, dtype=torch.bfloat16, device=DEV)
    st = F.new_status(DEV)
    F.kv_append(new, new, kpool, vpool, table, start_pos=14, status=st)      # crosses into page 1
    with pytest.raises(RuntimeError, match="page id"):
        F.check_status(st)
    torch.cuda.synchronize()
    assert kpool[0, 14:].eq(1).all() and kpool[1, :2].eq(1).all()            # sequence 0 written
    assert kpool[2, 14:].eq(1).all() and kpool[3].eq(0).all()                # bad page skipped
    st.zero_()
    F.kv_append(new, new, kpool, vpool, table, start_pos=30, status=st)      # past the table
    with pytest.raises(RuntimeError, match="page id"):
        F.check_status(st)


# ------------------------------------------------------------------------------------------
# generic score-mod interpreter (every opcode, running-max kernel and decode kernels)
# ------------------------------------------------------------------------------------------
MOD_CASES = {
    "tanh_add": ([ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_ADD, 0.5)], [("tanh", None), ("add", 0.5)]),
    "exp": ([ScoreMod(S.MOD_MUL, 0.5), ScoreMod(S.MOD_EXP)], [("mul", 0.5), ("exp", None)]),
    "exp2": ([ScoreMod(S.MOD_MUL, 0.5), ScoreMod(S.MOD_EXP2)], [("mul", 0.5), ("exp2", None)]),
    "sin": ([ScoreMod(S.MOD_MUL, 2.0), ScoreMod(S.MOD_SIN)], [("mul", 2.0), ("sin", None)]),
    "cos": ([ScoreMod(S.MOD_COS), ScoreMod(S.MOD_MUL, 3.0)], [("cos", None), ("mul", 3.0)]),
    "square": ([ScoreMod(S.MOD_SQUARE), ScoreMod(S.MOD_MUL, -0.25)],
               [("square", None), ("mul", -0.25)]),
    "div_relu": ([ScoreMod(S.MOD_ADD, 0.25), ScoreMod(S.MOD_DIV, 0.5), ScoreMod(S.MOD_RELU)],
                 [("add", 0.25), ("div", 0.5), ("relu", None)]),
}


@pytest.mark.parametrize("name", sorted(MOD_CASES))
def test_generic_score_mods_prefill_and_decode(name):
    """Every opcode of the score-mod interpreter, on the GPU, in the prefill kernel (generic
    mode) and in both decode kernels, against the eager fp32 computation of the same chain."""
    mods, ref_mods = MOD_CASES[name]
    D = 128
    q = randn_bf16(1, 4, 300, D, seed=1)
    k = randn_bf16(1, 2, 300, D, seed=2)
    v = randn_bf16(1, 2, 300, D, seed=3)
    st = F.new_status(DEV)
    out = F.prefill_attention(q.to(DEV), k.to(DEV), v.to(DEV), scale=D ** -0.5, mods=mods,
                              mask_kind=S.MASK_CAUSAL, status=st)
    F.check_status(st)
    want = O.attention_ref(q, k, v, scale=D ** -0.5, mods=ref_mods, mask="causal")
    assert max_err(out, want) <= TOL
    for G in (1, 4):                                   # FMA kernel / tensor-core kernel
        qd = randn_bf16(2, 2, G, D, seed=4)
        kd = randn_bf16(2, 2, 500, D, seed=5)
        vd = randn_bf16(2, 2, 500, D, seed=6)
        got = F.decode_attention(qd.to(DEV), kd.to(DEV), vd.to(DEV), scale=D ** -0.5, mods=mods)
        want = O.attention_ref(qd, kd, vd, scale=D ** -0.5, mods=ref_mods, batch_chunk=2)
        assert max_err(got, want) <= TOL


# ------------------------------------------------------------------------------------------
# the (batch x kv-head) partition on a real device
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("world", [2, 4])
def test_shard_units_on_device_concatenates_to_the_unsharded_result(world):
    """Two / four simulated ranks run their unit ranges one after the other on one GPU; the
    concatenation of their output slabs equals the unsharded launch bit for bit (same kernels,
    same per-unit arithmetic)."""
    w = dataclasses.replace(WORKLOADS["window_gqa_softcap"], B=2, S=640)
    q, k, v = (t.to(DEV) for t in make_inputs(w))
    kw = dict(scale=w.D ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL_WINDOW, window=w.window)
    full = F.prefill_attention(q, k, v, **kw)
    slabs = []
    for r in range(world):
        ql, kl, vl = sharding.shard_units(q, k, v, r, world)
        slabs.append(F.prefill_attention(ql, kl, vl, **kw))
    cat = torch.cat([s.reshape(-1) for s in slabs]).view_as(full)
    assert torch.equal(cat, full)
    # decode: shard by batch x kv-head as well
    wd = dataclasses.replace(WORKLOADS["decode"], B=4, Hq=8, Hkv=8, S=1024)
    qd, kd, vd = (t.to(DEV) for t in make_inputs(wd))
    full_d = F.decode_attention(qd.view(4, 8, 1, wd.D), kd, vd, scale=wd.D ** -0.5, splits=2)
    parts = []
    for r in range(world):
        ql, kl, vl = sharding.shard_units(qd, kd, vd, r, world)
        parts.append(F.decode_attention(ql, kl, vl, scale=wd.D ** -0.5, splits=2))
    assert torch.equal(torch.cat([p.reshape(-1) for p in parts]).view_as(full_d), full_d)


# ------------------------------------------------------------------------------------------
# paged K / V fused into the prefill tile loads
# ------------------------------------------------------------------------------------------
def _paged_prefill_case(B, Hq, Hkv, S_, D, P, seed=0):
    g = torch.Generator().manual_seed(seed)
    blocks = -(-S_ // P)
    n_pages = B * blocks + 9
    q = randn_bf16(B, Hq, S_, D, seed=seed + 1)
    kp = randn_bf16(n_pages, P, Hkv, D, seed=seed + 2)
    vp = randn_bf16(n_pages, P, Hkv, D, seed=seed + 3)
    kt = torch.randperm(n_pages, generator=g)[:B * blocks].view(B, blocks).to(torch.int32)
    vt = torch.randperm(n_pages, generator=g)[:B * blocks].view(B, blocks).to(torch.int32)
    return q, kp, vp, kt, vt


@pytest.mark.parametrize("B,Hq,Hkv,S_,D,P", [
    (2, 4, 4, 384, 64, 1), (2, 8, 2, 593, 128, 16), (1, 4, 2, 300, 128, 12), (3, 4, 4, 128, 64, 16),
])
@pytest.mark.parametrize("which", ["k", "v", "kv"])
def test_paged_prefill_fused_gather(B, Hq, Hkv, S_, D, P, which):
    """K and / or V of a causal prefill read through a block table inside the kernel: equal, bit
    for bit, to the same kernel on the gathered dense tensors (the gather only changes where the
    rows come from), and within tolerance of the oracle."""
    q, kp, vp, kt, vt = _paged_prefill_case(B, Hq, Hkv, S_, D, P)
    k_dense = O.paged_kv_ref(kp, kt)[:, :, :S_].to(torch.bfloat16)
    v_dense = O.paged_kv_ref(vp, vt)[:, :, :S_].to(torch.bfloat16)
    qd = q.to(DEV)
    kw = dict(scale=D ** -0.5, mask_kind=S.MASK_CAUSAL)
    k_arg = kp.to(DEV) if "k" in which else k_dense.to(DEV)
    v_arg = vp.to(DEV) if "v" in which else v_dense.to(DEV)
    st = F.new_status(DEV)
    out = F.prefill_attention(qd, k_arg, v_arg, status=st, seq_len=S_,
                              k_block_table=kt.to(DEV) if "k" in which else None,
                              v_block_table=vt.to(DEV) if "v" in which else None, **kw)
    F.check_status(st)
    dense = F.prefill_attention(qd, k_dense.to(DEV), v_dense.to(DEV), **kw)
    assert torch.equal(out, dense)
    want = O.attention_ref(q, k_dense, v_dense, mask="causal", batch_chunk=B)
    assert max_err(out, want) <= TOL


def test_paged_prefill_softcap_window_gqa_and_bad_page():
    q, kp, vp, kt, vt = _paged_prefill_case(2, 8, 2, 700, 128, 16, seed=4)
    k_dense = O.paged_kv_ref(kp, kt)[:, :, :700]
    v_dense = O.paged_kv_ref(vp, vt)[:, :, :700]
    st = F.new_status(DEV)
    kw = dict(scale=128 ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL_WINDOW, window=200,
              seq_len=700, status=st)
    out = F.prefill_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), k_block_table=kt.to(DEV),
                              v_block_table=vt.to(DEV), **kw)
    F.check_status(st)
    want = O.attention_ref(q, k_dense, v_dense, mods=O.softcap_mods(50.0), mask="window",
                           window=200, batch_chunk=2)
    assert max_err(out, want) <= TOL
    bad = kt.clone()
    bad[1, 5] = kp.shape[0] + 3
    F.prefill_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), k_block_table=bad.to(DEV),
                        v_block_table=vt.to(DEV), **kw)
    with pytest.raises(RuntimeError, match="page id"):
        F.check_status(st)
    torch.cuda.synchronize()
