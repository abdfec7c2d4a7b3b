"""GPU parity tests: the sm_100a kernels, called through the C ABI (loopfuse_b200.functional),
against the CPU oracle on the same seeded bf16 inputs. Tolerance for bf16 outputs: max-abs error
<= 2e-2; page-index and block-skip decisions bit-exact."""
import dataclasses

import pytest
import torch

from loopfuse_b200 import functional as F
from loopfuse_b200 import spec as S
from loopfuse_b200.spec import ScoreMod
from loopfuse_b200.variants import WORKLOADS, make_inputs
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-2
DEV = "cuda"


def randn_bf16(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def max_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return (got.float().cpu() - want.float()).abs().max().item()


SOFTCAP = [ScoreMod(S.MOD_DIV, 50.0), ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_MUL, 50.0)]


# ------------------------------------------------------------------------------------------
# decode
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,Hkv,G,Skv,D", [
    (2, 3, 1, 512, 128), (2, 2, 4, 300, 128), (1, 2, 8, 1000, 128), (3, 2, 2, 77, 64),
    (1, 1, 1, 1, 128), (2, 4, 1, 2048, 64), (1, 2, 4, 4096, 128),
])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_decode_matches_oracle(B, Hkv, G, Skv, D, splits):
    q = randn_bf16(B, Hkv, G, D, seed=1)
    k = randn_bf16(B, Hkv, Skv, D, seed=2)
    v = randn_bf16(B, Hkv, Skv, D, seed=3)
    st = F.new_status(DEV)
    out = F.decode_attention(q.to(DEV), k.to(DEV), v.to(DEV), scale=D ** -0.5, splits=splits,
                             status=st)
    F.check_status(st)
    want = O.attention_ref(q, k, v, batch_chunk=B)
    assert max_err(out, want) <= TOL


def test_decode_split_invariance():
    B, Hkv, G, Skv, D = 2, 4, 4, 2048, 128
    q, k, v = (randn_bf16(B, Hkv, n, D, seed=i).to(DEV)
               for i, n in ((1, G), (2, Skv), (3, Skv)))
    outs = [F.decode_attention(q, k, v, scale=D ** -0.5, splits=s).float()
            for s in (1, 2, 4, 8)]
    for o in outs[1:]:
        assert (o - outs[0]).abs().max().item() <= 4e-3   # one bf16 ulp at |x| < 0.5


def test_decode_softcap_and_strided_inputs():
    B, Hkv, G, Skv, D = 2, 2, 4, 640, 128
    q = randn_bf16(B, Hkv, G, D, seed=1, scale=3.0)
    kv = randn_bf16(B, Skv, 2, Hkv, D, seed=2, scale=3.0)      # K and V interleaved, [B,S,2,H,D]
    k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
    kvd = kv.to(DEV)
    out = F.decode_attention(q.to(DEV), kvd[:, :, 0].transpose(1, 2), kvd[:, :, 1].transpose(1, 2),
                             scale=D ** -0.5, mods=SOFTCAP)
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0), batch_chunk=B)
    assert max_err(out, want) <= TOL


def test_decode_config4_full_size_sample():
    w = WORKLOADS["decode"]
    q, k, v = make_inputs(w, batch=8)
    out = F.decode_attention(q.to(DEV).view(8, w.Hkv, 1, w.D), k.to(DEV), v.to(DEV),
                             scale=w.D ** -0.5)
    want = O.attention_ref(q, k, v, batch_chunk=8)
    assert max_err(out.view_as(want), want) <= TOL


def test_combine_entry_point_merges_partials():
    """lf_combine_f32 on hand-made partials: equals the log-sum-exp merge computed in fp32."""
    import ctypes as C
    from loopfuse_b200 import _native
    B, Hkv, G, D, splits = 2, 3, 4, 128, 5
    units = B * Hkv * G
    g = torch.Generator().manual_seed(4)
    part_o = torch.randn(units, splits, D, generator=g)
    m = torch.randn(units, splits, generator=g) * 3
    l = torch.rand(units, splits, generator=g) + 0.5
    m[0, 2] = float("-inf")          # an empty split contributes nothing
    l[0, 2] = 0.0
    part_o[0, 2] = 0.0
    w = torch.exp2(m - m.max(dim=1, keepdim=True).values)
    want = (part_o * w[..., None]).sum(1) / (l * w).sum(1, keepdim=True)
    po, ml = part_o.to(DEV), torch.stack([m, l], dim=-1).contiguous().to(DEV)
    out = torch.empty(B, Hkv, G, D, dtype=torch.bfloat16, device=DEV)
    strides = (C.c_int64 * 3)(*out.stride()[:3])
    rc = _native.load().lf_combine_f32(po.data_ptr(), ml.data_ptr(), out.data_ptr(), B, Hkv, G, D,
                                       splits, strides, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert max_err(out.view(units, D), want) <= TOL


# ------------------------------------------------------------------------------------------
# paged decode
# ------------------------------------------------------------------------------------------
def _paged_case(B, Hkv, G, D, page_size, pages_per_seq, seed=0, extra_pages=5):
    g = torch.Generator().manual_seed(seed)
    n_pages = B * pages_per_seq + extra_pages
    q = randn_bf16(B, Hkv, G, D, seed=seed + 1)
    kp = randn_bf16(n_pages, page_size, Hkv, D, seed=seed + 2)
    vp = randn_bf16(n_pages, page_size, Hkv, D, seed=seed + 3)
    table = torch.randperm(n_pages, generator=g)[:B * pages_per_seq].view(B, pages_per_seq)
    return q, kp, vp, table.to(torch.int32)


@pytest.mark.parametrize("B,Hkv,G,D,P,NP", [
    (2, 2, 4, 128, 16, 20), (3, 8, 4, 128, 16, 128), (2, 2, 1, 64, 1, 300), (1, 3, 8, 128, 8, 33),
    (2, 2, 2, 128, 12, 10),
])
def test_paged_decode_matches_oracle(B, Hkv, G, D, P, NP):
    q, kp, vp, table = _paged_case(B, Hkv, G, D, P, NP)
    st = F.new_status(DEV)
    out = F.paged_decode_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV),
                                   scale=D ** -0.5, status=st)
    F.check_status(st)
    want = O.attention_ref(q, O.paged_kv_ref(kp, table), O.paged_kv_ref(vp, table), batch_chunk=B)
    assert max_err(out, want) <= TOL


def test_paged_gather_is_bit_exact():
    q, kp, vp, table = _paged_case(3, 4, 1, 128, 16, 9)
    st = F.new_status(DEV)
    got = F.paged_gather(kp.to(DEV), table.to(DEV), status=st)
    F.check_status(st)
    rows = O.physical_rows(table, 16, 9 * 16)                       # [B, S]
    flat = kp.reshape(-1, 4, 128)                                   # [(page, slot), H, D]
    want = flat[rows].transpose(1, 2)                               # [B, H, S, D]
    assert torch.equal(got.cpu(), want)
    assert torch.equal(got.cpu(), O.paged_load_ref(kp, table).reshape(3, -1, 4, 128).transpose(1, 2))


def test_paged_decode_equals_dense_decode_on_gathered_kv_bitwise():
    q, kp, vp, table = _paged_case(2, 4, 4, 128, 16, 64)
    qd, kpd, vpd, td = q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV)
    k = F.paged_gather(kpd, td)
    v = F.paged_gather(vpd, td)
    for splits in (1, 4):
        a = F.paged_decode_attention(qd, kpd, vpd, td, scale=0.088, splits=splits)
        b = F.decode_attention(qd, k, v, scale=0.088, splits=splits)
        assert torch.equal(a, b)


def test_paged_decode_separate_tables_and_partial_last_page():
    B, Hkv, G, D, P, NP = 2, 2, 2, 128, 16, 12
    q, kp, vp, kt = _paged_case(B, Hkv, G, D, P, NP, seed=5)
    g = torch.Generator().manual_seed(99)
    vt = torch.randperm(kp.shape[0], generator=g)[:B * NP].view(B, NP).to(torch.int32)
    seq_len = NP * P - 5
    out = F.paged_decode_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), kt.to(DEV),
                                   block_table_v=vt.to(DEV), seq_len=seq_len, scale=D ** -0.5)
    k = O.paged_kv_ref(kp, kt)[:, :, :seq_len]
    v = O.paged_kv_ref(vp, vt)[:, :, :seq_len]
    assert max_err(out, O.attention_ref(q, k, v, batch_chunk=B)) <= TOL


def test_out_of_range_page_id_sets_status_and_does_not_fault():
    q, kp, vp, table = _paged_case(1, 2, 1, 128, 16, 8)
    bad = table.clone()
    bad[0, 3] = kp.shape[0] + 100
    st = F.new_status(DEV)
    F.paged_decode_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), bad.to(DEV), scale=1.0, status=st)
    with pytest.raises(RuntimeError, match="page id"):
        F.check_status(st)
    torch.cuda.synchronize()


def test_paged_config5_reduced_batch():
    w = dataclasses.replace(WORKLOADS["paged_decode_gqa"], B=8)
    q, kp, vp, table = make_inputs(w)
    out = F.paged_decode_attention(q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV),
                                   scale=w.D ** -0.5)
    want = O.workload_ref(w, (q, kp, vp, table))
    assert max_err(out, want) <= TOL


# ------------------------------------------------------------------------------------------
# prefill
# ------------------------------------------------------------------------------------------
def _prefill_case(B, Hq, Hkv, Sq, Skv, D, seed=0, scale=1.0):
    return (randn_bf16(B, Hq, Sq, D, seed=seed + 1, scale=scale),
            randn_bf16(B, Hkv, Skv, D, seed=seed + 2, scale=scale),
            randn_bf16(B, Hkv, Skv, D, seed=seed + 3))


def _run_prefill(q, k, v, **kw):
    st = F.new_status(DEV)
    out = F.prefill_attention(q.to(DEV), k.to(DEV), v.to(DEV), status=st, **kw)
    F.check_status(st, "prefill")
    return out


@pytest.mark.parametrize("S_", [17, 128, 129, 256, 593, 1024])
@pytest.mark.parametrize("D", [64, 128])
def test_prefill_causal(S_, D):
    q, k, v = _prefill_case(2, 2, 2, S_, S_, D)
    out = _run_prefill(q, k, v, scale=D ** -0.5, mask_kind=S.MASK_CAUSAL)
    want = O.attention_ref(q, k, v, mask="causal", batch_chunk=2)
    assert max_err(out, want) <= TOL


@pytest.mark.parametrize("S_", [100, 384, 640])
def test_prefill_no_mask(S_):
    q, k, v = _prefill_case(1, 3, 3, S_, S_, 128)
    out = _run_prefill(q, k, v, scale=128 ** -0.5)
    assert max_err(out, O.attention_ref(q, k, v)) <= TOL


def test_prefill_config1_full():
    w = WORKLOADS["causal_tiny"]
    q, k, v = make_inputs(w)
    out = _run_prefill(q, k, v, scale=w.D ** -0.5, mask_kind=S.MASK_CAUSAL)
    assert max_err(out, O.workload_ref(w, (q, k, v), batch_chunk=2)) <= TOL


KV_TILES = [64, 128]   # the two bounded-softcap kernels (64-key and 128-key KV tiles)


@pytest.mark.parametrize("kv_tile", KV_TILES)
@pytest.mark.parametrize("S_,scale_in", [(512, 1.0), (593, 3.0), (100, 1.0), (2048, 6.0)])
def test_prefill_softcap(S_, scale_in, kv_tile):
    q, k, v = _prefill_case(1, 4, 4, S_, S_, 128, scale=scale_in)
    out = _run_prefill(q, k, v, scale=128 ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL,
                       kv_tile=kv_tile)
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0), mask="causal")
    assert max_err(out, want) <= TOL


@pytest.mark.parametrize("kv_tile", KV_TILES)
@pytest.mark.parametrize("S_,W,G", [(1024, 256, 4), (593, 130, 2), (640, 258, 1), (300, 1024, 4),
                                    (512, 1, 1), (2048, 256, 4), (900, 64, 2),
                                    (593, 130, 4), (45, 16, 4), (97, 300, 4)])
def test_prefill_window_gqa_softcap(S_, W, G, kv_tile):
    q, k, v = _prefill_case(1, 2 * G, 2, S_, S_, 128, scale=2.0)
    out = _run_prefill(q, k, v, scale=128 ** -0.5, mods=SOFTCAP,
                       mask_kind=S.MASK_CAUSAL_WINDOW, window=W, kv_tile=kv_tile)
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0), mask="window", window=W)
    assert max_err(out, want) <= TOL


def test_prefill_generic_score_mods():
    q, k, v = _prefill_case(1, 2, 2, 256, 256, 64)
    mods = [ScoreMod(S.MOD_MUL, 3.5), ScoreMod(S.MOD_ADD, 1.0), ScoreMod(S.MOD_RELU),
            ScoreMod(S.MOD_ADD, -2.0)]
    out = _run_prefill(q, k, v, scale=0.125, mods=mods, mask_kind=S.MASK_CAUSAL)
    want = O.attention_ref(q, k, v, scale=0.125,
                           mods=[("mul", 3.5), ("add", 1.0), ("relu", None), ("add", -2.0)],
                           mask="causal")
    assert max_err(out, want) <= TOL


def test_prefill_rectangular_with_offset():
    # chunked prefill: 200 new queries against 456 keys, diagonal aligned bottom-right
    q, k, v = _prefill_case(1, 2, 2, 200, 456, 128)
    out = _run_prefill(q, k, v, scale=128 ** -0.5, mask_kind=S.MASK_CAUSAL, causal_offset=256)
    want = O.attention_ref(q, k, v, mask="causal", offset=256)
    assert max_err(out, want) <= TOL


def test_prefill_strided_views():
    B, H, S_, D = 2, 2, 300, 128
    qkv = randn_bf16(B, S_, 3, H, D, seed=7)                        # packed [B, S, 3, H, D]
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    d = qkv.to(DEV)
    out = F.prefill_attention(d[:, :, 0].transpose(1, 2), d[:, :, 1].transpose(1, 2),
                              d[:, :, 2].transpose(1, 2), scale=D ** -0.5,
                              mask_kind=S.MASK_CAUSAL)
    assert max_err(out, O.attention_ref(q, k, v, mask="causal", batch_chunk=B)) <= TOL


@pytest.mark.parametrize("kind,W,S_", [(S.MASK_CAUSAL, 0, 2048), (S.MASK_CAUSAL_WINDOW, 256, 2048),
                                       (S.MASK_CAUSAL_WINDOW, 130, 593), (S.MASK_NONE, 0, 400)])
def test_kernel_iterates_exactly_the_analysed_skip_ranges(kind, W, S_):
    """Block-skip decisions are bit-exact: the (lo, hi) each q-tile really iterated on the GPU
    == the analysis layer's table == the brute-force scan of the mask."""
    B, H, D = 1, 2, 64
    q, k, v = _prefill_case(B, H, H, S_, S_, D)
    n_qt = -(-S_ // S.TILE_Q)
    dbg = torch.full((B * H * n_qt * 2,), -1, dtype=torch.int32, device=DEV)
    _run_prefill(q, k, v, scale=0.125, mask_kind=kind, window=W, dbg_ranges=dbg)
    got = dbg.view(B * H, n_qt, 2).cpu()
    table = S.skip_table(kind, W, 0, S_, S_)
    mask = {S.MASK_NONE: "none", S.MASK_CAUSAL: "causal", S.MASK_CAUSAL_WINDOW: "window"}[kind]
    keep = O.keep_matrix(mask, W, S_, S_)
    for iq in range(n_qt):
        assert tuple(got[0, iq].tolist()) == table[iq] == tuple(got[1, iq].tolist())
        assert table[iq] == O.brute_force_skip_range(mask, W, S_, S_, S.TILE_Q, S.TILE_K, iq,
                                                     keep=keep)


@pytest.mark.parametrize("kv_tile", KV_TILES)
@pytest.mark.parametrize("kind,W,S_", [(S.MASK_CAUSAL, 0, 2048), (S.MASK_CAUSAL_WINDOW, 256, 2048),
                                       (S.MASK_CAUSAL_WINDOW, 130, 593), (S.MASK_NONE, 0, 400)])
def test_persistent_softcap_kernel_iterates_exactly_the_analysed_skip_ranges(kind, W, S_, kv_tile):
    """The same bit-exact check for the persistent kernels that softcap(50) selects (more work
    items than SMs, so every CTA walks several items), in units of the kernel's own KV tile."""
    B, H, D = 3, 32, 64
    q, k, v = _prefill_case(B, H, 8, S_, S_, D)
    kw = dict(scale=0.125, mods=SOFTCAP, mask_kind=kind, window=W, kv_tile=kv_tile)
    assert F.prefill_kv_tile(q.to(DEV), k.to(DEV), v.to(DEV), **kw) == kv_tile
    # Four query heads per kv head: under a window mask the 64-key kernel packs them into one
    # tile and walks the query rows in chunks of 32; the ranges are then per chunk.
    q_tile = F.prefill_q_tile(q.to(DEV), k.to(DEV), v.to(DEV), **kw)
    assert q_tile == (32 if kind == S.MASK_CAUSAL_WINDOW and kv_tile == 64 else S.TILE_Q)
    n_qt = -(-S_ // q_tile)
    dbg = torch.full((B * H * n_qt * 2,), -1, dtype=torch.int32, device=DEV)
    _run_prefill(q, k, v, dbg_ranges=dbg, **kw)
    got = dbg.view(B * H, n_qt, 2).cpu()
    table = S.skip_table(kind, W, 0, S_, S_, tile_q=q_tile, tile_k=kv_tile)
    mask = {S.MASK_NONE: "none", S.MASK_CAUSAL: "causal", S.MASK_CAUSAL_WINDOW: "window"}[kind]
    keep = O.keep_matrix(mask, W, S_, S_)
    for iq in range(n_qt):
        assert all(tuple(got[u, iq].tolist()) == table[iq] for u in range(B * H))
        assert table[iq] == O.brute_force_skip_range(mask, W, S_, S_, q_tile, kv_tile, iq,
                                                     keep=keep)


@pytest.mark.parametrize("kv_tile", KV_TILES)
@pytest.mark.parametrize("S_,W", [(593, 0), (1024, 200), (130, 64)])
def test_prefill_softcap_head_dim_64(S_, W, kv_tile):
    q, k, v = _prefill_case(2, 4, 2, S_, S_, 64, scale=1.5)
    kind = S.MASK_CAUSAL_WINDOW if W else S.MASK_CAUSAL
    out = _run_prefill(q, k, v, scale=64 ** -0.5, mods=SOFTCAP, mask_kind=kind, window=W,
                       kv_tile=kv_tile)
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0), mask="window" if W else "causal",
                           window=W, batch_chunk=2)
    assert max_err(out, want) <= TOL


@pytest.mark.parametrize("G", [2, 4])
@pytest.mark.parametrize("S_,W", [(1024, 200), (333, 96)])
def test_prefill_packed_gqa_layout_head_dim_64(S_, W, G):
    """Two or four query heads per kv head under a window mask at D = 64: the packed layout
    (128 / G rows of each head per tile), ragged sizes, more than one kv head and batch."""
    q, k, v = _prefill_case(2, 2 * G, 2, S_, S_, 64, scale=1.5)
    kw = dict(scale=64 ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL_WINDOW, window=W)
    assert F.prefill_q_tile(q.to(DEV), k.to(DEV), v.to(DEV), **kw) == 128 // G
    out = _run_prefill(q, k, v, **kw)
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0), mask="window", window=W,
                           batch_chunk=2)
    assert max_err(out, want) <= TOL


def test_prefill_softcap_large_cap_uses_running_max():
    """cap * log2(e) > 80: outside the fixed-reference range, the running-max kernel runs."""
    cap = 100.0
    mods = [ScoreMod(S.MOD_DIV, cap), ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_MUL, cap)]
    q, k, v = _prefill_case(1, 4, 2, 593, 593, 128, scale=2.0)
    out = _run_prefill(q, k, v, scale=128 ** -0.5, mods=mods, mask_kind=S.MASK_CAUSAL)
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(cap), mask="causal")
    assert max_err(out, want) <= TOL


@pytest.mark.parametrize("softcap", [0, 64, 128])   # 0: running-max kernel; else the KV tile
def test_prefill_rows_without_visible_keys_are_nan(softcap):
    """Diagonal shifted up by 200: query rows 0..199 see no key at all (NaN in the eager
    computation), row 200 sees key 0 only; the first 128-row tile has no KV block to visit."""
    q, k, v = _prefill_case(1, 2, 2, 384, 256, 128)
    mods = SOFTCAP if softcap else []
    out = _run_prefill(q, k, v, scale=128 ** -0.5, mods=mods, mask_kind=S.MASK_CAUSAL,
                       causal_offset=-200, kv_tile=softcap).float().cpu()
    want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0) if softcap else (),
                           mask="causal", offset=-200)
    assert torch.isnan(want[:, :, :200]).all() and not torch.isnan(want[:, :, 200:]).any()
    assert torch.isnan(out[:, :, :200]).all()
    assert (out[:, :, 200:] - want[:, :, 200:]).abs().max().item() <= TOL
    assert torch.equal(out[:, :, 200], v[:, :, 0].float())


@pytest.mark.parametrize("kv_tile", KV_TILES)
@pytest.mark.parametrize("S_,W", [(128, 0), (256, 0), (700, 64)])
def test_persistent_kernels_many_short_items(S_, W, kv_tile):
    """Work items of one or two KV blocks, many more of them than SMs: the hand-over between
    items (row-sum exchange through the output staging buffers, O hand-back, Q prefetch) runs
    back to back. Repeated launches must agree bit for bit with each other and with the oracle
    within the tolerance."""
    B, Hq, Hkv, D = 6, 64, 16, 128
    q, k, v = _prefill_case(B, Hq, Hkv, S_, S_, D)
    kind = S.MASK_CAUSAL_WINDOW if W else S.MASK_CAUSAL
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    st = F.new_status(DEV)
    kw = dict(scale=D ** -0.5, mods=SOFTCAP, mask_kind=kind, window=W, kv_tile=kv_tile, status=st)
    first = F.prefill_attention(qd, kd, vd, **kw).clone()
    for _ in range(20):
        again = F.prefill_attention(qd, kd, vd, **kw)
        assert torch.equal(again, first)
    F.check_status(st)
    want = O.attention_ref(q[:2], k[:2], v[:2], mods=O.softcap_mods(50.0),
                           mask="window" if W else "causal", window=W, batch_chunk=1)
    assert max_err(first[:2], want) <= TOL


def test_persistent_kernel_launches_on_two_streams():
    """Launches that overlap on the GPU use different ticket counters."""
    q, k, v = (t.to(DEV) for t in _prefill_case(2, 8, 8, 1024, 1024, 128))
    kw = dict(scale=128 ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL)
    ref = F.prefill_attention(q, k, v, **kw)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(2)]
    outs = []
    for i in range(6):
        with torch.cuda.stream(streams[i % 2]):
            outs.append(F.prefill_attention(q, k, v, **kw))
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, ref)


@pytest.mark.parametrize("kv_tile", KV_TILES)
def test_prefill_config2_full_size_sample(kv_tile):
    """cfg 2 at full size on the GPU (the launch the benchmark times). The oracle checks one
    head of every batch element (a different head each) plus the last head of the last element,
    so every region of the work queue is covered; it needs about a second per head on the CPU."""
    w = WORKLOADS["causal_softcap"]
    q, k, v = make_inputs(w)
    out = _run_prefill(q, k, v, scale=w.D ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL,
                       kv_tile=kv_tile)
    heads = [(b, (5 * b + 3) % w.Hq) for b in range(w.B)] + [(w.B - 1, w.Hq - 1), (0, 0)]
    for b, h in heads:
        want = O.attention_ref(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1],
                               mods=O.softcap_mods(50.0), mask="causal")
        assert max_err(out[b:b + 1, h:h + 1], want) <= TOL
    # size-independent property: row 0 attends to key 0 only, so out[..., 0, :] == v[..., 0, :]
    assert torch.equal(out[:, :, 0, :].cpu(), v[:, :, 0, :])


@pytest.mark.parametrize("kv_tile", KV_TILES)
def test_prefill_config3_full_size_sample(kv_tile):
    """cfg 3 at full size: one kv head (its four query heads) of every batch element, plus the
    last kv head of the last element."""
    w = WORKLOADS["window_gqa_softcap"]
    q, k, v = make_inputs(w)
    out = _run_prefill(q, k, v, scale=w.D ** -0.5, mods=SOFTCAP,
                       mask_kind=S.MASK_CAUSAL_WINDOW, window=w.window, kv_tile=kv_tile)
    g = w.group
    units = [(b, (3 * b + 1) % w.Hkv) for b in range(w.B)] + [(w.B - 1, w.Hkv - 1)]
    for b, hk in units:
        qs = slice(hk * g, (hk + 1) * g)
        want = O.attention_ref(q[b:b + 1, qs], k[b:b + 1, hk:hk + 1], v[b:b + 1, hk:hk + 1],
                               mods=O.softcap_mods(50.0), mask="window", window=w.window)
        assert max_err(out[b:b + 1, qs], want) <= TOL
    kv_rep = v[:, :, 0, :].repeat_interleave(w.group, dim=1)
    assert torch.equal(out[:, :, 0, :].cpu(), kv_rep)


def test_prefill_and_decode_replay_from_a_cuda_graph():
    """The entry points only enqueue work on the given stream (a memset node for the work-queue
    counter, kernel nodes with the tensor maps passed by value), so after one eager call they can
    be captured once and replayed on new data in the same buffers."""
    q, k, v = (t.to(DEV) for t in _prefill_case(1, 4, 2, 640, 640, 128))
    kw = dict(scale=128 ** -0.5, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL)
    qd = randn_bf16(2, 2, 4, 128, seed=21).to(DEV)
    kd, vd = (randn_bf16(2, 2, 777, 128, seed=s_).to(DEV) for s_ in (22, 23))
    ws = F.DecodeWorkspace()
    out_p = torch.empty_like(q)
    F.prefill_attention(q, k, v, out=out_p, **kw)             # first calls outside the capture
    out_d = F.decode_attention(qd, kd, vd, scale=0.09, workspace=ws)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        F.prefill_attention(q, k, v, out=out_p, **kw)
        out_d2 = F.decode_attention(qd, kd, vd, scale=0.09, workspace=ws, out=out_d)
    for seed in (31, 32):
        q.copy_(randn_bf16(*q.shape, seed=seed))
        qd.copy_(randn_bf16(*qd.shape, seed=seed + 10))
        g.replay()
        torch.cuda.synchronize()
        want_p = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0), mask="causal")
        assert max_err(out_p, want_p) <= TOL
        want_d = O.attention_ref(qd.reshape(2, 8, 1, 128), kd, vd, scale=0.09).reshape(2, 2, 4, 128)
        assert max_err(out_d2, want_d) <= TOL


def test_persistent_kernel_ticket_counters_wrap_around():
    """More launches than the library has work-queue counters (256): slots are reused in stream
    order and every launch still walks the whole queue."""
    q, k, v = (t.to(DEV) for t in _prefill_case(1, 8, 4, 512, 512, 64))
    kw = dict(scale=0.125, mods=SOFTCAP, mask_kind=S.MASK_CAUSAL)
    ref = F.prefill_attention(q, k, v, **kw).clone()
    out = torch.empty_like(ref)
    for i in range(600):
        if i % 100 == 99:
            out.zero_()
        F.prefill_attention(q, k, v, out=out, **kw)
        if i % 100 == 99:
            assert torch.equal(out, ref)


def test_bounded_device_wait_runs_out_and_reports():
    """A wait that can never complete (an mbarrier nobody arrives on) gives up after its limit,
    writes LF_DEV_TIMEOUT into the status word and the kernel returns: check_status raises, the
    context stays usable. The limit here is 2e5 clocks (~0.1 ms); the product kernels use the
    same wait with a limit of 4e8 clocks."""
    from loopfuse_b200 import _native
    st = F.new_status(DEV)
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    rc = _native.load().lf_selftest_wait_timeout(200_000, st.data_ptr(), waited.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 1 | (99 << 8)
    assert 200_000 <= int(waited.item()) < 400_000_000
    with pytest.raises(RuntimeError, match="bounded device-side wait ran out .site 99"):
        F.check_status(st)
    # the context is alive: a real kernel runs and is correct afterwards
    q, k, v = _prefill_case(1, 2, 2, 128, 128, 64)
    out = _run_prefill(q, k, v, scale=0.125, mask_kind=S.MASK_CAUSAL)
    assert max_err(out, O.attention_ref(q, k, v, scale=0.125, mask="causal")) <= TOL
