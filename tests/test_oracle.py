"""The CPU oracle against the fixtures generated from the reference itself
(tests/golden/make_golden.py): eager ops, eager attention functions, generated loop bounds."""
import json

import pytest
import torch

from oracle import attention_oracle as O


@pytest.fixture(scope="module")
def eager_ops(golden_dir):
    return torch.load(golden_dir / "eager_ops.pt")


@pytest.fixture(scope="module")
def eager_att(golden_dir):
    return torch.load(golden_dir / "eager_attention.pt")


@pytest.fixture(scope="module")
def skip_golden(golden_dir):
    with open(golden_dir / "skip_ranges.json") as f:
        return json.load(f)


def test_causal_mask_bit_exact(eager_ops):
    assert torch.equal(O.causal_mask_ref(eager_ops["x"]), eager_ops["causal_mask"])
    assert torch.equal(O.causal_mask_general(eager_ops["x"]), eager_ops["causal_mask"])


def test_sliding_mask_eager_bit_exact(eager_ops):
    x = eager_ops["x"]
    assert torch.equal(O.sliding_mask_eager_ref(x, 5), eager_ops["sliding_mask_w5"])
    assert torch.equal(O.sliding_mask_eager_ref(x, 64), eager_ops["sliding_mask_w64"])


def test_compiled_window_equals_causal_of_eager_window(eager_ops):
    # The compiled-kernel mask (0 <= i-j < W) is the reference's eager sliding mask
    # intersected with its causal mask.
    x = eager_ops["x"]
    assert torch.equal(O.sliding_mask_ref(x, 5), eager_ops["causal_of_sliding_w5"])
    assert torch.equal(O.causal_mask_general(O.sliding_mask_ref(x, 5)),
                       eager_ops["causal_of_sliding_w5"])


def test_paged_load_bit_exact(eager_ops):
    assert torch.equal(O.paged_load_ref(eager_ops["buffer"], eager_ops["table"]),
                       eager_ops["paged_load"])
    assert torch.equal(O.paged_load_ref(eager_ops["buffer4"], eager_ops["table4"]),
                       eager_ops["paged_load4"])


def test_physical_rows_match_gather(eager_ops):
    pool, table = eager_ops["buffer4"], eager_ops["table4"]      # [12, 4, 2, 8], [2, 6]
    P = pool.shape[1]
    rows = O.physical_rows(table, P, table.shape[1] * P)          # [2, 24]
    flat = pool.reshape(-1, *pool.shape[2:])
    gathered = eager_ops["paged_load4"].reshape(2, -1, *pool.shape[2:])
    assert torch.equal(flat[rows], gathered)


@pytest.mark.parametrize("name,kw", [
    ("causal", dict(mask="causal")),
    ("causal_softcap50", dict(mask="causal", mods=O.softcap_mods(50))),
    ("window24_gqa_softcap50", dict(mask="window", window=24, mods=O.softcap_mods(50))),
    ("decode", dict()),
])
def test_attention_matches_reference_eager(eager_att, name, kw):
    # 1e-4: fp32 matmul and softmax sum in an order that depends on the CPU and the thread count,
    # so fixtures made on one machine reproduce to about 1e-6..1e-5 on another, not bit for bit
    case = eager_att[name]
    out = O.attention_ref(case["q"], case["k"], case["v"], **kw)
    torch.testing.assert_close(out, case["out"], rtol=1e-4, atol=1e-4)


def test_paged_attention_matches_reference_eager(eager_att):
    case = eager_att["paged_gqa_decode_p4"]
    k = O.paged_kv_ref(case["k_pool"], case["block_table"])
    v = O.paged_kv_ref(case["v_pool"], case["block_table"])
    out = O.attention_ref(case["q"], k, v)
    torch.testing.assert_close(out, case["out"], rtol=1e-4, atol=1e-4)


def test_modified_attention_oracle_against_the_eager_bf16_graph():
    """The function of the reference's tests/test_accuracy.py:176-181 evaluated eagerly on bf16
    tensors (every op rounds to bf16) stays within bf16 noise of the oracle, which keeps only
    the roundings at the two bias additions."""
    import loopfuse_b200  # noqa: F401  (registers loopfuse::causal_mask, pinned by eager_ops.pt)
    g = torch.Generator().manual_seed(4)
    B, H, S, D = 2, 2, 96, 64
    mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
    Q, K, V, qb, ob = (mk(B, H, S, D) for _ in range(5))
    sb = mk(B, H, S, S)
    QK = (Q + qb) @ K.transpose(-2, -1) * (D ** -0.5)
    QK = QK * 3.5 + sb
    eager = torch.softmax(torch.ops.loopfuse.causal_mask(QK), dim=-1) @ V + ob
    want = O.modified_attention_ref(Q, K, V, qb, sb, ob)
    # (bf16 scores of magnitude ~10 carry steps of 0.06 into the softmax)
    torch.testing.assert_close(eager.float(), want, atol=0.15, rtol=0.05)


def test_chunking_does_not_change_result():
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(4, 2, 33, 16, generator=g) for _ in range(3))
    a = O.attention_ref(q, k, v, mask="causal", batch_chunk=1)
    b = O.attention_ref(q, k, v, mask="causal", batch_chunk=4)
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-4)


_MASK_OF = {"causal": ("causal", 0), "window256": ("window", 256),
            "causal_of_window256": ("window", 256), "window130": ("window", 130),
            "none": ("none", 0)}


def test_closed_forms_equal_generated_bounds(skip_golden):
    """reference_skip_range restates the expressions the reference's compiler generated."""
    for tab in skip_golden["tables"]:
        mask, window = _MASK_OF[tab["mask"]]
        for iq, (lo, hi) in enumerate(tab["ranges"]):
            got = O.reference_skip_range(mask, window, tab["S"], tab["tile_q"], tab["tile_k"], iq)
            assert got == (lo, hi), (tab["mask"], tab["S"], tab["tile_q"], tab["tile_k"], iq)


def test_generated_bounds_vs_brute_force(skip_golden):
    """Where the reference's bounds and the brute-force live-tile scan agree and where they do
    not: causal upper bounds always agree; the window lower bound drops one live corner tile
    exactly when tile_k divides (iq*tile_q - W + 2), which never happens for W=256 with
    power-of-two tiles >= 4 but does for W=130."""
    mismatches = {}
    for tab in skip_golden["tables"]:
        mask, window = _MASK_OF[tab["mask"]]
        S, tq, tk = tab["S"], tab["tile_q"], tab["tile_k"]
        keep = O.keep_matrix(mask, window, S, S)
        for iq, (lo, hi) in enumerate(tab["ranges"]):
            blo, bhi = O.brute_force_skip_range(mask, window, S, S, tq, tk, iq, keep=keep)
            assert hi == bhi, (tab["mask"], S, tq, tk, iq)
            if lo != blo:
                assert lo == blo + 1 and (iq * tq - window + 2) % tk == 0
                mismatches.setdefault(tab["mask"], 0)
                mismatches[tab["mask"]] += 1
    assert set(mismatches) <= {"window130"}
    assert mismatches.get("window130", 0) > 0


def test_kv_append_is_the_inverse_of_paged_load():
    """Appending rows through a permutation table and gathering them back with the reference's
    paged_load semantics returns the rows (the round trip that pins the page-index rule of the
    cache producer)."""
    g = torch.Generator().manual_seed(5)
    n_pages, P, Hkv, D, B, S = 24, 4, 2, 8, 3, 20
    pool = torch.zeros(n_pages, P, Hkv, D)
    table = torch.randperm(n_pages, generator=g)[:B * 6].view(B, 6).int()
    new = torch.randn(B, Hkv, S, D, generator=g)
    pool = O.kv_append_ref(pool, new[:, :, :13], table, 0)
    pool = O.kv_append_ref(pool, new[:, :, 13:], table, [13] * B)
    gathered = O.paged_load_ref(pool, table.long())           # [B, 6, P, Hkv, D]
    back = gathered.reshape(B, 6 * P, Hkv, D)[:, :S].transpose(1, 2)
    assert torch.equal(back, new)
    rows = O.physical_rows(table, P, S)                        # pool row of every (b, t)
    flat = pool.reshape(n_pages * P, Hkv, D)
    assert torch.equal(flat[rows.long()].transpose(1, 2), new)
