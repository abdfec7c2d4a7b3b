"""Host-side logic on the CPU: the eager custom ops, and the block-skip ranges (Python mirror,
C ABI, brute force, and the reference's generated bounds)."""
import json

import pytest
import torch

import loopfuse_b200  # noqa: F401  registers torch.ops.loopfuse.*
from loopfuse_b200 import spec as S
from oracle import attention_oracle as O


@pytest.fixture(scope="module")
def eager_ops(golden_dir):
    return torch.load(golden_dir / "eager_ops.pt")


def test_eager_causal_mask_matches_reference(eager_ops):
    assert torch.equal(torch.ops.loopfuse.causal_mask(eager_ops["x"]), eager_ops["causal_mask"])


def test_eager_sliding_mask_is_the_compiled_reference_mask(eager_ops):
    x = eager_ops["x"]
    got = torch.ops.loopfuse.sliding_mask(x, 5)
    # equals causal_mask(sliding_mask(.)) of the reference, and the reference's eager
    # sliding_mask wherever j <= i
    assert torch.equal(got, eager_ops["causal_of_sliding_w5"])
    lower = torch.tril(torch.ones(37, 37, dtype=torch.bool))
    assert torch.equal(got[..., lower], eager_ops["sliding_mask_w5"][..., lower])
    assert torch.equal(torch.ops.loopfuse.causal_mask(got), eager_ops["causal_of_sliding_w5"])


def test_eager_paged_load_matches_reference(eager_ops):
    assert torch.equal(torch.ops.loopfuse.paged_load(eager_ops["buffer"], eager_ops["table"]),
                       eager_ops["paged_load"])
    assert torch.equal(torch.ops.loopfuse.paged_load(eager_ops["buffer4"], eager_ops["table4"]),
                       eager_ops["paged_load4"])


def test_scan_max():
    x = torch.randn(3, 5, 11)
    run, fin = torch.ops.loopfuse.scan_max(x)
    assert torch.equal(run, torch.cummax(x, -1).values)
    assert torch.equal(fin, x.max(-1, keepdim=True).values)


def test_non_square_causal_mask_is_top_left_aligned():
    x = torch.zeros(1, 3, 7)
    got = torch.ops.loopfuse.causal_mask(x)
    assert torch.equal(got, O.causal_mask_general(x))
    assert got[0, 0, 0] == 0 and got[0, 0, 1] == float("-inf")


_KIND = {"none": S.MASK_NONE, "causal": S.MASK_CAUSAL, "window": S.MASK_CAUSAL_WINDOW}


@pytest.mark.parametrize("mask,window", [("none", 0), ("causal", 0), ("window", 32),
                                         ("window", 130), ("window", 256), ("window", 258),
                                         ("window", 1024), ("window", 5000)])
@pytest.mark.parametrize("s", [17, 129, 512, 593, 2048])
def test_skip_range_equals_brute_force(mask, window, s):
    keep = O.keep_matrix(mask, window, s, s)
    for tq in (64, 128):
        for tk in (64, 128):
            for iq in range(-(-s // tq)):
                want = O.brute_force_skip_range(mask, window, s, s, tq, tk, iq, keep=keep)
                got = S.skip_range(_KIND[mask], window, 0, s, s, tq, tk, iq)
                assert got == want, (mask, window, s, tq, tk, iq)


@pytest.mark.parametrize("sq,skv,off", [(100, 300, 200), (300, 100, 0), (64, 512, 448),
                                        (130, 130, -5)])
def test_skip_range_rectangular_and_offset(sq, skv, off):
    for mask, window in (("causal", 0), ("window", 70)):
        keep = O.keep_matrix(mask, window, sq, skv, off)
        for iq in range(-(-sq // 128)):
            want = O.brute_force_skip_range(mask, window, sq, skv, 128, 128, iq, keep=keep)
            got = S.skip_range(_KIND[mask], window, off, sq, skv, 128, 128, iq)
            assert got == want, (mask, sq, skv, off, iq)


def test_c_abi_skip_range_is_the_same_integers(native_lib):
    from loopfuse_b200._native import c_skip_range
    for kind, window in ((S.MASK_NONE, 0), (S.MASK_CAUSAL, 0), (S.MASK_CAUSAL_WINDOW, 256),
                         (S.MASK_CAUSAL_WINDOW, 130)):
        for s_q, s_kv, off in ((2048, 2048, 0), (593, 593, 0), (100, 300, 200), (130, 130, -5)):
            for tq, tk in ((128, 128), (64, 128)):
                for iq in range(-(-s_q // tq) + 1):   # one tile past the end as well
                    assert c_skip_range(kind, window, off, s_q, s_kv, tq, tk, iq) == \
                        S.skip_range(kind, window, off, s_q, s_kv, tq, tk, iq)


def test_skip_range_vs_reference_generated_bounds(golden_dir):
    """Same integers as the reference compiler's bounds for the benchmark masks (causal,
    window 256) at every tile shape; for window 130 the reference drops a live corner tile at
    some q-tiles (see tests/test_oracle.py), there the brute-force value is used."""
    with open(golden_dir / "skip_ranges.json") as f:
        tabs = json.load(f)["tables"]
    kinds = {"causal": (S.MASK_CAUSAL, 0), "window256": (S.MASK_CAUSAL_WINDOW, 256),
             "causal_of_window256": (S.MASK_CAUSAL_WINDOW, 256), "none": (S.MASK_NONE, 0)}
    checked = 0
    for tab in tabs:
        if tab["mask"] not in kinds:
            continue
        kind, window = kinds[tab["mask"]]
        for iq, (lo, hi) in enumerate(tab["ranges"]):
            got = S.skip_range(kind, window, 0, tab["S"], tab["S"], tab["tile_q"],
                               tab["tile_k"], iq)
            assert got == (lo, hi), (tab, iq)
            checked += 1
    assert checked > 300


def test_live_tile_counts_at_benchmark_shapes():
    # causal S=2048: 136 of 256 tiles at 128x128, 272 of 512 at the kernel's 128x64;
    # window 256: 45 of 256 and 90 of 512
    assert (S.TILE_Q, S.TILE_K) == (128, 64)
    for tk, n_causal, n_window in ((128, 136, 45), (64, 272, 90)):
        causal = S.skip_table(S.MASK_CAUSAL, 0, 0, 2048, 2048, 128, tk)
        window = S.skip_table(S.MASK_CAUSAL_WINDOW, 256, 0, 2048, 2048, 128, tk)
        assert sum(hi - lo for lo, hi in causal) == n_causal
        assert sum(hi - lo for lo, hi in window) == n_window
