"""Seeded random sweeps of shapes through the C ABI against the CPU oracle: window masks with
two / four grouped heads (the packed layout), ragged sizes, Sq != Skv with a causal offset, rows
without any visible key (NaN, as in the eager computation), plain and softcap scores, dense and
paged decode with forced split counts, the two-product scores. The fixed cases of the other test
files cover the benchmark geometries; these cover the corners between them."""
import random

import pytest
import torch

from loopfuse_b200 import functional as F, spec as S
from loopfuse_b200.spec import ScoreMod
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
SOFTCAP = [ScoreMod(S.MOD_DIV, 50.0), ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_MUL, 50.0)]


def _close_with_nan(out, want):
    out = out.float().cpu()
    if not torch.equal(torch.isnan(out), torch.isnan(want)):
        return False
    m = ~torch.isnan(want)
    return (not m.any()) or (out[m] - want[m]).abs().max().item() <= TOL


def test_random_prefill_shapes():
    rnd = random.Random(7)
    g = torch.Generator().manual_seed(7)
    st = F.new_status("cuda")
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    for _ in range(40):
        D, G, Hkv, B = rnd.choice([64, 128]), rnd.choice([1, 2, 4]), rnd.choice([1, 2, 3]), rnd.choice([1, 2])
        Sq = rnd.choice([1, 17, 31, 32, 33, 64, 100, 129, 257, 400, 777])
        Skv = Sq + rnd.choice([0, 0, 5, 64, 130])
        mask = rnd.choice(["window", "window", "causal", "none"])
        W = rnd.choice([1, 7, 32, 64, 100, 256, 1000])
        softcap = rnd.random() < 0.7
        q, k, v = mk(B, Hkv * G, Sq, D), mk(B, Hkv, Skv, D), mk(B, Hkv, Skv, D)
        kind = {"window": S.MASK_CAUSAL_WINDOW, "causal": S.MASK_CAUSAL, "none": S.MASK_NONE}[mask]
        out = F.prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5,
                                  mods=SOFTCAP if softcap else [], mask_kind=kind, window=W,
                                  causal_offset=Skv - Sq, status=st)
        want = O.attention_ref(q, k, v, mods=O.softcap_mods(50.0) if softcap else [], mask=mask,
                               window=W, offset=Skv - Sq, batch_chunk=B)
        assert _close_with_nan(out, want), dict(D=D, G=G, Hkv=Hkv, B=B, Sq=Sq, Skv=Skv, W=W,
                                                mask=mask, softcap=softcap)
    F.check_status(st)


def test_random_decode_shapes():
    rnd = random.Random(11)
    g = torch.Generator().manual_seed(11)
    st = F.new_status("cuda")
    ws = F.DecodeWorkspace()
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    for _ in range(30):
        D, G, Hkv, B = rnd.choice([64, 128]), rnd.choice([1, 2, 4, 8]), rnd.choice([1, 3, 8]), rnd.choice([1, 2, 5])
        Skv = rnd.choice([1, 15, 16, 17, 100, 1000, 4097])
        splits = rnd.choice([0, 0, 1, 2, 5])
        q = mk(B, Hkv, G, D)
        if rnd.random() < 0.5:
            k, v = mk(B, Hkv, Skv, D), mk(B, Hkv, Skv, D)
            out = F.decode_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5, splits=splits,
                                     workspace=ws, status=st)
            want = O.attention_ref(q, k, v, batch_chunk=8)
        else:
            P = rnd.choice([1, 4, 16, 24])
            blocks = -(-Skv // P)
            n_pages = B * blocks + 2
            kp, vp = mk(n_pages, P, Hkv, D), mk(n_pages, P, Hkv, D)
            table = torch.randperm(n_pages, generator=g)[:B * blocks].view(B, blocks).int()
            out = F.paged_decode_attention(q.cuda(), kp.cuda(), vp.cuda(), table.cuda(),
                                           seq_len=Skv, scale=D ** -0.5, splits=splits,
                                           workspace=ws, status=st)
            want = O.attention_ref(q, O.paged_kv_ref(kp, table)[:, :, :Skv],
                                   O.paged_kv_ref(vp, table)[:, :, :Skv], batch_chunk=8)
        assert (out.float().cpu() - want).abs().max().item() <= TOL, (D, G, Hkv, B, Skv, splits)
    F.check_status(st)


def test_random_two_product_shapes():
    rnd = random.Random(13)
    g = torch.Generator().manual_seed(13)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    for _ in range(10):
        D, Dpe, H = rnd.choice([64, 128]), rnd.choice([8, 16, 32, 64]), rnd.choice([1, 3])
        Sq = rnd.choice([5, 128, 200, 513])
        Skv = Sq + rnd.choice([0, 40])
        q, qp = mk(1, H, Sq, D), mk(1, H, Sq, Dpe)
        k, kp, v = mk(1, H, Skv, D), mk(1, H, Skv, Dpe), mk(1, H, Skv, D)
        out = F.prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=(D + Dpe) ** -0.5,
                                  q_pe=qp.cuda(), k_pe=kp.cuda())
        want = O.mla_attention_ref(q, qp, k, kp, v, mask="none")
        assert (out.float().cpu() - want).abs().max().item() <= TOL, (D, Dpe, H, Sq, Skv)
