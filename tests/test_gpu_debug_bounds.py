"""The range-checking build (liblf_sm100_dbg.so, -DLF_DEBUG_BOUNDS) on small ragged shapes.

compute-sanitizer cannot be used where these kernels are developed, so the library can be built
with every plain global index compared against its range before use; a violation is written to
the status word (LF_DEV_BOUNDS) and the access is clamped or skipped. The library is chosen when
it is loaded, so the cases run in a child process with LF_DEBUG_BOUNDS=1: ragged sizes in the
style of the reference's tests (S = 17, 129, 593; tests/test_accuracy.py:127), results against
the CPU oracle, status word zero.
"""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent("""
    import sys, torch
    sys.path.insert(0, %r)
    from loopfuse_b200 import _native, functional as F, spec as SP
    from oracle import attention_oracle as O
    assert _native.load().lf_debug_bounds() == 1
    TOL = 2e-2
    g = torch.Generator().manual_seed(21)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    st = F.new_status("cuda")
    for S in (17, 129, 593):
        for G in (1, 4):
            q, k, v = mk(2, 3, G, 128), mk(2, 3, S, 128), mk(2, 3, S, 128)
            for splits in (0, 3):
                out = F.decode_attention(q.cuda(), k.cuda(), v.cuda(), scale=128 ** -0.5,
                                         splits=splits, status=st)
                want = O.attention_ref(q, k, v, batch_chunk=8)
                assert (out.float().cpu() - want).abs().max().item() <= TOL, (S, G, splits)
        for P in (1, 16):
            blocks = -(-S // P)
            n_pages = 2 * blocks + 3
            kp, vp = mk(n_pages, P, 3, 64), mk(n_pages, P, 3, 64)
            table = torch.randperm(n_pages, generator=g)[:2 * blocks].view(2, blocks).int()  # disjoint pages
            q = mk(2, 3, 4, 64)
            out = F.paged_decode_attention(q.cuda(), kp.cuda(), vp.cuda(), table.cuda(), seq_len=S,
                                           scale=64 ** -0.5, status=st)
            kk = O.paged_kv_ref(kp, table)[:, :, :S]
            vv = O.paged_kv_ref(vp, table)[:, :, :S]
            want = O.attention_ref(q, kk, vv, batch_chunk=8)
            assert (out.float().cpu() - want).abs().max().item() <= TOL, (S, P)
            new = mk(2, 3, 5, 64)
            pos = [0, min(3, S - 5)] if S >= 8 else [0, 0]
            T = min(5, S)
            kpd, vpd = kp.cuda(), vp.cuda()
            F.kv_append(new[:, :, :T].cuda(), new[:, :, :T].cuda(), kpd, vpd, table.cuda(),
                        seq_pos=torch.tensor(pos, dtype=torch.int32).cuda(), status=st)
            wantp = O.kv_append_ref(kp, new[:, :, :T], table, pos)
            assert torch.equal(kpd.cpu(), wantp), (S, P)
        q, k, v = mk(1, 2, S, 64), mk(1, 2, S, 64), mk(1, 2, S, 64)
        S8 = -(-S // 8) * 8
        sb_full = mk(1, 2, S, S8)   # rows padded to 16 bytes; the kernel sees the [.., :S] view
        sb = sb_full[..., :S]
        out = F.prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=0.125, mask_kind=SP.MASK_CAUSAL,
                                  score_bias=sb_full.cuda()[..., :S], status=st)
        s = O.causal_mask_general(q.float() @ k.float().transpose(-2, -1) * 0.125 + sb.float())
        want = torch.softmax(s, dim=-1) @ v.float()
        assert (out.float().cpu() - want).abs().max().item() <= TOL, S
    torch.cuda.synchronize()
    assert int(st.item()) == 0, hex(int(st.item()))
    print("debug-bounds cases ok")
""") % str(ROOT)


@pytest.mark.gpu
def test_range_checking_build_runs_clean_on_ragged_shapes():
    env = dict(os.environ, LF_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "debug-bounds cases ok" in r.stdout


def test_range_checking_library_exports_the_same_abi():
    import ctypes as C
    from loopfuse_b200 import _native
    from loopfuse_b200.build import build_native
    dbg = C.CDLL(str(build_native(debug_bounds=True)))
    assert all(hasattr(dbg, n) for n in _native.EXPORTS)
    dbg.lf_debug_bounds.restype = C.c_int
    assert dbg.lf_debug_bounds() == 1
    assert _native.load().lf_debug_bounds() == (1 if os.environ.get("LF_DEBUG_BOUNDS", "0") not in ("", "0") else 0)
