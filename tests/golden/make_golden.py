"""Generate the golden fixtures in this folder FROM THE REFERENCE ITSELF.

Run in the build container, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference package (CODEGEN_ONLY mode: no GPU, no Triton launch) and writes
  eager_ops.pt        outputs of the reference's eager custom ops on seeded inputs
  eager_attention.pt  seeded inputs + outputs of small attention functions written like the
                      reference's benchmark/tests and run eagerly in fp32 with its ops
  skip_ranges.json    the loop-bound expressions its compiler generates for causal and
                      sliding-window attention, and those expressions evaluated on a grid of
                      (S, tile_q, tile_k, window) as integer tables
The fixtures are small (a few hundred KB) and are committed; the tests never need the reference.
The reference registers the same ``loopfuse::`` op namespace as loopfuse_b200, so this script
must not import loopfuse_b200.
"""
from __future__ import annotations

import json
import math
import os
import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    os.environ["CODEGEN_ONLY"] = "1"
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    import torch
    from loopfuse import loopfuse_backend  # the reference
    import loopfuse.torch_backend as ref_ops  # noqa: F401
    assert Path(sys.modules["loopfuse"].__file__).resolve().is_relative_to(Path(ref_root).resolve())

    ops = torch.ops.loopfuse

    # ---------------- eager ops ----------------
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(2, 3, 37, 37, generator=g)
    buf = torch.randn(50, 4, 8, generator=g)
    table = torch.randint(0, 50, (3, 7), generator=g, dtype=torch.int32)
    buf4 = torch.randn(12, 4, 2, 8, generator=g)
    table4 = torch.randperm(12, generator=g).view(2, 6).to(torch.int32)
    eager = {
        "x": x,
        "causal_mask": ops.causal_mask(x),
        "sliding_mask_w5": ops.sliding_mask(x, 5),
        "sliding_mask_w64": ops.sliding_mask(x, 64),
        "causal_of_sliding_w5": ops.causal_mask(ops.sliding_mask(x, 5)),
        "buffer": buf, "table": table, "paged_load": ops.paged_load(buf, table.long()),
        "buffer4": buf4, "table4": table4, "paged_load4": ops.paged_load(buf4, table4.long()),
    }
    torch.save(eager, HERE / "eager_ops.pt")

    # ---------------- eager attention functions ----------------
    def causal_fn(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(ops.causal_mask(qk), dim=-1) @ v

    def softcap_fn(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        qk = torch.tanh(qk / 50) * 50
        return torch.softmax(ops.causal_mask(qk), dim=-1) @ v

    def window_gqa_fn(q, k, v):
        hq, hk = q.shape[1], k.shape[1]
        k = k.repeat_interleave(hq // hk, dim=1)
        v = v.repeat_interleave(hq // hk, dim=1)
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        qk = torch.tanh(qk / 50) * 50
        m = ops.causal_mask(ops.sliding_mask(qk, 24))
        return torch.softmax(m, dim=-1) @ v

    def decode_fn(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(qk, dim=-1) @ v

    def paged_fn(q, kc, vc, bt):
        b = q.shape[0]
        k = ops.paged_load(kc, bt)
        v = ops.paged_load(vc, bt)
        k = k.reshape(b, -1, k.shape[-2], k.shape[-1]).transpose(1, 2)
        v = v.reshape(b, -1, v.shape[-2], v.shape[-1]).transpose(1, 2)
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(qk, dim=-1) @ v

    def rn(*shape):
        return torch.randn(*shape, generator=g)

    att = {}
    q, k, v = rn(1, 2, 48, 16), rn(1, 2, 48, 16), rn(1, 2, 48, 16)
    att["causal"] = {"q": q, "k": k, "v": v, "out": causal_fn(q, k, v)}
    # larger scores so that the softcap actually bends them
    q, k, v = 3 * rn(1, 2, 48, 16), 3 * rn(1, 2, 48, 16), rn(1, 2, 48, 16)
    att["causal_softcap50"] = {"q": q, "k": k, "v": v, "out": softcap_fn(q, k, v)}
    q, k, v = 3 * rn(1, 4, 80, 16), 3 * rn(1, 2, 80, 16), rn(1, 2, 80, 16)
    att["window24_gqa_softcap50"] = {"q": q, "k": k, "v": v, "out": window_gqa_fn(q, k, v)}
    q, k, v = rn(2, 2, 1, 16), rn(2, 2, 70, 16), rn(2, 2, 70, 16)
    att["decode"] = {"q": q, "k": k, "v": v, "out": decode_fn(q, k, v)}
    q, kc, vc = rn(2, 2, 4, 16), rn(12, 4, 2, 16), rn(12, 4, 2, 16)
    bt = torch.randperm(12, generator=g).view(2, 6)
    att["paged_gqa_decode_p4"] = {"q": q, "k_pool": kc, "v_pool": vc,
                                  "block_table": bt.to(torch.int32),
                                  "out": paged_fn(q, kc, vc, bt)}
    torch.save(att, HERE / "eager_attention.pt")

    # ---------------- generated loop bounds ----------------
    def compile_and_get_code(fn, *inputs):
        torch._dynamo.reset()
        torch._dynamo.mark_static(inputs[0], 3)
        torch._dynamo.mark_dynamic(inputs[0], 2)
        kd = torch.compile(fn, backend=loopfuse_backend, dynamic=True, mode=None)(*inputs)
        return kd.code

    def bounds(code):
        start = re.search(r"range_start = (.*)", code)
        end = re.search(r"range_end = (.*)", code)
        return (start.group(1).strip() if start else None,
                end.group(1).strip() if end else None)

    # Window sizes are literals: a closure variable would be traced as a symbolic integer.
    def window256_fn(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(ops.sliding_mask(qk, 256), dim=-1) @ v

    def causal_of_window256_fn(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(ops.causal_mask(ops.sliding_mask(qk, 256)), dim=-1) @ v

    def window130_fn(q, k, v):
        qk = q @ k.transpose(-2, -1) * (q.shape[-1] ** -0.5)
        return torch.softmax(ops.sliding_mask(qk, 130), dim=-1) @ v

    qkv = [torch.randn(2, 4, 512, 64) for _ in range(3)]
    exprs = {}
    exprs["causal"] = bounds(compile_and_get_code(causal_fn, *qkv))
    exprs["window256"] = bounds(compile_and_get_code(window256_fn, *qkv))
    exprs["causal_of_window256"] = bounds(compile_and_get_code(causal_of_window256_fn, *qkv))
    exprs["window130"] = bounds(compile_and_get_code(window130_fn, *qkv))
    exprs["none"] = bounds(compile_and_get_code(decode_fn, *qkv))

    def evaluate(expr, iq, tq, tk, s):
        """Evaluate a generated bound like the Triton kernel does: float math, then
        ``.to(tl.int32)`` truncates toward zero."""
        if expr is None:
            return None
        py = expr.replace("tl.maximum", "max").replace("tl.minimum", "min")
        py = py.replace("tl.cdiv", "cdiv").replace(".to(tl.int32)", ".trunc()")
        # variable names follow the user function's parameter names; make them canonical
        py = re.sub(r"index_\d+_[qQ]_dim2", "IQ", py)
        py = re.sub(r"tile_[qQ]_dim2", "TQ", py)
        py = re.sub(r"tile_[kK]_dim2", "TK", py)
        py = re.sub(r"\b[kKqQ]_dim2\b", "SEQ", py)

        class F(float):
            def trunc(self):
                return math.trunc(self)

            def _w(self, r):
                return F(r)

            def __add__(self, o): return F(float(self) + float(o))
            __radd__ = __add__
            def __mul__(self, o): return F(float(self) * float(o))
            __rmul__ = __mul__
            def __sub__(self, o): return F(float(self) - float(o))
            def __rsub__(self, o): return F(float(o) - float(self))
            def __truediv__(self, o): return F(float(self) / float(o))
            def __rtruediv__(self, o): return F(float(o) / float(self))
            def __neg__(self): return F(-float(self))

        env = {"max": max, "min": min, "cdiv": lambda a, b: -(-int(a) // int(b)),
               "IQ": F(iq), "TQ": F(tq), "TK": F(tk), "SEQ": s}
        return int(eval(py, {"__builtins__": {}}, env))

    tables = []
    for name, (e_lo, e_hi) in exprs.items():
        for s in (512, 593, 2048):
            for tq, tk in ((128, 128), (64, 64), (128, 64), (64, 128)):
                n_qt = -(-s // tq)
                rows = []
                for iq in range(n_qt):
                    lo = evaluate(e_lo, iq, tq, tk, s) if e_lo else 0
                    hi = evaluate(e_hi, iq, tq, tk, s) if e_hi else -(-s // tk)
                    rows.append([lo, hi])
                tables.append({"mask": name, "S": s, "tile_q": tq, "tile_k": tk, "ranges": rows})
    with open(HERE / "skip_ranges.json", "w") as f:
        json.dump({"expressions": {k: list(v) for k, v in exprs.items()}, "tables": tables}, f)
    print("expressions:")
    for k_, v_ in exprs.items():
        print(" ", k_, v_)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path to a checkout of tomatillos/loopfuse>")
    main(sys.argv[1])
