"""Run a few launches of one benchmark workload through the C ABI - the command line that
profilers (ncu) wrap. Usage:

    python -m loopfuse_b200.profile_case --workload causal_softcap --batch 2 --launches 3

``--batch`` shrinks the workload so that a multi-pass capture stays small; keep the tensors
above the 126 MB L2 when DRAM figures matter.
"""
from __future__ import annotations

import argparse
import dataclasses

import torch

from .variants import WORKLOADS, make_inputs


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="causal_softcap", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="0 = the workload's own batch")
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from bench import make_runner  # the same launch closures the benchmark times

    w = WORKLOADS[args.workload]
    if args.batch:
        w = dataclasses.replace(w, B=args.batch)
    inputs = tuple(t.cuda() for t in make_inputs(w))
    fn, launches_per_call, out = make_runner(w, inputs)
    for _ in range(args.launches):
        fn()
    torch.cuda.synchronize()
    print(f"{w.name}: B={w.B} {args.launches} calls x {launches_per_call} kernel(s), "
          f"out mean {out.float().mean().item():.6f}")


if __name__ == "__main__":
    main()
