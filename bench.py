#!/usr/bin/env python
"""Benchmark of the fused-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the hot path over one batch of synthetic input. The headline workload
(N=1) is "causal_softcap": causal + logit-softcap prefill, B=8 H=32 S=2048 D=128, bf16, reported
as TFLOP/s with the causal-adjusted FLOP count of the reference's benchmark
(tests/benchmark.py:110,186). For N>1 (launched by torchrun, one rank per GPU) every rank owns
its own batch of 8 sequences ((batch x kv-head) units are independent, so scaling is "weak"),
runs the K steps without any collective and the output slabs are gathered with ONE NCCL
all-gather at the end, inside the timed region.

One JSON line is printed by rank 0. Besides the contract keys it carries
  roofline      achieved vs measured peak of the dominant kernel (CUDA-event timed here)
  cpu_baseline  the eager fp32 CPU computation of the same functions, timed on a bounded sample
  e2e           the same metric through torch.compile(fn, backend=loopfuse_backend) with host
                buffers: H2D of q, k, v and D2H of the output inside the timed region
  others        kernel-only figures for the other benchmark configurations (decode in GB/s)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "prefill TFLOP/s (causal-adjusted FLOPs) per job; decode HBM GB/s under `others`"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one full-size launch of each
# workload's dominant kernel, from the ncu captures summarised under profiles/: captured on a
# smaller batch and scaled by the batch ratio (the traffic is proportional to the batch).
NCU_TRAFFIC_BYTES = {
    "causal_softcap": 4 * (100.74e6 + 15.15e6),
    "window_gqa_softcap": 2 * (100.74e6 + 36.01e6),
    "decode": 8 * (268.51e6 + 4.59e6),
    "paged_decode_gqa": 2 * (268.79e6 + 4.74e6),
}


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"])}, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: clocks are reported as unknown
            self._nv = None

    def _poll(self):
        nv = self._nv
        names = {
            nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(0.001)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


# --------------------------------------------------------------------------------------------
# CPU arm: the eager fp32 computation (oracle port of the reference's eager path)
# --------------------------------------------------------------------------------------------
def cpu_sample(workload):
    """Bounded sample of a workload for the CPU arm. The eager fp32 computation of the headline
    prefill configuration takes a few seconds on a multi-core host, so the sample is the whole
    configuration there; decode samples 16 sequences (KV upcast to fp32 costs memory)."""
    import dataclasses
    if workload.kind == "prefill":
        return workload
    return dataclasses.replace(workload, B=min(workload.B, 16))


def time_cpu(workload, steps: int, warmup: int) -> dict:
    """Time the eager fp32 CPU computation on a bounded sample with all host threads."""
    from loopfuse_b200.variants import make_inputs
    from oracle import attention_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    sample = cpu_sample(workload)
    inputs = make_inputs(sample)
    for _ in range(warmup):
        O.workload_ref(sample, inputs)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.workload_ref(sample, inputs)
        times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    if workload.kind == "prefill":
        value, unit = sample.flops() / dt / 1e12, "TFLOP/s"
    else:
        value, unit = sample.kv_bytes() / dt / 1e9, "GB/s"
    return {"value": value, "unit": unit, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample.kind} B={sample.B} Hq={sample.Hq} Hkv={sample.Hkv} S={sample.S} "
                      f"D={sample.D}, eager fp32, {steps} timed passes of {dt * 1e3:.0f} ms",
            "ms_per_step": dt * 1e3}


def run_reference_arm(args, workload) -> None:
    """`--impl reference`: the reference's own CPU implementation of the path (its eager fp32
    functions, restated in oracle/) on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps = max(1, min(args.steps, 5))
    warmup = max(1, min(args.warmup, 2))
    r = time_cpu(workload, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": r["unit"],
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload.name, "sample": r["sample"]},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": r["unit"], "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def make_runner(workload, inputs):
    """Closure that launches the workload's kernel(s) once through the C ABI; returns
    (fn, launches_per_call, out)."""
    from loopfuse_b200 import functional as F, spec as S
    from loopfuse_b200.spec import ScoreMod
    w = workload
    scale = w.D ** -0.5
    if w.kind == "prefill":
        q, k, v = inputs
        mods = ([ScoreMod(S.MOD_DIV, w.softcap), ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_MUL, w.softcap)]
                if w.softcap else [])
        kind = S.MASK_CAUSAL_WINDOW if w.window else S.MASK_CAUSAL
        out = torch.empty_like(q)

        def fn():
            F.prefill_attention(q, k, v, scale=scale, mods=mods, mask_kind=kind, window=w.window,
                                out=out)
        return fn, 1, out
    ws = F.DecodeWorkspace()
    if w.kind == "decode":
        q, k, v = inputs
        q4 = q.view(w.B, w.Hkv, w.group, w.D)
        out = torch.empty_like(q4)

        def fn():
            F.decode_attention(q4, k, v, scale=scale, out=out, workspace=ws)
    else:
        q, kp, vp, table = inputs
        out = torch.empty_like(q)

        def fn():
            F.paged_decode_attention(q, kp, vp, table, scale=scale, out=out, workspace=ws)
    from loopfuse_b200 import _native
    splits = _native.load().lf_decode_auto_splits(
        w.B, w.Hkv, w.group, w.S, w.D, w.page_size if w.kind == "paged_decode" else 0)
    return fn, (2 if splits > 1 else 1), out


def time_kernel(fn, steps: int, warmup: int) -> float:
    """Average milliseconds per call, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / steps


def run_ours(args, workload) -> None:
    import torch.distributed as dist
    from loopfuse_b200 import loopfuse_backend
    from loopfuse_b200.variants import WORKLOADS, make_inputs
    from loopfuse_b200.sharding import gather_output

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks, peak_kind = load_peaks()
    w = workload

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Two alternating input sets (1 GiB working set per pair of steps, far above the 126 MB L2),
    # resident in HBM before the timed region. Rank r owns sequences [r*B, (r+1)*B).
    sets = [tuple(t.to(dev) for t in make_inputs(w, seed=s, batch_offset=rank * w.B))
            for s in (0, 1)]
    runners = [make_runner(w, s) for s in sets]
    launches_per_call = runners[0][1]
    gathered = None
    if world > 1:
        gathered = torch.empty((world * w.B, *runners[0][2].shape[1:]), dtype=torch.bfloat16,
                               device=dev)

    align_token = torch.zeros(1, device=dev)
    for i in range(max(args.warmup, 3)):
        runners[i % 2][0]()
    if world > 1:
        dist.all_reduce(align_token)
        gather_output(runners[0][2], tuple(gathered.shape), out=gathered)
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev_compute_end = torch.cuda.Event(enable_timing=True)
    with sampler:
        if world > 1:
            # The host-side barrier above lets the ranks' CPUs leave milliseconds apart; a tiny
            # all-reduce enqueued ahead of the start event lines the GPU timelines up instead, so
            # that the one collective at the end does not wait for a rank whose host was late.
            dist.all_reduce(align_token)
        start.record()
        for i in range(args.steps):
            runners[i % 2][0]()
        ev_compute_end.record()
        if world > 1:   # the single collective of the path: gather the output slabs
            gather_output(runners[(args.steps - 1) % 2][2], tuple(gathered.shape), out=gathered)
        end.record()
        barrier()
    total_ms = start.elapsed_time(end)
    compute_ms = start.elapsed_time(ev_compute_end)
    t = torch.tensor([total_ms, compute_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, compute_ms = t.tolist()
    ms_per_step = total_ms / args.steps
    kernel_ms = compute_ms / args.steps
    if w.kind == "prefill":
        per_rank_work, unit, peak = w.flops() / 1e12, "TFLOP/s", peaks["bf16_tflops"]
        bound, roof_unit = "tensor", "TFLOP/s"
    else:
        per_rank_work, unit, peak = w.kv_bytes() / 1e9, "GB/s", peaks["hbm_gbs"]
        bound, roof_unit = "hbm", "GB/s"
    value = world * per_rank_work / (ms_per_step * 1e-3)
    achieved = per_rank_work / (kernel_ms * 1e-3)

    # ---- end to end through the public API: torch.compile(fn, backend=loopfuse_backend) with
    # pinned host buffers; H2D of the inputs and D2H of the output are inside the timed region.
    host_in = [t.cpu().pin_memory() for t in sets[0]]
    host_out = torch.empty(runners[0][2].shape if w.kind != "decode" else (w.B, w.Hq, 1, w.D),
                           dtype=torch.bfloat16).pin_memory()
    torch._dynamo.reset()
    compiled = torch.compile(w.fn(), backend=loopfuse_backend, dynamic=True)

    # Three streams, two buffer sets: the H2D copy of step i+1 and the D2H copy of step i-1
    # overlap the kernel of step i (PCIe is full duplex). Every step still copies its own inputs
    # in and its own result out inside the timed region.
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [[torch.empty_like(t, device=dev) for t in host_in] for _ in range(2)]
    host_outs = [host_out, torch.empty_like(host_out).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(n):
        for i in range(n):
            k = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_done[k])      # the kernel of step i-2 has read buffer k
                for d, h_ in zip(dev_in[k], host_in):
                    d.copy_(h_, non_blocking=True)
                ev_in[k].record(s_in)
            cur.wait_event(ev_in[k])
            out = compiled(*dev_in[k])
            ev_done[k].record(cur)
            out.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                if i >= 2:
                    s_out.wait_event(ev_out[k])
                host_outs[k].copy_(out.view(host_out.shape), non_blocking=True)
                ev_out[k].record(s_out)
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)

    cur.wait_stream(torch.cuda.current_stream(dev))
    e2e_run(3)
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    e2e_run(e2e_steps)
    e2.record()
    barrier()
    t = torch.tensor([s2.elapsed_time(e2)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = t.item() / e2e_steps
    e2e = {"value": world * per_rank_work / (e2e_ms * 1e-3), "unit": unit,
           "h2d_bytes_per_step": world * sum(t.numel() * t.element_size() for t in host_in),
           "d2h_bytes_per_step": world * host_out.numel() * host_out.element_size(),
           "ms_per_step": e2e_ms, "steps": e2e_steps}

    # ---- the other benchmark configurations, kernel-only, for context (rank 0, N=1 only)
    others = {}
    cpu = None
    if rank == 0 and world == 1 and not args.no_others:
        del sets, runners
        torch.cuda.empty_cache()
        for name, ow in WORKLOADS.items():
            if name == w.name:
                continue
            osets = [tuple(t.to(dev) for t in make_inputs(ow, seed=s)) for s in (0, 1)]
            orun = [make_runner(ow, s) for s in osets]
            calls = {"i": 0}

            def alt():
                orun[calls["i"] % 2][0]()
                calls["i"] += 1
            ms = time_kernel(alt, 20, 5)
            if ow.kind == "prefill":
                val, u, pk = ow.flops() / 1e12 / (ms * 1e-3), "TFLOP/s", peaks["bf16_tflops"]
            else:
                val, u, pk = ow.kv_bytes() / 1e9 / (ms * 1e-3), "GB/s", peaks["hbm_gbs"]
            others[name] = {"value": val, "unit": u, "ms": ms, "frac_of_peak": val / pk,
                            "peak": pk}
            del osets, orun
            torch.cuda.empty_cache()
        cpu = time_cpu(w, steps=2, warmup=1)
        cpu.pop("ms_per_step", None)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w.name, "kind": w.kind, "B_per_gpu": w.B, "Hq": w.Hq,
                       "Hkv": w.Hkv, "S": w.S, "D": w.D, "softcap": w.softcap, "window": w.window,
                       "page_size": w.page_size, "parallelism": f"units(batch x kv-head) x{world}",
                       "l2": "two alternating input sets, 1 GiB touched per pair of steps "
                             "(L2 is 126 MB); no explicit flush",
                       "collective": "one all-gather of the output slabs at the end of the timed "
                                     "region" if world > 1 else "none"},
            "clocks": sampler.summary(),
            "e2e": e2e,
            "gpu_launches": args.steps * launches_per_call,
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": roof_unit,
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(w.name),
                         "peak_source": f"{peak_kind} (burst figure: kernel timed alone)",
                         "kernel_ms": kernel_ms},
            "others": others,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if world > 1:
            line["gather_ms"] = total_ms - compute_ms
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="causal_softcap")
    ap.add_argument("--no-others", action="store_true",
                    help="skip the context figures for the other configurations")
    args = ap.parse_args()
    from loopfuse_b200.variants import WORKLOADS
    workload = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, workload)
    else:
        run_ours(args, workload)


if __name__ == "__main__":
    main()
