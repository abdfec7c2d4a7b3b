#!/usr/bin/env python
"""Benchmark of the fused-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--batch B] [--no-others] [--kernel-only]

A step is one pass of the hot path over one batch of synthetic input. The headline workload is
"causal_softcap": causal + logit-softcap prefill, B=8 H=32 S=2048 D=128, bf16, reported as
TFLOP/s with the causal-adjusted FLOP count of the reference's benchmark
(tests/benchmark.py:110,186). `--batch` shrinks the batch (profiling captures of a small case).

N > 1 (launched by torchrun, one rank per GPU, NCCL): (batch x kv-head) units are independent, so
every rank owns its own batch of 8 sequences ("weak" scaling) and computes with no collective in
the data path; `value` is the units of all ranks over the max-over-ranks time of K steps of that
sharded compute, and does not depend on K. What it costs to also replicate every step's output
on every rank is measured next to it and kept out of `value`: one NCCL all-gather of the output
slabs per step on a second stream (`with_gather_every_step`, the gather alone, its bus
bandwidth), the gathered tensor verified against the ranks' own slabs. The strong-scaling view
(one batch of 8 split over the ranks) is reported under `strong_scaling`.

One JSON line is printed by rank 0. Besides the contract keys it carries
  roofline      achieved vs measured peak of the dominant kernel (CUDA-event timed here)
  cpu_baseline  the eager fp32 CPU computation of the same function, timed on a bounded sample
  e2e           the same metric through torch.compile(fn, backend=loopfuse_backend) with pinned
                host buffers: H2D of the inputs and D2H of the output inside the timed region,
                with the measured pinned-copy ceiling of this host next to it
  sustained     the headline kernel launched back to back for >= 2 s, with the median SM clock
  worst_case    the headline kernel on inputs whose scores need the MUFU tanh in every block
  others        the other benchmark configurations (decode and paged decode in GB/s), each with
                its own roofline, e2e and cpu_baseline; at N > 1 every rank runs its own batch
"""
from __future__ import annotations

import argparse
import dataclasses
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
# workload's dominant kernel, from ncu captures of a smaller batch scaled by the batch ratio (the
# traffic is proportional to the batch).
NCU_TRAFFIC_BYTES = {
    "causal_softcap": 4 * (108.67e6 + 14.64e6),
    "window_gqa_softcap": 2 * (100.74e6 + 30.84e6),
    "decode": 8 * (268.51e6 + 4.03e6),
    "paged_decode_gqa": 2 * (268.79e6 + 5.29e6),
}
FULL_BATCH: dict = {}   # workload name -> batch of the benchmark configuration


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


def bind_to_gpu_numa_node(gpu_index: int) -> dict:
    """Pin this process (and so the pinned host buffers it first touches, and its copy-issuing
    thread) to the CPUs of the NUMA node the GPU hangs off. Only reads GPU properties."""
    info: dict = {"numa_node": None, "cpus": None}
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        dom, rest = bus.split(":", 1)   # sysfs uses a 4-digit domain, NVML an 8-digit one
        node = int(Path(f"/sys/bus/pci/devices/{dom[-4:].lower()}:{rest.lower()}/numa_node")
                   .read_text())
        if node < 0:
            return info
        cpulist = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
        cpus: set[int] = set()
        for part in cpulist.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            info = {"numa_node": node, "cpus": len(allowed)}
    except Exception as e:  # no sysfs / NVML: leave the affinity as it is
        info["error"] = type(e).__name__
    return info


def workload_config(w, world: int, extra: dict | None = None) -> dict:
    cfg = {"workload": w.name, "kind": w.kind, "B_per_gpu": w.B, "Hq": w.Hq, "Hkv": w.Hkv,
           "S": w.S, "D": w.D, "softcap": w.softcap, "window": w.window,
           "page_size": w.page_size, "parallelism": f"units(batch x kv-head) x{world}"}
    if extra:
        cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------------------------
# CPU arm: the eager fp32 computation (oracle port of the reference's eager path)
# --------------------------------------------------------------------------------------------
def cpu_sample(workload, small: bool):
    """Bounded sample of a workload for the CPU arm (throughput does not depend on the batch):
    prefill 2 sequences (the whole configuration for the tiny one), decode 16 sequences (the KV
    upcast to fp32 costs memory); `small` halves that for runs with many steps."""
    if workload.kind == "prefill":
        b = workload.B if workload.B <= 2 else (1 if small else 2)
    else:
        b = min(workload.B, 8 if small else 16)
    return dataclasses.replace(workload, B=b)


def time_cpu(workload, steps: int, warmup: int, small: bool = False) -> dict:
    """Time the eager fp32 CPU computation on a bounded sample with all host threads."""
    from loopfuse_b200.variants import make_inputs
    from oracle import attention_oracle as O
    torch.set_num_threads(len(os.sched_getaffinity(0)) or os.cpu_count() or 1)
    sample = cpu_sample(workload, small)
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
            "sample": f"{sample.kind} B={sample.B} of {workload.B} Hq={sample.Hq} Hkv={sample.Hkv} "
                      f"S={sample.S} D={sample.D}, eager fp32, {steps} timed passes of "
                      f"{dt * 1e3:.0f} ms",
            "ms_per_step": dt * 1e3}


def run_reference_arm(args, workload) -> None:
    """`--impl reference`: the reference's own CPU implementation of the path (its eager fp32
    functions, restated in oracle/) on the host cores; rank 0 only. Honours --steps/--warmup;
    every step is one pass over a bounded sample of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    r = time_cpu(workload, steps, warmup, small=steps > 10)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": r["unit"],
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(workload, args.gpus),
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": r["unit"], "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def softcap_mods(w):
    from loopfuse_b200 import spec as S
    from loopfuse_b200.spec import ScoreMod
    if not w.softcap:
        return []
    return [ScoreMod(S.MOD_DIV, w.softcap), ScoreMod(S.MOD_TANH), ScoreMod(S.MOD_MUL, w.softcap)]


class Runner:
    """Launches one workload once per call through the C ABI on fixed device buffers."""

    def __init__(self, w, inputs, q_scale: float = 1.0, sm_margin: int = 0):
        from loopfuse_b200 import _native, functional as F, spec as S
        self.w = w
        scale = w.D ** -0.5
        if w.kind == "prefill":
            q, k, v = inputs
            if q_scale != 1.0:
                q = (q.float() * q_scale).to(q.dtype)
            kind = S.MASK_CAUSAL_WINDOW if w.window else S.MASK_CAUSAL
            self.out = torch.empty_like(q)
            prep = F.PreparedPrefill(q, k, v, scale=scale, mods=softcap_mods(w), mask_kind=kind,
                                     window=w.window, out=self.out, sm_margin=sm_margin)
            self.launch = prep.run
            self.launches_per_call = 1
            return
        ws = F.DecodeWorkspace()
        if w.kind == "decode":
            q, k, v = inputs
            q4 = q.view(w.B, w.Hkv, w.group, w.D)
            self.out = out = torch.empty_like(q4)
            self.launch = lambda: F.decode_attention(q4, k, v, scale=scale, out=out, workspace=ws)
            page = 0
        else:
            q, kp, vp, table = inputs
            self.out = out = torch.empty_like(q)
            self.launch = lambda: F.paged_decode_attention(q, kp, vp, table, scale=scale, out=out,
                                                           workspace=ws)
            page = w.page_size
        splits = _native.load().lf_decode_auto_splits(w.B, w.Hkv, w.group, w.S, w.D, page)
        self.launches_per_call = 2 if splits > 1 else 1


def events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_runners(runners, steps: int, warmup: int) -> float:
    """Average milliseconds per step over `steps` launches that alternate between the runners
    (two input sets: far more than the 126 MB L2 is touched per pair of steps)."""
    for i in range(warmup):
        runners[i % len(runners)].launch()
    torch.cuda.synchronize()
    start, end = events()
    start.record()
    for i in range(steps):
        runners[i % len(runners)].launch()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / steps


def work_of(w) -> tuple[float, str, str]:
    """(algorithmic work of one step in T- or G-units, value unit, roofline bound)."""
    if w.kind == "prefill":
        return w.flops() / 1e12, "TFLOP/s", "tensor"
    return w.kv_bytes() / 1e9, "GB/s", "hbm"


def roofline_of(w, ms: float, peaks: dict, peak_kind: str) -> dict:
    work, unit, bound = work_of(w)
    achieved = work / (ms * 1e-3)
    peak = peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"]
    traffic = NCU_TRAFFIC_BYTES.get(w.name)
    if traffic:
        traffic *= w.B / FULL_BATCH.get(w.name, w.B)
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
            "frac": achieved / peak, "traffic": traffic,
            "peak_source": f"{peak_kind} (burst figure: kernel timed alone)", "kernel_ms": ms}


def max_over_ranks(values: list, dev, world: int) -> list:
    if world == 1:
        return values
    import torch.distributed as dist
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def copy_ceiling(dev, nbytes: int = 256 << 20) -> dict:
    """Plain pinned-memory copies between this host and this GPU, one cudaMemcpyAsync per
    direction, both directions at once (what the end-to-end loop does): GB/s per direction."""
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    seen: list = [[], []]
    for _ in range(5):
        torch.cuda.synchronize()
        a1, b1 = events()
        a2, b2 = events()
        with torch.cuda.stream(s1):
            a1.record()
            d_in.copy_(h_in, non_blocking=True)
            b1.record()
        with torch.cuda.stream(s2):
            a2.record()
            h_out.copy_(d_out, non_blocking=True)
            b2.record()
        torch.cuda.synchronize()
        seen[0].append(nbytes / 1e9 / (a1.elapsed_time(b1) * 1e-3))
        seen[1].append(nbytes / 1e9 / (a2.elapsed_time(b2) * 1e-3))
    # the median of five: other tenants of the host's memory and PCIe switches come and go, and
    # the best of a few tries would describe a quieter machine than the end-to-end loop sees
    best = [sorted(x)[len(x) // 2] for x in seen]
    return {"h2d_gbs": best[0], "d2h_gbs": best[1]}


def time_e2e(w, host_inputs, dev, steps: int, barrier) -> dict:
    """The workload through torch.compile(fn, backend=loopfuse_backend) with pinned host buffers.
    Three streams, two buffer sets: the H2D copy of step i+1 and the D2H copy of step i-1 overlap
    the kernel of step i (PCIe is full duplex). Every step still copies its own inputs in and
    its own result out inside the timed region."""
    from loopfuse_b200 import loopfuse_backend
    host_in = [t.pin_memory() for t in host_inputs]
    torch._dynamo.reset()
    compiled = torch.compile(w.fn(), backend=loopfuse_backend, dynamic=True)
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [[torch.empty_like(t, device=dev) for t in host_in] for _ in range(2)]
    host_outs: list = [None, None]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def run(n):
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
            if host_outs[k] is None:
                host_outs[k] = torch.empty(out.shape, dtype=out.dtype).pin_memory()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                if i >= 2:
                    s_out.wait_event(ev_out[k])
                host_outs[k].copy_(out, non_blocking=True)
                ev_out[k].record(s_out)
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)

    run(3)
    barrier()
    s2, e2 = events()
    s2.record()
    run(steps)
    e2.record()
    barrier()
    return {"ms": s2.elapsed_time(e2) / steps, "steps": steps,
            "h2d_bytes": sum(t.numel() * t.element_size() for t in host_in),
            "d2h_bytes": host_outs[0].numel() * host_outs[0].element_size()}


def run_ours(args, workload) -> None:
    import torch.distributed as dist
    from loopfuse_b200.variants import WORKLOADS, make_inputs
    from loopfuse_b200 import sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    affinity = bind_to_gpu_numa_node(physical_gpu_index(local_rank))
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks, peak_kind = load_peaks()
    for name, ww in WORKLOADS.items():
        FULL_BATCH[name] = ww.B
    w = workload
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Two alternating input sets, resident in HBM before any timed region. Rank r owns
    # sequences [r*B, (r+1)*B).
    host_sets = [make_inputs(w, seed=s, batch_offset=rank * w.B) for s in (0, 1)]
    sets = [tuple(t.to(dev) for t in hs) for hs in host_sets]
    runners = [Runner(w, s) for s in sets]
    work, unit, _ = work_of(w)

    # ---- kernel only: K steps, no collective; max over ranks
    align_token = torch.zeros(1, device=dev)
    for i in range(warmup):
        runners[i % 2].launch()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    start, end = events()
    with sampler:
        if world > 1:
            # The host-side barrier lets the ranks' CPUs leave milliseconds apart; a tiny
            # all-reduce enqueued ahead of the start event lines the GPU timelines up instead.
            dist.all_reduce(align_token)
        start.record()
        for i in range(steps):
            runners[i % 2].launch()
        end.record()
        barrier()
    kernel_ms = max_over_ranks([start.elapsed_time(end) / steps], dev, world)[0]
    launches = steps * runners[0].launches_per_call

    line: dict = {}
    ms_per_step = kernel_ms
    collective = "none"
    if world > 1 and not args.kernel_only:
        # ---- not part of `value`: what it costs to ALSO replicate every step's output on every
        # rank - an all-gather of the output slabs once per step on a second stream, the gather
        # of step i next to the kernel of step i+1. The path itself has no exchange step (the
        # (batch x kv-head) units are independent and a consumer of sharded attention output,
        # e.g. the output projection under tensor parallelism, reads the local slab), so `value`
        # is the rate of the sharded compute; these keys say what a caller who wants the full
        # tensor everywhere pays on top.
        # (With one CTA of the persistent prefill kernel resident on every SM the collective's
        # kernel cannot start before it ends, so the two serialise. `--sm-margin` leaves SMs
        # free, but NCCL's all-gather needs ~26 of them for its full rate: not worth it.)
        comm = torch.cuda.Stream(dev)
        cur = torch.cuda.current_stream(dev)
        piped = [Runner(w, s, sm_margin=args.sm_margin) for s in sets] if args.sm_margin else runners
        full_shape = (world * w.B, *runners[0].out.shape[1:])
        gathered = [torch.empty(full_shape, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ev_k = [torch.cuda.Event() for _ in range(2)]
        ev_g = [torch.cuda.Event() for _ in range(2)]

        def pipelined(n):
            for i in range(n):
                k = i % 2
                if i >= 2:
                    cur.wait_event(ev_g[k])       # gather i-2 has read out[k]
                piped[k].launch()
                ev_k[k].record(cur)
                with torch.cuda.stream(comm):
                    comm.wait_event(ev_k[k])
                    sharding.gather_output(piped[k].out, full_shape, out=gathered[k])
                    ev_g[k].record(comm)
            cur.wait_stream(comm)

        pipelined(3)
        barrier()
        dist.all_reduce(align_token)
        s1, e1 = events()
        s1.record()
        pipelined(steps)
        e1.record()
        barrier()
        # the collective alone, back to back
        dist.all_reduce(align_token)
        s2, e2 = events()
        s2.record()
        for i in range(steps):
            sharding.gather_output(piped[i % 2].out, full_shape, out=gathered[i % 2])
        e2.record()
        barrier()
        overlapped_ms, gather_ms = max_over_ranks(
            [s1.elapsed_time(e1) / steps, s2.elapsed_time(e2) / steps], dev, world)
        launches += (steps + 3) * runners[0].launches_per_call
        # Every slab of the gathered tensor equals the owning rank's output, bit for bit:
        # compare position-weighted integer checksums of the slabs.
        last = (steps - 1) % 2
        slabs = gathered[last].view(world, -1).view(torch.int16).to(torch.int64)
        weights = torch.arange(slabs.shape[1], device=dev, dtype=torch.int64) % 8191 + 1
        got = (slabs * weights).sum(dim=1)
        mine = (piped[last].out.reshape(-1).view(torch.int16).to(torch.int64) * weights).sum()
        all_mine = torch.empty(world, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(all_mine, mine.reshape(1))
        slab_bytes = runners[0].out.numel() * 2
        line.update({
            "kernel_only_per_gpu": work / (kernel_ms * 1e-3),
            "kernel_ms_per_step": kernel_ms,
            "gather_ms_per_step": gather_ms, "overlapped_ms_per_step": overlapped_ms,
            "gather_bus_gbs": slab_bytes * (world - 1) / 1e9 / (gather_ms * 1e-3),
            "gather_verified": bool(torch.equal(got, all_mine)),
            "with_gather_every_step": {"value": world * work / (overlapped_ms * 1e-3),
                                       "unit": unit, "ms_per_step": overlapped_ms},
            "sm_margin": args.sm_margin,
        })
        collective = ("none in the data path: `value` = units of all ranks / max-over-ranks time "
                      "of the sharded kernels, independent of --steps. Replicating every step's "
                      "output on every rank (one all-gather per step on a second stream) is "
                      "measured separately: with_gather_every_step, gather_ms_per_step, "
                      "overlapped_ms_per_step, gather_bus_gbs, gather_verified")
        del gathered, slabs, weights

        # ---- strong scaling: ONE batch of the configuration split over the ranks
        # ((batch x kv-head) units, contiguous ranges), slabs gathered, checked against the
        # unsharded launch.
        if w.kind == "prefill" and (w.B * w.Hkv) % world == 0:
            from loopfuse_b200 import functional as F, spec as S
            g_in = tuple(t.to(dev) for t in make_inputs(w, seed=0))
            ql, kl, vl = sharding.shard_units(*g_in, rank, world)
            kind = S.MASK_CAUSAL_WINDOW if w.window else S.MASK_CAUSAL
            local = F.PreparedPrefill(ql, kl, vl, scale=w.D ** -0.5, mods=softcap_mods(w),
                                      mask_kind=kind, window=w.window)
            full = torch.empty_like(g_in[0])
            for _ in range(3):
                local.run()
            barrier()
            dist.all_reduce(align_token)
            s3, e3 = events()
            m3 = torch.cuda.Event(enable_timing=True)
            s3.record()
            for _ in range(steps):
                local.run()
            m3.record()
            sharding.gather_output(local.out, tuple(full.shape), out=full)
            e3.record()
            barrier()
            k_ms, g_ms = max_over_ranks(
                [s3.elapsed_time(m3) / steps, m3.elapsed_time(e3)], dev, world)
            ref = Runner(w, g_in)
            ref.launch()
            torch.cuda.synchronize()
            line["strong_scaling"] = {
                "kernel_ms_per_step": k_ms, "value": work / (k_ms * 1e-3), "unit": unit,
                "gather_ms": g_ms, "verified": bool(torch.equal(full, ref.out)),
                "what": f"one batch of {w.B} split over {world} ranks by (batch x kv-head) "
                        "units; kernel time is the max over ranks, the gather is timed once"}
            launches += steps + 4
            del ref, full, local, g_in
        torch.cuda.empty_cache()

    value = world * work / (ms_per_step * 1e-3)

    line["e2e"] = None
    if not args.kernel_only:
        # ---- end to end through the public API
        barrier()
        ceiling = copy_ceiling(dev)
        e = time_e2e(w, host_sets[0], dev, max(3, min(steps, 10)), barrier)
        e_ms, neg_h2d, neg_d2h = max_over_ranks(
            [e["ms"], -ceiling["h2d_gbs"], -ceiling["d2h_gbs"]], dev, world)
        bound_ms = max(e["h2d_bytes"] / (-neg_h2d * 1e6), e["d2h_bytes"] / (-neg_d2h * 1e6))
        launches += (e["steps"] + 3) * runners[0].launches_per_call
        line["e2e"] = {"value": world * work / (e_ms * 1e-3), "unit": unit,
                       "h2d_bytes_per_step": world * e["h2d_bytes"],
                       "d2h_bytes_per_step": world * e["d2h_bytes"], "ms_per_step": e_ms,
                       "steps": e["steps"],
                       "copy_ceiling": {"h2d_gbs_per_gpu": -neg_h2d, "d2h_gbs_per_gpu": -neg_d2h,
                                        "ms_per_step_at_ceiling": bound_ms,
                                        "frac_of_ceiling": bound_ms / e_ms,
                                        "what": "slowest rank's pinned cudaMemcpyAsync rates, "
                                                "both directions at once"}}

    if not args.kernel_only and w.kind == "prefill":
        # ---- sustained: the headline kernel back to back for >= 2 s
        n_sus = max(steps, int(2200.0 / kernel_ms) + 1)
        sus = ClockSampler(physical_gpu_index(local_rank))
        barrier()
        s4, e4 = events()
        with sus:
            s4.record()
            for i in range(n_sus):
                runners[i % 2].launch()
            e4.record()
            torch.cuda.synchronize()
        sus_ms = max_over_ranks([s4.elapsed_time(e4) / n_sus], dev, world)[0]
        cs = sus.summary()
        line["sustained"] = {
            "launches": n_sus, "seconds": sus_ms * n_sus / 1e3, "ms_per_step": sus_ms,
            "value": work / (sus_ms * 1e-3), "unit": unit, "sm_mhz_median": cs["sm_mhz"],
            "reasons": cs["reasons"],
            "ms_times_mhz": sus_ms * cs["sm_mhz"] if cs["sm_mhz"] else None,
            "frac_of_sustained_peak": work / (sus_ms * 1e-3) / peaks["bf16_tflops_sustained"]}
        launches += n_sus
        # ---- worst case of the data-dependent path: queries scaled by 10, so that the scores
        # of every block leave the range of the polynomial tanh and take the MUFU form.
        if w.softcap:
            hard = [Runner(w, s, q_scale=10.0) for s in sets]
            hard_ms = max_over_ranks([time_runners(hard, steps, 3)], dev, world)[0]
            line["worst_case"] = {"ms_per_step": hard_ms, "value": work / (hard_ms * 1e-3),
                                  "unit": unit,
                                  "what": "queries x10: |score / softcap| > 0.4 in every 32 x 32 "
                                          "piece, MUFU tanh (2 more MUFU ops per score)"}
            launches += steps + 3
            del hard

    # ---- the other benchmark configurations (every rank runs its own batch at N > 1)
    others: dict = {}
    cpu = None
    if not args.no_others and not args.kernel_only:
        del sets, runners
        torch.cuda.empty_cache()
        for name, ow in WORKLOADS.items():
            if name == w.name:
                continue
            o_host = [make_inputs(ow, seed=s, batch_offset=rank * ow.B) for s in (0, 1)]
            orun = [Runner(ow, tuple(t.to(dev) for t in hs)) for hs in o_host]
            barrier()
            ms = max_over_ranks([time_runners(orun, 20, 5)], dev, world)[0]
            launches += 25 * orun[0].launches_per_call
            o_work, o_unit, _ = work_of(ow)
            entry = {"value": world * o_work / (ms * 1e-3), "unit": o_unit, "ms": ms,
                     "per_gpu": o_work / (ms * 1e-3),
                     "roofline": roofline_of(ow, ms, peaks, peak_kind)}
            del orun
            torch.cuda.empty_cache()
            oe = time_e2e(ow, o_host[0], dev, 4, barrier)
            oe_ms = max_over_ranks([oe["ms"]], dev, world)[0]
            entry["e2e"] = {"value": world * o_work / (oe_ms * 1e-3), "unit": o_unit,
                            "h2d_bytes_per_step": world * oe["h2d_bytes"],
                            "d2h_bytes_per_step": world * oe["d2h_bytes"], "ms_per_step": oe_ms}
            if rank == 0 and world == 1:
                c = time_cpu(ow, steps=2, warmup=1)
                c.pop("ms_per_step", None)
                entry["cpu_baseline"] = c
            others[name] = entry
            del o_host
            torch.cuda.empty_cache()
        if rank == 0 and world == 1:
            cpu = time_cpu(w, steps=2, warmup=1)
            cpu.pop("ms_per_step", None)

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, world, {
                "l2": "two alternating input sets, 1 GiB touched per pair of steps "
                      "(L2 is 126 MB); no explicit flush",
                "collective": collective, "host_affinity": affinity}),
            "clocks": sampler.summary(),
            "gpu_launches": launches,
            "roofline": roofline_of(w, kernel_ms, peaks, peak_kind),
        }
        out.update(line)
        out["others"] = others
        if cpu is not None:
            out["cpu_baseline"] = cpu
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="causal_softcap")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the batch per GPU (small cases for profiler captures)")
    ap.add_argument("--sm-margin", type=int, default=0,
                    help="SMs the prefill kernel leaves to the collective in the pipelined "
                         "multi-GPU loop (0: none - NCCL's all-gather moves ~16 GB/s per CTA "
                         "and needs about 26 SMs for the full NVLink rate, which costs the "
                         "kernel more than the overlap returns: measured)")
    ap.add_argument("--no-others", action="store_true",
                    help="skip the figures for the other configurations")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the kernel-timed region (what a profiler capture needs)")
    args = ap.parse_args()
    from loopfuse_b200.variants import WORKLOADS
    workload = WORKLOADS[args.workload]
    if args.batch:
        workload = dataclasses.replace(workload, B=args.batch)
    if args.impl == "reference":
        run_reference_arm(args, workload)
    else:
        run_ours(args, workload)


if __name__ == "__main__":
    main()
