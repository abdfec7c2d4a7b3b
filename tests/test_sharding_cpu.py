"""Multi-GPU host logic on the CPU: (batch x kv-head) unit partition, rank-local views and the
single all-gather, run as two gloo ranks. The per-rank computation is the CPU oracle here (the
kernels need a GPU); the point is that sharded results reassemble to the unsharded result bit for
bit and that a missing rank is detected on the host."""
import datetime
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from loopfuse_b200 import sharding
from loopfuse_b200.variants import WORKLOADS, make_inputs
from oracle import attention_oracle as O


def test_unit_range_partitions_contiguously():
    for n, world in ((256, 8), (64, 4), (8, 8), (2048, 2)):
        ranges = [sharding.unit_range(n, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert len({hi - lo for lo, hi in ranges}) == 1
    with pytest.raises(ValueError):
        sharding.unit_range(10, 0, 4)


def test_shard_units_are_views_of_whole_kv_groups():
    q = torch.randn(2, 8, 5, 16)
    k = torch.randn(2, 2, 7, 16)
    v = torch.randn(2, 2, 7, 16)
    ql, kl, vl = sharding.shard_units(q, k, v, rank=1, world=2)
    assert ql.shape == (2, 4, 5, 16) and kl.shape == (2, 1, 7, 16)
    # rank 1 owns batch element 1 (units 2, 3): q heads 0-3 with kv head 0, 4-7 with kv head 1
    assert torch.equal(ql[0], q[1, 0:4]) and torch.equal(ql[1], q[1, 4:8])
    assert torch.equal(kl[1, 0], k[1, 1]) and torch.equal(vl[0, 0], v[1, 0])
    assert ql.data_ptr() == q[1].data_ptr()


def _worker(rank, world, port, tmp, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=20 if mode == "ok" else 3))
    try:
        w = WORKLOADS["window_gqa_softcap"]
        import dataclasses
        w = dataclasses.replace(w, B=2, Hq=8, Hkv=2, S=96, D=32, window=40)
        q, k, v = (t.float() for t in make_inputs(w))
        full = O.workload_ref(w, (q, k, v), batch_chunk=2)
        ql, kl, vl = sharding.shard_units(q, k, v, rank, world)
        local = O.attention_ref(ql, kl, vl, mods=O.softcap_mods(w.softcap), mask="window",
                                window=w.window, batch_chunk=ql.shape[0])
        if mode == "missing_rank" and rank == 1:
            return                      # leaves between steps, never joins the collective
        try:
            out = sharding.gather_output(local, tuple(full.shape))
        except Exception as e:          # the surviving rank sees a host-side error, no hang
            torch.save({"error": type(e).__name__}, f"{tmp}/r{rank}.pt")
            return
        torch.save({"equal": torch.equal(out, full), "max_diff": (out - full).abs().max().item()},
                   f"{tmp}/r{rank}.pt")
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_reassemble_the_unsharded_result(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), "ok"), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["max_diff"] <= 1e-6, res


def test_missing_rank_is_detected_on_the_host(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), "missing_rank"), nprocs=2, join=True)
    res = torch.load(tmp_path / "r0.pt")
    assert "error" in res, res
