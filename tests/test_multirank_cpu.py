"""The bench's multi-rank bookkeeping on two gloo ranks (CPU): ranks work on
their own tensors with no data-path collective; only the timing is reduced,
as a maximum over ranks."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    my_step_seconds = 0.010 * (rank + 1)          # rank 1 is the slow one
    t = bench.max_over_ranks([my_step_seconds, 1.0 / (rank + 1)])
    value = bench.whole_job_gbps(world, 2 * 4 * (1 << 26), t[0])
    dist.barrier()
    if rank == 0:
        torch.save({"t": t, "value": value}, out)
    dist.destroy_process_group()


def test_two_ranks_report_slowest_rank_time(tmp_path):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["t"] == pytest.approx([0.020, 1.0])
    assert r["value"] == pytest.approx(2 * 2 * 4 * (1 << 26) / 0.020 / 1e9)


def test_single_rank_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.max_over_ranks([0.5, 2.0]) == [0.5, 2.0]
    assert bench.whole_job_gbps(1, 1e9, 0.5) == pytest.approx(2.0)
