"""world_size-2 gloo test of the replica aggregation used by the multi-GPU benchmark."""
import importlib
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.conftest import ROOT


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rep = importlib.import_module("little-gemma_b200.replicas")
    # fake per-rank measurements: rank r emitted 1000*(r+1) tokens in 500*(r+1) ms
    my = torch.tensor([1000.0 * (rank + 1), 500.0 * (rank + 1), 100.0, 1.0 + rank, 1.0], dtype=torch.float64)
    allv = [torch.zeros_like(my) for _ in range(world)]
    dist.barrier()
    dist.all_gather(allv, my)
    agg = rep.aggregate([v.tolist() for v in allv])
    if rank == 0:
        q.put((agg, rep.session_seed(0), rep.session_seed(1)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_replicas_aggregate_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    agg, s0, s1 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert agg["tok_s"] == pytest.approx(3000.0 / 1.0)        # 3000 tokens / slowest replica (1000 ms)
    assert agg["e2e_tok_s"] == pytest.approx(200.0 / 2.0)
    assert agg["identical"] == 1.0 and agg["n"] == 2.0
    assert s0 != s1


def test_aggregate_flags_a_diverging_replica():
    rep = importlib.import_module("little-gemma_b200.replicas")
    agg = rep.aggregate([[10, 1, 1, 1, 1], [10, 2, 1, 1, 0]])
    assert agg["identical"] == 0.0 and agg["max_ms"] == 2
    with pytest.raises(ValueError):
        rep.aggregate([])
