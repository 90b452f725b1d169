"""CPU-only, world_size 2 over gloo: the host side of the data-parallel step (bucket merging and the
sum-then-scale average), with the collective injected the way DataParallelTrainer injects NCCL."""
import os
import socket
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # spawned ranks re-import this file

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from weta_b200.trainer import GradBucketer


def test_bucketer_merges_adjacent_ranges():
    sent = []
    b = GradBucketer(lambda s, n: sent.append((s, n)), min_elems=100)
    for s, n in [(0, 10), (10, 30), (40, 70), (110, 5), (115, 0), (200, 10)]:
        b.add(s, n)
    b.flush()
    assert sent == [(0, 110), (110, 5), (200, 10)]
    assert sum(n for _, n in sent) == 125


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(rank)
    arena = torch.randn(1000)
    mine = arena.clone()
    b = GradBucketer(lambda s, n: dist.all_reduce(arena[s:s + n], op=dist.ReduceOp.SUM), min_elems=256)
    for s, n in [(0, 10), (10, 500), (510, 90), (600, 400)]:  # per-layer ranges, last layer first
        b.add(s, n)
    b.flush()
    arena *= 1.0 / world  # what Adam's grad_scale does
    gathered = [torch.zeros(1000) for _ in range(world)]
    dist.all_gather(gathered, mine)
    want = torch.stack(gathered).mean(0)
    out[rank] = bool(torch.allclose(arena, want, atol=1e-6)) and b.issued == [(0, 510), (510, 490)]
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_average_gradients():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out[0] and out[1]
