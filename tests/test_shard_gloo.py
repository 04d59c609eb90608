"""CPU test of the multi-GPU host logic with the gloo backend, world_size 2: session sharding, the barrier and the
max-over-ranks / sum-over-ranks reductions the benchmark uses.  No data-path collective exists to test."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkv_rsv_b200.shard import all_ranks_ok, max_over_ranks, owner_of, shard_sessions, sum_over_ranks


def test_shard_sessions_partition():
    for n in (0, 1, 7, 256, 1024):
        for w in (1, 2, 4, 8):
            parts = shard_sessions(n, w)
            flat = sorted(i for p in parts for i in p)
            assert flat == list(range(n))
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
            assert all(owner_of(i, w) == r for r, p in enumerate(parts) for i in p)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = shard_sessions(10, world)[rank]
    dist.barrier()
    slow = max_over_ranks(1.0 + rank, dist)          # rank 1 is the slow one
    total = sum_over_ranks(len(mine), dist)
    out.put((rank, slow, total, mine))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [g[1] for g in got] == [2.0, 2.0]           # both ranks see the slowest rank's time
    assert [g[2] for g in got] == [10.0, 10.0]         # aggregate = sum over ranks
    assert got[0][3] == [0, 2, 4, 6, 8] and got[1][3] == [1, 3, 5, 7, 9]


def _failing_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    log = []
    for step in range(3):
        ok = True
        try:
            if rank == 1 and step == 1:
                raise RuntimeError("this rank's step failed")  # a host-side failure between steps: nothing is in flight
            done = 10 * (step + 1)
        except RuntimeError:
            ok = False
        if not all_ranks_ok(ok, dist):
            log.append(("skipped", step))  # every rank leaves the leg together; no rank waits in a reduction for the failed one
            break
        log.append(("sum", step, sum_over_ranks(done, dist)))
    out.put((rank, log))
    dist.barrier()
    dist.destroy_process_group()


def test_a_rank_that_fails_between_steps_is_seen_by_the_others():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] == got[1] == [("sum", 0, 20.0), ("skipped", 1)]
