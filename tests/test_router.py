"""Host logic of the multi-GPU layout: the session router (no GPU, no collective) and, with the gloo backend at world size 2,
that one process per GPU replaying the same arrival list agrees on the placement without exchanging it."""
import os

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkv_rsv_b200.router import ReplicaSet, Router, place_arrivals
from rwkv_rsv_b200.shard import max_over_ranks, sum_over_ranks


def test_mod_policy_is_session_id_mod_n():
    r = Router(4, "mod")
    assert [r.admit(i, 10) for i in range(10)] == [i % 4 for i in range(10)]
    assert r.sessions == [3, 3, 2, 2] and r.load == [30.0, 30.0, 20.0, 20.0]


def test_least_loaded_balances_unequal_sessions_and_retire_frees_the_book():
    r = Router(3)
    assert [r.admit(i, c) for i, c in enumerate([100, 10, 10, 10, 10, 50])] == [0, 1, 2, 1, 2, 1]
    assert r.load == [100.0, 70.0, 20.0]
    assert r.retire(0) == 0 and r.load[0] == 0.0 and r.sessions[0] == 0
    assert r.admit(6, 5) == 0
    assert r.gpu_of(6) == 0 and r.most_and_least_loaded() == (1, 0)
    with pytest.raises(KeyError):
        r.admit(6, 1)
    with pytest.raises(KeyError):
        r.retire(0)


def test_ties_go_to_fewer_sessions_then_to_the_lower_index():
    r = Router(3)
    assert [r.admit(i, 0) for i in range(4)] == [0, 1, 2, 0]


def test_move_rehomes_a_session():
    r = Router(2)
    r.admit("a", 40)
    r.admit("b", 40)
    r.admit("c", 40)
    assert r.load == [80.0, 40.0]
    assert r.move("c", 1, remaining_cost=10) == 0
    assert r.load == [40.0, 50.0] and r.sessions == [1, 2] and r.gpu_of("c") == 1
    r.retire("c")
    assert r.load == [40.0, 40.0]


def test_virtual_time_drain_is_a_function_of_the_arrival_list():
    arrive, costs = [0.0, 0.0, 1.0, 1.0, 1.5], [100, 10, 10, 10, 10]
    # at t = 1 the 50 tok/s drain has emptied GPU 1 (10 tokens) and left GPU 0 with 50
    assert place_arrivals(arrive, costs, 2, "least_loaded", drain_rate=50.0) == [0, 1, 1, 1, 1]
    with pytest.raises(ValueError):
        place_arrivals([1.0, 0.5], [1, 1], 2, "least_loaded", drain_rate=1.0)


def test_arguments_are_checked():
    for bad in (lambda: Router(0), lambda: Router(2, "random"), lambda: Router(2, drain_rate=0.0), lambda: Router(2).admit(0, -1), lambda: Router(2).move(0, 1)):
        with pytest.raises((ValueError, KeyError)):
            bad()
    r = Router(2)
    r.admit(0, 1)
    with pytest.raises(ValueError):
        r.move(0, 2)


class _FakeSched:
    """A scheduler that finishes a session `work` steps after it was submitted and 'generates' its id."""

    def __init__(self):
        self.q, self.done, self.n, self.closed = {}, [], 0, False

    def submit(self, prompt, max_new, sp=None):
        self.q[self.n] = len(prompt) + max_new
        self.n += 1
        return self.n - 1

    def step(self):
        rows = len(self.q)
        for rid in list(self.q):
            self.q[rid] -= 10
            if self.q[rid] <= 0:
                del self.q[rid]
                self.done.append(rid)
        return rows, len(self.q) + len(self.done)

    def poll(self):
        d, self.done = self.done, []
        return d

    def result(self, rid):
        return np.asarray([rid], dtype=np.uint32)

    def sync(self):
        pass

    def close(self):
        self.closed = True


def test_replica_set_spreads_sessions_and_returns_every_result():
    scheds = [_FakeSched(), _FakeSched(), _FakeSched()]
    rs = ReplicaSet(scheds)
    rng = np.random.default_rng(0)
    sids = [rs.submit([0] * int(rng.integers(1, 200)), int(rng.integers(1, 100))) for _ in range(40)]
    assert all(s.n >= 8 for s in scheds)  # roughly a third each
    out = rs.run_until_done()
    assert sorted(out) == sids and rs.router.sessions == [0, 0, 0] and rs.router.where == {}
    rs.close()
    assert all(s.closed for s in scheds)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank builds the same seeded arrival list (as the benchmark does) and keeps the sessions placed on it
    rng = np.random.default_rng(3)
    n = 64
    arrive = np.cumsum(rng.exponential(1.0 / 64.0, size=n))
    cost = rng.integers(16, 2048, size=n) + rng.geometric(1.0 / 256.0, size=n)
    place = place_arrivals(arrive, cost, world, "least_loaded", drain_rate=4000.0)
    mine = [i for i, g in enumerate(place) if g == rank]
    dist.barrier()
    total = sum_over_ranks(len(mine), dist)
    work = float(sum(cost[i] for i in mine))
    slowest = max_over_ranks(work, dist)
    q.put((rank, mine, total, work, slowest, float(cost.sum())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_placement_without_exchanging_it():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, mine0, tot0, w0, slow0, all_work), (_, mine1, tot1, w1, slow1, _) = got
    assert sorted(mine0 + mine1) == list(range(64)) and not set(mine0) & set(mine1)  # a partition
    assert tot0 == tot1 == 64.0
    assert slow0 == slow1 == max(w0, w1)
    assert abs(w0 - w1) <= 0.25 * all_work  # unequal sessions, balanced work
