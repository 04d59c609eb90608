"""Multi-GPU layout: one full model replica per GPU, sessions sharded by id, no collective on the data path.

The reference is single-GPU (device 0 only, src/backend_cuda.rs:955-956); sessions are independent (per-session state,
read-only weights), so they shard across replicas without any exchange.  `torch.distributed` is used only to line the
ranks up (barrier) and to take the slowest rank's time.
"""


def shard_sessions(n_sessions, world_size):
    """Session ids owned by each rank: id mod world_size (sizes differ by at most one)."""
    return [list(range(r, n_sessions, world_size)) for r in range(world_size)]


def owner_of(session_id, world_size):
    return session_id % world_size


def max_over_ranks(value, dist=None, device=None):
    """The slowest rank's value (every rank gets it).  With no process group this is the value itself."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, dist=None, device=None):
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def all_ranks_ok(ok, dist=None, device=None):
    """True on every rank only if `ok` is true on every rank.  Called between steps (nothing in flight on any GPU): a rank whose
    step raised reports it here, and the others learn of it on the host before their next launch instead of waiting for it in a
    reduction that never comes."""
    return max_over_ranks(0.0 if ok else 1.0, dist, device) == 0.0
