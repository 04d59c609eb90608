"""Session router: which GPU replica serves which session.

The reference serves one GPU (device 0 only, src/backend_cuda.rs:955-956).  Sessions are independent - the state is per
session (src/gpu_model.rs:3920-3970), the weights are read-only - so N GPUs are N full replicas and the only multi-GPU
decision is the placement of a session at admission.  Nothing here touches a GPU: the router is plain host bookkeeping, and
no collective runs on the data path.

Two policies:

* ``"mod"``          - session id mod n_gpus (a fixed batch of equal sessions: the static-batch benchmark).
* ``"least_loaded"`` - the replica with the least outstanding work at admission, ties to the lower index (the Poisson
                       benchmark: prompt and generation lengths differ by two orders of magnitude).  The work of a session
                       is counted in tokens (prompt + generation budget) and leaves the book when the session retires
                       or, with ``drain_rate`` set, as virtual time passes.

The router is deterministic: the same sequence of calls gives the same placement.  One process per GPU can therefore
replay the same arrival list independently and agree on the placement without exchanging a byte (``drain_rate`` makes the
load book a function of the arrival times alone); a single front-end process uses ``retire`` instead.
"""


class Router:
    def __init__(self, n_gpus, policy="least_loaded", drain_rate=None):
        if n_gpus < 1:
            raise ValueError("n_gpus must be at least 1")
        if policy not in ("mod", "least_loaded"):
            raise ValueError("policy must be 'mod' or 'least_loaded'")
        if drain_rate is not None and not drain_rate > 0:
            raise ValueError("drain_rate must be positive")
        self.n_gpus, self.policy, self.drain_rate = int(n_gpus), policy, drain_rate
        self.load = [0.0] * self.n_gpus   # outstanding tokens per replica
        self.sessions = [0] * self.n_gpus  # sessions admitted and not retired
        self.where = {}                    # session id -> (gpu, cost)
        self._clock = 0.0

    def _drain(self, now):
        if self.drain_rate is None or now is None:
            return
        if now < self._clock:
            raise ValueError("arrival times must not decrease")
        dt, self._clock = now - self._clock, now
        self.load = [max(0.0, x - dt * self.drain_rate) for x in self.load]

    def admit(self, session_id, cost=1.0, now=None):
        """Places a session; returns its GPU.  `cost` = tokens of work (prompt + generation budget); `now` = arrival time in
        seconds when the load book drains by virtual time."""
        if session_id in self.where:
            raise KeyError(f"session {session_id} is already placed")
        if cost < 0:
            raise ValueError("cost must not be negative")
        self._drain(now)
        if self.policy == "mod":
            g = int(session_id) % self.n_gpus
        else:
            g = min(range(self.n_gpus), key=lambda i: (self.load[i], self.sessions[i], i))
        self.load[g] += float(cost)
        self.sessions[g] += 1
        self.where[session_id] = (g, float(cost))
        return g

    def gpu_of(self, session_id):
        return self.where[session_id][0]

    def retire(self, session_id):
        """The session has finished (or left): its work leaves the book.  With `drain_rate` the tokens have drained already."""
        g, cost = self.where.pop(session_id)
        self.sessions[g] -= 1
        if self.drain_rate is None:
            self.load[g] = max(0.0, self.load[g] - cost)
        return g

    def move(self, session_id, gpu, remaining_cost=None):
        """Re-homes a session (after its state was copied with State.slot_copy_from); returns the GPU it left."""
        if not 0 <= gpu < self.n_gpus:
            raise ValueError("gpu out of range")
        g, cost = self.where[session_id]
        c = cost if remaining_cost is None else float(remaining_cost)
        self.load[g] = max(0.0, self.load[g] - cost)
        self.sessions[g] -= 1
        self.load[gpu] += c
        self.sessions[gpu] += 1
        self.where[session_id] = (gpu, c)
        return g

    def most_and_least_loaded(self):
        order = sorted(range(self.n_gpus), key=lambda i: (self.load[i], i))
        return order[-1], order[0]


def place_arrivals(arrive, costs, n_gpus, policy="least_loaded", drain_rate=None):
    """Placement of a whole arrival list (times in seconds, non-decreasing; one cost per session): list of GPU indices.
    Every rank of a one-process-per-GPU job calls this with the same arguments and serves the sessions it is given."""
    r = Router(n_gpus, policy, drain_rate)
    return [r.admit(i, float(c), float(t)) for i, (t, c) in enumerate(zip(arrive, costs))]


class ReplicaSet:
    """One front-end process, one model replica and one continuous-batching scheduler per GPU.

    `submit` places the session with the router and hands it to that GPU's scheduler; `step` queues one packed step on every
    GPU (the schedulers queue their work on their own streams and return, so the GPUs run side by side under one host
    thread); `poll` returns the finished sessions as (session id, tokens) and takes their work off the router's book.
    `schedulers` = objects with the interface of rwkv_rsv_b200.Scheduler (submit / step / poll / result / sync / close)."""

    def __init__(self, schedulers, policy="least_loaded"):
        self.scheds = list(schedulers)
        self.router = Router(len(self.scheds), policy)
        self._local = {}   # (gpu, scheduler's request id) -> session id
        self._next = 0

    def submit(self, prompt, max_new, sp=None):
        sid, self._next = self._next, self._next + 1
        g = self.router.admit(sid, len(prompt) + int(max_new))
        self._local[(g, self.scheds[g].submit(prompt, max_new, sp))] = sid
        return sid

    def step(self):
        """One step on every GPU; returns (rows queued over all GPUs, sessions not yet finished)."""
        rows = active = 0
        for s in self.scheds:
            r, a = s.step()
            rows += r
            active += a
        return rows, active

    def poll(self):
        done = []
        for g, s in enumerate(self.scheds):
            for rid in s.poll():
                sid = self._local.pop((g, rid))
                self.router.retire(sid)
                done.append((sid, s.result(rid)))
        return done

    def run_until_done(self):
        out = {}
        while True:
            rows, active = self.step()
            out.update(self.poll())
            if active == 0:
                break
            if rows == 0:
                for s in self.scheds:
                    s.sync()
        out.update(self.poll())
        return out

    def close(self):
        for s in self.scheds:
            s.close()
