"""GPU parity of the continuous-batching scheduler: every session's tokens must equal what the single-session
API produces for it, whatever else shares its steps."""
import numpy as np
import pytest

import rwkv_rsv_b200 as rsv

pytestmark = pytest.mark.gpu


def single_session(bundle, prompt, max_new, sp):
    """Reference semantics: prefill the prompt, then token r from the previous token's logits with seed sp.seed + r and
    the r tokens generated so far as history (arg-max when sp is None)."""
    bundle.reset()
    out = []
    feed = list(prompt)
    for r in range(max_new):
        if sp is None:
            tok = bundle.infer_argmax(feed)
        else:
            spr = rsv.SamplerParams(sp.temperature, sp.top_k, sp.top_p, (sp.seed + r) & 0xFFFFFFFF, sp.repetition_penalty, sp.frequency_penalty,
                                    sp.presence_penalty)
            tok = bundle.infer_sample(feed, spr, out)
        out.append(tok)
        feed = [tok]
    return out


@pytest.fixture(scope="module")
def bundle(tiny_paths):
    return rsv.ModelBuilder(tiny_paths["int8"]).build()


def test_ragged_sessions_argmax(bundle):
    rng = np.random.default_rng(21)
    lens = [1, 7, 40, 3, 130, 16, 65]
    news = [5, 9, 3, 12, 4, 8, 1]
    prompts = [rng.integers(0, 4096, size=n).astype(np.uint32) for n in lens]
    want = [single_session(bundle, p, n, None) for p, n in zip(prompts, news)]
    sch = rsv.Scheduler(bundle.model, max_slots=3, chunk=16, max_rows=24, max_new_cap=16)   # fewer slots than sessions: they queue
    ids = [sch.submit(p, n) for p, n in zip(prompts, news)]
    done = sch.run_until_done()
    assert sorted(done) == sorted(ids)
    for i, rid in enumerate(ids):
        assert list(done[rid]) == want[i], f"session {i}"
    st = sch.stats()
    assert st["rows"] == sum(lens) + sum(n - 1 for n in news)     # every prompt token and every fed-back token is one row
    assert st["steps"] < st["rows"]                               # rows were packed several to a step


def test_sampling_sessions_and_late_arrivals(bundle):
    rng = np.random.default_rng(22)
    sps = [rsv.SamplerParams(top_p=0.9, seed=100), rsv.SamplerParams(temperature=0.7, top_k=40, seed=7, repetition_penalty=1.2),
           rsv.SamplerParams(top_p=0.5, seed=2**32 - 2), rsv.SamplerParams(seed=55, frequency_penalty=0.5, presence_penalty=0.2)]
    prompts = [rng.integers(0, 4096, size=n).astype(np.uint32) for n in (9, 33, 2, 70)]
    news = [10, 6, 8, 5]
    want = [single_session(bundle, p, n, sp) for p, n, sp in zip(prompts, news, sps)]
    sch = rsv.Scheduler(bundle.model, max_slots=4, chunk=32, max_rows=48, max_new_cap=16)
    ids = [sch.submit(prompts[0], news[0], sps[0]), sch.submit(prompts[1], news[1], sps[1])]
    done = {}
    for _ in range(3):                       # two sessions run alone for a few steps, then two more arrive
        sch.step()
    ids += [sch.submit(prompts[2], news[2], sps[2]), sch.submit(prompts[3], news[3], sps[3])]
    done.update(sch.run_until_done())
    for i, rid in enumerate(ids):
        assert list(done[rid]) == want[i], f"session {i}"


def test_mixed_argmax_and_sampling_in_one_step(bundle):
    rng = np.random.default_rng(23)
    p0, p1 = rng.integers(0, 4096, size=12).astype(np.uint32), rng.integers(0, 4096, size=5).astype(np.uint32)
    sp = rsv.SamplerParams(top_p=0.8, seed=9)
    want0, want1 = single_session(bundle, p0, 6, None), single_session(bundle, p1, 6, sp)
    sch = rsv.Scheduler(bundle.model, max_slots=2, chunk=8, max_rows=16, max_new_cap=8)
    a, b = sch.submit(p0, 6), sch.submit(p1, 6, sp)
    done = sch.run_until_done()
    assert list(done[a]) == want0 and list(done[b]) == want1


def test_scheduler_errors(bundle):
    sch = rsv.Scheduler(bundle.model, max_slots=2, chunk=8, max_rows=16, max_new_cap=8)
    with pytest.raises(rsv.RsvError, match="vocab"):
        sch.submit([1, 4096], 2)
    with pytest.raises(rsv.RsvError, match="empty"):
        sch.submit([], 2)
    with pytest.raises(rsv.RsvError, match="max_new"):
        sch.submit([1], 9)
    rid = sch.submit([1, 2, 3], 2)
    with pytest.raises(rsv.RsvError, match="not finished"):
        sch.result(rid)
    assert list(sch.run_until_done()) == [rid]
    with pytest.raises(rsv.RsvError, match="unknown"):
        sch.result(rid)
    with pytest.raises(rsv.RsvError):
        rsv.Scheduler(bundle.model, max_slots=4, chunk=8, max_rows=2)


def _replica_set_equals_single_sessions(path, devices, bundle):
    """A front end over one scheduler per model handle (rwkv_rsv_b200.router.ReplicaSet): sessions of very different sizes are
    placed least-loaded, every replica packs its own steps, and every session's tokens equal the single-session API's."""
    from rwkv_rsv_b200.router import ReplicaSet
    rng = np.random.default_rng(23)
    lens = [3, 90, 5, 17, 140, 2, 33, 8, 61, 12]
    news = [6, 3, 10, 5, 2, 9, 4, 7, 3, 8]
    sps = [None if i % 3 == 0 else rsv.SamplerParams(top_p=0.9, temperature=0.9, seed=1000 + i) for i in range(len(lens))]
    prompts = [rng.integers(0, 4096, size=n).astype(np.uint32) for n in lens]
    want = [single_session(bundle, p, n, sp) for p, n, sp in zip(prompts, news, sps)]
    models = [rsv.Model(path, device=d) for d in devices]
    rs = ReplicaSet([rsv.Scheduler(m, max_slots=3, chunk=32, max_rows=48, max_new_cap=16) for m in models])
    try:
        sids = [rs.submit(p, n, sp) for p, n, sp in zip(prompts, news, sps)]
        placed = [rs.router.gpu_of(s) for s in sids]
        assert set(placed) == set(range(len(devices)))             # both replicas got work ...
        work = [sum(lens[i] + news[i] for i in range(len(lens)) if placed[i] == g) for g in range(len(devices))]
        assert max(work) - min(work) <= max(l + n for l, n in zip(lens, news))  # ... balanced by tokens to within one session
        done = rs.run_until_done()
        assert sorted(done) == sids
        for i, sid in enumerate(sids):
            assert list(done[sid]) == want[i], f"session {i} on replica {placed[i]}"
        assert rs.router.sessions == [0] * len(devices)
    finally:
        rs.close()
        for m in models:
            m.close()


def test_replica_set_over_two_model_handles(bundle, tiny_paths):
    _replica_set_equals_single_sessions(tiny_paths["int8"], [0, 0], bundle)


def test_replica_set_over_two_gpus(bundle, tiny_paths):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _replica_set_equals_single_sessions(tiny_paths["int8"], [0, 1], bundle)
