#!/usr/bin/env python3
"""Benchmark of the batched RWKV-7 forward step (decode), 3B shape, int8 weights.

  python bench.py --gpus 1 --steps K --warmup W          # this repository's CUDA path
  python bench.py --impl reference --steps K --warmup W  # the reference algorithm's fp32 CPU path (the oracle)

One "step" = one decode step of `--batch` sessions per GPU (default 1: benchmark config 2, a 512-token
prompt prefilled and then an arg-max self-loop).  Prints ONE JSON line.
  value     decode tok/s summed over all GPUs, device-timed (CUDA events on the model's stream) with tokens
            and state resident in HBM (GPU self-loop, no host round-trip)
  e2e       the same metric through the host-buffer API: per step the tokens go host->device and the
            logits come back device->host
  roofline  the dominant kernel's algorithmic bytes / its mean device time, against the measured HBM peak
  cpu_baseline  the CPU oracle timed on this box (bounded sample; all cores and one core)
Further keys, each run by every rank (times = the slowest rank's, tokens summed): `batch_sweep` (decode at 1, 8, 64, 256, 1024
sessions per GPU), `batch_sweep_fixed_total` (N > 1: that many sessions in all, sharded by id mod N), `prefill` (one session's
2048 tokens in 512-token chunks per GPU), `continuous_batching` (benchmark config 3: 256 Poisson sessions per GPU, routed
least-loaded; `..._fixed_total` at N > 1), `other_weight_formats` (N = 1: fp16 and the reference's per-group int8 container at
batch 1 and 64), `timed_regions` (the timed region of K steps is repeated for about a second; the median is reported).
Inputs are synthetic: seeded random-init weights of the named shape, uniform random prompt tokens.
Every step streams all weights (3.1 GB at the 3B int8 shape), far more than the 126 MB L2, so no L2 flush
is needed between timed iterations.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_second"
UNIT = "tok/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--shape", default="3b", choices=["tiny", "3b", "7b"])
    ap.add_argument("--quant", default="int8", choices=["fp16", "int8", "int8g"],
                    help="int8: one (scale, zero) per output row; int8g: the reference container, one per row and group of 128 weights")
    ap.add_argument("--batch", type=int, default=1, help="sessions per GPU")
    ap.add_argument("--prompt", type=int, default=512, help="prompt tokens prefilled before decoding")
    ap.add_argument("--sweep", default="1,8,64,256,1024", help="batch sizes of the decode sweep, per GPU; '' disables it")
    ap.add_argument("--sweep-steps", type=int, default=32)
    ap.add_argument("--prefill", type=int, default=2048, help="prompt tokens of the timed chunked prefill, per GPU; 0 disables it")
    ap.add_argument("--continuous", type=int, default=256, help="sessions per GPU of the continuous-batching workload (benchmark config 3); 0 disables it")
    ap.add_argument("--other-format", type=int, default=1, help="1: also time batch 1 and 64 with the other weight formats (fp16, int8 per row, int8 per group), N=1 only")
    ap.add_argument("--cpu-seconds", type=float, default=20.0, help="time budget of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--model-dir", default=os.environ.get("RSV_BENCH_DIR", "/tmp/rsv_bench"))
    return ap.parse_args()


def model_path(args):
    return os.path.join(args.model_dir, f"rwkv7_{args.shape}_{args.quant}_seed0.st")


def ensure_model(args):
    import rwkv_rsv_b200 as rsv
    path = model_path(args)
    if not os.path.exists(path):
        os.makedirs(args.model_dir, exist_ok=True)
        tmp = path + f".tmp{os.getpid()}"
        rsv.write_synthetic(tmp, args.shape, seed=0, quant={"fp16": 0, "int8": 1, "int8g": 2}[args.quant])
        os.replace(tmp, path)
    return path


def shape_of(args):
    import rwkv_rsv_b200 as rsv
    return rsv.SHAPES[args.shape]


def algorithmic_bytes(sh, quant, B):
    """Dense algorithmic bytes of one decode step: every weight byte once, state read + written once per
    session, the embedding row and the logits per session."""
    L, C, F, V, H, N = sh["n_layer"], sh["n_embd"], sh["ffn_hidden"], sh["vocab"], sh["n_head"], sh["head_size"]
    mids = sh["w_mid"] + sh["a_mid"] + sh["v_mid"] + sh["g_mid"]
    big = L * (4 * C * C + 2 * C * F)
    if quant in ("int8", "int8g"):
        w = big + big // 128 * 4
    else:
        w = big * 2
    w += L * 2 * C * mids * 2 + L * 19 * C * 4 + V * C * 2
    s_rw = 2 * L * H * N * N * 4 + 2 * L * 2 * C * 4
    a = 2 * C + 2 * V * 4
    return w + B * (s_rw + a), w


# DRAM traffic of decode_stream_kernel per decoded token, from one ncu capture of a 4-token launch
# (dram__bytes_read.sum + dram__bytes_write.sum, divided by 4; summary under profiles/).  Every token streams the same weights,
# so the traffic of a launch is this figure times its tokens.
NCU_DRAM_BYTES_PER_TOKEN = {("3b", "int8", 1): 3.0933e9}


def kernel_bytes(sh, quant, B):
    """Algorithmic bytes of one launch of each weight-streaming kernel (weights once + activations in/out)."""
    C, F, V = sh["n_embd"], sh["ffn_hidden"], sh["vocab"]
    mids = sh["w_mid"] + sh["a_mid"] + sh["v_mid"] + sh["g_mid"]
    wb = (lambda m, k: m * k + m * k // 128 * 4) if quant in ("int8", "int8g") else (lambda m, k: m * k * 2)
    act = lambda n_in, n_out: 4 * B * (n_in + n_out)
    return {
        "linear_rkv_rank": 3 * wb(C, C) + C * mids * 2 + act(6 * C, 3 * C + mids),
        "linear_rank_back": C * mids * 2 + act(mids, 4 * C),
        "linear_att_out": wb(C, C) + act(C, 2 * C),
        "linear_ffn_key": wb(F, C) + act(C, F),
        "linear_ffn_value": wb(C, F) + act(F, 2 * C),
        "linear_head": V * C * 2 + act(C, V),
        "wkv7": B * (sh["n_head"] * 64 * 64 * 4 * 2 + 4 * 7 * C),
    }


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(path, sh, seconds, threads=None, prompt=8, single_tokens=3):
    """Times the CPU oracle (fp32, the reference's algorithm) on a bounded sample of the same workload."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    nthr = threads or (os.cpu_count() or 1)
    orc.set_threads(nthr)
    t0 = time.perf_counter()
    m = orc.OracleModel(path)
    load_s = time.perf_counter() - t0
    rng = np.random.default_rng(1)
    toks = rng.integers(0, sh["vocab"], size=prompt).astype(np.uint32)
    m.forward(toks[:2])  # warm-up: page in the weights
    tok, n, t0 = int(toks[-1]), 0, time.perf_counter()
    while True:
        tok = orc.argmax(m.forward([tok]))
        n += 1
        el = time.perf_counter() - t0
        if (el >= seconds and n >= 3) or n >= 4096:
            break
    # the reference's CPU path is single-threaded (no rayon in src/model.rs): the same oracle on one thread, a few tokens
    single = None
    if single_tokens > 0:
        orc.set_threads(1)
        t1 = time.perf_counter()
        k = 0
        while k < single_tokens:
            tok = orc.argmax(m.forward([tok]))
            k += 1
            if time.perf_counter() - t1 > 45.0:
                break
        single = {"value": k / (time.perf_counter() - t1), "unit": UNIT, "cores": 1, "tokens": k}
        orc.set_threads(nthr)
    res = {"value": n / el, "unit": UNIT, "cores": nthr, "kind": "port", "single_thread": single,
           "sample": f"{n} arg-max decode tokens of the same checkpoint after a {2}-token warm-up, fp32 CPU oracle, {nthr} OpenMP threads "
                     f"(model load {load_s:.1f} s not timed)"}
    m.close()
    return res, m


def run_reference(args):
    """--impl reference: the reference algorithm's own CPU implementation (the fp32 oracle; the Rust crate
    cannot be built in this image) on all host threads, same config and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    path = ensure_model(args)
    sh = shape_of(args)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    nthr = os.cpu_count() or 1
    orc.set_threads(nthr)
    m = orc.OracleModel(path)
    rng = np.random.default_rng(1)
    tok = int(rng.integers(0, sh["vocab"]))
    budget = 120.0
    t_w = time.perf_counter()
    for i in range(max(args.warmup, 1)):
        tok = orc.argmax(m.forward([tok]))
        if time.perf_counter() - t_w > budget / 4:
            break
    n, t0 = 0, time.perf_counter()
    while n < args.steps:
        tok = orc.argmax(m.forward([tok]))
        n += 1
        if time.perf_counter() - t0 > budget and n >= 3:
            break
    el = time.perf_counter() - t0
    v = n / el
    sample = f"{n} of the requested {args.steps} decode steps (time-bounded), batch 1, {nthr} OpenMP threads, oracle port of src/model.rs"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": n, "warmup": args.warmup,
        "ms_per_step": 1000.0 * el / n, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args, 1),
        "reference_note": "the CPU arm decodes from a fresh state (the cost of a decode step does not depend on the state's content); its prompt is not prefilled",
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": nthr, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def bench_config(args, B):
    """The `config` object of the JSON line: the same for the GPU arm and the reference arm."""
    return {"workload": workload_name(args), "shape": args.shape, "weights": args.quant, "batch_per_gpu": B, "prompt": args.prompt,
            "l2": "every step streams all weights (>> 126 MB L2); no flush needed", "sessions": "one full replica per GPU, no collective"}


def workload_name(args):
    return (f"RWKV-7 {args.shape} shape {args.quant}, random init seed 0: {args.prompt}-token uniform-random prompt prefill, then arg-max "
            f"GPU self-loop decode, batch {args.batch} per GPU")


def decode_run(rsv, model, state, seeds, steps):
    """Queues `steps` self-loop rounds; returns device ms (CUDA events on the model's stream)."""
    model.timer_start()
    t = model.submit_sample_selfloop_batch(state, seeds, steps, None)
    ms = model.timer_stop()
    out = model.collect_sample_selfloop_batch(t)
    return ms, out


def prefix_states(rsv, model, B, prompt, vocab, rng):
    """Per-slot prefix state: up to 8 distinct prompts are prefilled and their states tiled over the slots
    (the state's content does not change the work of a decode step)."""
    st = model.create_batch_state(B)
    nd = min(B, 8)
    small = model.create_batch_state(nd)
    prompts = [rng.integers(0, vocab, size=prompt).astype(np.uint32) for _ in range(nd)]
    seeds = model.forward_seq_batch(small, prompts)
    per = [small.slot_back(i) for i in range(nd)]
    for b in range(B):
        st.slot_load(b, per[b % nd])
    small.close()
    return st, np.asarray([seeds[b % nd] for b in range(B)], dtype=np.uint32)


def continuous_batching(rsv, model, sh, n_sessions, seed=3, rate=64.0, rank=0, world=1, dist=None, device=None, fixed_total=False):
    """Benchmark config 3: `n_sessions` sessions per GPU arrive as one Poisson process at `rate` requests per second and GPU (wall
    clock; with `fixed_total` both figures are totals over all GPUs: the arrival span, about n_sessions / rate seconds, then bounds
    the run from below however many GPUs serve it), prompt lengths log-uniform in 16..2048, generation lengths geometric with mean 256, top-p 0.9, temperature 1.0, one
    sampler seed per session; every scheduler step is a ragged mix of prompt chunks (<= 512 tokens per session) and one decode
    row per generating session.  With several GPUs every rank builds the same arrival list, places the sessions with the
    least-loaded router (rwkv_rsv_b200.router.place_arrivals: deterministic, nothing is exchanged) and serves its own; the
    clock starts at a barrier.  Returns tokens per second over the span from the first arrival to the last completion on the
    slowest rank."""
    from rwkv_rsv_b200.router import place_arrivals
    from rwkv_rsv_b200.shard import max_over_ranks, sum_over_ranks
    total = n_sessions if fixed_total else n_sessions * world
    rate_all = rate if fixed_total else rate * world
    rng = np.random.default_rng(seed)
    arrive = np.cumsum(rng.exponential(1.0 / rate_all, size=total))
    arrive -= arrive[0]
    plen = np.clip(np.exp(rng.uniform(np.log(16), np.log(2048), size=total)).astype(np.int64), 16, 2048)
    glen = np.clip(rng.geometric(1.0 / 256.0, size=total), 1, 2048)
    prompts = [rng.integers(0, sh["vocab"], size=int(n)).astype(np.uint32) for n in plen]
    # the router's book drains at about one GPU's measured rate on this workload (prompt + generated tokens per second)
    place = place_arrivals(arrive, plen + glen, world, "least_loaded", drain_rate=8000.0) if world > 1 else [0] * total
    mine = [i for i in range(total) if place[i] == rank]
    from rwkv_rsv_b200.shard import all_ranks_ok
    sched, failure = None, None
    try:
        sched = rsv.Scheduler(model, max_slots=max(len(mine), 1), chunk=512, max_new_cap=2048)
    except Exception as e:
        failure = str(e)
    if not all_ranks_ok(failure is None, dist, device):
        if sched:
            sched.close()
        raise RuntimeError(failure or "another rank could not create its scheduler")
    nxt, done, generated, steps, rows_total, max_rows = 0, 0, 0, 0, 0, 0
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    try:
        while done < len(mine):
            now = time.perf_counter() - t0
            while nxt < len(mine) and arrive[mine[nxt]] <= now:
                i = mine[nxt]
                sched.submit(prompts[i], int(glen[i]), rsv.SamplerParams(temperature=1.0, top_p=0.9, seed=1000 + i))
                nxt += 1
            rows, active = sched.step()
            steps += 1 if rows else 0
            rows_total += rows
            max_rows = max(max_rows, rows)
            for rid in sched.poll():
                generated += len(sched.result(rid))
                done += 1
            if rows == 0 and active == 0 and nxt < len(mine):
                time.sleep(max(0.0, min(0.002, arrive[mine[nxt]] - (time.perf_counter() - t0))))
            elif rows == 0:
                sched.sync()
        sched.sync()
    except Exception as e:  # reported to the other ranks below: they must not wait for this one in a reduction
        failure = str(e)
    el_own = time.perf_counter() - t0
    sched.close()
    if not all_ranks_ok(failure is None, dist, device):
        raise RuntimeError(failure or "another rank's scheduler failed")
    el = max_over_ranks(el_own, dist, device)
    gen_all = int(sum_over_ranks(generated, dist, device))
    assert gen_all == int(glen.sum()), "every session must produce its full generation length"
    per_rank = [int(sum(1 for g in place if g == r)) for r in range(world)]
    return {"sessions": total, "sessions_per_gpu": per_rank, "arrival_rate_per_s": rate_all, "arrival_span_s": float(arrive[-1]), "prompt_tokens": int(plen.sum()), "generated_tokens": gen_all,
            "seconds": el, "decode_tok_s": gen_all / el, "total_tok_s": (int(plen.sum()) + gen_all) / el, "steps_rank0": steps,
            "mean_rows_per_step_rank0": rows_total / max(steps, 1), "max_rows_per_step_rank0": max_rows,
            "placement": "one GPU" if world == 1 else "least-loaded at admission (virtual-time drain 8000 tok/s), replayed identically on every rank",
            "sampler": "top_p 0.9, temperature 1.0, seed 1000 + session", "prefill_chunk": 512}


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    import torch
    import rwkv_rsv_b200 as rsv
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sh = shape_of(args)
    if rank == 0:
        ensure_model(args)
    if dist:
        dist.barrier()
    path = model_path(args)
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    rng = np.random.default_rng(1000 + rank)

    model = rsv.Model(path, device=local)
    state, seeds = prefix_states(rsv, model, B, args.prompt, sh["vocab"], rng)

    # ---- device-resident decode: warm-up, then timed regions of exactly K steps each ----
    # A region of K steps can be far shorter than the clock sampler's period, so the region is repeated (R >= 3 times, about a
    # second in all) while the sampler runs; the reported time is the median region (each one the max over ranks), the spread is
    # reported beside it.
    from rwkv_rsv_b200.shard import max_over_ranks
    w_ms, _ = decode_run(rsv, model, state, seeds, W)
    torch.cuda.synchronize()
    w_ms = max_over_ranks(w_ms, dist, torch.device("cuda", local))  # the same on every rank: they must agree on the number of regions
    reps = int(min(25, max(3, np.ceil(1000.0 / max(w_ms / W * K, 1e-3)))))
    clocks = ClockSampler(local)
    clocks.start()
    region_ms, launches = [], 0
    for _ in range(reps):
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        model.clear_kernel_prof()
        ms_r, out = decode_run(rsv, model, state, seeds, K)
        launches = model.launch_count()
        torch.cuda.synchronize()
        region_ms.append(max_over_ranks(ms_r, dist, torch.device("cuda", local)))  # the slowest replica's device time
    clk = clocks.stop()
    ms = float(np.median(region_ms))
    value = world * B * K / (ms / 1000.0)

    # ---- end to end through the host-buffer API (batch 1: Bundle::infer_tokens per token) ----
    e2e = None
    if B == 1:
        tok_pin = torch.zeros(1, dtype=torch.int32).pin_memory()
        lg_pin = torch.zeros(sh["vocab"], dtype=torch.float32).pin_memory()
        tok_np, lg_np = tok_pin.numpy().view(np.uint32), lg_pin.numpy()
        lib = rsv.native()
        tok_np[0] = int(out[0, -1])
        import ctypes
        tp, lp = ctypes.c_void_p(tok_pin.data_ptr()), ctypes.c_void_p(lg_pin.data_ptr())
        for _ in range(W):
            assert lib.rsv_infer_tokens(model._h, state._h, tp, 1, lp) == 0
            tok_np[0] = int(lg_np.argmax())
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(K):
            rc = lib.rsv_infer_tokens(model._h, state._h, tp, 1, lp)
            tok_np[0] = int(lg_np.argmax())
        torch.cuda.synchronize()
        el = time.perf_counter() - t0
        assert rc == 0
        el = max_over_ranks(el, dist, torch.device("cuda", local))
        e2e = {"value": world * K / el, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4 * sh["vocab"],
               "api": "rsv_infer_tokens (Bundle::infer_tokens), one token in, logits out, host arg-max"}

    result = None
    if rank == 0:
        # ---- per-kernel device time -> roofline of the dominant kernel ----
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
        step_bytes, w_bytes = algorithmic_bytes(sh, args.quant, B)
        kb = kernel_bytes(sh, args.quant, B)
        # per-kernel device times of the multi-kernel path (CUDA event pair around every launch)
        model.clear_kernel_prof()
        model.prof_enable(True)
        decode_run(rsv, model, state, seeds, min(K, 16))
        model.prof_enable(False)
        prof = model.kernel_prof()
        tot = sum(v["ms"] for v in prof.values())
        kernels = {k: {"share": v["ms"] / tot, "us_per_launch": 1000.0 * v["ms"] / v["launches"],
                       "gbs": (kb[k] / (v["ms"] / v["launches"] / 1000.0) / 1e9) if k in kb else None} for k, v in prof.items()}
        if launches == 1:
            # the whole timed region was ONE launch of the persistent decode kernel: its duration is the timed region itself
            achieved = step_bytes * K / (ms / 1000.0) / 1e9
            per_tok = NCU_DRAM_BYTES_PER_TOKEN.get((args.shape, args.quant, B))
            traffic = per_tok * K if per_tok else None
            roofline = {"bound": "hbm", "kernel": "decode_stream_kernel", "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                        "frac": achieved / peak, "traffic": traffic, "bytes_per_launch": step_bytes * K, "ms_per_launch": ms, "share_of_step": 1.0,
                        "note": "one cooperative launch runs all timed steps; bytes = algorithmic bytes of a decode step x steps; "
                                "traffic = ncu DRAM bytes per token (4-token capture) x steps",
                        "step": {"bytes": step_bytes, "achieved": achieved, "frac": achieved / peak}, "multi_kernel_path": kernels}
        else:
            dom = max(prof.items(), key=lambda kv: kv[1]["ms"])
            dom_ms = dom[1]["ms"] / dom[1]["launches"]
            achieved = kb.get(dom[0], 0) / (dom_ms / 1000.0) / 1e9
            roofline = {"bound": "hbm", "kernel": dom[0], "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                        "traffic": None, "bytes_per_launch": kb.get(dom[0], 0), "ms_per_launch": dom_ms, "share_of_step": dom[1]["ms"] / tot,
                        "step": {"bytes": step_bytes, "achieved": step_bytes / (ms / K / 1000.0) / 1e9,
                                 "frac": step_bytes / (ms / K / 1000.0) / 1e9 / peak},
                        "kernels": kernels}
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench_config(args, B),
            "clocks": clk, "gpu_launches": launches, "e2e": e2e, "roofline": roofline,
            "timed_regions": {"count": reps, "ms_min": float(min(region_ms)), "ms_median": ms, "ms_max": float(max(region_ms))},
        }
    # ---- the other workloads: every rank runs its share, times are the slowest rank's, tokens are summed ----
    from rwkv_rsv_b200.shard import shard_sessions, sum_over_ranks
    dev = torch.device("cuda", local)
    peak_gbs = None
    try:
        peak_gbs = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs")
    except OSError:
        pass
    peak_gbs = peak_gbs or 6650.0
    legs = {}
    # decode batch sweep (benchmark config 4): b sessions on every GPU (weak) and, with several GPUs, b sessions in all, sharded
    # by session id mod N (strong: per-GPU batches shrink and move back toward the weight-stream regime)
    if args.sweep:
        def sweep_point(n_local):
            """`n_local` sessions on this rank (0: this rank only joins the barriers)."""
            ms_b = 0.0
            if n_local > 0:
                st_b, seeds_b = prefix_states(rsv, model, n_local, min(args.prompt, 256), sh["vocab"], rng)
                decode_run(rsv, model, st_b, seeds_b, 3)
                torch.cuda.synchronize()
            if dist:
                dist.barrier()
            if n_local > 0:
                ms_b, _ = decode_run(rsv, model, st_b, seeds_b, args.sweep_steps)
                st_b.close()
            return max_over_ranks(ms_b, dist, dev)
        weak, strong = {}, {}
        for b in [int(x) for x in args.sweep.split(",") if x]:
            if b == B:
                ms_b = ms / K * args.sweep_steps
            else:
                ms_b = sweep_point(b)
            bts, _ = algorithmic_bytes(sh, args.quant, b)
            weak[str(b)] = {"tok_s": world * b * args.sweep_steps / (ms_b / 1000.0), "ms_per_step": ms_b / args.sweep_steps,
                            "hbm_frac": bts / (ms_b / args.sweep_steps / 1000.0) / 1e9 / peak_gbs}
            if world > 1 and b >= world:
                share = len(shard_sessions(b, world)[rank])
                ms_s = sweep_point(share)
                strong[str(b)] = {"tok_s": b * args.sweep_steps / (ms_s / 1000.0), "ms_per_step": ms_s / args.sweep_steps, "sessions_per_gpu": b // world}
        legs["batch_sweep"] = weak
        if strong:
            legs["batch_sweep_fixed_total"] = strong
    # prompt prefill (the chunked sequence path, Bundle::infer with chunk 512): one session per GPU
    if args.prefill > 0:
        from rwkv_rsv_b200.shard import all_ranks_ok
        pms, perr = 0.0, None
        try:
            pb = rsv.Bundle(model)
            ptoks = rng.integers(0, sh["vocab"], size=args.prefill).astype(np.uint32)
            pb.infer_chunked(ptoks[:min(512, args.prefill)], 512)  # sizes the work buffers
            pb.reset()
        except Exception as e:  # an optional section must not cost the headline line
            perr = str(e)
        if all_ranks_ok(perr is None, dist, dev):
            if dist:
                dist.barrier()
            try:
                model.timer_start()
                pb.infer_chunked(ptoks, 512)
                pms = model.timer_stop()
                pb.state.close()
            except Exception as e:
                perr = str(e)
            ok = all_ranks_ok(perr is None, dist, dev)
            pms = max_over_ranks(pms, dist, dev)
            if ok:
                legs["prefill"] = {"tokens": int(args.prefill) * world, "chunk": 512, "ms": pms, "tok_s": world * args.prefill / (pms / 1000.0),
                                   "api": "rsv_infer_chunked (Bundle::infer, RnnOption::Last), one session per GPU"}
        if "prefill" not in legs:
            legs["prefill"] = {"error": perr or "another rank failed"}
    # continuous batching (benchmark config 3)
    if args.continuous > 0:
        try:
            legs["continuous_batching"] = continuous_batching(rsv, model, sh, args.continuous, rank=rank, world=world, dist=dist, device=dev)
        except Exception as e:  # raised on every rank together (see all_ranks_ok)
            legs["continuous_batching"] = {"error": str(e)}
        if world > 1:
            try:
                legs["continuous_batching_fixed_total"] = continuous_batching(rsv, model, sh, args.continuous, rank=rank, world=world, dist=dist, device=dev,
                                                                              fixed_total=True)
            except Exception as e:
                legs["continuous_batching_fixed_total"] = {"error": str(e)}
    if rank == 0:
        result.update(legs)
    state.close()
    model.close()
    # ---- the same shape with the other weight format (fp16 when the headline is int8): batch 1 and batch 64, one GPU only ----
    if rank == 0 and world == 1 and args.other_format:
        try:
            import copy
            legs2 = {}
            for q2 in [q for q in ("fp16", "int8", "int8g") if q != args.quant]:
                a2 = copy.copy(args)
                a2.quant = q2
                ensure_model(a2)
                m2 = rsv.Model(model_path(a2), device=local)
                leg = {}
                for b in (1, 64):
                    st_b, seeds_b = prefix_states(rsv, m2, b, 64, sh["vocab"], rng)
                    decode_run(rsv, m2, st_b, seeds_b, 3)
                    n = 64 if b == 1 else args.sweep_steps
                    ms_b, _ = decode_run(rsv, m2, st_b, seeds_b, n)
                    bts, _ = algorithmic_bytes(sh, q2, b)
                    leg[str(b)] = {"tok_s": b * n / (ms_b / 1000.0), "ms_per_step": ms_b / n, "hbm_frac": bts / (ms_b / n / 1000.0) / 1e9 / peak_gbs}
                    st_b.close()
                m2.close()
                legs2[q2] = leg
            result["other_weight_formats"] = legs2
        except Exception as e:  # an optional section must not cost the headline line
            result["other_weight_formats"] = {"error": str(e)}
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            result["cpu_baseline"], _ = cpu_baseline(path, sh, args.cpu_seconds)
        elif not args.no_cpu_baseline:
            result["cpu_baseline"] = None
        print(json.dumps(result))
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
