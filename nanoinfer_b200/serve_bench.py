"""The serving benchmark: many requests of random lengths through the continuous-batching
scheduler, beside a static-batching baseline, in the manner of the reference's ``metal-serve``
(crates/cli/src/metal_serve.rs).

The workload is the reference's (metal_serve.rs:97-131): request ``i`` arrives after an
exponential gap of mean ``1 / rate`` (``rate`` 0: everything at t = 0), with a prompt length uniform in
``[prompt_min, prompt_max]`` and a fixed output length uniform in ``[out_min, out_max]`` (no end
token), all from one xorshift generator seeded with ``seed``.  The reference cuts its prompts out of an
English text; here they are seeded random token ids of the same lengths.

Two policies run the same requests (metal_serve.rs:163-363):
  * ``static``: batches of ``max_batch`` in arrival order; a batch runs until its longest request is
    done, and a slot whose request ended early stays empty until then;
  * ``continuous``: the engine's scheduler (admission while a slot and pages are free, decode rows
    first, prompt portions under ``prefill_budget``).
For each the summary gives what the reference's does (metal_serve.rs:373-469): generated tokens per
second over the makespan, time to first token, time per output token and end-to-end latency at p50
and p99, iterations, rows computed, peak and mean pages in use, and a down-sampled iteration trace.
Times are the host's wall clock; the engine runs one step ahead of its reads, so a token's time is
when the host has read it.
"""
from __future__ import annotations

import json
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

_MASK64 = (1 << 64) - 1


class XorShift:
    """The workload generator of the reference (metal_serve.rs:82-95): xorshift64 (13, 7, 17)."""

    def __init__(self, seed: int):
        self.s = ((int(seed) * 0x9E3779B97F4A7C15) & _MASK64) | 1

    def next(self) -> int:
        s = self.s
        s ^= (s << 13) & _MASK64
        s ^= s >> 7
        s ^= (s << 17) & _MASK64
        self.s = s
        return s

    def unif(self) -> float:
        return (self.next() >> 11) / float(1 << 53)

    def range(self, lo: int, hi: int) -> int:
        return lo + self.next() % (hi - lo + 1)


@dataclass
class ServeRequest:
    id: int
    arrival: float
    prompt: List[int]
    out_len: int


@dataclass
class RequestLog:
    admitted: float = 0.0
    first_token: float = 0.0
    finished: float = 0.0
    generated: int = 0


@dataclass
class Iteration:
    t0: float
    dt: float
    decode_rows: int
    prefill_rows: int
    occupied: int
    kv_pages: int


@dataclass
class Outcome:
    logs: List[RequestLog]
    iters: List[Iteration] = field(default_factory=list)
    makespan: float = 0.0
    pages_peak: int = 0
    preemptions: int = 0


def workload(n_requests: int, prompt_min: int, prompt_max: int, out_min: int, out_max: int, rate: float, seed: int,
             vocab_size: int) -> List[ServeRequest]:
    import math

    rng = XorShift(seed)
    t, reqs = 0.0, []
    for i in range(n_requests):
        if rate > 0.0:
            t += -math.log(max(rng.unif(), 1e-12)) / rate
        n_prompt = rng.range(prompt_min, prompt_max)
        prompt = [rng.next() % vocab_size for _ in range(n_prompt)]
        reqs.append(ServeRequest(i, t, prompt, rng.range(out_min, out_max)))
    return reqs


def _run(engine, reqs: List[ServeRequest], static: bool, temperature: float = 0.0, top_k: int = 40,
         seed: int = 0) -> Outcome:
    """Feeds the requests to the engine as they arrive and steps it until all are done.  With a
    temperature every request samples from a generator of its own (seed + its id)."""
    from .sampling.sampler import SamplingParams

    sched, cache = engine.scheduler, engine.cache
    logs = [RequestLog() for _ in reqs]
    out = Outcome(logs)
    handle: Dict[int, object] = {}        # request id -> the engine's request
    rid_of: Dict[int, int] = {}           # id(engine's request) -> request id
    first_seen: Dict[int, bool] = {}
    nxt, done = 0, 0
    last_decode, last_prefill = sched.stats.decode_rows, sched.stats.prefill_rows
    pre0 = sched.stats.preemptions
    t_start = time.perf_counter()
    now = lambda: time.perf_counter() - t_start
    while done < len(reqs):
        t = now()
        # static batching takes the next batch only when the engine is empty
        may_add = not static or not engine.has_work()
        room = engine.scheduler.max_batch if static else len(reqs)
        while may_add and nxt < len(reqs) and reqs[nxt].arrival <= t and room > 0:
            r = reqs[nxt]
            handle[r.id] = engine.add_request(r.prompt, SamplingParams(max_new_tokens=r.out_len, temperature=temperature,
                                                                       top_k=top_k, seed=seed + r.id))
            rid_of[id(handle[r.id])] = r.id
            nxt += 1
            room -= 1
        if not engine.has_work():
            if nxt < len(reqs):
                time.sleep(max(0.0, min(reqs[nxt].arrival - now(), 0.01)))
            continue
        t0 = now()
        ended = engine.step()
        t1 = now()
        st = sched.stats
        used = cache.pages_used()
        pages = max(used) if used else 0
        out.iters.append(Iteration(t0, t1 - t0, st.decode_rows - last_decode, st.prefill_rows - last_prefill,
                                   len(sched.running), pages))
        last_decode, last_prefill = st.decode_rows, st.prefill_rows
        out.pages_peak = max(out.pages_peak, pages)
        for rid, h in handle.items():
            if rid not in first_seen:
                if h.admitted_order >= 0 and logs[rid].admitted == 0.0:
                    logs[rid].admitted = t0
                if h.output and h.output[0] >= 0:
                    first_seen[rid] = True
                    logs[rid].first_token = t1
        for h in ended:
            rid = rid_of.pop(id(h))
            logs[rid].finished = t1
            logs[rid].generated = len(h.output)
            if rid not in first_seen:
                first_seen[rid] = True
                logs[rid].first_token = t1
            del handle[rid]
            done += 1
    out.makespan = now()
    out.preemptions = sched.stats.preemptions - pre0
    return out


def run_continuous(engine, reqs: List[ServeRequest], **sampling) -> Outcome:
    return _run(engine, reqs, static=False, **sampling)


def run_static(engine, reqs: List[ServeRequest], **sampling) -> Outcome:
    return _run(engine, reqs, static=True, **sampling)


def _pct(xs: List[float], p: float) -> float:
    xs = sorted(xs)
    return xs[int(round((len(xs) - 1) * p))] if xs else 0.0


def summarise(name: str, reqs: List[ServeRequest], o: Outcome, page_size: int, gantt: int = 32,
              quiet: bool = False) -> dict:
    gen = sum(l.generated for l in o.logs)
    ttft = [l.first_token - r.arrival for r, l in zip(reqs, o.logs)]
    tpot = [(l.finished - l.first_token) / (r.out_len - 1) for r, l in zip(reqs, o.logs) if r.out_len > 1]
    e2e = [l.finished - r.arrival for r, l in zip(reqs, o.logs)]
    rows = sum(i.decode_rows + i.prefill_rows for i in o.iters)
    wasted = sum(max(0, i.occupied - i.decode_rows) for i in o.iters) if name == "static" else 0
    busy = sum(i.dt for i in o.iters)
    kv_avg = sum(i.kv_pages * i.dt for i in o.iters) / max(busy, 1e-12)
    stride = max(1, -(-len(o.iters) // 120))
    if not quiet:
        print(f"{name:<11} {gen / o.makespan:>8.0f} tok/s  makespan {o.makespan:>6.2f} s  iters {len(o.iters):>5}  "
              f"TTFT p50 {1e3 * _pct(ttft, 0.5):>7.1f} ms p99 {1e3 * _pct(ttft, 0.99):>7.1f} ms  "
              f"TPOT p50 {1e3 * _pct(tpot, 0.5):>6.2f} ms p99 {1e3 * _pct(tpot, 0.99):>6.2f} ms  "
              f"e2e p50 {_pct(e2e, 0.5):>6.2f} s  KV peak {o.pages_peak} pages")
    return {
        "policy": name,
        "throughput_tok_s": gen / o.makespan,
        "generated_tokens": gen,
        "makespan_s": o.makespan,
        "engine_busy_s": busy,
        "iterations": len(o.iters),
        "rows_computed": rows,
        "wasted_decode_rows": wasted,
        "preemptions": o.preemptions,
        "ttft_ms": {"p50": 1e3 * _pct(ttft, 0.5), "p99": 1e3 * _pct(ttft, 0.99)},
        "tpot_ms": {"p50": 1e3 * _pct(tpot, 0.5), "p99": 1e3 * _pct(tpot, 0.99)},
        "e2e_s": {"p50": _pct(e2e, 0.5), "p99": _pct(e2e, 0.99)},
        "kv_pages_peak": o.pages_peak,
        "kv_pages_avg_used": kv_avg,
        "kv_page_tokens": page_size,
        "gantt": [{"id": r.id, "arrival": r.arrival, "admitted": l.admitted, "first_token": l.first_token,
                   "finished": l.finished, "prompt_len": len(r.prompt), "out_len": r.out_len}
                  for r, l in list(zip(reqs, o.logs))[:gantt]],
        "iters": [{"t": i.t0, "dt": i.dt, "decode_rows": i.decode_rows, "prefill_rows": i.prefill_rows,
                   "occupied": i.occupied, "kv_pages": i.kv_pages} for i in o.iters[::stride]],
    }


def run_serving(model_dir: str, dtype: str = "bfloat16", requests: int = 128, max_batch: int = 32,
                prompt_min: int = 16, prompt_max: int = 256, out_min: int = 16, out_max: int = 256, rate: float = 0.0,
                prefill_budget: int = 256, kv_blocks: Optional[int] = None, seed: int = 7, temperature: float = 0.0,
                top_k: int = 40, gantt: int = 32, policies=("static", "continuous"), quiet: bool = False) -> dict:
    """The serving workload through the engine, once per policy; returns the summary (the options are
    those of the reference's ``metal-serve``: crates/cli/src/metal_serve.rs:33-79).  Every number that
    describes the model (context limit, vocabulary, bytes a step must read) is taken from the engine
    that was built, not from a configuration's field names."""
    from .bench_support import measured_peaks
    from .engine.engine import Engine
    from .measure import kv_bytes_per_position, weight_bytes_per_step

    page = 16

    def engine(n_blocks):
        return Engine(model_dir, dtype=dtype, max_tokens=n_blocks * page, max_batch=max_batch,
                      max_rows=max(512, prefill_budget + max_batch), prefill_budget=prefill_budget, page_size=page)

    probe_blocks = kv_blocks or max_batch * (-(-(prompt_max + out_max) // page)) + 8
    eng = engine(probe_blocks)
    limit, vocab = eng.model.max_positions, eng.model.vocab_size
    if limit is not None and prompt_max >= limit:
        raise ValueError(f"prompt_max must be below the context length {limit}")
    longest = prompt_max + out_max if limit is None else min(prompt_max + out_max, limit)
    n_blocks = kv_blocks or max_batch * (-(-longest // page)) + 8
    if n_blocks != probe_blocks:
        del eng
        torch_empty_cache()
        eng = engine(n_blocks)
    reqs = workload(requests, prompt_min, prompt_max, out_min, out_max, rate, seed, vocab)
    if limit is not None:   # an output that would pass the end of the context is cut there
        for r in reqs:
            r.out_len = max(1, min(r.out_len, limit - len(r.prompt)))
    total_in, total_out = sum(len(r.prompt) for r in reqs), sum(r.out_len for r in reqs)
    if not quiet:
        print(f"serve-bench: {requests} requests (prompt {prompt_min}-{prompt_max}, output {out_min}-{out_max}; "
              f"{total_in} prompt + {total_out} output tokens), rate {rate} req/s, max batch {max_batch}, "
              f"{n_blocks} KV pages, {dtype}", file=sys.stderr)
    sampling = {"temperature": temperature, "top_k": top_k, "seed": seed}
    run_continuous(eng, reqs[:min(len(reqs), 4)], **sampling)   # warm up: kernels built, first graphs captured
    peaks = measured_peaks()
    weights = weight_bytes_per_step(eng.model)
    page_bytes = sum(per_pos for per_pos, _ in kv_bytes_per_position(eng.cache)) * page
    out = []
    for name in policies:
        o = (run_static if name == "static" else run_continuous)(eng, reqs, **sampling)
        s = summarise(name, reqs, o, page, gantt, quiet=quiet)
        # what the steps had to read (every weight once a step, and the pages in use) over the time
        # the engine was busy, against the memory's rate
        must_read = sum(weights + i.kv_pages * page_bytes for i in o.iters)
        s["hbm_gbs"] = must_read / max(s["engine_busy_s"], 1e-12) / 1e9
        s["hbm_frac"] = s["hbm_gbs"] / peaks["hbm_gbs"]
        s["kv_pages_total"] = n_blocks
        out.append(s)
    return {"requests": requests, "max_batch": max_batch, "prefill_budget": prefill_budget, "kv_blocks": n_blocks,
            "dtype": dtype, "seed": seed, "rate": rate, "temperature": temperature, "top_k": top_k,
            "prompt_tokens": total_in, "output_tokens": total_out, "peaks": peaks["source"], "policies": out}


def torch_empty_cache() -> None:
    import torch
    torch.cuda.empty_cache()


def run_cli(args) -> int:
    from .bench_support import provenance

    try:
        summary = run_serving(args.weights, args.dtype, args.requests, args.max_batch, args.prompt_min, args.prompt_max,
                              args.out_min, args.out_max, args.rate, args.prefill_budget, args.kv_blocks, args.seed,
                              args.temperature, args.top_k, args.gantt)
    except ValueError as e:
        print(str(e), file=sys.stderr)
        return 2
    summary["note"] = args.note
    by = {s["policy"]: s for s in summary["policies"]}
    print(f"continuous / static throughput: {by['continuous']['throughput_tok_s'] / by['static']['throughput_tok_s']:.2f}x")
    stamp = provenance()
    summary.update(stamp)
    if args.summary:
        with open(args.summary, "w") as fh:
            json.dump(summary, fh)
    if args.out:
        with open(args.out, "a") as fh:
            for s in summary["policies"]:
                fh.write(json.dumps({"stage": f"serve-{s['policy']}", "dtype": args.dtype,
                                     "throughput_tok_s": s["throughput_tok_s"], "ttft_ms": s["ttft_ms"],
                                     "tpot_ms": s["tpot_ms"], "e2e_s": s["e2e_s"], "hbm_frac": s["hbm_frac"],
                                     "kv_pages_peak": s["kv_pages_peak"], "kv_pages_total": s["kv_pages_total"],
                                     "requests": args.requests, "max_batch": args.max_batch, "note": args.note,
                                     **stamp}) + "\n")
    return 0
