"""Measurement shared by ``bench.py`` and the ``bench`` command: timed decode steps and
prefill on the engine's own step function, with the byte and FLOP counts of the reference's
bench (crates/cli/src/bench.rs:261-271, crates/cli/src/metal_batch.rs:113-114,157-160), taken
from the built model (``measure.py``):
  * decode step bytes = every weight the step uses, once, plus the cached keys and values of
    the live requests;
  * FLOPs = 2 per weight element and row, the head counted once per logits row, plus the
    attention products 4 * heads * head size * keys per row and layer.
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess
import tempfile
import threading
import time
from typing import Dict, List, Optional, Tuple

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def repo_root() -> str:
    return os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def measured_peaks() -> Dict[str, float]:
    path = os.path.join(repo_root(), "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
        out = dict(FALLBACK_PEAKS)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if isinstance(raw.get(k), (int, float)):
                out[k] = float(raw[k])
        out["source"] = "measured"
        return out
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS)


def model_folder(preset: str, seed: int, dtype: torch.dtype, n_layer: Optional[int] = None) -> Tuple[str, object]:
    """A folder with seeded random weights of the preset's sizes (made once per process tree, in the
    temporary folder); ``n_layer`` may reduce the depth, never the layer sizes."""
    from .cli import _preset_path
    from .config.base import architecture_name
    from .registry import get_architecture
    from .weights.random_init import write_random_model

    with open(_preset_path(preset)) as fh:
        raw = json.load(fh)
    if n_layer is not None:
        raw["n_layer"] = int(n_layer)
    cfg = get_architecture(architecture_name(raw)).config_cls.from_dict(raw)
    key = hashlib.sha1(json.dumps([raw, seed, str(dtype)], sort_keys=True).encode()).hexdigest()[:12]
    d = os.path.join(tempfile.gettempdir(), f"nanoinfer_b200_model_{os.getuid()}_{key}")
    if not (os.path.isfile(os.path.join(d, "model.safetensors")) and os.path.isfile(os.path.join(d, "config.json"))):
        tmp = d + f".tmp{os.getpid()}"
        write_random_model(cfg, tmp, seed, dtype)
        if os.path.isdir(d):
            import shutil
            shutil.rmtree(tmp)
        else:
            os.rename(tmp, d)
    return d, cfg


# ----------------------------------------------------------------------------- counts
# (taken from the built model and its cache: ``measure.py``)
from .measure import kv_bytes, parameter_count, step_flops, weight_bytes_per_step  # noqa: E402


def vocabulary(eng) -> int:
    return eng.model.vocab_size


def context_limit(eng, default: int) -> int:
    return eng.model.max_positions or default


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons in the background during a timed region."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, period_ms: int = 10):
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.lines: List[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._read, daemon=True)
            self._t.start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> Dict[str, object]:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- workloads
class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so that the next step starts with a cold cache.
    The write (1 GiB, about 0.3 ms) also covers the host's preparation of the step that follows it
    on the stream: the events around the step then bracket device work only, whatever the host's
    speed (with a 256 MB write the host's packing could outlast it, and the gap was counted)."""

    def __init__(self, device, nbytes: int = 1 << 30):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def flush(self) -> None:
        self.buf.zero_()


def build_engine(model_dir: str, dtype: str, batch: int, context: int, max_rows: int):
    from .engine.engine import Engine

    return Engine(model_dir, dtype=dtype, max_tokens=batch * (context + 64), max_batch=max(batch, 1),
                  max_rows=max_rows, check_status=False)


def time_decode(eng, batch: int, prompt_len: int, steps: int, warmup: int, seed: int = 0,
                flush: bool = True, clocks: Optional["ClockSampler"] = None) -> Dict[str, float]:
    """Device time of decode steps at a fixed batch: ``batch`` requests are prefilled with
    ``prompt_len`` random tokens, then ``warmup + steps`` greedy decode steps run through the
    engine's step function and sampler; each timed step is bracketed by CUDA events, with an L2
    flush between steps."""
    from .engine.runner import StepItem

    vocab = vocabulary(eng)
    g = torch.Generator().manual_seed(seed)
    if clocks is not None:
        # clocks and throttle reasons under load: the sampler takes a moment to start, so it is started
        # before the batch's prompts are run and goes on through the warm-up and the timed steps
        clocks.start()
    reqs = [eng.cache.open_request() for _ in range(batch)]
    from .sampling.sampler import SamplingParams
    for r in reqs:
        eng.sampler.set_request(r.slot, SamplingParams(temperature=0.0))
    last = []
    budget = max(1, eng.runner.max_rows // max(1, prompt_len))
    for i in range(0, batch, budget):
        chunk = reqs[i:i + budget]
        items = [StepItem(r, torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), [prompt_len - 1])
                 for r in chunk]
        last += eng.runner.step(items, sampler=eng.sampler).tolist()
    flusher = L2Flusher(eng.device) if flush else None
    times = []
    ctx_sum = 0
    torch.cuda.synchronize()
    for s in range(warmup + steps):
        items = [StepItem(r, [t], [0]) for r, t in zip(reqs, last)]
        if flusher is not None:
            flusher.flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = eng.runner.step(items, sampler=eng.sampler)
        e1.record()
        last = toks.tolist()
        if s >= warmup:
            times.append(e0.elapsed_time(e1))
            ctx_sum += sum(r.n_tokens for r in reqs)
    clock_record = clocks.stop() if clocks is not None else None
    for r in reqs:
        eng.cache.close_request(r)
    ms = sum(times) / len(times)
    return {"clocks": clock_record, "ms_per_step": ms, "tokens_per_s": batch / (ms / 1e3), "mean_context": ctx_sum / (len(times) * batch),
            "steps": len(times), "launches_per_step": eng.runner.launches_last_step,
            "graph_replays": eng.runner.graph_replays}


def preheat(eng, seconds: float = 1.5, prompt_len: int = 512) -> int:
    """Keeps the GPU busy with untimed prefill steps for about ``seconds``: a device that has idled
    (while weights were made on the host, or after another program's pause) takes a moment to reach
    the clocks and power state it then holds, and the few warm-up steps of a timed loop are over
    sooner than that.  Returns the number of steps run."""
    import time

    from .engine.runner import StepItem

    limit = context_limit(eng, prompt_len + 1)
    n = max(1, min(prompt_len, limit - 1, eng.runner.max_rows))
    tokens = [(7 * i + 1) % vocabulary(eng) for i in range(n)]
    t0, steps = time.perf_counter(), 0
    while time.perf_counter() - t0 < seconds:
        r = eng.cache.open_request()
        eng.runner.step([StepItem(r, tokens, [n - 1])])
        eng.cache.close_request(r)
        steps += 1
        if steps % 8 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    return steps


def time_prefill(eng, n_prompts: int, prompt_len: int, runs: int, warmup: int, seed: int = 1) -> Dict[str, float]:
    """Device time of ONE step that prefills ``n_prompts`` prompts of ``prompt_len`` tokens."""
    from .engine.runner import StepItem

    vocab = vocabulary(eng)
    g = torch.Generator().manual_seed(seed)
    flusher = L2Flusher(eng.device)
    times = []
    if eng.runner.use_graphs:
        warmup = max(warmup, 4)   # the step function captures a step with prompts the fourth time it sees its shape
    for s in range(warmup + runs):
        reqs = [eng.cache.open_request() for _ in range(n_prompts)]
        items = [StepItem(r, torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), [prompt_len - 1])
                 for r in reqs]
        flusher.flush()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.runner.step(items)
        e1.record()
        torch.cuda.synchronize()
        if s >= warmup:
            times.append(e0.elapsed_time(e1))
        for r in reqs:
            eng.cache.close_request(r)
    times.sort()
    ms = times[len(times) // 2]
    tokens = n_prompts * prompt_len
    contexts = [p + 1 for _ in range(n_prompts) for p in range(prompt_len)]
    return {"ms": ms, "tokens": tokens, "tokens_per_s": tokens / (ms / 1e3),
            "flops": step_flops(eng.model, contexts, n_prompts)}


def time_e2e_decode(eng, batch: int, prompt_len: int, steps: int, warmup: int, seed: int = 2) -> Dict[str, float]:
    """Decode throughput through the public entry point: requests are added with host token lists,
    ``Engine.step`` runs scheduler, step function and sampler, and every step's tokens are read
    back to the host.  Wall-clock time around the timed steps, device idle before and after."""
    from .sampling.sampler import SamplingParams

    g = torch.Generator().manual_seed(seed)
    params = SamplingParams(max_new_tokens=warmup + steps + 1, temperature=0.0)
    for _ in range(batch):
        eng.add_request(torch.randint(0, vocabulary(eng), (prompt_len,), generator=g).tolist(), params)
    while any(r.n_pending > 1 for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()  # prefill
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    while eng.has_work():
        eng.step()
    return {"tokens_per_s": batch * steps / dt, "ms_per_step": dt / steps * 1e3,
            "h2d_bytes_per_step": eng.runner.last_meta_bytes, "d2h_bytes_per_step": 4 * batch}


def profile_step(eng, items, sampler=None, repeats: int = 3):
    """Per-kernel device time of one step, run eagerly ``repeats`` times (the requests are cut back
    after each run, so the same step is measured); returns {(launcher, label): (ms per step, calls)}."""
    from .kernels import ops

    graphs = eng.runner.use_graphs
    eng.runner.use_graphs = False
    lens = [it.request.n_tokens for it in items]
    try:
        eng.runner.step(items, sampler=sampler)
        for it, n in zip(items, lens):
            eng.cache.truncate(it.request, n)
        prof = ops.start_profile()
        for _ in range(repeats):
            eng.runner.step(items, sampler=sampler)
            for it, n in zip(items, lens):
                eng.cache.truncate(it.request, n)
        out = prof.summary()
    finally:
        ops.stop_profile()
        eng.runner.use_graphs = graphs
    return {k: (ms / repeats, n // repeats) for k, (ms, n) in out.items()}


def format_profile(table) -> str:
    total = sum(ms for ms, _ in table.values())
    lines = [f"{'kernel':<28}{'shape':<26}{'calls':>6}{'ms':>10}{'%':>7}"]
    for (name, label), (ms, n) in sorted(table.items(), key=lambda kv: -kv[1][0]):
        lines.append(f"{name[4:]:<28}{label if 'linear' in name else '':<26}{n:>6}{ms:>10.4f}{100 * ms / total:>7.1f}")
    lines.append(f"{'total':<60}{total:>10.4f}")
    return "\n".join(lines)


def print_profile(eng, prompt) -> None:
    """The per-kernel breakdown of a prefill of ``prompt`` and of one decode step after it."""
    import sys

    from .engine.runner import StepItem
    from .sampling.sampler import SamplingParams

    r = eng.cache.open_request()
    eng.sampler.set_request(r.slot, SamplingParams(temperature=0.0))
    pre = profile_step(eng, [StepItem(r, list(prompt), [len(prompt) - 1])], eng.sampler)
    print(f"-- prefill of {len(prompt)} tokens", file=sys.stderr)
    print(format_profile(pre), file=sys.stderr)
    eng.runner.step([StepItem(r, list(prompt), [len(prompt) - 1])], sampler=eng.sampler)
    dec = profile_step(eng, [StepItem(r, [int(prompt[-1])], [0])], eng.sampler)
    print(f"-- one decode step at context {len(prompt) + 1}", file=sys.stderr)
    print(format_profile(dec), file=sys.stderr)
    eng.cache.close_request(r)


# ----------------------------------------------------------------------------- the bench command
def run_cli_bench(args) -> int:
    import sys

    peaks = measured_peaks()
    bw = args.bandwidth_gbs or peaks["hbm_gbs"]
    batches = [int(b) for b in str(args.batch).split(",") if b]
    from .registry import load_config

    from .registry import get_architecture
    config = load_config(args.weights)
    limit = get_architecture(config.architecture).build_spec(config).max_positions
    if limit is not None and args.prompt_len + args.tokens + args.warmup > limit:
        print(f"prompt_len + tokens must be <= {limit}", file=sys.stderr)
        return 2
    results = []
    for b in batches:
        eng = build_engine(args.weights, args.dtype, b, args.prompt_len + args.tokens + args.warmup,
                           max_rows=max(2048, b))
        dec = time_decode(eng, b, args.prompt_len, args.tokens, max(3, args.warmup))
        pre = time_prefill(eng, 1, args.prompt_len, args.runs, max(1, args.warmup))
        step_bytes = weight_bytes_per_step(eng.model) + kv_bytes(eng.cache, [dec["mean_context"]] * b)
        ceiling = bw * 1e9 / step_bytes * b
        line = {"dtype": args.dtype, "batch": b, "prompt_len": args.prompt_len, "tokens": args.tokens,
                "decode_tok_s": dec["tokens_per_s"], "decode_ms_per_step": dec["ms_per_step"],
                "decode_gbs": step_bytes / (dec["ms_per_step"] / 1e3) / 1e9,
                "ceiling_tok_s": ceiling, "pct_of_ceiling": 100.0 * dec["tokens_per_s"] / ceiling,
                "prefill_tok_s": pre["tokens_per_s"], "note": args.note}
        print(f"{args.dtype} B={b}: prefill {pre['tokens_per_s']:.0f} tok/s | decode {dec['tokens_per_s']:.1f} tok/s "
              f"({line['decode_gbs']:.1f} GB/s) | {line['pct_of_ceiling']:.2f}% of {ceiling:.0f} tok/s ceiling")
        results.append(line)
        del eng
        torch.cuda.empty_cache()
    if args.out:
        with open(args.out, "a") as fh:
            for line in results:
                fh.write(json.dumps(line) + "\n")
    return 0
