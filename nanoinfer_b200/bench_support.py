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


def model_folder(preset: str, seed: int, dtype: torch.dtype, n_layer: Optional[int] = None,
                 overrides: Optional[Dict[str, object]] = None) -> Tuple[str, object]:
    """A folder with seeded random weights of the preset's sizes (made once per process tree, in the
    temporary folder); ``n_layer`` may reduce the depth, never the layer sizes; ``overrides`` replaces
    other keys of the preset's config.json (a longer context, for instance)."""
    from .cli import _preset_path
    from .config.base import architecture_name
    from .registry import get_architecture
    from .weights.random_init import write_random_model

    with open(_preset_path(preset)) as fh:
        raw = json.load(fh)
    if n_layer is not None:
        raw["n_layer"] = int(n_layer)
    raw.update(overrides or {})
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
        prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in chunk]
        # (a prompt longer than a step's rows goes in portions, one request at a time)
        for at in range(0, prompt_len, eng.runner.max_rows):
            n = min(eng.runner.max_rows, prompt_len - at)
            items = [StepItem(r, p[at:at + n], [n - 1] if at + n == prompt_len else []) for r, p in zip(chunk, prompts)]
            toks = eng.runner.step(items, sampler=eng.sampler)
        last += toks.tolist()
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
    back to the host.  Wall-clock time around the timed steps, device idle before and after.

    Prompts enter under the engine's row budget, so the requests begin to decode a few steps apart;
    prompts are that many tokens shorter than ``prompt_len`` and every request is given more new
    tokens than the run takes, so that all ``batch`` requests decode in every timed step (a request
    that ended inside the timed steps would leave a smaller batch of another shape behind).
    ``host_ms_per_step``: what the host spends on a step (scheduling, packing, launching,
    bookkeeping) without its waits for the device: where it is below the device's time per step,
    the host is hidden behind the device."""
    from .sampling.sampler import SamplingParams

    g = torch.Generator().manual_seed(seed)
    lag = -(-batch * prompt_len // max(1, min(eng.scheduler.prefill_budget, eng.runner.max_rows))) + 1
    prompt_len = max(1, prompt_len - lag)
    params = SamplingParams(max_new_tokens=warmup + steps + 2 * lag + 4, temperature=0.0)
    for _ in range(batch):
        eng.add_request(torch.randint(0, vocabulary(eng), (prompt_len,), generator=g).tolist(), params)
    while any(r.n_pending > 1 for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()  # prefill
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    eng.wait_seconds = 0.0
    rows = 0
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
        rows += len(eng.scheduler.running)
    host = time.perf_counter() - t0 - eng.wait_seconds
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    full = rows == batch * steps
    while eng.has_work():
        eng.step()
    return {"tokens_per_s": batch * steps / dt, "ms_per_step": dt / steps * 1e3, "host_ms_per_step": host / steps * 1e3,
            "all_rows_in_every_step": full,
            "h2d_bytes_per_step": eng.runner.last_meta_bytes, "d2h_bytes_per_step": 4 * batch}


# ----------------------------------------------------------------------------- provenance
def provenance() -> Dict[str, object]:
    """Where a number comes from: the commit and whether the tree was clean, the tools, the device
    and the time (the reference stamps its ledger lines the same way: crates/cli/src/bench.rs:151-175)."""
    def git(*args):
        try:
            return subprocess.run(["git", "-C", repo_root(), *args], capture_output=True, text=True, timeout=10).stdout.strip()
        except (OSError, subprocess.SubprocessError):
            return ""
    sha = git("rev-parse", "--short=12", "HEAD")
    dirty: Optional[bool] = bool(git("status", "--porcelain")) if sha else None
    if not sha:
        # a copy of the tree without its history (a snapshot sent to another machine): the build step
        # leaves the commit it was made from beside the kernel library
        try:
            with open(os.path.join(repo_root(), "nanoinfer_b200", "_build", "git_state.json")) as fh:
                state = json.load(fh)
            sha, dirty = state.get("git_sha") or "", state.get("git_dirty")
        except (OSError, ValueError):
            pass
    out: Dict[str, object] = {"git_sha": sha or None, "git_dirty": dirty,
                              "torch": torch.__version__, "cuda": torch.version.cuda,
                              "time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    if torch.cuda.is_available():
        out["gpu"] = torch.cuda.get_device_name(0)
    try:
        out["load_1m"] = os.getloadavg()[0]
    except OSError:
        pass
    return out


# ----------------------------------------------------------------------------- the per-op profile
def profile_step(eng, items, sampler=None, repeats: int = 3, phase: str = "decode"):
    """One step run eagerly ``repeats`` times under a trace recorder (the requests are cut back after
    each run, so the same step is measured); returns name -> (calls, ms, FLOPs, bytes) per step."""
    from . import trace

    graphs = eng.runner.use_graphs
    eng.runner.use_graphs = False
    lens = [it.request.n_tokens for it in items]
    try:
        eng.runner.step(items, sampler=sampler)
        for it, n in zip(items, lens):
            eng.cache.truncate(it.request, n)
        rec = trace.start()
        for _ in range(repeats):
            rec.begin_step(phase, sum(len(it.tokens) for it in items), 0)
            eng.runner.step(items, sampler=sampler)
            for it, n in zip(items, lens):
                eng.cache.truncate(it.request, n)
        table = rec.table()
    finally:
        trace.stop()
        eng.runner.use_graphs = graphs
    return {k: (n // repeats, ms / repeats, fl / repeats, by / repeats) for k, (n, ms, fl, by) in table.items()}


def print_profile(eng, prompt, out=None) -> None:
    """Where the time of a prefill of ``prompt`` and of one decode step after it goes, op by op, with
    each op's GFLOP/s, GB/s and fraction of the roofline (the reference's ``--profile``:
    crates/cli/src/report.rs:22-58)."""
    import sys

    from . import trace
    from .engine.runner import StepItem
    from .sampling.sampler import SamplingParams

    out = out or sys.stderr
    peaks = measured_peaks()
    r = eng.cache.open_request()
    eng.sampler.set_request(r.slot, SamplingParams(temperature=0.0))
    pre = profile_step(eng, [StepItem(r, list(prompt), [len(prompt) - 1])], eng.sampler, phase="prefill")
    print(trace.format_table(pre, peaks["hbm_gbs"], peaks["bf16_tflops"],
                             f"\nprefill of {len(prompt)} tokens (kernels launched one by one; peaks {peaks['source']})"), file=out)
    eng.runner.step([StepItem(r, list(prompt), [len(prompt) - 1])], sampler=eng.sampler)
    dec = profile_step(eng, [StepItem(r, [int(prompt[-1])], [0])], eng.sampler)
    print(trace.format_table(dec, peaks["hbm_gbs"], peaks["bf16_tflops"],
                             f"\none decode step at context {len(prompt) + 1}"), file=out)
    eng.cache.close_request(r)


# ----------------------------------------------------------------------------- the bench command
def decode_points(model_dir: str, dtype: str, batches, prompt_len: int, tokens: int, warmup: int = 3,
                  bandwidth_gbs: Optional[float] = None, runs: int = 3, profile: bool = False) -> List[dict]:
    """The reference's bench at each batch size (crates/cli/src/bench.rs:240-373,
    crates/cli/src/metal_batch.rs:113-160): ``batch`` requests with prompts of ``prompt_len`` tokens
    decode ``tokens`` tokens; tokens a second, the bytes a step must read over its time, and the
    share of the ceiling that the memory's rate sets; the pages the requests hold at the end of
    ``pages_total``."""
    import sys

    peaks = measured_peaks()
    bw = bandwidth_gbs or peaks["hbm_gbs"]
    out = []
    for b in batches:
        eng = build_engine(model_dir, dtype, b, prompt_len + tokens + warmup, max_rows=max(2048, b, prompt_len))
        dec = time_decode(eng, b, prompt_len, tokens, max(3, warmup))
        pre = time_prefill(eng, 1, prompt_len, runs, 1)
        step_bytes = weight_bytes_per_step(eng.model) + kv_bytes(eng.cache, [dec["mean_context"]] * b)
        ceiling = bw * 1e9 / step_bytes * b
        pages_total = [g.pool.n_pages for g in eng.cache.groups]
        pages_used = [-(-(prompt_len + tokens + warmup) // eng.cache.page_size) * b for _ in eng.cache.groups]
        out.append({"dtype": dtype, "batch": b, "prompt_len": prompt_len, "tokens": tokens,
                    "decode_tok_s": dec["tokens_per_s"], "decode_ms_per_step": dec["ms_per_step"],
                    "decode_gbs": step_bytes / (dec["ms_per_step"] / 1e3) / 1e9, "ceiling_tok_s": ceiling,
                    "frac_of_hbm": dec["tokens_per_s"] / ceiling, "peaks": peaks["source"],
                    "prefill_tok_s": pre["tokens_per_s"], "prefill_ms": pre["ms"],
                    "pages_used": pages_used, "pages_total": pages_total})
        if profile:
            print(f"-- batch {b}", file=sys.stderr)
            print_profile(eng, [(7 * i + 1) % vocabulary(eng) for i in range(prompt_len)])
        del eng
        torch.cuda.empty_cache()
    return out


def run_cli_bench(args) -> int:
    import sys

    from .registry import get_architecture, load_config

    batches = [int(b) for b in str(args.batch).split(",") if b]
    config = load_config(args.weights)
    limit = get_architecture(config.architecture).build_spec(config).max_positions
    if limit is not None and args.prompt_len + args.tokens + max(3, args.warmup) > limit:
        print(f"prompt_len + tokens + warm-up must be <= {limit}", file=sys.stderr)
        return 2
    results = decode_points(args.weights, args.dtype, batches, args.prompt_len, args.tokens, args.warmup,
                            args.bandwidth_gbs, args.runs, getattr(args, "profile", False))
    stamp = provenance()
    for line in results:
        line["note"] = args.note
        print(f"{args.dtype} B={line['batch']}: prefill {line['prefill_tok_s']:.0f} tok/s | decode "
              f"{line['decode_tok_s']:.1f} tok/s ({line['decode_gbs']:.1f} GB/s) | {100 * line['frac_of_hbm']:.2f}% of "
              f"{line['ceiling_tok_s']:.0f} tok/s ceiling | pages {line['pages_used']} of {line['pages_total']}")
    if args.out:
        with open(args.out, "a") as fh:
            for line in results:
                fh.write(json.dumps({**line, **stamp}) + "\n")
    return 0
