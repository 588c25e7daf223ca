"""Instrumentation: what every kernel launch of a step did, how long it took, and how close to the
roofline it ran.

The reference's forward pass reports every op to a trace sink with an estimate of the FLOPs and
bytes an ideal kernel would need (crates/core/src/trace.rs:52-115), and its ``--profile`` table and
``--trace-out`` file divide them by the measured time (crates/cli/src/report.rs:22-136).  Here
the kernel interface does the reporting: while a ``Recorder`` is active (``start``/``stop``), every
launcher call is bracketed by CUDA events and tagged with an ``Op``: kind, name, layer, shape, and
the same analytic counts.  Nothing is recorded, and nothing is paid, when no recorder is active.
Steps run eagerly while one is (a captured graph has no per-launch events).

Counts (a multiply-add is 2 FLOPs; bytes are what must be read and written once, in the dtypes the
engine uses):
  matmul   [M, K, N]: 2 M K N + M N FLOPs; weights + bias + input + output bytes
           (trace.rs:71-84, with the engine's element sizes instead of 4)
  attn     [queries, keys seen, width]: keys seen x (4 width + 5 heads) FLOPs; the queries, the
           outputs and every key and value of the requests once (trace.rs:101-115)
  ln, embed, kv_write, sample: elementwise, bytes in and out once (trace.rs:86-98)
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class Op:
    kind: str                      # embed | ln | matmul | attn | kv_write | lm_head | sample
    name: str                      # qkv, attn, attn_proj, fc, fc_proj, lm_head, ln, embed, ...
    dims: Tuple[int, int, int]
    flops: float
    bytes: float
    layer: int = -1                # index of the schedule entry, -1 outside the layers


@dataclass
class Event:
    op: Op
    launcher: str
    start: "torch.cuda.Event"
    end: "torch.cuda.Event"
    step: int


class Recorder:
    """Collects the launches of the steps run while it is active."""

    def __init__(self):
        self.events: List[Event] = []
        self.step = 0
        self.layer = -1
        self.name = ""
        self.origin = torch.cuda.Event(enable_timing=True)
        self.origin.record()
        #: (phase, rows, context after the step, first event index) per step
        self.steps: List[Tuple[str, int, int, int]] = []

    def begin_step(self, phase: str, rows: int, context: int) -> None:
        self.steps.append((phase, rows, context, len(self.events)))
        self.step = len(self.steps) - 1

    def add(self, op: Op, launcher: str, e0, e1) -> None:
        op.layer = self.layer
        if self.name and op.kind == "matmul":
            op.name = self.name
            if op.name == "lm_head":
                op.kind = "lm_head"
        self.events.append(Event(op, launcher, e0, e1, self.step))

    # ------------------------------------------------------------------ summaries
    def table(self, phase: Optional[str] = None) -> Dict[str, Tuple[int, float, float, float]]:
        """name -> (calls, ms, flops, bytes), over the steps of ``phase`` (all if None)."""
        torch.cuda.synchronize()
        out: Dict[str, Tuple[int, float, float, float]] = {}
        for e in self.events:
            if phase is not None and self.steps and self.steps[e.step][0] != phase:
                continue
            n, ms, fl, by = out.get(e.op.name, (0, 0.0, 0.0, 0.0))
            out[e.op.name] = (n + 1, ms + e.start.elapsed_time(e.end), fl + e.op.flops, by + e.op.bytes)
        return out


_current: Optional[Recorder] = None


def start() -> Recorder:
    global _current
    from .kernels import ops
    _current = ops._rec = Recorder()
    return _current


def stop() -> None:
    global _current
    from .kernels import ops
    _current = ops._rec = None


def current() -> Optional[Recorder]:
    return _current


def format_table(table, peak_gbs: float, peak_tflops: float, title: str = "") -> str:
    """The reference's per-op table (report.rs:39-57) with one more column: the fraction of the
    roofline, i.e. the time an ideal kernel would need (the slower of FLOPs / peak and bytes / peak)
    over the time measured."""
    total = sum(ms for _, ms, _, _ in table.values()) or 1e-12
    lines = []
    if title:
        lines.append(title)
    lines.append(f"  {'op':<11} {'calls':>6} {'ms':>10} {'share':>7} {'GFLOP/s':>10} {'GB/s':>9} {'of roof':>8}")
    for name, (n, ms, fl, by) in sorted(table.items(), key=lambda kv: -kv[1][1]):
        s = ms / 1e3 or 1e-12
        ideal = max(fl / (peak_tflops * 1e12), by / (peak_gbs * 1e9))
        lines.append(f"  {name:<11} {n:>6} {ms:>10.3f} {100 * ms / total:>6.1f}% {fl / s / 1e9:>10.1f} {by / s / 1e9:>9.1f} "
                     f"{ideal / s:>8.3f}")
    lines.append(f"  {'total':<11} {'':>6} {total:>10.3f}")
    return "\n".join(lines)


def write_jsonl(rec: Recorder, path: str, header: dict, tokens: List[dict], kv: Optional[dict] = None) -> None:
    """The run as one JSON object a line, in the reference's event schema (report.rs:69-136):
    ``run_start``, one ``op`` per launch (times in microseconds since the run began), ``kv``,
    one ``token`` per step, ``run_end``."""
    torch.cuda.synchronize()
    lines = [dict(t="run_start", run=0, ts_us=0, **header)]
    step_ms: Dict[int, float] = {}
    for e in rec.events:
        dur = e.start.elapsed_time(e.end)
        step_ms[e.step] = step_ms.get(e.step, 0.0) + dur
        lines.append({"t": "op", "run": 0, "tok": e.step, "layer": e.op.layer, "op": e.op.name, "kind": e.op.kind,
                      "start_us": round(1e3 * rec.origin.elapsed_time(e.start), 3), "dur_us": round(1e3 * dur, 3),
                      "flops": int(e.op.flops), "bytes": int(e.op.bytes), "shape": list(e.op.dims)})
    if kv:
        lines.append(dict(t="kv", run=0, **kv))
    prefill_ms, decode_ms, n_decode = 0.0, 0.0, 0
    for i, (phase, rows, context, _) in enumerate(rec.steps):
        tok = tokens[i] if i < len(tokens) else {}
        lines.append({"t": "token", "run": 0, "idx": i, "phase": phase, "dur_us": round(1e3 * step_ms.get(i, 0.0), 3),
                      "n_computed": rows, "context_len": context, **tok})
        if phase == "prefill":
            prefill_ms += step_ms.get(i, 0.0)
        else:
            decode_ms += step_ms.get(i, 0.0)
            n_decode += 1
    lines.append({"t": "run_end", "run": 0, "n_prompt": rec.steps[0][1] if rec.steps else 0, "n_gen": len(rec.steps),
                  "prefill_ms": prefill_ms, "decode_tok_s": n_decode / (decode_ms / 1e3) if decode_ms else 0.0})
    with open(path, "w") as fh:
        for line in lines:
            fh.write(json.dumps(line) + "\n")
