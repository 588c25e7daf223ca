"""Drives ``bin/trace_run`` as a user would: one JSON line per step on its standard input, the
next line only after ``done <step>`` came back, logits read from the files it writes."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class TraceSession:
    def __init__(self, model_dir, dtype, out_dir, max_tokens, vocab, extra=()):
        self.out_dir, self.vocab = str(out_dir), vocab
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", self.out_dir,
             "--max-tokens", str(max_tokens), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step_no = 0
        #: per request id: {position: logits row}
        self.logits = {}
        self.pos = {}

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want); positions follow from what was sent before."""
        rec = {"step": self.step_no, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.step_no}", f"trace_run answered {line!r} (exit code {self.proc.poll()})"
        n_want = sum(len(w) for _, _, w in entries)
        path = os.path.join(self.out_dir, f"{self.step_no}.f32")
        if n_want:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == n_want * self.vocab, f"{path}: {data.size} floats for {n_want} rows"
            rows = torch.from_numpy(data.reshape(n_want, self.vocab).copy())
            k = 0
            for i, t, w in entries:
                p0 = self.pos.get(i, 0)
                for j in w:
                    self.logits.setdefault(i, {})[p0 + j] = rows[k]
                    k += 1
        else:
            assert not os.path.exists(path)
        for i, t, _ in entries:
            self.pos[i] = self.pos.get(i, 0) + len(t)
        for i in end:
            self.pos.pop(i, None)
        self.step_no += 1

    def close(self):
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=60)
        assert rc == 0, f"trace_run exited with {rc}"

    def stacked(self, rid, n):
        """Logits of request ``rid`` at positions 0..n-1 as one tensor."""
        got = self.logits[rid]
        assert sorted(got) == list(range(n)), f"request {rid}: positions {sorted(got)[:5]}... of {n}"
        return torch.stack([got[p] for p in range(n)])

    def pages(self):
        """With ``--log-pages``: [{request id: [page ids per cache group]}] for every step."""
        with open(os.path.join(self.out_dir, "pages.jsonl")) as fh:
            return [json.loads(line)["pages"] for line in fh]


def max_diff(a, b):
    return float((a - b).abs().max())


def max_kl(ref, got):
    """The largest KL(plain || engine) of the next-token distributions over the rows, in float64
    (the reference's second measure of a reduced-precision path: crates/core/tests/reference.rs:29-45)."""
    lp = torch.log_softmax(ref.double(), dim=-1)
    lq = torch.log_softmax(got.double(), dim=-1)
    return float((lp.exp() * (lp - lq)).sum(-1).max())
