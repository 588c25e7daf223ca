"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step is a list of items; each item appends some tokens to one request and names the places
among them whose logits are wanted.  Items may be portions of prompts, cut anywhere, beside
single decoded tokens; one row of the batch is one token of one request, as in the reference's
batch engine (crates/metal/src/batch.rs:1-15, ``Batch::step`` batch.rs:259-315).  The step

  1. checks everything first (live request, tokens in the vocabulary, context and row limits,
     pages for ALL items) and changes nothing if a check fails (the reference checks as it
     goes, batch.rs:281-305);
  2. takes the pages, packs the row and entry tables into one pinned buffer and sends it to
     the device in one copy;
  3. runs the model on exactly these rows;
  4. commits the new lengths (batch.rs:270) and returns float32 logits [wanted, vocab] in the
     order of the items and of their ``want`` lists.  Sampling is a separate call on them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, PoolExhausted, RequestCache
from ..kernels import ops
from ..models.model import Model
from ..parts.base import StepContext, Workspace


class StepError(ValueError):
    """The step was refused; nothing was changed."""


class BadToken(StepError):
    pass


class ContextFull(StepError):
    pass


class TooManyRows(StepError):
    pass


@dataclass
class StepItem:
    request: RequestCache
    tokens: Sequence[int]
    #: indices into ``tokens`` whose logits are wanted (may be empty)
    want: Sequence[int] = field(default_factory=list)


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, max_rows: int = 2048, max_entries: int = 64,
                 check_status: bool = True):
        if model.device is None:
            raise ValueError("the model has no weights yet: load them first")
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_rows, self.max_entries = int(max_rows), int(max_entries)
        self.check_status = check_status
        self.workspace = Workspace(self.device)
        self.status = ops.status_word() if self.device.type == "cuda" else torch.zeros(1, dtype=torch.int32)
        n_tables = sum(self.max_entries * mb for mb in cache.max_blocks)
        cap = 7 * self.max_rows + 8 * self.max_entries + 16 + n_tables
        # A ring of pinned staging buffers: a buffer is written again only after the copy that
        # last read it has finished.
        on_gpu = self.device.type == "cuda"
        self._ring = []
        for _ in range(4):
            host = torch.empty(cap, dtype=torch.int32)
            if on_gpu:
                host = host.pin_memory()
            self._ring.append((host, host.numpy(), torch.cuda.Event() if on_gpu else None))
        self._ring_next = 0
        self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.last_meta_bytes = 0
        self.last_logit_slot = None

    # ------------------------------------------------------------------ checks
    def _validate(self, items: Sequence[StepItem]) -> int:
        if not items:
            raise StepError("a step needs at least one item")
        if len(items) > self.max_entries:
            raise TooManyRows(f"{len(items)} items > max_entries {self.max_entries}")
        vocab, limit = self.model.vocab_size, self.model.max_positions
        seen = set()
        n_rows = 0
        for it in items:
            r = it.request
            if not r.live:
                raise StepError("a request of the step is not live")
            if id(r) in seen:
                raise StepError("a request appears twice in one step")
            seen.add(id(r))
            n = len(it.tokens)
            if n == 0:
                raise StepError("empty work item")
            for t in it.tokens:
                if not 0 <= int(t) < vocab:
                    raise BadToken(f"token id {t} is out of vocabulary")
            if limit is not None and r.n_tokens + n > limit:
                raise ContextFull(f"context full: {r.n_tokens + n} tokens exceeds max {limit}")
            for w in it.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"want index {w} is outside the item's {n} tokens")
            n_rows += n
        if n_rows > self.max_rows:
            raise TooManyRows(f"{n_rows} rows > max_rows {self.max_rows}")
        return n_rows

    # ------------------------------------------------------------------ the step
    def step(self, items: Sequence[StepItem]) -> Optional[torch.Tensor]:
        T = self._validate(items)
        work = [(it.request, len(it.tokens)) for it in items]
        try:
            self.cache.append(work)  # all pages of the step, or none
        except PoolExhausted:
            raise
        E = len(items)
        M = sum(len(it.want) for it in items)

        # ---- pack the tables:
        # [tokens | positions | row_entry | entry_start | pos0 | slot | logit_rows | logit_slot | attention plan |
        #  block tables]
        host, buf, copied = self._ring[self._ring_next]
        self._ring_next = (self._ring_next + 1) % len(self._ring)
        if copied is not None:
            copied.synchronize()  # returns at once unless the GPU is four steps behind
        o_tok, o_pos, o_ent = 0, T, 2 * T
        o_start = 3 * T
        o_pos0 = o_start + E + 1
        o_slot = o_pos0 + E
        o_lrow = o_slot + E
        o_lslot = o_lrow + M
        o_plan = o_lslot + M
        row = 0
        lrow = o_lrow
        starts, pos0s, slots = [], [], []
        max_q = max_kv = 0
        for e, it in enumerate(items):
            n, p0 = len(it.tokens), it.request.n_tokens
            buf[o_tok + row:o_tok + row + n] = it.tokens
            buf[o_pos + row:o_pos + row + n] = np.arange(p0, p0 + n, dtype=np.int32)
            buf[o_ent + row:o_ent + row + n] = e
            for w in it.want:
                buf[lrow] = row + int(w)
                buf[lrow + M] = it.request.slot
                lrow += 1
            starts.append(row)
            pos0s.append(p0)
            slots.append(it.request.slot)
            max_q, max_kv = max(max_q, n), max(max_kv, p0 + n)
            row += n
        starts.append(row)
        buf[o_start:o_start + E + 1] = starts
        buf[o_pos0:o_pos0 + E] = pos0s
        buf[o_slot:o_slot + E] = slots
        # which rows are single decoded tokens, which are prompt portions (64-row tiles)
        plan = ops.AttentionPlan(starts, pos0s, self.device, into=buf)
        n_plan = len(plan.host)
        buf[o_plan:o_plan + n_plan] = plan.host
        o_tab = o_plan + n_plan
        o_tab += (-o_tab) % 4  # keep the tables 16-byte aligned
        tab_offsets = []
        o = o_tab
        for gi, mb in enumerate(self.cache.max_blocks):
            tab = buf[o:o + E * mb].reshape(E, mb)
            tab.fill(-1)
            for e, it in enumerate(items):
                blocks = it.request.blocks[gi]
                tab[e, :len(blocks)] = blocks
            tab_offsets.append(o)
            o += E * mb
        n_meta = o
        self.last_meta_bytes = 4 * n_meta
        dev = self._meta_dev
        dev[:n_meta].copy_(host[:n_meta], non_blocking=True)
        if copied is not None:
            copied.record()

        ctx = StepContext(
            n_rows=T, n_entries=E, max_rows=self.max_rows,
            tokens=dev[o_tok:o_tok + T], positions=dev[o_pos:o_pos + T], row_entry=dev[o_ent:o_ent + T],
            entry_start=dev[o_start:o_start + E + 1], entry_pos0=dev[o_pos0:o_pos0 + E],
            entry_slot=dev[o_slot:o_slot + E], status=self.status, workspace=self.workspace,
            host_entry_start=starts, host_entry_pos0=pos0s, host_entry_slot=slots,
            max_q_len=max_q, max_kv_len=max_kv,
        )
        plan.bind(dev[o_plan:o_plan + n_plan])
        ctx.attention_plan = plan
        tables = [dev[off:off + E * mb].view(E, mb) for off, mb in zip(tab_offsets, self.cache.max_blocks)]
        caches = self.cache.layer_views(tables)
        logit_rows = dev[o_lrow:o_lrow + M] if M else None
        #: the state slot of the request behind each logits row (for the sampler)
        self.last_logit_slot = dev[o_lslot:o_lslot + M] if M else None
        logits = self.model.forward(ctx, caches, self.cache.state_tensors, logit_rows, M)

        for it in items:
            self.cache.commit(it.request, len(it.tokens))
        self.steps_run += 1
        if self.check_status:
            self.raise_on_status()
        return logits

    def raise_on_status(self) -> None:
        """Read the device status word (this waits for the step) and raise if a kernel flagged a fault."""
        code = int(self.status.item())
        if code != ops.STATUS_OK:
            self.status.zero_()
            what = {ops.STATUS_BAD_PAGE: "a kernel met a page index outside its pool",
                    ops.STATUS_WAIT_TIMEOUT: "a kernel gave up waiting on a barrier"}.get(code, f"code {code}")
            raise RuntimeError(f"device status after step {self.steps_run}: {what}")
