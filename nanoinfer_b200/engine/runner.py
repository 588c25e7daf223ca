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
     order of the items and of their ``want`` lists, or, when a sampler is given, one sampled
     token per logits row.

Steps are launch-bound (a decode step is a hundred small kernels), so the kernels of a step are
captured in a CUDA graph the second time its shape is seen, and replayed from then on (the
reference keeps its decode loop on the GPU for the same reason, ``decode_resident``,
batch.rs:322-363).  What a graph bakes in is only the shape of the step: the tables it reads are
rewritten before every replay.
"""
from __future__ import annotations

import contextlib
import gc
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..kernels import ops
from ..models.model import Model
from ..parts.base import StepContext, StepLimits, Workspace


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


@dataclass
class _Layout:
    """Where each table of a step lies in the packed int32 buffer."""
    T: int
    E: int
    M: int
    n_plan: int
    tok: int = 0
    pos: int = 0
    ent: int = 0
    start: int = 0
    pos0: int = 0
    slot: int = 0
    lrow: int = 0
    lslot: int = 0
    plan: int = 0
    tabs: Tuple[int, ...] = ()
    total: int = 0


@dataclass
class _Captured:
    graph: "torch.cuda.CUDAGraph"
    logits: Optional[torch.Tensor]
    tokens: Optional[torch.Tensor]
    launches: int


#: batches of more than PAD_FROM single tokens are padded to a multiple of PAD_TO rows
PAD_FROM, PAD_TO = 8, 8
#: a step that carries prompt portions is filled up to a multiple of this many rows with rows of no
#: request (entry -1: no keys or values kept, no attention, nobody's logits), so that steps which differ
#: by a few tokens share a graph: a prompt of 70 tokens and one of 80 are both a step of 80 rows
PAD_ROWS_TO = 16


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, max_rows: int = 2048, max_entries: int = 64,
                 check_status: bool = True, use_graphs: bool = True, max_graphs: int = 96):
        if model.device is None:
            raise ValueError("the model has no weights yet: load them first")
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_rows, self.max_entries = int(max_rows), int(max_entries)
        self.check_status = check_status
        on_gpu = self.device.type == "cuda"
        # a mixer may plan its work on the host in ways that a graph would freeze: every mixer says
        # whether its launches follow from the step's shape alone
        self.use_graphs = bool(use_graphs) and on_gpu and model.capture_safe()
        self.max_graphs = max_graphs
        self.workspace = Workspace(self.device)
        #: what each kind of part derives on the host from a step's shape, by name
        self._planners = model.step_planners()
        # Scratch is sized here, once, for the largest step: a captured graph holds raw addresses,
        # so no buffer may move while graphs are live (the reference sizes every buffer once as
        # well, from max_rows and max_seqs: crates/metal/src/batch.rs:159-193).
        limit = model.max_positions or max(cache.max_blocks, default=0) * cache.page_size
        model.reserve(self.workspace, StepLimits(self.max_rows, self.max_entries, int(limit), model.dtype))
        self._graph_generation = self.workspace.generation
        self.status = ops.status_word() if on_gpu else torch.zeros(1, dtype=torch.int32)
        n_tables = sum(self.max_entries * mb for mb in cache.max_blocks)
        cap = 7 * self.max_rows + 8 * self.max_entries + 16 + n_tables
        # A ring of pinned staging buffers: a buffer is written again only after the copy that
        # last read it has finished.
        self._ring = []
        for _ in range(4):
            host = torch.empty(cap, dtype=torch.int32)
            if on_gpu:
                host = host.pin_memory()
            self._ring.append((host, host.numpy(), torch.cuda.Event() if on_gpu else None))
        self._ring_next = 0
        self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self._arange = np.arange(self.max_entries + 1, dtype=np.int32)
        self._graphs: Dict[tuple, _Captured] = {}
        #: how often the graphs had to be dropped because a scratch buffer was replaced
        self.graph_drops = 0
        self._seen: Dict[tuple, int] = {}
        self.steps_run = 0
        self.graph_replays = 0
        self.padded_steps = 0
        #: steps with prompt portions that were filled up with rows of no request
        self.row_padded_steps = 0
        self.last_meta_bytes = 0
        self.last_logit_slot = None
        #: kernel launches of the last step (counted by the kernel interface)
        self.launches_last_step = 0

    # ------------------------------------------------------------------ checks
    def _validate(self, items: Sequence[StepItem], feedback: bool = False) -> int:
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
                    # the one exception: a lone token -(slot + 1) stands for the token that the step
                    # before sampled for this request and that is still on the device
                    if feedback and n == 1 and int(t) == -(r.slot + 1):
                        continue
                    raise BadToken(f"token id {t} is out of vocabulary")
            if limit is not None and r.n_tokens + n > limit:
                raise ContextFull(f"context full: {r.n_tokens + n} tokens exceeds max {limit}")
            for w in it.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"want index {w} is outside the item's {n} tokens")
            if len(set(int(w) for w in it.want)) != len(it.want):
                raise StepError("a want index is given twice")   # (one logits row per place, whatever the mix)
            n_rows += n
        if n_rows > self.max_rows:
            raise TooManyRows(f"{n_rows} rows > max_rows {self.max_rows}")
        return n_rows

    # ------------------------------------------------------------------ packing
    def _layout(self, T: int, E: int, M: int, n_plan: int) -> _Layout:
        """[tokens | positions | row_entry | entry_start | pos0 | slot | logit_rows | logit_slot |
        attention plan | block tables], the tables 16-byte aligned."""
        lay = _Layout(T, E, M, n_plan)
        lay.tok, lay.pos, lay.ent = 0, T, 2 * T
        lay.start = 3 * T
        lay.pos0 = lay.start + E + 1
        lay.slot = lay.pos0 + E
        lay.lrow = lay.slot + E
        lay.lslot = lay.lrow + M
        lay.plan = lay.lslot + M
        o = lay.plan + n_plan
        o += (-o) % 4
        tabs = []
        for mb in self.cache.max_blocks:
            tabs.append(o)
            o += E * mb
        lay.tabs, lay.total = tuple(tabs), o
        return lay

    def _plans(self, starts, pos0s):
        """The step's plans by name, and their words in one list."""
        plans = {name: make(starts, pos0s, self.use_graphs) for name, make in self._planners.items()}
        words: List[int] = []
        for p in plans.values():
            words += p.words
        return plans, words

    def _drop_graphs(self) -> None:
        """A scratch buffer was replaced by a larger one: every captured graph may hold the old
        address.  Drop them all; only then is the replaced memory let go."""
        if self._graphs:
            self.graph_drops += 1
        self._graphs.clear()
        self._seen.clear()
        torch.cuda.synchronize(self.device)      # nothing in flight still uses the old buffers
        self.workspace.release_retired()
        self._graph_generation = self.workspace.generation

    def _context(self, lay: _Layout, plans, starts, pos0s, slots, max_q: int, max_kv: int, sampler=None):
        dev = self._meta_dev
        T, E, M = lay.T, lay.E, lay.M
        ctx = StepContext(
            n_rows=T, n_entries=E, max_rows=self.max_rows,
            tokens=dev[lay.tok:lay.tok + T], positions=dev[lay.pos:lay.pos + T], row_entry=dev[lay.ent:lay.ent + T],
            entry_start=dev[lay.start:lay.start + E + 1], entry_pos0=dev[lay.pos0:lay.pos0 + E],
            entry_slot=dev[lay.slot:lay.slot + E], status=self.status, workspace=self.workspace,
            host_entry_start=starts, host_entry_pos0=pos0s, host_entry_slot=slots,
            max_q_len=max_q, max_kv_len=max_kv, token_feedback=getattr(sampler, "last_token", None),
        )
        at = lay.plan
        for p in plans.values():
            p.bind(dev[at:at + len(p.words)] if p.words else None)
            at += len(p.words)
        ctx.plans = plans
        tables = [dev[off:off + E * mb].view(E, mb) for off, mb in zip(lay.tabs, self.cache.max_blocks)]
        caches = self.cache.layer_views(tables)
        logit_rows = dev[lay.lrow:lay.lrow + M] if M else None
        logit_slot = dev[lay.lslot:lay.lslot + M] if M else None
        return ctx, caches, logit_rows, logit_slot

    def _run(self, ctx, caches, logit_rows, logit_slot, M: int, sampler):
        with ops.bound_stream() if self.device.type == "cuda" else contextlib.nullcontext():
            logits = self.model.forward(ctx, caches, self.cache.state_tensors, logit_rows, M)
            tokens = sampler.sample(logits, logit_slot) if (sampler is not None and logits is not None) else None
        return logits, tokens

    # ------------------------------------------------------------------ the step
    def step(self, items: Sequence[StepItem], sampler=None) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits [wanted, vocab] (None if nothing is wanted), or with
        ``sampler`` the sampled tokens, int32 [wanted].  Either lives in the engine's scratch memory
        and is valid until the next step."""
        T = self._validate(items, feedback=sampler is not None and hasattr(sampler, "last_token"))
        self.cache.append([(it.request, len(it.tokens)) for it in items])  # all pages of the step, or none
        E = len(items)
        decode_only = T == E
        host, buf, copied = self._ring[self._ring_next]
        self._ring_next = (self._ring_next + 1) % len(self._ring)
        if copied is not None:
            copied.synchronize()  # returns at once unless the GPU is four steps behind

        want_rows: List[int] = []
        n_pad = 0
        if decode_only:
            pos0s = [it.request.n_tokens for it in items]
            slots = [it.request.slot for it in items]
            want_rows = [e for e, it in enumerate(items) if len(it.want)]
            tokens_in = [it.tokens[0] for it in items]
            # A batch of more than PAD_FROM single tokens, all wanted, is filled up to the next multiple
            # of PAD_TO with rows of a request that is none: token 0 at position 0, key and value
            # into the cache's spare page, state in its spare slot.  Batches that shrink and grow by
            # a request then share a graph instead of each running uncaptured, then being captured.
            if (self.use_graphs and self.cache.pad_slot is not None and E > PAD_FROM and len(want_rows) == E):
                n_pad = min(-(-E // PAD_TO) * PAD_TO, self.max_entries, self.max_rows) - E
                tokens_in += [0] * n_pad
                pos0s += [0] * n_pad
                slots += [self.cache.pad_slot] * n_pad
                want_rows += range(E, E + n_pad)
                E = T = E + n_pad
                self.padded_steps += 1 if n_pad else 0
            starts = self._arange[:E + 1].tolist()
            M = len(want_rows)
            max_q, max_kv = 1, max(pos0s) + 1
            plans, plan_words = self._plans(starts, pos0s)
            lay = self._layout(T, E, M, len(plan_words))
            buf[lay.tok:lay.tok + T] = tokens_in
            buf[lay.pos:lay.pos + T] = pos0s
            buf[lay.ent:lay.ent + T] = self._arange[:E]
            buf[lay.lrow:lay.lrow + M] = want_rows
            buf[lay.lslot:lay.lslot + M] = [slots[e] for e in want_rows]
        else:
            M = sum(len(it.want) for it in items)
            starts, pos0s, slots = [0], [], []
            max_q = max_kv = 0
            for it in items:
                n, p0 = len(it.tokens), it.request.n_tokens
                starts.append(starts[-1] + n)
                pos0s.append(p0)
                slots.append(it.request.slot)
                max_q, max_kv = max(max_q, n), max(max_kv, p0 + n)
            plans, plan_words = self._plans(starts, pos0s)
            n_real = T
            if self.use_graphs:
                T = min(-(-T // PAD_ROWS_TO) * PAD_ROWS_TO, self.max_rows)
            lay = self._layout(T, E, M, len(plan_words))
            if T > n_real:                      # rows of no request behind the last entry's
                buf[lay.tok + n_real:lay.tok + T] = 0
                buf[lay.pos + n_real:lay.pos + T] = 0
                buf[lay.ent + n_real:lay.ent + T] = -1
                self.row_padded_steps += 1
            lrow = lay.lrow
            for e, it in enumerate(items):
                a, n, p0 = starts[e], len(it.tokens), pos0s[e]
                buf[lay.tok + a:lay.tok + a + n] = it.tokens
                buf[lay.pos + a:lay.pos + a + n] = np.arange(p0, p0 + n, dtype=np.int32)
                buf[lay.ent + a:lay.ent + a + n] = e
                for w in it.want:
                    buf[lrow] = a + int(w)
                    buf[lrow + M] = slots[e]
                    lrow += 1
        buf[lay.start:lay.start + E + 1] = starts
        buf[lay.pos0:lay.pos0 + E] = pos0s
        buf[lay.slot:lay.slot + E] = slots
        if lay.n_plan:
            buf[lay.plan:lay.plan + lay.n_plan] = plan_words
        for gi, (off, mb) in enumerate(zip(lay.tabs, self.cache.max_blocks)):
            tab = buf[off:off + E * mb].reshape(E, mb)
            for e, it in enumerate(items):
                tab[e] = it.request.table_rows[gi]
            if n_pad:
                tab[E - n_pad:] = -1
                tab[E - n_pad:, 0] = self.cache.pad_page[gi]
        self.last_meta_bytes = 4 * lay.total
        self._meta_dev[:lay.total].copy_(host[:lay.total], non_blocking=True)
        if copied is not None:
            copied.record()
        self.last_logit_slot = self._meta_dev[lay.lslot:lay.lslot + M] if M else None

        # a graph bakes in the shape of the step only: row, entry and logits counts, and what each
        # plan says it fixes (for attention: how the rows split into single tokens and prompt tiles,
        # and the split of the decode keys)
        key = None
        if self.use_graphs:
            if self.workspace.generation != self._graph_generation:
                self._drop_graphs()
            key = (T, E, M, tuple((name, p.graph_key()) for name, p in plans.items()), id(sampler),
                   getattr(sampler, "any_sampled", None), getattr(sampler, "generation", None))
        elif self.workspace.retired:
            self.workspace.release_retired()     # no graphs: the stream's order alone protects old buffers
        cap = self._graphs.get(key) if key is not None else None
        if cap is not None:
            self._graphs[key] = self._graphs.pop(key)   # most recently used last
            cap.graph.replay()
            self.graph_replays += 1
            logits, tokens = cap.logits, cap.tokens
            self.launches_last_step = cap.launches
        else:
            args = self._context(lay, plans, starts, pos0s, slots, max_q, max_kv, sampler)
            n_seen = self._seen.get(key, 0) if key is not None else 0
            # A shape that was run already (scratch is sized, attributes are set) is captured: a batch
            # of single tokens the second time it comes, since it will come again step after step, and so
            # a lone prompt portion (filled up to 16 rows, its shape is one of a few dozen); other steps
            # with prompt portions the fourth time only (most such shapes of a serving mix come
            # once or twice, and a capture costs about two uncaptured steps).  The new graph takes the
            # place of the one that has not been used for the longest time if the table is full.
            if key is not None and n_seen >= (1 if decode_only or E == 1 else 3):
                while len(self._graphs) >= self.max_graphs:
                    del self._graphs[next(iter(self._graphs))]
                graph = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                # Nothing but kernel launches happens while capturing, but the garbage collector may
                # wake up at any allocation and release pinned memory or events of an engine that
                # is no longer used, which a strict capture does not survive: it stays off meanwhile.
                gc_was_on = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                        logits, tokens = self._run(*args, M, sampler)
                finally:
                    if gc_was_on:
                        gc.enable()
                if self.workspace.generation != self._graph_generation or (
                        getattr(sampler, "generation", None) != key[-1]):
                    # a buffer moved while the step was being captured (a shape that was run before
                    # never does this; a part that sizes scratch by something else might): the new
                    # graph mixes old and new addresses, so it is not kept, and the step runs plainly
                    del graph
                    self._drop_graphs()
                    logits, tokens = self._run(*args, M, sampler)
                else:
                    cap = _Captured(graph, logits, tokens, ops.launch_count() - before)
                    self._graphs[key] = cap
                    graph.replay()
                    self.graph_replays += 1
                    self.launches_last_step = cap.launches
            else:
                before = ops.launch_count()
                logits, tokens = self._run(*args, M, sampler)
                self.launches_last_step = ops.launch_count() - before
                if key is not None:
                    if len(self._seen) >= 64 * self.max_graphs:   # shapes that never came back
                        self._seen.clear()
                    self._seen[key] = n_seen + 1

        for it in items:
            self.cache.commit(it.request, len(it.tokens))
        self.steps_run += 1
        if self.check_status:
            self.raise_on_status()
        out = tokens if sampler is not None else logits
        return out[:M - n_pad] if n_pad and out is not None else out

    def raise_on_status(self) -> None:
        """Read the device status word (this waits for the step) and raise if a kernel flagged a fault."""
        code = int(self.status.item())
        if code != ops.STATUS_OK:
            self.status.zero_()
            what = {ops.STATUS_BAD_PAGE: "a kernel met a page index outside its pool",
                    ops.STATUS_WAIT_TIMEOUT: "a kernel gave up waiting on a barrier"}.get(code, f"code {code}")
            raise RuntimeError(f"device status after step {self.steps_run}: {what}")
