"""The continuous-batching scheduler: which requests run in the next step, and how many of
their tokens.

The policy is the reference's ``run_continuous`` (crates/cli/src/metal_serve.rs:255-363):
  * requests wait first-come first-served; one is admitted while a place in the batch is free
    and the pool can hold its prompt plus one token, with one spare page per running request
    as room to grow; admission stops at the first waiting request that does not fit
    (metal_serve.rs:283-293).  Pages that earlier admissions will still take for their prompts
    count as taken (the reference counts free pages only);
  * every step takes one row for each request that has a single pending token (a decoding
    request), then portions of prompts, oldest first, under a token budget of
    min(prefill_budget, max_rows - decode rows); several prompts may share a step and a
    prompt may be cut anywhere (metal_serve.rs:299-315);
  * the prediction after a portion that does not end the prompt is not a token
    (metal_serve.rs:333-340); a request ends after its fixed number of new tokens
    (metal_serve.rs:345-347), at its end token if one is set, or when the context is full
    (crates/cli/src/main.rs:192-194).

When pages run out the reference's step fails and the whole run aborts
(crates/metal/src/batch.rs:244-248, metal_serve.rs:318).  Here the scheduler never lets a
step ask for more pages than are free.  Decoding requests get their pages first; prompt
portions are then cut down to the pages that are left (or left out of the step).  If a
decoding request finds no page, or nothing at all can move, the most recently admitted
running request is preempted: its pages and slot go back, it returns to the FRONT of the
waiting queue, and when it is admitted again all its tokens so far (prompt and generated)
are computed again.  A request that cannot go on even with the whole pool to itself is
ended with the reason "too_long".

The scheduler is host-only: it sees the cache manager's page counts, never the device.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

from ..cache.manager import CacheManager, RequestCache
from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    id: int
    prompt: List[int]
    params: SamplingParams
    #: generated tokens; while the engine runs a step ahead of its reads the newest may be a negative
    #: stand-in (its value follows one step later); a finished request that was reported holds values only
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    finish_reason: Optional[str] = None
    cache: Optional[RequestCache] = None
    #: how many of ``tokens`` are in the cache
    n_computed: int = 0
    n_preemptions: int = 0
    admitted_order: int = -1

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def n_pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.n_computed

    def next_tokens(self, n: int) -> List[int]:
        """The next ``n`` tokens that are not in the cache yet (without building the whole list)."""
        a, p = self.n_computed, len(self.prompt)
        if a >= p:
            return self.output[a - p:a - p + n]
        return (self.prompt[a:a + n] + self.output[:max(0, a + n - p)])[:n]


@dataclass
class ScheduledItem:
    request: Request
    n_tokens: int
    #: the portion reaches the request's last token, so its last logits give the next token
    samples: bool = False
    #: where in the request's output the step's token was put (set when the step is recorded)
    output_index: int = -1

    def __post_init__(self):
        self.samples = self.n_tokens == self.request.n_pending


@dataclass
class SchedulerStats:
    steps: int = 0
    decode_rows: int = 0
    prefill_rows: int = 0
    preemptions: int = 0
    dropped_portions: int = 0
    peak_pages: int = 0


#: the longest lone prompt portion that runs as a step of its own (see ``Scheduler.portions_alone``)
PORTION_ALONE_MAX_ROWS = 256


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int = 64, max_rows: int = 2048,
                 prefill_budget: int = 2048, headroom_pages: int = 1, max_positions: Optional[int] = None):
        self.cache = cache
        self.max_batch, self.max_rows = int(max_batch), int(max_rows)
        self.prefill_budget, self.headroom_pages = int(prefill_budget), int(headroom_pages)
        self.max_positions = max_positions
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.stats = SchedulerStats()
        self._ids = itertools.count()
        self._order = itertools.count()
        #: called with (request) after a slot was given to it, so that per-slot state can be set
        self.on_admit = None
        #: A lone short prompt portion beside decoded tokens runs as a step of its own, by turns with the
        #: decoded tokens (never two such steps in a row while tokens wait to be decoded).  The engine sets
        #: this where steps replay as graphs: a step of decoded tokens alone replays one, a step of one
        #: portion alone repeats its shape (the step function fills it up to 16 rows) and soon does too,
        #: while the two in one step are a shape that never comes again and is launched kernel by kernel.
        self.portions_alone = False
        self._portion_ran_alone = False

    # ------------------------------------------------------------------ requests in and out
    def add(self, prompt: Sequence[int], params: SamplingParams) -> Request:
        if len(prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        req = Request(next(self._ids), list(prompt), params)
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _pages(self, n_tokens: int) -> int:
        return -(-n_tokens // self.cache.page_size)

    def _free_pages(self) -> int:
        free = self.cache.pages_free()
        return min(free) if free else 1 << 30

    def _total_pages(self) -> int:
        sizes = [g.pool.n_pages for g in self.cache.groups]
        return min(sizes) if sizes else 1 << 30

    def _finish(self, req: Request, reason: str) -> None:
        if req.cache is not None:
            self.cache.close_request(req.cache)
            req.cache = None
        if req in self.running:
            self.running.remove(req)
        # a request that was preempted waits in the queue while its last token is still read one
        # step late: an end token found then must take it out of the queue as well, or it would be
        # admitted again and go on past its end
        if req.state == WAITING and req in self.waiting:
            self.waiting.remove(req)
        req.state, req.finish_reason = FINISHED, reason

    def _preempt(self, req: Request) -> None:
        self.cache.close_request(req.cache)
        req.cache = None
        req.n_computed = 0
        req.n_preemptions += 1
        req.state = WAITING
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.stats.preemptions += 1

    # ------------------------------------------------------------------ one decision
    def _admit(self, finished: List[Request]) -> None:
        while self.waiting and len(self.running) < self.max_batch:
            req = self.waiting[0]
            n = len(req.tokens)
            if self._pages(n + 1) > self._total_pages() or (
                    self.max_positions is not None and n > self.max_positions):
                self.waiting.popleft()
                self._finish(req, "too_long")
                finished.append(req)
                continue
            # pages already promised to running requests whose prompts are not in the cache yet
            promised = sum(max(0, self._pages(len(r.prompt) + len(r.output) + 1)
                               - max((len(b) for b in r.cache.blocks), default=0)) for r in self.running)
            need = self._pages(n + 1) + self.headroom_pages * len(self.running) + promised
            if self._free_pages() < need or self.cache.slots.n_free == 0:
                break  # head of the line waits; nobody overtakes it
            self.waiting.popleft()
            req.cache = self.cache.open_request()
            req.state = RUNNING
            req.admitted_order = next(self._order)
            self.running.append(req)
            if self.on_admit is not None:
                self.on_admit(req)

    def schedule(self) -> List[ScheduledItem]:
        """Decide the next step.  Returns the items to run (none if nothing is left to run);
        requests ended without running are in ``self.ended_without_step``."""
        self.ended_without_step: List[Request] = []
        ps = self.cache.page_size
        while True:
            self._admit(self.ended_without_step)
            free = list(self.cache.pages_free())

            def take(req: Request, n: int) -> bool:
                need = self.cache.pages_needed(req.cache, n)
                if any(k > f for k, f in zip(need, free)):
                    return False
                for g, k in enumerate(need):
                    free[g] -= k
                return True

            def max_fit(req: Request) -> int:
                room = [(len(b) + f) * ps - req.cache.n_tokens for b, f in zip(req.cache.blocks, free)]
                return min(room) if room else 1 << 30

            items: List[ScheduledItem] = []
            portions: List[ScheduledItem] = []
            decode_rows, starved = 0, False
            for req in self.running:
                if req.n_pending == 1:
                    if take(req, 1):
                        items.append(ScheduledItem(req, 1))
                        decode_rows += 1
                    else:
                        starved = True
            if not starved:
                budget = min(self.prefill_budget, self.max_rows - decode_rows)
                for req in self.running:
                    if req.n_pending > 1 and budget > 0:
                        n = min(req.n_pending, budget, max_fit(req))
                        if n >= 1 and take(req, n):
                            portions.append(ScheduledItem(req, n))
                            budget -= n
                        else:
                            self.stats.dropped_portions += 1
                if (self.portions_alone and items and len(portions) == 1
                        and portions[0].n_tokens <= PORTION_ALONE_MAX_ROWS):
                    if self._portion_ran_alone:      # the decoded tokens' turn; the portion waits a step
                        portions = []
                    else:
                        items, decode_rows = [], 0
                    self._portion_ran_alone = not self._portion_ran_alone
                else:
                    self._portion_ran_alone = False
                items += portions
                if items or not self.running:
                    break
            # a decoding request found no page, or nothing at all can move: make room
            victim = max(self.running, key=lambda r: r.admitted_order)
            if len(self.running) == 1:
                # alone in the pool and still no room for one more token: it can never go on
                self._finish(victim, "too_long")
                self.ended_without_step.append(victim)
            else:
                self._preempt(victim)
        if items:
            self.stats.steps += 1
            self.stats.decode_rows += decode_rows
            self.stats.prefill_rows += sum(i.n_tokens for i in items) - decode_rows
        used = self.cache.pages_used()
        self.stats.peak_pages = max(self.stats.peak_pages, max(used) if used else 0)
        return items

    # ------------------------------------------------------------------ after the step
    def on_step_done(self, items: Sequence[ScheduledItem], sampled: Sequence[int]) -> List[Request]:
        """Record what a step produced.  ``sampled`` holds one token for every item whose
        ``samples`` is true, in order.  Returns the requests that ended.

        A token may be a negative stand-in for a value that the host has not read yet (the engine
        runs one step ahead of its reads): it counts as a token for the length and context rules,
        and ``on_tokens_read`` puts the value in later and applies the end-token rule then."""
        ended: List[Request] = []
        it = iter(sampled)
        for item in items:
            req = item.request
            takes_token = item.samples
            req.n_computed += item.n_tokens
            if not takes_token:
                continue  # mid-prompt portion: its prediction is not a token
            tok = int(next(it))
            req.output.append(tok)
            item.output_index = len(req.output) - 1
            p = req.params
            if p.eos_token_id is not None and tok == p.eos_token_id:
                reason = "eos"
            elif len(req.output) >= p.max_new_tokens:
                reason = "length"
            elif self.max_positions is not None and len(req.prompt) + len(req.output) > self.max_positions:
                reason = "context_full"  # the new token has no position left to be fed at
            else:
                continue
            self._finish(req, reason)
            ended.append(req)
        return ended

    def on_tokens_read(self, items: Sequence[ScheduledItem], values: Sequence[int]) -> List[Request]:
        """The values of a step's tokens that were recorded as stand-ins.  Returns the requests that
        end at their end token now (their later tokens, computed ahead, are dropped)."""
        ended: List[Request] = []
        it = iter(values)
        for item in items:
            if not item.samples:
                continue
            tok, req, idx = int(next(it)), item.request, item.output_index
            if idx < 0 or idx >= len(req.output) or req.output[idx] >= 0:
                continue  # the request ended at an earlier token, or the value is known already
            req.output[idx] = tok
            eos = req.params.eos_token_id
            if eos is None or tok != eos:
                continue
            del req.output[idx + 1:]       # what was computed ahead of the end token is dropped
            if req.state == FINISHED:
                req.finish_reason = "eos"  # it had ended meanwhile for another reason, at this token or a later one
                continue
            self._finish(req, "eos")
            ended.append(req)
        return ended
