"""The Python entry point: a model folder in, generated token ids out.

``Engine`` owns the model, the cache manager, the step function, the scheduler and the
sampler.  ``generate`` is the loop of the reference's ``generate`` command
(crates/cli/src/main.rs:151-195: feed the prompt, sample, feed the sampled token, until the
wanted number of tokens or a full context) run for many requests at once by the
continuous-batching scheduler (crates/cli/src/metal_serve.rs:255-363).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..sampling.sampler import Sampler, SamplingParams
from .runner import ModelRunner, StepItem
from .scheduler import Request, Scheduler

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


#: largest model (bytes of weights a step reads) for which a lone short prompt portion runs as a step of its own
PORTIONS_ALONE_MAX_WEIGHT_BYTES = 512 << 20


class Engine:
    def __init__(self, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", device: str = "cuda",
                 max_tokens: Optional[int] = None, max_batch: int = 64, max_rows: int = 2048,
                 prefill_budget: Optional[int] = None, page_size: int = 16, check_status: bool = False,
                 use_graphs: bool = True, run_ahead: bool = True):
        """``max_tokens``: how many tokens all live requests may hold in the cache together
        (default: ``max_batch`` full contexts).  ``prefill_budget``: most prompt tokens per step
        (default ``max_rows``).  ``run_ahead``: launch a step before the host has read the tokens
        of the step before it (they pass from sampler to embedding on the device), so that the
        host's scheduling and packing overlap the device's work; the tokens are the same."""
        from .. import load_model

        if isinstance(dtype, str):
            dtype = _DTYPES[dtype]
        self.device = torch.device(device)
        self.model = load_model(model_dir, dtype, self.device)
        limit = self.model.max_positions
        if max_tokens is None:
            max_tokens = max_batch * (limit if limit is not None else 2048)
        self.cache = CacheManager(self.model.kv_needs(), self.model.state_needs(), max_tokens=max_tokens,
                                  max_requests=max_batch, page_size=page_size, dtype=dtype, device=self.device,
                                  max_positions=limit, padding=True)
        self.runner = ModelRunner(self.model, self.cache, max_rows=max_rows, max_entries=max_batch,
                                  check_status=check_status, use_graphs=use_graphs)
        self.sampler = Sampler(self.cache.slots)
        self.scheduler = Scheduler(self.cache, max_batch=max_batch, max_rows=max_rows,
                                   prefill_budget=prefill_budget or max_rows, max_positions=limit)
        self.scheduler.on_admit = self._on_admit
        # (where a step of decoded tokens and a prompt portion together is bound by the host that launches it kernel
        # by kernel, not by the device: measured with requests arriving at a steady rate, GPT-2 small answers the
        # first token after 2 ms instead of 137 ms and a token takes 0.8 ms instead of 1.2 ms; at GPT-2 XL's size
        # such a step is bound by the device and the portion rides along for nothing, so it stays one step)
        from ..measure import weight_bytes_per_step
        self.scheduler.portions_alone = (self.runner.use_graphs
                                         and weight_bytes_per_step(self.model) <= PORTIONS_ALONE_MAX_WEIGHT_BYTES)
        self.eos_token_id = self.model.spec.eos_token_id
        self.run_ahead = bool(run_ahead) and self.device.type == "cuda"
        #: the step whose tokens the host has not read yet: (items, pinned buffer, event, count, ended)
        self._in_flight = None
        self._token_ring = []
        if self.run_ahead:
            for _ in range(3):
                self._token_ring.append((torch.empty(max(max_batch, 1), dtype=torch.int32).pin_memory(),
                                         torch.cuda.Event()))
        self._token_ring_next = 0
        #: seconds the host has spent waiting for the device to hand over a step's tokens (a caller
        #: that measures the host's own share of a step sets it to zero and reads it back)
        self.wait_seconds = 0.0

    def _on_admit(self, req: Request) -> None:
        self.sampler.set_request(req.cache.slot, req.params, n_draws_done=len(req.output))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        vocab = self.model.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is out of vocabulary")
        return self.scheduler.add([int(t) for t in prompt], params or SamplingParams())

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._in_flight is not None

    def step(self) -> List[Request]:
        """One scheduler decision and one model step.  Returns the requests that ended (with
        ``run_ahead``, those whose last token the host has read by now: one step later)."""
        if self.run_ahead:
            return self._step_ahead()
        items = self.scheduler.schedule()
        ended = list(self.scheduler.ended_without_step)
        if not items:
            return ended
        step_items = []
        for it in items:
            toks = it.request.next_tokens(it.n_tokens)
            step_items.append(StepItem(it.request.cache, toks, [it.n_tokens - 1] if it.samples else []))
        tokens = self.runner.step(step_items, sampler=self.sampler)
        sampled: List[int] = tokens.tolist() if tokens is not None else []
        ended += self.scheduler.on_step_done(items, sampled)
        return ended

    def _read_in_flight(self) -> List[Request]:
        """Wait for the step in flight, put its tokens in place of their stand-ins and return the
        requests that are now known to have ended."""
        if self._in_flight is None:
            return []
        items, host, event, n, ended = self._in_flight
        self._in_flight = None
        t0 = time.perf_counter()
        event.synchronize()
        self.wait_seconds += time.perf_counter() - t0
        ended = ended + self.scheduler.on_tokens_read(items, host[:n].tolist())
        return ended

    def _step_ahead(self) -> List[Request]:
        ended: List[Request] = []
        while True:
            items = self.scheduler.schedule()
            ended += self.scheduler.ended_without_step
            # A stand-in may only be the single token of a decoding request in its own slot; a
            # portion that holds one (a request that was preempted meanwhile) needs the value first.
            if self._in_flight is not None and any(
                    it.n_tokens > 1 and any(t < 0 for t in it.request.next_tokens(it.n_tokens)) for it in items):
                ended += self._read_in_flight()
                continue
            break
        if not items:
            return ended + self._read_in_flight()
        step_items, stand_ins = [], []
        for it in items:
            toks = it.request.next_tokens(it.n_tokens)
            step_items.append(StepItem(it.request.cache, toks, [it.n_tokens - 1] if it.samples else []))
            if it.samples:
                stand_ins.append(-(it.request.cache.slot + 1))
        tokens = self.runner.step(step_items, sampler=self.sampler)
        in_flight = None
        if tokens is not None:
            host, event = self._token_ring[self._token_ring_next]
            self._token_ring_next = (self._token_ring_next + 1) % len(self._token_ring)
            n = tokens.shape[0]
            host[:n].copy_(tokens, non_blocking=True)
            event.record()
            in_flight = [items, host, event, n, []]
        # the step's tokens count at once (lengths, pages, who runs next); their values follow
        done = self.scheduler.on_step_done(items, stand_ins)
        if in_flight is not None:
            in_flight[4] = done   # ended by length or context: reported once their last token is read
        ended += self._read_in_flight()   # the step before this one
        self._in_flight = in_flight
        return ended

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Generate for every prompt (token ids in, new token ids out), batched continuously."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        return [r.output for r in reqs]
