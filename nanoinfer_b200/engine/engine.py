"""The Python entry point: a model folder in, generated token ids out.

``Engine`` owns the model, the cache manager, the step function, the scheduler and the
sampler.  ``generate`` is the loop of the reference's ``generate`` command
(crates/cli/src/main.rs:151-195: feed the prompt, sample, feed the sampled token, until the
wanted number of tokens or a full context) run for many requests at once by the
continuous-batching scheduler (crates/cli/src/metal_serve.rs:255-363).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..sampling.sampler import Sampler, SamplingParams
from .runner import ModelRunner, StepItem
from .scheduler import Request, Scheduler

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


class Engine:
    def __init__(self, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", device: str = "cuda",
                 max_tokens: Optional[int] = None, max_batch: int = 64, max_rows: int = 2048,
                 prefill_budget: Optional[int] = None, page_size: int = 16, check_status: bool = False,
                 use_graphs: bool = True):
        """``max_tokens``: how many tokens all live requests may hold in the cache together
        (default: ``max_batch`` full contexts).  ``prefill_budget``: most prompt tokens per step
        (default ``max_rows``)."""
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
                                  max_positions=limit)
        self.runner = ModelRunner(self.model, self.cache, max_rows=max_rows, max_entries=max_batch,
                                  check_status=check_status, use_graphs=use_graphs)
        self.sampler = Sampler(self.cache.slots)
        self.scheduler = Scheduler(self.cache, max_batch=max_batch, max_rows=max_rows,
                                   prefill_budget=prefill_budget or max_rows, max_positions=limit)
        self.scheduler.on_admit = self._on_admit
        self.eos_token_id = self.model.spec.eos_token_id

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
        return self.scheduler.has_work()

    def step(self) -> List[Request]:
        """One scheduler decision and one model step.  Returns the requests that ended."""
        items = self.scheduler.schedule()
        ended = list(self.scheduler.ended_without_step)
        if not items:
            return ended
        step_items = []
        for it in items:
            r = it.request
            toks = r.tokens[r.n_computed:r.n_computed + it.n_tokens]
            step_items.append(StepItem(r.cache, toks, [it.n_tokens - 1] if it.samples else []))
        tokens = self.runner.step(step_items, sampler=self.sampler)
        sampled: List[int] = tokens.tolist() if tokens is not None else []
        ended += self.scheduler.on_step_done(items, sampled)
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
