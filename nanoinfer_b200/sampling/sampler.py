"""Sampling: greedy, temperature and top-k, with the reference's generator.

``SamplingParams`` carries the options of the reference's ``generate`` command
(crates/cli/src/main.rs:48-72: tokens 40, temperature 0.0 = greedy, top_k 40, seed 42) and
``Sampler`` runs the reference's rule on the device (crates/core/src/sampler.rs:59-78) with a
xorshift64* word per request (sampler.rs:46-57) kept in the request's state slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.manager import StateSlots
from ..kernels import ops

_MASK64 = (1 << 64) - 1


@dataclass
class SamplingParams:
    max_new_tokens: int = 40
    temperature: float = 0.0      # <= 0: greedy
    top_k: int = 40               # 0: the whole vocabulary
    seed: int = 42
    #: stop when this token is produced (None: never, as the reference, which has no EOS stop)
    eos_token_id: Optional[int] = None


def xorshift64star_state(seed: int, n_draws: int = 0) -> int:
    """The generator's state after ``n_draws`` draws from ``seed`` (crates/core/src/sampler.rs:46-57:
    the state starts at max(seed, 1))."""
    s = max(int(seed), 1) & _MASK64
    for _ in range(n_draws):
        s ^= s >> 12
        s ^= (s << 25) & _MASK64
        s ^= s >> 27
    return s


def _as_signed(u: int) -> int:
    return u - (1 << 64) if u >= (1 << 63) else u


class Sampler:
    """Per-slot sampling state on the device and the call that turns logits rows into tokens."""

    def __init__(self, slots: StateSlots):
        self.slots = slots
        self.rng = slots.register(("sampler", "rng"), (), torch.int64)
        self.temperature = slots.register(("sampler", "temperature"), (), torch.float32)
        self.top_k = slots.register(("sampler", "top_k"), (), torch.int32)
        #: the token last sampled for each slot: the next step's embedding can read it from here
        #: before the host has seen it
        self.last_token = slots.register(("sampler", "last_token"), (), torch.int32)
        #: the step's tokens and the kernel's two zero-invariant words per row.  Sized for 256 rows or
        #: one per slot; a call with more rows (logits wanted at many places of a prompt) replaces both,
        #: and ``generation`` tells holders of captured graphs that the old addresses are gone
        self.generation = 0
        self._size(max(256, slots.n_slots + 1))
        #: slots whose request samples with a temperature (a slot stays here until its next request)
        self._sampled_slots = set()

    def _size(self, n: int) -> None:
        dev = self.slots.device
        self._out = torch.zeros(n, dtype=torch.int32, device=dev)
        self._scratch = torch.zeros(2 * n, dtype=torch.int64, device=dev)

    def set_request(self, slot: int, params: SamplingParams, n_draws_done: int = 0) -> None:
        """Write a request's options into its slot; ``n_draws_done`` restores the generator of a
        request that sampled before (after a preemption)."""
        draws = n_draws_done if params.temperature > 0.0 else 0
        self.rng[slot] = _as_signed(xorshift64star_state(params.seed, draws))
        self.temperature[slot] = float(params.temperature)
        self.top_k[slot] = int(params.top_k)
        if params.temperature > 0.0:
            self._sampled_slots.add(slot)
        else:
            self._sampled_slots.discard(slot)

    @property
    def any_sampled(self) -> bool:
        """Whether some slot may hold a request that samples with a temperature: the kernel is then
        launched as clusters of blocks that share a sampled row."""
        return bool(self._sampled_slots)

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor) -> torch.Tensor:
        """One token per logits row (int32, on the device; valid until the next call)."""
        n = logits.shape[0]
        if n > self._out.numel():
            self._size(n)
            self.generation += 1
        ops.sample(logits, n, row_slot, self.temperature, self.top_k, self.rng, self._out, self._scratch,
                   self.last_token, teams=self.any_sampled)
        return self._out[:n]
