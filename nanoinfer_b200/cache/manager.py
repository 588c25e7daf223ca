"""The cache manager: keys and values in pages with a block table per request, and slots for
per-request state of fixed size.

Pages follow the reference's batch engine (crates/metal/src/batch.rs): a page holds a fixed
number of positions of EVERY layer of its group, keys and values (batch.rs:107-109); a free
list handed out from page 0 upward (batch.rs:174); pages are taken on demand before a step
(``ensure_blocks``, batch.rs:243-254), given back when a request ends (``free_seq``,
batch.rs:209-212) or is cut back (``truncate``, batch.rs:220-227), and reused at once.

Beyond the reference:
  * layers are sorted into GROUPS by what they need (key/value heads, head size, window); each
    group has a page pool, a device tensor and block tables of its own, so a group that keeps a
    window of keys gives pages back as the window passes them while another keeps all keys;
  * a step's allocation is all-or-nothing (the reference leaves a partial allocation behind
    when the pool runs out, batch.rs:243-254);
  * every request owns one STATE SLOT: an index into per-slot tensors of fixed size (a mixer's
    recurrent state, the sampler's generator word), given back with the request.
The bookkeeping is host-only and is tested without a GPU; the device tensors are optional.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KVCacheSpec, KVCacheView, StateSpec


class CacheError(RuntimeError):
    pass


class PoolExhausted(CacheError):
    """Not enough free pages (or no free slot) for what was asked; nothing was changed."""


class PagePool:
    """A fixed set of page ids with a LIFO free list.  Holding a page twice or freeing a page
    that is not held is an error, not a silent corruption."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        self._free: List[int] = list(range(self.n_pages - 1, -1, -1))  # page 0 is handed out first
        self._held = [False] * self.n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_used(self) -> int:
        return self.n_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise PoolExhausted("page pool exhausted")
        p = self._free.pop()
        if self._held[p]:
            raise CacheError(f"page {p} was on the free list while held")
        self._held[p] = True
        return p

    def give_back(self, page: int) -> None:
        if not 0 <= page < self.n_pages or not self._held[page]:
            raise CacheError(f"page {page} is given back but is not held")
        self._held[page] = False
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free once or held: none lost, none twice."""
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in self._free:
            if self._held[p]:
                raise CacheError(f"page {p} is free and held")
        if sum(self._held) + len(self._free) != self.n_pages:
            raise CacheError("a page was lost")


@dataclass
class CacheGroup:
    """Layers with the same need share page ids: page p of the group holds positions of all of them."""
    spec: KVCacheSpec
    owners: List[int]                      # schedule indices whose runs own a cache layer here
    page_size: int
    pool: PagePool
    tensor: Optional[torch.Tensor] = None  # [n_layers, n_pages, 2, n_kv_head, page_size, head_dim]

    def layer_of(self, schedule_index: int) -> int:
        return self.owners.index(schedule_index)

    def bytes_per_page(self, itemsize: int) -> int:
        return len(self.owners) * 2 * self.spec.n_kv_head * self.page_size * self.spec.head_dim * itemsize


@dataclass
class RequestCache:
    """What one request holds: its slot, its committed length, and per group the page of each
    logical block (-1 where the block was never taken or was given back behind a window)."""
    slot: int
    n_tokens: int = 0
    blocks: List[List[int]] = field(default_factory=list)
    live: bool = True
    #: per group, the block table row as the device wants it (int32 [max_blocks], -1 = no page):
    #: a mirror of ``blocks`` kept by the manager so that a step copies it in one piece
    table_rows: List[np.ndarray] = field(default_factory=list)

    def pages_held(self) -> int:
        return sum(1 for g in self.blocks for p in g if p >= 0)


class StateSlots:
    """Per-request state of fixed size: ``n_slots`` rows in every registered tensor."""

    def __init__(self, n_slots: int, device: Optional[torch.device], spare: int = 0):
        """``spare``: rows beyond the slots in every tensor, never handed out (rows that pad a step
        to the shape of a captured graph point there)."""
        self.n_slots = int(n_slots)
        self.spare = int(spare)
        self.device = device
        self._free: List[int] = list(range(self.n_slots - 1, -1, -1))
        self._held = [False] * self.n_slots
        self.tensors: Dict[object, torch.Tensor] = {}

    def register(self, key: object, shape: Tuple[int, ...], dtype: torch.dtype) -> Optional[torch.Tensor]:
        """A zeroed tensor [n_slots, *shape] addressed by slot; None when there is no device."""
        if self.device is None:
            return None
        t = torch.zeros((self.n_slots + self.spare, *shape), dtype=dtype, device=self.device)
        self.tensors[key] = t
        return t

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise PoolExhausted("no free state slot")
        s = self._free.pop()
        if self._held[s]:
            raise CacheError(f"slot {s} was free while held")
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots or not self._held[slot]:
            raise CacheError(f"slot {slot} is given back but is not held")
        self._held[slot] = False
        self._free.append(slot)

    def reset(self, slot: int, keys: Optional[Sequence[object]] = None) -> None:
        """Zero the slot's row in the registered tensors (all of them, or those named)."""
        for key, t in self.tensors.items():
            if keys is None or key in keys:
                t[slot].zero_()

    def check(self) -> None:
        if len(set(self._free)) != len(self._free) or sum(self._held) + len(self._free) != self.n_slots:
            raise CacheError("state slots are inconsistent")


class CacheManager:
    def __init__(self, kv_needs: Sequence[Tuple[int, KVCacheSpec]], state_needs: Sequence[Tuple[int, StateSpec]],
                 max_tokens: int, max_requests: int, page_size: int = 16,
                 dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None,
                 max_positions: Optional[int] = None, pages_per_group: Optional[Sequence[int]] = None,
                 padding: bool = False):
        """``max_tokens``: how many tokens live requests may hold together, each request's count
        rounded up to whole pages; every group's pool gets ``ceil(max_tokens / page_size)`` pages
        unless ``pages_per_group`` says otherwise.  ``device`` None: bookkeeping only.
        ``padding``: one page per group and one state slot more than the pools hand out
        (``pad_page``, ``pad_slot``): the step function points the rows there with which it pads a
        batch of single tokens to the shape of a captured graph.  No request ever holds them."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = int(page_size)
        self.dtype, self.device = dtype, device
        self.max_positions = max_positions
        n_default = max(1, -(-int(max_tokens) // self.page_size))
        by_spec: Dict[KVCacheSpec, List[int]] = {}
        for idx, spec in kv_needs:
            by_spec.setdefault(spec, []).append(idx)
        self.groups: List[CacheGroup] = []
        for gi, (spec, owners) in enumerate(by_spec.items()):
            n_pages = int(pages_per_group[gi]) if pages_per_group is not None else n_default
            group = CacheGroup(spec, owners, self.page_size, PagePool(n_pages))
            if device is not None:
                group.tensor = torch.zeros(
                    (len(owners), n_pages + (1 if padding else 0), 2, spec.n_kv_head, self.page_size, spec.head_dim),
                    dtype=dtype, device=device)
            self.groups.append(group)
        self._group_of: Dict[int, int] = {idx: gi for gi, g in enumerate(self.groups) for idx in g.owners}
        self.pad_page: Optional[List[int]] = [g.pool.n_pages for g in self.groups] if padding else None
        self.pad_slot: Optional[int] = int(max_requests) if padding else None
        self.slots = StateSlots(max_requests, device, spare=1 if padding else 0)
        self.state_tensors: Dict[int, torch.Tensor] = {}
        for idx, spec in state_needs:
            t = self.slots.register(("state", idx), tuple(spec.shape), spec.dtype)
            if t is not None:
                self.state_tensors[idx] = t
        self._state_keys = [("state", idx) for idx, _ in state_needs]
        self._live: List[RequestCache] = []
        # the longest block table a request can have, per group
        self.max_blocks = [self._max_blocks(g) for g in self.groups]

    def _max_blocks(self, g: CacheGroup) -> int:
        limit = self.max_positions if self.max_positions is not None else g.pool.n_pages * self.page_size
        return max(1, -(-limit // self.page_size))

    # ------------------------------------------------------------------ requests
    def open_request(self) -> RequestCache:
        slot = self.slots.take()
        self.slots.reset(slot, self._state_keys)
        req = RequestCache(slot=slot, blocks=[[] for _ in self.groups],
                           table_rows=[np.full(mb, -1, dtype=np.int32) for mb in self.max_blocks])
        self._live.append(req)
        return req

    def close_request(self, req: RequestCache) -> None:
        """Give back everything the request holds."""
        self._require_live(req)
        for g, blocks, row in zip(self.groups, req.blocks, req.table_rows):
            for p in blocks:
                if p >= 0:
                    g.pool.give_back(p)
            blocks.clear()
            row.fill(-1)
        self.slots.give_back(req.slot)
        req.live = False
        req.n_tokens = 0
        self._live.remove(req)

    def _require_live(self, req: RequestCache) -> None:
        if not req.live:
            raise CacheError("the request is not live")

    # ------------------------------------------------------------------ pages
    def _first_needed_block(self, g: CacheGroup, pos0: int) -> int:
        """The first logical block that a query at position ``pos0`` (or later) still reads."""
        if g.spec.window <= 0:
            return 0
        return max(0, pos0 - g.spec.window + 1) // self.page_size

    def pages_needed(self, req: RequestCache, n_new: int) -> List[int]:
        """Pages per group that appending ``n_new`` tokens would take from the pool."""
        self._require_live(req)
        out = []
        end = req.n_tokens + n_new
        n_blocks = -(-end // self.page_size)
        for g, blocks in zip(self.groups, req.blocks):
            out.append(max(0, n_blocks - len(blocks)))
        return out

    def can_append(self, work: Sequence[Tuple[RequestCache, int]]) -> bool:
        need = [0] * len(self.groups)
        for req, n in work:
            for gi, k in enumerate(self.pages_needed(req, n)):
                need[gi] += k
        return all(need[gi] <= g.pool.n_free for gi, g in enumerate(self.groups))

    def append(self, work: Sequence[Tuple[RequestCache, int]]) -> None:
        """Take the pages that every (request, new tokens) of a step needs: all of them or none."""
        for req, n in work:
            self._require_live(req)
            if n <= 0:
                raise CacheError("a step must append at least one token")
            if self.max_positions is not None and req.n_tokens + n > self.max_positions:
                raise CacheError(f"context full: {req.n_tokens + n} tokens exceeds max {self.max_positions}")
        if not self.can_append(work):
            raise PoolExhausted("KV cache pool exhausted: the step needs more pages than are free")
        for req, n in work:
            n_blocks = -(-(req.n_tokens + n) // self.page_size)
            for g, blocks, row in zip(self.groups, req.blocks, req.table_rows):
                while len(blocks) < n_blocks:
                    page = g.pool.take()
                    row[len(blocks)] = page
                    blocks.append(page)

    def commit(self, req: RequestCache, n_new: int) -> None:
        """The step ran: the request is ``n_new`` tokens longer; pages a window has passed go back."""
        self._require_live(req)
        req.n_tokens += n_new
        for g, blocks, row in zip(self.groups, req.blocks, req.table_rows):
            if g.spec.window > 0:
                first = self._first_needed_block(g, req.n_tokens)  # the next query stands at n_tokens
                for b in range(min(first, len(blocks))):
                    if blocks[b] >= 0:
                        g.pool.give_back(blocks[b])
                        blocks[b] = -1
                        row[b] = -1

    def truncate(self, req: RequestCache, n_tokens: int) -> None:
        """Forget positions from ``n_tokens`` on; pages wholly past it go back
        (crates/metal/src/batch.rs:220-227).  Not possible behind a window or with mixer state."""
        self._require_live(req)
        if n_tokens > req.n_tokens or n_tokens < 0:
            raise CacheError("truncate: bad length")
        if self._state_keys and n_tokens != req.n_tokens:
            raise CacheError("truncate: a mixer keeps per-request state, which cannot be rolled back")
        keep = -(-n_tokens // self.page_size)
        for g, blocks, row in zip(self.groups, req.blocks, req.table_rows):
            if g.spec.window > 0 and n_tokens < req.n_tokens:
                first = self._first_needed_block(g, n_tokens)
                if any(blocks[b] < 0 for b in range(first, min(keep, len(blocks)))):
                    raise CacheError("truncate: pages behind the window were already given back")
            while len(blocks) > keep:
                p = blocks.pop()
                row[len(blocks)] = -1
                if p >= 0:
                    g.pool.give_back(p)
        req.n_tokens = n_tokens

    # ------------------------------------------------------------------ views and accounting
    def group_index(self, schedule_index: int) -> int:
        return self._group_of[schedule_index]

    def layer_views(self, block_tables: Sequence[torch.Tensor]) -> Dict[int, KVCacheView]:
        """A KVCacheView per owning schedule index, given this step's block table of each group."""
        views: Dict[int, KVCacheView] = {}
        for gi, g in enumerate(self.groups):
            for li, idx in enumerate(g.owners):
                views[idx] = KVCacheView(g.tensor[li], block_tables[gi], self.page_size, g.spec.window)
        return views

    @property
    def live_requests(self) -> List[RequestCache]:
        return list(self._live)

    def pages_free(self) -> List[int]:
        return [g.pool.n_free for g in self.groups]

    def pages_used(self) -> List[int]:
        return [g.pool.n_used for g in self.groups]

    def nbytes(self) -> int:
        return sum(g.tensor.numel() * g.tensor.element_size() for g in self.groups if g.tensor is not None)

    def check(self) -> None:
        """Invariants: every page is free or held by exactly one live request; slots likewise."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = [p for r in self._live for p in r.blocks[gi] if p >= 0]
            if len(set(held)) != len(held):
                raise CacheError(f"group {gi}: a page is held twice")
            if len(held) != g.pool.n_used:
                raise CacheError(f"group {gi}: {g.pool.n_used} pages are out but requests hold {len(held)}")
            for r in self._live:
                row = r.table_rows[gi]
                if list(row[:len(r.blocks[gi])]) != r.blocks[gi] or (row[len(r.blocks[gi]):] != -1).any():
                    raise CacheError(f"group {gi}: a block table row does not mirror the request's pages")
        self.slots.check()
        if len({r.slot for r in self._live}) != len(self._live):
            raise CacheError("two live requests share a slot")
