"""What a model is put together from: the interfaces of the parts and their registries.

A part (norm, mixer, feed-forward, position encoding, embedding, head) takes all of
its sizes and constants as constructor arguments, declares the parameters it wants
(``param_specs``), receives them (``bind``) and runs on the rows of one step
(``forward``).  No part knows which model it is in: the architecture's builder
chooses a part per layer by its registered name and tells the loader which tensor
of the checkpoint feeds which parameter.

The reference passes constants as arguments in places (eps to layernorm, head count
and size to attention: crates/core/src/stages/blocks.rs:43,76) and fixes the rest in
code (GELU kind, 4C: blocks.rs:113-137); here all of them are parameters.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, Type

import torch

# ----------------------------------------------------------------------------- parameter specs
#: kinds of parameters: how the loader stores them for a given engine dtype
MATRIX = "matrix"   # [out, in] operand of a matrix product: the engine's dtype
TABLE = "table"     # rows looked up by index (embeddings): the engine's dtype
VECTOR = "vector"   # biases and norm parameters: always 32-bit
INT_TABLE = "int_table"  # integer tables: int32

#: how the random-weights mode fills a parameter
INIT_NORMAL = "normal"              # N(0, std)
INIT_ONE_PLUS_NORMAL = "one_plus"   # 1 + N(0, std)   (norm scales)
INIT_ZEROS = "zeros"


@dataclass(frozen=True)
class ParamSpec:
    key: str                 # the part's own name for the parameter
    shape: Tuple[int, ...]   # the shape the part computes with
    kind: str = MATRIX
    init: str = INIT_NORMAL


@dataclass(frozen=True)
class TensorRef:
    """Where a parameter lives in the checkpoint: the tensor's name, and whether the file
    stores it transposed ([in, out], as GPT-2's Conv1D does: crates/core/src/weights.rs:1-9)."""
    name: str
    transposed: bool = False


@dataclass(frozen=True)
class KVCacheSpec:
    """A mixer's need of paged keys and values."""
    n_kv_head: int
    head_dim: int
    window: int = 0          # 0: all keys; w > 0: the last w positions only


@dataclass(frozen=True)
class StateSpec:
    """A mixer's need of per-request state of fixed size (one tensor of `shape` per request)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ----------------------------------------------------------------------------- the parts
class Part:
    """Base of all parts."""

    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded parameters, keyed as in ``param_specs``."""
        self.params = params

    def prepare(self, dtype: torch.dtype, device: torch.device) -> None:
        """Called once after ``bind`` with the engine's dtype."""
        self.dtype, self.device = dtype, device

    def reserve(self, workspace: "Workspace", limits: "StepLimits") -> None:
        """Optional: size the part's scratch for the largest step ahead of time
        (``workspace.reserve``), so that no buffer has to grow once steps are captured in graphs.
        A part that does not is still safe: a buffer that grows later makes the step function drop
        its graphs."""

    def matrix_flops_per_row(self) -> float:
        """FLOPs this part's matrix products spend on one row: 2 per element of every ``matrix``
        parameter unless the part says otherwise (a routed feed-forward counts the experts a row
        visits; a head, whose matrix is a ``table``, counts it all)."""
        total = 0
        for spec in self.param_specs():
            if spec.kind == MATRIX or isinstance(self, Head):
                n = 1
                for d in spec.shape:
                    n *= int(d)
                total += n
        return 2.0 * total

    def step_planner(self) -> Optional[Tuple[str, Callable[..., "StepPlan"]]]:
        """Optional: (name, factory) of what this kind of part derives on the host from the shape
        of a step.  The step function calls ``factory(entry_start, entry_pos0, for_graph)`` once
        per step and name (parts that give the same name share the plan), sends the plan's words to
        the device with the step's other tables, and hands it to the parts as ``ctx.plans[name]``."""
        return None


@dataclass(frozen=True)
class StepLimits:
    """The largest step the engine will run: what scratch is sized for."""
    max_rows: int
    max_entries: int
    max_positions: int
    dtype: torch.dtype


class StepPlan:
    """What a kind of part works out on the host from the shape of a step (which rows are single
    decoded tokens, how work is cut into tiles): ``words`` are int32 values that travel to the
    device with the step's tables, ``bind`` receives the device tensor that holds them, and
    ``graph_key`` names everything about the plan that a captured graph of the step bakes in: two
    steps whose keys are equal run the same launches with the same sizes.  ``for_graph`` asks the
    factory to round what may be rounded (a key range, say) so that steps share graphs."""

    words: List[int] = []

    def graph_key(self) -> tuple:
        return (len(self.words),)

    def bind(self, buf: Optional[torch.Tensor]) -> None:
        pass


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, n_rows: int,
                rows: Optional[torch.Tensor] = None) -> None:
        """out[:n_rows] = norm(x[rows] or x[:n_rows]); x is the 32-bit residual stream."""
        raise NotImplementedError

    def as_input(self, x: torch.Tensor, ctx: "StepContext", dtype: torch.dtype,
                 rows: Optional[torch.Tensor] = None):
        """Optional: this norm of ``x`` in a form that a following matrix product accepts as its
        activations and may fold into its own kernel (``kernels.ops.NormInput``).  None: the norm
        cannot be folded, and is run by ``forward``."""
        return None


class PositionEncoding(Part):
    """Either adds to the embeddings (``additive_table``/``on_embedding``) or transforms
    queries and keys inside a mixer (``on_qk``); a part may do neither or both."""

    def additive_table(self) -> Optional[torch.Tensor]:
        """A [positions, width] table to be added to the token embeddings, if that is all it does."""
        return None

    def max_positions(self) -> Optional[int]:
        return None

    def on_embedding(self, x: torch.Tensor, ctx: "StepContext") -> None:
        pass

    def on_qk(self, q: torch.Tensor, k: torch.Tensor, ctx: "StepContext") -> None:
        pass


class Mixer(Part):
    """Mixes information across positions (attention here).  ``forward`` reads the normed
    rows ``xn`` and ADDS its output to the 32-bit residual stream ``x`` in place.

    A part that sets ``takes_norm_input = True`` may be given ``xn`` as a foldable norm input
    (``Norm.as_input``) instead of a tensor, and passes it on to its first matrix product."""

    takes_norm_input = False

    def kv_spec(self) -> Optional[KVCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def flops_per_key(self) -> float:
        """FLOPs spent per row and visible key beyond the matrix products (attention: the score
        and the weighted sum, 4 per query head and head element)."""
        return 0.0

    @property
    def capture_safe(self) -> bool:
        """Whether ``forward`` only enqueues work whose shape follows from the step's shape and its
        plans' graph keys, reading everything else (tokens, positions, slots, tables) on the device,
        so that a step may be captured in a CUDA graph and replayed with other contents.  A mixer
        without state of its own is; one with state says so itself if it is (a ``forward`` that
        loops over ``ctx.host_entry_slot`` on the host is not)."""
        return self.state_spec() is None

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: "StepContext", cache: Optional["KVCacheView"],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        raise NotImplementedError


class FeedForward(Part):
    """Per-row transformation; ``forward`` ADDS its output to the residual stream ``x``.
    ``takes_norm_input`` as for mixers."""

    takes_norm_input = False

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: "StepContext") -> None:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx: "StepContext", x: torch.Tensor, position: Optional[PositionEncoding]) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, h: torch.Tensor, out: torch.Tensor, n_rows: int, ctx: "StepContext") -> None:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError


# ----------------------------------------------------------------------------- registries
class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Type[Part]] = {}

    def register(self, name: str) -> Callable[[Type[Part]], Type[Part]]:
        def deco(cls: Type[Part]) -> Type[Part]:
            if name in self._items and self._items[name] is not cls:
                raise ValueError(f"{self.what} {name!r} is already registered")
            self._items[name] = cls
            return cls
        return deco

    def build(self, name: str, **kwargs: Any) -> Part:
        if name not in self._items:
            raise KeyError(f"unknown {self.what} {name!r}; registered: {sorted(self._items)}")
        return self._items[name](**kwargs)

    def names(self) -> List[str]:
        return sorted(self._items)


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


# ----------------------------------------------------------------------------- what a step shows to the parts
@dataclass
class KVCacheView:
    """One cache layer as a mixer sees it during a step."""
    layer: torch.Tensor          # [n_pages, 2, n_kv_head, page_size, head_dim]
    block_table: torch.Tensor    # int32 [n_entries, max_blocks]; -1 where no page is held
    page_size: int
    window: int


@dataclass
class StepContext:
    """The rows of one step.  Row t is token ``tokens[t]`` at position ``positions[t]`` of batch
    entry ``row_entry[t]``; an entry's rows are consecutive and in order.  Behind the last entry's rows
    there may be rows of no request (``row_entry[t] == -1``, token 0 at position 0): the step function
    fills a step up with them so that its shape repeats.  They pass through every row-wise part like
    any row; a part that keeps something per request (keys and values, state) leaves them out, and
    nobody reads what they produce.  ``entry_start[-1]`` is the number of rows that belong to requests."""
    n_rows: int
    n_entries: int
    max_rows: int                # the most rows a step may bring: scratch is sized for it
    tokens: torch.Tensor         # int32 [n_rows]
    positions: torch.Tensor      # int32 [n_rows]
    row_entry: torch.Tensor      # int32 [n_rows]
    entry_start: torch.Tensor    # int32 [n_entries + 1]: first row of each entry
    entry_pos0: torch.Tensor     # int32 [n_entries]: position of the entry's first row
    entry_slot: torch.Tensor     # int32 [n_entries]: the request's state slot
    status: torch.Tensor         # int32 [1]: device status word (0 = fine)
    workspace: "Workspace"
    # the same on the host, for parts that plan their launches
    host_entry_start: List[int] = field(default_factory=list)
    host_entry_pos0: List[int] = field(default_factory=list)
    host_entry_slot: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    #: the schedule entry that is running (set by the model's forward pass; -1 outside the layers)
    layer: int = -1
    #: the step's plans by name (``Part.step_planner``); a part that finds none builds its own
    plans: Dict[str, StepPlan] = field(default_factory=dict)
    #: int32 [slots]: the token last sampled for each slot, left on the device by the sampler; a
    #: negative entry -(s + 1) of ``tokens`` stands for ``token_feedback[s]``
    token_feedback: Optional[torch.Tensor] = None


class Workspace:
    """Named scratch buffers that live as long as the engine: a part asks for a buffer by name,
    shape and dtype and gets the same memory every step.

    A captured CUDA graph holds the raw addresses of the buffers its kernels were given, so a
    buffer must not move while a graph that uses it can still be replayed.  Scratch is therefore
    sized ahead where its bound is known (``reserve``, called by the step function at construction
    with the largest step).  Should a larger buffer be asked for all the same, the old one is not
    freed but kept in ``retired`` and ``generation`` goes up: whoever holds graphs compares the
    generation before every replay, drops its graphs when it changed, and only then calls
    ``release_retired``.  Nothing that a live graph can write to is ever handed out again."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        # the views handed out, by (name, shape, dtype): a step asks for the same ones again and
        # again, and making a view costs more than a launch's share of a step
        self._views: Dict[tuple, torch.Tensor] = {}
        #: goes up whenever a buffer that was handed out before is replaced by a larger one
        self.generation = 0
        #: replaced buffers, kept alive until ``release_retired``
        self.retired: List[torch.Tensor] = []

    def _buffer(self, name: str, n: int, dtype: torch.dtype, zeroed: bool) -> torch.Tensor:
        buf = self._bufs.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if buf is not None:
                self.retired.append(buf)
                self.generation += 1
            make = torch.zeros if zeroed else torch.empty
            buf = make(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[name] = buf
            for k in [k for k in self._views if k[0] == name]:   # views of the buffer that was replaced
                del self._views[k]
        return buf

    def reserve(self, name: str, n: int, dtype: torch.dtype, zeroed: bool = False) -> None:
        """Make sure that buffer ``name`` holds at least ``n`` elements from now on."""
        self._buffer(name, int(n), dtype, zeroed)

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        view = self._buffer(name, n, dtype, False)[:n].view(*shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[key] = view
        return view

    def get_zeroed(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Like ``get``, but the memory is zero when first handed out (and whenever it has to grow);
        for counters that a kernel finds zero and leaves zero."""
        n = 1
        for s in shape:
            n *= int(s)
        return self._buffer(name, n, dtype, True)[:n].view(*shape)

    def release_retired(self) -> None:
        """Free the buffers that were replaced.  Only when nothing can refer to them any more: the
        caller has dropped every graph captured before the current generation."""
        self.retired.clear()

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())
