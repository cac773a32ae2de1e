"""What a part is, what it may ask of the engine, and the registries parts live in.

A model is put together from parts: a *mixer* (attention and its kin), a
*feed-forward*, *norms*, a *position encoding*, and a *block* that arranges them
around the residual stream. A part takes every size and constant as a constructor
parameter, declares the tensors it wants by local name, and never learns which
model it is in. Each kind of part has one registry from a name to a class, so a
layer is data: ``PartSpec("gated_gqa_attention", {...})``.

Interfaces
----------
Every part:
    ``tensors() -> {local_name: TensorSpec}``   what it loads
    ``load(tensors, runtime)``                  receives exactly those, on the device
Mixer additionally (class attributes `graph_safe` / `graph_safe_mixed`: its forward does no
host-side work per request in a step of single tokens / in any step, so such steps may be
captured into CUDA graphs):
    ``kv_spec() -> KVSpec | None``              rows it keeps per position, in pages
    ``state_spec() -> StateSpec | None``        fixed-size state it keeps per request
    ``initial_state() -> Tensor | None``        what that state starts as (None: zeros)
    ``forward(h, ctx: LayerContext) -> branch`` h, branch: [tokens, hidden] engine dtype
FeedForward:  ``forward(h, ctx) -> branch``
              A mixer or feed-forward whose `forward` gives `h` to one ``ops.linear`` or
              ``ops.linear_swiglu`` and to nothing else may set ``takes_pending = True``; `h` can
              then be an ``ops.PendingStep`` (a residual step that product runs in its own kernel).
Norm:         ``forward(x) -> h`` and the attributes ``weight``, ``eps`` that the
              fused residual kernel reads (``weight is None`` means weightless)
Position:     ``table() -> float32[rotary_dims / 2] | None`` of inverse frequencies
Embedding:    ``forward(token_ids, positions) -> x`` float32 [tokens, hidden]
Block:        ``entry_norm`` and ``forward(x, h, ctx, exit_norm) -> (x, h_next)``
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part loads. `kind` decides the dtype it is kept in:
    ``matrix`` follows the engine's dtype (bfloat16 or float32), ``vector`` is always
    float32 (norm weights: a stored 32-bit value is never rounded), ``table_i32`` is
    an integer table kept as int32."""

    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class KVSpec:
    """What a mixer keeps in the paged cache for every position.

    rows:    the tensors of one position, each `(heads, width)`: an attention mixer keeps two
             equal ones (its keys and its values), a mixer with a latent cache one, a mixer
             whose keys and values differ in width two unequal ones.
    window:  how many of the latest positions can still be read (None: all of them).
    stride:  positions per stored row (1: one row for every position; n: one row for every
             n positions, as a mixer that keeps a compressed history would want).
    Layers with equal specs share one group of pages."""

    rows: tuple[tuple[int, int], ...]
    window: int | None = None
    stride: int = 1

    def __post_init__(self) -> None:
        if not self.rows or any(h < 1 or w < 1 for h, w in self.rows):
            raise ValueError(f"a cache row needs positive (heads, width) entries, got {self.rows}")
        if self.stride < 1 or (self.window is not None and self.window < 1):
            raise ValueError("stride and window must be at least 1")

    @classmethod
    def keys_and_values(cls, kv_heads: int, head_dim: int, window: int | None = None) -> "KVSpec":
        """`kv_heads` keys and as many values of `head_dim` each per position."""
        return cls(((kv_heads, head_dim), (kv_heads, head_dim)), window)

    @property
    def uniform(self) -> bool:
        return all(row == self.rows[0] for row in self.rows)

    @property
    def elements_per_position(self) -> int:
        return sum(h * w for h, w in self.rows)

    def stored(self, positions: int) -> int:
        """Rows that `positions` positions occupy."""
        return -(-positions // self.stride)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per request (one slot per live request). A request's
    state starts as `Mixer.initial_state()` says (zeros unless overridden)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PartSpec:
    """A part as data: the registered name of its class and its parameters."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # params may hold tuples only; good enough for caching
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


class Part:
    """Base of every part. Sub-classes take their sizes and constants as parameters."""

    def tensors(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor], runtime: "Runtime") -> None:
        self.runtime = runtime


class Mixer(Part):
    takes_pending = False
    """True when `forward` hands `h` straight to `ops.linear` or `ops.linear_swiglu` and uses it
    nowhere else: `h` may then be an `ops.PendingStep`, which that product runs in its own kernel."""

    def kv_spec(self) -> KVSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def initial_state(self) -> torch.Tensor | None:
        """What a request's state slot holds before its first step: a tensor of the
        `StateSpec`'s shape, or None for zeros."""
        return None

    def forward(self, h: torch.Tensor, ctx: "LayerContext") -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class FeedForward(Part):
    takes_pending = False  # as for a Mixer

    def forward(self, h: torch.Tensor, ctx: "LayerContext") -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Norm(Part):
    weight: torch.Tensor | None = None
    eps: float = 0.0

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Position(Part):
    def table(self) -> torch.Tensor | None:  # pragma: no cover
        raise NotImplementedError


class Embedding(Part):
    """Turns the step's tokens into the float32 residual stream. It is told where each
    token stands, so an encoding that is added to the embeddings (learned absolute
    positions, say) is a part like any other."""

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Block(Part):
    entry_norm: Norm | None = None

    def forward(self, x, h, ctx: "LayerContext", exit_norm: Norm | None):  # pragma: no cover
        raise NotImplementedError


@dataclass
class Runtime:
    """Where and in what precision the engine runs. `dtype` is the dtype of matrices,
    activations and cache pages; reductions are 32-bit in both."""

    dtype: torch.dtype
    device: torch.device

    @property
    def exact(self) -> bool:
        """True on the 32-bit path: no reduced-precision matrix mode anywhere."""
        return self.dtype == torch.float32


class Registry:
    """One registry per kind of part: name -> class."""

    def __init__(self, what: str) -> None:
        self.what = what
        self._classes: dict[str, Callable[..., Part]] = {}

    def register(self, name: str, cls: Callable[..., Part] | None = None):
        def put(c):
            if name in self._classes and self._classes[name] is not c:
                raise ValueError(f"{self.what} {name!r} is already registered")
            self._classes[name] = c
            return c

        return put if cls is None else put(cls)

    def build(self, spec: PartSpec) -> Part:
        try:
            cls = self._classes[spec.kind]
        except KeyError:
            raise KeyError(f"no {self.what} named {spec.kind!r}; known: {sorted(self._classes)}") from None
        return cls(**spec.params)

    def names(self) -> list[str]:
        return sorted(self._classes)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


@dataclass
class KVView:
    """One cache entry's pages as a mixer sees them in a step.

    pages:        a group whose rows are all `(heads, width)` (keys and values of equal
                  shape, or a single latent row): [num_pages, len(rows), heads, page_size,
                  width], so index 1 of axis 1 is an attention mixer's V; a group of
                  unequal rows: [num_pages, elements per page], row i of a page being the
                  `[heads_i, page_size, width_i]` block that `row(i)` views
    block_table:  int32 [num_seqs, max_pages]; physical page of each logical page of
                  each request, -1 where a page was given back (behind a window)
    slot_mapping: int64 [tokens]; page * page_size + offset where this step's token goes
    writes:       False when this entry reads another entry's cache
    spec:         the `KVSpec` the pages were made for
    """

    pages: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    page_size: int
    window: int | None
    writes: bool = True
    spec: KVSpec | None = None

    def row(self, index: int) -> torch.Tensor:
        """Row `index` of every page: [num_pages, heads, page_size, width]."""
        if self.pages.dim() == 5:
            return self.pages[:, index]
        rows = self.spec.rows
        start = sum(h * w for h, w in rows[:index]) * self.page_size
        heads, width = rows[index]
        return self.pages[:, start: start + heads * width * self.page_size].view(-1, heads, self.page_size, width)

@dataclass
class StepContext:
    """The batch of one step: tokens of several requests, flattened.

    Device tensors are int32 unless said otherwise. Host mirrors (`q_lens`,
    `seq_lens_host`) are for parts that must loop over requests on the host; kernels
    read the device copies, so a captured graph can be replayed with new values.
    """

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # [tokens]
    positions: torch.Tensor  # [tokens] absolute position of each token in its request
    cu_seqlens: torch.Tensor  # [num_seqs + 1] offsets of each request's tokens in the batch
    seq_lens: torch.Tensor  # [num_seqs] tokens of the request held after this step
    state_slots: torch.Tensor  # [num_seqs] slot of per-request state (padding rows: the scratch slot)
    fresh: torch.Tensor  # [num_seqs] 1 where this is the request's first portion
    logit_rows: torch.Tensor  # [wanted] rows of the batch whose logits are wanted
    q_lens: list[int]
    seq_lens_host: list[int]
    max_q_len: int
    max_seq_len: int
    decode_only: bool
    groups: dict[int, tuple[torch.Tensor, torch.Tensor]]  # group -> (block_table, slot_mapping)
    workspace: Any = None


@dataclass
class LayerContext:
    """What one schedule entry's parts see: the batch, this entry's cache pages and
    this entry's per-request state."""

    step: StepContext
    kv: KVView | None
    state: torch.Tensor | None  # [num_slots, *StateSpec.shape]
    entry: int
    exit_may_pend: bool = False  # whatever takes this entry's h takes a pending residual step too
