"""What a part is, what memory it may ask for, and what a step hands it.

A model is a list of blocks; a block is an arrangement of a mixer, a feed-forward and norms.
No part knows which model it is in: each takes its sizes and constants as parameters, declares
the per-request memory it needs as ``StateSpec``s, and reads the step's layout from a
``StepContext``. The cache manager allocates what the specs ask for; the step function fills
the context. (Counterpart in the reference: Tokenomos models/contract.py:19-137.)

State memory comes in two shapes:

- paged, growing with the sequence: ``PagedKV`` (every position kept) and ``WindowKV`` (only the
  last ``window`` positions are ever read, pages behind the window are given back). Specs with
  equal ``group`` share one pool's page numbering and one block table per request;
- fixed size per request: ``SlotState``, a row ``[*shape]`` of a ``[slots, *shape]`` tensor,
  row 0 being the null row that padded sequences point at. A request that starts at position
  0 must read its row as zeros: parts check ``seq_ctx == 0`` (or positions) instead of relying
  on a cleared row.

``SharedState`` owns nothing: the call reads the state of another call of the layer list.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Protocol, runtime_checkable

import torch


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position: ``[pages, 2, kv_heads, page, head_dim]``."""

    kv_heads: int
    head_dim: int

    @property
    def group(self) -> tuple:
        return ("full",)


@dataclass(frozen=True)
class WindowKV:
    """Keys and values of which only the last ``window`` positions are read."""

    kv_heads: int
    head_dim: int
    window: int

    @property
    def group(self) -> tuple:
        return ("window", self.window)


@dataclass(frozen=True)
class SlotState:
    """Fixed-size state per request: a row of ``[slots, *shape]``; ``dtype`` None = work dtype."""

    shape: tuple[int, ...]
    dtype: torch.dtype | None = None


@dataclass(frozen=True)
class SharedState:
    """No memory of its own: reads state ``name`` of call ``source`` of the layer list."""

    source: int
    name: str = "kv"


StateSpec = PagedKV | WindowKV | SlotState | SharedState
# (index of the call in the model's layer list, name of the state within the part)
StateKey = tuple[int, str]


@dataclass
class HostLayout:
    """The step's layout as Python lists, for parts that plan launches on the host."""

    seq_lens: list[int]          # new tokens of each sequence in this step
    seq_ctx: list[int]           # tokens of each sequence already in the cache
    seq_slot: list[int]          # state row of each sequence
    decode_only: bool            # every sequence brings exactly one token
    longest: int = 0             # upper bound of (cached + new) tokens over the sequences


@dataclass
class StepContext:
    """One step's packed token layout: sequences back to back, ``T`` tokens, ``S`` sequences.

    Device tensors (int32): ``positions`` [T], ``tok_seq`` [T], ``cu_seqlens`` [S + 1],
    ``seq_ctx`` [S] (tokens already cached = position of the sequence's first new token),
    ``seq_slot`` [S]. ``block_tables[group]`` [S, blocks]: page of each block of positions, per
    cache group. ``states[(call, name)]``: the tensor the cache manager built for that spec
    (for a ``SharedState`` the source's tensor); ``state_groups[(call, name)]``: the cache group of
    a paged state, the key into ``block_tables``.
    ``tiles(kind, size)``: device tile lists cut from the sequences (cached per step).
    ``scratch``: per-step values parts share (rotary tables and the like).
    """

    n_tokens: int
    n_seqs: int
    positions: torch.Tensor
    tok_seq: torch.Tensor
    cu_seqlens: torch.Tensor
    seq_ctx: torch.Tensor
    seq_slot: torch.Tensor
    block_tables: dict[tuple, torch.Tensor]
    states: dict[StateKey, torch.Tensor]
    state_groups: dict[StateKey, tuple]
    page_size: int
    host: HostLayout
    tile_source: object = None
    scratch: dict = field(default_factory=dict)

    def tiles(self, size: int, which: str = "all"):
        """Runs of at most ``size`` tokens of one sequence: device int32 arrays
        ``(seq, first token in the batch, offset in the sequence's portion, tokens)``.
        ``which``: ``all`` sequences, or only the ``multi``-token ones (prompt portions)."""
        return self.tile_source.tiles(size, which)

    def singles(self) -> torch.Tensor:
        """Device int32 indices (into the packed tokens) of the sequences that bring exactly one
        token (decoded tokens)."""
        return self.tile_source.singles()


@runtime_checkable
class Mixer(Protocol):
    """A block's token mixer (attention, short conv, anything with per-request state)."""

    def state_specs(self) -> dict[str, StateSpec]: ...

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        """``x`` [T, width] normed input -> [T, width]; ``call`` keys ``ctx.states``."""
        ...


@runtime_checkable
class FeedForward(Protocol):
    def forward(self, x: torch.Tensor) -> torch.Tensor: ...


@runtime_checkable
class Norm(Protocol):
    """A norm that can take the residual add with it (one kernel)."""

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor | None,
                 pre: "Norm | None" = None) -> tuple[torch.Tensor, torch.Tensor]:
        """``stream = residual + [pre](x)``; returns ``(norm(stream), stream)``."""
        ...


@runtime_checkable
class PositionEncoding(Protocol):
    """Whatever turns positions into what a mixer applies to its queries and keys."""

    def tables(self, ctx: StepContext) -> object: ...
