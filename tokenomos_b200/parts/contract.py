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

A spec says what the cache manager has to do for it through three attributes, so a part may
bring a spec class of its own: ``storage`` (``"paged"``, ``"slot"`` or ``"shared"``); for paged
storage ``group`` (specs with equal groups share page numbers and block tables), ``window``
(None: every position is kept) and ``page_shape(page_size)`` (the shape of one page); for slot
storage ``shape`` and ``dtype``; for shared storage ``source`` and ``name``.

Captured steps. With ``graphs=True`` the engine records a step's kernels once per shape and
replays them with new contents in the same device buffers. A part can be recorded if its
``forward`` launches the same kernels whatever the batch holds: it reads the batch only from the
device tensors of the ``StepContext``, from ``ctx.tiles`` / ``ctx.singles`` and from the two host
facts that are fixed for a shape, ``ctx.host.decode_only`` and ``ctx.host.longest``. Such a part
sets ``capture_safe = True``. The per-sequence lists of ``ctx.host`` do not exist in a captured
step and raise ``LayoutUnavailable`` there; a model with any part that is not ``capture_safe``
is never captured (the engine runs its steps eagerly).
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
    storage = "paged"
    window = None

    @property
    def group(self) -> tuple:
        return ("full",)

    def page_shape(self, page_size: int) -> tuple[int, ...]:
        return (2, self.kv_heads, page_size, self.head_dim)


@dataclass(frozen=True)
class WindowKV:
    """Keys and values of which only the last ``window`` positions are read."""

    kv_heads: int
    head_dim: int
    window: int
    storage = "paged"

    @property
    def group(self) -> tuple:
        return ("window", self.window)

    def page_shape(self, page_size: int) -> tuple[int, ...]:
        return (2, self.kv_heads, page_size, self.head_dim)


@dataclass(frozen=True)
class SlotState:
    """Fixed-size state per request: a row of ``[slots, *shape]``; ``dtype`` None = work dtype."""

    shape: tuple[int, ...]
    dtype: torch.dtype | None = None
    storage = "slot"


@dataclass(frozen=True)
class SharedState:
    """No memory of its own: reads state ``name`` of call ``source`` of the layer list."""

    source: int
    name: str = "kv"
    storage = "shared"


# the specs the framework's own parts use; any object with the attributes above is one too
StateSpec = PagedKV | WindowKV | SlotState | SharedState
# (index of the call in the model's layer list, name of the state within the part)
StateKey = tuple[int, str]


class LayoutUnavailable(RuntimeError):
    """A part asked for the per-sequence host lists of a captured step, which has none."""


class HostLayout:
    """What the host knows of a step's layout. ``decode_only`` (every sequence brings exactly
    one token) and ``longest`` (an upper bound of cached + new tokens over the sequences) are
    always there. ``seq_lens`` (new tokens of each sequence), ``seq_ctx`` (tokens already cached)
    and ``seq_slot`` (state rows) are Python lists for parts that plan launches on the host;
    a captured step is recorded once for every batch of its shape, so there they raise."""

    def __init__(self, seq_lens: list[int], seq_ctx: list[int], seq_slot: list[int],
                 decode_only: bool, longest: int = 0, captured: bool = False):
        self._lists = (seq_lens, seq_ctx, seq_slot)
        self.decode_only, self.longest, self.captured = decode_only, longest, captured

    @classmethod
    def of_captured_step(cls, decode_only: bool, longest: int) -> "HostLayout":
        return cls([], [], [], decode_only, longest, captured=True)

    def _list(self, i: int, name: str) -> list[int]:
        if self.captured:
            raise LayoutUnavailable(
                f"ctx.host.{name} does not exist in a captured step: the step is recorded once and "
                "replayed for every batch of its shape. Read the layout from the context's device "
                "tensors, or leave capture_safe unset on the part so that its model runs eagerly")
        return self._lists[i]

    @property
    def seq_lens(self) -> list[int]:
        return self._list(0, "seq_lens")

    @property
    def seq_ctx(self) -> list[int]:
        return self._list(1, "seq_ctx")

    @property
    def seq_slot(self) -> list[int]:
        return self._list(2, "seq_slot")


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


@dataclass(frozen=True)
class HeadLayout:
    """What a position encoding needs to know of the projection it is handed: ``qkv`` rows hold
    ``heads`` query heads, then ``kv_heads`` key heads, then ``kv_heads`` value heads, each of
    ``head_dim`` (``kv_heads`` 0: queries only); the per-head norm weights (float32 [head_dim] or
    None) and eps that go with them."""

    heads: int
    kv_heads: int
    head_dim: int
    q_norm: torch.Tensor | None
    k_norm: torch.Tensor | None
    eps: float


@runtime_checkable
class PositionEncoding(Protocol):
    """Owns everything between the fused q/k/v projection and attention over the cache: how
    position enters the queries and keys, and the write of the new keys and values. Attention
    calls it once per layer and step and knows nothing of rotations or tables."""

    def encode_qk(self, qkv: torch.Tensor, ctx: StepContext, heads: HeadLayout,
                  pool: torch.Tensor | None, table: torch.Tensor | None) -> torch.Tensor:
        """``qkv`` [T, (H + 2 Hkv) D] (rows may be strided) -> the queries [T, H, D] as attention
        will use them (normed, position applied), contiguous. The step's keys (treated likewise)
        and values are written into ``pool`` [pages, 2, Hkv, P, D] at each token's position,
        through ``table`` (the block table of the layer's cache group); ``pool`` None: the layer
        has no keys of its own."""
        ...

    # Optional. An encoding that is nothing but a rotate-half rotation of the first R columns of
    # every q and k head by ``position * frequency`` may say so:
    #
    #     def rotate_half_frequencies(self) -> torch.Tensor      # [R / 2] float32, on the device
    #
    # A mixer is then free to apply norm, rotation and cache write inside a kernel of its own
    # (attention does, in steps where every sequence brings one token) instead of calling
    # ``encode_qk``; both ways give the same bits. Encodings without the method are always
    # called through ``encode_qk``.
