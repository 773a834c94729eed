"""Block arrangements and the stack that runs the layer list.

``PreNormBlock``: ``x = N1(r); r += mixer(x); x = N2(r); r += ffn(x)`` with the residual stream
carried as ``(h, residual)`` so that each add happens inside the next norm's kernel; with
sandwich norms the mixer's and the feed-forward's outputs pass a post-norm before the add
(Tokenomos models/blocks/decoder.py:104-125, 173-180).

``Stack``: embedding, the layer list (data: entries may name a block twice, or read another
entry's state), final norm and head applied only to the rows whose logits are wanted.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import SharedState, StateKey, StateSpec, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import DEFAULT_TUNING, Tuning, register
from tokenomos_b200.parts.spec import LayerCall


class PreNormBlock:
    def __init__(self, mixer, ffn, pre_mixer, pre_ffn, post_mixer=None, post_ffn=None):
        self.mixer, self.ffn = mixer, ffn
        self.pre_mixer, self.pre_ffn = pre_mixer, pre_ffn
        self.post_mixer, self.post_ffn = post_mixer, post_ffn
        # the arrangement itself launches nothing; it can be recorded if all its parts can
        self.capture_safe = all(getattr(part, "capture_safe", False)
                                for part in (mixer, ffn, pre_mixer, pre_ffn, post_mixer, post_ffn)
                                if part is not None)
        # A sublayer whose part offers it runs without a norm kernel when the step is small:
        # the pre-norm's weight moves into the part's first projection now (``fold_norm``), the
        # norm that stays has weight one, and ``forward_stream`` takes the un-normed stream and
        # returns stream + part(norm(stream)) with both the statistics and the add inside its
        # own kernels. Without post-norms only: they sit between the part and the add.
        self.eps_mixer = self.eps_ffn = None
        if post_mixer is None and post_ffn is None:
            self.pre_mixer, self.eps_mixer = self._fold(pre_mixer, mixer)
            self.pre_ffn, self.eps_ffn = self._fold(pre_ffn, ffn)

    @staticmethod
    def _fold(norm, part):
        """(the norm that is left, eps if ``part`` took the weight else None)."""
        if not (hasattr(norm, "folded") and hasattr(part, "fold_norm") and hasattr(part, "forward_stream")):
            return norm, None
        weight, eps, unit = norm.folded()
        return (unit, eps) if part.fold_norm(weight) else (norm, None)

    @staticmethod
    def _stream(h, residual):
        """The residual stream with ``h`` (a part's output not yet added, or None) in it."""
        if h is None:
            return residual
        if residual is None:
            return h if h.is_contiguous() else h.contiguous()
        return ops.add_rmsnorm(h, residual, None, 0.0)[1]

    def forward(self, h, residual, pending, ctx: StepContext, call: int):
        """``h``: the block before's output still to be added to ``residual`` (None: it is in the
        stream already); ``pending``: that block's post-norm still to apply to ``h``. Returns this
        block's output (or None), the stream and its own pending post-norm."""
        rows = (h if h is not None else residual).shape[0]
        if self.eps_mixer is not None and pending is None and self.mixer.can_stream(rows, ctx):
            residual = self.mixer.forward_stream(self._stream(h, residual), self.eps_mixer, ctx, call)
            h = None
        else:
            if h is None:
                h, residual = residual, None
            x, residual = self.pre_mixer.add_norm(h, residual, pending)
            h = self.mixer.forward(x, ctx, call)
        if self.eps_ffn is not None and self.ffn.can_stream(rows):
            return None, self.ffn.forward_stream(self._stream(h, residual), self.eps_ffn), None
        if h is None:
            h, residual = residual, None
        x, residual = self.pre_ffn.add_norm(h, residual, self.post_mixer)
        return self.ffn.forward(x), residual, self.post_ffn


@register("block", "prenorm")
def build_prenorm(parts: dict) -> PreNormBlock:
    return PreNormBlock(parts["mixer"], parts["ffn"], parts["pre_mixer_norm"],
                        parts["pre_ffn_norm"], parts.get("post_mixer_norm"),
                        parts.get("post_ffn_norm"))


class Stack:
    def __init__(self, embedding: torch.Tensor, blocks: list, order: list[LayerCall], final_norm,
                 head: Linear | None, tuning: Tuning = DEFAULT_TUNING, embed_scale: float | None = None,
                 logit_softcap: float | None = None, suppress: tuple[int, ...] = ()):
        self.embedding = embedding
        self.embed_scale = None if embed_scale is None else float(embed_scale)
        self.logit_softcap = None if logit_softcap is None else float(logit_softcap)
        if self.logit_softcap is not None and self.logit_softcap <= 0:
            raise ValueError(f"a logit soft cap of {logit_softcap}: it must be positive")
        bad = [t for t in suppress if not 0 <= int(t) < embedding.shape[0]]
        if bad:
            raise ValueError(f"suppressed token ids {bad} outside the vocabulary of {embedding.shape[0]}")
        self.suppress = (torch.tensor([int(t) for t in suppress], dtype=torch.int32, device=embedding.device)
                         if suppress else None)
        self.blocks = blocks
        self.order = list(order)
        self.final_norm = final_norm
        self.head = head if head is not None else Linear(embedding, tuning=tuning)
        self.tied = head is None
        self.vocab, self.width = embedding.shape
        self.dtype = embedding.dtype
        for i, call in enumerate(self.order):
            if not 0 <= call.block < len(blocks):
                raise ValueError(f"layer list entry {i} names block {call.block} of {len(blocks)}")
            if call.state_from is not None and not 0 <= call.state_from < i:
                raise ValueError(f"layer list entry {i} reads the state of entry {call.state_from}, "
                                 "which must come earlier in the list")

    @property
    def capture_safe(self) -> bool:
        """Whether a step of this model may be recorded as a CUDA graph: every block (and so
        every part in it) and the final norm say so."""
        return all(getattr(part, "capture_safe", False) for part in (*self.blocks, self.final_norm))

    def not_capture_safe(self) -> list[str]:
        """The kinds of the parts that keep this model from being recorded."""
        out = []
        for block in (*self.blocks, self.final_norm):
            if not getattr(block, "capture_safe", False):
                inner = [type(p).__name__ for p in vars(block).values()
                         if hasattr(p, "forward") and not getattr(p, "capture_safe", False)]
                out.extend(inner or [type(block).__name__])
        return sorted(set(out))

    def state_specs(self) -> dict[StateKey, StateSpec]:
        """Per entry of the layer list, the memory its mixer asks for. An entry that reads
        another's state contributes ``SharedState`` specs pointing at it."""
        out: dict[StateKey, StateSpec] = {}
        for i, call in enumerate(self.order):
            for name, spec in self.blocks[call.block].mixer.state_specs().items():
                if call.state_from is not None:
                    spec = SharedState(call.state_from, name)
                out[(i, name)] = spec
        return out

    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        h = ops.gather_rows(self.embedding, ids)
        return h if self.embed_scale is None else ops.scale_rows(h, self.embed_scale)

    def embed_fed(self, ids_host: torch.Tensor, use_prev: torch.Tensor, last_token: torch.Tensor,
                  slot: torch.Tensor) -> torch.Tensor:
        """Embedding rows of a decode step whose ids may still be on the device: row r takes
        ``last_token[slot[r]]`` where ``use_prev[r]`` is set, else ``ids_host[r]``."""
        h = ops.gather_rows_select(self.embedding, ids_host, use_prev, last_token, slot)
        return h if self.embed_scale is None else ops.scale_rows(h, self.embed_scale)

    def forward(self, h: torch.Tensor, ctx: StepContext):
        """Runs the layer list; returns ``(h, residual, pending)`` of the last block: the final
        norm takes the last add with it, on the wanted rows only (``logits``)."""
        residual, pending = None, None
        for i, call in enumerate(self.order):
            h, residual, pending = self.blocks[call.block].forward(h, residual, pending, ctx, i)
        return h, residual, pending

    def logits(self, out, rows: torch.Tensor | None) -> torch.Tensor:
        """Float32 logits [len(rows), vocab] at token rows ``rows`` (int32) of the step; None:
        at every row, in order."""
        h, residual, pending = out
        if h is None:                    # the last block's output is in the stream already
            h, residual = residual, None
        if rows is not None:
            h = ops.gather_rows(h, rows)
            if residual is not None:
                residual = ops.gather_rows(residual, rows)
        y, _ = self.final_norm.add_norm(h, residual, pending)
        out = self.head(y, out_dtype=torch.float32)
        if self.logit_softcap is not None or self.suppress is not None:
            ops.logit_options(out, self.logit_softcap, self.suppress)
        return out
