"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere. It holds pages
for the new positions, packs the tokens back to back, uploads the layout (one pinned buffer,
one copy), runs embedding -> layer list -> final norm and head on the wanted rows only, and
advances the requests' lengths. It runs only the tokens it is given; everything earlier comes
from the cache that earlier steps left. The reference's engine builds the same packed layout
(Tokenomos models/contract.py:66-97, core/engine.py:501-595) but never mixes prompt portions
with decoded tokens in one forward; here that is the normal case.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from tokenomos_b200.cache.manager import CacheManager, OutOfPages
from tokenomos_b200.parts.contract import HostLayout, StepContext


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the places among them (indices
    into ``tokens``) whose logits are wanted."""

    rid: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


class _Tiles:
    """Cuts the step's sequences into runs of at most ``size`` tokens, on demand, once per size."""

    def __init__(self, seq_lens: list[int], device, upload):
        self.seq_lens, self.device, self.upload = seq_lens, device, upload
        self.cache: dict[int, tuple] = {}

    def tiles(self, size: int):
        if size not in self.cache:
            seq, tok0, off, n = [], [], [], []
            start = 0
            for s, length in enumerate(self.seq_lens):
                for o in range(0, length, size):
                    seq.append(s)
                    tok0.append(start + o)
                    off.append(o)
                    n.append(min(size, length - o))
                start += length
            k = len(seq)
            flat = self.upload(seq + tok0 + off + n)
            self.cache[size] = (flat[:k], flat[k:2 * k], flat[2 * k:3 * k], flat[3 * k:])
        return self.cache[size]


class StepFunction:
    def __init__(self, model, cache: CacheManager, staging_ints: int = 1 << 20):
        self.model, self.cache = model, cache
        self.device = cache.device
        # pinned staging for the layout, used round-robin so that a copy still in flight is
        # never overwritten (each buffer is reused only after `ring` later uploads)
        self._ring = [torch.empty(staging_ints, dtype=torch.int32).pin_memory()
                      if self.device.type == "cuda" else torch.empty(staging_ints, dtype=torch.int32)
                      for _ in range(4)]
        self._ring_events = [None] * len(self._ring)
        self._ring_pos = 0
        self.steps = 0

    def _upload(self, values: list[int]) -> torch.Tensor:
        """Host ints -> device int32 tensor through pinned memory, without a sync."""
        n = len(values)
        i = self._ring_pos
        self._ring_pos = (i + 1) % len(self._ring)
        buf = self._ring[i]
        if n > buf.numel():
            buf = self._ring[i] = (torch.empty(2 * n, dtype=torch.int32).pin_memory()
                                   if self.device.type == "cuda" else torch.empty(2 * n, dtype=torch.int32))
            self._ring_events[i] = None
        if self._ring_events[i] is not None:
            self._ring_events[i].synchronize()
        buf[:n] = torch.tensor(values, dtype=torch.int32)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        out.copy_(buf[:n], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._ring_events[i] = ev
        return out

    def layout(self, entries: list[StepEntry]) -> tuple[StepContext, torch.Tensor, torch.Tensor]:
        """Hold pages for the entries' tokens and build the step's context; returns it with the
        token ids [T] and the wanted rows [R] (both device int32). All or nothing: the pages the
        whole step needs are counted first, and ``OutOfPages`` is raised before any is taken."""
        cache = self.cache
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if not e.tokens:
                raise ValueError(f"request {e.rid!r} brings no tokens")
            bad = [w for w in e.want if not 0 <= w < len(e.tokens)]
            if bad:
                raise ValueError(f"request {e.rid!r}: wanted places {bad} outside its {len(e.tokens)} tokens")
            vocab = self.model.vocab
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.rid!r}: token id outside 0..{vocab - 1}")
        short = {}
        for g in cache.groups:
            need = sum(cache.pages_needed(e.rid, len(e.tokens))[g] for e in entries)
            if need > cache.free_pages(g):
                short[g] = (need, cache.free_pages(g))
        if short:
            raise OutOfPages(f"the step needs pages (group: needed, free) {short}")
        for e in entries:
            cache.extend(e.rid, len(e.tokens))

        seq_lens = [len(e.tokens) for e in entries]
        seq_ctx = [cache.length(e.rid) for e in entries]
        seq_slot = [cache.slot(e.rid) for e in entries]
        S, T = len(entries), sum(seq_lens)
        cu = [0]
        for n in seq_lens:
            cu.append(cu[-1] + n)
        positions, tok_seq, ids, want = [], [], [], []
        for s, e in enumerate(entries):
            positions.extend(range(seq_ctx[s], seq_ctx[s] + seq_lens[s]))
            tok_seq.extend([s] * seq_lens[s])
            ids.extend(e.tokens)
            want.extend(cu[s] + w for w in e.want)
        groups = list(cache.groups)
        width = max(1, max(-(-(c + n) // cache.page_size) for c, n in zip(seq_ctx, seq_lens)))
        tables = []
        for g in groups:
            for e in entries:
                row = cache.block_table(e.rid, g)
                tables.extend(row[:width] + [0] * (width - len(row)))
        flat = self._upload(positions + tok_seq + cu + seq_ctx + seq_slot + ids + want + tables)
        o = 0

        def take(n):
            nonlocal o
            part = flat[o:o + n]
            o += n
            return part

        d_pos, d_tok_seq, d_cu = take(T), take(T), take(S + 1)
        d_ctx, d_slot, d_ids, d_want = take(S), take(S), take(T), take(len(want))
        block_tables = {g: take(S * width).view(S, width) for g in groups}
        host = HostLayout(seq_lens, seq_ctx, seq_slot, all(n == 1 for n in seq_lens))
        ctx = StepContext(
            n_tokens=T, n_seqs=S, positions=d_pos, tok_seq=d_tok_seq, cu_seqlens=d_cu,
            seq_ctx=d_ctx, seq_slot=d_slot, block_tables=block_tables, states=cache.states,
            state_groups=cache.state_groups, page_size=cache.page_size, host=host,
            tile_source=_Tiles(seq_lens, self.device, self._upload))
        return ctx, d_ids, d_want

    @torch.no_grad()
    def run(self, entries: list[StepEntry], commit: bool = True) -> torch.Tensor | None:
        """Run one step; returns float32 logits [wanted, vocab] in the order of the entries and
        of their ``want`` lists (None when nothing is wanted). ``commit`` False leaves advancing
        the requests' lengths to the caller (the scheduler does it when it takes the tokens)."""
        ctx, ids, want = self.layout(entries)
        out = self.model.forward(self.model.embed(ids), ctx)
        logits = self.model.logits(out, want) if want.numel() else None
        if commit:
            for e in entries:
                self.cache.commit(e.rid, len(e.tokens))
        self.steps += 1
        return logits
