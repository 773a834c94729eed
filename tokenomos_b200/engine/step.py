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

import contextlib
import gc
import itertools
from dataclasses import dataclass, field

import numpy as np
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


@contextlib.contextmanager
def _no_collection():
    """No garbage collection while a CUDA graph is captured: a collector that ran in the middle
    and freed an older engine's graph would destroy a graph during the capture, which CUDA
    refuses, and the capture would be lost (seen when an engine was built after others had
    gone). The collector runs once before instead."""
    gc.collect()
    was = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was:
            gc.enable()


def _forget_capture_run() -> None:
    """The run that warms a step up before it is captured works on an all-zero layout: no tile,
    every token of the dummy sequence, outputs that no kernel wrote. What the sampler made of
    such logits (a row without a finite value is reported) says nothing about a real step."""
    from tokenomos_b200 import ops

    torch.cuda.synchronize()
    ops.sample_status()


class _Tiles:
    """Cuts the step's sequences into runs of at most ``size`` tokens, on demand, once per size."""

    def __init__(self, seq_lens: list[int], device, upload, asked: set | None = None):
        self.seq_lens, self.device, self.upload = seq_lens, device, upload
        self.cache: dict[int, tuple] = {}
        self.asked = asked          # every (size, which) any step's parts have asked for

    @staticmethod
    def cut(seq_lens: list[int], size: int, which: str):
        """Host arrays (sequence, first token, offset in the portion, tokens) of the tiles, in
        the order of the sequences; ``which`` other than "all" leaves single-token sequences out."""
        lens = np.asarray(seq_lens, dtype=np.int64)
        starts = np.cumsum(lens) - lens
        counts = -(-lens // size)
        if which != "all":
            counts = np.where(lens > 1, counts, 0)
        seq = np.repeat(np.arange(len(lens)), counts)
        first = np.cumsum(counts) - counts                     # each sequence's first tile
        off = (np.arange(len(seq)) - first[seq]) * size
        tok0 = starts[seq] + off
        n = np.minimum(size, lens[seq] - off)
        return tuple(a.astype(np.int32) for a in (seq, tok0, off, n))

    def tiles(self, size: int, which: str = "all"):
        key = (size, which)
        if self.asked is not None:
            self.asked.add(key)
        if key not in self.cache:
            seq, tok0, off, n = self.cut(self.seq_lens, size, which)
            k = len(seq)
            if k == 0:
                empty = torch.empty(0, dtype=torch.int32, device=self.device)
                self.cache[key] = (empty, empty, empty, empty)
            else:
                flat = self.upload(np.concatenate((seq, tok0, off, n)))
                self.cache[key] = (flat[:k], flat[k:2 * k], flat[2 * k:3 * k], flat[3 * k:])
        return self.cache[key]

    def singles(self):
        if self.asked is not None:
            self.asked.add("singles")
        if "singles" not in self.cache:
            idx, start = [], 0
            for length in self.seq_lens:
                if length == 1:
                    idx.append(start)
                start += length
            self.cache["singles"] = (self.upload(idx) if idx else
                                     torch.empty(0, dtype=torch.int32, device=self.device))
        return self.cache["singles"]


DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 96, 128, 192, 256, 384, 512)


class _ConstTiles:
    """Tiles of a decode-only step: one token per sequence, whatever size is asked for."""

    def __init__(self, arange: torch.Tensor, zeros: torch.Tensor, ones: torch.Tensor):
        self.value = (arange, arange, zeros, ones)
        self.none = (arange[:0], arange[:0], arange[:0], arange[:0])

    def tiles(self, size: int, which: str = "all"):
        return self.value if which == "all" else self.none

    def singles(self):
        return self.value[0]


class _DecodeGraph:
    """One captured decode step for ``rows`` sequences: a static layout buffer in, tokens out.

    The token a row feeds is either given by the host or, when the step that sampled it is still
    in flight, taken on the device from ``last_token[slot]``, which the sampler of every step
    writes; so the host may queue a step before it has read the tokens of the one before."""

    RING = 2     # host staging buffers: step n + 1 is packed while step n's copy may be pending

    def __init__(self, step_fn: "StepFunction", rows: int):
        cache, dev = step_fn.cache, step_fn.device
        self.rows = rows
        self.width = cache.max_blocks
        self.groups = list(cache.groups)
        b = rows
        # layout of the int32 buffer the host fills each step
        self.off = {}
        o = 0
        for name, n in (("positions", b), ("seq_ctx", b), ("seq_slot", b), ("ids_host", b),
                        ("use_prev", b), ("sampling", 6 * b)):
            self.off[name] = (o, n)
            o += n
        for g in self.groups:
            self.off[("table", g)] = (o, b * self.width)
            o += b * self.width
        self.size = o
        self.host = [torch.zeros(self.size, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.host_np = [h.numpy() for h in self.host]
        # what each staging buffer's block-table rows hold: (request, entries written) per row
        self.host_rows = [{g: [(None, 0, 0)] * b for g in self.groups} for _ in range(self.RING)]
        self.tokens_host = [torch.zeros(b, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.turn = 0
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(b, dtype=torch.int32, device=dev)
        arange = torch.arange(b + 1, dtype=torch.int32, device=dev)
        zeros = torch.zeros(b, dtype=torch.int32, device=dev)
        ones = torch.ones(b, dtype=torch.int32, device=dev)
        self.last_token = step_fn.last_token

        def view(name):
            a, n = self.off[name]
            return self.dev[a:a + n]

        self.ctx = StepContext(
            n_tokens=b, n_seqs=b, positions=view("positions"), tok_seq=arange[:b],
            cu_seqlens=arange, seq_ctx=view("seq_ctx"), seq_slot=view("seq_slot"),
            block_tables={g: view(("table", g)).view(b, self.width) for g in self.groups},
            states=cache.states, state_groups=cache.state_groups, page_size=cache.page_size,
            host=HostLayout.of_captured_step(True, cache.max_len),
            tile_source=_ConstTiles(arange[:b], zeros, ones))
        self.ids_host, self.use_prev = view("ids_host"), view("use_prev")
        self.sampling = view("sampling")
        self.graph = None
        self.launches = 0

    def body(self, model):
        from tokenomos_b200 import ops
        from tokenomos_b200.sampling import sampler

        h = model.embed_fed(self.ids_host, self.use_prev, self.last_token, self.ctx.seq_slot)
        out = model.forward(h, self.ctx)
        logits = model.logits(out, None)          # every row is wanted, in order
        sampler.sample_packed(logits, self.sampling, self.tokens,
                              scatter=(self.ctx.seq_slot, self.last_token))

    def capture(self, model):
        from tokenomos_b200.ops import _lib

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.body(model)              # warm-up outside the capture (library handles, sizes)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = _lib.calls()
        with _no_collection(), torch.cuda.graph(graph):
            self.body(model)
        self.launches = _lib.calls() - before
        self.graph = graph
        _forget_capture_run()


class DecodeHandle:
    """A decode step in flight: ``tokens()`` waits for it and returns the sampled tokens."""

    def __init__(self, event, host_tokens: torch.Tensor, n: int):
        self.event, self.host_tokens, self.n = event, host_tokens, n
        self._tokens = None

    def tokens(self) -> list[int]:
        if self._tokens is None:
            self.event.synchronize()
            self._tokens = self.host_tokens[:self.n].tolist()
        return self._tokens


STEP_TOKEN_BUCKETS = (32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384)
STEP_SEQ_BUCKETS = (4, 16, 64, 128, 256, 512, 1024)


class _FixedTiles:
    """Tile lists of a captured step: device arrays of the greatest length the bucket allows,
    refilled before every replay; entries past the step's own are empty tiles (0 tokens) and
    negative token indices, which the kernels skip."""

    def __init__(self, views: dict):
        self.views = views

    def tiles(self, size: int, which: str = "all"):
        return self.views[(size, which)]

    def singles(self):
        return self.views["singles"]


class _StepGraph:
    """One captured step for any mix of prompt portions and single tokens that fits ``tokens``
    packed tokens and ``seqs`` sequences: a static layout buffer in, sampled tokens out.

    A step with fewer tokens is padded with a dummy sequence on the null slot and the null page
    (its tokens are carried through the row-wise kernels and belong to no tile); unused sequences
    are empty. Logits are taken at one row per sequence at most (the row whose token is sampled);
    unused rows repeat row 0. As in the decode graph, the id of a single token may come from
    ``last_token`` on the device."""

    RING = 2

    def __init__(self, step_fn: "StepFunction", tokens: int, seqs: int, tile_keys: set):
        cache, dev = step_fn.cache, step_fn.device
        self.tokens_cap, self.seqs_cap = tokens, seqs
        self.width = cache.max_blocks
        self.groups = list(cache.groups)
        T, S = tokens, seqs
        self.off = {}
        o = 0

        def field_(name, n):
            nonlocal o
            self.off[name] = (o, n)
            o += n

        for name, n in (("positions", T), ("tok_seq", T), ("ids_host", T), ("use_prev", T), ("tok_slot", T),
                        ("cu", S + 1), ("seq_ctx", S), ("seq_slot", S), ("want", S), ("want_slot", S),
                        ("sampling", 6 * S)):
            field_(name, n)
        for g in self.groups:
            field_(("table", g), S * self.width)
        self.tile_keys = sorted(k for k in tile_keys if k != "singles")
        self.tile_cap = {}
        for key in self.tile_keys:
            self.tile_cap[key] = T // key[0] + S + 1
            field_(("tiles", key), 4 * self.tile_cap[key])
        field_("singles", S)
        self.size = o
        self.host = [torch.zeros(self.size, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.host_np = [h.numpy() for h in self.host]
        # what each staging buffer's block-table rows hold: (request, entries written) per row
        self.table_rows = [{g: [(None, 0)] * S for g in self.groups} for _ in range(self.RING)]
        self.windowless = {g: cache.groups[g].window is None for g in self.groups}
        self.tokens_host = [torch.zeros(S, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.turn = 0
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros(S, dtype=torch.int32, device=dev)
        self.last_token = step_fn.last_token

        def view(name):
            a, n = self.off[name]
            return self.dev[a:a + n]

        views = {"singles": view("singles")}
        for key in self.tile_keys:
            flat, k = view(("tiles", key)), self.tile_cap[key]
            views[key] = (flat[:k], flat[k:2 * k], flat[2 * k:3 * k], flat[3 * k:])
        self.ctx = StepContext(
            n_tokens=T, n_seqs=S, positions=view("positions"), tok_seq=view("tok_seq"),
            cu_seqlens=view("cu"), seq_ctx=view("seq_ctx"), seq_slot=view("seq_slot"),
            block_tables={g: view(("table", g)).view(S, self.width) for g in self.groups},
            states=cache.states, state_groups=cache.state_groups, page_size=cache.page_size,
            host=HostLayout.of_captured_step(False, cache.max_len), tile_source=_FixedTiles(views))
        self.view = view
        self.graph = None
        self.launches = 0

    def body(self, model):
        from tokenomos_b200.sampling import sampler

        v = self.view
        h = model.embed_fed(v("ids_host"), v("use_prev"), self.last_token, v("tok_slot"))
        out = model.forward(h, self.ctx)
        logits = model.logits(out, v("want"))
        sampler.sample_packed(logits, v("sampling"), self.sampled,
                              scatter=(v("want_slot"), self.last_token))

    def capture(self, model, pool):
        from tokenomos_b200.ops import _lib

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.body(model)              # warm-up outside the capture (library handles, sizes)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = _lib.calls()
        with _no_collection(), torch.cuda.graph(graph, pool=pool):
            self.body(model)
        self.launches = _lib.calls() - before
        self.graph = graph
        _forget_capture_run()

    def fill(self, turn: int, entries: list[StepEntry], states: list, sampling_rows: list[tuple],
             fed_on_device: list[bool]) -> int:
        """Write the step's layout into staging buffer ``turn``; returns the wanted-row count."""
        from tokenomos_b200.sampling import sampler

        h, T, S = self.host_np[turn], self.tokens_cap, self.seqs_cap
        n = len(entries)
        lens = [len(e.tokens) for e in entries]
        total = sum(lens)
        pad = T - total
        lens_np = np.asarray(lens, dtype=np.int32)
        ctx_np = np.asarray([st.length for st in states], dtype=np.int32)
        slot_np = np.asarray([st.slot for st in states], dtype=np.int32)
        cu = np.zeros(n + 1, dtype=np.int32)
        np.cumsum(lens_np, out=cu[1:])

        def put(name, values, fill=0):
            o, cap = self.off[name]
            k = len(values)
            h[o:o + k] = values
            h[o + k:o + cap] = fill

        put("positions", np.arange(total, dtype=np.int32) + np.repeat(ctx_np - cu[:-1], lens_np))
        put("tok_seq", np.repeat(np.arange(n, dtype=np.int32), lens_np), n)       # padding: the dummy sequence
        use_prev = np.repeat(np.asarray(fed_on_device, dtype=np.int32), lens_np)
        ids = np.fromiter(itertools.chain.from_iterable(e.tokens for e in entries), dtype=np.int32, count=total)
        ids[use_prev != 0] = 0               # a token fed on the device has no value on the host
        put("ids_host", ids)
        put("use_prev", use_prev)
        put("tok_slot", np.repeat(slot_np, lens_np))
        put("cu", cu, T)                         # the dummy sequence takes the rest; then empty ones
        put("seq_ctx", ctx_np)
        put("seq_slot", slot_np)
        want, want_slot = [], []
        for i, e in enumerate(entries):
            for w in e.want:
                want.append(int(cu[i]) + w)
                want_slot.append(int(slot_np[i]))
        put("want", want)
        put("want_slot", want_slot)
        o, _ = self.off["sampling"]
        sampler.pack_rows_into(h[o:o + 6 * S], sampling_rows, S)
        # block tables: a row that held the same request the last time this staging buffer was
        # used only gets its new entries (a window group's entries also turn to 0: rewritten)
        for g in self.groups:
            o, _ = self.off[("table", g)]
            held = self.table_rows[turn][g]
            incremental = self.windowless[g]
            for i, (e, st) in enumerate(zip(entries, states)):
                row = st.tables[g]
                base = o + i * self.width
                held_rid, held_len = held[i]
                if incremental and held_rid == (e.rid, st.epoch) and held_len <= len(row):
                    if held_len < len(row):
                        h[base + held_len:base + len(row)] = row[held_len:]
                else:
                    h[base:base + len(row)] = row
                    if held_len > len(row):
                        h[base + len(row):base + held_len] = 0
                held[i] = ((e.rid, st.epoch), len(row))
            for i in range(n, S):
                if held[i][1]:
                    h[o + i * self.width:o + i * self.width + held[i][1]] = 0
                if held[i][0] is None:
                    break                    # rows beyond were cleared before
                held[i] = (None, 0)
        for key in self.tile_keys:
            seq, tok0, off, cnt = _Tiles.cut(lens, key[0], key[1])
            o, _ = self.off[("tiles", key)]
            k, cap = len(seq), self.tile_cap[key]
            for j, (values, fill) in enumerate(((seq, 0), (tok0, 0), (off, 1), (cnt, 0))):
                h[o + j * cap:o + j * cap + k] = values
                h[o + j * cap + k:o + (j + 1) * cap] = fill
        singles = [int(cu[i]) for i, m in enumerate(lens) if m == 1]
        put("singles", singles, -1)
        return len(want)


class StepFunction:
    def __init__(self, model, cache: CacheManager, staging_ints: int = 1 << 20):
        self.model, self.cache = model, cache
        self.device = cache.device
        self._graphs: dict[int, _DecodeGraph] = {}
        self._step_graphs: dict[tuple, _StepGraph] = {}
        self._step_graph_uses: dict[tuple, int] = {}
        self._graph_pool = None
        self._tile_keys: set = set()     # what the model's parts ask the tile source for
        self._tiles_known = False        # an eager step with a prompt portion has run: the set is complete
        # a mixed step's bucket is captured once this many steps have fallen into it
        self.capture_after = 2
        # the token each request's last step sampled, by state slot (slot 0: padded rows)
        self.last_token = torch.zeros(cache.max_requests + 1, dtype=torch.int32, device=self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # pinned staging for the layout, used round-robin so that a copy still in flight is
        # never overwritten (each buffer is reused only after `ring` later uploads)
        self._ring = [torch.empty(staging_ints, dtype=torch.int32).pin_memory()
                      if self.device.type == "cuda" else torch.empty(staging_ints, dtype=torch.int32)
                      for _ in range(4)]
        self._ring_events = [None] * len(self._ring)
        self._ring_pos = 0
        self.steps = 0
        if self.device.type == "cuda":
            from tokenomos_b200 import ops
            if ops.checks_enabled():         # the debug build: tell the kernels the pools' sizes
                ops.set_check_bounds(cache.num_pages, cache.max_requests + 1)

    def _upload(self, values) -> torch.Tensor:
        """Host ints (a list, or a numpy int32 array) -> device int32 tensor through pinned
        memory, without a sync."""
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
        buf.numpy()[:n] = values
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        out.copy_(buf[:n], non_blocking=True)
        self.h2d_bytes += 4 * n
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._ring_events[i] = ev
        return out

    def _reserve(self, entries: list[StepEntry]) -> None:
        """Check the entries and hold pages for their tokens. All or nothing: the pages the
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

    def layout(self, entries: list[StepEntry]) -> tuple[StepContext, torch.Tensor, torch.Tensor]:
        """Hold pages for the entries' tokens (``_reserve``) and build the step's context; returns
        it with the token ids [T] and the wanted rows [R] (both device int32)."""
        cache = self.cache
        self._reserve(entries)
        seq_lens = [len(e.tokens) for e in entries]
        seq_ctx = [cache.length(e.rid) for e in entries]
        seq_slot = [cache.slot(e.rid) for e in entries]
        S, T = len(entries), sum(seq_lens)
        cu = [0]
        for n in seq_lens:
            cu.append(cu[-1] + n)
        want = []
        for s, e in enumerate(entries):
            want.extend(cu[s] + w for w in e.want)
        lens_np = np.asarray(seq_lens, dtype=np.int32)
        starts = np.repeat(np.asarray(seq_ctx, dtype=np.int32) - np.asarray(cu[:-1], dtype=np.int32), lens_np)
        positions = np.arange(T, dtype=np.int32) + starts
        tok_seq = np.repeat(np.arange(S, dtype=np.int32), lens_np)
        ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int32, count=T)
        groups = list(cache.groups)
        width = max(1, max(-(-(c + n) // cache.page_size) for c, n in zip(seq_ctx, seq_lens)))
        tables = np.zeros((len(groups), S, width), dtype=np.int32)
        for gi, g in enumerate(groups):
            for si, e in enumerate(entries):
                row = cache.block_table(e.rid, g)
                tables[gi, si, :min(width, len(row))] = row[:width]
        flat = self._upload(np.concatenate((
            positions, tok_seq, np.asarray(cu, dtype=np.int32), np.asarray(seq_ctx, dtype=np.int32),
            np.asarray(seq_slot, dtype=np.int32), ids, np.asarray(want, dtype=np.int32),
            tables.reshape(-1))))
        o = 0

        def take(n):
            nonlocal o
            part = flat[o:o + n]
            o += n
            return part

        d_pos, d_tok_seq, d_cu = take(T), take(T), take(S + 1)
        d_ctx, d_slot, d_ids, d_want = take(S), take(S), take(T), take(len(want))
        block_tables = {g: take(S * width).view(S, width) for g in groups}
        host = HostLayout(seq_lens, seq_ctx, seq_slot, all(n == 1 for n in seq_lens),
                          max(c + n for c, n in zip(seq_ctx, seq_lens)))
        ctx = StepContext(
            n_tokens=T, n_seqs=S, positions=d_pos, tok_seq=d_tok_seq, cu_seqlens=d_cu,
            seq_ctx=d_ctx, seq_slot=d_slot, block_tables=block_tables, states=cache.states,
            state_groups=cache.state_groups, page_size=cache.page_size, host=host,
            tile_source=_Tiles(seq_lens, self.device, self._upload, self._tile_keys))
        return ctx, d_ids, d_want

    @torch.no_grad()
    def run(self, entries: list[StepEntry], commit: bool = True) -> torch.Tensor | None:
        """Run one step; returns float32 logits [wanted, vocab] in the order of the entries and
        of their ``want`` lists (None when nothing is wanted). ``commit`` False leaves advancing
        the requests' lengths to the caller (the scheduler does it when it takes the tokens)."""
        ctx, ids, want = self.layout(entries)
        out = self.model.forward(self.model.embed(ids), ctx)
        if not ctx.host.decode_only:
            self._tiles_known = True
        logits = self.model.logits(out, want) if want.numel() else None
        if commit:
            for e in entries:
                self.cache.commit(e.rid, len(e.tokens))
        self.steps += 1
        return logits

    # ---- decode-only steps through a CUDA graph ----

    def decode_graph(self, rows: int) -> _DecodeGraph:
        """The captured decode step of the smallest bucket that holds ``rows`` sequences."""
        bucket = next((b for b in DECODE_BUCKETS if b >= rows), rows)
        bucket = min(bucket, max(rows, self.cache.max_requests))
        g = self._graphs.get(bucket)
        if g is None:
            g = self._graphs[bucket] = _DecodeGraph(self, bucket)
            g.capture(self.model)
        return g

    @torch.no_grad()
    def launch_decode_graph(self, entries: list[StepEntry], sampling_rows: list[tuple],
                            fed_on_device: list[bool] | None = None,
                            commit: bool = False, reserved: bool = False) -> DecodeHandle:
        """Queue one decode step for entries of one token each and return at once: the layout
        goes up in one copy from pinned memory, the captured graph (token select, embedding ...
        sampled token) replays, the tokens come back in one copy; ``handle.tokens()`` waits for
        them. ``fed_on_device[i]``: entry i's token is the one its previous step sampled, which
        the host may not have read yet; the device takes it from ``last_token``. Rows of the
        bucket beyond the entries point at the null slot and the null page. ``reserved``: the
        caller (the scheduler's plan) already holds the pages and has checked the entries."""
        if not reserved:
            for e in entries:
                if len(e.tokens) != 1:
                    raise ValueError("the decode graph takes one token per request")
                self.cache.extend(e.rid, 1)
        return self.launch_decode_ids([e.rid for e in entries], [e.tokens[0] for e in entries],
                                      sampling_rows, fed_on_device, commit)

    @torch.no_grad()
    def launch_decode_ids(self, rids: list, tokens: list[int], sampling_rows: list[tuple],
                          fed_on_device: list[bool] | None = None, commit: bool = False) -> DecodeHandle:
        """``launch_decode_graph`` for requests whose pages are held already, given as parallel
        lists (request ids, the one token each feeds): what the engine's loop calls every decode
        step, without building an entry per request."""
        from tokenomos_b200.sampling import sampler

        cache = self.cache
        n = len(rids)
        g = self.decode_graph(n)
        turn = g.turn
        g.turn = (turn + 1) % g.RING
        h, rows_held, b, width = g.host_np[turn], g.host_rows[turn], g.rows, g.width
        requests = cache.requests
        states = [requests[rid] for rid in rids]
        lengths = [st.length for st in states]
        for name, values in (("positions", lengths), ("seq_ctx", lengths),
                             ("seq_slot", [st.slot for st in states]),
                             ("ids_host", tokens),
                             ("use_prev", [int(f) for f in fed_on_device] if fed_on_device else [0] * n)):
            o, _ = g.off[name]
            h[o:o + n] = values
            h[o + n:o + b] = 0
        o, _ = g.off["sampling"]
        sampler.pack_rows_into(h[o:o + 6 * b], sampling_rows, b)
        # block tables: a row that held the same request the last time this staging buffer was
        # used only gets its new entries (a window group's entries also turn to 0: rewritten)
        for grp in g.groups:
            o, _ = g.off[("table", grp)]
            held = rows_held[grp]
            incremental = cache.groups[grp].window is None
            for i, (rid, st) in enumerate(zip(rids, states)):
                row = st.tables[grp]
                have = len(row)
                held_rid, held_epoch, held_len = held[i]
                if incremental and held_len <= have and held_rid == rid and held_epoch == st.epoch:
                    if held_len == have:
                        continue                 # the common case: the same pages as last time
                    base = o + i * width
                    h[base + held_len:base + have] = row[held_len:]
                else:
                    base = o + i * width
                    h[base:base + have] = row
                    h[base + have:base + width] = 0
                held[i] = (rid, st.epoch, have)
            for i in range(n, b):
                if held[i][0] is not None:
                    h[o + i * width:o + (i + 1) * width] = 0
                    held[i] = (None, 0, 0)
        g.dev.copy_(g.host[turn], non_blocking=True)
        g.graph.replay()
        g.tokens_host[turn].copy_(g.tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.h2d_bytes += 4 * g.size
        self.d2h_bytes += 4 * b
        self.steps += 1
        if commit:
            for rid in rids:
                cache.commit(rid, 1)
        return DecodeHandle(event, g.tokens_host[turn], n)

    # ---- any step through a CUDA graph ----

    @staticmethod
    def _bucket(value: int, buckets: tuple) -> int | None:
        for b in buckets:
            if value <= b:
                return b
        return None

    def step_graph_for(self, entries: list[StepEntry]) -> "_StepGraph | None":
        """The captured step that takes ``entries`` (prompt portions beside single tokens, one
        wanted row per entry at most), capturing it when its bucket has been met
        ``capture_after`` times; None while it is not worth a capture, or if no bucket fits."""
        total = sum(len(e.tokens) for e in entries)
        if any(len(e.want) > 1 for e in entries) or not self._tiles_known:
            return None
        tokens = self._bucket(total, STEP_TOKEN_BUCKETS)
        # a step that does not fill its bucket needs one more sequence: the dummy one
        seqs = self._bucket(len(entries) + (0 if tokens == total else 1), STEP_SEQ_BUCKETS)
        if tokens is None or seqs is None:
            return None
        key = (tokens, seqs)
        g = self._step_graphs.get(key)
        if g is None:
            uses = self._step_graph_uses.get(key, 0) + 1
            self._step_graph_uses[key] = uses
            if uses <= self.capture_after:
                return None
            g = _StepGraph(self, tokens, seqs, self._tile_keys)
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            g.capture(self.model, self._graph_pool)
            self._step_graphs[key] = g
        elif not self._tile_keys <= set(g.tile_keys) | {"singles"}:
            return None          # a part asked for tiles the capture did not know: run eagerly
        return g

    def capture_shapes(self, decode_rows: int, step_tokens: int, step_seqs: int) -> tuple[int, int]:
        """Record ahead of time what serving would record at first use: the decode step of every
        bucket up to ``decode_rows`` sequences, and the mixed step of every (token, sequence)
        bucket a step of at most ``step_tokens`` tokens and ``step_seqs`` sequences can fall
        into. Mixed shapes need to know which tile lists the model's parts ask for, which the
        first eager step with a prompt portion tells; without one they are left for later.
        Returns how many decode and mixed shapes are now recorded."""
        for b in DECODE_BUCKETS:
            bucket = min(b, max(1, self.cache.max_requests))
            if bucket not in self._graphs:
                self.decode_graph(bucket)
            if b >= decode_rows:
                break
        if self._tiles_known:
            top_tokens = self._bucket(step_tokens, STEP_TOKEN_BUCKETS)
            top_seqs = self._bucket(step_seqs + 1, STEP_SEQ_BUCKETS)      # + the dummy sequence
            below = 0
            for seqs in STEP_SEQ_BUCKETS:
                if top_seqs is None or seqs > top_seqs:
                    break
                for tokens in STEP_TOKEN_BUCKETS:
                    if top_tokens is None or tokens > top_tokens:
                        break
                    # a step of this sequence bucket has more than `below` sequences (one of
                    # them may be the dummy), each with a token
                    if tokens < below or (tokens, seqs) in self._step_graphs:
                        continue
                    g = _StepGraph(self, tokens, seqs, self._tile_keys)
                    if self._graph_pool is None:
                        self._graph_pool = torch.cuda.graph_pool_handle()
                    g.capture(self.model, self._graph_pool)
                    self._step_graphs[(tokens, seqs)] = g
                below = seqs
        return len(self._graphs), len(self._step_graphs)

    def launch_step_graph(self, g: "_StepGraph", entries: list[StepEntry], sampling_rows: list[tuple],
                          fed_on_device: list[bool], reserved: bool = False) -> DecodeHandle:
        """Queue one step through its captured graph and return at once (see
        ``launch_decode_graph``): ``handle.tokens()`` waits for the sampled tokens, in the order
        of the entries that want one."""
        cache = self.cache
        if not reserved:
            self._reserve(entries)
        turn = g.turn
        g.turn = (turn + 1) % g.RING
        states = [cache.requests[e.rid] for e in entries]
        wanted = g.fill(turn, entries, states, sampling_rows, fed_on_device)
        g.dev.copy_(g.host[turn], non_blocking=True)
        g.graph.replay()
        g.tokens_host[turn].copy_(g.sampled, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.h2d_bytes += 4 * g.size
        self.d2h_bytes += 4 * g.seqs_cap
        self.steps += 1
        return DecodeHandle(event, g.tokens_host[turn], wanted)

    def run_decode_graph(self, entries: list[StepEntry], sampling_rows: list[tuple],
                         commit: bool = False) -> list[int]:
        """``launch_decode_graph`` and wait: the sampled token of each entry."""
        return self.launch_decode_graph(entries, sampling_rows, None, commit).tokens()
