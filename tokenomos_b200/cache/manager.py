"""The cache manager: pages of keys and values with a block table per request, and slots for
per-request state of fixed size.

What the model asks for arrives as ``StateSpec``s keyed by (entry of the layer list, name).
Paged specs are sorted into *groups* by what they keep (every position, or a window of the last
``w``); each group has its own pool of page numbers and its own block table per request, and
every layer of the group indexes its own tensor ``[pages, 2, kv_heads, page, head_dim]`` with
the group's page numbers. Pages return to the group's pool when the request ends, or, in a
window group, as soon as no later query can see them, and are handed out again (lowest number
first, so runs are reproducible). Page 0 of every pool and slot 0 are never handed out: padded
rows of a batch point there. Fixed-size state (``SlotState``) is a row ``[*shape]`` per request
in a ``[slots, *shape]`` tensor; a request starting at position 0 reads it as zeros by
contract, so rows are not cleared on reuse.

The bookkeeping is plain host code and is tested without a GPU (``device="meta"`` or "cpu");
the reference keeps the same books on the device (Tokenomos core/state.py:19-46,
core/pools.py:90-108, kernels/engine/slots.py:20-108).
"""

from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field

import torch

from tokenomos_b200.parts.contract import StateKey, StateSpec


class OutOfPages(RuntimeError):
    """A request needs more pages (or a slot) than the pool has free right now."""


class CacheError(RuntimeError):
    """The manager's books were used wrongly (unknown request, double free, ...)."""


class FreeList:
    """Numbers ``first .. count-1``, handed out lowest first, each held at most once."""

    def __init__(self, count: int, first: int = 1):
        self.count, self.first = count, first
        self._heap = list(range(first, count))
        heapq.heapify(self._heap)
        self._held: set[int] = set()

    def __len__(self) -> int:
        return len(self._heap)

    def take(self) -> int:
        if not self._heap:
            raise OutOfPages("pool is empty")
        n = heapq.heappop(self._heap)
        self._held.add(n)
        return n

    def give(self, n: int) -> None:
        if n not in self._held:
            raise CacheError(f"{n} given back but not held (freed twice, or never taken)")
        self._held.remove(n)
        heapq.heappush(self._heap, n)

    @property
    def held(self) -> set[int]:
        return self._held


@dataclass
class Group:
    """Paged layers that keep the same positions: one page numbering, one block table."""

    key: tuple
    window: int | None
    pages: FreeList
    members: list[StateKey] = field(default_factory=list)


@dataclass
class RequestState:
    slot: int
    length: int = 0                                   # tokens in the cache
    reserved: int = 0                                 # tokens pages are held for (>= length)
    tables: dict[tuple, list[int]] = field(default_factory=dict)  # group -> page per block (0: none)
    epoch: int = 0                                    # distinguishes two lives of one request id
    # per group: blocks below this index have been given back (a window has passed them); every
    # block from here to the end of the table holds a page
    first_live: dict[tuple, int] = field(default_factory=dict)
    # tokens the tables of every group already reach (the shortest table times the page size):
    # an extension below this needs no page
    held_tokens: int = 0


class CacheManager:
    def __init__(self, specs: dict[StateKey, StateSpec], page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype, device, max_len: int | None = None,
                 poison: bool = False):
        """``num_pages``: pages of each group's pool, the null page included. ``max_requests``:
        live requests (slots 1..max_requests). ``max_len``: longest sequence (sets the block
        table's width; default: what the pool could hold). ``poison`` (for tests): every page
        and every state row that no live request holds is kept full of NaN (all of them at the
        start, each again when it is given back), so that a kernel that reads a position it must
        not read, or a stale state row, shows in the logits; the null page and the null row stay
        zero."""
        if page_size < 1 or num_pages < 2 or max_requests < 1:
            raise ValueError("cache: page_size >= 1, num_pages >= 2 (page 0 is the null page), "
                             "max_requests >= 1")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device = dtype, torch.device(device)
        self.max_len = max_len or (num_pages - 1) * page_size
        self.max_blocks = -(-self.max_len // page_size)
        self.specs = dict(specs)
        self.groups: dict[tuple, Group] = {}
        self.states: dict[StateKey, torch.Tensor] = {}
        self.state_groups: dict[StateKey, tuple] = {}
        self.slots = FreeList(max_requests + 1, first=1)
        self.requests: dict[object, RequestState] = {}
        # what a spec needs is said by the spec itself (``storage`` and the attributes that go
        # with it, see parts.contract), so a part may bring a spec class of its own
        for key, spec in specs.items():
            storage = getattr(spec, "storage", None)
            if storage == "paged":
                g = self.groups.get(spec.group)
                if g is None:
                    g = self.groups[spec.group] = Group(spec.group, spec.window, FreeList(num_pages))
                elif g.window != spec.window:
                    raise ValueError(f"state {key}: cache group {spec.group} holds a window of "
                                     f"{g.window}, this spec asks for {spec.window}")
                g.members.append(key)
                shape = (num_pages, *spec.page_shape(page_size))
                self.states[key] = torch.zeros(shape, dtype=dtype, device=self.device)
                self.state_groups[key] = spec.group
            elif storage == "slot":
                self.states[key] = torch.zeros((max_requests + 1, *spec.shape),
                                               dtype=spec.dtype or dtype, device=self.device)
            elif storage != "shared":
                raise ValueError(f"state {key}: a spec's storage is 'paged', 'slot' or 'shared', "
                                 f"not {storage!r}")
        for key, spec in specs.items():
            if spec.storage == "shared":
                src = (spec.source, spec.name)
                if src not in self.states:
                    raise ValueError(f"state {key} reads {src}, which owns no memory")
                self.states[key] = self.states[src]
                if src in self.state_groups:
                    self.state_groups[key] = self.state_groups[src]

        # the groups whose pages a window gives back as a request advances
        self._windowed = [(k, g) for k, g in self.groups.items() if g.window is not None]
        self.poison = bool(poison)
        if self.poison:
            for key, spec in specs.items():
                if spec.storage != "shared" and self.states[key].dtype.is_floating_point:
                    self.states[key][1:] = float("nan")

    def _poison_pages(self, group: Group, pages: list[int]) -> None:
        if pages:
            index = torch.tensor(pages, dtype=torch.long, device=self.device)
            for key in group.members:
                self.states[key].index_fill_(0, index, float("nan"))

    def _poison_slot(self, slot: int) -> None:
        for key, spec in self.specs.items():
            if spec.storage == "slot" and self.states[key].dtype.is_floating_point:
                self.states[key][slot] = float("nan")

    # ---- sizes ----

    def bytes_per_page(self) -> int:
        """Bytes one page costs across every paged layer (all groups)."""
        total = 0
        for key, spec in self.specs.items():
            if spec.storage == "paged":
                total += math.prod(spec.page_shape(self.page_size)) * self.dtype.itemsize
        return total

    def bytes_per_slot(self) -> int:
        """Bytes one request's fixed-size state rows cost across every layer."""
        total = 0
        for key, spec in self.specs.items():
            if spec.storage == "slot":
                total += math.prod(spec.shape) * (spec.dtype or self.dtype).itemsize
        return total

    def free_pages(self, group: tuple | None = None) -> int:
        """Free pages of ``group``, or the smallest count over the groups."""
        if group is not None:
            return len(self.groups[group].pages)
        return min((len(g.pages) for g in self.groups.values()), default=1 << 30)

    def free_slots(self) -> int:
        return len(self.slots)

    # ---- a request's life ----

    def admit(self, rid) -> RequestState:
        """Give ``rid`` a slot (no pages yet)."""
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already live")
        if not len(self.slots):
            raise OutOfPages("no free slot")
        self._epoch = getattr(self, "_epoch", 0) + 1
        st = RequestState(self.slots.take(), tables={k: [] for k in self.groups}, epoch=self._epoch)
        if not self.groups:
            st.held_tokens = self.max_len          # nothing is paged: no extension needs a page
        self.requests[rid] = st
        return st

    def _first_needed_block(self, g: Group, ctx: int) -> int:
        """First block a query at position ``ctx`` or later can read in group ``g``."""
        if g.window is None:
            return 0
        return max(0, ctx - g.window + 1) // self.page_size

    def pages_needed(self, rid, n_new: int) -> dict[tuple, int]:
        """Pages each group must still hand out so ``rid`` can take ``n_new`` more tokens."""
        st = self._get(rid)
        end_block = -(-(st.length + n_new) // self.page_size)
        need = {}
        for k, g in self.groups.items():
            # blocks [first_live, len(table)) hold pages; the step needs [lo, end_block)
            lo = max(self._first_needed_block(g, st.length), st.first_live.get(k, 0))
            have = max(0, min(len(st.tables[k]), end_block) - lo)
            need[k] = max(0, end_block - lo - have)
        return need

    def _already_held(self, st: RequestState, n_new: int) -> bool:
        """Every group's table already reaches the block of position ``length + n_new - 1`` (the
        common case of a decoded token inside its last page): nothing to count or to take."""
        end_block = -(-(st.length + n_new) // self.page_size)
        for table in st.tables.values():
            if len(table) < end_block:
                return False
        return True

    def can_extend(self, rid, n_new: int) -> bool:
        st = self._get(rid)
        if st.length + n_new > self.max_len:
            return False
        if self._already_held(st, n_new):
            return True
        return all(n <= len(self.groups[k].pages) for k, n in self.pages_needed(rid, n_new).items())

    def try_extend(self, rid, n_new: int) -> bool:
        """``can_extend`` and, if it can, ``extend``, in one call: what the scheduler asks for
        every running request every step. The common case, a decoded token inside its last page,
        is two comparisons."""
        st = self.requests.get(rid)
        if st is None:
            raise CacheError(f"request {rid!r} is not live")
        end = st.length + n_new
        if end <= st.held_tokens and end <= self.max_len:
            if end > st.reserved:
                st.reserved = end
            return True
        if not self.can_extend(rid, n_new):
            return False
        self.extend(rid, n_new)
        return True

    def extend(self, rid, n_new: int) -> None:
        """Hold pages for positions ``[length, length + n_new)`` in every group; all or nothing."""
        st = self._get(rid)
        if st.length + n_new > self.max_len:
            raise OutOfPages(f"request {rid!r}: {st.length} + {n_new} tokens exceed the longest "
                             f"sequence the block table holds ({self.max_len})")
        if self._already_held(st, n_new):
            st.reserved = max(st.reserved, st.length + n_new)
            return
        need = self.pages_needed(rid, n_new)
        short = {k: (n, len(self.groups[k].pages)) for k, n in need.items()
                 if n > len(self.groups[k].pages)}
        if short:
            raise OutOfPages(f"request {rid!r} needs pages (group: needed, free) {short}")
        end_block = -(-(st.length + n_new) // self.page_size)
        for k, g in self.groups.items():
            table = st.tables[k]
            # a table only grows at its end: blocks behind a window were given back for good
            for _ in range(len(table), end_block):
                table.append(g.pages.take())
        st.reserved = max(st.reserved, st.length + n_new)
        st.held_tokens = min(len(t) for t in st.tables.values()) * self.page_size

    def commit(self, rid, n_new: int) -> None:
        """The step wrote ``n_new`` tokens: advance, and give back what a window has passed."""
        st = self._get(rid)
        if st.length + n_new > st.reserved:
            raise CacheError(f"request {rid!r}: commit of {n_new} tokens beyond what was extended")
        st.length += n_new
        for k, g in self._windowed:
            table = st.tables[k]
            passed = min(self._first_needed_block(g, st.length), len(table))
            if self.poison:
                self._poison_pages(g, [table[b] for b in range(st.first_live.get(k, 0), passed)])
            for b in range(st.first_live.get(k, 0), passed):
                g.pages.give(table[b])
                table[b] = 0
            st.first_live[k] = max(st.first_live.get(k, 0), passed)

    def release(self, rid) -> None:
        """The request ended: its pages and its slot go back."""
        st = self.requests.pop(rid, None)
        if st is None:
            raise CacheError(f"request {rid!r} is not live (released twice?)")
        for k, g in self.groups.items():
            for page in st.tables[k]:
                if page:
                    g.pages.give(page)
            if self.poison:
                self._poison_pages(g, [page for page in st.tables[k] if page])
        if self.poison:
            self._poison_slot(st.slot)
        self.slots.give(st.slot)

    def _get(self, rid) -> RequestState:
        st = self.requests.get(rid)
        if st is None:
            raise CacheError(f"request {rid!r} is not live")
        return st

    def length(self, rid) -> int:
        return self._get(rid).length

    def slot(self, rid) -> int:
        return self._get(rid).slot

    def block_table(self, rid, group: tuple) -> list[int]:
        return self._get(rid).tables[group]

    # ---- invariants (tests call this after every operation) ----

    def check(self) -> None:
        """No page lost, none held twice: per group, pages held by requests and free pages
        partition ``1 .. num_pages-1``; same for slots."""
        for k, g in self.groups.items():
            held = [p for st in self.requests.values() for p in st.tables[k] if p]
            if len(held) != len(set(held)):
                raise CacheError(f"group {k}: a page is held twice")
            if set(held) != g.pages.held:
                raise CacheError(f"group {k}: pages held by requests differ from the pool's books")
            free = set(g.pages._heap)
            if len(free) != len(g.pages._heap) or free & set(held):
                raise CacheError(f"group {k}: a page is both free and held, or free twice")
            if free | set(held) != set(range(1, self.num_pages)):
                raise CacheError(f"group {k}: a page is lost")
        slots = [st.slot for st in self.requests.values()]
        if len(slots) != len(set(slots)) or set(slots) != self.slots.held:
            raise CacheError("slots: held twice or lost")
