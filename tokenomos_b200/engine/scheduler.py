"""The scheduler: which requests run in the next step, and with how many of their tokens.

Every step is one mixed batch under a token budget: first one token for each request that is
decoding (oldest first), then the next portion of each request still reading its prompt, then
new admissions in arrival order while a slot, the pages for the whole prompt and budget remain.
The reference admits and prefills to completion before its next decode step and never mixes
(Tokenomos core/engine.py:402-419,720-746); its token budget per prefill forward
(``prefill_budget``) is this scheduler's budget per step.

Pages run out (decided here, tested in tests/test_scheduler.py):

1. a request whose prompt plus ``max_new`` can never fit the pool or the block table is refused
   at ``add`` (as Tokenomos core/engine.py:605-617 refuses at submit);
2. nothing new is admitted while the pages for its whole prompt (plus one token) are not free;
3. if a running request cannot get the page its next token or portion needs, the *newest*
   running request is preempted: pages and slot go back, the request returns to the front of
   the waiting queue and is later recomputed from its prompt plus the tokens it has generated.
   The oldest request always proceeds, so the queue drains. Sampling is keyed by (seed, number
   of tokens generated), so a recomputed request continues with the same tokens.
   (The reference lets the newest rows sit out with their state intact instead,
   core/engine.py:843-858; recomputing needs no pages held by idle rows.)

The scheduler owns no device memory and runs no kernel: ``plan`` returns what to run,
``commit`` takes the sampled tokens. Both are plain host code.
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field

from tokenomos_b200.cache.manager import CacheManager, OutOfPages

MAX_STOPS = 8


@dataclass(eq=False)      # requests are compared by identity (membership tests in the queues)
class Request:
    """One generation request (names as Tokenomos core/engine.py:50-66)."""

    prompt: list[int]
    max_new: int = 256
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int = 0
    stop: tuple[int, ...] = ()
    on_done: object = None
    on_tokens: object = None
    # filled by the scheduler
    rid: int = -1
    output: list[int] = field(default_factory=list)
    computed: int = 0          # tokens of prompt + output that are in the cache
    finish: str | None = None  # "stop" | "length"
    preemptions: int = 0
    arrival: int = -1
    result: object = None
    # tokens sampled on the device whose values the host has not read yet (a step in flight)
    inflight: int = 0

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    def span(self, start: int, count: int) -> list[int]:
        """``tokens[start:start + count]`` without joining the two lists."""
        n = len(self.prompt)
        if start + count <= n:
            return self.prompt[start:start + count]
        if start >= n:
            return self.output[start - n:start - n + count]
        return self.prompt[start:] + self.output[:start + count - n]

    @property
    def total(self) -> int:
        """Tokens of the sequence so far, those still in flight included."""
        return len(self.prompt) + len(self.output) + self.inflight

    @property
    def pending(self) -> int:
        """Tokens (known or in flight) not yet in the cache."""
        return self.total - self.computed

    @property
    def sampled_all(self) -> bool:
        """Every token the request may generate has been sampled (some may be in flight)."""
        return len(self.output) + self.inflight >= self.max_new


@dataclass(slots=True)
class Planned:
    """One request's share of the next step: tokens ``[start, start + count)`` of prompt +
    output; ``sample``: the share reaches the end of what is known, so its last position's
    logits are sampled. ``fed_on_device``: the share is the one token an earlier step sampled
    and the host has not read yet; the device feeds it."""

    req: Request
    start: int
    count: int
    sample: bool
    fed_on_device: bool = False


class NeedsDrain(Exception):
    """The plan needs token values that are still in flight (a preemption, or a share that is
    not a single decoded token): read the steps in flight first, then plan again."""


class Scheduler:
    def __init__(self, cache: CacheManager, token_budget: int = 2048, max_seqs: int | None = None):
        if token_budget < 1:
            raise ValueError("token_budget must be at least 1")
        self.cache = cache
        self.token_budget = token_budget
        self.max_seqs = max_seqs or cache.max_requests
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in admission order (oldest first)
        self._ids = itertools.count()
        self._arrivals = itertools.count()
        self.stats = {"steps": 0, "preemptions": 0, "admitted": 0, "finished": 0}

    # ---- requests in ----

    def check(self, req: Request) -> None:
        """Raise ``ValueError`` for a request this engine can never serve."""
        cache = self.cache
        if req.max_new < 1:
            raise ValueError(f"max_new {req.max_new}: a reply has at least one token")
        if not req.prompt:
            raise ValueError("empty prompt")
        if len(req.stop) > MAX_STOPS:
            raise ValueError(f"{len(req.stop)} stop tokens (at most {MAX_STOPS})")
        total = len(req.prompt) + req.max_new
        if total > cache.max_len:
            raise ValueError(f"request too long: {len(req.prompt)} + {req.max_new} tokens exceed "
                             f"the longest sequence ({cache.max_len})")
        held = (cache.num_pages - 1) * cache.page_size
        if total > held:
            raise ValueError(f"request needs {total} tokens of the {held} the page pool holds")

    def add(self, req: Request) -> None:
        self.check(req)
        req.rid = next(self._ids)
        req.arrival = next(self._arrivals)
        self.waiting.append(req)

    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- one step ----

    def _pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.cache.page_size)

    def _preempt(self, victim: Request) -> None:
        self.running.remove(victim)
        self.cache.release(victim.rid)
        victim.computed = 0
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        self.stats["preemptions"] += 1

    def _outstanding(self) -> int:
        """Pages the running requests will still ask for to finish reading what they know."""
        total = 0
        for req in self.running:
            held = self._pages_for(self.cache.requests[req.rid].reserved)
            total += max(0, self._pages_for(req.total + 1) - held)
        return total

    def inflight(self) -> bool:
        return any(r.inflight for r in self.running)

    def plan(self) -> list[Planned]:
        """Decide the next step and hold its pages (``CacheManager.extend``)."""
        cache, budget = self.cache, self.token_budget
        planned: list[Planned] = []
        # 1 and 2: running requests, oldest first; a decoding one takes one token, one still
        # reading its prompt a portion of what is left of the budget. Victims are always the
        # newest, which this loop has not planned yet.
        preempted = False                     # membership tests only once somebody has left
        try_extend = cache.try_extend
        for req in tuple(self.running):
            if preempted and req not in self.running:       # preempted while serving an older one
                continue
            if budget <= 0:
                break
            total = len(req.prompt) + len(req.output) + req.inflight
            count = min(total - req.computed, budget)
            if count <= 0 or len(req.output) + req.inflight >= req.max_new:
                # nothing left to compute: its last token is sampled (in flight until the next
                # delivery), and the cache entry of a token nobody will follow is never read
                continue
            fed = req.inflight > 0
            if fed and not (count == 1 and req.inflight == 1):
                raise NeedsDrain("only a single decoded token can be fed on the device")
            while not try_extend(req.rid, count):
                if self.inflight():
                    raise NeedsDrain("a preemption needs every token value on the host")
                victim = self.running[-1]
                if victim is req and len(self.running) == 1:
                    raise OutOfPages(f"request {req.rid} cannot get its pages although it is "
                                     "alone in the pool")
                self._preempt(victim)
                preempted = True
                if victim is req:
                    break
            if preempted and req not in self.running:
                continue
            sample = req.computed + count == total and len(req.output) + req.inflight < req.max_new
            planned.append(Planned(req, req.computed, count, sample, fed))
            budget -= count
        # 3: admissions, in arrival order (a preempted request is at the front)
        while self.waiting and budget > 0 and len(self.running) < self.max_seqs:
            req = self.waiting[0]
            need = self._pages_for(len(req.prompt) + len(req.output) + 1)
            if need + self._outstanding() > cache.free_pages() or cache.free_slots() < 1:
                break
            self.waiting.popleft()
            cache.admit(req.rid)
            count = min(req.pending, budget)
            cache.extend(req.rid, count)
            self.running.append(req)
            self.stats["admitted"] += 1
            planned.append(Planned(req, 0, count, count == len(req.tokens)))
            budget -= count
        if not planned and (self.running or self.waiting):
            if self.inflight():
                raise NeedsDrain("nothing to run until the steps in flight are read")
            raise OutOfPages("the scheduler can run nothing: the pool is too small for the "
                             "oldest request")
        self.stats["steps"] += bool(planned)
        return planned

    def launch(self, planned: list[Planned]) -> None:
        """The step has been handed to the device: advance every planned request's length; the
        tokens it samples are in flight until ``deliver``."""
        commit = self.cache.commit
        for p in planned:
            req, count = p.req, p.count
            commit(req.rid, count)
            req.computed += count
            if p.sample:
                req.inflight += 1

    def deliver(self, planned: list[Planned], sampled: list[int]) -> list[Request]:
        """The sampled tokens of a launched step (one per share with ``sample``, in order):
        append them, finish and free what is done. A request that an earlier delivery finished
        (a stop token seen one step late) drops its token."""
        it = iter(sampled)
        finished = []
        for p in planned:
            if not p.sample:
                continue
            req = p.req
            tok = int(next(it))
            req.inflight -= 1
            if req.finish is not None:
                continue
            req.output.append(tok)
            if req.on_tokens is not None:
                req.on_tokens([tok])
            if tok in req.stop:
                req.finish = "stop"
            elif len(req.output) >= req.max_new:
                req.finish = "length"
            if req.finish is not None:
                self.running.remove(req)
                self.cache.release(req.rid)
                self.stats["finished"] += 1
                finished.append(req)
        return finished

    def commit(self, planned: list[Planned], sampled: list[int]) -> list[Request]:
        """``launch`` and ``deliver`` in one call, for a step whose tokens are read at once."""
        self.launch(planned)
        return self.deliver(planned, sampled)
