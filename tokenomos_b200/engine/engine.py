"""The engine: cache manager + step function + scheduler + sampler behind ``submit`` / ``run``.

Per host iteration: take new requests off the inbox, let the scheduler plan one mixed step
(decode tokens and prompt portions under the token budget), run it through the step function,
sample the rows whose share reached the end of their known tokens, read the sampled tokens
back, and let the scheduler finish and free. Keyword arguments follow the reference's
``Engine`` where it has them: ``slots``, ``page``, ``max_len``, ``pages``, ``prefill_budget``,
``graphs`` (Tokenomos core/engine.py:148-184).
"""

from __future__ import annotations

import queue
import threading
import time
import warnings
from dataclasses import dataclass, field

import torch

from collections import deque

from tokenomos_b200 import ops
from tokenomos_b200.cache.manager import CacheManager

from tokenomos_b200.engine.scheduler import NeedsDrain, Planned, Request, Scheduler
from tokenomos_b200.engine.step import StepEntry, StepFunction
from tokenomos_b200.sampling import sampler


def _nvtx_push(name: str) -> None:
    """An NVTX range around a phase of the host loop (``plan``, ``launch``, ``wait``, ``deliver``,
    ``idle``; the reference marks ``admit / decode / wait / idle``, Tokenomos
    core/engine.py:692,752,763,794), so that a timeline shows which side a step waited on.
    Without a profiler attached a range costs a fraction of a microsecond."""
    torch.cuda.nvtx.range_push(name)


def _nvtx_pop() -> None:
    torch.cuda.nvtx.range_pop()


@dataclass
class Result:
    tokens: list[int]
    finish: str


@dataclass
class Stats:
    steps: int = 0
    decode_steps: int = 0          # steps in which every row brought one token
    graph_steps: int = 0           # mixed steps that replayed a captured graph
    prefill_tokens: int = 0
    generated: int = 0
    preemptions: int = 0
    wall_s: float = 0.0
    # (perf_counter, rows, tokens) at each step's start
    stamps: list = field(default_factory=list)


class Engine:
    def __init__(self, model, slots: int = 64, page: int = 16, max_len: int = 4096,
                 pages: int | None = None, prefill_budget: int = 2048, graphs: bool = True,
                 kv_fraction: float = 0.8, device: str = "cuda", poison: bool = False,
                 warmup: bool = False):
        """``slots``: live requests. ``page``: tokens per cache page. ``max_len``: longest
        sequence (prompt + reply). ``pages``: pages per cache group, the null page included
        (None: ``kv_fraction`` of the free memory, at most what ``slots`` sequences of
        ``max_len`` need). ``prefill_budget``: tokens per step. ``graphs``: steps replay
        captured CUDA graphs (decode-only steps per batch-size bucket, mixed steps per token and
        sequence bucket). ``poison`` (for tests): the cache manager keeps every page and state
        row that no request holds full of NaN. ``warmup``: call ``warmup()`` before
        the first request is served."""
        self.model = model
        self.device = torch.device(device)
        specs = model.state_specs()
        if pages is None:
            # the fixed-size state rows come first, the pages share what is left (as the
            # reference sizes its pools, Tokenomos core/pools.py:34-68)
            probe = CacheManager(specs, page, 2, 1, model.dtype, "meta", max_len)
            per_page = max(1, probe.bytes_per_page())
            free = torch.cuda.mem_get_info(self.device)[0] - (slots + 1) * probe.bytes_per_slot()
            if free <= 0:
                raise ValueError(f"{slots} state rows of {probe.bytes_per_slot()} bytes exceed the free "
                                 "memory: fewer slots")
            pages = int(free * kv_fraction) // per_page
            pages = max(2, min(pages, slots * -(-max_len // page) + 1))
        self.cache = CacheManager(specs, page, pages, slots, model.dtype, self.device, max_len,
                                  poison=poison)
        self.step_fn = StepFunction(model, self.cache)
        self.scheduler = Scheduler(self.cache, prefill_budget, slots)
        # a step is recorded as a CUDA graph only if every part of the model can be (see
        # parts.contract: capture_safe); otherwise every step runs eagerly
        self.graphs = bool(graphs) and model.capture_safe
        if graphs and not self.graphs:
            warnings.warn("graphs=True, but these parts are not capture_safe: "
                          f"{', '.join(model.not_capture_safe())}; every step runs eagerly", stacklevel=2)
        # decode steps queued on the device whose tokens the host has not read: (plan, handle)
        self._inflight: deque = deque()
        self.depth = 1
        self._checked_at = 0       # stats.steps when the kernels' error word was last read
        self.inbox: queue.Queue[Request] = queue.Queue()
        self.stats = Stats()
        self.prefill_budget, self.slots = prefill_budget, slots
        # ``trace_on()``: one record per step from then on (``trace_take`` hands them over)
        self.trace: list[dict] | None = None
        self._trace_lock = threading.Lock()
        self._wait_s = 0.0
        self._nvtx = self.device.type == "cuda"
        if warmup:
            self.warmup()

    # ---- tracing ----

    def trace_on(self) -> None:
        """Record every step from now on: its kind (``decode``, ``mixed``: a captured mixed step,
        ``eager``), rows, tokens, the captured bucket it replayed, the host's milliseconds to
        plan it, to launch it and waiting for older steps' tokens, and (from two CUDA events
        around the step) its milliseconds on the device. Opt-in, as the reference's per-iteration
        records are (Tokenomos core/engine.py:270-298): the two events cost a few microseconds
        a step."""
        with self._trace_lock:
            self.trace = []

    def trace_take(self) -> list[dict]:
        """The records of the steps finished since the last take, device times filled in (waits
        for their events). Any thread."""
        with self._trace_lock:
            if self.trace is None:
                return []
            records, self.trace = self.trace, []
        out = []
        for rec in records:
            start, end = rec.pop("_events")
            end.synchronize()
            rec["gpu_ms"] = round(start.elapsed_time(end), 4)
            out.append(rec)
        return out

    def _trace_begin(self, t0: float, kind: str, rows: int, tokens: int, bucket) -> dict | None:
        if self._nvtx:
            _nvtx_push("launch")
        if self.trace is None:
            return None
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        now = time.perf_counter()
        return {"step": self.stats.steps, "kind": kind, "rows": rows, "tokens": tokens, "bucket": bucket,
                "captured": kind != "eager", "plan_ms": round((now - t0) * 1e3, 4), "_t": now,
                "_events": (start, None)}

    def _trace_end(self, rec: dict | None) -> None:
        if self._nvtx:
            _nvtx_pop()
        if rec is None:
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        rec["_events"] = (rec["_events"][0], end)
        rec["launch_ms"] = round((time.perf_counter() - rec.pop("_t")) * 1e3, 4)
        rec["wait_ms"] = round(self._wait_s * 1e3, 4)        # waiting for older steps, since the last record
        self._wait_s = 0.0
        with self._trace_lock:
            if self.trace is not None:
                self.trace.append(rec)

    def _deliver_older(self, finished: list[Request]) -> None:
        """Read the tokens of every step in flight beyond ``depth`` (waits for them) and let the
        scheduler take them."""
        while len(self._inflight) > self.depth:
            old_planned, old_handle = self._inflight.popleft()
            if self._nvtx:
                _nvtx_push("wait")
            t = time.perf_counter()
            tokens = old_handle.tokens()
            self._wait_s += time.perf_counter() - t
            if self._nvtx:
                _nvtx_pop()
                _nvtx_push("deliver")
            finished += self.scheduler.deliver(old_planned, tokens)
            if self._nvtx:
                _nvtx_pop()

    def warmup(self) -> tuple[int, int]:
        """Touch every kernel variant and record every step shape serving will meet, before the
        first request (the reference's engine does the same before it serves, Tokenomos
        core/engine.py:635-664): two short requests run one eager mixed step (it builds the
        kernel library if need be, loads the library handles and tells which tile lists the
        model's parts ask for), then the decode step of every batch-size bucket up to ``slots``
        and the mixed step of every (token, sequence) bucket under the token budget are
        captured. Without it each shape is captured when serving first meets it (a mixed one
        the third time). Returns the numbers of decode and mixed shapes recorded; the statistics
        start afresh."""
        vocab, cache = self.model.vocab, self.cache
        longest = min(cache.max_len, (cache.num_pages - 1) * cache.page_size) - 2
        count = min(2, self.slots)
        n = max(2, min(longest // max(1, count), self.prefill_budget // 2 + 3))
        was, self.graphs = self.graphs, False
        try:
            self.generate([Request([(7 * i + r) % vocab for i in range(n)], max_new=2) for r in range(count)])
        finally:
            self.graphs = was
        recorded = (0, 0)
        if self.graphs:
            recorded = self.step_fn.capture_shapes(self.slots, self.prefill_budget, self.slots)
        torch.cuda.synchronize(self.device)
        self.stats = Stats()
        self._checked_at = 0
        return recorded

    # ---- requests in ----

    def submit(self, req: Request) -> None:
        """Queue ``req`` (any thread). A request the engine can never serve fails here."""
        vocab = self.model.vocab
        if req.prompt and (min(req.prompt) < 0 or max(req.prompt) >= vocab):
            raise ValueError(f"prompt token id outside 0..{vocab - 1}")
        self.scheduler.check(req)
        self.inbox.put(req)

    # ---- one iteration ----

    def _take_inbox(self) -> None:
        while True:
            try:
                self.scheduler.add(self.inbox.get_nowait())
            except queue.Empty:
                return

    # a continuously busy engine reads the kernels' error words this often (steps)
    CHECK_EVERY = 512

    def _check_kernels(self) -> None:
        """The tcgen05 kernels bound every wait on a barrier instead of hanging, and record
        where they gave up. Reading the words waits for the device, so it happens where the host
        waits anyway: before the last replies of a batch are handed out, when the engine drains,
        and every ``CHECK_EVERY`` steps of an engine that never goes idle."""
        if self.stats.steps == self._checked_at or self.cache.device.type != "cuda":
            return
        self._checked_at = self.stats.steps
        for what, where in (("GEMM", ops.gemm_tc_status()), ("attention", ops.attention_prefill_tc_status())):
            if where:
                ops.clear_tickets()      # a CTA that gave up may have left its tile's ticket drawn
                raise RuntimeError(f"a tcgen05 {what} kernel gave up waiting on a barrier (place {where}); "
                                   "the tokens of the steps since the last check are not to be trusted")
        if ops.checks_enabled():
            found = ops.checks_status()
            if found:
                raise RuntimeError(f"index check: {found}")
        row = ops.sample_status()
        if row:
            raise RuntimeError(f"the sampler met a row of logits without a finite value (row {row - 1} of "
                               "its step) and answered token 0: the model's weights or its cache hold NaN")

    def _finish(self, finished: list[Request]) -> list[Request]:
        if finished and self.scheduler.idle():
            self._check_kernels()            # nothing is in flight: the check costs nothing
        for req in finished:
            req.result = Result(list(req.output), req.finish)
            if req.on_done is not None:
                req.on_done(req)
        return finished

    def _drain(self) -> list[Request]:
        finished = []
        while self._inflight:
            planned, handle = self._inflight.popleft()
            finished += self.scheduler.deliver(planned, handle.tokens())
        return finished

    def drain(self) -> list[Request]:
        """Read every step in flight: after this the host knows every sampled token. Also a
        place where a kernel that gave up waiting on a barrier turns into an exception."""
        finished = self._finish(self._drain())
        self._check_kernels()
        return finished

    def _decode_step(self, planned, finished: list[Request], t0: float = 0.0) -> list[Request]:
        """Every request decodes one token: the captured decode graph, queued without waiting
        for the step before it. One pass over the plan builds what the graph's layout needs."""
        rids, tokens, rows, fed = [], [], [], []
        for p in planned:
            r = p.req
            rids.append(r.rid)
            fed.append(p.fed_on_device)
            if p.fed_on_device:
                tokens.append(0)
            else:
                at = p.start - len(r.prompt)
                tokens.append(r.output[at] if at >= 0 else r.prompt[p.start])
            rows.append((r.temperature, r.top_p, r.top_k, r.min_p, r.seed, len(r.output) + r.inflight))
        n = len(planned)
        self.stats.stamps.append((time.perf_counter(), n, n))
        self.stats.steps += 1
        self.stats.decode_steps += 1
        bucket = self.step_fn.decode_graph(n).rows if self.trace is not None else None
        rec = self._trace_begin(t0, "decode", n, n, bucket)
        handle = self.step_fn.launch_decode_ids(rids, tokens, rows, fed)
        self._trace_end(rec)
        self.scheduler.launch(planned)
        self._inflight.append((planned, handle))
        self.stats.generated += n
        self._deliver_older(finished)
        self.stats.preemptions = self.scheduler.stats["preemptions"]
        return self._finish(finished)

    @torch.no_grad()
    def step(self) -> list[Request]:
        """Plan and queue one step; returns the requests that finished meanwhile. A step in
        which every request decodes one token replays a CUDA graph and is not waited for: its
        tokens are read while the next step runs (the host stays one step behind the device, as
        the reference's loop does, Tokenomos core/engine.py:1-14); a request that a stop token
        ends therefore decodes one token too many, which is dropped. Any other step (prompt
        portions, a preemption) first reads what is in flight and then runs synchronously."""
        finished: list[Request] = []
        t0 = time.perf_counter()
        if self.stats.steps - self._checked_at >= self.CHECK_EVERY:
            self._check_kernels()
        if self._nvtx:
            _nvtx_push("plan")
        try:
            try:
                planned = self.scheduler.plan()
            except NeedsDrain:
                finished += self._drain()
                if self.scheduler.idle():
                    return self._finish(finished)
                planned = self.scheduler.plan()
        finally:
            if self._nvtx:
                _nvtx_pop()
        if not planned:
            return self._finish(finished + self._drain())
        def entries_of(planned):
            entries, rows = [], []
            for p in planned:
                r = p.req
                toks = [0] * p.count if p.fed_on_device else r.span(p.start, p.count)
                entries.append(StepEntry(r.rid, toks, [p.count - 1] if p.sample else []))
                if p.sample:
                    rows.append((r.temperature, r.top_p, r.top_k, r.min_p, r.seed,
                                 len(r.output) + r.inflight))
            return entries, rows

        decode_only = all(p.count == 1 and p.sample for p in planned)
        if self.graphs and decode_only:
            return self._decode_step(planned, finished, t0)
        entries, rows = entries_of(planned)
        # a captured step (decode-only, or a mixed one whose bucket has been captured) is queued
        # without waiting for the step before it; anything else runs eagerly and needs every
        # token on the host first
        graph = None
        if self.graphs and not decode_only:
            graph = self.step_fn.step_graph_for(entries)
        if not (self.graphs and (decode_only or graph is not None)) and (
                self._inflight or any(p.fed_on_device for p in planned)):
            # undo nothing (pages stay held), read what is in flight, plan again with the tokens known
            finished += self._drain()
            planned = self.scheduler.plan() if not self.scheduler.idle() else []
            if not planned:
                return self._finish(finished)
            decode_only = all(p.count == 1 and p.sample for p in planned)
            entries, rows = entries_of(planned)
            graph = None
        tokens_in_step = sum(p.count for p in planned)
        self.stats.stamps.append((time.perf_counter(), len(planned), tokens_in_step))
        self.stats.steps += 1
        if all(p.count == 1 for p in planned):
            self.stats.decode_steps += 1
        else:
            self.stats.prefill_tokens += sum(p.count for p in planned if p.count > 1)
        if self.graphs and (decode_only or graph is not None):
            fed = [p.fed_on_device for p in planned]
            if decode_only:
                bucket = self.step_fn.decode_graph(len(planned)).rows if self.trace is not None else None
                rec = self._trace_begin(t0, "decode", len(planned), tokens_in_step, bucket)
                handle = self.step_fn.launch_decode_graph(entries, rows, fed, reserved=True)
            else:
                rec = self._trace_begin(t0, "mixed", len(planned), tokens_in_step,
                                        [graph.tokens_cap, graph.seqs_cap])
                handle = self.step_fn.launch_step_graph(graph, entries, rows, fed, reserved=True)
                self.stats.graph_steps += 1
            self._trace_end(rec)
            self.scheduler.launch(planned)
            self._inflight.append((planned, handle))
            self.stats.generated += len(rows)
            self._deliver_older(finished)
        else:
            rec = self._trace_begin(t0, "eager", len(planned), tokens_in_step, None)
            logits = self.step_fn.run(entries, commit=False)
            sampled_dev = None
            if rows:
                packed = self.step_fn._upload(sampler.pack_rows(rows))
                slots = self.step_fn._upload([self.cache.slot(p.req.rid) for p in planned if p.sample])
                sampled_dev = sampler.sample_packed(logits, packed, scatter=(slots, self.step_fn.last_token))
            self._trace_end(rec)
            sampled: list[int] = sampled_dev.tolist() if sampled_dev is not None else []
            self.stats.generated += len(sampled)
            finished += self.scheduler.commit(planned, sampled)
        self.stats.preemptions = self.scheduler.stats["preemptions"]
        return self._finish(finished)

    def run(self, stop: threading.Event | None = None) -> None:
        """The engine's loop. Without ``stop`` it returns once every queued request is answered;
        with ``stop`` (an event, for a worker thread) it keeps serving, sleeping on the inbox for
        a moment whenever there is nothing to do, until the event is set."""
        start = time.perf_counter()
        while True:
            self._take_inbox()
            if self.scheduler.idle():
                self.drain()
                if stop is None or stop.is_set():
                    break
                if self._nvtx:
                    _nvtx_push("idle")
                try:
                    self.scheduler.add(self.inbox.get(timeout=0.02))
                except queue.Empty:
                    continue
                finally:
                    if self._nvtx:
                        _nvtx_pop()
            self.step()
        self.stats.wall_s += time.perf_counter() - start

    def generate(self, requests: list[Request]) -> list[Result]:
        """The replies to ``requests``, in their order: queues them all, then runs the loop on the
        caller's thread until nothing is left to do."""
        for r in requests:
            self.submit(r)
        self.run()
        return [r.result for r in requests]
