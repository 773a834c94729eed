"""The scheduler's decisions (no GPU): admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out. A fake step stands in for the
model: the next token is a function of the whole history, so any scheduling must give the same
replies."""

from __future__ import annotations

import random
from collections import deque

import pytest
import torch

from tokenomos_b200.cache.manager import CacheManager
from tokenomos_b200.engine.scheduler import NeedsDrain, Request, Scheduler
from tokenomos_b200.parts.contract import PagedKV, SlotState

SPECS = {(0, "conv"): SlotState((2, 8)), (1, "kv"): PagedKV(2, 16)}


def fake_next(tokens: list[int]) -> int:
    h = 17
    for t in tokens:
        h = (h * 31 + t) % 1009
    return h % 50


def drive(sched: Scheduler, log=None, limit=10000):
    """Run the scheduler to the end; checks the cache's books and the plan's shape each step."""
    steps = 0
    while not sched.idle():
        planned = sched.plan()
        assert planned
        assert sum(p.count for p in planned) <= sched.token_budget
        assert len({p.req.rid for p in planned}) == len(planned)
        for p in planned:
            assert p.count >= 1 and p.start == p.req.computed
            assert sched.cache.length(p.req.rid) == p.start
        sampled = [fake_next(p.req.tokens[:p.start + p.count]) for p in planned if p.sample]
        if log is not None:
            log.append([(p.req.rid, p.start, p.count, p.sample) for p in planned])
        sched.commit(planned, sampled)
        sched.cache.check()
        steps += 1
        assert steps < limit
    return steps


def make(pages=200, page=4, slots=8, budget=16, max_len=400):
    cache = CacheManager(SPECS, page, pages, slots, torch.float32, "meta", max_len)
    return Scheduler(cache, budget)


def expected(prompt, max_new, stop=()):
    out, toks = [], list(prompt)
    while len(out) < max_new:
        t = fake_next(toks)
        out.append(t)
        toks.append(t)
        if t in stop:
            break
    return out


def test_prompt_is_cut_into_portions_under_the_budget_then_decoded():
    s = make(budget=16)
    r = Request(list(range(40)), max_new=3)
    s.add(r)
    log = []
    drive(s, log)
    assert [step[0][1:] for step in log] == [(0, 16, False), (16, 16, False), (32, 8, True),
                                             (40, 1, True), (41, 1, True)]
    assert r.output == expected(r.prompt, 3) and r.finish == "length"
    assert s.cache.free_pages() == 199 and s.cache.free_slots() == 8


def test_decode_tokens_go_first_and_prompts_share_what_is_left():
    s = make(budget=10)
    a, b = Request([1, 2, 3], max_new=20), Request(list(range(30)), max_new=2)
    s.add(a)
    log = []
    planned = s.plan()
    s.commit(planned, [fake_next(a.prompt)])
    s.add(b)
    drive(s, log)
    # a decodes one token a step and comes first; b's prompt takes the other 9 tokens of the budget
    assert log[0] == [(a.rid, 3, 1, True), (b.rid, 0, 9, False)]
    assert log[1] == [(a.rid, 4, 1, True), (b.rid, 9, 9, False)]
    assert a.output == expected(a.prompt, 20) and b.output == expected(b.prompt, 2)


def test_stop_token_ends_a_request_and_is_kept():
    s = make()
    prompt = [5, 6, 7]
    full = expected(prompt, 12)
    stop = full[4]
    r = Request(prompt, max_new=12, stop=(stop,))
    s.add(r)
    drive(s)
    assert r.finish == "stop" and r.output == full[:full.index(stop) + 1]


def test_requests_that_can_never_fit_are_refused():
    s = make(pages=6, page=4, max_len=100)      # 20 tokens
    with pytest.raises(ValueError, match="page pool"):
        s.add(Request(list(range(15)), max_new=10))
    with pytest.raises(ValueError, match="empty prompt"):
        s.add(Request([], max_new=1))
    with pytest.raises(ValueError, match="at least one token"):
        s.add(Request([1], max_new=0))
    with pytest.raises(ValueError, match="stop tokens"):
        s.add(Request([1], max_new=1, stop=tuple(range(9))))
    s2 = make(max_len=20)
    with pytest.raises(ValueError, match="longest sequence"):
        s2.add(Request(list(range(15)), max_new=10))


def test_admission_waits_for_pages_and_slots():
    s = make(pages=9, page=4, slots=2, budget=64)   # 32 tokens
    a, b, c = (Request(list(range(10)), max_new=4) for _ in range(3))
    for r in (a, b, c):
        s.add(r)
    log = []
    drive(s, log)
    assert {x[0] for x in log[0]} == {a.rid, b.rid}      # two slots: c waits for a finisher
    first_c = next(i for i, step in enumerate(log) if any(x[0] == c.rid for x in step))
    assert first_c >= 4
    for r in (a, b, c):
        assert r.output == expected(r.prompt, 4)


def test_pages_run_out_newest_is_preempted_and_recomputed_with_the_same_tokens():
    # 11 usable pages of 4 = 44 tokens; three requests that each grow to 26 tokens
    s = make(pages=12, page=4, slots=4, budget=32)
    reqs = [Request([i + 1] * 6, max_new=20) for i in range(3)]
    for r in reqs:
        s.add(r)
    log = []
    drive(s, log)
    assert s.stats["preemptions"] >= 1
    assert reqs[0].preemptions == 0                       # the oldest always proceeds
    assert max(r.preemptions for r in reqs[1:]) >= 1
    for r in reqs:
        assert r.output == expected(r.prompt, 20) and r.finish == "length"
    # a preempted request restarts from position 0 with its generated tokens as prompt
    victim = next(r for r in reqs if r.preemptions)
    restarts = [x for step in log for x in step if x[0] == victim.rid and x[1] == 0]
    assert len(restarts) == victim.preemptions + 1 and restarts[-1][2] > 6
    assert s.cache.free_pages() == 11 and s.cache.free_slots() == 4


@pytest.mark.parametrize("seed", range(6))
def test_random_loads_give_the_same_replies_as_a_roomy_pool(seed):
    rng = random.Random(seed)
    specs = [(rng.randint(1, 30), rng.randint(1, 25)) for _ in range(12)]
    tight = make(pages=rng.choice([30, 40, 60]), page=rng.choice([2, 4]), slots=rng.choice([2, 3, 5]),
                 budget=rng.choice([7, 16, 40]), max_len=80)
    reqs = [Request([rng.randint(0, 49) for _ in range(p)], max_new=n) for p, n in specs]
    pending = list(reqs)
    # requests arrive while others run
    while pending or not tight.idle():
        for _ in range(rng.randint(0, 2)):
            if pending:
                tight.add(pending.pop(0))
        if tight.idle():
            continue
        planned = tight.plan()
        sampled = [fake_next(p.req.tokens[:p.start + p.count]) for p in planned if p.sample]
        tight.commit(planned, sampled)
        tight.cache.check()
    for r in reqs:
        assert r.output == expected(r.prompt, r.max_new)
    assert tight.cache.free_slots() == tight.cache.max_requests


class FakeDevice:
    """Stands in for the GPU when the host runs a step behind it: per request it keeps the
    tokens that have gone through the "model" and the token its last step sampled (what
    ``last_token[slot]`` holds on the device), which a share with ``fed_on_device`` feeds without
    the host knowing its value."""

    def __init__(self):
        self.seen: dict[int, list[int]] = {}
        self.last: dict[int, int] = {}

    def run(self, planned) -> list[int]:
        sampled = []
        for p in planned:
            r = p.req
            if p.start == 0:
                self.seen[r.rid] = []
            history = self.seen[r.rid]
            assert len(history) == p.start
            if p.fed_on_device:
                assert p.count == 1 and r.inflight == 1
                history.append(self.last[r.rid])
            else:
                assert r.inflight == 0            # every value of the share is known on the host
                history.extend(r.span(p.start, p.count))
            if p.sample:
                self.last[r.rid] = fake_next(history)
                sampled.append(self.last[r.rid])
        return sampled


def drive_async(sched: Scheduler, arrivals=None, depth=1, log=None, limit=10000):
    """``plan -> launch`` with ``deliver`` ``depth`` steps behind, as the engine's loop does with
    captured steps; ``NeedsDrain`` delivers everything in flight first. Returns (steps, drains)."""
    dev, inflight = FakeDevice(), deque()
    arrivals = deque(arrivals or [])
    steps = drains = 0

    def deliver_all():
        while inflight:
            sched.deliver(*inflight.popleft())

    while arrivals or not sched.idle():
        if arrivals:
            sched.add(arrivals.popleft())
        try:
            planned = sched.plan()
        except NeedsDrain:
            assert inflight
            deliver_all()
            drains += 1
            continue
        assert planned
        if log is not None:
            log.append([(p.req.rid, p.start, p.count, p.sample, p.fed_on_device) for p in planned])
        sampled = dev.run(planned)
        sched.launch(planned)
        inflight.append((planned, sampled))
        while len(inflight) > depth:
            sched.deliver(*inflight.popleft())
        sched.cache.check()
        steps += 1
        assert steps < limit
    deliver_all()
    return steps, drains


def test_one_step_behind_gives_the_same_replies_and_no_step_for_a_sampled_out_request():
    """The in-flight protocol without a GPU. A request whose every token is sampled is not
    planned again: a reply of N tokens takes one step for the prompt and N - 1 decode steps, and
    every step after the prompt's is decode-only (planning the finished request once more, for
    the cache entry of its last token, made this count N + 1 and the last step a mixed one)."""
    s = make(budget=64)
    r = Request(list(range(10)), max_new=6)
    s.add(r)
    log = []
    steps, drains = drive_async(s, log=log)
    assert r.output == expected(r.prompt, 6) and r.finish == "length"
    assert steps == 6 and drains == 1            # the drain: nothing to run, the last token in flight
    assert [step[0][1:] for step in log[1:]] == [(10 + i, 1, True, True) for i in range(5)]
    assert s.cache.free_pages() == 199 and s.cache.free_slots() == 8


def test_one_step_behind_sees_a_stop_token_late_and_drops_the_extra_token():
    s = make(budget=64)
    prompt = [3, 1, 4, 1, 5]
    full = expected(prompt, 30)
    stop = full[4]
    want = expected(prompt, 30, stop=(stop,))
    r = Request(prompt, max_new=30, stop=(stop,))
    s.add(r)
    log = []
    steps, _ = drive_async(s, log=log)
    assert r.output == want and r.finish == "stop"
    # the stop token is sampled by step len(want) - 1 (counting from 0) and read one step later:
    # exactly one step more than the synchronous drive takes
    assert steps == len(want) + 1


@pytest.mark.parametrize("seed", range(6))
def test_one_step_behind_random_loads_match_the_synchronous_drive(seed):
    """Random arrivals into a tight pool: preemptions force ``NeedsDrain``, stops are seen late,
    and the replies equal those of the plain drive (and of no scheduling at all)."""
    rng = random.Random(100 + seed)
    specs = [(rng.randint(1, 30), rng.randint(1, 25)) for _ in range(12)]
    stops = tuple(rng.sample(range(50), 3))
    sched = make(pages=rng.choice([30, 40, 60]), page=rng.choice([2, 4]), slots=rng.choice([2, 3, 5]),
                 budget=rng.choice([7, 16, 40]), max_len=80)
    reqs = [Request([rng.randint(0, 49) for _ in range(p)], max_new=n, stop=stops) for p, n in specs]
    drive_async(sched, arrivals=reqs, depth=rng.choice([1, 1, 2]))
    for r in reqs:
        assert r.output == expected(r.prompt, r.max_new, stops), r.rid
        assert r.finish == ("stop" if r.output[-1] in stops else "length")
        assert r.inflight == 0
    assert sched.cache.free_slots() == sched.cache.max_requests
    assert sched.cache.free_pages() == sched.cache.num_pages - 1


def test_decode_attention_split_rule():
    """How many CTAs share a decoded token's keys: about 1,024 keys each; more splits while the GPU
    would stay empty (never below 128 keys a split); never more CTAs than fit in a few waves."""
    from tokenomos_b200.parts.attention import Attention
    from tokenomos_b200.parts.registry import Tuning
    f, t = Attention.decode_splits, Tuning()
    assert f(8, 8, 4096) == 4 and f(64, 8, 4096) == 4 and f(8, 8, 16384) == 16    # 1,024 keys a CTA
    assert f(1, 8, 4096) == 32 and f(1, 8, 100) == 1 and f(8, 8, 1024) == 4       # filling the GPU
    assert f(1, 8, 32768) == 32 and f(64, 8, 32768) == 4                           # the CTA cap
    for rows in (1, 2, 3, 8, 17, 64, 256, 1000):
        for kv in (1, 2, 8):
            prev = 0
            for longest in (1, 64, 128, 129, 500, 2048, 4096, 10 ** 5):
                n = f(rows, kv, longest)
                assert 1 <= n <= max(1, -(-longest // t.decode_min_keys))
                assert n * rows * kv <= t.decode_ctas_per_sm * t.sm_count + rows * kv
                assert n >= prev                    # a longer context never gets fewer splits
                prev = n


def test_one_kernel_decode_attention_split_rule():
    """The one-kernel form's splits: as many as keep every CTA resident at once (two an SM), never
    below 128 keys a split, at least one."""
    from tokenomos_b200.parts.attention import Attention
    from tokenomos_b200.parts.registry import Tuning
    f, t = Attention.fused_splits, Tuning()
    assert f(8, 8, 4096) == 4 and f(8, 8, 32768) == 4 and f(8, 8, 300) == 3
    assert f(1, 8, 4096) == 32 and f(1, 8, 32768) == 37 and f(2, 8, 4096) == 18 and f(4, 8, 4096) == 9
    assert f(8, 32, 4096) == 1 and f(8, 64, 4096) == 1              # more CTAs than fit even unsplit: one each
    for rows in (1, 2, 3, 5, 8):
        for kv in (1, 2, 3, 8):
            for longest in (1, 127, 128, 129, 2048, 10 ** 5):
                n = f(rows, kv, longest)
                assert 1 <= n <= max(1, -(-longest // t.decode_min_keys))
                assert n == 1 or n * rows * kv <= t.decode_fused_ctas_per_sm * t.sm_count
    half = Tuning(sm_count=74)
    assert f(8, 8, 4096, half) == 2


def test_prefill_attention_split_rule():
    """How many CTAs may share one tile's keys in the tcgen05 prefill kernel: as many as fill the
    GPU once, within the scratch memory's budget, 16 at most, one when the step has many tiles."""
    from tokenomos_b200.parts.attention import Attention
    from tokenomos_b200.parts.registry import Tuning
    f = Attention.prefill_splits
    assert f(2048, 64, 32, 8) == 1 and f(8192, 256, 32, 8) == 1          # a step that fills the GPU by itself
    assert f(512, 16, 32, 8) == 2 and f(128, 4, 32, 8) == 9 and f(32, 1, 32, 8) == 16
    assert f(128, 69, 32, 8) == 3                                          # a captured step's long list: the memory budget
    assert f(128, 4, 32, 8, Tuning(prefill_split_ctas_per_sm=0)) == 1      # switched off
    for tokens in (1, 2, 31, 32, 33, 500, 5000):
        for entries in (1, 5, 70, 300):
            for kv in (1, 2, 8):
                n = f(tokens, entries, 32, kv)
                assert 1 <= n <= 16
                assert n == 1 or entries * kv * n * 128 * 66 * 4 <= 64 << 20
