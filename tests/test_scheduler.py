"""The scheduler's decisions (no GPU): admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out. A fake step stands in for the
model: the next token is a function of the whole history, so any scheduling must give the same
replies."""

from __future__ import annotations

import random

import pytest
import torch

from tokenomos_b200.cache.manager import CacheManager
from tokenomos_b200.engine.scheduler import Request, Scheduler
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


def test_decode_attention_split_rule():
    """How many CTAs share a decoded token's keys: about 1,024 keys each; more splits while the GPU
    would stay empty (never below 128 keys a split); never more CTAs than fit in a few waves."""
    from tokenomos_b200.parts.attention import Attention
    f = Attention.decode_splits
    assert f(8, 8, 4096) == 4 and f(64, 8, 4096) == 4 and f(8, 8, 16384) == 16    # 1,024 keys a CTA
    assert f(1, 8, 4096) == 32 and f(1, 8, 100) == 1 and f(8, 8, 1024) == 4       # filling the GPU
    assert f(1, 8, 32768) == 32 and f(64, 8, 32768) == 4                           # the CTA cap
    for rows in (1, 2, 3, 8, 17, 64, 256, 1000):
        for kv in (1, 2, 8):
            prev = 0
            for longest in (1, 64, 128, 129, 500, 2048, 4096, 10 ** 5):
                n = f(rows, kv, longest)
                assert 1 <= n <= max(1, -(-longest // Attention.DECODE_MIN_KEYS))
                assert n * rows * kv <= Attention.DECODE_CTAS + rows * kv
                assert n >= prev                    # a longer context never gets fewer splits
                prev = n
