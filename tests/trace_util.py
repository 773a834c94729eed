"""Builds replay traces (the JSON steps ``bin/trace_run`` reads) and runs them, either in this
process through the framework's step function or through the ``bin/trace_run`` program."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one after the other; every position wanted."""
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [rid]})
    return steps


def tail_decoded(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        cut = max(1, len(ids) - tail)
        cuts = [0, cut] + list(range(cut + 1, len(ids) + 1))
        for a, b in zip(cuts[:-1], cuts[1:]):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": ids[a:b], "want": list(range(b - a))}],
                "end": [rid] if b == len(ids) else []})
    return steps


def portions(requests: dict[str, list[int]], sizes=(7, 2, 19, 3, 2, 31, 5, 2, 64, 11)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, ids in requests.items():
        a, k = 0, 0
        while a < len(ids):
            b = min(len(ids), a + sizes[k % len(sizes)])
            if len(ids) - b == 1:        # never leave a lone last token: portions have >= 2
                b = len(ids)
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": ids[a:b], "want": list(range(b - a))}],
                "end": [rid] if b == len(ids) else []})
            a, k = b, k + 1
    return steps


def mixed(requests: dict[str, list[int]], live: int = 4, seed: int = 0, decode_tail: int = 12,
          sizes=(9, 2, 23, 4, 16, 2, 40)) -> list[dict]:
    """Up to ``live`` requests at a time: portions of some beside single (decoded) tokens of
    others; a request is sometimes left out of a step; finished requests end and the next one
    starts, so pages and slots are used again."""
    import random

    rng = random.Random(seed)
    waiting = list(requests.items())
    active: dict[str, int] = {}
    steps = []
    while waiting or active:
        while waiting and len(active) < live:
            rid, _ = waiting.pop(0)
            active[rid] = 0
        entries, ended = [], []
        for rid in list(active):
            ids, done = requests[rid], active[rid]
            if len(active) > 1 and rng.random() < 0.2:
                continue                                   # sits this step out
            left = len(ids) - done
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.choice(sizes), left - decode_tail)
                n = max(n, min(2, left))
            entries.append({"id": rid, "tokens": ids[done:done + n], "want": list(range(n))})
            active[rid] = done + n
            if active[rid] == len(ids):
                ended.append(rid)
                del active[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def max_live_tokens(steps: list[dict], page: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of ``page``."""
    held: dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // page) * page for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def collect(steps: list[dict], per_step: dict[int, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Per request, the logits rows in position order (every position was wanted once)."""
    rows: dict[str, list] = {}
    for s in steps:
        if not any(e["want"] for e in s["entries"]):
            continue
        block, o = per_step[s["step"]], 0
        for e in s["entries"]:
            n = len(e["want"])
            rows.setdefault(e["id"], []).append(block[o:o + n])
            o += n
        assert o == block.shape[0]
    return {rid: torch.cat(parts) for rid, parts in rows.items()}


def run_in_process(folder, dtype: str, steps: list[dict], max_tokens: int, page: int,
                   max_requests: int = 8, poison: bool = True) -> dict[int, torch.Tensor]:
    """Drive the framework's own loader, cache manager and step function with the trace."""
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    conf = models.configure(folder, work=dtype)
    model = models.load(folder, "cuda", conf)
    pages = -(-max_tokens // page) + 1
    # every page and state row that no request holds is full of NaN: a read past a request's
    # own positions, or of a state row the request before left, shows in the logits
    cache = CacheManager(model.state_specs(), page, pages, max_requests, conf.work, "cuda",
                         max_len=max(max_tokens, page), poison=poison)
    step_fn = StepFunction(model, cache)
    out = {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in cache.requests:
                cache.admit(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = step_fn.run(entries)
        if logits is not None:
            out[s["step"]] = logits.double().cpu()
        for rid in s["end"]:
            cache.release(rid)
        cache.check()
    assert not cache.requests
    return out


def run_program(folder, dtype: str, steps: list[dict], max_tokens: int, out_dir: Path, vocab: int,
                page: int | None = None) -> dict[int, torch.Tensor]:
    """Run ``bin/trace_run`` as a user would: steps on stdin, ``done`` lines on stdout, files."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    if page is not None:
        cmd += ["--page-size", str(page)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    done = [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps], proc.stdout[-2000:]
    out = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if wanted:
            arr = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            out[s["step"]] = torch.from_numpy(arr.astype(np.float64))
        else:
            assert not path.exists()
    return out
