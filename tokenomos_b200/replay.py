"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing and has no forward pass, cache or loader of its own: it drives the model
registry, the weight loader, the cache manager and the step function that generation uses.
Steps come on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch. For a step in which something is wanted the logits at the
wanted places are written to ``<out>/<step>.f32`` as little-endian float32 ``[wanted, vocab]``,
in the order of the entries and of ``want``. After every step a line ``done <step>`` is printed
and flushed. ``end`` names requests that are finished after the step: their pages and slot go
back to the pools and are used again. ``--max-tokens`` sizes the page pool (each request's
tokens rounded up to whole pages).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files go to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (sizes the page pool)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-requests", type=int, default=8, help="live requests (state slots)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import numpy as np
    import torch

    from tokenomos_b200 import models, ops
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    torch.cuda.set_device(args.device)
    ops.available()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    conf = models.configure(args.model, work=args.dtype)
    model = models.load(args.model, args.device, conf)
    page = args.page_size
    pages = -(-args.max_tokens // page) + 1          # + the null page
    cache = CacheManager(model.state_specs(), page, pages, args.max_requests, conf.work,
                         args.device, max_len=max(args.max_tokens, page))
    step_fn = StepFunction(model, cache)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        entries = []
        for e in obj.get("entries", []):
            rid = e["id"]
            if rid not in cache.requests:
                cache.admit(rid)
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        if entries:
            logits = step_fn.run(entries)
            if logits is not None:
                arr = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                arr.tofile(out / f"{obj['step']}.f32")
        for rid in obj.get("end", []):
            if rid in cache.requests:
                cache.release(rid)
        print(f"done {obj['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
