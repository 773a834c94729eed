"""Trace replay against the plain implementation, in 32-bit and in bfloat16: each request alone
and whole; most of it in one step and the last 32 tokens one by one; portions of changing size
down to two tokens; mixed, up to four live requests, with so few pages that they are used
again; long decoding; the first tokens of a sequence. The logits at a position must not depend
on how the tokens were cut, on what else was in the batch, or on which pages held them."""

from __future__ import annotations

import pytest
import torch

import plain_lfm3
import trace_util
from conftest import TINY

pytestmark = pytest.mark.gpu

# Tolerances, relative to the largest |logit| of the request. 32-bit: accumulation order only.
# bfloat16: the 16-bit path rounds activations after every kernel; measured errors against the
# float64 oracle are 0.3 % (A) to 2.4 % (C) of the scale, so 4 % is a real bound, and two
# bfloat16 runs that only differ in cutting must agree far closer than either does with the oracle.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
TOL_SAME_DTYPE = {"float32": 1e-5, "bfloat16": 2e-2}

LENGTHS = {"A": [5, 17, 33, 70, 96, 41], "B": [1, 9, 40, 64, 130, 57], "C": [3, 26, 75, 50, 110, 38],
           "D": [2, 31, 150, 65, 200, 90]}


def requests_for(name: str) -> dict[str, list[int]]:
    vocab = TINY[name]["config"]["vocab_size"]
    g = torch.Generator().manual_seed(1234 + ord(name))
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist()
            for i, n in enumerate(LENGTHS[name])}


_oracle_cache: dict = {}


def oracle(name: str, folder, requests) -> dict[str, torch.Tensor]:
    if name not in _oracle_cache:
        config, w = plain_lfm3.read_folder(folder)
        _oracle_cache[name] = {rid: plain_lfm3.forward_logits(config, w, ids)
                               for rid, ids in requests.items()}
    return _oracle_cache[name]


def compare(got: dict, want: dict, tol: float, what: str):
    for rid, ref in want.items():
        assert rid in got, (what, rid)
        assert got[rid].shape == ref.shape, (what, rid, got[rid].shape, ref.shape)
        assert torch.isfinite(got[rid]).all(), (what, rid)
        if ref.numel() == 0:
            continue
        err = (got[rid] - ref).abs().amax(dim=1)
        scale = ref.abs().max().item()
        bad = (err > tol * scale).nonzero()
        assert bad.numel() == 0, (f"{what}: request {rid}: first wrong position {int(bad[0])} of "
                                  f"{len(err)}: error {err[int(bad[0])].item():.3e}, "
                                  f"allowed {tol * scale:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_way_of_cutting(name, dtype, model_folders):
    folder = model_folders[name][torch.bfloat16]
    page = TINY[name]["page"]
    reqs = requests_for(name)
    want = oracle(name, folder, reqs)
    results = {}
    for mode, steps in (("whole", trace_util.whole(reqs)),
                        ("tail", trace_util.tail_decoded(reqs, 32)),
                        ("portions", trace_util.portions(reqs)),
                        ("mixed", trace_util.mixed(reqs, live=4, seed=ord(name)))):
        # the pool holds exactly what the trace's live requests need, so pages are used again
        max_tokens = trace_util.max_live_tokens(steps, 64)
        per_step = trace_util.run_in_process(folder, dtype, steps, max_tokens, page)
        got = trace_util.collect(steps, per_step)
        compare(got, want, TOL[dtype], f"{name} {dtype} {mode}")
        results[mode] = got
    for mode in ("tail", "portions", "mixed"):
        compare(results[mode], results["whole"], TOL_SAME_DTYPE[dtype], f"{name} {dtype} {mode} vs whole")


def test_mixed_trace_really_mixes_and_reuses(model_folders):
    """The mixed trace is what it claims: portions beside single tokens, requests left out,
    at most four live, and a pool too small to hold every request at once."""
    reqs = requests_for("B")
    steps = trace_util.mixed(reqs, live=4, seed=ord("B"))
    assert any(len(s["entries"]) > 1 and {len(e["tokens"]) == 1 for e in s["entries"]} == {True, False}
               for s in steps)
    live, worst = set(), 0
    for s in steps:
        live |= {e["id"] for e in s["entries"]}
        worst = max(worst, len(live))
        live -= set(s["end"])
    assert worst == 4
    assert trace_util.max_live_tokens(steps, 64) < sum(-(-len(v) // 64) * 64 for v in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype, model_folders):
    """One token prompts, two token prompts, and 300 tokens decoded one by one across many
    pages and far past the window."""
    name = "C"
    folder = model_folders[name][torch.bfloat16]
    vocab = TINY[name]["config"]["vocab_size"]
    g = torch.Generator().manual_seed(99)
    reqs = {"one": torch.randint(0, vocab, (1,), generator=g).tolist(),
            "two": torch.randint(0, vocab, (2,), generator=g).tolist(),
            "long": torch.randint(0, vocab, (300,), generator=g).tolist()}
    config, w = plain_lfm3.read_folder(folder)
    want = {rid: plain_lfm3.forward_logits(config, w, ids) for rid, ids in reqs.items()}
    steps = trace_util.tail_decoded(reqs, tail=298)
    per_step = trace_util.run_in_process(folder, dtype, steps, trace_util.max_live_tokens(steps),
                                         TINY[name]["page"])
    compare(trace_util.collect(steps, per_step), want, TOL[dtype], f"long decoding {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, model_folders, tmp_path):
    """The program itself, as a user runs it: stdin, ``done`` lines, logits files."""
    name = "B"
    folder = model_folders[name][torch.bfloat16]
    reqs = requests_for(name)
    want = oracle(name, folder, reqs)
    steps = trace_util.mixed(reqs, live=3, seed=5)
    # a step that wants nothing writes no file
    steps[0]["entries"][0]["want"] = []
    got_steps = trace_util.run_program(folder, dtype, steps, trace_util.max_live_tokens(steps),
                                       tmp_path / "out", TINY[name]["config"]["vocab_size"])
    rows = trace_util.collect(steps, got_steps)
    first = steps[0]["entries"][0]
    trimmed = dict(want)
    trimmed[first["id"]] = want[first["id"]][len(first["tokens"]):]
    compare(rows, trimmed, TOL[dtype], f"trace_run {dtype}")
