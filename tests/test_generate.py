"""Generation through the entry points: greedy replies equal the plain implementation's,
seeded sampling repeats and is the same alone or in a batch, stop tokens end a reply, running
out of pages changes nothing but the speed, the command line prints what the API returns."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_lfm3
from conftest import TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


# How far below the plain implementation's best logit a 16-bit greedy token may lie, per
# configuration: two to four times the worst gap measured on a B200 over 192 generated tokens
# each (A 0.000, B 0.012, C 0.035, D 0.005 nats, with 192, 187, 185 and 190 of the tokens the
# plain implementation's own argmax). The reference holds its engine to 0.15 nats against its
# dense forward (Tokenomos tests/core/test_engine.py:98-102).
MARGIN_BF16 = {"A": 0.02, "B": 0.05, "C": 0.08, "D": 0.04}


def prompts_for(name, lengths, seed=0):
    vocab = TINY[name]["config"]["vocab_size"]
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def teacher_forced_ok(config, w, prompt, reply, margin):
    """Never compare free-running streams across implementations: each generated token must be
    the plain implementation's argmax given the same history, or within ``margin`` of it."""
    logits = plain_lfm3.forward_logits(config, w, prompt + reply)
    for i, tok in enumerate(reply):
        row = logits[len(prompt) + i - 1]
        if int(row.argmax()) != tok:
            assert row.max().item() - row[tok].item() <= margin, (i, tok, int(row.argmax()))


@pytest.mark.parametrize("work", ["fp32", "bf16"])
@pytest.mark.parametrize("name, lengths, steps", [("A", [5, 17, 33], 16), ("B", [1, 9, 40, 64], 24)])
def test_greedy_generation_through_llm(name, lengths, steps, work, model_folders):
    margin = 1e-4 if work == "fp32" else MARGIN_BF16[name]
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders[name][torch.bfloat16]
    config, w = plain_lfm3.read_folder(folder)
    prompts = prompts_for(name, lengths)
    with LLM(str(folder), work=work, page=TINY[name]["page"], max_len=256, slots=4, pages=40,
             prefill_budget=48, poison=True) as llm:
        outs = llm.generate(prompts, SamplingParams(max_tokens=steps))
    for prompt, out in zip(prompts, outs):
        assert out.prompt_tokens == len(prompt) and out.finish == "length"
        assert len(out.token_ids) == steps
        teacher_forced_ok(config, w, prompt, out.token_ids, margin)
        if work == "fp32":
            assert out.token_ids == plain_lfm3.generate_greedy(config, w, prompt, steps)


@pytest.mark.parametrize("name, work, margin", [("A", "fp32", 1e-4), ("B", "fp32", 1e-4),
                                                ("D", "bf16", MARGIN_BF16["D"]), ("C", "bf16", MARGIN_BF16["C"])])
def test_mixed_steps_through_captured_graphs(name, work, margin, model_folders):
    """Prompt portions beside decoded tokens, replayed from captured steps (fixed-size layouts
    padded with a dummy sequence, empty tiles and unused rows) and queued one step ahead of the
    host: the same tokens as the eager steps, and the plain implementation's."""
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders[name][torch.bfloat16]
    config, w = plain_lfm3.read_folder(folder)
    prompts = prompts_for(name, [37, 5, 64, 18, 51, 9, 70, 26], seed=4)
    kw = dict(work=work, page=TINY[name]["page"], max_len=128, slots=5, pages=60, prefill_budget=24,
              poison=True)
    p = SamplingParams(max_tokens=20)
    with LLM(str(folder), graphs=False, **kw) as llm:
        eager = llm.generate(prompts, p)
    with LLM(str(folder), graphs=True, **kw) as llm:
        llm.engine.step_fn.capture_after = 0
        graphed = llm.generate(prompts, p)
        again = llm.generate(prompts, p)
        assert llm.engine.stats.graph_steps > 10
        llm.engine.cache.check()
    for prompt, a, b, c in zip(prompts, eager, graphed, again):
        assert b.token_ids == c.token_ids
        teacher_forced_ok(config, w, prompt, b.token_ids, margin)
        if work == "fp32":
            assert a.token_ids == b.token_ids


def test_mixed_step_whose_bucket_has_as_many_tokens_as_sequences(model_folders):
    """Forty requests, most of them decoding beside one prompt portion: such a step falls into the
    captured bucket of 64 tokens and 64 sequences, whose layout has as many tokens as sequences
    without being one token per sequence. The parts must not take it for a decode step."""
    from tokenomos_b200 import LLM, SamplingParams
    name = "D"                   # head size 64: the tensor-core attention kernels, the fused conv
    folder = model_folders[name][torch.bfloat16]
    config, w = plain_lfm3.read_folder(folder)
    prompts = prompts_for(name, [3 + (i * 7) % 11 for i in range(39)] + [50], seed=9)
    kw = dict(work="bf16", page=TINY[name]["page"], max_len=96, slots=40, pages=200, prefill_budget=58,
              poison=True)
    p = SamplingParams(max_tokens=12)
    with LLM(str(folder), graphs=True, **kw) as llm:
        llm.engine.step_fn.capture_after = 0
        outs = llm.generate(prompts, p)
        shapes = set(llm.engine.step_fn._step_graphs)
        llm.engine.cache.check()
    assert (64, 64) in shapes, shapes
    for prompt, o in zip(prompts, outs):
        teacher_forced_ok(config, w, prompt, o.token_ids, MARGIN_BF16[name])


def test_warmup_records_every_step_shape_before_the_first_request(model_folders):
    """``warmup=True``: the decode step of every batch bucket up to ``slots`` and the mixed step
    of every (token, sequence) bucket under the budget are captured before serving (the
    reference warms its engine up the same way and tests it, Tokenomos
    tests/core/test_engine.py:172-194); serving then records nothing more and gives the tokens
    of an engine that captured as it went."""
    from tokenomos_b200 import LLM, SamplingParams
    name = "D"
    folder = model_folders[name][torch.bfloat16]
    prompts = prompts_for(name, [37, 5, 64, 18, 51, 9, 70, 26], seed=4)
    kw = dict(work="fp32", page=TINY[name]["page"], max_len=128, slots=5, pages=60, prefill_budget=24)
    p = SamplingParams(max_tokens=12)
    with LLM(str(folder), graphs=True, **kw) as llm:
        llm.engine.step_fn.capture_after = 0
        lazy = llm.generate(prompts, p)
    with LLM(str(folder), graphs=True, warmup=True, **kw) as llm:
        step_fn = llm.engine.step_fn
        decode, mixed = set(step_fn._graphs), set(step_fn._step_graphs)
        assert decode == {1, 2, 4, 5}                          # buckets up to the 5 slots
        assert mixed == {(32, 4), (32, 16)}                    # 24 tokens at most, 5 + 1 sequences
        assert llm.engine.stats.steps == 0
        # the runs that warm a shape up work on an empty layout; what the sampler made of their
        # logits must not be held against the first real step
        from tokenomos_b200 import ops
        assert ops.sample_status() == 0
        warm = llm.generate(prompts, p)
        assert set(step_fn._graphs) == decode and set(step_fn._step_graphs) == mixed
        assert llm.engine.stats.graph_steps > 0
    assert [o.token_ids for o in warm] == [o.token_ids for o in lazy]


def test_trace_records_say_what_every_step_was(model_folders):
    """``trace_on`` / ``trace_take``: one record per step with its kind, rows, tokens, the captured
    bucket it replayed, host milliseconds to plan and launch it and device milliseconds from two
    CUDA events; nothing is recorded before ``trace_on``, and the records account for every
    token the steps ran."""
    from tokenomos_b200 import LLM, SamplingParams
    name = "D"
    folder = model_folders[name][torch.bfloat16]
    prompts = prompts_for(name, [37, 5, 64, 18], seed=4)
    kw = dict(work="bf16", page=TINY[name]["page"], max_len=128, slots=4, pages=40, prefill_budget=24)
    with LLM(str(folder), graphs=True, warmup=True, **kw) as llm:
        llm.generate(prompts[:1], SamplingParams(max_tokens=3))
        assert llm.engine.trace_take() == []
        llm.engine.trace_on()
        before = llm.engine.stats.steps
        outs = llm.generate(prompts, SamplingParams(max_tokens=8))
        records = llm.engine.trace_take()
        assert len(records) == llm.engine.stats.steps - before
        assert llm.engine.trace_take() == []
    kinds = {r["kind"] for r in records}
    assert "decode" in kinds and "mixed" in kinds
    for r in records:
        assert set(r) >= {"step", "kind", "rows", "tokens", "bucket", "captured", "plan_ms", "launch_ms",
                          "wait_ms", "gpu_ms"}
        assert r["gpu_ms"] > 0 and r["plan_ms"] >= 0 and r["rows"] <= r["tokens"]
        if r["kind"] == "decode":
            assert r["captured"] and r["rows"] == r["tokens"] <= r["bucket"]
        if r["kind"] == "mixed":
            assert r["captured"] and r["tokens"] <= r["bucket"][0] and r["rows"] <= r["bucket"][1]
    # every prompt token and every generated token but each reply's last went through a step
    ran = sum(r["tokens"] for r in records)
    assert ran == sum(len(p) for p in prompts) + sum(len(o.token_ids) - 1 for o in outs)


def test_seeded_sampling_repeats_alone_and_in_batches(model_folders):
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders["B"][torch.bfloat16]
    prompts = prompts_for("B", [1, 9, 40, 64], seed=1)
    p = SamplingParams(max_tokens=24, temperature=0.8, seed=1234)
    with LLM(str(folder), work="fp32", page=8, max_len=128, slots=4, pages=60) as llm:
        batch = llm.generate(prompts, p)
        again = llm.generate(prompts, p)
        alone = [llm.generate([x], p)[0] for x in prompts]
        other = llm.generate(prompts, SamplingParams(max_tokens=24, temperature=0.8, seed=99))
    assert [o.token_ids for o in batch] == [o.token_ids for o in again]
    assert [o.token_ids for o in batch] == [o.token_ids for o in alone]
    assert [o.token_ids for o in batch] != [o.token_ids for o in other]
    greedy_like = sum(o.token_ids == batch[0].token_ids for o in batch)
    assert greedy_like == 1


def test_stop_token_and_refusals(model_folders):
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders["A"][torch.bfloat16]
    prompt = prompts_for("A", [12])[0]
    with LLM(str(folder), work="fp32", page=16, max_len=64, slots=2, pages=6) as llm:
        free = llm.generate([prompt], SamplingParams(max_tokens=12))[0]
        stop = free.token_ids[5]
        cut = llm.generate([prompt], SamplingParams(max_tokens=12, stop_token_ids=(stop,)))[0]
        first = free.token_ids.index(stop)
        assert cut.finish == "stop" and cut.token_ids == free.token_ids[:first + 1]
        with pytest.raises(ValueError, match="longest sequence"):
            llm.generate([prompt], SamplingParams(max_tokens=60))
        with pytest.raises(ValueError, match="token id"):
            llm.generate([[10 ** 6]], SamplingParams(max_tokens=2))
        with pytest.raises(ValueError, match="tokenizer.json"):
            llm.generate(["text"], SamplingParams(max_tokens=2))
        # the engine still serves after refusals
        assert llm.generate([prompt], SamplingParams(max_tokens=12))[0].token_ids == free.token_ids


def test_pages_run_out_same_tokens_as_a_roomy_pool(model_folders):
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders["A"][torch.bfloat16]
    prompts = prompts_for("A", [20, 31, 9, 27, 14, 22], seed=3)
    p = SamplingParams(max_tokens=30, temperature=0.7, seed=5)
    with LLM(str(folder), work="fp32", page=16, max_len=64, slots=6, pages=40) as llm:
        roomy = llm.generate(prompts, p)
        assert llm.engine.stats.preemptions == 0
    # 8 usable pages of 16 tokens: the six requests cannot all stay resident
    with LLM(str(folder), work="fp32", page=16, max_len=64, slots=6, pages=9, poison=True) as llm:
        tight = llm.generate(prompts, p)
        assert llm.engine.stats.preemptions > 0
        llm.engine.cache.check()
        assert llm.engine.cache.free_pages() == 8
    assert [o.token_ids for o in tight] == [o.token_ids for o in roomy]


@pytest.mark.parametrize("graphs", [True, False])
def test_pages_run_out_in_bfloat16_with_captured_mixed_steps(graphs, model_folders):
    """Preemption and recomputation on the 16-bit kernels (head size 64: the tensor-core
    attention, the fused conv), with mixed steps captured and in flight when the pool runs dry.
    A recomputed request sees its earlier tokens through other kernels (a prompt portion instead
    of single tokens), so in 16 bits the replies are held to the plain implementation by teacher
    forcing, not to the roomy pool's stream."""
    from tokenomos_b200 import LLM, SamplingParams
    name = "D"
    folder = model_folders[name][torch.bfloat16]
    config, w = plain_lfm3.read_folder(folder)
    prompts = prompts_for(name, [20, 31, 9, 27, 14, 22], seed=3)
    p = SamplingParams(max_tokens=30)
    # 8 usable pages of 16 tokens: the six requests cannot all stay resident
    with LLM(str(folder), work="bf16", page=16, max_len=64, slots=6, pages=9, prefill_budget=40,
             graphs=graphs, poison=True) as llm:
        llm.engine.step_fn.capture_after = 0
        tight = llm.generate(prompts, p)
        assert llm.engine.stats.preemptions > 0
        assert llm.engine.stats.graph_steps > 0 or not graphs
        llm.engine.cache.check()
        assert llm.engine.cache.free_pages() == 8
    for prompt, o in zip(prompts, tight):
        assert len(o.token_ids) == 30
        teacher_forced_ok(config, w, prompt, o.token_ids, MARGIN_BF16[name])


def test_a_kernel_that_gave_up_on_a_barrier_fails_the_waiting_caller(model_folders, monkeypatch):
    """The tcgen05 kernels bound their waits and leave a word where they gave up; the engine
    reads it before it hands out the last replies of a batch. The word is made on the host here
    (no kernel is made to wait): the status call is replaced by one that reports place 2."""
    from tokenomos_b200 import LLM, SamplingParams, ops
    folder = model_folders["A"][torch.bfloat16]
    with LLM(str(folder), work="bf16", page=16, max_len=64, slots=2, pages=6) as llm:
        ok = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=3))
        assert len(ok[0].token_ids) == 3 and llm.failure is None
        monkeypatch.setattr(ops, "gemm_tc_status", lambda: 2)
        # a ticket that such a kernel left drawn must not reach the next launch
        drawn = ops._decode_tickets(8, torch.device("cuda", torch.cuda.current_device()))
        drawn[3] = 1
        with pytest.raises(RuntimeError, match="engine thread failed") as err:
            llm.generate([[1, 2, 3]], SamplingParams(max_tokens=3))
        assert "gave up waiting on a barrier (place 2)" in str(err.value.__cause__)
        assert isinstance(llm.failure, RuntimeError)
        assert int(drawn.abs().sum()) == 0


@pytest.mark.filterwarnings("ignore::pytest.PytestUnhandledThreadExceptionWarning")
def test_engine_thread_failure_surfaces(model_folders):
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders["A"][torch.bfloat16]
    with LLM(str(folder), work="fp32", page=16, max_len=64, slots=2, pages=6) as llm:
        def boom(*a, **k):
            raise RuntimeError("injected")
        llm.engine.step = boom
        with pytest.raises(RuntimeError, match="engine thread failed"):
            llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2))
        assert isinstance(llm.failure, RuntimeError)


def test_command_line(model_folders, tmp_path):
    from tokenomos_b200 import LLM, SamplingParams
    folder = model_folders["A"][torch.bfloat16]
    cmd = [sys.executable, "-m", "tokenomos_b200.generate", "--model", str(folder),
           "--prompt-ids", "1,2,3,4", "--prompt-ids", "9,8", "--max-tokens", "6",
           "--arch-kw", '{"work": "fp32"}', "--engine-kw", '{"page": 16, "max_len": 64, "slots": 2, "pages": 8}']
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    with LLM(str(folder), work="fp32", page=16, max_len=64, slots=2, pages=8) as llm:
        want = llm.generate([[1, 2, 3, 4], [9, 8]], SamplingParams(max_tokens=6))
    assert [ln["token_ids"] for ln in lines] == [o.token_ids for o in want]
    assert [ln["prompt_tokens"] for ln in lines] == [4, 2]
