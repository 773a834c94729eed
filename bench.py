"""Decode and prefill throughput of the LFM3 1.2B-size configuration on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers 16]

A step is one decode step: every live request brings one token, the engine's captured step
(embedding to sampled token) runs once. ``value`` is decoded tokens per second at ``--batch``
requests whose prompts of 2,048 random tokens were prefilled first; it is timed on the device
with CUDA events around exactly K steps after W warm-up steps (each step's layout is packed and
uploaded by the host and its tokens are read back, one step behind the device as in serving). ``e2e`` is the same rate through
``LLM.generate`` (host token ids in, host token ids out; every step uploads its layout from
pinned memory and reads its tokens back). The line also carries the prefill of one 2,048-token
prompt, the decode step's HBM roofline, and decode rates at batch 1 and 64. Weights are random
(N(0, 0.02), bfloat16), token ids synthetic; there is no dataset or checkpoint behind it.
Method after the reference's own decode bench (Tokenomos bench/decode.py:90-118,154-177:
random prompts, greedy, steady-state step time; prefill of 2,048-token prompts).
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: the 1.2B-size LFM3 configuration
CONFIG_1P2B = {
    "architectures": ["Lfm3ForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 16,
    "layer_types": ["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv",
                    "conv", "full_attention", "conv", "full_attention", "conv", "full_attention",
                    "conv", "full_attention", "conv"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 8192, "vocab_size": 65536, "rope_theta": 1000000.0, "norm_eps": 1e-5,
    "conv_L_cache": 3, "conv_bias": False, "tie_embedding": True,
    # what the reference's declaration reads beside the keys above (Tokenomos
    # models/lfm3/arch.py:61-67,98; models/load/checkpoint.py:160-165): the rotary parameters per
    # attention kind, the tying flag under its other name, and a per-head output gate, whose
    # 32 x 2048 matrix per attention layer is under 0.1 % of a step's bytes. Both arms run this
    # one folder.
    "rope_parameters": {"full_attention": {"rope_type": "default", "rope_theta": 1000000.0}},
    "tie_word_embeddings": True, "attention_gate": True,
}
PROMPT = 2048
CONTEXT = 4096
# the far end of "decode to 4,096": prompts this long, decoded until the context is full
PROMPT_FAR = 3584
# device time the timed blocks of a decode measurement cover at least
MIN_TIMED_MS = 200.0

# BASELINE.json configs[3] and configs[4]: serving workloads on the 350M- and 2.6B-size models
ATTN_AT_16 = (2, 5, 8, 10, 12, 14)
ATTN_AT_30 = (2, 6, 10, 14, 18, 21, 24, 27)
WORKLOADS = {
    "mixed350m": dict(
        config={**CONFIG_1P2B, "hidden_size": 1024, "num_attention_heads": 16, "intermediate_size": 4608,
                "layer_types": ["full_attention" if i in ATTN_AT_16 else "conv" for i in range(16)]},
        requests=256, prompt=(64, 2048), new_tokens=256, max_len=4096, slots=256, budget=2048),
    "chunked2p6b": dict(
        config={**CONFIG_1P2B, "num_hidden_layers": 30, "intermediate_size": 10752,
                "layer_types": ["full_attention" if i in ATTN_AT_30 else "conv" for i in range(30)]},
        requests=64, prompt=(4096, 4096), new_tokens=64, max_len=8192, slots=64, budget=512),
}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Clocks:
    """Samples nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
        mhz = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": float(self.samples[0][1]) if self.samples else None,
                "reasons": reasons, "samples": len(self.samples)}


def lfm3_tensor_shapes(config: dict) -> list[tuple[str, tuple, bool]]:
    """(name, shape, is a norm weight) of every tensor of an LFM3 text folder, from the
    config.json keys alone (names as Tokenomos models/lfm3/arch.py:76-126). Stated here, apart
    from either engine's declaration, because both arms of the bench load the folder it makes:
    each arm's loader then checks the list against its own."""
    d, H, Hkv = config["hidden_size"], config["num_attention_heads"], config["num_key_value_heads"]
    D = config.get("head_dim", d // H)
    I, V, W = config["intermediate_size"], config["vocab_size"], config["conv_L_cache"]
    out = [("model.embed_tokens.weight", (V, d), False)]
    for i, kind in enumerate(config["layer_types"]):
        p = f"model.layers.{i}."
        if kind == "conv":
            out += [(p + "conv.in_proj.weight", (3 * d, d), False), (p + "conv.out_proj.weight", (d, d), False),
                    (p + "conv.conv.weight", (d, 1, W), False)]
            if config.get("conv_bias"):
                out.append((p + "conv.conv.bias", (d,), False))
        else:
            a = p + "self_attn."
            out += [(a + "q_proj.weight", (H * D, d), False), (a + "k_proj.weight", (Hkv * D, d), False),
                    (a + "v_proj.weight", (Hkv * D, d), False), (a + "o_proj.weight", (d, H * D), False),
                    (a + "q_norm.weight", (D,), True), (a + "k_norm.weight", (D,), True)]
            if config.get("attention_gate"):
                out.append((a + "gate_proj.weight", (H, d), False))
        out += [(p + "feed_forward.w1.weight", (I, d), False), (p + "feed_forward.w3.weight", (I, d), False),
                (p + "feed_forward.w2.weight", (d, I), False), (p + "operator_norm.weight", (d,), True),
                (p + "ffn_norm.weight", (d,), True)]
    out.append(("model.embedding_norm.weight", (d,), True))
    if not config.get("tie_word_embeddings", config.get("tie_embedding", True)):
        out.append(("lm_head.weight", (V, d), False))
    return out


def write_folder(folder: Path, layers: int, config: dict | None = None) -> dict:
    """The configuration's model folder with random weights drawn on the GPU: matrices, the
    embedding and conv taps N(0, 0.02), norm weights 1, bfloat16, seed 0 (a CPU draw of 1.2 G
    values takes far longer). Imports neither engine."""
    import torch
    from safetensors.torch import save_file

    config = dict(config or CONFIG_1P2B)
    config["layer_types"] = config["layer_types"][:layers]
    config["num_hidden_layers"] = len(config["layer_types"])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    tensors = {}
    for name, shape, is_norm in lfm3_tensor_shapes(config):
        if is_norm:
            tensors[name] = torch.ones(shape, dtype=torch.bfloat16)
        else:
            t = torch.randn(shape, generator=gen, dtype=torch.float32, device="cuda") * 0.02
            tensors[name] = t.to(torch.bfloat16).cpu()
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file(tensors, str(folder / "model.safetensors"))
    return config


def weight_bytes(model, cfg) -> int:
    """Bytes of weights a decode step reads once: every layer's matrices and vectors, the final
    norm, and the head (the tied embedding matrix is read whole by the head)."""
    total = 0
    seen = set()

    def add(t):
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            return t.numel() * t.element_size()
        return 0

    for block in model.blocks:
        for part in (block.mixer, block.ffn):
            for v in vars(part).values():
                if hasattr(v, "weight") and hasattr(v.weight, "numel"):
                    total += add(v.weight)
                elif hasattr(v, "numel"):
                    total += add(v)
    total += add(model.head.weight)
    return total


def kv_bytes_per_token(cfg) -> int:
    n_attn = len(cfg.attention_layers())
    return n_attn * 2 * cfg.num_key_value_heads * cfg.head_dim * 2


def make_engine(model, batch: int, page: int, prompt: int = PROMPT, context: int = CONTEXT):
    from tokenomos_b200.engine.engine import Engine
    pages = batch * (context // page) + 2
    return Engine(model, slots=batch, page=page, max_len=context, pages=pages, prefill_budget=prompt,
                  graphs=True)


def device_decode(model, cfg, batch: int, steps: int, warmup: int, page: int, seed: int = 0,
                  prompt: int = PROMPT, context: int = CONTEXT) -> dict:
    """K decode steps timed on the device: prefill ``batch`` prompts, then replay the captured
    decode step with the layout advanced on the host each step (the same work ``LLM.generate``
    does, minus the scheduler)."""
    import torch

    from tokenomos_b200.engine.step import StepEntry
    from tokenomos_b200.ops import _lib

    eng = make_engine(model, batch, page, prompt, context)
    step_fn, cache = eng.step_fn, eng.cache
    g = torch.Generator().manual_seed(seed)
    last = []
    for r in range(batch):
        ids = torch.randint(0, cfg.vocab_size, (prompt,), generator=g).tolist()
        cache.admit(r)
        step_fn.run([StepEntry(r, ids, [])])
        last.append(int(ids[-1]))
    rows = [(0.0, 1.0, 0, 0.0, 0, 0)] * batch
    pending = []

    def one(first=False):
        # queue a step before the one before it has been read: its tokens are fed on the device
        entries = [StepEntry(r, [last[r]] if first else [0], []) for r in range(batch)]
        pending.append(step_fn.launch_decode_graph(entries, rows, [not first] * batch, commit=True))
        while len(pending) > 1:
            pending.pop(0).tokens()

    one(first=True)
    for _ in range(warmup - 1):
        one()
    torch.cuda.synchronize()
    ctx_start = cache.length(0)
    calls0 = _lib.calls()
    # blocks of exactly K steps, each between two CUDA events with a synchronize on both sides;
    # the block is repeated until MIN_TIMED_MS of device time are covered (three blocks at
    # least, as long as the context has room) and the median block is the result
    blocks = []
    room = context - ctx_start - 2
    while True:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one()
        end.record()
        torch.cuda.synchronize()
        blocks.append(start.elapsed_time(end))
        room -= steps
        if room < steps or len(blocks) >= 64 or (len(blocks) >= 3 and sum(blocks) >= MIN_TIMED_MS):
            break
    while pending:
        pending.pop(0).tokens()
    ms = statistics.median(blocks) / steps
    graph = step_fn.decode_graph(batch)
    out = {"ms_per_step": ms, "tok_s": batch / ms * 1e3, "ctx_start": ctx_start,
           "ctx_end": cache.length(0), "launches_per_step": graph.launches,
           "host_calls": _lib.calls() - calls0, "blocks": len(blocks),
           "timed_ms": sum(blocks)}
    for r in range(batch):
        cache.release(r)
    del eng
    torch.cuda.empty_cache()
    return out


def device_prefill(model, cfg, page: int, reps: int = 3, tokens: int = PROMPT) -> dict:
    """One prompt of ``tokens`` tokens as one step, timed on the device with CUDA events around
    the step function's call (layout packed and uploaded by the host, embedding to the sampled
    first token), the median of ``reps``: through the captured step of its shape, which is how a
    warmed-up engine runs it, and eagerly (kernel by kernel from the host) beside it."""
    import torch

    from tokenomos_b200.engine.step import StepEntry

    eng = make_engine(model, 1, page, tokens, max(CONTEXT, 2 * tokens))
    step_fn, cache = eng.step_fn, eng.cache
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (tokens,), generator=g).tolist()
    greedy = [(0.0, 1.0, 0, 0.0, 0, 0)]

    def eager(rid):
        step_fn.run([StepEntry(rid, ids, [tokens - 1])])

    def captured(rid):
        entries = [StepEntry(rid, ids, [tokens - 1])]
        graph = step_fn.step_graph_for(entries)
        step_fn.launch_step_graph(graph, entries, greedy, [False]).tokens()
        cache.commit(rid, tokens)

    def timed(fn) -> float:
        times = []
        for i in range(reps + 2):
            cache.admit(i)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            fn(i)
            end.record()
            torch.cuda.synchronize()
            cache.release(i)
            if i >= 2:
                times.append(start.elapsed_time(end))
        return statistics.median(times)

    eager_ms = timed(eager)
    step_fn.capture_after = 0            # as after Engine.warmup(): the shape is captured
    fits = eng.graphs and step_fn.step_graph_for([StepEntry("probe", ids, [tokens - 1])]) is not None
    ms = timed(captured) if fits else eager_ms       # (no captured shape beyond 16,384 tokens)
    flops = prefill_flops(cfg.to_dict(), tokens)
    del eng
    torch.cuda.empty_cache()
    return {"ms": ms, "eager_ms": eager_ms, "tokens": tokens, "tok_s": tokens / ms * 1e3, "flops": flops}


def e2e_decode(llm, cfg, batch: int, steps: int, warmup: int) -> dict:
    """The same decode through the Python entry point: ``LLM.generate`` with host token ids in
    and out; the engine thread schedules, uploads each step's layout from pinned memory and
    reads each step's tokens back."""
    import torch

    from tokenomos_b200.api.llm import SamplingParams

    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (PROMPT,), generator=g).tolist() for _ in range(batch)]
    llm.engine.stats.stamps.clear()
    outs = llm.generate(prompts, SamplingParams(max_tokens=warmup + steps + batch + 1))
    assert all(len(o.token_ids) == warmup + steps + batch + 1 for o in outs)
    stamps = llm.engine.stats.stamps
    decode = [i for i, (_, rows, toks) in enumerate(stamps) if rows == batch and toks == batch]
    first = decode[warmup]
    last = decode[min(warmup + steps, len(decode) - 1)]
    n = last - first
    seconds = stamps[last][0] - stamps[first][0]
    graph = llm.engine.step_fn.decode_graph(batch)
    return {"value": batch * n / seconds, "unit": "tokens/s", "steps": n,
            "h2d_bytes_per_step": 4 * graph.size, "d2h_bytes_per_step": 4 * graph.rows,
            "ms_per_step": seconds / n * 1e3}


def profile_case(mode: str, layers: int, batch: int, ctx: int, steps: int, page: int) -> None:
    """A small case for a profiler: ``layers`` layers of the configuration, a cache filled to
    ``ctx`` positions per request without running a prefill (its contents do not matter to a
    kernel's duration), then ``steps`` eager decode steps or one prefill of 2,048 tokens."""
    import tempfile

    import torch

    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    with tempfile.TemporaryDirectory(prefix="tokenomos_b200_profile_") as tmp:
        folder = Path(tmp) / "model"
        write_folder(folder, layers)
        model = models.load(folder, "cuda", models.configure(folder, work="bf16"))
    pages = batch * (-(-(ctx + PROMPT + steps) // page)) + 2
    cache = CacheManager(model.state_specs(), page, pages, batch, torch.bfloat16, "cuda",
                         max_len=ctx + PROMPT + steps + page)
    step_fn = StepFunction(model, cache)
    for r in range(batch):
        cache.admit(r)
        if ctx:
            cache.extend(r, ctx)
            cache.commit(r, ctx)
    g = torch.Generator().manual_seed(0)
    if mode == "decode_graph":
        # the captured decode step exactly as serving replays it (token select ... sampling)
        rows = [(0.0, 1.0, 0, 0.0, 0, 0)] * batch
        for _ in range(steps):
            step_fn.run_decode_graph([StepEntry(r, [1 + r], []) for r in range(batch)], rows, commit=True)
    elif mode == "decode":
        for _ in range(steps):
            step_fn.run([StepEntry(r, [int(torch.randint(0, 1000, (1,), generator=g))], [0])
                         for r in range(batch)])
    else:
        ids = torch.randint(0, model.vocab, (PROMPT,), generator=g).tolist()
        for _ in range(steps):
            step_fn.run([StepEntry(0, ids, [PROMPT - 1])])
            cache.release(0)
            cache.admit(0)
    torch.cuda.synchronize()
    print(f"profile case done: {mode} layers={layers} batch={batch} ctx={ctx} steps={steps}")


def kernel_case(name: str) -> None:
    """One kernel alone for a profiler, over operands that rotate through more than the L2 holds:
    ``gemm_tc64``: the tcgen05 product of 64 rows with a [6144, 2048] matrix, 16 launches;
    ``conv_tile``: the tiled gated short conv over a 2,048-token portion of 2,048 channels (width 3,
    tiles of 16 tokens), 20 launches in a CUDA graph that is replayed five times;
    ``attn_portions`` (a measurement, not a profiler case): the tcgen05 prefill attention on
    portions behind cached contexts, with a tile's keys shared by 1 to 16 CTAs."""
    import torch

    from tokenomos_b200 import ops

    ops.available()
    dev, bf16 = "cuda", torch.bfloat16
    if name == "attn_portions":
        # the tcgen05 prefill attention on a portion of T tokens behind C cached positions (32
        # heads of 64 over 8 KV heads, one sequence), with up to `split` CTAs sharing a tile's
        # keys: CUDA events around 10 launches, after 3
        H, Hkv, D, P = 32, 8, 64, 16
        per = ops.attention_prefill_tc_tokens(H, Hkv)
        for T, C in ((512, 0), (512, 3584), (512, 32256), (128, 4096), (128, 32640), (32, 32640), (2048, 0), (2048, 30720)):
            q = torch.randn(T, H, D, device=dev, dtype=bf16)
            pages = (C + T) // P + 2
            pool = torch.randn(pages, 2, Hkv, P, D, device=dev, dtype=bf16)
            out = torch.empty_like(q)
            pos = torch.arange(C, C + T, dtype=torch.int32, device=dev)
            seq = torch.zeros(T, dtype=torch.int32, device=dev)
            table = torch.arange(1, pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
            t0 = torch.arange(0, T, per, dtype=torch.int32, device=dev)
            nt = torch.full((t0.numel(),), per, dtype=torch.int32, device=dev)
            flops = 4.0 * H * D * sum(C + i + 1 for i in range(T))
            line = f"portion {T:5d} behind {C:6d} ({t0.numel() * Hkv:4d} CTAs unsplit):"
            for split in (1, 2, 4, 8, 16):
                if split > 1 and t0.numel() * Hkv * split > 4 * 296:
                    continue
                for _ in range(3):
                    ops.attention_prefill_tc(q, pool, out, pos, seq, table, t0, nt, None, D ** -0.5, None, split)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(10):
                    ops.attention_prefill_tc(q, pool, out, pos, seq, table, t0, nt, None, D ** -0.5, None, split)
                b.record()
                torch.cuda.synchronize()
                us = a.elapsed_time(b) / 10 * 1e3
                line += f"  x{split}: {us:7.1f} us ({flops / us / 1e6:5.0f} TFLOP/s)"
            print(line, flush=True)
        if ops.attention_prefill_tc_status():
            raise RuntimeError("the tcgen05 attention reported an error")
    elif name == "gemm_tc64":
        ws = [torch.randn(6144, 2048, device=dev, dtype=bf16) * 0.02 for _ in range(8)]
        x = torch.randn(64, 2048, device=dev, dtype=bf16)
        for i in range(16):
            ops.gemm_tc(x, ws[i % 8])
        torch.cuda.synchronize()
        if ops.gemm_tc_status():
            raise RuntimeError("the tcgen05 product reported an error")
    else:
        tokens, width, taps, tile = 2048, 2048, 3, 16
        ins = [torch.randn(tokens, 3 * width, device=dev, dtype=bf16) for _ in range(10)]
        w = torch.randn(width, taps, device=dev)
        state = torch.zeros(4, taps - 1, width, device=dev, dtype=bf16)
        i32 = dict(dtype=torch.int32, device=dev)
        cu, ctx0, slot = torch.tensor([0, tokens], **i32), torch.zeros(1, **i32), torch.ones(1, **i32)
        seq, off = torch.zeros(tokens // tile, **i32), torch.arange(0, tokens, tile, **i32)
        n = torch.full((tokens // tile,), tile, **i32)

        def calls():
            for i in range(20):
                ops.conv_gated(ins[i % 10], w, None, state, cu, ctx0, slot, seq, off, n, 0, tile, off)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            calls()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            calls()
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
    print(f"kernel case done: {name}")


def ingraph_table(layers: int, batch: int, ctx: int, page: int) -> None:
    """What each kind of kernel costs *inside* the captured decode step, where launches overlap
    through programmatic dependent launch and a kernel's cold, serialised time under a profiler
    says little: the step is captured once whole and once per kind with that kind's launches
    left out (their outputs stay unwritten, which changes no launch that follows), each graph is
    replayed and timed with CUDA events, and the difference is the kind's cost in the step.
    Prints one line per kind: launches, microseconds, microseconds per launch, share, and for
    matrix products the bytes of the matrix over that time."""
    import tempfile

    import torch
    import torch.nn.functional as F

    import tokenomos_b200.parts.linear as linear_part
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepFunction
    from tokenomos_b200.ops import _lib
    from tokenomos_b200.sampling import sampler

    with tempfile.TemporaryDirectory(prefix="tokenomos_b200_profile_") as tmp:
        folder = Path(tmp) / "model"
        write_folder(folder, layers)
        model = models.load(folder, "cuda", models.configure(folder, work="bf16"))
    pages = batch * (-(-(ctx + 64) // page)) + 2
    cache = CacheManager(model.state_specs(), page, pages, batch, torch.bfloat16, "cuda", max_len=ctx + 64)
    for r in range(batch):
        cache.admit(r)
        cache.extend(r, ctx + 1)
        cache.commit(r, ctx)
    real_call, real_linear, real_mm = _lib.call, F.linear, torch.mm
    seen: dict[str, int] = {}
    sizes: dict[str, int] = {}

    def key_of(name, args):
        if name in ("tk_gemm_skinny", "tk_gemm_tc_decode", "tk_gemm_skinny_conv"):
            extra = ""
            if name == "tk_gemm_skinny":
                extra = (" swiglu" if args[11] else "") + (" +norm" if args[12] > 0 else "") + (" +add" if args[13] else "")
            k = f"{name[3:]}[{args[8]}x{args[9]}]{extra}"
            sizes[k] = 2 * args[8] * args[9]
            return k
        return name[3:]

    def timed_step(skip=None, record=False) -> float:
        def call(name, *args):
            k = key_of(name, args)
            if record and name not in _lib._QUERIES:
                seen[k] = seen.get(k, 0) + 1
            return 0 if k == skip else real_call(name, *args)

        def lin(x, w, b=None):
            k = f"library[{w.shape[0]}x{w.shape[1]}]"
            sizes[k] = 2 * w.shape[0] * w.shape[1]
            if record:
                seen[k] = seen.get(k, 0) + 1
            if k == skip:
                return torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
            return real_linear(x, w, b)

        def mm(a, b, out_dtype=None):
            k = f"library[{b.shape[1]}x{b.shape[0]}]"
            sizes[k] = 2 * b.shape[0] * b.shape[1]
            if record:
                seen[k] = seen.get(k, 0) + 1
            if k == skip:
                return torch.empty(a.shape[0], b.shape[1], dtype=out_dtype or a.dtype, device=a.device)
            return real_mm(a, b, out_dtype=out_dtype) if out_dtype else real_mm(a, b)

        _lib.call, linear_part.F.linear, torch.mm = call, lin, mm
        try:
            graph = StepFunction(model, cache).decode_graph(batch)
        finally:
            _lib.call, linear_part.F.linear, torch.mm = real_call, real_linear, real_mm
        h = graph.host_np[0]
        states = [cache.requests[r] for r in range(batch)]
        for name, values in (("positions", [st.length for st in states]), ("seq_ctx", [st.length for st in states]),
                             ("seq_slot", [st.slot for st in states]), ("ids_host", [5] * batch),
                             ("use_prev", [0] * batch)):
            o, _ = graph.off[name]
            h[o:o + batch] = values
        o, _ = graph.off["sampling"]
        sampler.pack_rows_into(h[o:o + 6 * graph.rows], [(0.0, 1.0, 0, 0.0, 0, 0)] * batch, graph.rows)
        for grp in graph.groups:
            o, _ = graph.off[("table", grp)]
            for i, st in enumerate(states):
                row = st.tables[grp]
                h[o + i * graph.width:o + i * graph.width + len(row)] = row
        graph.dev.copy_(graph.host[0])
        torch.cuda.synchronize()
        for _ in range(5):
            graph.graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(20):
                graph.graph.replay()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end) / 20 * 1e3)
        return statistics.median(times)

    whole = timed_step(record=True)
    # the step is run once to warm up and once to be captured: every kind was counted twice
    print(f"decode step, batch {batch}, {ctx} cached positions, {layers} layers: {whole:.1f} us, "
          f"{sum(seen.values()) // 2} launches")
    rows = []
    for k, n in seen.items():
        rows.append((whole - timed_step(skip=k), k, n // 2))
    print(f"  {'kind':46s} launches      us   us each   share   matrix GB/s")
    for cost, k, n in sorted(rows, reverse=True):
        rate = f"{sizes[k] * n / cost / 1e3:10.0f}" if k in sizes and cost > 0 else ""
        print(f"  {k:46s} {n:6d} {cost:9.1f} {cost / max(n, 1):8.2f} {100 * cost / whole:6.1f}%  {rate}")
    print(f"  the kinds sum to {sum(r[0] for r in rows):.1f} us of the step's {whole:.1f}")


def chunked_prefill(model, cfg, page: int, prompt: int, budget: int, max_new: int = 2) -> dict:
    """One long prompt through the engine in portions of ``budget`` tokens, as the scheduler cuts
    it (late portions are few tiles behind a long context): wall clock of the whole call, one
    request, the better of two calls after the engine has warmed up."""
    import torch

    from tokenomos_b200.engine.engine import Engine
    from tokenomos_b200.engine.scheduler import Request

    eng = Engine(model, slots=2, page=page, max_len=prompt + 64, prefill_budget=budget, graphs=True, warmup=True)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (prompt,), generator=g).tolist()
    best = None
    for _ in range(2):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.generate([Request(ids, max_new=max_new)])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    del eng
    torch.cuda.empty_cache()
    return {"prompt": prompt, "portion": budget, "ms": round(best * 1e3, 1), "tok_s": round(prompt / best, 1)}


def run_sweep(model, cfg, page: int, pk: dict) -> int:
    """Decode at other batch sizes and context lengths, prefill at other lengths: one JSON line
    of points, each with its fraction of the roofline (decode: bytes the step must read over the
    measured copy bandwidth; prefill: flops over the measured bf16 GEMM rate)."""
    conv_layers = sum(k == "conv" for k in cfg.layer_types)
    out = {"sweep": "1.2B-size LFM3, bf16, random weights", "decode": [], "prefill": []}
    for ctx in (512, 8192, 32768):
        for batch in (1, 8, 64):
            r = device_decode(model, cfg, batch, 32, 4, page, prompt=ctx, context=ctx + 64)
            mid = (r["ctx_start"] + r["ctx_end"]) / 2
            nbytes = (weight_bytes(model, cfg) + batch * mid * kv_bytes_per_token(cfg)
                      + batch * conv_layers * 2 * (cfg.conv_L_cache - 1) * cfg.hidden_size * 2)
            out["decode"].append({"batch": batch, "ctx": ctx, "ms": round(r["ms_per_step"], 4),
                                  "tok_s": round(r["tok_s"], 1),
                                  "frac_hbm": round(nbytes / (r["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3)})
    for n in (512, 8192, 32768):
        r = device_prefill(model, cfg, page, reps=2, tokens=n)
        out["prefill"].append({"tokens": n, "ms": round(r["ms"], 3), "tok_s": round(r["tok_s"], 1),
                               "frac_bf16": round(r["flops"] / (r["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 3)})
    out["chunked_prefill"] = [chunked_prefill(model, cfg, page, prompt, budget)
                              for prompt, budget in ((32000, 512), (32000, 128), (8000, 512))]
    print(json.dumps(out))
    return 0


def run_workload(name: str, page: int, trace_path: str | None = None) -> int:
    """A whole serving workload through ``LLM.generate`` (continuous batching: prompts are cut
    into portions under the token budget and run beside the decoding requests): wall-clock
    tokens per second, prompt and generated."""
    import tempfile

    import torch

    from tokenomos_b200.api.llm import LLM, SamplingParams

    w = WORKLOADS[name]
    tmp = tempfile.TemporaryDirectory(prefix="tokenomos_b200_bench_")
    folder = Path(tmp.name) / name
    write_folder(folder, len(w["config"]["layer_types"]), w["config"])
    g = torch.Generator().manual_seed(0)
    lo, hi = w["prompt"]
    lengths = torch.randint(lo, hi + 1, (w["requests"],), generator=g).tolist()
    vocab = w["config"]["vocab_size"]
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
    pages = sum(-(-(n + w["new_tokens"] + 1) // page) for n in lengths) + 2
    t0 = time.perf_counter()
    llm = LLM(str(folder), work="bf16", slots=w["slots"], page=page, max_len=w["max_len"], pages=pages,
              prefill_budget=w["budget"], graphs=True, warmup=True)
    warmup_seconds = time.perf_counter() - t0
    shapes_after_warmup = len(llm.engine.step_fn._step_graphs) + len(llm.engine.step_fn._graphs)
    clocks = Clocks()
    try:
        # the engine warmed up before serving (every step shape the budget allows is captured
        # then); the first pass shows what is left of the start-up cost
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        llm.generate(prompts, SamplingParams(max_tokens=w["new_tokens"]))
        torch.cuda.synchronize()
        first_seconds = time.perf_counter() - t0
        steps_before = llm.engine.stats.steps
        decode_before, graph_before = llm.engine.stats.decode_steps, llm.engine.stats.graph_steps
        clocks.start()
        # three steady-state passes, the median reported: the loop is host-bound in places, and
        # the host is a shared machine
        passes = []
        for _ in range(3):
            t0 = time.perf_counter()
            outs = llm.generate(prompts, SamplingParams(max_tokens=w["new_tokens"]))
            torch.cuda.synchronize()
            passes.append(time.perf_counter() - t0)
        seconds = sorted(passes)[1]
        if trace_path:
            # one more pass with a record per step: kind, rows, tokens, bucket, host and device ms
            llm.engine.trace_on()
            llm.generate(prompts, SamplingParams(max_tokens=w["new_tokens"]))
            Path(trace_path).write_text(json.dumps(llm.engine.trace_take()))
        steps_per_pass = (llm.engine.stats.steps - steps_before) // 3
        decode_per_pass = (llm.engine.stats.decode_steps - decode_before) // 3
        graph_per_pass = (llm.engine.stats.graph_steps - graph_before) // 3
    finally:
        clock_report = clocks.stop()
        stats = llm.engine.stats
        llm_graphs = dict(llm.engine.step_fn._step_graphs)
        llm.close()
        tmp.cleanup()
    generated = sum(len(o.token_ids) for o in outs)
    print(json.dumps({
        "workload": name, "metric": "tokens/s over the whole call (prompt + generated)",
        "value": round((sum(lengths) + generated) / seconds, 1), "unit": "tokens/s",
        "generated_per_s": round(generated / seconds, 1), "seconds": round(seconds, 3),
        "passes_seconds": [round(t, 3) for t in passes], "first_pass_seconds": round(first_seconds, 3),
        "warmup_seconds": round(warmup_seconds, 3), "shapes_after_warmup": shapes_after_warmup,
        "captured_step_shapes": len(llm_graphs), "graph_steps": graph_per_pass,
        "requests": w["requests"], "prompt_tokens": sum(lengths), "generated": generated,
        "steps": steps_per_pass, "decode_steps": decode_per_pass, "preemptions": stats.preemptions,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {"layers": len(w["config"]["layer_types"]), "hidden_size": w["config"]["hidden_size"],
                   "intermediate_size": w["config"]["intermediate_size"], "max_len": w["max_len"],
                   "slots": w["slots"], "token_budget": w["budget"], "page_size": page},
        "clocks": clock_report}))
    return 0


def bench_config(layers: int, batch: int, config: dict) -> dict:
    """The ``config`` record of the JSON line: every size, flat; the same for both arms."""
    return {
        "model": "LFM3 1.2B-size (BASELINE configs[2]) + per-head output gate", "global_batch": batch,
        "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
        "layers": layers, "layers_of_config": 16, "hidden_size": config["hidden_size"],
        "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"],
        "head_dim": config["head_dim"], "intermediate_size": config["intermediate_size"],
        "vocab_size": config["vocab_size"], "conv_L_cache": config["conv_L_cache"],
        "attention_gate": bool(config.get("attention_gate")),
        "l2": "inputs larger than L2 (weights read every step)",
    }


REF_ROOT = ROOT / "baseline" / "_ref"


def reference_arm(args, warmup: int) -> dict:
    """The same metric on the unmodified reference: its Python package as copied from its
    ``src`` folder into ``baseline/_ref`` (its wheel needs maturin and a Rust toolchain, which
    the offline wheelhouse lacks; the Rust module serves the JSON grammar only, Tokenomos
    api/llm.py:27, and is stubbed with empty modules). The path is the reference's own decode
    bench (Tokenomos bench/decode.py:62-137): ``models.load``, ``Engine(...)``, ``warmup()``,
    ``generate`` of random prompts; the steady decode step is the median gap between the stamps
    of consecutive decode-step enqueues with every row live, the prefill the device time of one
    2,048-token request with one new token. Nothing of tokenomos_b200 is imported here."""
    import tempfile
    import types

    sys.path.insert(0, str(REF_ROOT))
    for name in ("tokenomos._rs", "tokenomos._rs.grammar"):
        sys.modules.setdefault(name, types.ModuleType(name))
    import torch
    from tokenomos import models
    from tokenomos.core.engine import Engine, Request

    torch.cuda.set_device(0)
    tmp = tempfile.TemporaryDirectory(prefix="tokenomos_ref_bench_")
    folder = Path(tmp.name) / "lfm3_1p2b_random"
    config = write_folder(folder, args.layers)
    model = models.load(str(folder), "cuda", models.configure(str(folder), work="bf16"))
    vocab = config["vocab_size"]
    g = torch.Generator().manual_seed(2)
    clocks = Clocks()
    clocks.start()

    def engine(batch: int, new: int, prompt: int):
        page = 32                                        # the reference's default
        max_len = prompt + new + 8
        eng = Engine(model, slots=batch, page=page, max_len=max_len, new_cap=new, reserve_new=new,
                     pages=batch * -(-max_len // page) + 8, graphs=True)
        eng.warmup()
        return eng

    def decode(batch: int, steps: int, prompt: int) -> dict:
        # enough decode steps for the K-step block to repeat as in the other arm
        new = warmup + 8 + max(3 * steps, int(MIN_TIMED_MS / 0.5))
        new = min(new, CONTEXT - prompt - 8) if prompt == PROMPT_FAR else new
        eng = engine(batch, new, prompt)
        reqs = [Request(torch.randint(0, vocab, (prompt,), generator=g).tolist(), max_new=new)
                for _ in range(batch)]
        eng.generate([Request(list(r.prompt), max_new=4) for r in reqs[:8]])
        eng.stats = type(eng.stats)()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        results = eng.generate(reqs)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert all(len(r.tokens) == new for r in results)
        st = eng.stats.stamps                            # (perf_counter, bucket, rows bound)
        full = [i for i, (_, _, r) in enumerate(st) if r == batch]
        lo, hi = full[0] + warmup, full[-1] - 2
        gaps = [st[i + 1][0] - st[i][0] for i in range(lo, hi) if st[i][2] == batch and st[i + 1][2] == batch]
        step_ms = statistics.median(gaps) * 1e3
        span = st[hi][0] - st[lo][0]
        out = {"ms_per_step": step_ms, "tok_s": batch / step_ms * 1e3, "steady_steps": len(gaps),
               "span_tok_s": batch * (hi - lo) / span, "wall_s": wall,
               "d2h_bytes_per_step": 4 * int(eng.ev_dev.numel())}
        if batch == args.batch and prompt == PROMPT:
            times = []
            for i in range(5):
                one = Request(torch.randint(0, vocab, (PROMPT,), generator=g).tolist(), max_new=1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                eng.generate([one])
                b.record()
                torch.cuda.synchronize()
                if i >= 2:
                    times.append(a.elapsed_time(b))
            out["prefill_ms"] = statistics.median(times)
        del eng
        torch.cuda.empty_cache()
        return out

    main_run = decode(args.batch, args.steps, PROMPT)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode(b, min(args.steps, 64), PROMPT)["tok_s"], 1)
        for b in (1, args.batch, 64):
            points[f"decode_b{b}_far"] = round(decode(b, min(args.steps, 64), PROMPT_FAR)["tok_s"], 1)
    clock_report = clocks.stop()
    tmp.cleanup()
    pk = peaks()
    flops = prefill_flops(config, PROMPT)
    return {
        "impl": "reference",
        "metric": METRIC, "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": bench_config(args.layers, args.batch, config),
        "engine": {"page_size": 32, "timing": "median gap between decode-step enqueues, every row live "
                   f"({main_run['steady_steps']} steps), the host one step ahead of the device"},
        "clocks": clock_report,
        "e2e": {"value": round(main_run["span_tok_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": main_run["d2h_bytes_per_step"],
                "ms_per_step": round(args.batch / main_run["span_tok_s"] * 1e3, 4)},
        "prefill": {"value": round(PROMPT / main_run["prefill_ms"] * 1e3, 1), "tokens": PROMPT,
                    "ms": round(main_run["prefill_ms"], 3),
                    "frac": round(flops / (main_run["prefill_ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "points": points,
    }


def run_reference(args, warmup: int) -> int:
    if not (REF_ROOT / "tokenomos" / "__init__.py").exists():
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref/tokenomos is absent: the reference's wheel cannot be built "
                          "offline (its backend is maturin, pyproject.toml:1-3), and its Python "
                          "package was not copied there"}))
        return 0
    try:
        line = reference_arm(args, warmup)
    except Exception as e:  # noqa: BLE001 - the arm reports why it could not run
        text = " ".join(f"{type(e).__name__}: {e}".split())
        print(json.dumps({"impl": "reference", "unavailable": text[:400]}))
        return 0
    print(json.dumps(line))
    return 0


def prefill_flops(config: dict, tokens: int) -> float:
    """Flops of one prompt of ``tokens``: 2 * tokens * parameters of every matrix the tokens
    pass (the head runs on one row), plus causal attention (q.k and p.v over half the square)."""
    d, inter = config["hidden_size"], config["intermediate_size"]
    H, Hkv, D = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    flops = 0.0
    for kind in config["layer_types"]:
        per_tok = 3 * d * inter
        if kind == "conv":
            per_tok += 3 * d * d + d * d
        else:
            per_tok += (H + 2 * Hkv) * D * d + H * D * d
            flops += 2 * 2 * H * D * tokens * (tokens + 1) / 2
        flops += 2 * tokens * per_tok
    return flops + 2 * config["vocab_size"] * d


METRIC = "decode tokens/s (1.2B-size LFM3, batch 8, context 2048+)"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="run a whole serving workload of BASELINE.json (configs[3] / configs[4]) instead")
    ap.add_argument("--profile", default=None, choices=["decode", "decode_graph", "prefill", "ingraph"],
                    help="run only a small case for a profiler (see profile_case) and exit; ingraph: "
                         "the cost of each kind of kernel inside the captured decode step (ingraph_table)")
    ap.add_argument("--kernel", default=None, choices=["gemm_tc64", "conv_tile", "attn_portions"],
                    help="run only one kernel over rotating operands for a profiler (see kernel_case) and exit")
    ap.add_argument("--ctx", type=int, default=2048, help="--profile: positions already cached")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=16, help="layers of the 16 the configuration has")
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--trace", default=None,
                    help="--workload: write one JSON record per step of an extra pass to this file")
    ap.add_argument("--sweep", action="store_true",
                    help="decode and prefill at other batch sizes and context lengths instead")
    args = ap.parse_args()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus > 1 is not built")
        return 2
    warmup = max(3, args.warmup)
    if args.impl == "reference":
        return run_reference(args, warmup)

    import torch

    from tokenomos_b200 import ops

    torch.cuda.set_device(0)
    ops.available()
    if args.kernel:
        kernel_case(args.kernel)
        return 0
    if args.profile == "ingraph":
        ingraph_table(args.layers, args.batch, args.ctx, args.page)
        return 0
    if args.profile:
        profile_case(args.profile, args.layers, args.batch, args.ctx, args.steps, args.page)
        return 0
    if args.workload:
        return run_workload(args.workload, args.page, args.trace)
    pk = peaks()
    import tempfile

    from tokenomos_b200.api.llm import LLM

    tmp = tempfile.TemporaryDirectory(prefix="tokenomos_b200_bench_")
    folder = Path(tmp.name) / "lfm3_1p2b_random"
    config = write_folder(folder, args.layers)
    pages = args.batch * (CONTEXT // args.page) + 2
    llm = LLM(str(folder), work="bf16", slots=args.batch, page=args.page, max_len=CONTEXT,
              pages=pages, prefill_budget=PROMPT, graphs=True)
    model, cfg = llm.model, llm.model.config
    if args.sweep:
        rc = run_sweep(model, cfg, args.page, pk)
        llm.close()
        tmp.cleanup()
        return rc
    clocks = Clocks()
    clocks.start()
    main_run = device_decode(model, cfg, args.batch, args.steps, warmup, args.page)
    prefill = device_prefill(model, cfg, args.page)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(device_decode(model, cfg, b, min(args.steps, 64), warmup,
                                                         args.page)["tok_s"], 1)
        for b in (1, args.batch, 64):
            points[f"decode_b{b}_far"] = round(device_decode(
                model, cfg, b, min(args.steps, 64), warmup, args.page, prompt=PROMPT_FAR)["tok_s"], 1)
        # a 32,000-token prompt served in portions of 512 tokens (tokens a second over the call)
        try:
            points["prefill_32k_by_512"] = chunked_prefill(model, cfg, args.page, 32000, 512)["tok_s"]
        except Exception as exc:  # the line above it must not be lost to this point
            print(f"bench.py: the chunked prefill point failed: {exc}", file=sys.stderr)
            points["prefill_32k_by_512"] = None
        # the 2,048-token prompt as the reference arm times it: one request with one new token
        # through the engine's own generate call, wall clock
        try:
            points["prefill_2048_through_engine_ms"] = chunked_prefill(model, cfg, args.page, PROMPT, PROMPT, 1)["ms"]
        except Exception as exc:
            print(f"bench.py: the prefill-through-the-engine point failed: {exc}", file=sys.stderr)
            points["prefill_2048_through_engine_ms"] = None
    e2e = e2e_decode(llm, cfg, args.batch, args.steps, warmup)
    clock_report = clocks.stop()
    llm.close()
    tmp.cleanup()

    ctx_mid = (main_run["ctx_start"] + main_run["ctx_end"]) / 2
    conv_layers = sum(k == "conv" for k in cfg.layer_types)
    step_bytes = (weight_bytes(model, cfg) + args.batch * ctx_mid * kv_bytes_per_token(cfg)
                  + args.batch * conv_layers * 2 * (cfg.conv_L_cache - 1) * cfg.hidden_size * 2)
    achieved = step_bytes / (main_run["ms_per_step"] * 1e-3) / 1e9
    line = {
        "impl": "ours",
        "metric": METRIC,
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": bench_config(args.layers, args.batch, config),
        "engine": {"page_size": args.page, "decode_ctx_start": main_run["ctx_start"],
                   "decode_ctx_end": main_run["ctx_end"], "timed_blocks": main_run["blocks"],
                   "timed_ms": round(main_run["timed_ms"], 1),
                   "timing": "median of blocks of exactly `steps` steps, CUDA events around each"},
        "clocks": clock_report,
        "e2e": {k: (round(v, 4 if k == "ms_per_step" else 1) if isinstance(v, float) else v)
                for k, v in e2e.items()},
        "gpu_launches": main_run["launches_per_step"] * args.steps,
        "prefill": {"value": round(prefill["tok_s"], 1), "tokens": PROMPT, "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "eager_ms": round(prefill["eager_ms"], 3),
                    "how": "one captured step (layout upload to sampled token), as a warmed-up engine runs it"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "peaks": pk["source"]},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
