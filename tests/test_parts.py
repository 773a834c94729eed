"""Each part alone against the plain implementation's function for it; the layer list as data
(a block run twice, a layer reading another layer's cache); and a toy mixer with state of its
own, defined here, registered, built and stepped without touching the framework's files."""

from __future__ import annotations

import json

import pytest
import torch

import plain_lfm3
from conftest import TINY

pytestmark = pytest.mark.gpu


def _ctx_for(model_or_specs, page, seq_lens, dtype, pages=64, slots=4):
    """A cache manager and a step function's layout for fresh sequences of ``seq_lens``."""
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    class _M:
        vocab = 1 << 30
    specs = model_or_specs
    cache = CacheManager(specs, page, pages, slots, dtype, "cuda", max_len=512)
    step = StepFunction(_M(), cache)
    entries = []
    for i, n in enumerate(seq_lens):
        cache.admit(i)
        entries.append(StepEntry(i, [0] * n, []))
    ctx, _, _ = step.layout(entries)
    return ctx, cache, step


def _close(got, want, dtype, what):
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    got, want = got.double().cpu(), want.double()
    scale = max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    assert err <= tol * scale, f"{what}: error {err:.3e}, allowed {tol * scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixers_and_ffn_alone(name, dtype, model_folders):
    """Every block's mixer and feed-forward, fed the same normed input as the plain functions."""
    from tokenomos_b200 import models
    folder = model_folders[name][torch.bfloat16]
    config, w = plain_lfm3.read_folder(folder)
    s = plain_lfm3.settings(config)
    model = models.load(folder, "cuda", models.configure(folder, work=dtype))
    lens = [13, 1, 30]
    ctx, cache, _ = _ctx_for(model.state_specs(), TINY[name]["page"], lens, dtype)
    d = config["hidden_size"]
    x = torch.randn(sum(lens), d).to(dtype)
    for i, kind in enumerate(s["layer_types"]):
        block = model.blocks[i]
        p = f"model.layers.{i}."
        # each part is fed what its own pre-norm makes of x. In a 16-bit model the norm's weight
        # lives in the part's first projection (the block folds it in when it is built) and the
        # norm that is left has weight one; the pair must still equal norm-with-weight then part.
        folded = dtype == torch.bfloat16 and not s["sandwich"]
        assert (block.eps_mixer is not None) == folded and (block.eps_ffn is not None) == folded
        for norm, weight in ((block.pre_mixer, f"{p}operator_norm.weight"), (block.pre_ffn, f"{p}ffn_norm.weight")):
            plain_weight = torch.ones_like(w[weight]) if folded else w[weight]
            _close(norm(x.cuda()), plain_lfm3.rmsnorm(x.double(), plain_weight, s["eps"]), dtype,
                   f"{name} layer {i} {weight}")
        xs = torch.split(plain_lfm3.rmsnorm(x.double(), w[f"{p}operator_norm.weight"], s["eps"]), lens)
        got = block.mixer.forward(block.pre_mixer(x.cuda()), ctx, i)
        if kind == "conv":
            want = torch.cat([plain_lfm3.short_conv(v, w, f"{p}conv.", s, torch.float64) for v in xs])
        else:
            want = torch.cat([plain_lfm3.attention(v, w, f"{p}self_attn.", s, kind, torch.float64)
                              for v in xs])
        _close(got, want, dtype, f"{name} layer {i} {kind}")
        got = block.ffn.forward(block.pre_ffn(x.cuda()))
        normed = plain_lfm3.rmsnorm(x.double(), w[f"{p}ffn_norm.weight"], s["eps"])
        _close(got, plain_lfm3.swiglu(normed, w, f"{p}feed_forward.", torch.float64), dtype,
               f"{name} layer {i} ffn")


def test_rope_part_matches_the_plain_tables():
    from tokenomos_b200.parts.rope import Rope
    for D, angles, theta in ((16, 8, 1e4), (24, 12, 1e6), (32, 8, 5e4)):
        rope = Rope(D, angles, theta, "cpu")
        pos = torch.tensor([0, 1, 77, 4095])
        f = pos.float()[:, None] * rope.inv_freq[None]
        cos, sin = plain_lfm3.rope_tables(pos, D, angles, theta, torch.float64)
        assert torch.equal(torch.cat((f, f), -1).double().cos(), cos)
        assert (rope.inv_freq[angles:] == 0).all() and rope.inv_freq.numel() == D // 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_list_is_data(dtype, model_folders):
    """Run block 1 twice and let the last attention layer read block 1's cache instead of having
    keys of its own: the stack follows the list; each entry has its own state unless it shares."""
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction
    from tokenomos_b200.parts.spec import LayerCall
    name = "B"
    folder = model_folders[name][torch.bfloat16]
    config, w = plain_lfm3.read_folder(folder)
    model = models.load(folder, "cuda", models.configure(folder, work=dtype))
    # B's layers: conv, attn, conv, conv, attn, attn. New list: 0, 1, 1, 2, 3, 4
    model.order = [LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(2), LayerCall(3), LayerCall(4)]
    specs = model.state_specs()
    assert (1, "kv") in specs and (2, "kv") in specs and (3, "conv") in specs
    ids = torch.randint(0, config["vocab_size"], (45,)).tolist()
    # the plain implementation of the same list: a config and weights with layer 1 duplicated
    config2 = json.loads(json.dumps(config))
    lt = config["layer_types"]
    config2["layer_types"] = [lt[0], lt[1], lt[1], lt[2], lt[3], lt[4]]
    config2["num_hidden_layers"] = 6
    w2 = {}
    mapping = {0: 0, 1: 1, 2: 1, 3: 2, 4: 3, 5: 4}
    for new, old in mapping.items():
        for k, v in w.items():
            if k.startswith(f"model.layers.{old}."):
                w2[k.replace(f"model.layers.{old}.", f"model.layers.{new}.", 1)] = v
    for k, v in w.items():
        if not k.startswith("model.layers."):
            w2[k] = v
    want = plain_lfm3.forward_logits(config2, w2, ids)
    cache = CacheManager(specs, 8, 40, 2, dtype, "cuda", max_len=128)
    step = StepFunction(model, cache)
    cache.admit("a")
    outs = [step.run([StepEntry("a", ids[a:b], list(range(b - a)))])
            for a, b in ((0, 20), (20, 21), (21, 45))]
    _close(torch.cat(outs), want, dtype, "layer list with a block twice")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shared_kv_layer_reads_another_layers_cache(dtype):
    """A queries-only attention layer (``kv_source``) over the cache an earlier entry wrote."""
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction
    from tokenomos_b200.parts.attention import Attention
    from tokenomos_b200.parts.contract import SharedState
    from tokenomos_b200.parts.linear import Linear
    from tokenomos_b200.parts.rope import Rope
    H, Hkv, D, d = 4, 2, 16, 40
    rope = Rope(D, D // 2, 1e4, "cuda")
    mk = lambda *shape: (torch.randn(*shape) * 0.2).to(dtype)  # noqa: E731
    wq, wk, wv, wo, wq2, wo2 = mk(H * D, d), mk(Hkv * D, d), mk(Hkv * D, d), mk(d, H * D), mk(H * D, d), mk(d, H * D)
    owner = Attention(Linear.fused([wq.cuda(), wk.cuda(), wv.cuda()]), Linear(wo.cuda()), H, Hkv, D, rope, 1e-5)
    reader = Attention(Linear(wq2.cuda()), Linear(wo2.cuda()), H, Hkv, D, rope, 1e-5, kv_source=0)
    assert reader.state_specs() == {"kv": SharedState(0, "kv")}
    specs = {(0, "kv"): owner.state_specs()["kv"], (1, "kv"): reader.state_specs()["kv"]}
    ctx, cache, _ = _ctx_for(specs, 4, [9, 2], dtype)
    x = torch.randn(11, d).to(dtype)
    owner.forward(x.cuda(), ctx, 0)
    got = reader.forward(x.cuda(), ctx, 1)
    # plain: the reader's queries over the owner's (rotated) keys and values
    want = []
    for xs in torch.split(x.double(), [9, 2]):
        T = xs.shape[0]
        cos, sin = plain_lfm3.rope_tables(torch.arange(T), D, D // 2, 1e4, torch.float64)
        q = plain_lfm3.rotate((xs @ wq2.double().T).view(T, H, D), cos, sin)
        k = plain_lfm3.rotate((xs @ wk.double().T).view(T, Hkv, D), cos, sin).repeat_interleave(2, 1)
        v = (xs @ wv.double().T).view(T, Hkv, D).repeat_interleave(2, 1)
        sc = torch.einsum("ihd,jhd->hij", q, k) * D ** -0.5
        sc = sc.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool))[None], float("-inf"))
        want.append(torch.einsum("hij,jhd->ihd", sc.softmax(-1), v).reshape(T, H * D) @ wo2.double().T)
    _close(got, torch.cat(want), dtype, "shared KV reader")


def _toy_folder(tmp_path, mixer, ffn, seed=4):
    import toy_parts
    from tokenomos_b200.weights import write_model_folder
    raw = toy_parts.toy_config(mixer, ffn)
    return raw, write_model_folder(tmp_path / f"toy_{mixer}_{ffn}", raw, seed=seed, std=0.3)


def _toy_weights(folder):
    from safetensors.torch import load_file
    return {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}


@pytest.mark.parametrize("mixer, ffn", [("ema_host", "swiglu"), ("ema_device", "swiglu"),
                                        ("attention_scaled", "routed"), ("attention_learned", "routed")])
def test_toy_parts_register_build_and_step(mixer, ffn, tmp_path):
    """Parts defined in ``tests/toy_parts.py`` (a mixer with state of its own, once planned on
    the host and once from device tensors with a state spec class of its own; a feed-forward that
    routes tokens to experts; two position encodings, one of them not a rotation and with a
    tensor of its own) are registered, named by a new architecture's declaration, loaded from a
    model folder and stepped whole, in portions and beside another request, with no change to the
    framework's files. The logits agree with each other and with the plain restatement."""
    import toy_parts
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    raw, folder = _toy_folder(tmp_path, mixer, ffn)
    model = models.load(folder, "cuda", models.configure(folder, work="fp32"))
    kinds = {"ema_host": toy_parts.EmaMixerHost, "ema_device": toy_parts.EmaMixerDevice}
    if mixer in kinds:
        assert isinstance(model.blocks[0].mixer, kinds[mixer])
        assert model.capture_safe == (mixer == "ema_device")
    else:
        want_rope = toy_parts.ScaledRope if mixer == "attention_scaled" else toy_parts.LearnedPosition
        assert isinstance(model.blocks[1].mixer.rope, want_rope) and model.capture_safe
        assert isinstance(model.blocks[0].ffn, toy_parts.RoutedFFN)
    cache = CacheManager(model.state_specs(), 4, 24, 3, torch.float32, "cuda", max_len=64, poison=True)
    if mixer.startswith("ema"):
        assert tuple(cache.states[(1, "ema")].shape) == (4, raw["width"])
        assert cache.states[(1, "ema")].dtype == torch.float32
    step = StepFunction(model, cache)
    T = 21
    ids = torch.randint(0, raw["vocab_size"], (T,)).tolist()
    cache.admit("w")
    whole = step.run([StepEntry("w", ids, list(range(T)))])
    cache.release("w")
    cache.admit("other")      # takes the slot and the pages "w" had
    step.run([StepEntry("other", [1, 2, 3], [])])
    cache.admit("p")
    parts = [step.run([StepEntry("p", ids[a:b], list(range(b - a))), StepEntry("other", [7], [])][:1 + (a > 0)])
             for a, b in ((0, 6), (6, 7), (7, 9), (9, T))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-5)
    want = toy_parts.toy_forward(raw, _toy_weights(folder), ids)
    assert (whole.double().cpu() - want).abs().max().item() < 2e-4 * want.abs().max().item()


@pytest.mark.parametrize("mixer, ffn", [("ema_host", "swiglu"), ("ema_device", "swiglu"),
                                        ("attention_scaled", "routed"), ("attention_learned", "routed")])
def test_toy_architectures_generate_through_the_entry_point_with_and_without_graphs(mixer, ffn, tmp_path):
    """The same toy models through ``LLM.generate``: scheduler, mixed steps, captured CUDA graphs.
    With ``graphs=True`` a model whose parts are all ``capture_safe`` is recorded and replayed
    (the device-side EMA, the routed feed-forward, both position encodings); the host-planned EMA
    is not ``capture_safe``, the engine says so in a warning and runs it eagerly. Either way the
    tokens equal the eager engine's, and every token is the plain restatement's choice given the
    same history."""
    import warnings

    import toy_parts
    from tokenomos_b200 import LLM, SamplingParams

    raw, folder = _toy_folder(tmp_path, mixer, ffn, seed=11)
    w = _toy_weights(folder)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for n in (9, 3, 17, 6, 12)]
    kw = dict(work="fp32", page=4, max_len=48, slots=3, pages=40, prefill_budget=10, poison=True)
    p = SamplingParams(max_tokens=10)
    with LLM(str(folder), graphs=False, **kw) as llm:
        eager = llm.generate(prompts, p)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        with LLM(str(folder), graphs=True, **kw) as llm:
            llm.engine.step_fn.capture_after = 0
            graphed = llm.generate(prompts, p)
            stats = llm.engine.stats
            captured = llm.engine.graphs
    if mixer == "ema_host":
        assert not captured and stats.graph_steps == 0
        assert any("not capture_safe: EmaMixerHost" in str(c.message) for c in caught)
    else:
        assert captured and stats.graph_steps > 0 and stats.decode_steps > 0
    for prompt, a, b in zip(prompts, eager, graphed):
        assert a.token_ids == b.token_ids
        logits = toy_parts.toy_forward(raw, w, prompt + b.token_ids)
        for i, tok in enumerate(b.token_ids):
            row = logits[len(prompt) + i - 1]
            assert row.max().item() - row[tok].item() <= 1e-4, (mixer, i, tok, int(row.argmax()))


@pytest.mark.parametrize("work, dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
def test_options_around_the_layer_stack_are_data_of_the_model(work, dtype, tmp_path):
    """An embedding scale, a soft cap on the logits and a list of ids that are never produced come
    from the architecture's declaration (``ModelSpec``), with no change to ``Stack``: a toy
    configuration sets all three; stepping whole and in portions, eagerly and through captured
    graphs, agrees with the plain restatement, and sampling at a high temperature never yields a
    suppressed id."""
    import toy_parts
    from tokenomos_b200 import LLM, SamplingParams, models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction
    from tokenomos_b200.weights import write_model_folder

    raw = toy_parts.toy_config("attention_scaled", "swiglu", embed_scale=3.5, logit_softcap=4.0,
                               suppress=[0, 7, 59])
    folder = write_model_folder(tmp_path / "toy_options", raw, seed=3, std=0.3)
    model = models.load(folder, "cuda", models.configure(folder, work=work))
    assert model.embed_scale == 3.5 and model.logit_softcap == 4.0 and model.suppress.tolist() == [0, 7, 59]
    cache = CacheManager(model.state_specs(), 4, 24, 2, dtype, "cuda", max_len=64, poison=True)
    step = StepFunction(model, cache)
    T = 19
    ids = torch.randint(0, raw["vocab_size"], (T,)).tolist()
    cache.admit("w")
    whole = step.run([StepEntry("w", ids, list(range(T)))])
    cache.release("w")
    cache.admit("p")
    parts = torch.cat([step.run([StepEntry("p", ids[a:b], list(range(b - a)))]) for a, b in ((0, 5), (5, 7), (7, T))])
    want = toy_parts.toy_forward(raw, _toy_weights(folder), ids)
    kept = [t for t in range(raw["vocab_size"]) if t not in raw["suppress"]]
    assert torch.isneginf(whole[:, raw["suppress"]]).all() and torch.isneginf(parts[:, raw["suppress"]]).all()
    assert whole[:, kept].abs().max().item() <= 4.0            # the cap holds
    tol = 2e-4 if dtype == torch.float32 else 4e-2
    scale = want[:, kept].abs().max().item()
    assert (whole.double().cpu()[:, kept] - want[:, kept]).abs().max().item() < tol * scale
    assert (parts.double().cpu()[:, kept] - want[:, kept]).abs().max().item() < tol * scale
    # through the entry point, captured: the suppressed ids never come out, and eager == captured
    prompts = [ids[:9], ids[3:8], ids[5:]]
    kw = dict(work=work, page=4, max_len=48, slots=3, pages=40, prefill_budget=10, poison=True)
    p = SamplingParams(max_tokens=8, temperature=1.5, seed=2)
    with LLM(str(folder), graphs=False, **kw) as llm:
        eager = llm.generate(prompts, p)
    with LLM(str(folder), graphs=True, **kw) as llm:
        llm.engine.step_fn.capture_after = 0
        graphed = llm.generate(prompts, p)
        assert llm.engine.stats.graph_steps > 0
    for a, b in zip(eager, graphed):
        if dtype == torch.float32:       # (in bfloat16 a sampled token may sit on a rounding edge)
            assert a.token_ids == b.token_ids
        assert not (set(a.token_ids) | set(b.token_ids)) & set(raw["suppress"])


@pytest.mark.filterwarnings("ignore::pytest.PytestUnhandledThreadExceptionWarning")
def test_a_part_that_reads_host_lists_in_a_captured_step_fails_loudly(tmp_path):
    """A mixer that claims ``capture_safe`` but plans from ``ctx.host``'s per-sequence lists would
    be recorded once and then replay the first batch's plan for ever. The lists do not exist in a
    captured step: the first capture raises, and the caller sees it."""
    from tokenomos_b200 import LLM, SamplingParams
    from tokenomos_b200.parts.contract import LayoutUnavailable

    raw, folder = _toy_folder(tmp_path, "ema_lying", "swiglu")
    with LLM(str(folder), work="fp32", page=4, max_len=32, slots=2, pages=20, graphs=True) as llm:
        with pytest.raises(RuntimeError, match="engine thread failed") as err:
            llm.generate([[1, 2, 3]], SamplingParams(max_tokens=4))
        assert isinstance(err.value.__cause__, LayoutUnavailable)
        assert "ctx.host.seq_lens does not exist in a captured step" in str(err.value.__cause__)


def test_linear_adds_its_bias_in_32_bit_on_every_route():
    """A projection's bias is float32 and joins the 32-bit sum before the one rounding, whichever
    kernel ``route`` picks for the row count (the weight-streaming kernel, the tcgen05 kernel,
    the library). Inputs that make the difference visible: the product cancels the bias's
    16-bit part exactly, so the result is the part of the bias that bfloat16 cannot hold; a
    route that rounds the bias first gives zero instead."""
    from tokenomos_b200.parts.linear import Linear

    N, K = 64, 8192
    g = torch.Generator().manual_seed(3)
    bias = (1.0 + 0.5 * torch.rand(N, generator=g)).float()
    coarse = bias.to(torch.bfloat16)
    w = torch.zeros(N, K, dtype=torch.bfloat16)
    w[:, 0] = -coarse                                  # x = e_0 makes the product -bf16(bias)
    lin = Linear(w.cuda(), bias.cuda())
    want = (bias.double() - coarse.double())
    assert want.abs().min().item() > 0
    for rows, route in ((1, "skinny"), (8, "skinny"), (16, "tc"), (65, "library")):
        x = torch.zeros(rows, K, dtype=torch.bfloat16)
        x[:, 0] = 1.0
        got = lin(x.cuda()).double().cpu()
        assert lin.routed.get(route, 0) > 0, (rows, route, lin.routed)
        err = (got - want[None]).abs().max().item()
        assert err <= 2 ** -8 * want.abs().max().item(), (rows, route, err)
        got32 = lin(x.cuda(), out_dtype=torch.float32).double().cpu()
        assert (got32 - want[None]).abs().max().item() <= 1e-6, (rows, route)
