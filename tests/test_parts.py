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
    xs = torch.split(x.double(), lens)
    for i, kind in enumerate(s["layer_types"]):
        block = model.blocks[i]
        got = block.mixer.forward(x.cuda(), ctx, i)
        p = f"model.layers.{i}."
        if kind == "conv":
            want = torch.cat([plain_lfm3.short_conv(v, w, f"{p}conv.", s, torch.float64) for v in xs])
        else:
            want = torch.cat([plain_lfm3.attention(v, w, f"{p}self_attn.", s, kind, torch.float64)
                              for v in xs])
        _close(got, want, dtype, f"{name} layer {i} {kind}")
        got = block.ffn.forward(x.cuda())
        _close(got, plain_lfm3.swiglu(x.double(), w, f"{p}feed_forward.", torch.float64), dtype,
               f"{name} layer {i} ffn")
        norm = block.pre_mixer
        _close(norm(x.cuda()), plain_lfm3.rmsnorm(x.double(), w[f"{p}operator_norm.weight"], s["eps"]),
               dtype, f"{name} layer {i} norm")


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


def test_toy_mixer_with_its_own_state_registers_builds_and_steps(tmp_path):
    """A mixer defined here: an exponential moving average over the sequence with one state row
    per request (its running value). It is registered with the parts registry, named by a new
    architecture's declaration, loaded from a model folder and stepped in portions, with no
    change to the framework's files."""
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction
    from tokenomos_b200.parts.contract import SlotState
    from tokenomos_b200.parts.registry import register
    from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_NORM, ROLE_VECTOR, BlockSpec,
                                           LayerCall, ModelSpec, PartSpec, TensorDecl)
    from tokenomos_b200.weights import write_model_folder

    class EmaMixer:
        def __init__(self, decay: torch.Tensor):
            self.decay = torch.sigmoid(decay)          # [width], float32

        def state_specs(self):
            return {"ema": SlotState((self.decay.numel(),), torch.float32)}

        def forward(self, x, ctx, call):
            state = ctx.states[(call, "ema")]
            out = torch.empty_like(x)
            start = 0
            for s, n in enumerate(ctx.host.seq_lens):
                slot = ctx.host.seq_slot[s]
                run = state[slot].clone() if ctx.host.seq_ctx[s] > 0 else torch.zeros_like(state[slot])
                for t in range(start, start + n):
                    run = self.decay * run + (1 - self.decay) * x[t].float()
                    out[t] = run.to(x.dtype)
                state[slot] = run
                start += n
            return out

    register("mixer", "toy_ema", lambda params, tensors, rt: EmaMixer(tensors["decay"]))

    class ToyConfig:
        def __init__(self, width, vocab, layers, eps):
            self.width, self.vocab, self.layers, self.eps = width, vocab, layers, eps

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["width"], raw["vocab_size"], raw["layers"], raw["eps"])

    class ToyArch:
        names = ("ToyEmaForCausalLM",)
        config_class = ToyConfig

        def declare(self, cfg, tensor_names=()):
            def norm(name):
                return PartSpec("rmsnorm", {"eps": cfg.eps},
                                {"weight": TensorDecl(f"{name}.weight", (cfg.width,), ROLE_NORM)})
            blocks = []
            for i in range(cfg.layers):
                p = f"toy.{i}."
                blocks.append(BlockSpec("prenorm", {
                    "mixer": PartSpec("toy_ema", {}, {"decay": TensorDecl(f"{p}decay", (cfg.width,), ROLE_VECTOR)}),
                    "ffn": PartSpec("swiglu", {}, {
                        "gate": TensorDecl(f"{p}w1.weight", (2 * cfg.width, cfg.width)),
                        "up": TensorDecl(f"{p}w3.weight", (2 * cfg.width, cfg.width)),
                        "down": TensorDecl(f"{p}w2.weight", (cfg.width, 2 * cfg.width))}),
                    "pre_mixer_norm": norm(f"{p}n1"), "pre_ffn_norm": norm(f"{p}n2"),
                    "post_mixer_norm": None, "post_ffn_norm": None}))
            return ModelSpec(cfg.width, cfg.vocab,
                             TensorDecl("toy.embed.weight", (cfg.vocab, cfg.width), ROLE_EMBEDDING),
                             tuple(blocks), tuple(LayerCall(i) for i in range(cfg.layers)),
                             norm("toy.final"), None)

    models.register(ToyArch())
    raw = {"architectures": ["ToyEmaForCausalLM"], "width": 24, "vocab_size": 50, "layers": 2, "eps": 1e-5}
    folder = write_model_folder(tmp_path / "toy", raw, seed=4, std=0.3)
    model = models.load(folder, "cuda", models.configure(folder, work="fp32"))
    assert isinstance(model.blocks[0].mixer, EmaMixer)
    cache = CacheManager(model.state_specs(), 4, 8, 3, torch.float32, "cuda", max_len=64)
    assert tuple(cache.states[(1, "ema")].shape) == (4, 24)
    step = StepFunction(model, cache)
    ids = torch.randint(0, 50, (19,)).tolist()
    cache.admit("w")
    whole = step.run([StepEntry("w", ids, list(range(19)))])
    cache.release("w")
    cache.admit("other")      # takes the slot "w" had, and leaves its state behind
    step.run([StepEntry("other", [1, 2, 3], [])])
    cache.admit("p")
    parts = [step.run([StepEntry("p", ids[a:b], list(range(b - a))), StepEntry("other", [7], [])][:1 + (a > 0)])
             for a, b in ((0, 5), (5, 6), (6, 19))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-5)
    # and against a plain restatement of the toy model
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    r = w["toy.embed.weight"][ids]
    for i in range(2):
        p = f"toy.{i}."
        x = plain_lfm3.rmsnorm(r, w[f"{p}n1.weight"], 1e-5)
        decay = torch.sigmoid(w[f"{p}decay"].float()).double()
        run, m = torch.zeros(24, dtype=torch.float64), []
        for t in range(19):
            run = decay * run + (1 - decay) * x[t]
            m.append(run)
        r = r + torch.stack(m)
        x = plain_lfm3.rmsnorm(r, w[f"{p}n2.weight"], 1e-5)
        r = r + plain_lfm3.swiglu(x, w, p, torch.float64)
    want = plain_lfm3.rmsnorm(r, w["toy.final.weight"], 1e-5) @ w["toy.embed.weight"].T
    assert (whole.double().cpu() - want).abs().max().item() < 1e-4 * want.abs().max().item()


def test_toy_routed_ffn_and_toy_position_encoding_register_build_and_step(tmp_path):
    """Two more parts defined here, with no change to the framework's files: a feed-forward that
    routes every token to one of three small experts (router logits and probabilities in 32-bit)
    and a position encoding (rotary angles of positions divided by a factor), both registered
    with the parts registry and named by a new architecture's declaration beside the framework's
    own attention mixer. The model is loaded from a folder and stepped whole, in portions and
    beside another request; the logits agree with each other and with a plain restatement."""
    from tokenomos_b200 import models, ops
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction
    from tokenomos_b200.parts.linear import Linear
    from tokenomos_b200.parts.registry import register
    from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_NORM, BlockSpec, LayerCall, ModelSpec,
                                           PartSpec, TensorDecl)
    from tokenomos_b200.weights import write_model_folder

    E, FACTOR = 3, 4.0

    class RoutedFFN:
        def __init__(self, router, experts):
            self.router = router.float()                      # [E, width]
            self.experts = experts                            # [(gate_up Linear, down Linear)]

        def forward(self, x):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros_like(x)
            for e, (gate_up, down) in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    y = down(ops.swiglu(gate_up(x[rows].contiguous())))
                    out[rows] = (weight[rows, None] * y.float()).to(x.dtype)
            return out

    def build_routed(params, tensors, rt):
        experts = [(Linear.fused([tensors[f"gate{e}"], tensors[f"up{e}"]]), Linear(tensors[f"down{e}"]))
                   for e in range(params["experts"])]
        return RoutedFFN(tensors["router"], experts)

    class ScaledRope:
        """Rotary tables of ``position / factor``: the kernels multiply positions by
        ``inv_freq``, so dividing the frequencies does it."""

        def __init__(self, head_dim, theta, factor, device):
            idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
            self.inv_freq = (1.0 / (theta ** (idx / head_dim)) / factor).to(device).contiguous()
            self.dim = head_dim

        def tables(self, ctx):
            return self.inv_freq

    register("feed_forward", "toy_routed", build_routed)
    register("position", "toy_scaled_rope",
             lambda params, tensors, rt: ScaledRope(params["head_dim"], params["theta"], params["factor"], rt.device))

    class ToyConfig:
        def __init__(self, raw):
            self.width, self.vocab, self.layers, self.eps = raw["width"], raw["vocab_size"], raw["layers"], raw["eps"]
            self.heads, self.kv_heads, self.head_dim, self.inter = raw["heads"], raw["kv_heads"], raw["head_dim"], raw["inter"]

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

    class ToyArch:
        names = ("ToyRoutedForCausalLM",)
        config_class = ToyConfig

        def declare(self, c, tensor_names=()):
            def norm(name, n):
                return PartSpec("rmsnorm", {"eps": c.eps}, {"weight": TensorDecl(f"{name}.weight", (n,), ROLE_NORM)})
            blocks = []
            for i in range(c.layers):
                p = f"toy.{i}."
                H, Hkv, D, d = c.heads, c.kv_heads, c.head_dim, c.width
                mixer = PartSpec("attention", {
                    "heads": H, "kv_heads": Hkv, "head_dim": D, "eps": c.eps, "window": None,
                    "position": {"kind": "toy_scaled_rope", "params": {"head_dim": D, "theta": 100.0, "factor": FACTOR}},
                }, {"q": TensorDecl(f"{p}q.weight", (H * D, d)), "k": TensorDecl(f"{p}k.weight", (Hkv * D, d)),
                    "v": TensorDecl(f"{p}v.weight", (Hkv * D, d)), "o": TensorDecl(f"{p}o.weight", (d, H * D)),
                    "q_norm": TensorDecl(f"{p}qn.weight", (D,), ROLE_NORM),
                    "k_norm": TensorDecl(f"{p}kn.weight", (D,), ROLE_NORM)})
                ffn_tensors = {"router": TensorDecl(f"{p}router.weight", (E, d))}
                for e in range(E):
                    ffn_tensors[f"gate{e}"] = TensorDecl(f"{p}e{e}.w1.weight", (c.inter, d))
                    ffn_tensors[f"up{e}"] = TensorDecl(f"{p}e{e}.w3.weight", (c.inter, d))
                    ffn_tensors[f"down{e}"] = TensorDecl(f"{p}e{e}.w2.weight", (d, c.inter))
                blocks.append(BlockSpec("prenorm", {
                    "mixer": mixer, "ffn": PartSpec("toy_routed", {"experts": E}, ffn_tensors),
                    "pre_mixer_norm": norm(f"{p}n1", d), "pre_ffn_norm": norm(f"{p}n2", d),
                    "post_mixer_norm": None, "post_ffn_norm": None}))
            return ModelSpec(c.width, c.vocab, TensorDecl("toy.embed.weight", (c.vocab, c.width), ROLE_EMBEDDING),
                             tuple(blocks), tuple(LayerCall(i) for i in range(c.layers)),
                             norm("toy.final", c.width), None)

    models.register(ToyArch())
    raw = {"architectures": ["ToyRoutedForCausalLM"], "width": 40, "vocab_size": 60, "layers": 2, "eps": 1e-5,
           "heads": 4, "kv_heads": 2, "head_dim": 16, "inter": 24}
    folder = write_model_folder(tmp_path / "toy_routed", raw, seed=7, std=0.3)
    model = models.load(folder, "cuda", models.configure(folder, work="fp32"))
    assert isinstance(model.blocks[0].ffn, RoutedFFN)
    assert isinstance(model.blocks[1].mixer.rope, ScaledRope)
    cache = CacheManager(model.state_specs(), 4, 24, 3, torch.float32, "cuda", max_len=64)
    step = StepFunction(model, cache)
    T = 21
    ids = torch.randint(0, 60, (T,)).tolist()
    cache.admit("w")
    whole = step.run([StepEntry("w", ids, list(range(T)))])
    cache.release("w")
    cache.admit("other")
    step.run([StepEntry("other", [1, 2, 3], [])])
    cache.admit("p")
    parts = [step.run([StepEntry("p", ids[a:b], list(range(b - a))), StepEntry("other", [7], [])][:1 + (a > 0)])
             for a, b in ((0, 6), (6, 7), (7, 9), (9, T))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-5)

    # the plain restatement: same formulas, float64, whole sequence
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    H, Hkv, D = 4, 2, 16
    r = w["toy.embed.weight"][ids]
    cos, sin = plain_lfm3.rope_tables(torch.arange(T) / FACTOR, D, D // 2, 100.0, torch.float64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for i in range(2):
        p = f"toy.{i}."
        x = plain_lfm3.rmsnorm(r, w[f"{p}n1.weight"], 1e-5)
        q = plain_lfm3.rmsnorm((x @ w[f"{p}q.weight"].T).view(T, H, D), w[f"{p}qn.weight"], 1e-5)
        k = plain_lfm3.rmsnorm((x @ w[f"{p}k.weight"].T).view(T, Hkv, D), w[f"{p}kn.weight"], 1e-5)
        q, k = plain_lfm3.rotate(q, cos, sin), plain_lfm3.rotate(k, cos, sin).repeat_interleave(H // Hkv, 1)
        v = (x @ w[f"{p}v.weight"].T).view(T, Hkv, D).repeat_interleave(H // Hkv, 1)
        sc = (torch.einsum("ihd,jhd->hij", q, k) * D ** -0.5).masked_fill(~causal[None], float("-inf"))
        r = r + torch.einsum("hij,jhd->ihd", sc.softmax(-1), v).reshape(T, H * D) @ w[f"{p}o.weight"].T
        x = plain_lfm3.rmsnorm(r, w[f"{p}n2.weight"], 1e-5)
        probs = torch.softmax(x @ w[f"{p}router.weight"].T, dim=-1)
        weight, choice = probs.max(dim=-1)
        f = torch.zeros_like(x)
        for t in range(T):
            e = int(choice[t])
            g, u = x[t] @ w[f"{p}e{e}.w1.weight"].T, x[t] @ w[f"{p}e{e}.w3.weight"].T
            f[t] = weight[t] * ((torch.nn.functional.silu(g) * u) @ w[f"{p}e{e}.w2.weight"].T)
        r = r + f
    want = plain_lfm3.rmsnorm(r, w["toy.final.weight"], 1e-5) @ w["toy.embed.weight"].T
    assert (whole.double().cpu() - want).abs().max().item() < 2e-4 * want.abs().max().item()
