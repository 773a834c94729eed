"""Toy parts and a toy architecture, defined in the tests and registered with the framework's
registries without touching its files: what a user who adds a mixer, a feed-forward, a
position encoding or a state kind writes. They are slow torch code on purpose (the point is the
interface, not the kernels) and never become anybody's model.

- ``EmaMixerHost``: an exponential moving average over the sequence with one state row per
  request, planned on the host from ``ctx.host``'s lists, so it is not ``capture_safe``.
- ``EmaMixerDevice``: the same mixer reading the layout from the context's device tensors
  only: ``capture_safe``, so its model runs through captured CUDA graphs. Its state comes from
  a spec class of its own (``RunningState``), which the cache manager has never heard of.
- ``EmaMixerLying``: the host form that claims to be ``capture_safe``: must fail loudly.
- ``RoutedFFN``: every token goes to one of three experts (router in 32-bit).
- ``ScaledRope``: rotary angles of ``position / factor``.
- ``LearnedPosition``: no rotation at all: a learned row per position is added to every query
  and key head before their norm; a position part with a tensor of its own.

``ToyArch`` assembles them by config keys; ``toy_forward`` is its plain float64 restatement.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

import plain_lfm3
from tokenomos_b200 import models, ops
from tokenomos_b200.parts.contract import HeadLayout, SlotState, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import register
from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_NORM, ROLE_VECTOR, BlockSpec, LayerCall,
                                       ModelSpec, PartSpec, TensorDecl)

EXPERTS, FACTOR, THETA, MAX_POS = 3, 4.0, 100.0, 96


# ---- state of a kind the framework does not ship ----------------------------------------------

@dataclass(frozen=True)
class RunningState:
    """One float32 row per request, described to the cache manager by attributes alone."""

    width: int
    storage = "slot"
    dtype = torch.float32

    @property
    def shape(self) -> tuple[int, ...]:
        return (self.width,)


# ---- mixers -----------------------------------------------------------------------------------

class EmaMixerHost:
    def __init__(self, decay: torch.Tensor):
        self.decay = torch.sigmoid(decay)          # [width], float32

    def state_specs(self):
        return {"ema": SlotState((self.decay.numel(),), torch.float32)}

    def forward(self, x, ctx: StepContext, call: int):
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


class EmaMixerLying(EmaMixerHost):
    capture_safe = True          # not true: forward reads ctx.host's lists


class EmaMixerDevice:
    """The same recurrence with the batch read from device tensors: token t belongs to sequence
    ``tok_seq[t]`` whose state row is ``seq_slot[...]``; a token at position 0 starts from zero.
    The number of tokens is the step's (or the captured shape's) capacity; padded tokens belong
    to a dummy sequence on the null row."""

    capture_safe = True

    def __init__(self, decay: torch.Tensor):
        self.decay = torch.sigmoid(decay)

    def state_specs(self):
        return {"ema": RunningState(self.decay.numel())}

    def forward(self, x, ctx: StepContext, call: int):
        state = ctx.states[(call, "ema")]
        slots = ctx.seq_slot.long()[ctx.tok_seq.long().clamp(max=ctx.seq_slot.numel() - 1)]
        fresh = (ctx.positions == 0)
        out = torch.empty_like(x)
        for t in range(x.shape[0]):
            slot = slots[t:t + 1]
            before = torch.where(fresh[t], torch.zeros_like(state[0]), state.index_select(0, slot)[0])
            run = self.decay * before + (1 - self.decay) * x[t].float()
            out[t] = run.to(x.dtype)
            state.index_copy_(0, slot, run[None])
        return out


# ---- feed-forward -----------------------------------------------------------------------------

class RoutedFFN:
    """Top-1 routing: every expert runs on every token and a mask keeps the chosen one's output,
    which costs three times the work and needs no list of rows on the host."""

    capture_safe = True

    def __init__(self, router: torch.Tensor, experts: list):
        self.router = router.float()                      # [E, width]
        self.experts = experts                            # [(gate_up Linear, down Linear)]

    def forward(self, x):
        probs = torch.softmax(x.float() @ self.router.T, dim=-1)
        weight, choice = probs.max(dim=-1)
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e, (gate_up, down) in enumerate(self.experts):
            y = down(ops.swiglu(gate_up(x)))
            out += torch.where((choice == e)[:, None], weight[:, None] * y.float(), 0.0)
        return out.to(x.dtype)


# ---- position encodings -----------------------------------------------------------------------

class ScaledRope:
    capture_safe = True

    def __init__(self, head_dim: int, theta: float, factor: float, device):
        idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (theta ** (idx / head_dim)) / factor).to(device).contiguous()

    def encode_qk(self, qkv, ctx: StepContext, heads: HeadLayout, pool, table):
        return ops.qk_norm_rope_write(qkv, pool, heads.q_norm, heads.k_norm, heads.eps, self.inv_freq,
                                      ctx.positions, ctx.tok_seq, table, heads.heads, heads.kv_heads,
                                      heads.head_dim, ctx.page_size)


class LearnedPosition:
    """``q_h += table[pos]`` and ``k_h += table[pos]`` for every head, then the heads' norms; no
    rotation (the framework's kernel is asked for angle 0 and does the norm and the cache write)."""

    capture_safe = True

    def __init__(self, table: torch.Tensor, head_dim: int):
        self.table = table                                               # [MAX_POS, head_dim]
        self.no_rotation = torch.zeros(head_dim // 2, dtype=torch.float32, device=table.device)

    def encode_qk(self, qkv, ctx: StepContext, heads: HeadLayout, pool, table):
        H, Hkv, D = heads.heads, heads.kv_heads, heads.head_dim
        rows = self.table.index_select(0, ctx.positions.long().clamp(max=self.table.shape[0] - 1))
        moved = qkv.contiguous().clone()
        moved[:, :(H + Hkv) * D] += rows.to(qkv.dtype).repeat(1, H + Hkv)
        return ops.qk_norm_rope_write(moved, pool, heads.q_norm, heads.k_norm, heads.eps,
                                      self.no_rotation, ctx.positions, ctx.tok_seq, table, H, Hkv, D,
                                      ctx.page_size)


def _build_routed(params, tensors, rt):
    experts = [(Linear.fused([tensors[f"gate{e}"], tensors[f"up{e}"]]), Linear(tensors[f"down{e}"]))
               for e in range(params["experts"])]
    return RoutedFFN(tensors["router"], experts)


register("mixer", "toy_ema_host", lambda params, tensors, rt: EmaMixerHost(tensors["decay"]))
register("mixer", "toy_ema_device", lambda params, tensors, rt: EmaMixerDevice(tensors["decay"]))
register("mixer", "toy_ema_lying", lambda params, tensors, rt: EmaMixerLying(tensors["decay"]))
register("feed_forward", "toy_routed", _build_routed)
register("position", "toy_scaled_rope",
         lambda params, tensors, rt: ScaledRope(params["head_dim"], params["theta"], params["factor"], rt.device))
register("position", "toy_learned",
         lambda params, tensors, rt: LearnedPosition(tensors["table"], params["head_dim"]))


# ---- the architecture -------------------------------------------------------------------------

class ToyConfig:
    def __init__(self, raw: dict):
        self.raw = raw
        for key in ("width", "vocab_size", "layers", "eps", "mixer", "ffn"):
            setattr(self, key, raw[key])
        self.heads, self.kv_heads, self.head_dim = raw.get("heads", 4), raw.get("kv_heads", 2), raw.get("head_dim", 16)
        self.inter = raw.get("inter", 2 * raw["width"])
        self.embed_scale, self.logit_softcap = raw.get("embed_scale"), raw.get("logit_softcap")
        self.suppress = tuple(raw.get("suppress", ()))

    @classmethod
    def from_dict(cls, raw: dict) -> "ToyConfig":
        return cls(raw)


class ToyArch:
    """``mixer``: ``ema_host`` | ``ema_device`` | ``ema_lying`` | ``attention_scaled`` |
    ``attention_learned``; ``ffn``: ``swiglu`` | ``routed``."""

    names = ("ToyForCausalLM",)
    config_class = ToyConfig

    def declare(self, c: ToyConfig, tensor_names=()) -> ModelSpec:
        d = c.width

        def norm(name: str, n: int) -> PartSpec:
            return PartSpec("rmsnorm", {"eps": c.eps}, {"weight": TensorDecl(f"{name}.weight", (n,), ROLE_NORM)})

        blocks = []
        for i in range(c.layers):
            p = f"toy.{i}."
            if c.mixer.startswith("ema_"):
                mixer = PartSpec(f"toy_{c.mixer}", {}, {"decay": TensorDecl(f"{p}decay", (d,), ROLE_VECTOR)})
            else:
                H, Hkv, D = c.heads, c.kv_heads, c.head_dim
                tensors = {"q": TensorDecl(f"{p}q.weight", (H * D, d)), "k": TensorDecl(f"{p}k.weight", (Hkv * D, d)),
                           "v": TensorDecl(f"{p}v.weight", (Hkv * D, d)), "o": TensorDecl(f"{p}o.weight", (d, H * D)),
                           "q_norm": TensorDecl(f"{p}qn.weight", (D,), ROLE_NORM),
                           "k_norm": TensorDecl(f"{p}kn.weight", (D,), ROLE_NORM)}
                if c.mixer == "attention_scaled":
                    position = {"kind": "toy_scaled_rope", "params": {"head_dim": D, "theta": THETA, "factor": FACTOR}}
                else:
                    position = {"kind": "toy_learned", "params": {"head_dim": D}}
                    tensors["position.table"] = TensorDecl(f"{p}pos.table", (MAX_POS, D), ROLE_VECTOR)
                mixer = PartSpec("attention", {"heads": H, "kv_heads": Hkv, "head_dim": D, "eps": c.eps,
                                               "window": None, "position": position}, tensors)
            if c.ffn == "routed":
                ffn_tensors = {"router": TensorDecl(f"{p}router.weight", (EXPERTS, d))}
                for e in range(EXPERTS):
                    ffn_tensors[f"gate{e}"] = TensorDecl(f"{p}e{e}.w1.weight", (c.inter, d))
                    ffn_tensors[f"up{e}"] = TensorDecl(f"{p}e{e}.w3.weight", (c.inter, d))
                    ffn_tensors[f"down{e}"] = TensorDecl(f"{p}e{e}.w2.weight", (d, c.inter))
                ffn = PartSpec("toy_routed", {"experts": EXPERTS}, ffn_tensors)
            else:
                ffn = PartSpec("swiglu", {}, {"gate": TensorDecl(f"{p}w1.weight", (c.inter, d)),
                                              "up": TensorDecl(f"{p}w3.weight", (c.inter, d)),
                                              "down": TensorDecl(f"{p}w2.weight", (d, c.inter))})
            blocks.append(BlockSpec("prenorm", {
                "mixer": mixer, "ffn": ffn, "pre_mixer_norm": norm(f"{p}n1", d), "pre_ffn_norm": norm(f"{p}n2", d),
                "post_mixer_norm": None, "post_ffn_norm": None}))
        return ModelSpec(d, c.vocab_size, TensorDecl("toy.embed.weight", (c.vocab_size, d), ROLE_EMBEDDING),
                         tuple(blocks), tuple(LayerCall(i) for i in range(c.layers)), norm("toy.final", d), None,
                         embed_scale=c.embed_scale, logit_softcap=c.logit_softcap, suppress=tuple(c.suppress))


models.register(ToyArch())


def toy_config(mixer: str, ffn: str, **over) -> dict:
    raw = {"architectures": ["ToyForCausalLM"], "width": 40, "vocab_size": 60, "layers": 2, "eps": 1e-5,
           "heads": 4, "kv_heads": 2, "head_dim": 16, "inter": 24, "mixer": mixer, "ffn": ffn}
    raw.update(over)
    return raw


# ---- the plain restatement --------------------------------------------------------------------

def toy_forward(raw: dict, w: dict, ids: list[int]) -> torch.Tensor:
    """Float64 logits [T, vocab] of the toy model on one whole sequence (``w``: name -> float64)."""
    c = ToyConfig(raw)
    T, d = len(ids), c.width
    H, Hkv, D = c.heads, c.kv_heads, c.head_dim
    r = w["toy.embed.weight"][ids]
    if c.embed_scale is not None:
        r = r * c.embed_scale
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for i in range(c.layers):
        p = f"toy.{i}."
        x = plain_lfm3.rmsnorm(r, w[f"{p}n1.weight"], c.eps)
        if c.mixer.startswith("ema_"):
            decay = torch.sigmoid(w[f"{p}decay"].float()).double()
            run, m = torch.zeros(d, dtype=torch.float64), []
            for t in range(T):
                run = decay * run + (1 - decay) * x[t]
                m.append(run)
            r = r + torch.stack(m)
        else:
            q = (x @ w[f"{p}q.weight"].T).view(T, H, D)
            k = (x @ w[f"{p}k.weight"].T).view(T, Hkv, D)
            if c.mixer == "attention_learned":
                rows = w[f"{p}pos.table"][:T]
                q, k = q + rows[:, None, :], k + rows[:, None, :]
            q = plain_lfm3.rmsnorm(q, w[f"{p}qn.weight"], c.eps)
            k = plain_lfm3.rmsnorm(k, w[f"{p}kn.weight"], c.eps)
            if c.mixer == "attention_scaled":
                cos, sin = plain_lfm3.rope_tables(torch.arange(T) / FACTOR, D, D // 2, THETA, torch.float64)
                q, k = plain_lfm3.rotate(q, cos, sin), plain_lfm3.rotate(k, cos, sin)
            k = k.repeat_interleave(H // Hkv, 1)
            v = (x @ w[f"{p}v.weight"].T).view(T, Hkv, D).repeat_interleave(H // Hkv, 1)
            sc = (torch.einsum("ihd,jhd->hij", q, k) * D ** -0.5).masked_fill(~causal[None], float("-inf"))
            r = r + torch.einsum("hij,jhd->ihd", sc.softmax(-1), v).reshape(T, H * D) @ w[f"{p}o.weight"].T
        x = plain_lfm3.rmsnorm(r, w[f"{p}n2.weight"], c.eps)
        if c.ffn == "routed":
            probs = torch.softmax(x @ w[f"{p}router.weight"].T, dim=-1)
            weight, choice = probs.max(dim=-1)
            f = torch.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                g, u = x[t] @ w[f"{p}e{e}.w1.weight"].T, x[t] @ w[f"{p}e{e}.w3.weight"].T
                f[t] = weight[t] * ((torch.nn.functional.silu(g) * u) @ w[f"{p}e{e}.w2.weight"].T)
            r = r + f
        else:
            r = r + plain_lfm3.swiglu(x, w, p, torch.float64)
    logits = plain_lfm3.rmsnorm(r, w["toy.final.weight"], c.eps) @ w["toy.embed.weight"].T
    if c.logit_softcap is not None:
        logits = c.logit_softcap * torch.tanh(logits / c.logit_softcap)
    if c.suppress:
        logits[:, list(c.suppress)] = float("-inf")
    return logits
