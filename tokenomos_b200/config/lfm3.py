"""Typed configuration of the LFM3 hybrid conv text decoder, read from ``config.json``.

Every size and constant the model uses comes from here: nothing is hard-coded in the parts or
the kernels. The keys follow the reference's declaration (``models/lfm3/arch.py:57-131`` of
Tokenomos reads ``norm_eps``, ``head_dim``, ``rope_parameters``, ``layer_types``, ``conv_bias``,
``num_attention_heads``, ``num_key_value_heads``, ``sliding_window``, ``use_sandwich_norm``), and
its checkpoint reader (``models/load/checkpoint.py:156-165``: ``text_config`` if present, the
top-level ``tie_word_embeddings`` wins). Spellings the benchmark configurations use are accepted
beside them: a top-level ``rope_theta`` instead of ``rope_parameters``, ``tie_embedding`` for
``tie_word_embeddings``, ``head_dim`` defaulting to ``hidden_size / num_attention_heads``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

LAYER_KINDS = ("conv", "full_attention", "sliding_attention")


class ConfigError(ValueError):
    """A ``config.json`` that cannot describe a model: the message names every fault found."""


@dataclass(frozen=True)
class RopeParams:
    """Rotary parameters of one attention kind (``rope_parameters[kind]`` in config.json)."""

    theta: float
    partial_rotary_factor: float = 1.0

    def angles(self, head_dim: int) -> int:
        """Number of non-zero frequencies: the rest of ``head_dim // 2`` rotate by zero."""
        return int(self.partial_rotary_factor * head_dim) // 2


@dataclass(frozen=True)
class Lfm3Config:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    layer_types: tuple[str, ...]
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    norm_eps: float
    conv_L_cache: int
    conv_bias: bool
    tie_embedding: bool
    rope: dict[str, RopeParams] = field(default_factory=dict)
    sliding_window: int | None = None
    use_sandwich_norm: bool = False
    # None: decided by the checkpoint (present iff ``gate_proj`` tensors are stored)
    attention_gate: bool | None = None

    # ---- reading ----

    @classmethod
    def from_dict(cls, raw: dict) -> "Lfm3Config":
        """Build from a parsed ``config.json``; raises ``ConfigError`` listing every fault."""
        text = raw.get("text_config", raw)
        errors: list[str] = []

        def need(key: str, kind):
            if key not in text:
                errors.append(f"missing key {key!r}")
                return None
            v = text[key]
            if kind is int and (isinstance(v, bool) or not isinstance(v, int)):
                errors.append(f"{key!r} must be an integer, got {v!r}")
                return None
            if kind is float and (isinstance(v, bool) or not isinstance(v, (int, float))):
                errors.append(f"{key!r} must be a number, got {v!r}")
                return None
            return v

        archs = raw.get("architectures") or text.get("architectures")
        if not archs:
            errors.append("missing key 'architectures'")
            arch = ""
        else:
            arch = archs[0]
        d = need("hidden_size", int)
        n_layers = need("num_hidden_layers", int)
        heads = need("num_attention_heads", int)
        kv_heads = need("num_key_value_heads", int)
        inter = need("intermediate_size", int)
        vocab = need("vocab_size", int)
        eps = need("norm_eps", float)
        width = need("conv_L_cache", int)
        kinds = text.get("layer_types")
        if kinds is None:
            errors.append("missing key 'layer_types'")
            kinds = []
        elif not isinstance(kinds, list) or not all(isinstance(k, str) for k in kinds):
            errors.append("'layer_types' must be a list of strings")
            kinds = []
        for i, k in enumerate(kinds):
            if k not in LAYER_KINDS:
                errors.append(f"layer_types[{i}] = {k!r}: known kinds are {list(LAYER_KINDS)}")
        if n_layers is not None and kinds and n_layers != len(kinds):
            errors.append(f"num_hidden_layers = {n_layers} but layer_types has {len(kinds)} entries")

        head_dim = text.get("head_dim")
        if head_dim is None and d is not None and heads:
            if d % heads:
                errors.append(f"hidden_size {d} is not divisible by num_attention_heads {heads}")
            head_dim = d // heads
        if heads is not None and kv_heads is not None and (kv_heads < 1 or heads % kv_heads):
            errors.append(
                f"num_key_value_heads {kv_heads} must divide num_attention_heads {heads}"
            )
        if isinstance(head_dim, int) and head_dim % 2:
            errors.append(f"head_dim {head_dim} must be even (rotate-half RoPE)")
        if width is not None and width < 2:
            errors.append(f"conv_L_cache {width} must be at least 2")
        for name, v in (("hidden_size", d), ("intermediate_size", inter), ("vocab_size", vocab),
                        ("num_attention_heads", heads)):
            if v is not None and v < 1:
                errors.append(f"{name} {v} must be positive")
        if eps is not None and eps <= 0:
            errors.append(f"norm_eps {eps} must be positive")

        # rotary: per attention kind, or one top-level theta for all kinds
        rope: dict[str, RopeParams] = {}
        attn_kinds = sorted({k for k in kinds if k != "conv" and k in LAYER_KINDS})
        params = text.get("rope_parameters")
        if params is not None:
            # either {kind: {...}} or one flat {rope_theta: ...} for every kind
            flat = "rope_theta" in params
            for kind in attn_kinds:
                p = params if flat else params.get(kind)
                if p is None:
                    errors.append(f"rope_parameters has no entry for {kind!r}")
                    continue
                if p.get("rope_type", "default") != "default":
                    errors.append(f"rope_parameters[{kind!r}]: rope_type {p['rope_type']!r} "
                                  "(only 'default' is built)")
                if "rope_theta" not in p:
                    errors.append(f"rope_parameters[{kind!r}] lacks 'rope_theta'")
                    continue
                rope[kind] = RopeParams(float(p["rope_theta"]),
                                        float(p.get("partial_rotary_factor", 1.0)))
        elif "rope_theta" in text:
            for kind in attn_kinds:
                rope[kind] = RopeParams(float(text["rope_theta"]),
                                        float(text.get("partial_rotary_factor", 1.0)))
        elif attn_kinds:
            errors.append("missing key 'rope_theta' (or 'rope_parameters')")
        for kind, p in rope.items():
            if not (0.0 < p.partial_rotary_factor <= 1.0):
                errors.append(f"partial_rotary_factor {p.partial_rotary_factor} of {kind!r} "
                              "must be in (0, 1]")
            if p.theta <= 0:
                errors.append(f"rope_theta {p.theta} of {kind!r} must be positive")

        window = text.get("sliding_window")
        if "sliding_attention" in kinds:
            if not isinstance(window, int) or isinstance(window, bool) or window < 1:
                errors.append("layer_types names 'sliding_attention' but 'sliding_window' is "
                              f"{window!r}")

        if "tie_word_embeddings" in raw:
            tied = raw["tie_word_embeddings"]
        elif "tie_embedding" in raw:
            tied = raw["tie_embedding"]
        else:
            tied = text.get("tie_word_embeddings", text.get("tie_embedding", True))

        if errors:
            raise ConfigError("config.json: " + "; ".join(errors))
        return cls(
            architecture=arch,
            hidden_size=d,
            num_hidden_layers=n_layers,
            layer_types=tuple(kinds),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=int(head_dim),
            intermediate_size=inter,
            vocab_size=vocab,
            norm_eps=float(eps),
            conv_L_cache=width,
            conv_bias=bool(text.get("conv_bias", False)),
            tie_embedding=bool(tied),
            rope=rope,
            sliding_window=window if isinstance(window, int) else None,
            use_sandwich_norm=bool(text.get("use_sandwich_norm", False)),
            attention_gate=text.get("attention_gate"),
        )

    @classmethod
    def from_folder(cls, path: str | Path) -> "Lfm3Config":
        return cls.from_dict(json.loads((Path(path) / "config.json").read_text("utf-8")))

    # ---- writing (the random-weights mode writes a real model folder) ----

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": "lfm3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "layer_types": list(self.layer_types),
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "norm_eps": self.norm_eps,
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": self.conv_bias,
            "tie_word_embeddings": self.tie_embedding,
            "use_sandwich_norm": self.use_sandwich_norm,
            "rope_parameters": {
                kind: {
                    "rope_type": "default",
                    "rope_theta": p.theta,
                    "partial_rotary_factor": p.partial_rotary_factor,
                }
                for kind, p in self.rope.items()
            },
        }
        if self.sliding_window is not None:
            out["sliding_window"] = self.sliding_window
        if self.attention_gate is not None:
            out["attention_gate"] = self.attention_gate
        return out

    # ---- derived ----

    @property
    def kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def attention_layers(self) -> list[int]:
        return [i for i, k in enumerate(self.layer_types) if k != "conv"]
