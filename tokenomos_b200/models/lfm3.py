"""The LFM3 hybrid conv text decoder as a declaration: configuration -> ``ModelSpec``.

Per layer, ``layer_types[i]`` picks the mixer: ``conv`` a gated short convolution of
``conv_L_cache`` taps, ``full_attention`` / ``sliding_attention`` grouped-query attention with
per-head q/k RMSNorm and rotary encoding (a window of ``sliding_window`` positions on the
sliding ones, an optional per-head sigmoid gate). Every layer has a SwiGLU feed-forward
(``w1`` gate, ``w3`` up, ``w2`` down), pre-norms ``operator_norm`` and ``ffn_norm``, and with
``use_sandwich_norm`` post-norms after the mixer and the feed-forward. Final
``embedding_norm``; the head is the embedding unless untied (``lm_head``).
Tensor names and wiring: Tokenomos models/lfm3/arch.py:49-131.
"""

from __future__ import annotations

from tokenomos_b200.config.lfm3 import Lfm3Config
from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_MATRIX, ROLE_NORM, ROLE_VECTOR,
                                       BlockSpec, LayerCall, ModelSpec, PartSpec, TensorDecl)


class Lfm3:
    names = ("Lfm3ForCausalLM", "Lfm3VlForConditionalGeneration", "Lfm2ForCausalLM")
    config_class = Lfm3Config

    @staticmethod
    def root(tensor_names) -> str:
        """Prefix of the text stack's tensors: a vision-language folder nests it."""
        nested = "model.language_model.embed_tokens.weight"
        return "model.language_model." if nested in tensor_names else "model."

    def declare(self, cfg: Lfm3Config, tensor_names=()) -> ModelSpec:
        """``tensor_names``: the names a model folder holds, when there is one: they settle the
        prefix and whether the attention layers have the optional gate."""
        root = self.root(tensor_names)
        d, D = cfg.hidden_size, cfg.head_dim
        H, Hkv, I, W = (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size,
                        cfg.conv_L_cache)
        gate = cfg.attention_gate
        if gate is None:
            gate = any(n.endswith("self_attn.gate_proj.weight") for n in tensor_names)

        def norm(name: str, width: int) -> PartSpec:
            return PartSpec("rmsnorm", {"eps": cfg.norm_eps},
                            {"weight": TensorDecl(f"{name}.weight", (width,), ROLE_NORM)})

        blocks = []
        for i, kind in enumerate(cfg.layer_types):
            p = f"{root}layers.{i}."
            if kind == "conv":
                c = f"{p}conv."
                tensors = {
                    "in_proj": TensorDecl(f"{c}in_proj.weight", (3 * d, d)),
                    "out_proj": TensorDecl(f"{c}out_proj.weight", (d, d)),
                    "conv": TensorDecl(f"{c}conv.weight", (d, 1, W), ROLE_VECTOR),
                    "in_proj_bias": TensorDecl(f"{c}in_proj.bias", (3 * d,), ROLE_VECTOR, optional=True),
                    "out_proj_bias": TensorDecl(f"{c}out_proj.bias", (d,), ROLE_VECTOR, optional=True),
                }
                if cfg.conv_bias:
                    tensors["conv_bias"] = TensorDecl(f"{c}conv.bias", (d,), ROLE_VECTOR)
                mixer = PartSpec("short_conv", {"dim": d, "width": W}, tensors)
            else:
                a = f"{p}self_attn."
                rope = cfg.rope[kind]
                tensors = {
                    "q": TensorDecl(f"{a}q_proj.weight", (H * D, d)),
                    "k": TensorDecl(f"{a}k_proj.weight", (Hkv * D, d)),
                    "v": TensorDecl(f"{a}v_proj.weight", (Hkv * D, d)),
                    "o": TensorDecl(f"{a}o_proj.weight", (d, H * D)),
                    "q_norm": TensorDecl(f"{a}q_norm.weight", (D,), ROLE_NORM),
                    "k_norm": TensorDecl(f"{a}k_norm.weight", (D,), ROLE_NORM),
                }
                if gate:
                    tensors["gate"] = TensorDecl(f"{a}gate_proj.weight", (H, d))
                mixer = PartSpec(
                    "attention",
                    {
                        "heads": H, "kv_heads": Hkv, "head_dim": D, "eps": cfg.norm_eps,
                        "window": cfg.sliding_window if kind == "sliding_attention" else None,
                        "position": {"kind": "rope",
                                     "params": {"head_dim": D, "angles": rope.angles(D),
                                                "theta": rope.theta}},
                    },
                    tensors)
            f = f"{p}feed_forward."
            ffn = PartSpec("swiglu", {"width": d, "inter": I}, {
                "gate": TensorDecl(f"{f}w1.weight", (I, d)),
                "up": TensorDecl(f"{f}w3.weight", (I, d)),
                "down": TensorDecl(f"{f}w2.weight", (d, I)),
            })
            sandwich = cfg.use_sandwich_norm
            blocks.append(BlockSpec("prenorm", {
                "mixer": mixer,
                "ffn": ffn,
                "pre_mixer_norm": norm(f"{p}operator_norm", d),
                "pre_ffn_norm": norm(f"{p}ffn_norm", d),
                "post_mixer_norm": norm(f"{p}post_operator_norm", d) if sandwich else None,
                "post_ffn_norm": norm(f"{p}post_ffn_norm", d) if sandwich else None,
            }))
        return ModelSpec(
            width=d,
            vocab=cfg.vocab_size,
            embedding=TensorDecl(f"{root}embed_tokens.weight", (cfg.vocab_size, d), ROLE_EMBEDDING),
            blocks=tuple(blocks),
            order=tuple(LayerCall(i) for i in range(len(blocks))),
            final_norm=norm(f"{root}embedding_norm", d),
            head=None if cfg.tie_embedding else TensorDecl("lm_head.weight", (cfg.vocab_size, d),
                                                           ROLE_MATRIX),
            # a vision-language folder also stores its vision tower and projector, and a tied
            # checkpoint may store a copy of the head: neither belongs to the text stack
            scope=(root,) if cfg.tie_embedding else (root, "lm_head."),
        )
