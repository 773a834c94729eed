"""Typed configuration and the architecture registry (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C
from tokenomos_b200 import models
from tokenomos_b200.config import ConfigError, Lfm3Config


def test_reads_every_size_from_config():
    a, b = Lfm3Config.from_dict(TINY_A), Lfm3Config.from_dict(TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 4, 1, 24)
    assert a.conv_L_cache == 3 and b.conv_L_cache == 4
    assert a.tie_embedding and not b.tie_embedding
    assert not a.conv_bias and b.conv_bias
    assert a.rope["full_attention"].theta == 10000.0 and b.rope["full_attention"].theta == 1e6
    assert a.norm_eps == 1e-5 and b.norm_eps == 1e-6
    assert a.attention_layers() == [2] and b.attention_layers() == [1, 4, 5]


def test_head_dim_defaults_to_width_over_heads():
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert Lfm3Config.from_dict(raw).head_dim == 16


def test_rope_parameters_per_kind_and_partial_rotation():
    c = Lfm3Config.from_dict(TINY_C)
    assert c.rope["sliding_attention"].angles(c.head_dim) == 8
    assert c.rope["full_attention"].angles(c.head_dim) == 16
    assert c.sliding_window == 11 and c.use_sandwich_norm and c.attention_gate is True


def test_text_config_nesting_and_top_level_tie_flag_wins():
    raw = {"architectures": ["Lfm3VlForConditionalGeneration"], "tie_word_embeddings": False,
           "text_config": {k: v for k, v in TINY_A.items() if k != "architectures"}}
    c = Lfm3Config.from_dict(raw)
    assert c.hidden_size == 64 and c.tie_embedding is False


def test_round_trip_through_to_dict():
    c = Lfm3Config.from_dict(TINY_C)
    assert Lfm3Config.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change, needle", [
    ({"layer_types": ["conv", "attn", "conv", "conv"]}, "layer_types[1]"),
    ({"num_hidden_layers": 5}, "num_hidden_layers = 5"),
    ({"num_key_value_heads": 3}, "must divide"),
    ({"conv_L_cache": 1}, "at least 2"),
    ({"head_dim": 15}, "must be even"),
    ({"norm_eps": 0}, "norm_eps"),
    ({"hidden_size": "64"}, "must be an integer"),
])
def test_faults_are_named(change, needle):
    with pytest.raises(ConfigError) as e:
        Lfm3Config.from_dict({**TINY_A, **change})
    assert needle in str(e.value)


def test_every_fault_is_listed_at_once():
    raw = {k: v for k, v in TINY_A.items() if k not in ("hidden_size", "vocab_size", "norm_eps")}
    with pytest.raises(ConfigError) as e:
        Lfm3Config.from_dict(raw)
    for key in ("hidden_size", "vocab_size", "norm_eps"):
        assert key in str(e.value)


def test_sliding_layer_needs_a_window_and_rope_needs_default_type():
    raw = dict(TINY_C)
    del raw["sliding_window"]
    with pytest.raises(ConfigError, match="sliding_window"):
        Lfm3Config.from_dict(raw)
    raw = json.loads(json.dumps(TINY_C))
    raw["rope_parameters"]["full_attention"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="rope_type"):
        Lfm3Config.from_dict(raw)


def test_registry_maps_names_to_declarations(tmp_path):
    assert "Lfm3ForCausalLM" in models.ARCHS
    (tmp_path / "config.json").write_text(json.dumps({**TINY_A, "architectures": ["NoSuchModel"]}))
    with pytest.raises(ValueError, match="no declaration for 'NoSuchModel'"):
        models.configure(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    conf = models.configure(tmp_path, work="fp32")
    assert conf.work == torch.float32 and conf.config.hidden_size == 64
    with pytest.raises(ValueError, match="work dtype"):
        models.configure(tmp_path, work="fp8")


def test_declaration_lists_layers_by_config():
    conf = Lfm3Config.from_dict(TINY_B)
    spec = models.ARCHS["Lfm3ForCausalLM"].declare(conf)
    kinds = [b.parts["mixer"].kind for b in spec.blocks]
    assert kinds == ["short_conv", "attention", "short_conv", "short_conv", "attention", "attention"]
    assert spec.head is not None and spec.head.shape == (1000, 96)
    assert [c.block for c in spec.order] == list(range(6))
    names = {d.name for d in spec.tensor_decls()}
    assert "model.layers.0.conv.conv.bias" in names and "model.layers.1.self_attn.q_norm.weight" in names


@pytest.mark.parametrize("change, needle", [({"conv_L_cache": 9}, "9 taps"),
                                            ({"head_dim": 272}, "head size of 272"),
                                            ({"hidden_size": 51264, "num_attention_heads": 4, "head_dim": 16},
                                             "width of 51264")])
def test_sizes_no_kernel_takes_are_refused_when_the_model_is_built(change, needle):
    """What the configuration allows and a kernel does not take is refused when the model is put
    together (``models.load`` / ``from_tensors``), with the limit named, not at the first step."""
    import torch

    from conftest import TINY_A
    from tokenomos_b200 import models
    from tokenomos_b200.weights import random_tensors

    raw = dict(TINY_A, **change)
    conf = models.Configured(models.ARCHS["Lfm3ForCausalLM"], Lfm3Config.from_dict(raw), torch.float32)
    decls = conf.arch.declare(conf.config).tensor_decls()
    tensors = {d.name: torch.zeros(d.shape, device="meta") for d in decls if not d.optional}
    with pytest.raises(ValueError, match=needle):
        models.from_tensors(conf, tensors, device="meta")
