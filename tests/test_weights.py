"""Weights by tensor name: dtypes kept, one error for every mismatch, random-weights folders."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B
from tokenomos_b200 import models
from tokenomos_b200.config import Lfm3Config
from tokenomos_b200.weights import Checkpoint, WeightError, load_tensors, write_model_folder


def _decls(config):
    return models.ARCHS["Lfm3ForCausalLM"].declare(Lfm3Config.from_dict(config)).tensor_decls()


def test_random_folder_is_reproducible_and_complete(tmp_path):
    a = write_model_folder(tmp_path / "a", TINY_B, seed=7, std=0.05, norm_std=0.1)
    b = write_model_folder(tmp_path / "b", TINY_B, seed=7, std=0.05, norm_std=0.1)
    c = write_model_folder(tmp_path / "c", TINY_B, seed=8, std=0.05, norm_std=0.1)
    ta, tb, tc = (load_file(str(p / "model.safetensors")) for p in (a, b, c))
    assert set(ta) == {d.name for d in _decls(TINY_B) if not d.optional}
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert any(not torch.equal(ta[k], tc[k]) for k in ta)
    w = ta["model.layers.1.self_attn.q_proj.weight"]
    assert abs(w.std().item() - 0.05) < 0.01
    n = ta["model.layers.0.operator_norm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.1 and n.std().item() > 0.01
    assert json.loads((a / "config.json").read_text())["hidden_size"] == 96


def test_dtypes_kept(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_A, seed=0, dtype=torch.bfloat16)
    ckpt = Checkpoint(folder)
    for work in (torch.bfloat16, torch.float32):
        t = load_tensors(ckpt, _decls(TINY_A), work, "cpu")
        assert t["model.embed_tokens.weight"].dtype == work
        assert t["model.layers.2.self_attn.q_proj.weight"].dtype == work
        # vectors (norm weights, conv taps) are float32 whatever the work dtype
        assert t["model.layers.0.operator_norm.weight"].dtype == torch.float32
        assert t["model.layers.0.conv.conv.weight"].dtype == torch.float32
    # bfloat16 values read into float32 are exactly the stored values
    raw = load_file(str(folder / "model.safetensors"))["model.embed_tokens.weight"]
    t = load_tensors(ckpt, _decls(TINY_A), torch.float32, "cpu")
    assert torch.equal(t["model.embed_tokens.weight"], raw.float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_A, seed=0)
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    del tensors["model.layers.1.conv.in_proj.weight"]
    del tensors["model.embedding_norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(3)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    save_file(tensors, str(path))
    with pytest.raises(WeightError) as e:
        load_tensors(Checkpoint(folder), _decls(TINY_A), torch.float32, "cpu")
    msg = str(e.value)
    assert "2 missing" in msg and "model.layers.1.conv.in_proj.weight" in msg
    assert "model.embedding_norm.weight" in msg
    assert "1 unexpected" in msg and "model.layers.9.extra.weight" in msg
    assert "1 with a wrong shape" in msg and "stored [16, 64]" in msg and "[32, 64]" in msg


def test_vision_language_folder_loads_its_text_stack_and_ignores_the_rest(tmp_path):
    """A multimodal folder nests the text stack under ``model.language_model.`` and stores a
    vision tower and a projector beside it; a tied checkpoint may also store ``lm_head.weight``.
    None of those is the text model's business. A stray tensor *under* the text stack's prefix
    still is (checked by adding one: the load must then fail)."""
    folder = write_model_folder(tmp_path / "m", TINY_A, seed=0)
    path = folder / "model.safetensors"
    tensors = {k.replace("model.", "model.language_model.", 1): v for k, v in load_file(str(path)).items()}
    tensors["model.vision_tower.patch_embed.weight"] = torch.zeros(4, 3)
    tensors["model.multi_modal_projector.linear.weight"] = torch.zeros(5)
    tensors["lm_head.weight"] = torch.zeros(TINY_A["vocab_size"], TINY_A["hidden_size"])
    save_file(tensors, str(path))
    cfg = {"architectures": ["Lfm3VlForConditionalGeneration"], "text_config": TINY_A,
           "vision_config": {"hidden_size": 8}}
    (folder / "config.json").write_text(json.dumps(cfg))
    ckpt = Checkpoint(folder)
    arch = models.architecture_of(cfg)
    spec = arch.declare(arch.config_class.from_dict(cfg), ckpt.names())
    assert spec.scope == ("model.language_model.",)
    got = load_tensors(ckpt, spec.tensor_decls(), torch.float32, "cpu", spec.scope)
    assert "model.language_model.embed_tokens.weight" in got and "lm_head.weight" not in got
    assert not any("vision" in k or "projector" in k for k in got)
    tensors["model.language_model.layers.0.stray.weight"] = torch.zeros(2)
    save_file(tensors, str(path))
    with pytest.raises(WeightError, match="1 unexpected: model.language_model.layers.0.stray.weight"):
        load_tensors(Checkpoint(folder), spec.tensor_decls(), torch.float32, "cpu", spec.scope)


def test_conv_width_must_match_config(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_A, seed=0)
    cfg = json.loads((folder / "config.json").read_text())
    cfg["conv_L_cache"] = 4
    (folder / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(WeightError, match="conv.conv.weight"):
        load_tensors(Checkpoint(folder), _decls(cfg), torch.float32, "cpu")


def test_sharded_folder_reads_like_a_single_file(tmp_path):
    folder = write_model_folder(tmp_path / "m", TINY_A, seed=3)
    tensors = load_file(str(folder / "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {k: ("model-00001-of-00002.safetensors" if i < half else
                                "model-00002-of-00002.safetensors") for i, k in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    (folder / "model.safetensors").unlink()
    got = load_tensors(Checkpoint(folder), _decls(TINY_A), torch.float32, "cpu")
    assert all(torch.equal(got[k], tensors[k].float().reshape(got[k].shape)) for k in names)


def test_missing_files_are_named(tmp_path):
    with pytest.raises(FileNotFoundError, match="config.json"):
        Checkpoint(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        Checkpoint(tmp_path)
