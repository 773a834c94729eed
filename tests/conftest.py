"""Shared test set-up: the ``gpu`` marker, the two tiny configurations, model folders made in
temporary places, and the tolerances every comparison uses."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations of the architecture that differ in every size and option: head counts
# and groups, sizes that are no power of two, number of layers, vocabulary, eps, conv width and
# bias, tying, rotary base, page size; B also has sliding-window layers with a partial rotation,
# sandwich norms and the attention gate.
TINY_A = {
    "architectures": ["Lfm3ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 4,
    "layer_types": ["conv", "conv", "full_attention", "conv"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 192, "vocab_size": 512, "rope_theta": 10000.0, "norm_eps": 1e-5,
    "conv_L_cache": 3, "conv_bias": False, "tie_embedding": True,
}
TINY_B = {
    "architectures": ["Lfm3ForCausalLM"], "hidden_size": 96, "num_hidden_layers": 6,
    "layer_types": ["conv", "full_attention", "conv", "conv", "full_attention", "full_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 24,
    "intermediate_size": 256, "vocab_size": 1000, "rope_theta": 1000000.0, "norm_eps": 1e-6,
    "conv_L_cache": 4, "conv_bias": True, "tie_embedding": False,
}
# a third one for what A and B do not have: a window, partial rotation, sandwich norms, the gate,
# 3 query heads per KV head, a page size that does not divide the window
TINY_C = {
    "architectures": ["Lfm3ForCausalLM"], "hidden_size": 80, "num_hidden_layers": 5,
    "layer_types": ["sliding_attention", "conv", "full_attention", "sliding_attention", "conv"],
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
    "intermediate_size": 112, "vocab_size": 300, "norm_eps": 1e-5, "conv_L_cache": 2,
    "conv_bias": True, "tie_word_embeddings": True, "sliding_window": 11,
    "use_sandwich_norm": True, "attention_gate": True,
    "rope_parameters": {
        "full_attention": {"rope_type": "default", "rope_theta": 50000.0},
        "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0,
                              "partial_rotary_factor": 0.5},
    },
}
# a fourth one whose attention takes the tensor-core kernels in bfloat16 (head size 64, groups of
# four), with a window that spans several pages
TINY_D = {
    "architectures": ["Lfm3ForCausalLM"], "hidden_size": 128, "num_hidden_layers": 4,
    "layer_types": ["full_attention", "conv", "sliding_attention", "full_attention"],
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 160, "vocab_size": 400, "rope_theta": 500000.0, "norm_eps": 1e-5,
    "conv_L_cache": 3, "conv_bias": False, "tie_embedding": True, "sliding_window": 40,
}
TINY = {
    "A": dict(config=TINY_A, seed=0, std=0.02, norm_std=0.0, page=16),
    "B": dict(config=TINY_B, seed=1, std=0.05, norm_std=0.1, page=8),
    "C": dict(config=TINY_C, seed=2, std=0.08, norm_std=0.2, page=4),
    "D": dict(config=TINY_D, seed=3, std=0.06, norm_std=0.1, page=16),
}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> {dtype -> folder}: each tiny model written once per stored dtype. The bfloat16
    folder holds the float32 folder's values rounded, so both work dtypes read the same model
    when they read the bfloat16 one."""
    from tokenomos_b200.weights import write_model_folder

    out = {}
    for name, case in TINY.items():
        out[name] = {}
        for dtype in (torch.float32, torch.bfloat16):
            folder = tmp_path_factory.mktemp(f"tiny_{name}_{str(dtype).split('.')[-1]}")
            write_model_folder(folder, case["config"], case["seed"], case["std"],
                               case["norm_std"], dtype)
            out[name][dtype] = folder
    return out


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
