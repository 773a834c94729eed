"""The plain implementation against the reference's own code (golden logits made on the CPU by
``tests/golden/make_golden.py``), and against itself where the goldens do not reach."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import pytest
import torch
from safetensors import safe_open

import plain_lfm3
from tokenomos_b200.weights import write_model_folder

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["ref_tiny_a", "ref_tiny_b"])
def test_plain_matches_reference_code(name, tmp_path):
    meta = json.loads((GOLDEN / f"{name}.json").read_text())
    folder = write_model_folder(tmp_path / name, meta["config"], meta["seed"], meta["std"],
                                meta["norm_std"], torch.float32)
    digest = hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()[:16]
    # the only link to the reference's own output must not vanish quietly: if this torch draws
    # other random weights than the one the goldens were made with, remake the goldens
    # (tests/golden/make_golden.py) instead of skipping
    assert digest == meta["weights_sha256_16"], (
        f"{name}: the regenerated weights ({digest}) are not the ones the golden logits were made "
        f"with ({meta['weights_sha256_16']}): rerun tests/golden/make_golden.py")
    config, w = plain_lfm3.read_folder(folder)
    with safe_open(GOLDEN / f"{name}.safetensors", "pt") as f:
        for i, ids in enumerate(meta["ids"]):
            want = f.get_tensor(f"logits.{i}").double()
            got = plain_lfm3.forward_logits(config, w, ids)
            scale = want.abs().max().item()
            assert (got - want).abs().max().item() < 2e-5 * max(scale, 1.0), (name, i)


def test_plain_is_causal_and_prefix_stable(model_folders):
    """Logits at a position do not change when tokens are appended after it."""
    config, w = plain_lfm3.read_folder(model_folders["C"][torch.float32])
    ids = torch.randint(0, config["vocab_size"], (30,)).tolist()
    full = plain_lfm3.forward_logits(config, w, ids)
    short = plain_lfm3.forward_logits(config, w, ids[:19])
    assert (full[:19] - short).abs().max().item() < 1e-10


def test_plain_window_matters(model_folders):
    """Negative control: widening the window changes the logits beyond the window's reach."""
    config, w = plain_lfm3.read_folder(model_folders["C"][torch.float32])
    ids = torch.randint(0, config["vocab_size"], (40,)).tolist()
    base = plain_lfm3.forward_logits(config, w, ids)
    wide = dict(config, sliding_window=1000)
    other = plain_lfm3.forward_logits(wide, w, ids)
    window = config["sliding_window"]
    assert (base[:window] - other[:window]).abs().max().item() < 1e-10
    assert (base[window + 5:] - other[window + 5:]).abs().max().item() > 1e-6


def test_plain_float32_close_to_float64(model_folders):
    config, w = plain_lfm3.read_folder(model_folders["B"][torch.float32])
    ids = torch.randint(0, config["vocab_size"], (25,)).tolist()
    a = plain_lfm3.forward_logits(config, w, ids, torch.float64)
    b = plain_lfm3.forward_logits(config, w, ids, torch.float32).double()
    assert (a - b).abs().max().item() < 1e-4 * a.abs().max().item()
