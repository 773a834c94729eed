"""Makes the golden logits under this folder by running KohakuBlueleaf/Tokenomos's own model
code on the CPU (its Triton kernels under the Triton interpreter) on tiny random LFM3 models.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference <Tokenomos checkout>/src

Each case writes ``<name>.json``: the config.json dict, the seed and scales the random weights
were drawn with (``tokenomos_b200.weights.write_model_folder`` regenerates the folder), a
checksum of the weights and the token ids; and ``<name>.safetensors``: the float32 logits
Tokenomos's ``models.reference.forward_logits`` returned, one tensor per sequence. ``tests/test_plain.py`` regenerates each folder in
a temporary place and holds ``tests/plain_lfm3.py`` to these logits.

The reference's declaration always reads ``rope_parameters``, ``head_dim`` and a ``gate_proj``
tensor per attention layer (models/lfm3/arch.py:61-67,98), so the golden configs have them.
Its ``fp32`` work dtype keeps linear weights in float16; to get true float32 weights the script
sets ``floats.matmul`` to the identity before anything is built (core/floats.py:28-35).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import tempfile
import types
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

CASES = {
    # differs from the next in every size and option
    "ref_tiny_a": dict(
        config={
            "architectures": ["Lfm3ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 4,
            "layer_types": ["conv", "conv", "full_attention", "conv"],
            "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
            "intermediate_size": 192, "vocab_size": 512, "norm_eps": 1e-5, "conv_L_cache": 3,
            "conv_bias": False, "tie_word_embeddings": True, "attention_gate": True,
            "rope_parameters": {"full_attention": {"rope_type": "default", "rope_theta": 10000.0}},
        },
        seed=0, std=0.02, norm_std=0.0, lengths=[5, 17, 33]),
    "ref_tiny_b": dict(
        config={
            "architectures": ["Lfm3ForCausalLM"], "hidden_size": 96, "num_hidden_layers": 6,
            "layer_types": ["conv", "full_attention", "conv", "sliding_attention",
                            "full_attention", "sliding_attention"],
            "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 24,
            "intermediate_size": 256, "vocab_size": 1000, "norm_eps": 1e-6, "conv_L_cache": 4,
            "conv_bias": True, "tie_word_embeddings": False, "attention_gate": True,
            "sliding_window": 7, "use_sandwich_norm": True,
            "rope_parameters": {
                "full_attention": {"rope_type": "default", "rope_theta": 1000000.0},
                "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0,
                                      "partial_rotary_factor": 0.5},
            },
        },
        seed=1, std=0.05, norm_std=0.1, lengths=[1, 9, 40]),
}


def weights_checksum(folder: Path) -> str:
    return hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()[:16]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="the src folder of a Tokenomos checkout")
    args = ap.parse_args()
    if os.environ.get("TRITON_INTERPRET") != "1":
        raise SystemExit("run with TRITON_INTERPRET=1: the reference's kernels are Triton")
    sys.path.insert(0, args.reference)
    # the reference's only native module (JSON grammar) is not built here and not needed
    for name in ("tokenomos._rs", "tokenomos._rs.grammar"):
        sys.modules[name] = types.ModuleType(name)
    from tokenomos.core import floats
    floats.matmul = lambda dtype: dtype   # true float32 weights
    from tokenomos import models
    from tokenomos.models import reference

    from tokenomos_b200.weights import write_model_folder

    for name, case in CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_model_folder(Path(tmp) / name, case["config"], case["seed"],
                                        case["std"], case["norm_std"], torch.float32)
            model = models.load(str(folder), "cpu", models.configure(str(folder), work="fp32"))
            gen = torch.Generator().manual_seed(case["seed"] + 100)
            vocab = case["config"]["vocab_size"]
            seqs = [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in case["lengths"]]
            logits = reference.forward_logits(model, seqs, "cpu")
            out = {
                "config": case["config"], "seed": case["seed"], "std": case["std"],
                "norm_std": case["norm_std"], "weights_sha256_16": weights_checksum(folder),
                "ids": seqs,
            }
            (HERE / f"{name}.json").write_text(json.dumps(out, indent=1))
            save_file({f"logits.{i}": t.float().contiguous() for i, t in enumerate(logits)},
                      str(HERE / f"{name}.safetensors"))
            print(name, [tuple(t.shape) for t in logits], float(max(t.abs().max() for t in logits)))


if __name__ == "__main__":
    main()
