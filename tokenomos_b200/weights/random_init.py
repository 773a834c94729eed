"""Random weights from a configuration and a seed: either a real model folder (``config.json``
+ ``model.safetensors``, so that the loader path is the one exercised) or tensors in memory.

The reference has no such mode (its benches load real checkpoints and randomise the prompts,
Tokenomos bench/decode.py:90-95); this one follows the benchmark configurations' wording:
matrices, embeddings, conv taps and biases ``N(0, std)``, norm weights ``1`` or
``1 + N(0, norm_std)``. Tensors are drawn in the fixed order of the model's declaration from one
generator, so a seed names one model on any machine.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from tokenomos_b200.parts.spec import ROLE_NORM, ROLE_TABLE, TensorDecl


def random_tensors(decls: list[TensorDecl], seed: int, std: float = 0.02, norm_std: float = 0.0,
                   dtype: torch.dtype = torch.float32, device="cpu",
                   include_optional: bool = False) -> dict[str, torch.Tensor]:
    """Draw every declared tensor. Values are drawn in float32 and rounded once to ``dtype``
    (so a bfloat16 folder read back in float32 holds exactly the bfloat16 values)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for d in decls:
        if d.optional and not include_optional:
            continue
        if d.role == ROLE_TABLE:
            out[d.name] = torch.zeros(d.shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(d.shape, generator=gen, dtype=torch.float32, device=device)
        if d.role == ROLE_NORM:
            t = 1.0 + t * norm_std
        else:
            t = t * std
        out[d.name] = t.to(dtype)
    return out


def write_model_folder(folder: str | Path, config: dict, seed: int, std: float = 0.02,
                       norm_std: float = 0.0, dtype: torch.dtype = torch.float32) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json dict whose
    ``architectures`` names a registered architecture)."""
    from tokenomos_b200 import models  # late: models imports the parts, which import the kernels

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = models.architecture_of(config)
    cfg = arch.config_class.from_dict(config)
    spec = arch.declare(cfg)
    tensors = random_tensors(spec.tensor_decls(), seed, std, norm_std, dtype)
    stored = dict(config)
    stored.setdefault("torch_dtype", str(dtype).replace("torch.", ""))
    (folder / "config.json").write_text(json.dumps(stored, indent=1), "utf-8")
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
