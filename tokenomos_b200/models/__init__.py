"""Architectures: one registry from a folder's ``architectures`` name to its declaration, and
``load``, which builds a folder's model (Tokenomos models/__init__.py:19-85 has the same three
verbs: ``register``, ``configure``, ``load``).

An architecture is an object with ``names`` (the config.json names it serves), ``config_class``
(a typed configuration with ``from_dict``) and ``declare(config, tensor_names) -> ModelSpec``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from tokenomos_b200.models.lfm3 import Lfm3
from tokenomos_b200.parts import build_model
from tokenomos_b200.parts.registry import Runtime, Tuning
from tokenomos_b200.weights.checkpoint import Checkpoint, load_tensors

ARCHS: dict[str, object] = {}

WORK_DTYPES = {
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
    "fp32": torch.float32, "float32": torch.float32,
}


def register(arch) -> None:
    for name in arch.names:
        ARCHS[name] = arch


def architecture_of(raw_config: dict):
    names = raw_config.get("architectures") or raw_config.get("text_config", {}).get("architectures")
    if not names:
        raise ValueError("config.json has no 'architectures' entry")
    if names[0] not in ARCHS:
        raise ValueError(f"no declaration for {names[0]!r}; known: {sorted(ARCHS)}")
    return ARCHS[names[0]]


@dataclass
class Configured:
    """A folder's architecture with its typed configuration and the work dtype chosen."""

    arch: object
    config: object
    work: torch.dtype


def configure(path: str | Path, work: str | torch.dtype | None = None) -> Configured:
    """The declaration of folder ``path``'s architecture. ``work``: ``bf16`` (default) or
    ``fp32``, the storage type of activations, matrices and caches."""
    raw = json.loads((Path(path) / "config.json").read_text("utf-8"))
    arch = architecture_of(raw)
    if isinstance(work, str):
        if work not in WORK_DTYPES:
            raise ValueError(f"work dtype {work!r}; known: {sorted(WORK_DTYPES)}")
        work = WORK_DTYPES[work]
    return Configured(arch, arch.config_class.from_dict(raw), work or torch.bfloat16)


def load(path: str | Path, device: torch.device | str = "cuda", arch: Configured | None = None,
         tuning: Tuning | None = None):
    """The model in folder ``path`` (config.json + safetensors), chosen by its ``architectures``
    name unless ``arch`` (from ``configure``) is given. ``tuning``: the kernel-choice thresholds
    (default: the device's)."""
    conf = arch or configure(path)
    ckpt = Checkpoint(path)
    spec = conf.arch.declare(conf.config, ckpt.names())
    rt = Runtime(conf.work, torch.device(device), tuning or Tuning.for_device(device))
    tensors = load_tensors(ckpt, spec.tensor_decls(), rt.dtype, rt.device, spec.scope)
    model = build_model(spec, tensors, rt)
    model.config = conf.config
    model.spec = spec
    return model


def from_tensors(conf: Configured, tensors: dict, device: torch.device | str = "cuda"):
    """A model from tensors already in memory (the random-weights mode without a folder)."""
    spec = conf.arch.declare(conf.config, tensors.keys())
    rt = Runtime(conf.work, torch.device(device), Tuning.for_device(device))
    model = build_model(spec, tensors, rt)
    model.config = conf.config
    model.spec = spec
    return model


register(Lfm3())
