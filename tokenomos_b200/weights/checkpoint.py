"""A model folder: ``config.json`` and safetensors (one file, or shards behind an index), read
by tensor name (Tokenomos models/load/checkpoint.py:138-174 reads the same two layouts).

``load_tensors`` checks the folder against the model's tensor declarations before it reads
anything and raises one ``WeightError`` that lists every missing tensor, every unexpected
tensor and every wrong shape. How tensors are kept:

- matrices and embeddings in the work dtype (bfloat16 or float32);
- norm weights, biases and conv taps in float32: a value stored in 32-bit stays 32-bit, a
  16-bit one widens exactly;
- integer tables as int32.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_MATRIX, ROLE_NORM, ROLE_TABLE,
                                       ROLE_VECTOR, TensorDecl)


class WeightError(ValueError):
    """The folder's tensors do not match the model: the message lists every difference."""


_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "F64": torch.float64, "I32": torch.int32, "I64": torch.int64, "I16": torch.int16,
              "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


class Checkpoint:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        cfg = self.path / "config.json"
        if not cfg.exists():
            raise FileNotFoundError(f"{self.path}: no config.json")
        self.config = json.loads(cfg.read_text("utf-8"))
        index = self.path / "model.safetensors.index.json"
        single = self.path / "model.safetensors"
        self._files: dict[str, object] = {}
        if index.exists():
            self.weight_map: dict[str, str] = json.loads(index.read_text("utf-8"))["weight_map"]
        elif single.exists():
            with safe_open(single, "pt") as f:
                self.weight_map = dict.fromkeys(f.keys(), single.name)
        else:
            raise FileNotFoundError(f"{self.path}: neither model.safetensors nor "
                                    "model.safetensors.index.json")

    def _file(self, name: str):
        if name not in self._files:
            self._files[name] = safe_open(self.path / name, "pt", device="cpu")
        return self._files[name]

    def names(self) -> list[str]:
        return list(self.weight_map)

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._file(self.weight_map[name]).get_slice(name).get_shape())

    def stored_dtype(self, name: str) -> torch.dtype:
        code = self._file(self.weight_map[name]).get_slice(name).get_dtype()
        return _ST_DTYPES.get(code, torch.float32)

    def get(self, name: str) -> torch.Tensor:
        return self._file(self.weight_map[name]).get_tensor(name)


def check(source, decls: list[TensorDecl], scope: tuple[str, ...] = ()) -> None:
    """Raise ``WeightError`` unless ``source`` (``names()``, ``shape(name)``) holds the declared
    tensors (optional ones may be absent) with the declared shapes, and nothing undeclared
    under the name prefixes in ``scope`` (empty: under any name)."""
    have = set(source.names())
    declared = {d.name: d for d in decls}
    missing = sorted(n for n, d in declared.items() if n not in have and not d.optional)
    unexpected = sorted(n for n in have - set(declared)
                        if not scope or any(n.startswith(prefix) for prefix in scope))
    wrong = []
    for n, d in declared.items():
        if n in have:
            got = tuple(source.shape(n))
            if got != tuple(d.shape):
                wrong.append(f"{n}: stored {list(got)}, the configuration needs {list(d.shape)}")
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: " + ", ".join(missing))
        if unexpected:
            parts.append(f"{len(unexpected)} unexpected: " + ", ".join(unexpected))
        if wrong:
            parts.append(f"{len(wrong)} with a wrong shape: " + "; ".join(wrong))
        raise WeightError("model tensors do not match the configuration — " + " | ".join(parts))


def kept_dtype(decl: TensorDecl, stored: torch.dtype, work: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in (see the module docstring)."""
    if decl.role == ROLE_TABLE or not stored.is_floating_point:
        return torch.int32
    if decl.role in (ROLE_NORM, ROLE_VECTOR):
        return torch.float32
    if decl.role in (ROLE_MATRIX, ROLE_EMBEDDING):
        return work
    raise ValueError(f"tensor role {decl.role!r}")


def load_tensors(source, decls: list[TensorDecl], work: torch.dtype, device,
                 scope: tuple[str, ...] = ()) -> dict:
    """name -> tensor on ``device`` for every declared tensor ``source`` holds, after ``check``."""
    check(source, decls, scope)
    out = {}
    for d in decls:
        if not source.has(d.name):
            continue
        t = source.get(d.name)
        out[d.name] = t.to(device=device, dtype=kept_dtype(d, t.dtype, work)).contiguous()
    return out
