"""A model as data: which parts each block is made of, which tensors they read, and the order
in which the blocks run.

An architecture's declaration turns its configuration into a ``ModelSpec``. The weight loader
checks a model folder against the spec's tensor declarations (and the random-weights mode
generates exactly those), and ``parts.build`` turns the spec plus tensors into runnable parts
through the registries in ``parts.registry``. Nothing in a spec is specific to one model:
another architecture is another function that returns a ``ModelSpec``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

# roles decide how a tensor is kept and how the random-weights mode fills it
ROLE_MATRIX = "matrix"        # work dtype; N(0, std)
ROLE_EMBEDDING = "embedding"  # work dtype; N(0, std)
ROLE_NORM = "norm"            # float32 vector; 1 (+ N(0, norm_std))
ROLE_VECTOR = "vector"        # float32 vector or small table (biases, conv taps); N(0, std)
ROLE_TABLE = "table"          # integer table; int32
ROLES = (ROLE_MATRIX, ROLE_EMBEDDING, ROLE_NORM, ROLE_VECTOR, ROLE_TABLE)


@dataclass(frozen=True)
class TensorDecl:
    """One tensor of the checkpoint: its name, the exact shape it must have, how it is kept."""

    name: str
    shape: tuple[int, ...]
    role: str = ROLE_MATRIX
    optional: bool = False


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry ``kind``, its sizes and constants, and its tensors by role name.
    ``family``: the registry the kind is looked up in (``mixer``, ``feed_forward``, ``norm``,
    ``position``); None: the family the slot's name implies (``parts.build.SLOT_FAMILY``), which
    covers the slots of the arrangements that ship. An arrangement with slots of its own (a
    second mixer, an extra branch) names the family on each of their parts."""

    kind: str
    params: dict = field(default_factory=dict)
    tensors: dict[str, TensorDecl] = field(default_factory=dict)
    family: str | None = None


@dataclass(frozen=True)
class BlockSpec:
    """A block: the arrangement ``kind`` and the parts it arranges, by slot name."""

    kind: str
    parts: dict[str, PartSpec | None]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the layer list: run block ``block``; ``state_from`` names an earlier entry
    of the list whose state this one reads instead of owning one (None: its own)."""

    block: int
    state_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab: int
    embedding: TensorDecl
    blocks: tuple[BlockSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: TensorDecl | None  # None: the head is the embedding (tied)
    # name prefixes the model owns in its folder: a stored tensor under one of them that the
    # model does not declare is an error; tensors elsewhere (another tower of a multimodal
    # folder, a stored copy of a tied head) are not this model's business. Empty: every name.
    scope: tuple[str, ...] = ()
    # options around the layer stack that some architectures have (None / empty: absent):
    # the embedding rows times a constant (rounded to the work type, as is the product); the
    # logits through ``cap * tanh(logits / cap)``; token ids whose logits are -inf
    embed_scale: float | None = None
    logit_softcap: float | None = None
    suppress: tuple[int, ...] = ()

    def tensor_decls(self) -> list[TensorDecl]:
        """Every tensor the model reads, in a fixed order (the order random weights are drawn)."""
        out = [self.embedding]
        for block in self.blocks:
            for part in block.parts.values():
                if part is not None:
                    out.extend(part.tensors.values())
        out.extend(self.final_norm.tensors.values())
        if self.head is not None:
            out.append(self.head)
        seen: dict[str, TensorDecl] = {}
        for d in out:
            if d.name in seen and seen[d.name] != d:
                raise ValueError(f"tensor {d.name!r} declared twice with different shapes or roles")
            seen[d.name] = d
        return list(seen.values())
