"""``ModelSpec`` + tensors -> ``Stack``: every part is built by the registry entry of its kind."""

from __future__ import annotations

from tokenomos_b200.parts.block import Stack
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, builder_of
from tokenomos_b200.parts.spec import BlockSpec, ModelSpec, PartSpec

# the registry family of the slots the shipped arrangements use; a part in any other slot
# names its family itself (``PartSpec.family``)
SLOT_FAMILY = {
    "mixer": "mixer",
    "ffn": "feed_forward",
    "pre_mixer_norm": "norm",
    "pre_ffn_norm": "norm",
    "post_mixer_norm": "norm",
    "post_ffn_norm": "norm",
}


def _part(family: str, spec: PartSpec, tensors: dict, rt: Runtime):
    mine = {role: tensors[d.name] for role, d in spec.tensors.items() if d.name in tensors}
    return builder_of(family, spec.kind)(spec.params, mine, rt)


def _block(spec: BlockSpec, tensors: dict, rt: Runtime):
    parts = {}
    for slot, part in spec.parts.items():
        if part is None:
            continue
        family = part.family or SLOT_FAMILY.get(slot)
        if family is None:
            raise ValueError(f"block slot {slot!r}: its part names no family, and the slot is not one "
                             f"of {sorted(SLOT_FAMILY)}")
        parts[slot] = _part(family, part, tensors, rt)
    return builder_of("block", spec.kind)(parts)


def build_model(spec: ModelSpec, tensors: dict, rt: Runtime) -> Stack:
    """``tensors``: name -> tensor on ``rt.device``, kept as the weight loader keeps them."""
    blocks = [_block(b, tensors, rt) for b in spec.blocks]
    final_norm = _part("norm", spec.final_norm, tensors, rt)
    head = Linear(tensors[spec.head.name], tuning=rt.tuning) if spec.head is not None else None
    return Stack(tensors[spec.embedding.name], blocks, list(spec.order), final_norm, head,
                 tuning=rt.tuning, embed_scale=spec.embed_scale, logit_softcap=spec.logit_softcap,
                 suppress=spec.suppress)
