"""Parts a model is put together from: mixers, feed-forwards, norms, position encodings, block
arrangements; ``build_model`` turns a ``ModelSpec`` and its tensors into a runnable ``Stack``."""

from tokenomos_b200.parts import attention, block, ffn, norm, rope, shortconv  # noqa: F401  (register)
from tokenomos_b200.parts.build import build_model
from tokenomos_b200.parts.registry import Runtime, register

__all__ = ["build_model", "register", "Runtime"]
