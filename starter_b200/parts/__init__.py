"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""

from .registry import CATEGORIES, build_part, part_class, register_part
from . import norm, rope, attention, mlp, block  # noqa: F401  (each registers its kind)

__all__ = ["CATEGORIES", "build_part", "part_class", "register_part"]
