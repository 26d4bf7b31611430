"""Weights by tensor name, checked against what the model expects.

The reference pops each tensor by its name, fuses q/k/v and gate/up, ties the
output head to the embedding when the file has no ``lm_head.weight``, and
rejects leftovers (engine/model.py:100-128); each fault raises on its own.
Here the model's parts declare the tensors they want, the file is compared
with that list once, and a single error names every missing tensor, every
unexpected tensor and every wrong shape.

Dtypes: a tensor stored in bfloat16 stays bfloat16 and one stored in 32-bit
stays 32-bit for a bfloat16 run; a float32 run widens everything; integer
tensors become int32.
"""

from __future__ import annotations

from pathlib import Path
from typing import Dict, Tuple

import torch

from ..parts.registry import part_class
from .safetensors_io import SafetensorsFile


class WeightsError(ValueError):
    """The checkpoint does not hold what the model needs; the message lists every fault."""


def expected_tensors(spec, names) -> Tuple[Dict[str, Tuple[int, ...]], Dict[str, Tuple[int, ...]]]:
    """({name: shape} that must be there, {name: shape} that may be there) for a model."""
    required: Dict[str, Tuple[int, ...]] = {names.embedding: (spec.vocab_size, spec.hidden_size)}
    optional: Dict[str, Tuple[int, ...]] = {}
    (optional if spec.tie_embeddings else required)[names.lm_head] = (spec.vocab_size, spec.hidden_size)
    norm_cls = part_class("norm", spec.final_norm.kind)
    for role, shape in norm_cls.weight_shapes(spec.final_norm).items():
        required[names.final_norm[role]] = tuple(shape)
    if len(names.layers) != len(spec.layers):
        raise WeightsError(f"{len(names.layers)} layers are named for {len(spec.layers)} layers")
    for block_spec, block_names in zip(spec.layers, names.layers):
        block_cls = part_class("block", block_spec.kind)
        for part_name, category, sub in block_cls.sub_parts(block_spec):
            for role, shape in part_class(category, sub.kind).weight_shapes(sub).items():
                try:
                    required[block_names[part_name][role]] = tuple(shape)
                except KeyError:
                    raise WeightsError(f"the architecture names no tensor for {part_name}.{role}") from None
    return required, optional


def check_tensors(found: Dict[str, Tuple[int, ...]], required, optional, where: str) -> None:
    missing = sorted(n for n in required if n not in found)
    unexpected = sorted(n for n in found if n not in required and n not in optional)
    wrong = sorted((n, found[n], want) for n, want in {**optional, **required}.items()
                   if n in found and tuple(found[n]) != tuple(want))
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where} does not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): "
                     + ", ".join(f"{n} is {list(have)}, expected {list(want)}" for n, have, want in wrong))
    raise WeightsError("\n".join(lines))


def to_run_dtype(t: torch.Tensor, run_dtype: torch.dtype, name: str) -> torch.Tensor:
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return t.to(torch.int32)
    if run_dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    raise WeightsError(f"{name} is stored as {t.dtype}; a bfloat16 run takes bfloat16 or 32-bit tensors "
                       "(run with dtype float32 to widen it)")


class Checkpoint:
    """A source of tensors by name: a mapped model.safetensors, or anything with ``entries`` and ``get``."""

    def __init__(self, source, where: str):
        self.source = source
        self.where = where

    @classmethod
    def open(cls, folder) -> "Checkpoint":
        path = Path(folder) / "model.safetensors"
        return cls(SafetensorsFile(path), str(path))

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {name: tuple(shape) for name, (_, shape) in self.source.entries.items()}

    def check(self, spec, names) -> None:
        required, optional = expected_tensors(spec, names)
        check_tensors(self.shapes(), required, optional, self.where)

    def has(self, name: str) -> bool:
        return name in self.source.entries

    def load(self, name: str, run_dtype: torch.dtype, device) -> torch.Tensor:
        stored = self.source.get(name)
        t = to_run_dtype(stored, run_dtype, name).to(device).contiguous()
        # never hand out a view of the file's mapping: it dies with the file
        return t.clone() if t.data_ptr() == stored.data_ptr() and t.numel() else t

    def close(self) -> None:
        close = getattr(self.source, "close", None)
        if close:
            close()
