"""Weights by tensor name, checked against what the model expects.

The reference reads every ``*.safetensors`` shard of the folder, sorted, into
one dict by name (engine/model.py:67-75), pops each tensor by its name, fuses
q/k/v and gate/up, ties the output head to the embedding when the file has no
``lm_head.weight``, and rejects leftovers (engine/model.py:100-128); each
fault raises on its own.  Here the shards are mapped, not read (a tensor is
materialised when it is asked for), the model's parts declare the tensors
they want, the folder is compared with that list once, and a single error
names every missing tensor, every unexpected tensor, every wrong shape and
every tensor that two shards both hold.

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


def check_tensors(found: Dict[str, Tuple[int, ...]], required, optional, where: str, duplicates=None) -> None:
    """``duplicates``: {name: [files that hold it]} for names stored more than once."""
    duplicates = duplicates or {}
    missing = sorted(n for n in required if n not in found)
    unexpected = sorted(n for n in found if n not in required and n not in optional)
    wrong = sorted((n, found[n], want) for n, want in {**optional, **required}.items()
                   if n in found and tuple(found[n]) != tuple(want))
    if not (missing or unexpected or wrong or duplicates):
        return
    lines = [f"{where} does not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): "
                     + ", ".join(f"{n} is {list(have)}, expected {list(want)}" for n, have, want in wrong))
    if duplicates:
        lines.append(f"  stored more than once ({len(duplicates)}): "
                     + ", ".join(f"{n} in {' and '.join(files)}" for n, files in sorted(duplicates.items())))
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


class ShardedSource:
    """Every ``*.safetensors`` file of a folder, sorted by name, as one source of tensors by name.

    No index file is read: the shards' own headers say what each holds, as in
    the reference (engine/model.py:67-75).  There a name in two shards is
    silently taken from the later one; here it is kept in ``duplicates`` and
    reported with the other faults.
    """

    def __init__(self, folder):
        self.folder = Path(folder)
        paths = sorted(self.folder.glob("*.safetensors"))
        if not paths:
            raise FileNotFoundError(f"no *.safetensors file in {self.folder}: a model folder holds config.json and "
                                    "model.safetensors (or its shards)")
        self.files = []
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
        self.duplicates: Dict[str, list] = {}
        self._home: Dict[str, SafetensorsFile] = {}
        try:
            for path in paths:
                shard = SafetensorsFile(path)
                self.files.append(shard)
                for name, entry in shard.entries.items():
                    if name in self._home:
                        self.duplicates.setdefault(name, [self._home[name].path.name]).append(path.name)
                        continue
                    self.entries[name] = entry
                    self._home[name] = shard
        except Exception:
            self.close()
            raise

    def get(self, name: str) -> torch.Tensor:
        return self._home[name].get(name)

    def close(self) -> None:
        for shard in self.files:
            shard.close()
        self.files, self.entries, self._home = [], {}, {}


class Checkpoint:
    """A source of tensors by name: a folder's mapped shards, or anything with ``entries`` and ``get``."""

    def __init__(self, source, where: str):
        self.source = source
        self.where = where

    @classmethod
    def open(cls, folder) -> "Checkpoint":
        source = ShardedSource(folder)
        where = str(source.files[0].path) if len(source.files) == 1 else \
            f"{folder} ({len(source.files)} safetensors files)"
        return cls(source, where)

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {name: tuple(shape) for name, (_, shape) in self.source.entries.items()}

    def check(self, spec, names) -> None:
        required, optional = expected_tensors(spec, names)
        check_tensors(self.shapes(), required, optional, self.where, getattr(self.source, "duplicates", None))

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
