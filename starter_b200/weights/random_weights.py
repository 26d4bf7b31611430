"""Random weights from a configuration and a seed.

Matrices are N(0, 0.02) and norm weights 1 + N(0, 0.1), as the tiny test
model of the reference is filled (tests/tiny.py:24-30, there with 0.05 and
0.1).  Each tensor's values depend on (seed, tensor name) only, so they do
not change with the order tensors are made in, nor with which other tensors
exist.  ``write_model_folder`` writes config.json and model.safetensors;
``RandomSource`` hands the same tensors out without a file.
"""

from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Dict, Tuple

import torch

from ..config.registry import save_config
from .loader import expected_tensors
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return int.from_bytes(digest, "little") >> 1


class RandomSource:
    """Tensors of a model by name, made on demand.  Same interface as a mapped safetensors file."""

    def __init__(self, config, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu"):
        spec, names = config.model_spec(), config.tensor_names()
        required, _ = expected_tensors(spec, names)
        self.seed = int(seed)
        self.dtype = dtype
        self.device = torch.device(device)
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {n: (dtype, s) for n, s in required.items()}

    def get(self, name: str) -> torch.Tensor:
        _, shape = self.entries[name]
        gen = torch.Generator(device=self.device)
        gen.manual_seed(_tensor_seed(self.seed, name))
        noise = torch.randn(shape, generator=gen, dtype=torch.float32, device=self.device)
        if len(shape) == 1:
            return (1.0 + NORM_STD * noise).to(self.dtype)
        return (MATRIX_STD * noise).to(self.dtype)


def write_model_folder(config, seed: int, folder, dtype: torch.dtype = torch.bfloat16, shards: int = 1,
                       device="cpu") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights.

    ``shards`` > 1 writes ``model-0000i-of-0000n.safetensors`` files instead, the
    tensors dealt out in order in runs of about equal bytes, the way published
    checkpoints are laid out (no index file: the loader needs none).  ``device``
    is where the numbers are drawn (a GPU draws a large model in seconds; its
    generator gives other values than the CPU's for the same seed).
    """
    folder = Path(folder)
    save_config(config, folder)
    source = RandomSource(config, seed, dtype=dtype, device=device)
    items = list(source.entries.items())
    if shards <= 1:
        write_safetensors(folder / "model.safetensors", items, source.get)
        return folder
    sizes = [torch.Size(shape).numel() for _, (_, shape) in items]
    per_shard, groups, run = sum(sizes) / shards, [[]], 0
    for item, size in zip(items, sizes):
        if run >= per_shard * len(groups) and len(groups) < shards:
            groups.append([])
        groups[-1].append(item)
        run += size
    for i, group in enumerate(groups):
        write_safetensors(folder / f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors", group, source.get)
    return folder
