"""Shared fixtures: tiny Qwen3 configurations with random weights in temporary folders.

Tests marked ``gpu`` need a B200 and the compiled extension; everything else
runs on a CPU.
"""

import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from starter_b200.config import config_from_dict  # noqa: E402
from starter_b200.weights import write_model_folder  # noqa: E402

# Tiny A and B are the two small configurations the benchmark description names; W adds
# sliding-window layers.  They differ in every size and option.  M and N have the head sizes (128, 64)
# that the tensor-core attention kernels take, so that the engine as a whole runs on those kernels too
# (fused decode attention, tcgen05 and mma.sync prefill attention, with and without a window).
TINY = {
    "A": dict(hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, vocab_size=256, rms_norm_eps=1e-6, rope_theta=10000.0,
              tie_word_embeddings=True, seed=0),
    "B": dict(hidden_size=96, intermediate_size=224, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, vocab_size=389, rms_norm_eps=1e-5, rope_theta=1000000.0,
              tie_word_embeddings=False, seed=1),
    "W": dict(hidden_size=80, intermediate_size=112, num_hidden_layers=4, num_attention_heads=10,
              num_key_value_heads=5, head_dim=48, vocab_size=301, rms_norm_eps=3e-6, rope_theta=500000.0,
              tie_word_embeddings=False, use_sliding_window=True, sliding_window=40,
              layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"], seed=2),
    "M": dict(hidden_size=512, intermediate_size=1408, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=2, head_dim=128, vocab_size=5003, rms_norm_eps=1e-6, rope_theta=1000000.0,
              tie_word_embeddings=True, use_sliding_window=True, sliding_window=70,
              layer_types=["full_attention", "sliding_attention", "full_attention"], seed=3),
    "N": dict(hidden_size=384, intermediate_size=1000, num_hidden_layers=2, num_attention_heads=6,
              num_key_value_heads=3, head_dim=64, vocab_size=3001, rms_norm_eps=1e-5, rope_theta=10000.0,
              tie_word_embeddings=False, seed=4),
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the compiled extension")


def tiny_raw(name: str) -> dict:
    raw = dict(TINY[name])
    raw.pop("seed")
    raw["architectures"] = ["Qwen3ForCausalLM"]
    return raw


class TinyFolders(dict):
    """name -> folder with config.json and model.safetensors in bfloat16.  ``for_dtype(name, "float32")``
    is a folder of the same configuration whose weights are stored in 32-bit and are not bfloat16
    numbers, split over three shard files: a 32-bit run that rounded a weight through bfloat16
    anywhere could not match the plain implementation on it."""

    def __init__(self, factory):
        super().__init__()
        self._factory = factory
        self._wide = {}

    def for_dtype(self, name: str, dtype: str):
        if dtype != "float32":
            return self[name]
        if name not in self._wide:
            folder = self._factory.mktemp(f"tiny_{name}_f32")
            write_model_folder(config_from_dict(tiny_raw(name)), TINY[name]["seed"], folder, dtype=torch.float32, shards=3)
            self._wide[name] = folder
        return self._wide[name]


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    out = TinyFolders(tmp_path_factory)
    for name in TINY:
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        write_model_folder(config_from_dict(tiny_raw(name)), TINY[name]["seed"], folder)
        out[name] = folder
    return out


def random_tokens(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
