"""One registry from an architecture's name to its typed configuration.

``config.json`` names its architecture in ``architectures[0]``; that name picks
the configuration class, and the class says how the model is put together
(``model_spec``) and what its tensors are called in a checkpoint
(``tensor_names``).  The reference hard-wires one model
(engine/model.py:96-130); the name lookup is this library's own.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Type


class ConfigError(ValueError):
    """A configuration that is missing a key, inconsistent, or asks for an option that is not built."""


@dataclass
class TensorNames:
    """Checkpoint names of every tensor of a model, by part and role.

    ``layers[i]`` maps a part of layer i ("mixer_norm", "mixer", "ff_norm",
    "ff") to {role: checkpoint name}; the roles are the ones the part class
    declares in ``weight_shapes``.
    """

    embedding: str
    lm_head: str
    final_norm: Dict[str, str]
    layers: List[Dict[str, Dict[str, str]]] = field(default_factory=list)


class ModelConfig:
    """Base of typed configurations.  A subclass reads its own config.json keys."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def model_spec(self):
        raise NotImplementedError

    def tensor_names(self) -> TensorNames:
        raise NotImplementedError


_ARCHITECTURES: Dict[str, Type[ModelConfig]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig]) -> None:
    """Make ``name`` (as it stands in config.json's ``architectures``) buildable."""
    _ARCHITECTURES[name] = config_cls


def architecture_names() -> List[str]:
    return sorted(_ARCHITECTURES)


def config_from_dict(raw: dict) -> ModelConfig:
    names = raw.get("architectures")
    if not isinstance(names, list) or not names:
        raise ConfigError("config.json has no 'architectures' list; known architectures: "
                          + ", ".join(architecture_names()))
    name = names[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; known architectures: " + ", ".join(architecture_names()))
    return _ARCHITECTURES[name].from_dict(raw)


def load_config(folder) -> ModelConfig:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and model.safetensors")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(raw)


def save_config(config: ModelConfig, folder) -> None:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
