"""Typed configuration, read from config.json, and the architecture registry."""

from .registry import (ConfigError, ModelConfig, TensorNames, architecture_names, config_from_dict, load_config,
                       register_architecture, save_config)
from .specs import AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, NormSpec, RopeSpec

__all__ = ["ConfigError", "ModelConfig", "TensorNames", "architecture_names", "config_from_dict", "load_config",
           "register_architecture", "save_config", "AttentionSpec", "BlockSpec", "GatedMLPSpec", "ModelSpec",
           "NormSpec", "RopeSpec"]
