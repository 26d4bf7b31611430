"""Qwen3 dense decoder ("Qwen3ForCausalLM"): configuration, layer arrangement, tensor names.

What the reference reads from config.json (engine/model.py:39-52): hidden_size,
intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads,
head_dim (default hidden_size // num_attention_heads), vocab_size, rms_norm_eps,
rope_theta, tie_word_embeddings (default False).  Layer order
(OPTIMIZATION_GUIDE.md:60-69): pre-norm attention branch with per-head RMSNorm
of q and k and rotary positions, then pre-norm SwiGLU branch.  Tensor names
(engine/model.py:102-125).

Beyond the reference, the sliding-window keys of the same config.json
(use_sliding_window, sliding_window, max_window_layers, layer_types) are
read: a layer named "sliding_attention" sees the last ``sliding_window`` keys.
Options with no implementation here (biases, rope scaling, another
activation) are refused when the configuration is read.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.registry import ConfigError, ModelConfig, TensorNames, register_architecture
from ..config.specs import AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, NormSpec, RopeSpec

_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "vocab_size", "rms_norm_eps")


def _positive_int(raw: dict, key: str) -> int:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    layer_windows: Tuple[Optional[int], ...] = ()

    architecture = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in raw]
        rope = raw.get("rope_parameters") if isinstance(raw.get("rope_parameters"), dict) else {}
        theta = raw.get("rope_theta", rope.get("rope_theta"))
        if theta is None:
            missing.append("rope_theta")
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads")
        layers = _positive_int(raw, "num_hidden_layers")
        head_dim = raw.get("head_dim") or hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})")
        if not isinstance(head_dim, int) or head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim must be a positive even integer, got {head_dim!r}")
        eps = float(raw["rms_norm_eps"])
        if not eps > 0.0 or not float(theta) > 0.0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not built: the projections have no bias here")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act={raw['hidden_act']!r} is not built: the feed-forward is SwiGLU")
        scaling = raw.get("rope_scaling")
        if scaling is None and rope:
            scaling = rope if rope.get("rope_type", "default") != "default" else None
        if scaling is not None and scaling.get("rope_type", scaling.get("type", "default")) != "default":
            raise ConfigError(f"rope scaling {scaling!r} is not built: only the default rotary table is")
        return cls(
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_positive_int(raw, "vocab_size"),
            rms_norm_eps=eps,
            rope_theta=float(theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            layer_windows=cls._windows(raw, layers),
        )

    @staticmethod
    def _windows(raw: dict, layers: int) -> Tuple[Optional[int], ...]:
        window = raw.get("sliding_window")
        types = raw.get("layer_types")
        if types is not None:
            if len(types) != layers:
                raise ConfigError(f"layer_types has {len(types)} entries for {layers} layers")
            unknown = sorted(set(types) - {"full_attention", "sliding_attention"})
            if unknown:
                raise ConfigError(f"layer_types holds unknown kinds: {unknown}")
            sliding = [t == "sliding_attention" for t in types]
        else:
            first = raw.get("max_window_layers", 0) or 0
            sliding = [bool(raw.get("use_sliding_window", False)) and i >= first for i in range(layers)]
        if any(sliding):
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"sliding layers need a positive integer sliding_window, got {window!r}")
            return tuple(window if s else None for s in sliding)
        return tuple(None for _ in range(layers))

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        windows = self.layer_windows or tuple(None for _ in range(self.num_hidden_layers))
        if any(w is not None for w in windows):
            out["use_sliding_window"] = True
            out["sliding_window"] = next(w for w in windows if w is not None)
            out["layer_types"] = ["sliding_attention" if w is not None else "full_attention" for w in windows]
        else:
            out["use_sliding_window"] = False
            out["sliding_window"] = None
        return out

    def model_spec(self) -> ModelSpec:
        windows = self.layer_windows or tuple(None for _ in range(self.num_hidden_layers))
        norm = NormSpec(size=self.hidden_size, eps=self.rms_norm_eps)
        head_norm = NormSpec(size=self.head_dim, eps=self.rms_norm_eps)
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = AttentionSpec(
                hidden_size=self.hidden_size,
                num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim,
                scale=1.0 / math.sqrt(self.head_dim),  # engine/model.py:130
                qk_norm=head_norm,
                position=RopeSpec(theta=self.rope_theta, rotary_dim=self.head_dim),
                window=windows[i],
            )
            ff = GatedMLPSpec(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)
            layers.append(BlockSpec(mixer_norm=norm, mixer=mixer, ff_norm=norm, ff=ff))
        return ModelSpec(
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            layers=tuple(layers),
            final_norm=norm,
            tie_embeddings=self.tie_word_embeddings,
        )

    def tensor_names(self) -> TensorNames:
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append({
                "mixer_norm": {"weight": p + "input_layernorm.weight"},
                "mixer": {
                    "q": p + "self_attn.q_proj.weight",
                    "k": p + "self_attn.k_proj.weight",
                    "v": p + "self_attn.v_proj.weight",
                    "o": p + "self_attn.o_proj.weight",
                    "q_norm": p + "self_attn.q_norm.weight",
                    "k_norm": p + "self_attn.k_norm.weight",
                },
                "ff_norm": {"weight": p + "post_attention_layernorm.weight"},
                "ff": {
                    "gate": p + "mlp.gate_proj.weight",
                    "up": p + "mlp.up_proj.weight",
                    "down": p + "mlp.down_proj.weight",
                },
            })
        return TensorNames(
            embedding="model.embed_tokens.weight",
            lm_head="lm_head.weight",
            final_norm={"weight": "model.norm.weight"},
            layers=layers,
        )


register_architecture(Qwen3Config.architecture, Qwen3Config)
