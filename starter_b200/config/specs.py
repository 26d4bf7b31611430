"""Typed descriptions of the parts a model is put together from.

A spec is plain data: every size and constant a part needs, and nothing about
the model the part sits in.  An architecture turns its ``config.json`` into a
``ModelSpec``; the builder turns each spec into a part by looking its ``kind``
up in the part registry.  A new kind of part is a new spec class with a
``kind`` of its own plus one registered part class; nothing here has to change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm over the last axis: y = w * x * rsqrt(mean(x^2) + eps)."""

    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding, rotate-half pairing (d, d + rotary_dim/2),
    angle(p, j) = p / theta**(2j / rotary_dim)."""

    theta: float
    rotary_dim: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a key/value cache.

    ``window``: a query at position p sees the keys n with p - window < n <= p;
    None means every earlier key.  ``kv_from``: index of another layer whose
    cache this layer reads instead of projecting and storing keys and values.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[Any] = None
    window: Optional[int] = None
    kv_from: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: x += mixer(norm(x)); x += ff(norm(x)) for kind "prenorm"."""

    mixer_norm: Any
    mixer: Any
    ff_norm: Any
    ff: Any
    kind: str = "prenorm"


@dataclass(frozen=True)
class ModelSpec:
    """A decoder: embedding, layers, the order they run in, final norm, output head.

    ``schedule`` lists layer indices in execution order; an index may appear
    more than once: the layer then runs again with the same weights, and each occurrence keeps
    a cache entry of its own.

    Three optional constants of the outer model, None where an architecture has none (Qwen3 has
    none): ``embedding_scale`` multiplies the embedded rows, ``logit_scale`` the logits, and
    ``logit_softcap`` c turns a logit x into c * tanh(x / c), after the scale.
    """

    hidden_size: int
    vocab_size: int
    layers: Tuple[BlockSpec, ...]
    final_norm: Any
    tie_embeddings: bool
    schedule: Tuple[int, ...] = field(default=())
    embedding_scale: Optional[float] = None
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None

    def execution_order(self) -> Tuple[int, ...]:
        return self.schedule if self.schedule else tuple(range(len(self.layers)))
