"""Registry of part classes, by category and kind.

Categories: "norm", "position", "mixer", "ff", "block".  A spec's ``kind``
picks the class.  Every part class offers

* ``weight_shapes(spec) -> {role: shape}``: the tensors it wants, by role;
* ``__init__(spec, weights, runtime)``: ``weights`` maps role -> tensor in the
  run's dtype on the run's device; ``runtime`` carries dtype, device and kernels.

and, by category,

* norm:     ``forward(x) -> y`` and ``add_forward(x, delta) -> y`` (x += delta in place, then norm);
* position: ``prepare(n_positions)`` and ``fused_rotary()`` or ``apply(ctx, q, k)``;
* mixer:    ``cache_request()`` and ``forward(ctx, h, layer_cache) -> [rows, hidden]``;
* ff:       ``forward(ctx, h) -> [rows, hidden]``;
* block:    ``forward(ctx, stream, layer_cache)`` on a ``ResidualStream``.

A part never learns which model it is in: it sees its spec, its weights, the
step's context and its own layer's cache view.
"""

from __future__ import annotations

from typing import Dict, Tuple

_PARTS: Dict[Tuple[str, str], type] = {}
CATEGORIES = ("norm", "position", "mixer", "ff", "block")


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")
    _PARTS[(category, kind)] = cls


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise KeyError(f"no {category} part of kind {kind!r} is registered; known: {known}") from None


def build_part(category: str, spec, weights, runtime):
    return part_class(category, spec.kind)(spec, weights, runtime)
