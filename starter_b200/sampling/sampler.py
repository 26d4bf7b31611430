"""Token selection: greedy, or temperature with optional top-k.

The reference selects greedily, ``argmax`` inside the captured step
(engine/engine.py:204,207), lowest index on ties (engine/kernels/topk.py:4-5).
Temperature and top-k are this library's addition.  A draw is a pure
function of the 32-bit logits and a uniform number keyed by (seed, request,
step), so a request's tokens do not depend on the batch it ran in, on its
slot, or on how many requests ran before it.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 selects greedily; top_k 0 keeps the whole vocabulary."""

    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


def select(ops, logits, params: SamplingParams, request_ids=None, steps=None, advance=False):
    """Tokens (int32, on the device) for logits [rows, vocab].  ``request_ids`` and ``steps``
    (int32, on the device) key the uniform number of each row when sampling."""
    if params.greedy:
        return ops.argmax(logits)
    return ops.sample(logits, params.temperature, params.top_k, params.seed, request_ids, steps, advance=advance)
