"""Root-mean-square norm (kind "rmsnorm").

Formula of the reference's kernels (engine/kernels/rmsnorm.py:31-45,
engine/kernels/add_rmsnorm.py:21-29): the mean of squares and the scaling are
32-bit; in bfloat16 the normalised value is rounded before the weight multiply.
"""

from __future__ import annotations

from .registry import register_part


class RMSNorm:
    @staticmethod
    def weight_shapes(spec):
        return {"weight": (spec.size,)}

    def __init__(self, spec, weights, runtime):
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = weights["weight"]
        self.ops = runtime.ops

    def forward(self, x):
        return self.ops.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, x, delta):
        """x += delta in place (32-bit sum, stored in x's dtype), then the norm of the new x."""
        return self.ops.add_rmsnorm(x, delta, self.weight, self.eps)

    def folded(self, dtype):
        """(weight, eps) for a product that takes this norm in its prologue (``ops.linear(..., norm=)``), or None when
        the weight is kept in another type than the rows (a 32-bit weight in a bfloat16 run: the norm runs on its own)."""
        return (self.weight, self.eps) if self.weight.dtype == dtype else None


register_part("norm", "rmsnorm", RMSNorm)
