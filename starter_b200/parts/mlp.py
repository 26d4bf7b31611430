"""Dense gated feed-forward (kind "gated_mlp"): down(silu(gate(x)) * up(x)).

The reference fuses gate and up into one [2I, H] matrix, gate half first
(engine/model.py:116, engine/kernels/swiglu.py:5-6), and rounds gate, up,
silu(gate) and the product to bfloat16 (engine/kernels/swiglu.py:21-24).
"""

from __future__ import annotations

import torch

from .registry import register_part


class GatedMLP:
    @staticmethod
    def weight_shapes(spec):
        return {
            "gate": (spec.intermediate_size, spec.hidden_size),
            "up": (spec.intermediate_size, spec.hidden_size),
            "down": (spec.hidden_size, spec.intermediate_size),
        }

    def __init__(self, spec, weights, runtime):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not built; only 'silu' is")
        self.hidden_size = spec.hidden_size
        self.intermediate_size = spec.intermediate_size
        self.ops = runtime.ops
        self.w_gate_up = self.ops.prepare_matrix(torch.cat([weights["gate"], weights["up"]], dim=0), halves=2)
        self.w_down = self.ops.prepare_matrix(weights["down"])
        self.takes_fold = spec.hidden_size % 8 == 0 and spec.intermediate_size % 8 == 0

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, norm=None, residual=None):
        """h is the normed input; with ``norm`` it is the residual itself and the norm is taken inside the first
        product; with ``residual`` the result is added to that tensor instead of being returned on its own."""
        if norm is None and residual is None:
            return self.ops.linear(self.ops.linear_swiglu(h, self.w_gate_up), self.w_down)
        act = self.ops.linear_swiglu(h, self.w_gate_up, norm=norm)
        return self.ops.linear(act, self.w_down, add_to=residual)


register_part("ff", "gated_mlp", GatedMLP)
