"""Rotary position encoding (kind "rope"), rotate-half pairing.

Tables as the reference builds them (engine/model.py:78-93): inv_freq in
32-bit, angle = position * inv_freq in 32-bit, cos and sin taken in 32-bit and
only then rounded to the run's dtype.  Columns d and d + D/2 share an angle,
so the table holds D/2 columns.
"""

from __future__ import annotations

import torch

from .registry import register_part


class RotaryEmbedding:
    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        self.runtime = runtime
        self.cos = None
        self.sin = None

    def prepare(self, n_positions: int) -> None:
        """Build (or grow) the tables to cover positions 0..n_positions-1."""
        if self.cos is not None and self.cos.shape[0] >= n_positions:
            return
        d = self.rotary_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
        positions = torch.arange(n_positions, dtype=torch.float32)
        angles = positions[:, None] * inv_freq[None, :]
        rt = self.runtime
        self.cos = angles.cos().to(rt.dtype).to(rt.device).contiguous()
        self.sin = angles.sin().to(rt.dtype).to(rt.device).contiguous()

    def fused_rotary(self):
        """(cos, sin, rotary_dim) for the kernel that norms, rotates and stores in one pass."""
        return self.cos, self.sin, self.rotary_dim


register_part("position", "rope", RotaryEmbedding)
