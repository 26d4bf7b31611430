"""Causal grouped-query attention over the paged cache (kind "attention").

Steps of the reference's attention branch (engine/model.py:291-295,202-206):
fused q/k/v projection with rows laid out [q heads | k heads | v heads]
(engine/kernels/rope.py:46,75,89); per-head RMSNorm of q and k, rotary
positions, and the write of k and v into the cache in one kernel
(engine/kernels/rope.py:95-144); attention of the new rows over the cache,
query head h reading key/value head h // (heads / kv_heads)
(engine/kernels/attention.py:24-92); output projection.

Sizes, scale, window, the norm's eps and the position encoding all come from
the spec.  A layer with ``kv_from`` projects queries only and reads the
cache of the layer it names.

The position part is either rotary (it offers ``fused_rotary()``: norm,
rotation and the cache write then run in one kernel) or anything with
``apply(ctx, q, k) -> (q, k)`` over the normed heads (q [rows, heads, D], k
[rows, kv_heads, D], or None for a layer that stores none): the steps then
run one after another.  A layer without a position part rotates nothing.
"""

from __future__ import annotations

import torch

from ..cache.cache import KVRequest, SharedRequest
from .registry import build_part, register_part


class Attention:
    @staticmethod
    def weight_shapes(spec):
        hq, hkv, d, h = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.hidden_size
        shapes = {"q": (hq * d, h), "o": (h, hq * d)}
        if spec.kv_from is None:
            shapes["k"] = (hkv * d, h)
            shapes["v"] = (hkv * d, h)
        if spec.qk_norm is not None:
            shapes["q_norm"] = (d,)
            if spec.kv_from is None:
                shapes["k_norm"] = (d,)
        return shapes

    def __init__(self, spec, weights, runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} key/value heads evenly")
        if spec.qk_norm is not None and spec.qk_norm.size != spec.head_dim:
            raise ValueError("the per-head norm must have the head's size")
        self.spec = spec
        self.ops = runtime.ops
        self.num_heads = spec.num_heads
        self.num_kv_heads = spec.num_kv_heads
        self.head_dim = spec.head_dim
        self.scale = float(spec.scale)
        self.window = spec.window
        self.stores_kv = spec.kv_from is None
        mats = [weights["q"]] + ([weights["k"], weights["v"]] if self.stores_kv else [])
        self.w_qkv = self.ops.prepare_matrix(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0])
        self.w_o = self.ops.prepare_matrix(weights["o"])
        self.norm_eps = float(spec.qk_norm.eps) if spec.qk_norm is not None else 0.0
        self.q_norm = weights.get("q_norm")
        self.k_norm = weights.get("k_norm")
        self.position = build_part("position", spec.position, {}, runtime) if spec.position is not None else None
        self.takes_fold = spec.hidden_size % 8 == 0 and (spec.num_heads * spec.head_dim) % 8 == 0
        self.fused_position = self.position is None or hasattr(self.position, "fused_rotary")
        if not self.fused_position and not hasattr(self.position, "apply"):
            raise ValueError("a position part offers fused_rotary() or apply(ctx, q, k)")

    def cache_request(self):
        if not self.stores_kv:
            return SharedRequest(self.spec.kv_from)
        return KVRequest(self.num_kv_heads, self.head_dim, self.window)

    def prepare(self, cache) -> None:
        if self.position is not None:
            self.position.prepare(cache.max_seq_tokens)

    def _positions_applied(self, ctx, qkv):
        """q/k/v rows with the per-head norm taken and the position part's ``apply`` run over q and k."""
        rows, d, hq = qkv.shape[0], self.head_dim, self.num_heads
        hkv = self.num_kv_heads if self.stores_kv else 0
        q = qkv[:, :hq * d].reshape(rows * hq, d).contiguous()
        k = qkv[:, hq * d:(hq + hkv) * d].reshape(rows * hkv, d).contiguous() if hkv else None
        if self.q_norm is not None:
            q = self.ops.rmsnorm(q, self.q_norm, self.norm_eps)
        if k is not None and self.k_norm is not None:
            k = self.ops.rmsnorm(k, self.k_norm, self.norm_eps)
        q, k = self.position.apply(ctx, q.view(rows, hq, d), k.view(rows, hkv, d) if k is not None else None)
        pieces = [q.reshape(rows, hq * d)]
        if hkv:
            pieces += [k.reshape(rows, hkv * d), qkv[:, (hq + hkv) * d:]]
        return torch.cat(pieces, dim=1).contiguous()

    def _out(self, a, residual):
        return self.ops.linear(a, self.w_o) if residual is None else self.ops.linear(a, self.w_o, add_to=residual)

    def forward(self, ctx, h, layer_cache, norm=None, residual=None):
        """h is the normed input; with ``norm`` it is the residual itself and the norm is taken inside the q/k/v
        product; with ``residual`` the output projection adds to that tensor instead of returning its own."""
        qkv = self.ops.linear(h, self.w_qkv) if norm is None else self.ops.linear(h, self.w_qkv, norm=norm)
        if not self.fused_position:
            n_kv = self.num_kv_heads if self.stores_kv else 0
            q = self.ops.qk_norm_rope_store(ctx, self._positions_applied(ctx, qkv), layer_cache, self.num_heads, n_kv,
                                            self.head_dim, None, None, 0.0, None)
            a = self.ops.attention(ctx, q, layer_cache, self.num_heads, self.scale, self.window)
            return self._out(a, residual)
        rotary = self.position.fused_rotary() if self.position is not None else None
        n_kv = self.num_kv_heads if self.stores_kv else 0
        a = None
        one_call = getattr(self.ops, "qk_attention", None)   # optional: both steps in one kernel where the ops have it
        if one_call is not None:
            a = one_call(ctx, qkv, layer_cache, self.num_heads, n_kv, self.head_dim, self.q_norm, self.k_norm,
                         self.norm_eps, rotary, self.scale, self.window, then=self.w_o)
        if a is None:
            q = self.ops.qk_norm_rope_store(ctx, qkv, layer_cache, self.num_heads, n_kv, self.head_dim,
                                            self.q_norm, self.k_norm, self.norm_eps, rotary)
            a = self.ops.attention(ctx, q, layer_cache, self.num_heads, self.scale, self.window)
        return self._out(a, residual)


register_part("mixer", "attention", Attention)
