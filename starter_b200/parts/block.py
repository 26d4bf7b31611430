"""A layer's arrangement (kind "prenorm"): x += mixer(norm(x)); x += ff(norm(x)).

Order of the reference's layer (OPTIMIZATION_GUIDE.md:60-69,
engine/model.py:289-298).  Each branch leaves its output on the residual
stream; the sum is taken by the next norm.
"""

from __future__ import annotations

from .registry import build_part, register_part


class PreNormBlock:
    @staticmethod
    def sub_parts(spec):
        """(name, category, spec) of the parts this block is made of."""
        return (("mixer_norm", "norm", spec.mixer_norm), ("mixer", "mixer", spec.mixer),
                ("ff_norm", "norm", spec.ff_norm), ("ff", "ff", spec.ff))

    def __init__(self, spec, weights, runtime):
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        return self.mixer.cache_request()

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        self.ff.prepare(cache)

    def forward(self, ctx, stream, layer_cache) -> None:
        stream.push(self.mixer.forward(ctx, stream.normed(self.mixer_norm), layer_cache))
        stream.push(self.ff.forward(ctx, stream.normed(self.ff_norm)))


register_part("block", "prenorm", PreNormBlock)
