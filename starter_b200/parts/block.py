"""A layer's arrangement (kind "prenorm"): x += mixer(norm(x)); x += ff(norm(x)).

Order of the reference's layer (OPTIMIZATION_GUIDE.md:60-69,
engine/model.py:289-298).  Each branch leaves its output on the residual
stream; the sum is taken by the next norm.

Where the kernels can (``ops.folds``: the few rows of a decode step), a branch
takes both ends itself, as the reference's decode path does
(engine/model.py:186-210): a part with ``takes_fold`` gets ``residual=`` (the
stream, to which its last product adds its result, leaving the statistics of
the new rows in ``stream.stats``) and, once such statistics exist, the residual
un-normed together with ``norm=`` (weight, eps, statistics: what its first
product folds into its prologue).  A norm offers ``folded(dtype)`` for that;
parts or norms without these run the plain order.
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
        self.folds = getattr(runtime.ops, "folds", None)
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        return self.mixer.cache_request()

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        self.ff.prepare(cache)

    def _branch(self, ctx, stream, norm, part, *args) -> None:
        fold = None
        if (self.folds is not None and getattr(part, "takes_fold", False) and hasattr(norm, "folded")
                and self.folds(stream.x.shape[0], stream.x.dtype)):
            fold = norm.folded(stream.x.dtype)
        if fold is None:
            stream.push(part.forward(ctx, stream.normed(norm), *args))
        elif stream.pending is None and stream.stats is not None:
            part.forward(ctx, stream.x, *args, norm=fold + (stream.stats,), residual=stream)
        else:   # nothing has left the rows' statistics yet (a model's first branch): the norm runs on its own
            part.forward(ctx, stream.normed(norm), *args, residual=stream)

    def forward(self, ctx, stream, layer_cache) -> None:
        self._branch(ctx, stream, self.mixer_norm, self.mixer, layer_cache)
        self._branch(ctx, stream, self.ff_norm, self.ff)


register_part("block", "prenorm", PreNormBlock)
