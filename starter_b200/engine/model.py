"""A decoder put together from parts, as its ModelSpec says.

Reference forward (engine/model.py:280-299, 322-331): embedding, the layers,
final norm on the rows whose logits are wanted, output head.  Here the layers
are parts built from specs, and the order they run in is the spec's list.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..config.registry import load_config
from ..parts.registry import build_part, part_class
from ..weights.loader import Checkpoint, WeightsError
from .context import ResidualStream, Runtime, StepContext


class DecoderModel:
    def __init__(self, spec, names, checkpoint: Checkpoint, runtime: Runtime):
        checkpoint.check(spec, names)
        self.spec = spec
        self.runtime = runtime
        ops, dtype, device = runtime.ops, runtime.dtype, runtime.device

        def load(name):
            return checkpoint.load(name, dtype, device)

        self.embedding = load(names.embedding).contiguous()   # a table to gather rows from: no product reads it ...
        if checkpoint.has(names.lm_head):
            # engine/model.py:103-107: an lm_head in the file is used even when the config ties.
            self.lm_head = ops.prepare_matrix(load(names.lm_head))
        elif spec.tie_embeddings:
            self.lm_head = ops.prepare_matrix(self.embedding)   # ... unless it is the output head as well (same tensor)
        else:
            raise WeightsError(f"{checkpoint.where}: {names.lm_head} is missing and the embeddings are not tied")
        norm_cls = part_class("norm", spec.final_norm.kind)
        self.final_norm = norm_cls(spec.final_norm,
                                   {r: load(names.final_norm[r]) for r in norm_cls.weight_shapes(spec.final_norm)}, runtime)
        self.blocks = []
        for block_spec, block_names in zip(spec.layers, names.layers):
            block_cls = part_class("block", block_spec.kind)
            weights = {}
            for part_name, category, sub in block_cls.sub_parts(block_spec):
                roles = part_class(category, sub.kind).weight_shapes(sub)
                weights[part_name] = {role: load(block_names[part_name][role]) for role in roles}
            self.blocks.append(block_cls(block_spec, weights, runtime))
        self.order = spec.execution_order()
        for i in self.order:
            if not 0 <= i < len(self.blocks):
                raise ValueError(f"the execution order names layer {i}; the model has {len(self.blocks)} layers")

    # ---- construction ------------------------------------------------------------------

    @classmethod
    def from_folder(cls, folder, runtime: Runtime) -> "DecoderModel":
        config = load_config(folder)
        checkpoint = Checkpoint.open(folder)
        try:
            model = cls(config.model_spec(), config.tensor_names(), checkpoint, runtime)
        finally:
            checkpoint.close()
        model.config = config
        return model

    @classmethod
    def from_source(cls, config, source, runtime: Runtime, where: str = "weight source") -> "DecoderModel":
        model = cls(config.model_spec(), config.tensor_names(), Checkpoint(source, where), runtime)
        model.config = config
        return model

    def parts(self):
        """Every part object of the model: the final norm, each block, and what each block is made of."""
        yield self.final_norm
        for block, block_spec in zip(self.blocks, self.spec.layers):
            yield block
            for name, _, _ in type(block).sub_parts(block_spec):
                part = getattr(block, name, None)
                if part is not None:
                    yield part

    # ---- cache -------------------------------------------------------------------------

    def cache_requests(self) -> List[object]:
        """What each entry of the execution order asks of the cache.  A layer that is named twice runs
        with the same weights but keeps a cache entry per occurrence (otherwise the second run would
        overwrite what the first run of a later step has to read).  A mixer that reads another layer's
        cache gets the entry of that layer's latest earlier occurrence."""
        from ..cache.cache import SharedRequest
        requests = []
        for pos, i in enumerate(self.order):
            req = self.blocks[i].cache_request()
            if isinstance(req, SharedRequest):
                earlier = [p for p in range(pos) if self.order[p] == req.layer]
                if not earlier:
                    raise ValueError(f"layer {i} reads the cache of layer {req.layer}, which has not run before it")
                req = SharedRequest(earlier[-1])
            requests.append(req)
        return requests

    def prepare(self, cache) -> None:
        """Size position tables and workspaces for the cache the model will run on."""
        for block in self.blocks:
            block.prepare(cache)

    # ---- forward -----------------------------------------------------------------------

    def hidden(self, ctx: StepContext, tokens: torch.Tensor) -> ResidualStream:
        """Run the step's rows through every layer; returns the residual stream before the final norm."""
        x = ctx.ops.embed(tokens, self.embedding, ctx.status)
        if self.spec.embedding_scale is not None:
            x = (x.float() * self.spec.embedding_scale).to(x.dtype)
        stream = ResidualStream(x)
        for pos, i in enumerate(self.order):
            self.blocks[i].forward(ctx, stream, ctx.cache.layers[pos])
        return stream

    def logits(self, ctx: StepContext, stream: ResidualStream, rows: Optional[torch.Tensor]) -> torch.Tensor:
        """32-bit logits [len(rows), vocab] at the given rows (all rows when None)."""
        ops = ctx.ops
        x, delta = stream.x, stream.pending
        if rows is not None:
            x = ops.gather_rows(x, rows)
            delta = ops.gather_rows(delta, rows) if delta is not None else None
        h = self.final_norm.add_forward(x, delta) if delta is not None else self.final_norm.forward(x)
        logits = ops.linear(h, self.lm_head, out_float32=True)
        if self.spec.logit_scale is not None:
            logits = logits * self.spec.logit_scale
        if self.spec.logit_softcap is not None:
            logits = torch.tanh(logits / self.spec.logit_softcap) * self.spec.logit_softcap
        return logits
