"""What another architecture may ask of the outer model and of the attention part without editing them:
constants of the outer model (embedding scale, logit scale, logit soft cap) and a position encoding that is
not rotary.  The parts here are toys defined in this file; they are no model of anyone's."""

import dataclasses
import math
from dataclasses import dataclass

import torch

from conftest import TINY, random_tokens, tiny_raw
from emulated_ops import EmulatedOps
from helpers import run_tail_by_one, run_whole
from starter_b200.config import ModelConfig, config_from_dict
from starter_b200.engine.context import Runtime
from starter_b200.engine.model import DecoderModel
from starter_b200.engine.session import Session
from starter_b200.parts import register_part
from starter_b200.weights import RandomSource


def _session(config, spec_change=None, seed=1, dtype="float32"):
    """A session over ``config`` whose model spec is passed through ``spec_change`` first."""
    if spec_change is not None:
        base = config.model_spec()
        changed = spec_change(base)
        config = _WithSpec(config, changed)
    return Session((config, RandomSource(config, seed)), dtype=dtype, device="cpu", ops=EmulatedOps(), max_tokens=64 * 6,
                   max_seqs=3)


class _WithSpec(ModelConfig):
    """A configuration that answers with another model spec (same tensors)."""

    def __init__(self, config, spec):
        self._config, self._spec = config, spec

    def model_spec(self):
        return self._spec

    def tensor_names(self):
        return self._config.tensor_names()


def test_outer_model_constants():
    cfg = config_from_dict(tiny_raw("B"))                       # untied: the embedding's scale does not reach the head
    seqs = random_tokens(TINY["B"]["vocab_size"], (9, 70), seed=2)
    plain_logits = run_whole(_session(cfg), seqs)

    capped = run_whole(_session(cfg, lambda s: dataclasses.replace(s, logit_scale=0.5, logit_softcap=0.05)), seqs)
    for got, base in zip(capped, plain_logits):
        assert torch.allclose(got, 0.05 * torch.tanh(0.5 * base / 0.05), atol=1e-6)
        assert float(got.abs().max()) <= 0.05

    # An embedding scale is the same as a table that holds the scaled rows.
    scaled_session = _session(cfg, lambda s: dataclasses.replace(s, embedding_scale=3.0))
    table_session = _session(cfg)
    table_session.model.embedding.mul_(3.0)
    a, b = run_whole(scaled_session, seqs), run_whole(table_session, seqs)
    assert all(torch.allclose(x, y, atol=1e-5) for x, y in zip(a, b))
    assert not torch.allclose(a[0], plain_logits[0], atol=1e-3)


@dataclass(frozen=True)
class OffsetPositionSpec:
    """A toy absolute position encoding: q and k get sin(position * rate) * strength added to every element."""
    rate: float
    strength: float
    kind: str = "toy_offset_position"


class OffsetPosition:
    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        self.spec = spec

    def prepare(self, n_positions):
        pass

    def apply(self, ctx, q, k):
        slots = ctx.seq_slot.long()[ctx.row_seq.long()]
        pos = ctx.lengths.long()[slots] + torch.arange(ctx.n_rows, device=q.device) - ctx.cu_q.long()[ctx.row_seq.long()]
        add = (torch.sin(pos.float() * self.spec.rate) * self.spec.strength).to(q.dtype)[:, None, None]
        return q + add, (k + add if k is not None else None)


register_part("position", "toy_offset_position", OffsetPosition)


def test_attention_with_a_position_part_that_is_not_rotary():
    """The attention part runs a position part that only offers apply(ctx, q, k): per-head norm, the part's
    own encoding, the cache write and attention one after another.  Whole prompts and token-by-token steps
    agree (the keys in the cache carry their own positions), and the encoding matters."""
    cfg = config_from_dict(tiny_raw("A"))

    def swap(strength):
        def change(spec):
            layers = tuple(dataclasses.replace(b, mixer=dataclasses.replace(
                b.mixer, position=OffsetPositionSpec(rate=0.37, strength=strength))) for b in spec.layers)
            return dataclasses.replace(spec, layers=layers)
        return change

    seqs = random_tokens(TINY["A"]["vocab_size"], (40, 70, 9), seed=3)
    sess = _session(cfg, swap(0.5))
    assert not sess.model.blocks[0].mixer.fused_position
    whole = run_whole(sess, seqs, together=True)
    tail = run_tail_by_one(sess, seqs, tail=20)
    scale = max(float(w.abs().max()) for w in whole)
    for a, b in zip(whole, tail):
        assert float((a - b).abs().max()) <= 1e-4 * scale
    other = run_whole(_session(cfg, swap(0.0)), seqs, together=True)
    assert float((whole[0] - other[0]).abs().max()) > 1e-3 * scale
