"""A toy architecture defined here, in the test: a mixer with state of its own beside attention
layers, a layer that runs twice, and a layer that reads another layer's cache.  It is registered,
built, stepped and run through generation without a change to the library's files.  It is no
model of anyone's: it shows that the interfaces of the parts are enough."""

import math
from dataclasses import dataclass

import pytest
import torch

from starter_b200.cache import StateRequest
from starter_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelConfig, ModelSpec, NormSpec, RopeSpec,
                                 TensorNames, config_from_dict, register_architecture)
from starter_b200.engine import Engine, Session, StepEntry
from starter_b200.parts import register_part
from starter_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    state_size: int
    decay: float
    kind: str = "toy_decay"


class DecayMixer:
    """state <- decay * state + W_in h_t ;  out_t = W_out state.  The state lives in the cache's
    fixed-size area, one record per sequence, and is zero when a sequence starts."""

    @staticmethod
    def weight_shapes(spec):
        return {"w_in": (spec.state_size, spec.hidden_size), "w_out": (spec.hidden_size, spec.state_size)}

    def __init__(self, spec, weights, runtime):
        self.spec, self.ops = spec, runtime.ops
        self.w_in = self.ops.prepare_matrix(weights["w_in"])
        self.w_out = self.ops.prepare_matrix(weights["w_out"])

    def cache_request(self):
        return StateRequest((self.spec.state_size,), "float32")

    def prepare(self, cache):
        pass

    capturable = False   # forward reads device values on the host: decoding must run step by step

    def forward(self, ctx, h, layer_cache):
        u = self.ops.linear(h, self.w_in).float()
        cu, slots = ctx.cu_q.tolist(), ctx.seq_slot.tolist()
        states = torch.empty_like(u)
        for b, slot in enumerate(slots):
            s = layer_cache.state[slot]
            for r in range(cu[b], cu[b + 1]):
                s = self.spec.decay * s + u[r]
                states[r] = s
            layer_cache.state[slot] = s
        return self.ops.linear(states.to(h.dtype), self.w_out)


register_part("mixer", "toy_decay", DecayMixer)


class GraphDecayMixer(DecayMixer):
    """The same mixer with its one-token step written in tensor operations only (state records gathered and
    scattered by the step's slot vector), so that a decode step with it can be captured and replayed."""

    capturable = True

    def forward(self, ctx, h, layer_cache):
        if not ctx.is_decode:
            return super().forward(ctx, h, layer_cache)
        u = self.ops.linear(h, self.w_in).float()
        slots = ctx.seq_slot.long()                      # padding rows name the null slot's record
        s = self.spec.decay * layer_cache.state[slots] + u
        layer_cache.state.index_copy_(0, slots, s)
        return self.ops.linear(s.to(h.dtype), self.w_out)


register_part("mixer", "toy_decay_graph", GraphDecayMixer)


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    hidden: int
    state: int
    vocab: int
    decay: float
    mixer_kind: str = "toy_decay"
    architecture = "ToyDecayForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(hidden=raw["hidden"], state=raw["state"], vocab=raw["vocab"], decay=raw["decay"],
                   mixer_kind=raw.get("mixer_kind", "toy_decay"))

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden": self.hidden, "state": self.state, "vocab": self.vocab,
                "decay": self.decay, "mixer_kind": self.mixer_kind}

    def model_spec(self):
        norm = NormSpec(size=self.hidden, eps=1e-5)
        ff = GatedMLPSpec(hidden_size=self.hidden, intermediate_size=2 * self.hidden)
        att = dict(hidden_size=self.hidden, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                   position=RopeSpec(theta=10000.0, rotary_dim=16))
        layers = (
            BlockSpec(mixer_norm=norm, mixer=DecaySpec(self.hidden, self.state, self.decay, self.mixer_kind),
                      ff_norm=norm, ff=ff),
            BlockSpec(mixer_norm=norm, mixer=AttentionSpec(**att), ff_norm=norm, ff=ff),
            BlockSpec(mixer_norm=norm, mixer=AttentionSpec(kv_from=1, **att), ff_norm=norm, ff=ff),
        )
        # layer 0 runs twice (same weights, same state record); layer 2 reads the cache of layer 1
        return ModelSpec(hidden_size=self.hidden, vocab_size=self.vocab, layers=layers, final_norm=norm,
                         tie_embeddings=True, schedule=(0, 1, 2, 0))

    def tensor_names(self):
        layers = []
        for i, mixer in enumerate(({"w_in": "w_in", "w_out": "w_out"}, {"q": "q", "k": "k", "v": "v", "o": "o"},
                                   {"q": "q", "o": "o"})):
            p = f"layers.{i}."
            layers.append({"mixer_norm": {"weight": p + "n1"}, "mixer": {r: p + n for r, n in mixer.items()},
                           "ff_norm": {"weight": p + "n2"}, "ff": {"gate": p + "gate", "up": p + "up", "down": p + "down"}})
        return TensorNames(embedding="embed", lm_head="head", final_norm={"weight": "norm"}, layers=layers)


register_architecture(ToyConfig.architecture, ToyConfig)


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    folder = tmp_path_factory.mktemp("toy")
    cfg = config_from_dict({"architectures": ["ToyDecayForCausalLM"], "hidden": 48, "state": 24, "vocab": 97, "decay": 0.9})
    assert isinstance(cfg, ToyConfig)
    write_model_folder(cfg, 3, folder)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_steps_the_same_in_every_cutting(toy_folder, dtype):
    sess = Session(toy_folder, dtype=dtype, max_tokens=64 * 6, max_seqs=3, verbose=False)
    assert len(sess.cache.groups) == 2                      # one state group, one key/value group (layer 2 shares it)
    assert sess.cache.layers[2] is sess.cache.layers[1]
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (40, 9, 70)]
    slots = [sess.cache.alloc() for _ in seqs]
    whole = sess.stepper.step([StepEntry(s, t, list(range(len(t)))) for s, t in zip(slots, seqs)])
    whole = [w.float().cpu() for w in torch.split(whole, [len(t) for t in seqs])]
    for s in slots:
        sess.cache.free(s)
    scale = max(float(w.abs().max()) for w in whole)
    tol = (1e-4 if dtype == "float32" else 3e-2) * scale
    # token by token, in slots that were used before: the state must have been reset and must carry over
    for i, t in enumerate(seqs):
        slot = sess.cache.alloc()
        rows = [sess.stepper.step([StepEntry(slot, [tok], [0])]) for tok in t]
        sess.cache.free(slot)
        assert float((torch.cat(rows).float().cpu() - whole[i]).abs().max()) <= tol, f"request {i} token by token"
    # the state matters: a different decay gives different logits
    assert float(whole[0][-1].abs().max()) > 0
    sess.cache.check()


def test_toy_model_generates_through_the_entry_point(toy_folder):
    eng = Engine(toy_folder, dtype="float32", max_batch=2, max_context=64, use_graphs=False)
    outs = eng.generate_all([[1, 2, 3], [4, 5, 6, 7, 8], [9]], 6)
    assert [len(o) for o in outs] == [6, 6, 6]
    solo = Engine(toy_folder, dtype="float32", max_batch=1, max_context=64, use_graphs=False)
    assert solo.generate_all([[1, 2, 3], [4, 5, 6, 7, 8], [9]], 6) == outs


def test_state_mixer_under_captured_graphs(toy_folder, tmp_path):
    """A mixer that says it cannot be captured makes the loop decode step by step; one written in tensor
    operations decodes through replayed graphs, its state records updated inside them, and gives the same
    tokens as the step-by-step loop, for prompts of unequal length and a sequence that stops early."""
    prompts = [[1, 2, 3], [4, 5, 6, 7, 8], [9]]
    plain_loop = Engine(toy_folder, dtype="float32", max_batch=4, max_context=64, use_graphs=True)
    assert plain_loop.generator.use_graphs is False
    want = plain_loop.generate_all(prompts, 12)
    cfg = config_from_dict({"architectures": ["ToyDecayForCausalLM"], "hidden": 48, "state": 24, "vocab": 97, "decay": 0.9,
                            "mixer_kind": "toy_decay_graph"})
    write_model_folder(cfg, 3, tmp_path)                       # same seed and tensor names: the same weights
    eng = Engine(tmp_path, dtype="float32", max_batch=4, max_context=64, use_graphs=True)
    assert eng.generator.use_graphs is True
    assert eng.generate_all(prompts, 12) == want
    assert eng.generate_all(prompts, 12) == want              # state records were reset when the slots were taken again
    stop = {want[1][4]}
    stopped = eng.generate_all(prompts, 12, stop_token_ids=stop)
    for got, full in zip(stopped, want):
        cut = next((i for i, t in enumerate(full) if t in stop), len(full) - 1)
        assert got == full[:cut + 1]
    eng.session.cache.check()
