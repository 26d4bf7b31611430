"""Two more toy parts defined here, in the test: a feed-forward that routes every row to one of several
experts (32-bit router logits), and a position encoding of its own (angles that grow linearly with the
column, over half of the head only).  They are registered, built into a toy architecture beside the
library's own parts, stepped in every cutting and run through generation without a change to the
library's files.  They are no model of anyone's: they show that the interfaces of the parts are enough."""

from dataclasses import dataclass

import pytest
import torch

from starter_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelConfig, ModelSpec, NormSpec, RopeSpec,
                                 TensorNames, config_from_dict, register_architecture)
from starter_b200.engine import Engine, Session, StepEntry
from starter_b200.parts import build_part, register_part
from starter_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class LinearAnglesSpec:
    step: float
    rotary_dim: int
    kind: str = "toy_linear_angles"


class LinearAngles:
    """angle(position, j) = position * step * (j + 1): a rotary table with frequencies of its own, over the first
    ``rotary_dim`` columns of a head.  The attention part only asks for fused_rotary()."""

    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.cos = self.sin = None

    def prepare(self, n_positions):
        if self.cos is not None and self.cos.shape[0] >= n_positions:
            return
        j = torch.arange(1, self.spec.rotary_dim // 2 + 1, dtype=torch.float32)
        angles = torch.arange(n_positions, dtype=torch.float32)[:, None] * (self.spec.step * j)[None, :]
        self.cos = angles.cos().to(self.runtime.dtype).to(self.runtime.device).contiguous()
        self.sin = angles.sin().to(self.runtime.dtype).to(self.runtime.device).contiguous()

    def fused_rotary(self):
        return self.cos, self.sin, self.spec.rotary_dim


register_part("position", "toy_linear_angles", LinearAngles)


@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    intermediate_size: int
    n_experts: int
    kind: str = "toy_routed"


class RoutedFF:
    """Every row goes to the expert with the largest router logit (32-bit logits, lowest index on ties) and is
    scaled by that expert's softmax probability: out = p_e * down_e(silu(up_e(h)))."""

    @staticmethod
    def weight_shapes(spec):
        e, i, h = spec.n_experts, spec.intermediate_size, spec.hidden_size
        return {"router": (e, h), "up": (e * i, h), "down": (e * h, i)}

    def __init__(self, spec, weights, runtime):
        self.spec, self.ops = spec, runtime.ops
        e, i, h = spec.n_experts, spec.intermediate_size, spec.hidden_size
        self.router = self.ops.prepare_matrix(weights["router"])
        self.up = [self.ops.prepare_matrix(weights["up"][k * i:(k + 1) * i]) for k in range(e)]
        self.down = [self.ops.prepare_matrix(weights["down"][k * h:(k + 1) * h]) for k in range(e)]

    def prepare(self, cache):
        pass

    def forward(self, ctx, h):
        logits = self.ops.linear(h, self.router, out_float32=True)
        choice = logits.argmax(dim=-1)
        gate = torch.softmax(logits, dim=-1).gather(1, choice[:, None])
        out = torch.zeros_like(h)
        for k in range(self.spec.n_experts):
            rows = (choice == k).nonzero().flatten()
            if rows.numel():
                u = self.ops.linear(h.index_select(0, rows).contiguous(), self.up[k])
                a = torch.nn.functional.silu(u.float()).to(h.dtype)
                d = self.ops.linear(a, self.down[k]).float() * gate.index_select(0, rows)
                out.index_copy_(0, rows, d.to(h.dtype))
        return out


register_part("ff", "toy_routed", RoutedFF)


@dataclass(frozen=True)
class ToyRoutedConfig(ModelConfig):
    hidden: int
    inter: int
    experts: int
    vocab: int
    step: float
    architecture = "ToyRoutedForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(hidden=raw["hidden"], inter=raw["inter"], experts=raw["experts"], vocab=raw["vocab"], step=raw["step"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden": self.hidden, "inter": self.inter, "experts": self.experts,
                "vocab": self.vocab, "step": self.step}

    def model_spec(self):
        norm = NormSpec(size=self.hidden, eps=1e-5)
        toy_att = AttentionSpec(hidden_size=self.hidden, num_heads=3, num_kv_heads=1, head_dim=32, scale=0.2,
                                qk_norm=NormSpec(size=32, eps=1e-5), position=LinearAnglesSpec(self.step, 16))
        own_att = AttentionSpec(hidden_size=self.hidden, num_heads=2, num_kv_heads=2, head_dim=64, scale=0.125,
                                position=RopeSpec(theta=10000.0, rotary_dim=64))
        layers = (
            BlockSpec(mixer_norm=norm, mixer=toy_att, ff_norm=norm, ff=RoutedSpec(self.hidden, self.inter, self.experts)),
            BlockSpec(mixer_norm=norm, mixer=own_att, ff_norm=norm,
                      ff=GatedMLPSpec(hidden_size=self.hidden, intermediate_size=self.inter)),
        )
        return ModelSpec(hidden_size=self.hidden, vocab_size=self.vocab, layers=layers, final_norm=norm, tie_embeddings=False)

    def tensor_names(self):
        def att(p, norms):
            names = {r: p + r for r in ("q", "k", "v", "o")}
            if norms:
                names.update({"q_norm": p + "qn", "k_norm": p + "kn"})
            return names
        layers = [
            {"mixer_norm": {"weight": "l0.n1"}, "mixer": att("l0.", True), "ff_norm": {"weight": "l0.n2"},
             "ff": {"router": "l0.router", "up": "l0.up", "down": "l0.down"}},
            {"mixer_norm": {"weight": "l1.n1"}, "mixer": att("l1.", False), "ff_norm": {"weight": "l1.n2"},
             "ff": {"gate": "l1.gate", "up": "l1.up", "down": "l1.down"}},
        ]
        return TensorNames(embedding="embed", lm_head="head", final_norm={"weight": "norm"}, layers=layers)


register_architecture(ToyRoutedConfig.architecture, ToyRoutedConfig)
RAW = {"architectures": ["ToyRoutedForCausalLM"], "hidden": 40, "inter": 56, "experts": 3, "vocab": 83, "step": 0.05}


@pytest.fixture(scope="module")
def routed_folder(tmp_path_factory):
    folder = tmp_path_factory.mktemp("toy_routed")
    cfg = config_from_dict(RAW)
    assert isinstance(cfg, ToyRoutedConfig)
    write_model_folder(cfg, 5, folder)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_model_steps_the_same_in_every_cutting(routed_folder, dtype):
    sess = Session(routed_folder, dtype=dtype, max_tokens=64 * 8, max_seqs=3, verbose=False)
    assert len(sess.cache.groups) == 2                      # two key/value groups: the layers' head sizes differ
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 83, (n,), generator=g).tolist() for n in (70, 11, 33)]
    slots = [sess.cache.alloc() for _ in seqs]
    whole = sess.stepper.step([StepEntry(s, t, list(range(len(t)))) for s, t in zip(slots, seqs)])
    whole = [w.float().cpu() for w in torch.split(whole, [len(t) for t in seqs])]
    for s in slots:
        sess.cache.free(s)
    scale = max(float(w.abs().max()) for w in whole)
    tol = (1e-4 if dtype == "float32" else 3e-2) * scale
    # a prefix in one step, the rest token by token, in slots that were used before
    for i, t in enumerate(seqs):
        slot = sess.cache.alloc()
        cut = len(t) // 2
        rows = [sess.stepper.step([StepEntry(slot, t[:cut], list(range(cut)))])]
        rows += [sess.stepper.step([StepEntry(slot, [tok], [0])]) for tok in t[cut:]]
        sess.cache.free(slot)
        assert float((torch.cat(rows).float().cpu() - whole[i]).abs().max()) <= tol, f"request {i}, prefix then token by token"
    # positions matter: the same tokens one position later give other logits
    slot = sess.cache.alloc()
    shifted = sess.stepper.step([StepEntry(slot, [seqs[1][0]] + seqs[1], list(range(1, len(seqs[1]) + 1)))]).float().cpu()
    sess.cache.free(slot)
    if dtype == "float32":
        assert float((shifted - whole[1]).abs().max()) > 10 * tol
    sess.stepper.raise_on_status()
    sess.cache.check()


def test_routed_feed_forward_alone_against_its_formula(routed_folder):
    """The part by itself, 32-bit, against the formula written out; every expert gets rows."""
    sess = Session(routed_folder, dtype="float32", max_tokens=64, max_seqs=1, verbose=False)
    ff = sess.model.blocks[0].ff
    assert isinstance(ff, RoutedFF)
    h = torch.randn(50, 40, generator=torch.Generator().manual_seed(3)).cuda() * 3
    got = ff.forward(None, h)
    logits = h @ ff.router.T
    choice = logits.argmax(-1)
    assert set(choice.tolist()) == {0, 1, 2}
    want = torch.zeros_like(h)
    for r in range(h.shape[0]):
        k = int(choice[r])
        p = torch.softmax(logits[r], -1)[k]
        want[r] = p * (ff.down[k] @ torch.nn.functional.silu(ff.up[k] @ h[r]))
    assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max())


def test_position_part_alone_and_through_the_entry_point(routed_folder):
    sess = Session(routed_folder, dtype="float32", max_tokens=64 * 2, max_seqs=1, verbose=False)
    position = sess.model.blocks[0].mixer.position
    assert isinstance(position, LinearAngles)
    cos, sin, rotary_dim = position.fused_rotary()
    assert rotary_dim == 16 and cos.shape[1] == 8 and cos.shape[0] >= 128
    want = torch.cos(torch.tensor(100.0 * 0.05 * 3))
    assert abs(float(cos[100, 2]) - float(want)) < 1e-6
    eng = Engine(routed_folder, dtype="float32", max_batch=2, max_context=64, use_graphs=False)
    outs = eng.generate_all([[1, 2, 3], [4, 5, 6, 7, 8], [9]], 5)
    solo = Engine(routed_folder, dtype="float32", max_batch=1, max_context=64, use_graphs=False)
    assert solo.generate_all([[1, 2, 3], [4, 5, 6, 7, 8], [9]], 5) == outs
