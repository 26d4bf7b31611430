"""The layer sizes that are benchmarked (hidden 2,560, 32/8 heads of 128, intermediate 9,728, vocabulary
151,936), with 2 of the 36 layers, through the engine as the shape rules drive it: no rule is bent here.

At these sizes the rules pick what no tiny configuration reaches: the down projection cut into K slices
that meet in a cluster, four-warp blocks for gate/up, sixteen key splits through scratch at batch 1, the
balanced decode attention with the separate rotary kernel, cuBLAS products and the TMA + tcgen05 output
head at batch 64, tile-major copies of every matrix, the output projection's weights asked for from the
attention kernel.  The bfloat16 engine is held against the float32 engine on the same weights and, for a
short prompt and the decode steps after it, against the plain implementation.
"""

import pytest
import torch

from conftest import random_tokens
from helpers import TOLERANCE
from plain import qwen3_plain as plain
from starter_b200.config import config_from_dict
from starter_b200.engine.check import compare_dtypes
from starter_b200.engine.session import Session
from starter_b200.engine.step import StepEntry
from starter_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu

SIZES_4B_2_LAYERS = dict(architectures=["Qwen3ForCausalLM"], hidden_size=2560, intermediate_size=9728, num_hidden_layers=2,
                         num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rms_norm_eps=1e-6,
                         rope_theta=5000000.0, tie_word_embeddings=True)


def test_bfloat16_against_float32_at_the_benchmark_sizes():
    """Prompts of 319 (one token before a page's end) and 2,048 tokens, then six forced tokens at batch 1, 8 and 64."""
    report = compare_dtypes(config_from_dict(SIZES_4B_2_LAYERS), seed=0, prompt_lengths=(300, 2048), decode_batches=(1, 8, 64),
                            decode_steps=6)
    print(report)
    assert report["positions"] == 7 * (1 + 8 + 64)
    assert report["within_tolerance"], report
    assert report["max_rel_diff"] <= TOLERANCE["bfloat16"]
    assert report["argmax_agreement"] >= 0.5, report       # near-flat random logits: most, not all, choices agree


def test_bfloat16_against_plain_at_the_benchmark_sizes(tmp_path):
    """A prompt of 300 tokens whole, then decode across the page boundary at 320, batch 3 with unequal lengths."""
    cfg = config_from_dict(SIZES_4B_2_LAYERS)
    write_model_folder(cfg, 0, tmp_path, device="cuda")
    raw, tensors = plain.read_folder(tmp_path)
    seqs = random_tokens(cfg.vocab_size, (326, 70, 131), seed=31)
    ref = [plain.forward(raw, tensors, s, "bfloat16") for s in seqs]
    scale = max(float(r.abs().max()) for r in ref)
    sess = Session(tmp_path, dtype="bfloat16", max_tokens=64 * 12, max_seqs=3, verbose=False)
    cut = [300, 60, 120]
    slots = [sess.cache.alloc() for _ in seqs]
    rows = {i: [] for i in range(3)}
    out = sess.stepper.step([StepEntry(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, cut)])
    for i, part in enumerate(torch.split(out, cut)):
        rows[i].append(part.float().cpu())
    for t in range(26):
        live = [i for i in range(3) if cut[i] + t < len(seqs[i])]
        out = sess.stepper.step([StepEntry(slots[i], [seqs[i][cut[i] + t]], [0]) for i in live])
        for j, i in enumerate(live):
            rows[i].append(out[j:j + 1].float().cpu())
    sess.stepper.raise_on_status()
    for i in range(3):
        got = torch.cat(rows[i])
        assert got.shape == ref[i].shape
        worst = float((got - ref[i]).abs().max())
        assert worst <= TOLERANCE["bfloat16"] * scale, f"request {i}: {worst:.3g} of scale {scale:.3g}"
        assert float((got.argmax(-1) == ref[i].argmax(-1)).float().mean()) >= 0.5
