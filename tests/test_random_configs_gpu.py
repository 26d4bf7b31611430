"""Configurations drawn at random (head sizes, groups, widths, windows, vocabularies, step and row limits)
through every cutting in bfloat16, against the plain implementation, with freed pages poisoned.  The draw
is seeded: the same twelve configurations every time."""

import random

import pytest

from conftest import random_tokens
from helpers import assert_close, make_session, plain_logits, run_ragged_batches, run_tail_by_one, run_whole
from starter_b200.config import config_from_dict
from starter_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu


def draw(case: int):
    rng = random.Random(1000 + case)
    head_dim = rng.choice([64, 128, 128, 64, 48, 32])
    kv_heads = rng.choice([1, 2, 3, 4])
    heads = kv_heads * rng.choice([1, 2, 3, 4, 6, 8])
    layers = rng.choice([1, 2, 3])
    window = rng.choice([None, None, 40, 70, 130])
    raw = dict(architectures=["Qwen3ForCausalLM"], hidden_size=rng.choice([192, 256, 320, 520]),
               intermediate_size=rng.choice([264, 512, 1000]), num_hidden_layers=layers, num_attention_heads=heads,
               num_key_value_heads=kv_heads, head_dim=head_dim, vocab_size=rng.choice([301, 1000, 4099]),
               rms_norm_eps=rng.choice([1e-6, 1e-5]), rope_theta=rng.choice([1e4, 1e6]),
               tie_word_embeddings=rng.choice([True, False]))
    if window:
        raw.update(use_sliding_window=True, sliding_window=window,
                   layer_types=[rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)])
    lengths = [rng.choice([1, 2, 5, 33, 63, 64, 65, 100, 129, 200, 260]) for _ in range(6)]
    limits = dict(max_step_tokens=rng.choice([48, 128, 512]), max_rows=rng.choice([100, 8192]))
    return raw, lengths, limits, rng.choice([2, 3, 4])


@pytest.mark.parametrize("case", range(12))
def test_a_random_configuration_in_every_cutting(tmp_path, case):
    raw, lengths, limits, batch = draw(case)
    write_model_folder(config_from_dict(raw), case, tmp_path)
    seqs = random_tokens(raw["vocab_size"], lengths, seed=case)
    dtype = "bfloat16"
    ref = plain_logits(tmp_path, seqs, dtype)
    sess = make_session(tmp_path, dtype, max_tokens=64 * 24, max_seqs=4, **limits)
    what = f"{raw}, lengths {lengths}, {limits}"
    assert_close(run_whole(sess, seqs), ref, dtype, "alone and whole: " + what)
    assert_close(run_tail_by_one(sess, seqs), ref, dtype, "tail one by one: " + what)
    assert_close(run_ragged_batches(sess, seqs, batch_size=batch, poison=True), ref, dtype, "ragged batches, poisoned: " + what)
    assert sess.cache.slots.n_held == 0
