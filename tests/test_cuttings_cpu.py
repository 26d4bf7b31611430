"""The step function's host side (cache paging, ragged batches, chunked steps, slot reuse),
driven on a CPU through the emulated kernels and compared with the plain implementation."""

import pytest

from conftest import TINY, random_tokens
from emulated_ops import EmulatedOps
from helpers import assert_close, make_session, plain_logits, run_ragged_batches, run_tail_by_one, run_whole

LENGTHS = (5, 150, 77, 1, 64, 65)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_every_cutting_matches_plain(tiny_folders, name, dtype):
    folder = tiny_folders.for_dtype(name, dtype)
    seqs = random_tokens(TINY[name]["vocab_size"], LENGTHS, seed=11)
    ref = plain_logits(folder, seqs, dtype)
    # max_step_tokens below the longest request: its prompt runs as several forward passes
    sess = make_session(folder, dtype, ops=EmulatedOps(), max_tokens=64 * 10, max_seqs=4, max_step_tokens=48, max_rows=100)
    assert_close(run_whole(sess, seqs), ref, dtype, "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], dtype, "one ragged step")
    assert_close(run_tail_by_one(sess, seqs), ref, dtype, "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, dtype, "ragged batches, freed pages poisoned")
    assert_close(run_whole(sess, seqs[:2]), ref[:2], dtype, "whole again, in poisoned slots")
    assert sess.cache.slots.n_held == 0
