"""The engine on the GPU against the plain implementation, in every way of cutting the work."""

import pytest
import torch

from conftest import TINY, random_tokens
from helpers import assert_close, make_session, plain_logits, run_ragged_batches, run_tail_by_one, run_whole

pytestmark = pytest.mark.gpu
LENGTHS = (5, 150, 77, 1, 64, 65, 33)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_every_cutting_matches_plain(tiny_folders, name, dtype):
    folder = tiny_folders.for_dtype(name, dtype)
    seqs = random_tokens(TINY[name]["vocab_size"], LENGTHS, seed=11)
    ref = plain_logits(folder, seqs, dtype)
    sess = make_session(folder, dtype, max_tokens=64 * 10, max_seqs=4, max_step_tokens=48, max_rows=100)
    assert_close(run_whole(sess, seqs), ref, dtype, "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], dtype, "one ragged step")
    assert_close(run_tail_by_one(sess, seqs), ref, dtype, "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, dtype, "ragged batches, freed pages poisoned")
    assert_close(run_whole(sess, seqs[:2]), ref[:2], dtype, "whole again, in poisoned slots")
    assert sess.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tiny_folders, dtype):
    """Sequences of one, two and three tokens, alone and in one step: position 0 has a single key."""
    folder = tiny_folders.for_dtype("B", dtype)
    seqs = random_tokens(TINY["B"]["vocab_size"], (1, 2, 3, 1), seed=13)
    ref = plain_logits(folder, seqs, dtype)
    sess = make_session(folder, dtype, max_tokens=64 * 4, max_seqs=4)
    assert_close(run_whole(sess, seqs), ref, dtype, "alone")
    assert_close(run_whole(sess, seqs, together=True), ref, dtype, "together")
    assert_close(run_tail_by_one(sess, seqs), ref, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dependent_launch_changes_no_bit(tiny_folders, dtype):
    """Kernels that may start before their predecessor has ended (the default) give the very same logits as
    kernels that run strictly one after another: every one of them waits before it touches earlier results."""
    folder = tiny_folders["A"]
    seqs = random_tokens(TINY["A"]["vocab_size"], (150, 9, 64), seed=17)
    got = {}
    for on in (False, True):
        sess = make_session(folder, dtype, max_tokens=64 * 8, max_seqs=4, dependent_launch=on)
        got[on] = run_whole(sess, seqs, together=True) + run_tail_by_one(sess, seqs)
    for a, b in zip(got[False], got[True]):
        assert torch.equal(a, b)
    assert_close(got[True][:3], plain_logits(folder, seqs, dtype), dtype, "dependent launch")


@pytest.mark.parametrize("route", ["stream", "balanced", "balanced fused", "slices", "folded", "folded slices"])
def test_other_kernel_routes_through_the_whole_engine(tiny_folders, monkeypatch, route):
    """The shape rules send the test configurations to a few of the kernels only.  Here the rules are bent so
    that the whole engine runs on the others: the TMA + tcgen05 product for every matrix (batches of 12), the
    balanced decode attention (with the q/k preparation as a kernel of its own, the default, and inside it), and K slices / key splits that meet in
    clusters; and the decode products that take the norm before them and the residual sum after them into
    themselves (off by default: slower than the norm kernel as measured).  Freed pages are poisoned between batches."""
    from starter_b200.csrc.ops import get_ops
    ops = get_ops(verbose=False)
    if route == "stream":
        monkeypatch.setattr(ops, "STREAM_MIN_WORK", 0)
        monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 0)
        batch = 12
    elif route.startswith("balanced"):
        monkeypatch.setattr(ops, "force_decode_route", "balanced")
        monkeypatch.setattr(ops, "fuse_qk_balanced", route == "balanced fused")
        batch = 5
    elif route == "slices":
        monkeypatch.setattr(ops, "skinny_splits", lambda blocks, K: 3)
        monkeypatch.setattr(ops, "decode_splits", lambda *a: 3)
        batch = 4
    else:
        monkeypatch.setattr(ops, "FOLD_MAX_ROWS", 16)
        if route == "folded slices":
            monkeypatch.setattr(ops, "skinny_splits", lambda blocks, K: 3)
        batch = 5 if route == "folded" else 11
        folded = []
        inner = ops._skinny

        def watched(a, w, n_out, gate_up, out_float32, norm=None, add_to=None):
            folded.append((norm is not None and len(norm) == 3, add_to is not None))
            return inner(a, w, n_out, gate_up, out_float32, norm, add_to)
        monkeypatch.setattr(ops, "_skinny", watched)
    folder, dtype = tiny_folders["M"], "bfloat16"
    lengths = (5, 150, 77, 1, 64, 65, 33, 90, 129, 12, 70, 200, 3)
    seqs = random_tokens(TINY["M"]["vocab_size"], lengths, seed=19)
    ref = plain_logits(folder, seqs, dtype)
    sess = make_session(folder, dtype, max_tokens=64 * 40, max_seqs=batch, max_step_tokens=96)
    before = ops.launches
    assert_close(run_ragged_batches(sess, seqs, batch_size=batch, poison=True), ref, dtype, f"ragged batches, route {route}")
    assert ops.launches > before
    assert sess.cache.slots.n_held == 0
    if route.startswith("folded"):   # norms were read from the statistics that the sums left, and sums were taken
        assert (True, False) in folded and (False, True) in folded
