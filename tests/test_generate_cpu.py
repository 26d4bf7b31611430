"""The generation loop's decisions, on a CPU: batch planning, stop tokens, sequences that end
earlier, batches one after another, and token-exact agreement with the plain loop."""

import pytest

from conftest import TINY, random_tokens
from emulated_ops import EmulatedOps
from plain import qwen3_plain as plain
from starter_b200.cache import PAGE
from starter_b200.engine import BatchLimits, Engine, GenerationError, plan_batches


def test_plan_batches_respects_slots_and_pages():
    limits = BatchLimits(max_seqs=3, max_pages=10, max_seq_tokens=640)
    assert plan_batches([5, 9, 12, 1], 8, limits) == [[0, 1, 2], [3]]
    # 200 + 99 tokens = 5 pages each: two fit ten pages, the third starts a new batch
    assert plan_batches([200, 200, 200], 100, limits) == [[0, 1], [2]]
    assert plan_batches([], 4, limits) == []
    with pytest.raises(GenerationError, match="empty"):
        plan_batches([3, 0], 4, limits)
    with pytest.raises(GenerationError, match="exceed"):
        plan_batches([640], 2, limits)
    assert plan_batches([640], 1, limits) == [[0]]       # the last new token is never stored
    with pytest.raises(GenerationError, match="cache holds"):
        plan_batches([600], 10, BatchLimits(max_seqs=3, max_pages=5, max_seq_tokens=1000))


def engine_for(folder, dtype, **kw):
    return Engine(folder, dtype=dtype, device="cpu", ops=EmulatedOps(), **kw)


def test_greedy_generation_matches_plain_loop(tiny_folders):
    """Tiny A: batch of 3 with prompts of 5, 9 and 12 tokens, 8 greedy steps."""
    prompts = random_tokens(256, (5, 9, 12), seed=3)
    cfg, tensors = plain.read_folder(tiny_folders["A"])
    want = plain.generate(cfg, tensors, prompts, 8, "float32")
    eng = engine_for(tiny_folders["A"], "float32", max_batch=4, max_context=64)
    steps = list(eng.generate(prompts, 8))
    assert len(steps) == 8 and all(len(s) == 3 for s in steps)      # README.md:60-64
    assert [[s[b] for s in steps] for b in range(3)] == want
    assert eng.session.cache.slots.n_held == 0
    assert list(eng.generate(prompts, 0)) == []


def test_sampled_generation_matches_plain_loop(tiny_folders):
    """Tiny B: batch of 4 with prompts of 1, 7, 16 and 23 tokens, 10 steps at temperature 0.8."""
    prompts = random_tokens(389, (1, 7, 16, 23), seed=4)
    cfg, tensors = plain.read_folder(tiny_folders["B"])
    want = plain.generate(cfg, tensors, prompts, 10, "float32", temperature=0.8, top_k=20, seed=99)
    eng = engine_for(tiny_folders["B"], "float32", max_batch=4, max_context=64)
    assert eng.generate_all(prompts, 10, temperature=0.8, top_k=20, seed=99) == want
    # a request's tokens do not depend on the batch it runs in: one slot, four batches
    solo = engine_for(tiny_folders["B"], "float32", max_batch=1, max_context=64)
    assert solo.generate_all(prompts, 10, temperature=0.8, top_k=20, seed=99) == want


def test_stop_tokens_end_sequences_early(tiny_folders):
    prompts = random_tokens(256, (5, 9, 12), seed=3)
    cfg, tensors = plain.read_folder(tiny_folders["A"])
    free_run = plain.generate(cfg, tensors, prompts, 8, "float32")
    stop = {free_run[0][2], free_run[2][5]}
    want = plain.generate(cfg, tensors, prompts, 8, "float32", stop_token_ids=stop)
    assert len(want[0]) <= 3 and any(len(w) < 8 for w in want)
    eng = engine_for(tiny_folders["A"], "float32", max_batch=4, max_context=64)
    steps = list(eng.generate(prompts, 8, stop_token_ids=stop))
    got = [[s[b] for s in steps if s[b] is not None] for b in range(3)]
    assert got == want
    assert len(steps) == max(len(w) for w in want)                   # the loop ends with the last sequence
    for b in range(3):                                               # once ended, a sequence stays ended
        seen_none = False
        for s in steps:
            seen_none |= s[b] is None
            assert not (seen_none and s[b] is not None)
    assert eng.generate_all(prompts, 8, stop_token_ids=stop) == want


def test_batches_one_after_another_reuse_slots(tiny_folders):
    prompts = random_tokens(256, (3, 70, 20, 9, 41), seed=5)
    cfg, tensors = plain.read_folder(tiny_folders["A"])
    want = plain.generate(cfg, tensors, prompts, 5, "float32")
    eng = engine_for(tiny_folders["A"], "float32", max_batch=2, max_context=128)
    assert eng.generate_all(prompts, 5) == want
    assert eng.session.cache.slots.n_held == 0 and eng.session.cache.groups[0].pages.n_held == 0
    with pytest.raises(GenerationError, match="do not fit one batch"):
        list(eng.generate(prompts, 5))
    with pytest.raises(GenerationError, match="exceed"):
        eng.generate_all([list(range(200))], 5)
    assert eng.session.cache.slots.n_held == 0


def test_slots_come_back_when_the_caller_stops_listening(tiny_folders):
    eng = engine_for(tiny_folders["A"], "float32", max_batch=2, max_context=64)
    gen = eng.generate(random_tokens(256, (4, 6), seed=6), 10)
    next(gen)
    gen.close()
    assert eng.session.cache.slots.n_held == 0
    eng.session.cache.check()


def test_very_unequal_lengths_are_told_from_the_rest():
    """The hint that lets the kernels choose: the longest sequence holds more than three times the mean number of
    cache pages.  Lengths within a page of one another are equal, a single sequence is never unequal."""
    from starter_b200.engine.context import lengths_uneven
    assert not lengths_uneven([])
    assert not lengths_uneven([100000])
    assert not lengths_uneven([1, 63, 40, 7])                 # one page each
    assert not lengths_uneven([4096] * 64)
    assert not lengths_uneven([64, 2048, 700, 1300, 90, 1999])   # uniform in [64, 2048]: the longest is twice the mean
    assert lengths_uneven([16384] + [256] * 63)
    assert lengths_uneven([4096] + [256] * 7)
    assert not lengths_uneven([4096, 256])                    # two sequences: the longest can be at most twice the mean
