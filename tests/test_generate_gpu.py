"""Generation through the entry point on the GPU: greedy and sampled, with CUDA graphs and
without, against the plain loop; long decoding; stop tokens; slots used again."""

import pytest
import torch

from conftest import TINY, random_tokens
from plain import qwen3_plain as plain
from starter_b200.engine import Engine
from starter_b200.sampling import SamplingParams

pytestmark = pytest.mark.gpu


def tokens_agree(got, want, cfg, tensors, prompts, dtype, margin):
    """Token-exact, except where the plain logits hold a near-tie that rounding may flip:
    then the engine's token must be within ``margin`` of the plain maximum, and the
    comparison goes on along the engine's own sequence."""
    for b, (g, w) in enumerate(zip(got, want)):
        if g == w:
            continue
        assert len(g) == len(w)
        seq = list(prompts[b])
        for t, tok in enumerate(g):
            logits = plain.forward(cfg, tensors, seq, dtype)[-1]
            gap = float(logits.max() - logits[tok])
            assert gap <= margin * float(logits.abs().max()), f"request {b}, new token {t}: {tok} is {gap:.3g} below the maximum"
            seq.append(tok)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_tiny_a(tiny_folders, dtype, graphs):
    prompts = random_tokens(256, (5, 9, 12), seed=3)
    cfg, tensors = plain.read_folder(tiny_folders["A"])
    want = plain.generate(cfg, tensors, prompts, 8, dtype)
    eng = Engine(tiny_folders["A"], dtype=dtype, max_batch=4, max_context=128, use_graphs=graphs)
    steps = list(eng.generate(prompts, 8))
    assert len(steps) == 8 and all(len(s) == 3 and None not in s for s in steps)
    got = [[s[b] for s in steps] for b in range(3)]
    tokens_agree(got, want, cfg, tensors, prompts, dtype, 1e-4 if dtype == "float32" else 2e-2)
    again = list(eng.generate(prompts, 8))                                  # second call: state reset
    assert [[s[b] for s in again] for b in range(3)] == got
    assert eng.session.cache.slots.n_held == 0


@pytest.mark.parametrize("graphs", [False, True])
def test_sampled_tiny_b(tiny_folders, graphs):
    prompts = random_tokens(389, (1, 7, 16, 23), seed=4)
    eng = Engine(tiny_folders["B"], dtype="float32", max_batch=4, max_context=128, use_graphs=graphs)
    got = eng.generate_all(prompts, 10, temperature=0.8, seed=99)
    # The draw is a function of the logits: feed the engine's own sequences to the plain model and
    # redo every draw from the plain logits; a draw near an edge of the running sum may differ.
    cfg, tensors = plain.read_folder(tiny_folders["B"])
    for r, (p, new) in enumerate(zip(prompts, got)):
        assert len(new) == 10
        seq = list(p)
        for step, tok in enumerate(new):
            logits = plain.forward(cfg, tensors, seq, "float32")[-1]
            want, margin = plain.sample(logits, 0.8, 0, plain.uniform_from_counter(99, r, step))
            if margin > 1e-4:
                assert tok == want, f"request {r} step {step}: {tok} != {want} (margin {margin:.2g})"
            seq.append(tok)
    solo = Engine(tiny_folders["B"], dtype="float32", max_batch=1, max_context=128, use_graphs=graphs)
    assert solo.generate_all(prompts, 10, temperature=0.8, seed=99) == got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphs_and_eager_agree_over_a_long_decode(tiny_folders, dtype):
    """200 new tokens cross several cache pages; both ways of running the steps give the same tokens."""
    prompts = random_tokens(301, (3, 50, 64), seed=7)
    outs = []
    for graphs in (False, True):
        eng = Engine(tiny_folders["W"], dtype=dtype, max_batch=4, max_context=320, use_graphs=graphs)
        outs.append(eng.generate_all(prompts, 200))
    assert outs[0] == outs[1]
    cfg, tensors = plain.read_folder(tiny_folders["W"])
    if dtype == "float32":
        want = plain.generate(cfg, tensors, prompts[:1], 200, dtype)
        tokens_agree(outs[0][:1], want, cfg, tensors, prompts[:1], dtype, 1e-4)


def test_stop_tokens_and_slot_reuse(tiny_folders):
    prompts = random_tokens(256, (5, 9, 12, 30, 2), seed=3)
    cfg, tensors = plain.read_folder(tiny_folders["A"])
    free_run = plain.generate(cfg, tensors, prompts, 12, "float32")
    stop = {free_run[0][2], free_run[3][6]}
    want = plain.generate(cfg, tensors, prompts, 12, "float32", stop_token_ids=stop)
    for graphs in (False, True):
        eng = Engine(tiny_folders["A"], dtype="float32", max_batch=2, max_context=128, use_graphs=graphs)
        got = eng.generate_all(prompts, 12, stop_token_ids=stop)
        tokens_agree(got, want, cfg, tensors, prompts, "float32", 1e-4)
        assert eng.session.cache.slots.n_held == 0
        eng.session.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["M", "N"])
def test_greedy_on_the_tensor_core_kernels(tiny_folders, name, graphs):
    """The configurations whose head sizes put prefill and decode on the tensor-core attention kernels (the decode
    one with the q/k preparation inside), with unequal prompts, a window in M, replayed graphs and not."""
    dtype = "bfloat16"
    prompts = random_tokens(TINY[name]["vocab_size"], (70, 5, 131, 1), seed=23)
    cfg, tensors = plain.read_folder(tiny_folders[name])
    want = plain.generate(cfg, tensors, prompts, 10, dtype)
    eng = Engine(tiny_folders[name], dtype=dtype, max_batch=4, max_context=192, use_graphs=graphs)
    steps = list(eng.generate(prompts, 10))
    got = [[s[b] for s in steps] for b in range(len(prompts))]
    tokens_agree(got, want, cfg, tensors, prompts, dtype, 2e-2)
    again = list(eng.generate(prompts[:2], 10))                             # fewer requests, slots used again
    assert [[s[b] for s in again] for b in range(2)] == got[:2]
    assert eng.session.cache.slots.n_held == 0


def test_ended_sequences_leave_the_captured_batch(tiny_folders):
    """Under graphs a sequence that meets a stop token stops being computed: the loop drains the steps in
    flight and goes on with the graph of a smaller batch, and the survivors' tokens do not change."""
    prompts = random_tokens(389, (5, 9, 12, 30, 2, 17, 40, 3), seed=5)
    eng = Engine(tiny_folders["B"], dtype="float32", max_batch=8, max_context=128, use_graphs=True)
    free_run = eng.generate_all(prompts, 24, temperature=1.0, seed=11)       # sampled: the sequences do not repeat themselves
    decoder = eng.generator._decoder(SamplingParams(temperature=1.0))
    assert decoder.history == [[8, 23]]                      # one graph of 8 rows for all 23 decode steps
    # stop tokens that end six of the eight sequences early, at different steps, none of them within the first three
    early = {t for seq in free_run for t in seq[:3]}
    stop = set()
    for b in range(6):
        stop.add(next(t for t in free_run[b][3 + 2 * b:] if t not in early))
    got = eng.generate_all(prompts, 24, stop_token_ids=stop, temperature=1.0, seed=11)
    for b, (g, full) in enumerate(zip(got, free_run)):
        cut = next((i for i, t in enumerate(full) if t in stop), len(full) - 1)
        assert g == full[:cut + 1], f"request {b}"
    sizes = [size for size, _ in decoder.history]
    assert sizes[0] == 8 and sizes == sorted(sizes, reverse=True) and sizes[-1] <= 2, decoder.history
    assert sum(steps for _, steps in decoder.history) <= 23 + 3 * (len(sizes) - 1)   # at most the steps in flight are redone
    eager = Engine(tiny_folders["B"], dtype="float32", max_batch=8, max_context=128, use_graphs=False)
    assert eager.generate_all(prompts, 24, stop_token_ids=stop, temperature=1.0, seed=11) == got
    assert eng.session.cache.slots.n_held == 0
    eng.session.cache.check()


def test_a_new_seed_replays_the_same_graphs(tiny_folders):
    """Temperature, top-k and seed are data on the device: runs that differ in them share one set of captured graphs,
    and each gives the tokens of the step-by-step loop with the same settings."""
    prompts = random_tokens(389, (1, 7, 16), seed=6)
    eng = Engine(tiny_folders["B"], dtype="float32", max_batch=4, max_context=128, use_graphs=True)
    eager = Engine(tiny_folders["B"], dtype="float32", max_batch=4, max_context=128, use_graphs=False)
    outs = []
    for temperature, top_k, seed in [(0.8, 0, 1), (0.8, 0, 2), (1.3, 5, 2 ** 40 + 7), (0.8, 0, 1)]:
        outs.append(eng.generate_all(prompts, 10, temperature=temperature, top_k=top_k, seed=seed))
        assert outs[-1] == eager.generate_all(prompts, 10, temperature=temperature, top_k=top_k, seed=seed)
    assert outs[0] == outs[3] and outs[0] != outs[1]
    assert set(eng.generator._decoders) == {False}           # one decoder for every sampled run
    assert list(eng.generator._decoders[False].buckets) == [(4, False)]   # (sequences, very unequal lengths)
    eng.generate_all(prompts, 4)
    assert set(eng.generator._decoders) == {False, True}


def test_a_bad_token_raises_through_the_entry_point(tiny_folders):
    """A token id outside the vocabulary sets a status bit in the kernel instead of reading out of range; the
    loop raises it as StepError, with graphs and without, and the engine serves the next call."""
    from starter_b200.engine.step import StepError
    for graphs in (False, True):
        eng = Engine(tiny_folders["A"], dtype="float32", max_batch=2, max_context=64, use_graphs=graphs)
        with pytest.raises(StepError, match="outside the vocabulary"):
            eng.generate_all([[1, 2, 300]], 4)
        assert eng.session.cache.slots.n_held == 0
        assert len(eng.generate_all([[1, 2, 3]], 4)[0]) == 4


def test_a_captured_step_brings_its_status_with_its_tokens(tiny_folders):
    """Fed a token id outside the vocabulary, a replayed step raises its status bit in the word that is copied
    to the host with the step's tokens: the error comes before those tokens are handed out."""
    from starter_b200.engine.graph import GraphDecoder
    from starter_b200.engine.session import Session
    from starter_b200.engine.step import StepEntry, StepError
    sess = Session(tiny_folders["A"], dtype="float32", max_tokens=256, max_seqs=2, verbose=False)
    slot = sess.cache.alloc()
    sess.stepper.step([StepEntry(slot, [1, 2, 3], [])])
    sess.cache.reserve(slot, 16)
    decoder = GraphDecoder(sess, SamplingParams())
    with pytest.raises(StepError, match="outside the vocabulary"):
        list(decoder.run([slot], [256], [0], 1, 4))
    sess.cache.free(slot)
    slot = sess.cache.alloc()                                  # the same graph serves the next batch
    sess.stepper.step([StepEntry(slot, [1, 2, 3], [])])
    sess.cache.reserve(slot, 16)
    assert len(list(decoder.run([slot], [7], [0], 1, 4))) == 4
    sess.cache.free(slot)


def test_batches_of_very_unequal_lengths_take_the_kernel_that_shares_pages_out(tiny_folders, monkeypatch):
    """A batch whose longest sequence is several times the mean is served by the decode attention that shares all
    pages out evenly, in a graph of its own; a batch of equal lengths keeps the kernel whose blocks per sequence
    are a matter of shapes.  Both give the tokens of the plain implementation."""
    from starter_b200.csrc.ops import get_ops
    from starter_b200.engine.context import lengths_uneven
    assert lengths_uneven([900, 5, 7, 3, 9, 4, 6, 8]) and not lengths_uneven([100, 90, 120, 80]) and not lengths_uneven([500])
    ops = get_ops(verbose=False)
    monkeypatch.setattr(ops, "fuse_qk", False)
    calls = []
    inner = ops._balanced_scratch
    monkeypatch.setattr(ops, "_balanced_scratch", lambda *a: (calls.append(1), inner(*a))[1])
    folder = tiny_folders["M"]
    cfg, tensors = plain.read_folder(folder)
    eng = Engine(folder, dtype="bfloat16", max_batch=8, max_context=768)
    for lengths, balanced in (((600, 5, 7, 3, 9, 4, 6, 8), True), ((40, 44, 38, 41, 39, 45, 42, 40), False)):
        prompts = random_tokens(TINY["M"]["vocab_size"], lengths, seed=31)
        calls.clear()
        got = eng.generate_all(prompts, 6)
        assert bool(calls) == balanced, f"lengths {lengths}: the balanced kernel ran {len(calls)} times"
        tokens_agree(got, plain.generate(cfg, tensors, prompts, 6, "bfloat16"), cfg, tensors, prompts, "bfloat16", 2e-2)
    assert eng.session.cache.slots.n_held == 0
    assert set(eng.generator._decoder(SamplingParams()).buckets) == {(8, True), (8, False)}   # a graph for each kind of batch
