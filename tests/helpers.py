"""Ways of cutting the same requests into steps, shared by CPU and GPU tests."""

from __future__ import annotations

import torch

from starter_b200.engine.session import Session
from starter_b200.engine.step import StepEntry

from plain import qwen3_plain as plain

# Largest |difference| allowed, as a fraction of the largest |logit| of the plain implementation.
# float32: both sides are true 32-bit, the orders of summation differ.  bfloat16: both sides round
# at the same places, but a sum that lands on the other side of a rounding edge moves a value by
# one bfloat16 step (2^-8 relative), and a few of those meet in a logit.  Measured over the tiny
# configurations in every cutting: 0.003 to 0.010 of the scale; the reference allows itself 0.03
# against another implementation (tests/test_engine.py:50-53 there).
TOLERANCE = {"float32": 1e-4, "bfloat16": 2e-2}


def make_session(folder, dtype, ops=None, device=None, **kw):
    if ops is None:
        return Session(folder, dtype=dtype, device=device or "cuda:0", verbose=False, **kw)
    return Session(folder, dtype=dtype, device=device or "cpu", ops=ops, **kw)


def plain_logits(folder, seqs, dtype):
    cfg, tensors = plain.read_folder(folder)
    return [plain.forward(cfg, tensors, s, dtype) for s in seqs]


def run_whole(sess, seqs, together=False):
    """Each request alone and whole (or all of them in one ragged step); logits at every position."""
    outs = []
    groups = [list(range(len(seqs)))] if together else [[i] for i in range(len(seqs))]
    outs = [None] * len(seqs)
    for group in groups:
        slots = [sess.cache.alloc() for _ in group]
        out = sess.stepper.step([StepEntry(sl, seqs[i], list(range(len(seqs[i])))) for sl, i in zip(slots, group)])
        for i, part in zip(group, torch.split(out, [len(seqs[i]) for i in group])):
            outs[i] = part.float().cpu()
        for sl in slots:
            sess.cache.free(sl)
    sess.stepper.raise_on_status()
    sess.cache.check()
    return outs


def run_tail_by_one(sess, seqs, tail=32):
    """All but the last ``tail`` tokens in one step, then the rest one token a step; requests one after another."""
    outs = []
    for s in seqs:
        slot = sess.cache.alloc()
        cut = max(1, len(s) - tail)
        parts = [sess.stepper.step([StepEntry(slot, s[:cut], list(range(cut)))])]
        for t in s[cut:]:
            parts.append(sess.stepper.step([StepEntry(slot, [t], [0])]))
        outs.append(torch.cat(parts).float().cpu())
        sess.cache.free(slot)
    sess.stepper.raise_on_status()
    sess.cache.check()
    return outs


def poison_cache(sess):
    """Fill every key/value page with NaN (only when no sequence is live): a read of a page that a
    finished sequence left behind then shows in the logits."""
    assert sess.cache.slots.n_held == 0
    for g in sess.cache.groups:
        if hasattr(g, "k"):
            g.k.fill_(float("nan"))
            g.v.fill_(float("nan"))


def run_ragged_batches(sess, seqs, batch_size, prefix_fraction=0.5, poison=False):
    """Batches of unequal requests, one after another: a ragged first step with a prefix of each
    request, then one token per live request per step; shorter requests end earlier and leave."""
    outs = [None] * len(seqs)
    for b0 in range(0, len(seqs), batch_size):
        ids = list(range(b0, min(b0 + batch_size, len(seqs))))
        slots = {i: sess.cache.alloc() for i in ids}
        cut = {i: max(1, int(len(seqs[i]) * prefix_fraction)) for i in ids}
        parts = {i: [] for i in ids}
        out = sess.stepper.step([StepEntry(slots[i], seqs[i][:cut[i]], list(range(cut[i]))) for i in ids])
        for i, part in zip(ids, torch.split(out, [cut[i] for i in ids])):
            parts[i].append(part)
        t = 0
        while True:
            live = [i for i in ids if cut[i] + t < len(seqs[i])]
            if not live:
                break
            out = sess.stepper.step([StepEntry(slots[i], [seqs[i][cut[i] + t]], [0]) for i in live])
            for j, i in enumerate(live):
                parts[i].append(out[j:j + 1])
            for i in ids:  # a request that just ended gives its slot back while the others go on
                if cut[i] + t + 1 == len(seqs[i]) and i in slots:
                    sess.cache.free(slots.pop(i))
            t += 1
        for i in list(slots):
            sess.cache.free(slots.pop(i))
        for i in ids:
            outs[i] = torch.cat(parts[i]).float().cpu()
        if poison:
            poison_cache(sess)
    sess.stepper.raise_on_status()
    sess.cache.check()
    return outs


def assert_close(got, ref, dtype, what):
    scale = max(float(r.abs().max()) for r in ref)
    for i, (g, r) in enumerate(zip(got, ref)):
        assert g.shape == r.shape, f"{what}: request {i} has shape {tuple(g.shape)}, expected {tuple(r.shape)}"
        diff = (g - r).abs()
        worst = float(diff.max())
        if not worst <= TOLERANCE[dtype] * scale:
            pos = int(diff.max(dim=1).values.argmax())
            raise AssertionError(f"{what}: request {i} (length {len(r)}) differs by {worst:.3g} "
                                 f"(allowed {TOLERANCE[dtype] * scale:.3g}); first worst position {pos}")
