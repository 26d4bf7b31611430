"""The generation loop above the step function.

The reference runs one batch of equal-length prompts for exactly
``max_new_tokens`` steps: one prefill, then one decode per step, each token
copied to pinned host memory behind an event while the next step is already
queued (engine/engine.py:388-419), and it never stops at a token
(README.md:60-64).  Here prompts may be unequal, a set of stop tokens ends a
sequence early, ended sequences leave the batch, and more requests than fit
run as batches one after another, their slots used again.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Iterator, List, Optional, Sequence

import torch

from ..cache.cache import PAGE
from ..sampling.sampler import SamplingParams, select
from .step import StepEntry


class GenerationError(ValueError):
    """A request that cannot be served (empty prompt, longer than the cache allows)."""


@dataclass
class BatchLimits:
    max_seqs: int        # sequences a batch may hold
    max_pages: int       # cache pages a batch may hold
    max_seq_tokens: int  # tokens one sequence may hold


def pages_needed(prompt_len: int, max_new_tokens: int) -> int:
    """Pages a request holds at its longest: the prompt and every new token but the last,
    which is returned and never fed back."""
    return (prompt_len + max(max_new_tokens - 1, 0) + PAGE - 1) // PAGE


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, limits: BatchLimits) -> List[List[int]]:
    """Requests, in order, packed into batches that fit the slots and the pages."""
    batches: List[List[int]] = []
    current: List[int] = []
    pages = 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise GenerationError(f"request {i} has an empty prompt")
        if n + max_new_tokens - 1 > limits.max_seq_tokens:
            raise GenerationError(f"request {i}: {n} prompt tokens + {max_new_tokens} new tokens exceed the "
                                  f"{limits.max_seq_tokens} tokens a sequence may hold")
        need = pages_needed(n, max_new_tokens)
        if need > limits.max_pages:
            raise GenerationError(f"request {i} needs {need * PAGE} tokens of cache; the cache holds {limits.max_pages * PAGE}")
        if current and (len(current) == limits.max_seqs or pages + need > limits.max_pages):
            batches.append(current)
            current, pages = [], 0
        current.append(i)
        pages += need
    if current:
        batches.append(current)
    return batches


class Generator:
    """Generation over a Session: batches of unequal prompts, stop tokens, early finishers."""

    def __init__(self, session, use_graphs: bool = True):
        self.session = session
        # a part that cannot run inside a captured graph (it reads device values on the host, say) sets
        # ``capturable = False``; decoding then runs step by step
        self.use_graphs = (use_graphs and session.device.type == "cuda"
                           and all(getattr(part, "capturable", True) for part in session.model.parts()))
        self._decoders = {}

    def limits(self) -> BatchLimits:
        cache = self.session.cache
        return BatchLimits(max_seqs=cache.n_slots, max_pages=cache.tokens_free() // PAGE, max_seq_tokens=cache.max_seq_tokens)

    # ---- one batch -----------------------------------------------------------------------

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                       sampling: SamplingParams = SamplingParams(), stop_token_ids: Iterable[int] = (),
                       request_ids: Optional[Sequence[int]] = None) -> Iterator[List[Optional[int]]]:
        """Yield, per step, one new token per sequence (None for a sequence that has ended).

        All prompts run in one step; then every live sequence adds one token a step.  A sequence
        ends after ``max_new_tokens`` tokens or with its first stop token, which is its last output.
        The loop ends when every sequence has ended.  Slots are given back however the loop ends.
        """
        sess = self.session
        cache, stepper, ops = sess.cache, sess.stepper, sess.runtime.ops
        B = len(prompts)
        if max_new_tokens < 1 or B == 0:  # engine/engine.py:586-587
            return
        stop = frozenset(int(t) for t in stop_token_ids)
        ids = list(request_ids) if request_ids is not None else list(range(B))
        batches = plan_batches([len(p) for p in prompts], max_new_tokens, self.limits())
        if len(batches) != 1:
            raise GenerationError(f"{B} requests do not fit one batch ({cache.n_slots} slots, "
                                  f"{cache.tokens_free()} free tokens of cache); use run() for batches one after another")
        slots = [cache.alloc() for _ in range(B)]
        try:
            for s, p in zip(slots, prompts):
                cache.reserve(s, len(p) + max_new_tokens - 1)
            dev = sess.device
            req_dev = torch.tensor(ids, dtype=torch.int32, device=dev)
            logits = stepper.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
            step_dev = torch.zeros(B, dtype=torch.int32, device=dev)
            tokens = select(ops, logits, sampling, req_dev, step_dev).tolist()
            stepper.raise_on_status()
            live = list(range(B))
            produced = 1
            while True:
                out: List[Optional[int]] = [None] * B
                for j, b in enumerate(live):
                    out[b] = tokens[j]
                yield out
                live_next, feed = [], []
                for j, b in enumerate(live):
                    if tokens[j] not in stop and produced < max_new_tokens:
                        live_next.append(b)
                        feed.append(tokens[j])
                if not live_next:
                    return
                if self.use_graphs:
                    decoder = self._decoder(sampling)
                    for step_tokens in decoder.run([slots[b] for b in live_next], feed, [ids[b] for b in live_next],
                                                   produced, max_new_tokens - produced, stop, sampling):
                        out = [None] * B
                        for b, t in zip(live_next, step_tokens):
                            out[b] = t
                        if any(t is not None for t in out):
                            yield out
                    return
                live = live_next
                logits = stepper.step([StepEntry(slots[b], [t], [0]) for b, t in zip(live, feed)])
                req_dev = torch.tensor([ids[b] for b in live], dtype=torch.int32, device=dev)
                step_dev = torch.full((len(live),), produced, dtype=torch.int32, device=dev)
                tokens = select(ops, logits, sampling, req_dev, step_dev).tolist()
                stepper.raise_on_status()
                produced += 1
        finally:
            for s in slots:
                cache.free(s)

    def _decoder(self, sampling: SamplingParams):
        """One set of captured graphs for greedy runs, one for sampled runs: temperature, top-k and seed
        are data that the sampling kernel reads on the device, so a new seed captures nothing."""
        from .graph import GraphDecoder
        dec = self._decoders.get(sampling.greedy)
        if dec is None:
            dec = self._decoders[sampling.greedy] = GraphDecoder(self.session, sampling.greedy)
        return dec

    # ---- many requests -------------------------------------------------------------------

    def run(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, sampling: SamplingParams = SamplingParams(),
            stop_token_ids: Iterable[int] = ()) -> List[List[int]]:
        """New tokens of every request; requests run as batches one after another."""
        outputs: List[List[int]] = [[] for _ in prompts]
        if max_new_tokens < 1:
            return outputs
        for batch in plan_batches([len(p) for p in prompts], max_new_tokens, self.limits()):
            for step in self.generate_batch([prompts[i] for i in batch], max_new_tokens, sampling, stop_token_ids,
                                            request_ids=batch):
                for i, tok in zip(batch, step):
                    if tok is not None:
                        outputs[i].append(tok)
        return outputs
