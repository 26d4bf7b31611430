"""Decode steps captured as CUDA graphs and replayed with the host a few steps behind.

The reference captures ``tok.copy_(decode().argmax(-1))`` once per plan and
replays it, copying each step's tokens to pinned host memory behind an event
and waiting on that event only after the next steps are queued
(engine/engine.py:198-218, 401-419).  The same here, over this library's step:
a graph per batch size holds embedding, layers, final norm, output head, token
selection, the feed of the new token into the next step's input, and the
length update; everything a replay needs lives in device buffers that the
host fills once per batch.  Batch sizes are rounded up to a power of two; the
rows added that way belong to the cache's null slot and change no result.
"""

from __future__ import annotations

from typing import Iterator, List, Optional, Sequence

import torch

from ..sampling.sampler import SamplingParams, select
from .context import StepContext


def bucket_size(n: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return b


class _Bucket:
    def __init__(self, session, size: int, sampling: SamplingParams):
        self.session = session
        self.size = size
        self.sampling = sampling
        dev = session.device
        cache = session.cache
        i32 = dict(dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(size, **i32)
        self.seq_slot = torch.full((size,), cache.null_slot, **i32)
        self.cu_q = torch.arange(size + 1, **i32)
        self.row_seq = torch.arange(size, **i32)
        self.request_ids = torch.zeros(size, **i32)
        self.steps = torch.zeros(size, **i32)
        self.ctx = StepContext(
            runtime=session.runtime, cache=cache, n_seqs=size, n_rows=size, max_q_len=1,
            kv_bound=cache.max_seq_tokens, seq_slot=self.seq_slot, cu_q=self.cu_q, row_seq=self.row_seq,
            lengths=cache.lengths, status=session.stepper.status)
        self.graph: Optional[torch.cuda.CUDAGraph] = None

    def body(self) -> None:
        model, ops = self.session.model, self.session.runtime.ops
        stream = model.hidden(self.ctx, self.tokens)
        logits = model.logits(self.ctx, stream, None)
        new = select(ops, logits, self.sampling, self.request_ids, self.steps, advance=True)
        ops.advance_lengths(self.ctx)
        self.tokens.copy_(new)

    def capture(self) -> None:
        # One pass outside the graph, with every row on the null slot: libraries set themselves up
        # and nothing of a live sequence is touched.
        self.session.cache.flush()
        side = torch.cuda.Stream(device=self.session.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.body()

    def load(self, slots: Sequence[int], tokens: Sequence[int], request_ids: Sequence[int], first_step: int) -> None:
        cache = self.session.cache
        pad = self.size - len(slots)
        packed = torch.tensor(list(slots) + [cache.null_slot] * pad + list(tokens) + [0] * pad
                              + list(request_ids) + [0] * pad + [first_step] * self.size, dtype=torch.int32)
        packed = packed.pin_memory().to(self.session.device, non_blocking=True).view(4, self.size)
        self.seq_slot.copy_(packed[0])
        self.tokens.copy_(packed[1])
        self.request_ids.copy_(packed[2])
        self.steps.copy_(packed[3])


class GraphDecoder:
    """Runs the decode steps of one batch through a captured graph, ``depth`` steps in flight."""

    def __init__(self, session, sampling: SamplingParams, depth: int = 3):
        self.session = session
        self.sampling = sampling
        self.depth = depth
        self.buckets = {}

    def bucket(self, n: int) -> _Bucket:
        size = bucket_size(n)
        b = self.buckets.get(size)
        if b is None:
            b = self.buckets[size] = _Bucket(self.session, size, self.sampling)
            b.capture()
        return b

    def run(self, slots: Sequence[int], tokens: Sequence[int], request_ids: Sequence[int], first_step: int,
            n_steps: int, stop=frozenset()) -> Iterator[List[Optional[int]]]:
        """Feed ``tokens`` and decode ``n_steps`` steps; yields each step's new tokens in the order of
        ``slots`` (None for a sequence that has met a stop token).  Ends early when all have."""
        sess = self.session
        cache = sess.cache
        n = len(slots)
        b = self.bucket(n)
        cache.flush()
        b.load(slots, tokens, request_ids, first_step)
        host = torch.empty((self.depth, b.size), dtype=torch.int32, pin_memory=True)
        events = [torch.cuda.Event() for _ in range(self.depth)]
        live = [True] * n
        launched = yielded = 0
        while yielded < n_steps:
            while launched < n_steps and launched - yielded < self.depth:
                b.graph.replay()
                host[launched % self.depth].copy_(b.tokens, non_blocking=True)
                events[launched % self.depth].record()
                for s in slots:
                    cache.advance_host(s, 1)
                launched += 1
            events[yielded % self.depth].synchronize()
            toks = host[yielded % self.depth][:n].tolist()
            yielded += 1
            out = [t if alive else None for t, alive in zip(toks, live)]
            for i, t in enumerate(toks):
                if live[i] and t in stop:
                    live[i] = False
            yield out
            if not any(live):
                break
        sess.stepper.raise_on_status()
