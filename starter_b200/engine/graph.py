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

What the reference does not have: temperature, top-k and seed are read by the
sampling kernel from a small device buffer that the host fills per batch, so
one graph per batch size serves every sampled run (and one more the greedy
ones); a sequence that meets a stop token leaves the captured batch (its row
is pointed at the null slot, and once the live sequences fit a smaller batch
size the steps in flight are drained and the rest moves to that graph); each
step's status word comes to the host with the step's tokens and is checked
before they are handed out.
"""

from __future__ import annotations

import struct
from contextlib import nullcontext
from typing import Iterator, List, Optional, Sequence

import torch

from ..sampling.sampler import SamplingParams, select
from .context import StepContext, lengths_uneven
from .step import raise_status_bits


def bucket_size(n: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return b


class _Bucket:
    """Device buffers and the captured graph of one batch size."""

    def __init__(self, session, size: int, greedy: bool, uneven: bool = False):
        self.session = session
        self.size = size
        self.greedy = greedy
        self.uneven = uneven     # captured for batches of very unequal lengths (the kernels may be others)
        dev = session.device
        cache = session.cache
        i32 = dict(dtype=torch.int32, device=dev)
        self.out = torch.zeros(size + 1, **i32)      # the step's tokens, then its status word: one copy brings both
        self.tokens = self.out[:size]
        self.status = self.out[size:]
        self.seq_slot = torch.full((size,), cache.null_slot, **i32)
        self.cu_q = torch.arange(size + 1, **i32)
        self.row_seq = torch.arange(size, **i32)
        self.request_ids = torch.zeros(size, **i32)
        self.steps = torch.zeros(size, **i32)
        self.sample_params = torch.zeros(4, **i32)   # temperature (float bits), top_k, seed low, seed high
        self.ctx = StepContext(
            runtime=session.runtime, cache=cache, n_seqs=size, n_rows=size, max_q_len=1,
            kv_bound=cache.max_seq_tokens, seq_slot=self.seq_slot, cu_q=self.cu_q, row_seq=self.row_seq,
            lengths=cache.lengths, status=self.status, uneven=uneven)
        self.graph: Optional[torch.cuda.CUDAGraph] = None

    def body(self) -> None:
        model, ops = self.session.model, self.session.runtime.ops
        into = getattr(ops, "status_into", None)
        with into(self.status) if into is not None else nullcontext():
            stream = model.hidden(self.ctx, self.tokens)
            logits = model.logits(self.ctx, stream, None)
            if self.greedy:
                new = ops.argmax(logits)
            else:
                new = ops.sample(logits, 1.0, 0, 0, self.request_ids, self.steps, advance=True,
                                 device_params=self.sample_params)
            ops.advance_lengths(self.ctx)
        self.tokens.copy_(new)

    def capture(self) -> None:
        # One pass outside the graph, with every row on the null slot: libraries set themselves up
        # and nothing of a live sequence is touched.
        self.session.cache.flush()
        self.sample_params.copy_(torch.tensor(pack_sampling(SamplingParams(temperature=1.0)), dtype=torch.int32))
        side = torch.cuda.Stream(device=self.session.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.status.zero_()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.body()

    def load(self, slots: Sequence[int], tokens: Sequence[int], request_ids: Sequence[int], first_step: int,
             sampling: SamplingParams = SamplingParams()) -> None:
        cache = self.session.cache
        pad = self.size - len(slots)
        packed = torch.tensor(list(slots) + [cache.null_slot] * pad + list(tokens) + [0] * pad
                              + list(request_ids) + [0] * pad + [first_step] * self.size + pack_sampling(sampling),
                              dtype=torch.int32)
        packed = packed.pin_memory().to(self.session.device, non_blocking=True)
        rows = packed[:4 * self.size].view(4, self.size)
        self.seq_slot.copy_(rows[0])
        self.tokens.copy_(rows[1])
        self.request_ids.copy_(rows[2])
        self.steps.copy_(rows[3])
        self.sample_params.copy_(packed[4 * self.size:])
        self.status.zero_()

    def retire(self, rows: Sequence[int]) -> None:
        """Point these rows at the null slot for every replay launched from now on (in stream order:
        steps already in flight still see the sequences)."""
        idx = torch.tensor(list(rows), dtype=torch.long).pin_memory().to(self.session.device, non_blocking=True)
        self.seq_slot.index_fill_(0, idx, self.session.cache.null_slot)


def pack_sampling(sampling: SamplingParams) -> List[int]:
    """temperature's float bits, top_k, and the two halves of the seed, as four int32 values."""
    def signed(v):
        return v - (1 << 32) if v >= 1 << 31 else v
    (t_bits,) = struct.unpack("<I", struct.pack("<f", float(sampling.temperature) or 1.0))
    seed = int(sampling.seed) & ((1 << 64) - 1)
    return [signed(t_bits), int(sampling.top_k), signed(seed & 0xffffffff), signed(seed >> 32)]


class GraphDecoder:
    """Runs the decode steps of one batch through captured graphs, ``depth`` steps in flight.

    One decoder serves every greedy run, another every sampled run: what differs between sampled
    runs is data in a device buffer.  ``history`` lists [batch size of the graph, steps replayed]
    of the last run, in order."""

    def __init__(self, session, sampling=SamplingParams(), depth: int = 3):
        self.session = session
        self.greedy = sampling.greedy if isinstance(sampling, SamplingParams) else bool(sampling)
        self.default_sampling = sampling if isinstance(sampling, SamplingParams) else SamplingParams()
        self.depth = depth
        self.buckets = {}
        self.history: List[List[int]] = []

    def new_bucket(self, n: int, uneven: bool = False) -> _Bucket:
        """Buffers for ``n`` sequences with every row on the null slot, nothing captured."""
        return _Bucket(self.session, bucket_size(n), self.greedy, uneven)

    def bucket(self, n: int, uneven: bool = False) -> _Bucket:
        """The captured graph for ``n`` sequences; one more per size for batches of very unequal lengths, captured
        when the first such batch comes."""
        size = bucket_size(n)
        b = self.buckets.get((size, uneven))
        if b is None:
            b = self.buckets[(size, uneven)] = self.new_bucket(size, uneven)
            b.capture()
        return b

    def run(self, slots: Sequence[int], tokens: Sequence[int], request_ids: Sequence[int], first_step: int,
            n_steps: int, stop=frozenset(), sampling: Optional[SamplingParams] = None) -> Iterator[List[Optional[int]]]:
        """Feed ``tokens`` and decode ``n_steps`` steps; yields each step's new tokens in the order of
        ``slots`` (None for a sequence that has met a stop token).  Ends early when all have.

        A sequence that has ended stops reading its cache with the next step that is launched; its
        slot stays held until the caller frees it."""
        sess = self.session
        sampling = self.default_sampling if sampling is None else sampling
        if sampling.greedy != self.greedy:
            raise ValueError("this decoder's graphs were captured for the other kind of token selection")
        n = len(slots)
        last = list(tokens)
        live = list(range(n))          # sequences still decoding, in the order of the bucket's rows
        self.history = []
        try:
            yield from self._run(slots, last, live, request_ids, first_step, n_steps, stop, sampling)
        finally:
            # However the loop ends (all steps handed out, every sequence stopped, the caller gone, an error): the
            # device finishes what is in flight before the caller frees the slots those steps still write to.
            torch.cuda.current_stream(sess.device).synchronize()
        sess.stepper.raise_on_status()

    def _run(self, slots, last, live, request_ids, first_step, n_steps, stop, sampling):
        sess = self.session
        cache = sess.cache
        n = len(slots)
        done_steps = 0
        while live and done_steps < n_steps:
            matters = getattr(sess.runtime.ops, "uneven_matters", None)
            uneven = (lengths_uneven([cache.lengths_host[slots[i]] + 1 for i in live])
                      and (matters is None or matters(bucket_size(len(live)))))
            b = self.bucket(len(live), uneven)
            cache.flush()
            b.load([slots[i] for i in live], [last[i] for i in live], [request_ids[i] for i in live],
                   first_step + done_steps, sampling)
            record = [b.size, 0]
            self.history.append(record)
            rows = list(live)                       # row r of this bucket is sequence rows[r]
            reading = set(rows)                     # sequences whose rows still point at their slots
            alive = set(rows)
            host = torch.empty((self.depth, b.size + 1), dtype=torch.int32, pin_memory=True)
            events = [torch.cuda.Event() for _ in range(self.depth)]
            launched = yielded = 0
            budget = n_steps - done_steps
            drain = False
            while yielded < budget:
                while not drain and launched < budget and launched - yielded < self.depth:
                    b.graph.replay()
                    host[launched % self.depth].copy_(b.out, non_blocking=True)
                    events[launched % self.depth].record()
                    for i in reading:
                        cache.advance_host(slots[i], 1)
                    launched += 1
                if yielded == launched:
                    break
                events[yielded % self.depth].synchronize()
                values = host[yielded % self.depth].tolist()
                yielded += 1
                if values[b.size]:
                    b.status.zero_()
                    raise_status_bits(values[b.size])
                out: List[Optional[int]] = [None] * n
                ended = []
                for r, i in enumerate(rows):
                    if i in alive:
                        out[i] = last[i] = values[r]
                        if values[r] in stop:
                            alive.discard(i)
                            ended.append(r)
                yield out
                if ended and alive and not drain:
                    if bucket_size(len(alive)) < b.size:
                        drain = True                # what is in flight is handed out, the rest runs on a smaller graph
                    else:
                        b.retire(ended)
                        reading -= {rows[r] for r in ended}
                if not alive:
                    break
            record[1] = launched
            done_steps += yielded
            live = [i for i in rows if i in alive]
