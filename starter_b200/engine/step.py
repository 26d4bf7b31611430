"""The step function: a ragged batch of new tokens through the model, from the cache.

The reference has two step functions over fixed shapes: ``Plan.prefill`` for B
prompts of one length from position 0 and ``Plan.decode`` for one token each
(engine/model.py:280-303, 322-331), and rejects unequal prompts
(engine/engine.py:584-585).  Here one function takes, per sequence, whatever
new tokens it brings (a whole prompt, a piece of one, or one token), appends
them at the sequence's own length, and returns 32-bit logits at the rows
that were asked for.  Only the given tokens run; everything earlier is read
from the cache.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..cache.cache import Cache
from .context import StepContext

STATUS_BAD_TOKEN = 1
STATUS_NO_PAGE = 2
STATUS_TIMEOUT = 4
STATUS_MESSAGES = {
    STATUS_BAD_TOKEN: "a token id is outside the vocabulary",
    STATUS_NO_PAGE: "a row had no cache page reserved for its position",
    STATUS_TIMEOUT: "a wait inside a kernel ran out of time; the step's results are not valid",
}


class StepError(RuntimeError):
    """A kernel of the step flagged bad input instead of reading or writing out of range."""


def raise_status_bits(bits: int) -> None:
    """Raise StepError for a status word with bits set."""
    if bits:
        what = [msg for bit, msg in STATUS_MESSAGES.items() if bits & bit] or [f"status {bits}"]
        raise StepError("; ".join(what))


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, the places among them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Stepper:
    def __init__(self, model, cache: Cache, max_rows: int = 8192):
        self.model = model
        self.cache = cache
        self.runtime = model.runtime
        self.max_rows = int(max_rows)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.runtime.device)
        model.prepare(cache)

    # ---- host side -----------------------------------------------------------------------

    def _upload(self, values: List[int]) -> torch.Tensor:
        t = torch.tensor(values, dtype=torch.int32)
        if self.runtime.device.type == "cuda":
            return t.pin_memory().to(self.runtime.device, non_blocking=True)
        return t

    def make_context(self, slots: Sequence[int], q_lens: Sequence[int]) -> StepContext:
        """Describe a batch on the device.  Sequence b brings q_lens[b] rows for slot slots[b]."""
        cache = self.cache
        cu = [0]
        row_seq: List[int] = []
        for b, n in enumerate(q_lens):
            cu.append(cu[-1] + n)
            row_seq.extend([b] * n)
        B, M = len(slots), cu[-1]
        packed = self._upload(list(slots) + cu + row_seq)
        kv_bound = max(cache.lengths_host[s] + n for s, n in zip(slots, q_lens))
        return StepContext(
            runtime=self.runtime, cache=cache, n_seqs=B, n_rows=M, max_q_len=max(q_lens), kv_bound=kv_bound,
            seq_slot=packed[:B], cu_q=packed[B:2 * B + 1], row_seq=packed[2 * B + 1:], lengths=cache.lengths,
            status=self.status,
        )

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch; returns logits [wanted, vocab] in the order of
        the entries and of each entry's ``want`` (None when nothing is wanted)."""
        cache = self.cache
        seen = set()
        for e in entries:
            if not cache.slots.holds(e.slot) or e.slot in seen:
                raise ValueError(f"slot {e.slot} is not held, or appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise ValueError(f"slot {e.slot} brings no tokens")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"wanted place {w} is outside the {len(e.tokens)} tokens that slot {e.slot} brings")
            cache.reserve(e.slot, cache.lengths_host[e.slot] + len(e.tokens))
        done = [0] * len(entries)
        pieces: List[torch.Tensor] = []
        keys: List[tuple] = []  # (entry index, place) of every row of `pieces`, in their order
        while any(done[i] < len(e.tokens) for i, e in enumerate(entries)):
            room = self.max_rows
            part = []
            for i, e in enumerate(entries):
                n = min(len(e.tokens) - done[i], cache.step_limit, room)
                if n > 0:
                    part.append((i, done[i], n))
                    room -= n
            logits, part_keys = self._forward(entries, part)
            if logits is not None:
                pieces.append(logits)
                keys.extend(part_keys)
            for i, _, n in part:
                done[i] += n
        if not pieces:
            return None
        out = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
        wanted = [(i, w) for i, e in enumerate(entries) for w in e.want]
        if keys != wanted:
            where = {k: r for r, k in enumerate(keys)}
            index = torch.tensor([where[k] for k in wanted], dtype=torch.long, device=out.device)
            out = out.index_select(0, index)
        return out

    def _forward(self, entries, part):
        """One forward pass over ``part`` = [(entry index, first token, count)]."""
        cache = self.cache
        slots = [entries[i].slot for i, _, _ in part]
        q_lens = [n for _, _, n in part]
        tokens: List[int] = []
        want_rows: List[int] = []
        keys: List[tuple] = []
        row = 0
        for i, first, n in part:
            tokens.extend(int(t) for t in entries[i].tokens[first:first + n])
            for w in sorted(set(entries[i].want)):
                if first <= w < first + n:
                    want_rows.append(row + w - first)
                    keys.append((i, w))
            row += n
        cache.flush()
        ctx = self.make_context(slots, q_lens)
        packed = self._upload(tokens + want_rows)
        stream = self.model.hidden(ctx, packed[:len(tokens)])
        logits = None
        if want_rows:
            rows = None if want_rows == list(range(len(tokens))) else packed[len(tokens):]
            logits = self.model.logits(ctx, stream, rows)
        self.advance(ctx, slots, q_lens)
        # an entry may list a place twice: repeat its row
        if want_rows:
            dup = [(i, w) for i, first, n in part for w in entries[i].want if first <= w < first + n]
            if dup != keys:
                where = {k: r for r, k in enumerate(keys)}
                index = torch.tensor([where[k] for k in dup], dtype=torch.long, device=logits.device)
                logits, keys = logits.index_select(0, index), dup
        return logits, keys

    def advance(self, ctx: StepContext, slots, q_lens) -> None:
        """lengths[slot] += rows, on the device by a kernel and on the host's mirror."""
        ctx.ops.advance_lengths(ctx)
        for s, n in zip(slots, q_lens):
            self.cache.advance_host(s, n)

    def raise_on_status(self) -> None:
        """Read the kernels' status word (this waits for the device) and raise if any bit is set."""
        bits = int(self.status.item())
        if bits:
            self.status.zero_()
        read = getattr(self.runtime.ops, "read_kernel_status", None)
        if read is not None:
            bits |= read()
        raise_status_bits(bits)
