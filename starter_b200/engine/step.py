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

import array

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..cache.cache import Cache
from .context import StepContext, lengths_uneven

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


def _int32_tensor(values) -> torch.Tensor:
    """A sequence of token ids as a 1-D int32 tensor on the host.  A list of Python ints goes through the array
    module: four times faster than torch's own conversion (33 against 133 us for 2,048 ids)."""
    if isinstance(values, torch.Tensor):
        return values.to(dtype=torch.int32, device="cpu").reshape(-1)
    if isinstance(values, (list, tuple)) and values:
        try:
            return torch.frombuffer(array.array("i", values), dtype=torch.int32)
        except (TypeError, OverflowError):
            pass   # not plain ints (or beyond 32 bits): the general conversion says what is wrong
    return torch.as_tensor(values, dtype=torch.int32).reshape(-1)


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
        self.staging = cache.staging   # the batch's description goes up in one copy (cache/staging.py)
        model.prepare(cache)

    # ---- host side -----------------------------------------------------------------------

    def _describe(self, slots: Sequence[int], q_lens: Sequence[int], tail: Sequence[torch.Tensor] = ()):
        """(context of the batch on the device, the tail parts on the device): sequence b brings q_lens[b] rows for
        slot slots[b]; everything goes up in one copy."""
        cache = self.cache
        B = len(slots)
        cu = [0]
        for n in q_lens:
            cu.append(cu[-1] + int(n))
        M = cu[-1]
        head = torch.frombuffer(array.array("i", [*slots, *cu]), dtype=torch.int32)   # the short arrays in one piece
        if B == 1:
            row_seq = torch.zeros(M, dtype=torch.int32)
        else:
            row_seq = torch.repeat_interleave(torch.arange(B, dtype=torch.int32), torch.as_tensor(list(q_lens)), output_size=M)
        head, row_seq, *rest = self.staging.upload([head, row_seq, *tail])
        seq_slot, cu_q = head[:B], head[B:]
        kv_bound = max(cache.lengths_host[s] + n for s, n in zip(slots, q_lens))
        ctx = StepContext(
            runtime=self.runtime, cache=cache, n_seqs=B, n_rows=M, max_q_len=max(q_lens), kv_bound=kv_bound,
            seq_slot=seq_slot, cu_q=cu_q, row_seq=row_seq, lengths=cache.lengths, status=self.status,
            uneven=lengths_uneven([cache.lengths_host[s] + n for s, n in zip(slots, q_lens)]),
        )
        return ctx, rest

    def make_context(self, slots: Sequence[int], q_lens: Sequence[int]) -> StepContext:
        """Describe a batch on the device.  Sequence b brings q_lens[b] rows for slot slots[b]."""
        return self._describe(slots, q_lens)[0]

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
        tokens: List[torch.Tensor] = []
        want_rows: List[int] = []
        keys: List[tuple] = []
        row = 0
        for i, first, n in part:
            tokens.append(_int32_tensor(entries[i].tokens[first:first + n]))
            for w in sorted(set(entries[i].want)):
                if first <= w < first + n:
                    want_rows.append(row + w - first)
                    keys.append((i, w))
            row += n
        cache.flush()
        ctx, (token_ids, rows_wanted) = self._describe(slots, q_lens, [torch.cat(tokens) if len(tokens) > 1 else tokens[0],
                                                                          torch.as_tensor(want_rows, dtype=torch.int32)])
        stream = self.model.hidden(ctx, token_ids)
        logits = None
        if want_rows:
            rows = None if want_rows == list(range(row)) else rows_wanted
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
