"""The cache: one slot per sequence, paged keys and values per layer group, fixed-size state.

The reference keeps ``k_cache, v_cache [layers, batch, kv_heads, cap, head_dim]``
with one batch row per sequence and a device ``pos[batch]``
(engine/model.py:229-235).  Here

* a **slot** is a sequence's record: its length (tokens held) and, per group,
  its row of a page table;
* storage is in **pages** of ``PAGE`` tokens, so that the memory is bounded by
  the tokens that live sequences hold, whatever their number and lengths;
* layers with the same needs form a **group** with storage of its own: a
  full-attention group keeps every key, a window group keeps a ring of pages
  that covers the window plus the longest step, a state group keeps a
  fixed-size record per slot and layer;
* one extra **null slot** with one null page takes the writes of padding rows.

Page layout of a key/value group: ``[layer_in_group, page, kv_head, PAGE, head_dim]``.
Position p of a sequence lives in logical page ``p // PAGE`` at offset
``p % PAGE``; logical page j is physical page ``table[slot, j]`` for a full
group and ``table[slot, j % ring_pages]`` for a window group.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .allocator import CacheError, IndexAllocator
from .staging import HostStaging

PAGE = 64


@dataclass(frozen=True)
class KVRequest:
    """A mixer's need for keys and values: every key (window None) or the last ``window``."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A mixer's need for a fixed-size record per sequence, zero when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class SharedRequest:
    """A mixer that reads the cache of another layer and stores nothing itself.  In a mixer's answer
    ``layer`` is a layer index; in the list a Cache is built from, it is an index into that list."""

    layer: int


class KVGroup:
    def __init__(self, request: KVRequest, layers: Sequence[int], n_slots: int, pool_pages: int,
                 table_width: int, max_step_tokens: int, dtype: torch.dtype, device):
        self.request = request
        self.layers = list(layers)
        self.n_slots = n_slots
        if request.window is None:
            self.ring_pages = 0
            self.table_width = table_width
        else:
            # A step writes positions [s, s+T) and reads keys from s - window + 1 on: those span at
            # most (T + window - 2) // PAGE + 2 logical pages, which must be distinct ring entries.
            self.ring_pages = min((max_step_tokens + request.window - 2) // PAGE + 2, table_width)
            self.table_width = self.ring_pages
            pool_pages = min(pool_pages, n_slots * self.ring_pages)
        self.pool_pages = pool_pages
        self.null_page = pool_pages
        shape = (len(self.layers), pool_pages + 1, request.num_kv_heads, PAGE, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages = IndexAllocator(pool_pages, "cache page")
        self.table_host = torch.full((n_slots + 1, self.table_width), -1, dtype=torch.int32)
        self.table_host[n_slots, :] = self.null_page
        self.table = self.table_host.to(device)
        self._held: Dict[int, List[int]] = {}
        self._dirty = set()

    def pages_for(self, n_tokens: int) -> int:
        need = (n_tokens + PAGE - 1) // PAGE
        return min(need, self.ring_pages) if self.ring_pages else need

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Make sure the slot has the pages that ``n_tokens`` tokens need."""
        held = self._held.setdefault(slot, [])
        need = self.pages_for(n_tokens)
        if need > self.table_width:
            raise CacheError(f"a sequence of {n_tokens} tokens needs {need} pages; the page table holds "
                             f"{self.table_width} per sequence")
        if need - len(held) > self.pages.n_free:
            raise CacheError(f"the cache is full: {need - len(held)} more pages of {PAGE} tokens are needed, "
                             f"{self.pages.n_free} of {self.pool_pages} are free")
        if len(held) < need:
            first = len(held)
            while len(held) < need:
                held.append(self.pages.take())
            self.table_host[slot, first:need] = torch.tensor(held[first:], dtype=torch.int32)   # one write, not one per page
            self._dirty.add(slot)

    def release(self, slot: int) -> None:
        for page in self._held.pop(slot, []):
            self.pages.give_back(page)
        self.table_host[slot, :] = -1
        self._dirty.add(slot)

    def flush(self, staging) -> None:
        """Bring the device page table up to date with the host's: the changed rows go up in one copy."""
        if self._dirty:
            rows = torch.tensor(sorted(self._dirty), dtype=torch.int32)
            idx, data = staging.upload([rows, self.table_host[rows.long()]])
            self.table[idx] = data
            self._dirty.clear()

    def capacity_tokens(self) -> int:
        return self.pool_pages * PAGE

    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class StateGroup:
    def __init__(self, request: StateRequest, layers: Sequence[int], n_slots: int, run_dtype: torch.dtype, device):
        self.request = request
        self.layers = list(layers)
        dtype = run_dtype if request.dtype == "run" else getattr(torch, request.dtype)
        self.data = torch.zeros((len(self.layers), n_slots + 1) + tuple(request.shape), dtype=dtype, device=device)

    def reset(self, slot: int) -> None:
        self.data[:, slot].zero_()

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()


@dataclass
class LayerCache:
    """What one layer sees of the cache: its group and its index in the group's storage."""

    group: object
    index: int

    @property
    def is_kv(self) -> bool:
        return isinstance(self.group, KVGroup)

    @property
    def k(self) -> torch.Tensor:
        return self.group.k[self.index]

    @property
    def v(self) -> torch.Tensor:
        return self.group.v[self.index]

    @property
    def state(self) -> torch.Tensor:
        return self.group.data[self.index]


class Cache:
    """Slots, lengths, and the groups' storage for one model.

    ``requests[i]`` is what the i-th entry of the model's execution order asked for (a
    KVRequest, StateRequest, SharedRequest naming an earlier entry, or None).  ``max_tokens`` bounds the tokens all live sequences
    hold together, each sequence's count rounded up to ``PAGE``; ``max_seq_tokens``
    bounds one sequence; ``max_step_tokens`` bounds the tokens one sequence
    brings in one forward pass (it sizes the ring of a window group).
    """

    def __init__(self, requests: Sequence[object], n_slots: int, max_tokens: int, dtype: torch.dtype, device,
                 max_seq_tokens: Optional[int] = None, max_step_tokens: int = 1024):
        if n_slots <= 0 or max_tokens <= 0:
            raise CacheError("a cache needs at least one slot and one token of room")
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_slots = int(n_slots)
        self.null_slot = self.n_slots
        self.max_step_tokens = int(max_step_tokens)
        pool_pages = (int(max_tokens) + PAGE - 1) // PAGE
        self.max_seq_tokens = int(max_seq_tokens) if max_seq_tokens else pool_pages * PAGE
        table_width = min(pool_pages, (self.max_seq_tokens + PAGE - 1) // PAGE)
        self.max_seq_tokens = min(self.max_seq_tokens, table_width * PAGE)
        self.slots = IndexAllocator(self.n_slots, "sequence slot")
        self.groups: List[object] = []
        self.layers: List[Optional[LayerCache]] = [None] * len(requests)
        by_request: Dict[object, List[int]] = {}
        for i, req in enumerate(requests):
            if isinstance(req, (KVRequest, StateRequest)):
                by_request.setdefault(req, []).append(i)
        for req, layer_ids in by_request.items():
            if isinstance(req, KVRequest):
                group = KVGroup(req, layer_ids, self.n_slots, pool_pages, table_width, self.max_step_tokens, dtype, device)
            else:
                group = StateGroup(req, layer_ids, self.n_slots, dtype, device)
            self.groups.append(group)
            for j, i in enumerate(layer_ids):
                self.layers[i] = LayerCache(group, j)
        for i, req in enumerate(requests):
            if isinstance(req, SharedRequest):
                if not 0 <= req.layer < len(requests) or self.layers[req.layer] is None:
                    raise CacheError(f"layer {i} wants to read the cache of layer {req.layer}, which has none")
                self.layers[i] = self.layers[req.layer]
        # Only a ring of pages limits how many tokens a sequence may bring in one forward pass.
        self.has_rings = any(isinstance(g, KVGroup) and g.ring_pages for g in self.groups)
        self.step_limit = self.max_step_tokens if self.has_rings else (1 << 30)
        self.lengths_host: List[int] = [0] * (self.n_slots + 1)
        self.lengths = torch.zeros(self.n_slots + 1, dtype=torch.int32, device=device)
        self._dirty_lengths = set()
        self.staging = HostStaging(device)   # changed page-table rows and lengths go up through it

    # ---- slots -------------------------------------------------------------------------

    def alloc(self) -> int:
        """Take a slot for a new sequence: length 0, fixed-size state zero, no pages yet."""
        slot = self.slots.take()
        self.lengths_host[slot] = 0
        self._dirty_lengths.add(slot)
        for g in self.groups:
            if isinstance(g, StateGroup):
                g.reset(slot)
        return slot

    def free(self, slot: int) -> None:
        """Give a slot and its pages back.  Freeing a slot that is not held is an error."""
        self.slots.give_back(slot)
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.release(slot)
        self.lengths_host[slot] = 0
        self._dirty_lengths.add(slot)

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Make room for the sequence in ``slot`` to hold ``n_tokens`` tokens."""
        if not self.slots.holds(slot):
            raise CacheError(f"slot {slot} is not held")
        if n_tokens > self.max_seq_tokens:
            raise CacheError(f"a sequence of {n_tokens} tokens exceeds the cache's limit of {self.max_seq_tokens} per sequence")
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.reserve(slot, n_tokens)

    def assume_length(self, slot: int, n_tokens: int) -> None:
        """Declare that the slot already holds ``n_tokens`` tokens (pages reserved, contents as they
        are).  For benchmarks that start from a synthetic context instead of a real prompt."""
        self.reserve(slot, n_tokens)
        self.lengths_host[slot] = int(n_tokens)
        self._dirty_lengths.add(slot)

    def advance_host(self, slot: int, n: int) -> None:
        """Mirror on the host what the step's kernel did to the device lengths."""
        self.lengths_host[slot] += n

    def flush(self) -> None:
        """Bring device page tables and the lengths of newly taken or freed slots up to date."""
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.flush(self.staging)
        if self._dirty_lengths:
            rows = sorted(self._dirty_lengths)
            idx, vals = self.staging.upload([torch.tensor(rows, dtype=torch.int32),
                                             torch.tensor([self.lengths_host[r] for r in rows], dtype=torch.int32)])
            self.lengths[idx] = vals
            self._dirty_lengths.clear()

    # ---- accounting --------------------------------------------------------------------

    def tokens_free(self) -> int:
        """Tokens of room left in the tightest full-attention group (a window group needs less)."""
        frees = [g.pages.n_free * PAGE for g in self.groups if isinstance(g, KVGroup) and not g.ring_pages]
        if not frees:
            frees = [g.pages.n_free * PAGE for g in self.groups if isinstance(g, KVGroup)]
        return min(frees) if frees else 1 << 60

    def nbytes(self) -> int:
        return sum(g.nbytes() for g in self.groups)

    def check(self) -> None:
        """No slot or page is lost or held twice."""
        self.slots.check()
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.pages.check()
                held = [p for pages in g._held.values() for p in pages]
                if len(set(held)) != len(held) or len(held) != g.pages.n_held:
                    raise CacheError("a cache page is held by two slots or by none")
                for slot in g._held:
                    if g._held[slot] and not self.slots.holds(slot):
                        raise CacheError(f"slot {slot} is free but still holds pages")
