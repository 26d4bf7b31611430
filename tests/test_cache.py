"""The cache on the host: no slot or page lost, held twice or freed twice; rings; accounting."""

import random

import pytest
import torch

from starter_b200.cache import PAGE, Cache, CacheError, IndexAllocator, KVRequest, SharedRequest, StateRequest


def test_allocator_never_loses_or_doubles():
    alloc = IndexAllocator(5, "thing")
    held = [alloc.take() for _ in range(5)]
    assert sorted(held) == list(range(5)) and held == list(range(5))   # lowest first
    with pytest.raises(CacheError, match="no free thing"):
        alloc.take()
    alloc.give_back(3)
    with pytest.raises(CacheError, match="not held"):
        alloc.give_back(3)
    assert alloc.take() == 3
    rng = random.Random(0)
    held = set(range(5))
    for _ in range(500):
        if held and rng.random() < 0.5:
            i = rng.choice(sorted(held))
            alloc.give_back(i)
            held.remove(i)
        elif alloc.n_free:
            i = alloc.take()
            assert i not in held
            held.add(i)
        alloc.check()
        assert alloc.n_free + alloc.n_held == 5


def make(requests, **kw):
    return Cache(requests, dtype=torch.float32, device="cpu", **kw)


def test_groups_by_need_and_shared_layers():
    full, win = KVRequest(2, 16), KVRequest(2, 16, window=40)
    cache = make([full, win, full, win, SharedRequest(0), StateRequest((3, 4)), None], n_slots=3, max_tokens=64 * 6,
                 max_step_tokens=48)
    assert len(cache.groups) == 3
    assert cache.layers[0].group is cache.layers[2].group and cache.layers[0].index == 0 and cache.layers[2].index == 1
    assert cache.layers[1].group is cache.layers[3].group and cache.layers[1].group is not cache.layers[0].group
    assert cache.layers[4] is cache.layers[0] and cache.layers[6] is None
    assert cache.layers[1].group.ring_pages == (48 + 40 - 2) // PAGE + 2
    assert cache.layers[5].state.shape == (4, 3, 4)   # slots + the null slot
    with pytest.raises(CacheError):
        make([SharedRequest(1), None], n_slots=1, max_tokens=64)


def test_slots_and_pages_are_given_back_and_used_again():
    cache = make([KVRequest(1, 8)], n_slots=2, max_tokens=64 * 4)
    a, b = cache.alloc(), cache.alloc()
    with pytest.raises(CacheError, match="no free sequence slot"):
        cache.alloc()
    cache.reserve(a, 65)
    cache.reserve(b, 64)
    assert cache.groups[0].pages.n_held == 3 and cache.tokens_free() == 64
    with pytest.raises(CacheError, match="cache is full"):
        cache.reserve(b, 64 * 3)
    cache.check()
    cache.free(a)
    with pytest.raises(CacheError, match="not held"):
        cache.free(a)
    with pytest.raises(CacheError, match="not held"):
        cache.reserve(a, 1)
    c = cache.alloc()
    assert c == a and cache.lengths_host[c] == 0
    cache.reserve(c, 64 * 3)
    cache.flush()
    table = cache.groups[0].table
    assert sorted(table[c, :3].tolist() + table[b, :1].tolist()) == [0, 1, 2, 3]
    assert table[cache.null_slot, 0] == cache.groups[0].null_page
    cache.check()
    cache.free(b)
    cache.free(c)
    assert cache.groups[0].pages.n_free == 4 and cache.slots.n_free == 2
    assert bool((cache.groups[0].table_host[:2] == -1).all())


def test_window_group_keeps_a_ring():
    cache = make([KVRequest(1, 8, window=10)], n_slots=2, max_tokens=64 * 100, max_step_tokens=64)
    g = cache.groups[0]
    assert g.ring_pages == (64 + 10 - 2) // PAGE + 2 == 3
    s = cache.alloc()
    cache.reserve(s, 5000)          # far more tokens than the ring holds
    assert g.pages.n_held == 3
    assert g.pool_pages == 2 * 3    # never more pages than the slots' rings


def test_state_is_zero_for_a_new_sequence():
    cache = make([StateRequest((4,))], n_slots=2, max_tokens=64)
    s = cache.alloc()
    cache.layers[0].state[s] += 5.0
    cache.free(s)
    assert cache.alloc() == s and float(cache.layers[0].state[s].abs().sum()) == 0.0


def test_limits():
    cache = make([KVRequest(1, 8)], n_slots=4, max_tokens=64 * 8, max_seq_tokens=100)
    assert cache.max_seq_tokens == 100
    s = cache.alloc()
    cache.reserve(s, 100)
    with pytest.raises(CacheError, match="exceeds"):
        cache.reserve(s, 101)


def test_random_traffic_keeps_the_books():
    cache = make([KVRequest(1, 8), KVRequest(1, 8, window=20)], n_slots=5, max_tokens=64 * 12, max_step_tokens=32)
    rng = random.Random(1)
    live = {}
    for _ in range(400):
        r = rng.random()
        if r < 0.3 and cache.slots.n_free:
            live[cache.alloc()] = 0
        elif r < 0.6 and live:
            s = rng.choice(sorted(live))
            cache.free(s)
            del live[s]
        elif live:
            s = rng.choice(sorted(live))
            want = live[s] + rng.randint(1, 150)
            try:
                cache.reserve(s, want)
                live[s] = want
            except CacheError:
                pass
        cache.check()
        full = cache.groups[0]
        assert full.pages.n_held == sum((n + PAGE - 1) // PAGE for n in live.values())
    for s in list(live):
        cache.free(s)
    cache.check()
    assert all(g.pages.n_held == 0 for g in cache.groups)


def test_staging_keeps_what_it_was_given_and_the_step_reads_token_lists():
    """The host-to-device staging lays the parts side by side and hands back views in their shapes and order; what
    goes up is what the tensors held at the call, whatever the host writes to them afterwards.  (On the CPU the
    "device" is the host: the parts are copied.)  Token ids given as lists, tuples, tensors or other integers all
    become the same int32 tensor."""
    from starter_b200.cache.staging import HostStaging
    from starter_b200.engine.step import _int32_tensor

    staging = HostStaging("cpu")
    a = torch.tensor([3, 1, 2], dtype=torch.int32)
    b = torch.arange(6, dtype=torch.int32).view(2, 3)
    empty = torch.empty(0, dtype=torch.int32)
    got_a, got_empty, got_b = staging.upload([a, empty, b])
    a[0] = 99
    b[1, 2] = 99
    assert got_a.tolist() == [3, 1, 2] and got_b.tolist() == [[0, 1, 2], [3, 4, 5]] and got_empty.numel() == 0
    assert staging.upload([]) == []

    import numpy as np
    want = [5, 0, 151935]
    for given in (want, tuple(want), torch.tensor(want), torch.tensor(want, dtype=torch.int64), np.array(want),
                  [np.int64(v) for v in want], []):
        out = _int32_tensor(given)
        assert out.dtype == torch.int32 and out.dim() == 1 and out.tolist() == (want if len(given) else [])
    with pytest.raises(Exception):
        _int32_tensor([1, "two"])
