"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some callers of the kernels cannot allocate device memory (they run inside another framework's
memory plan, or are handed their buffers and nothing else).  For them the library exports
``sb_attn_decode_noalloc``: the split-key decode attention with its scratch in a fixed array
inside the library instead of in buffers the caller allocates.  This test calls that symbol
with ctypes, twice in a row on different inputs, both with enough splits to go through the
array, and wants each result bit-equal to the ordinary entry point ``sb_attn_decode`` given
scratch from torch (the same kernel runs either way) and close to a plain torch restatement of
attention.  Between the two calls it fills the array with ones, so that the second call only
passes if the entry point clears the counters it shares with every earlier call.  It also
checks, on the host alone, that calls too large for the array or for the merge are refused
with a message.  The file's name makes pytest collect it last.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p
from types import SimpleNamespace

import pytest
import torch

from starter_b200.cache import Cache, KVRequest

pytestmark = pytest.mark.gpu

MAX_COUNTERS, MAX_FLOATS = 4096, 4 * 1024 * 1024   # attn_decode_noalloc.h


class _DeviceBytes:
    """A view of raw device memory for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _setup(heads, kv_heads, head_dim, lengths, seed):
    from starter_b200.csrc.ops import SbBatch, SbKV
    dtype = torch.bfloat16
    cache = Cache([KVRequest(kv_heads, head_dim)], n_slots=len(lengths), max_tokens=64 * 40, dtype=dtype, device="cuda",
                  max_seq_tokens=1024)
    g = torch.Generator().manual_seed(seed)
    group = cache.groups[0]
    group.k.copy_(torch.randn(group.k.shape, generator=g).to(dtype))
    group.v.copy_(torch.randn(group.v.shape, generator=g).to(dtype))
    slots = [cache.alloc() for _ in lengths]
    for s, n in zip(slots, lengths):
        cache.assume_length(s, n)
        cache.reserve(s, n + 1)
    cache.flush()
    n = len(lengths)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    keep = dict(seq_slot=i32(slots), cu_q=i32(list(range(n + 1))), row_seq=i32(list(range(n))), cache=cache)
    batch = SbBatch(keep["seq_slot"].data_ptr(), keep["cu_q"].data_ptr(), keep["row_seq"].data_ptr(),
                    cache.lengths.data_ptr(), n, n, cache.null_slot, 0)
    kv = SbKV(group.k[0].data_ptr(), group.v[0].data_ptr(), group.table.data_ptr(), group.table_width, 0, kv_heads, head_dim)
    q = torch.randn(n, heads * head_dim, generator=g).to(dtype).cuda()
    return keep, batch, kv, q


def _plain_attention(keep, q, heads, head_dim):
    """The torch restatement of attention over the same cache: the new token sits at position lengths[slot]."""
    from emulated_ops import EmulatedOps
    cache = keep["cache"]
    ctx = SimpleNamespace(cache=cache, seq_slot=keep["seq_slot"], cu_q=keep["cu_q"], row_seq=keep["row_seq"],
                          lengths=cache.lengths, n_rows=q.shape[0], n_seqs=q.shape[0])
    return EmulatedOps().attention(ctx, q, cache.layers[0], heads, 1.0 / math.sqrt(head_dim), None)


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from starter_b200.csrc.build import load
    from starter_b200.csrc.ops import SbBatch, SbKV
    lib = load(verbose=False)
    ordinary = lib.sb_attn_decode
    ordinary.argtypes = [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]
    ordinary.restype = c_int
    noalloc = lib.sb_attn_decode_noalloc
    noalloc.argtypes = [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p]
    noalloc.restype = c_int
    message = lib.sb_attn_decode_noalloc_error
    message.restype = ctypes.c_char_p
    scratch_address = lib.sb_attn_decode_noalloc_scratch
    scratch_address.restype = c_void_p
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    # two calls in a row, with different shapes, both with more than 8 splits: their partial results and their
    # counters go through the fixed array (up to 8 splits would merge in shared memory and never touch it)
    for call, (heads, kv_heads, head_dim, lengths, n_splits, seed) in enumerate([(8, 2, 128, [700, 5, 64, 300], 12, 1),
                                                                                (4, 4, 64, [1000, 0, 129], 10, 2)]):
        keep, batch, kv, q = _setup(heads, kv_heads, head_dim, lengths, seed)
        n = len(lengths)
        scale = 1.0 / math.sqrt(head_dim)
        partial = torch.empty(n * heads * n_splits * (head_dim + 2), dtype=torch.float32, device="cuda")
        counters = torch.zeros(n * kv_heads, dtype=torch.int32, device="cuda")
        want = torch.empty_like(q)
        assert ordinary(q.data_ptr(), want.data_ptr(), batch, kv, heads, scale, 0, n_splits, partial.data_ptr(),
                        counters.data_ptr(), stream) == 0
        got = torch.full_like(q, float("nan"))
        code = noalloc(q.data_ptr(), got.data_ptr(), batch, kv, heads, scale, 0, n_splits, stream)
        assert code == 0, message().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), f"call {call}: the same kernel with the same splits gave other bits"
        plain = _plain_attention(keep, q, heads, head_dim)
        assert float((got.float() - plain.float()).abs().max()) <= 1.6e-2 * float(plain.float().abs().max())
        if call == 0:
            # What an interrupted or foreign use could leave behind: every counter and every partial result
            # non-zero.  The next call must not depend on what the array holds.
            address = scratch_address()
            assert address, "the first call sets the array's address up"
            dirty = torch.as_tensor(_DeviceBytes(address, MAX_COUNTERS * 4 + MAX_FLOATS * 4), device="cuda")
            dirty.fill_(1)
            torch.cuda.synchronize()

    # Refusals are decided on the host, before anything is launched.
    keep, batch, kv, q = _setup(8, 2, 128, [10] * 40, 3)
    # more scratch than the fixed array holds
    big = SbBatch(batch.seq_slot, batch.cu_q, batch.row_seq, batch.lengths, 4000, 4000, batch.null_slot, 0)
    code = noalloc(q.data_ptr(), q.data_ptr(), big, kv, 8, 1.0, 0, 64, stream)
    assert code == -1 and b"scratch" in message()
    # more splits than the merge has shared memory for (one sequence keeps the scratch within the array)
    one = SbBatch(batch.seq_slot, batch.cu_q, batch.row_seq, batch.lengths, 1, 1, batch.null_slot, 0)
    most = lib.sb_attn_decode_max_splits(8, 2, 128)
    assert 8 < most < 4000
    code = noalloc(q.data_ptr(), q.data_ptr(), one, kv, 8, 1.0, 0, most + 1, stream)
    assert code == -1 and b"splits" in message()
    partial = torch.empty(1, dtype=torch.float32, device="cuda")
    counters = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert ordinary(q.data_ptr(), q.data_ptr(), one, kv, 8, 1.0, 0, most + 1, partial.data_ptr(), counters.data_ptr(),
                    stream) != 0
    no_heads = SbKV(kv.k, kv.v, kv.table, kv.table_width, 0, 0, 128)
    assert noalloc(q.data_ptr(), q.data_ptr(), one, no_heads, 8, 1.0, 0, 4, stream) != 0
    torch.cuda.synchronize()
