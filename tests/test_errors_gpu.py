"""What the kernels refuse and what they flag: sizes no kernel takes raise KernelError before a launch;
bad input sets a bit in the step's status word, which the step function raises as StepError; a wait inside
a TMA/tcgen05 kernel that runs out of time ends by itself and says so.  Nothing here faults or hangs."""

import pytest
import torch

from conftest import TINY
from starter_b200.cache import Cache, KVRequest
from starter_b200.engine.session import Session
from starter_b200.engine.step import STATUS_NO_PAGE, STATUS_TIMEOUT, StepEntry, StepError
from test_kernels_gpu import make_ctx, rand

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from starter_b200.csrc.ops import get_ops
    return get_ops(verbose=False)


def test_a_row_without_a_page_is_flagged_not_written(tiny_folders):
    """The page table of a live sequence loses its entries (as a fault in the host's books would cause): the
    kernel that stores keys and values skips the rows that have no page, raises the bit, and the step function
    turns it into StepError.  The session then serves another sequence."""
    sess = Session(tiny_folders["B"], dtype="float32", max_tokens=64 * 4, max_seqs=2, verbose=False)
    slot = sess.cache.alloc()
    sess.cache.reserve(slot, 70)
    sess.cache.flush()
    for group in sess.cache.groups:
        group.table[slot].fill_(-1)
    before = [g.k.clone() for g in sess.cache.groups]
    sess.stepper.step([StepEntry(slot, list(range(70)), [69])])
    with pytest.raises(StepError, match="no cache page"):
        sess.stepper.raise_on_status()
    assert all(torch.equal(g.k, b) for g, b in zip(sess.cache.groups, before))   # nothing was stored anywhere
    sess.cache.free(slot)
    other = sess.cache.alloc()
    assert sess.stepper.step([StepEntry(other, [1, 2, 3], [2])]).shape == (1, TINY["B"]["vocab_size"])
    sess.stepper.raise_on_status()
    sess.cache.free(other)
    assert STATUS_NO_PAGE == 2


def test_sizes_no_kernel_takes_are_refused(ops):
    from starter_b200.csrc.ops import KernelError
    dtype = torch.float32
    cache = Cache([KVRequest(1, 320)], n_slots=1, max_tokens=128, dtype=dtype, device="cuda", max_seq_tokens=128)
    slot = cache.alloc()
    cache.reserve(slot, 4)
    cache.flush()
    ctx = make_ctx(cache, ops, [slot], [4], dtype)
    with pytest.raises(KernelError, match="head sizes up to 256"):
        ops.attention(ctx, rand((4, 2 * 320), dtype, 1), cache.layers[0], 2, 0.1, None)
    with pytest.raises(KernelError, match="head sizes up to 512"):
        ops.qk_norm_rope_store(ctx, rand((4, 3 * 640), dtype, 2), cache.layers[0], 1, 1, 640, None, None, 0.0, None)
    # a rotary table that ends before the step's last position
    cache = Cache([KVRequest(2, 32)], n_slots=1, max_tokens=128, dtype=dtype, device="cuda", max_seq_tokens=128)
    slot = cache.alloc()
    cache.reserve(slot, 20)
    cache.flush()
    ctx = make_ctx(cache, ops, [slot], [20], dtype)
    cos = torch.ones(10, 16, device="cuda")
    with pytest.raises(KernelError, match="covers 10 positions, the step reaches 20"):
        ops.qk_norm_rope_store(ctx, rand((20, 8 * 32), dtype, 3), cache.layers[0], 4, 2, 32, None, None, 0.0, (cos, cos, 32))
    with pytest.raises(KernelError, match="float32 or bfloat16"):
        ops.linear(torch.ones(2, 8, dtype=torch.float16, device="cuda"), torch.ones(4, 8, dtype=torch.float16, device="cuda"))
    with pytest.raises(KernelError, match="two axes"):
        ops.prepare_matrix(torch.ones(4, device="cuda"))


def test_a_wait_that_runs_out_ends_by_itself(ops):
    """The bounded wait of the TMA/tcgen05 kernels, on the device: a barrier is armed for bytes that nobody
    sends, the wait gives up after its limit (here about a millisecond), raises the time-out bit and the block's
    abort flag, a second waiting thread sees the flag and leaves, and the kernel returns.  The next launches
    (the tcgen05 product among them) run as if nothing had happened."""
    import ctypes
    from ctypes import c_longlong, c_void_p
    probe = ops.lib.sb_wait_probe
    probe.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p]
    probe.restype = ctypes.c_int
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(3, dtype=torch.int64, device="cuda")
    limit = 2_000_000                                          # clock cycles: about a millisecond
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    assert probe(status.data_ptr(), out.data_ptr(), limit, stream) == 0
    torch.cuda.synchronize()
    gave_up, follower_left, cycles = out.tolist()
    assert gave_up == 1 and follower_left == 1
    assert limit <= cycles < 50 * limit
    assert int(status.item()) == STATUS_TIMEOUT
    assert probe(status.data_ptr(), out.data_ptr(), 1 << 40, stream) != 0    # a probe that would wait long is refused
    # the context is intact: the product that uses the same barriers still gives right numbers
    a, w = rand((24, 512), torch.bfloat16, 5), rand((256, 512), torch.bfloat16, 6)
    got = ops._stream_product(a, w, 256, False, True)
    want = a.float() @ w.float().T
    assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())
    assert ops.read_kernel_status() == 0
