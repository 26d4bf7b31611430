"""Each CUDA kernel alone against its plain torch restatement, at sizes other than the models'."""

import math

import pytest
import torch

from emulated_ops import EmulatedOps
from starter_b200.cache import Cache, KVRequest
from starter_b200.engine.context import Runtime, StepContext

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from starter_b200.csrc.ops import get_ops
    return get_ops(verbose=False)


@pytest.fixture(scope="module")
def ref():
    return EmulatedOps()


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


def close(got, want, dtype, what, rel=None):
    rel = rel if rel is not None else (2e-5 if dtype == torch.float32 else 1.6e-2)
    scale = float(want.float().abs().max()) + 1e-30
    err = float((got.float() - want.float()).abs().max())
    assert err <= rel * scale, f"{what}: {err:.3g} > {rel * scale:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_and_gather(ops, ref, dtype):
    table = rand((301, 72), dtype, 0)
    tokens = torch.tensor([5, 300, 0, 17, 5], dtype=torch.int32).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    assert torch.equal(ops.embed(tokens, table, status), ref.embed(tokens, table, status.clone()))
    assert int(status) == 0
    bad = torch.tensor([5, 301, -1], dtype=torch.int32).cuda()
    ops.embed(bad, table, status)
    assert int(status) == 1
    rows = torch.tensor([4, 0, 4, 2], dtype=torch.int32).cuda()
    x = rand((5, 72), dtype, 1)
    assert torch.equal(ops.gather_rows(x, rows), x[rows.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [16, 200, 2560, 5000])
def test_rmsnorm(ops, ref, dtype, width):
    x = rand((7, width), dtype, 2, 3.0)
    w = (1 + 0.1 * rand((width,), torch.float32, 3)).to(dtype)
    close(ops.rmsnorm(x, w, 1e-5), ref.rmsnorm(x, w, 1e-5), dtype, "rmsnorm")
    d = rand((7, width), dtype, 4)
    x1, x2 = x.clone(), x.clone()
    y1, y2 = ops.add_rmsnorm(x1, d, w, 1e-6), ref.add_rmsnorm(x2, d, w, 1e-6)
    assert torch.equal(x1, x2), "residual sum"
    close(y1, y2, dtype, "add_rmsnorm")
    if dtype == torch.bfloat16:  # a norm weight stored in 32-bit stays 32-bit
        close(ops.rmsnorm(x, w.float(), 1e-5), ref.rmsnorm(x, w.float(), 1e-5), dtype, "rmsnorm, 32-bit weight")


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, ref, dtype):
    gu = rand((5, 2 * 331), dtype, 5, 2.0)
    close(ops.swiglu(gu), ref.swiglu(gu), dtype, "swiglu", rel=1e-6 if dtype == torch.float32 else 8e-3)
    if dtype == torch.bfloat16:   # both roundings where the formula has them (engine/kernels/swiglu.py:21-24); exp may differ in its last bit
        big = rand((300, 2 * 1000), dtype, 6, 2.0)
        same = float((ops.swiglu(big) == ref.swiglu(big)).float().mean())
        assert same >= 0.999, f"only {same:.5f} of the values have the restatement's bits"
        fused = ops.linear_swiglu(rand((8, 512), dtype, 7), rand((2 * 640, 512), dtype, 8, 0.05))
        assert fused.shape == (8, 640)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 389, 96), (5, 70, 33), (130, 257, 160), (64, 1000, 4096), (300, 512, 1024),
                                   (8, 6144, 2560), (16, 2560, 9728), (3, 1000, 4096), (11, 100, 1160)])
def test_linear(ops, ref, dtype, shape):
    M, N, K = shape
    a, w = rand((M, K), dtype, 6), rand((N, K), dtype, 7, 0.05)
    close(ops.linear(a, w), ref.linear(a, w), dtype, "linear")
    close(ops.linear(a, w, out_float32=True), ref.linear(a, w, out_float32=True), dtype, "linear, 32-bit out",
          rel=2e-5 if dtype == torch.float32 else 2e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 2 * 224, 96), (7, 2 * 9728, 2560), (16, 2 * 100, 1160), (40, 2 * 330, 72)])
def test_linear_swiglu(ops, ref, dtype, shape):
    M, N2, K = shape
    h, w = rand((M, K), dtype, 8), rand((N2, K), dtype, 9, 0.05)
    close(ops.linear_swiglu(h, w), ref.linear_swiglu(h, w), dtype, "linear + swiglu")


def make_ctx(cache, ops, slots, q_lens, dtype):
    rt = Runtime(dtype=dtype, device=torch.device("cuda"), ops=ops)
    cu = [0]
    row_seq = []
    for b, n in enumerate(q_lens):
        cu.append(cu[-1] + n)
        row_seq += [b] * n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return StepContext(runtime=rt, cache=cache, n_seqs=len(slots), n_rows=cu[-1], max_q_len=max(q_lens),
                       kv_bound=max(cache.lengths_host[s] + n for s, n in zip(slots, q_lens)), seq_slot=i32(slots),
                       cu_q=i32(cu), row_seq=i32(row_seq), lengths=cache.lengths,
                       status=torch.zeros(1, dtype=torch.int32).cuda())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(6, 3, 48, None), (4, 1, 16, 9), (8, 8, 128, None), (2, 2, 80, 70),
                                                            (8, 2, 128, None), (6, 1, 64, None), (4, 2, 64, 40),
                                                            (20, 1, 128, 90)])
def test_store_and_attention(ops, ref, dtype, heads, kv_heads, head_dim, window):
    """Two steps over three sequences of unequal length: rope + store + attention against the
    torch restatement working on a second, identical cache."""
    req = KVRequest(kv_heads, head_dim, window)
    caches = [Cache([req], n_slots=4, max_tokens=64 * 12, dtype=dtype, device="cuda", max_step_tokens=100) for _ in range(2)]
    half = head_dim // 2
    ang = torch.arange(400, dtype=torch.float32)[:, None] / (10000.0 ** (torch.arange(half).float() / half))[None]
    rotary = (ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda(), head_dim)
    qn = (1 + 0.1 * rand((head_dim,), torch.float32, 8)).to(dtype)
    kn = (1 + 0.1 * rand((head_dim,), torch.float32, 9)).to(dtype)
    slots = [[c.alloc() for _ in range(3)] for c in caches]
    assert slots[0] == slots[1]
    for step, q_lens in enumerate([(70, 3, 100), (1, 1, 5)]):
        outs = []
        for c, o in zip(caches, (ops, ref)):
            for s, n in zip(slots[0], q_lens):
                c.reserve(s, c.lengths_host[s] + n)
            c.flush()
            ctx = make_ctx(c, ops, slots[0], q_lens, dtype)
            qkv = rand((sum(q_lens), (heads + 2 * kv_heads) * head_dim), dtype, 20 + step)
            q = o.qk_norm_rope_store(ctx, qkv, c.layers[0], heads, kv_heads, head_dim, qn, kn, 1e-6, rotary)
            a = o.attention(ctx, q, c.layers[0], heads, 1.0 / math.sqrt(head_dim), window)
            o.advance_lengths(ctx)
            for s, n in zip(slots[0], q_lens):
                c.advance_host(s, n)
            assert int(ctx.status) == 0
            outs.append((q, a))
        close(outs[0][0], outs[1][0], dtype, f"q after norm and rope, step {step}", rel=1e-5 if dtype == torch.float32 else 8e-3)
        if dtype == torch.bfloat16:   # the kernel rounds where the formula rounds: (nearly) every value has its bits
            same = float((outs[0][0] == outs[1][0]).float().mean())
            assert same >= 0.998, f"only {same:.5f} of q's values have the restatement's bits"
        close(outs[0][1], outs[1][1], dtype, f"attention, step {step}")
        close(caches[0].groups[0].k, caches[1].groups[0].k, dtype, "stored keys", rel=1e-5 if dtype == torch.float32 else 8e-3)
        assert torch.equal(caches[0].groups[0].v, caches[1].groups[0].v), "stored values"
        assert torch.equal(caches[0].lengths, caches[1].lengths)


def test_attention_finds_a_far_key(ops):
    """One key among hundreds is made to stand out: the output must be its value."""
    dtype, heads, head_dim = torch.float32, 2, 32
    cache = Cache([KVRequest(1, head_dim, None)], n_slots=2, max_tokens=64 * 8, dtype=dtype, device="cuda")
    slot = cache.alloc()
    n = 300
    cache.reserve(slot, n)
    cache.flush()
    ctx = make_ctx(cache, ops, [slot], [n], dtype)
    qkv = rand((n, (heads + 2) * head_dim), dtype, 30, 0.1)
    qkv[:, heads * head_dim:(heads + 1) * head_dim] = 0.01 * rand((n, head_dim), dtype, 31)
    qkv[37, heads * head_dim:(heads + 1) * head_dim] = 10.0  # key 37 is large ...
    qkv[-1, :heads * head_dim] = 10.0                        # ... and the last query points at it
    q = ops.qk_norm_rope_store(ctx, qkv, cache.layers[0], heads, 1, head_dim, None, None, 0.0, None)
    a = ops.attention(ctx, q, cache.layers[0], heads, 1.0, None)
    want = qkv[37, (heads + 1) * head_dim:]
    assert torch.allclose(a[-1, :head_dim], want, atol=1e-5) and torch.allclose(a[-1, head_dim:], want, atol=1e-5)


def test_argmax_ties_and_sampling(ops):
    logits = rand((5, 1000), torch.float32, 40)
    logits[1, 700] = logits[1, 20] = 50.0   # equal maxima: the lower index wins
    logits[2, 999] = 60.0
    got = ops.argmax(logits).cpu()
    want = logits.cpu().argmax(-1)
    want[1] = 20
    assert got.tolist() == want.tolist()
    assert ops.argmax(rand((3, 151936), torch.float32, 41)).tolist() == rand((3, 151936), torch.float32, 41).argmax(-1).tolist()


@pytest.mark.parametrize("top_k", [0, 1, 7, 50])
def test_sampling_matches_plain(ops, top_k):
    from plain import qwen3_plain as plain
    vocab, rows = 389, 16
    logits = rand((rows, vocab), torch.float32, 50, 2.0)
    logits[3, 100] = logits[3, 200] = logits[3, 300] = float(logits[3].max()) + 0.5  # ties at the edge of the kept set
    req = torch.arange(rows, dtype=torch.int32).cuda() + 5
    steps = torch.full((rows,), 3, dtype=torch.int32).cuda()
    got = ops.sample(logits, 0.8, top_k, 1234, req, steps, advance=True).tolist()
    assert steps.tolist() == [4] * rows
    for r in range(rows):
        u = plain.uniform_from_counter(1234, 5 + r, 3)
        tok, margin = plain.sample(logits[r].cpu(), 0.8, top_k, u)
        if margin > 1e-5:  # a draw this far from an edge cannot be flipped by 32-bit rounding
            assert got[r] == tok, f"row {r}: {got[r]} != {tok} (margin {margin:.2g})"


def poison_beyond(cache, slots, lengths_after):
    """NaN in every cache position of a sequence's last page that lies beyond the tokens it will hold after the
    step: what a page's former owner may have left there must not reach any result."""
    g = cache.groups[0]
    for s, n in zip(slots, lengths_after):
        if n % 64 == 0:
            continue
        lp = (n - 1) // 64
        if g.ring_pages:
            lp %= g.ring_pages
        page = int(g.table_host[s, lp])
        g.k[:, page, :, n % 64:] = float("nan")
        g.v[:, page, :, n % 64:] = float("nan")


@pytest.mark.parametrize("splits", [None, 1, 3, 5, 6, 7, 12])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(8, 2, 128, None), (16, 1, 64, None), (6, 3, 64, 100), (4, 4, 128, 700)])
def test_decode_attention(ops, ref, monkeypatch, heads, kv_heads, head_dim, window, splits):
    """One new token per sequence over contexts of 0 to 1500 tokens, against the torch restatement;
    in the longest sequence one far key is made to stand out."""
    dtype = torch.bfloat16
    if splits is None:   # the balanced kernel, whatever the number of pairs
        monkeypatch.setattr(ops, "force_decode_route", "balanced")
    else:                # the split-key kernel with a fixed number of splits
        monkeypatch.setattr(ops, "decode_balanced", False)
        monkeypatch.setattr(ops, "decode_splits", lambda *a: splits)
    cache = Cache([KVRequest(kv_heads, head_dim, window)], n_slots=6, max_tokens=64 * 60, dtype=dtype, device="cuda",
                  max_seq_tokens=1600, max_step_tokens=64)
    g = cache.groups[0]
    g.k.copy_(rand(tuple(g.k.shape), dtype, 60))
    g.v.copy_(rand(tuple(g.v.shape), dtype, 61))
    lengths = [0, 63, 64, 700, 1500]
    slots = [cache.alloc() for _ in lengths]
    for s, n in zip(slots, lengths):
        cache.assume_length(s, n)
        cache.reserve(s, n + 1)
    cache.flush()
    poison_beyond(cache, slots, [n + 1 for n in lengths])
    ctx = make_ctx(cache, ops, slots, [1] * len(lengths), dtype)
    qkv = rand((len(lengths), (heads + 2 * kv_heads) * head_dim), dtype, 62)
    if window is None:  # key 37 of the last sequence is large and the new query of head 0 points at it
        lp, off = 37 // 64, 37 % 64
        page = int(g.table_host[slots[-1], lp])
        g.k[0, page, 0, off] = 4.0
        qkv[-1, :head_dim] = 4.0
    outs = []
    for o in (ops, ref):
        k0, v0 = g.k.clone(), g.v.clone()
        q = o.qk_norm_rope_store(ctx, qkv, cache.layers[0], heads, kv_heads, head_dim, None, None, 0.0, None)
        outs.append(o.attention(ctx, q, cache.layers[0], heads, 1.0 / math.sqrt(head_dim), window))
        g.k.copy_(k0)
        g.v.copy_(v0)
    close(outs[0], outs[1], dtype, "decode attention")
    if window is None:
        want = g.v[0, int(g.table_host[slots[-1], 0]), 0, 37].float()
        assert float((outs[0][-1, :head_dim].float() - want).abs().max()) < 0.05 * float(want.abs().max())


@pytest.mark.parametrize("splits", [None, 1, 3, 8, 11])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window,norm,rotary,store", [
    (8, 2, 128, None, torch.bfloat16, True, True), (16, 1, 64, None, torch.float32, True, True),
    (6, 3, 64, 100, None, True, True), (4, 4, 128, 700, torch.bfloat16, False, True),
    (12, 2, 128, None, torch.bfloat16, True, False)])
def test_decode_attention_with_preparation_inside(ops, ref, monkeypatch, heads, kv_heads, head_dim, window, norm, rotary,
                                                  store, splits):
    """The decode kernel that norms, rotates and stores q and k itself, against the two separate calls of the
    torch restatement: the attention's output and what it left in the cache.  Lengths put the new token at
    the start of a page, at its end, and in a sequence's first position."""
    dtype = torch.bfloat16
    if splits is None:   # the balanced kernel (equal shares of all pages per block), with the preparation inside as well
        monkeypatch.setattr(ops, "force_decode_route", "balanced")
        monkeypatch.setattr(ops, "fuse_qk_balanced", True)   # off by default: slower in the step than a kernel of its own
    else:
        monkeypatch.setattr(ops, "decode_balanced", False)
        monkeypatch.setattr(ops, "decode_splits", lambda *a: splits)
    cache = Cache([KVRequest(kv_heads, head_dim, window)], n_slots=6, max_tokens=64 * 60, dtype=dtype, device="cuda",
                  max_seq_tokens=1600, max_step_tokens=64)
    g = cache.groups[0]
    g.k.copy_(rand(tuple(g.k.shape), dtype, 80))
    g.v.copy_(rand(tuple(g.v.shape), dtype, 81))
    lengths = [0, 63, 64, 700, 1500]
    slots = [cache.alloc() for _ in lengths]
    for s, n in zip(slots, lengths):
        cache.assume_length(s, n)
        cache.reserve(s, n + 1)
    cache.flush()
    poison_beyond(cache, slots, [n + 1 for n in lengths])
    ctx = make_ctx(cache, ops, slots, [1] * len(lengths), dtype)
    n_kv = kv_heads if store else 0
    qkv = rand((len(lengths), (heads + 2 * n_kv) * head_dim), dtype, 82)
    q_w = k_w = None
    if norm is not None:
        q_w, k_w = 1.0 + rand((head_dim,), norm, 83, 0.2), 1.0 + rand((head_dim,), norm, 84, 0.2)
    tables = None
    if rotary:
        angle = torch.arange(1600, dtype=torch.float32, device="cuda")[:, None] * \
            (10000.0 ** (-torch.arange(head_dim // 2, dtype=torch.float32, device="cuda") * 2 / head_dim))[None, :]
        tables = (angle.cos().to(dtype), angle.sin().to(dtype), head_dim)
    scale = 1.0 / math.sqrt(head_dim)
    k0, v0 = g.k.clone(), g.v.clone()
    got = ops.qk_attention(ctx, qkv, cache.layers[0], heads, n_kv, head_dim, q_w, k_w, 1e-5, tables, scale, window)
    assert got is not None, "the step is of the kind the fused kernel serves"
    k_got, v_got = g.k.clone(), g.v.clone()
    g.k.copy_(k0)
    g.v.copy_(v0)
    q = ref.qk_norm_rope_store(ctx, qkv, cache.layers[0], heads, n_kv, head_dim, q_w, k_w, 1e-5, tables)
    want = ref.attention(ctx, q, cache.layers[0], heads, scale, window)
    close(got, want, dtype, "decode attention with q/k preparation inside")
    assert torch.equal(k_got.isnan(), g.k.isnan())          # the poison beyond the sequences stays where it was
    close(k_got.nan_to_num(), g.k.nan_to_num(), dtype, "keys left in the cache")
    same = float((k_got.nan_to_num() == g.k.nan_to_num()).float().mean())
    assert same >= 0.9999, f"only {same:.6f} of the cache's keys have the restatement's bits"   # all but a few of the new rows
    assert torch.equal(v_got.nan_to_num(), g.v.nan_to_num())
    assert int(ctx.status.item()) == 0
    if not store:
        assert torch.equal(k_got.nan_to_num(), k0.nan_to_num())


@pytest.mark.parametrize("M", [1, 5, 8, 11, 16, 19, 24, 29, 32])
@pytest.mark.parametrize("splits,tiled,warps", [(1, False, 8), (3, False, 8), (2, True, 8), (1, True, 4), (2, False, 4), (8, False, 4),
                                                (11, False, 8), (3, True, 8), (11, True, 4), (5, True, 8), (6, False, 4), (7, True, 4)])
def test_skinny_product_variants(ops, ref, M, splits, tiled, warps):
    """The weight-streaming product with every row tile, K slicing, way of meeting (cluster, scratch) and weight
    layout (row-major, tile-major copy), with and without the SwiGLU epilogue, at sizes that are no multiples
    of its tiles."""
    dtype = torch.bfloat16
    try:
        ops.force_skinny = (splits, tiled, warps)
        a, w = rand((M, 4104), dtype, 70), rand((2 * 1000, 4104), dtype, 71, 0.05)
        if tiled:   # a copy for each pairing of rows: the whole matrix as one, and as [gate; up]
            w_pairs = w.clone()
            assert ops.prepare_matrix(w) is w and ops.prepare_matrix(w_pairs, halves=2) is w_pairs
            assert w._sb_tiled[1] == 1 and w_pairs._sb_tiled[1] == 2
            close(ops._skinny(a, w_pairs, 1000, True, False), ref.linear_swiglu(a, w), dtype, "skinny + swiglu, tile-major")
        close(ops._skinny(a, w, 2000, False, False), ref.linear(a, w), dtype, "skinny")
        close(ops._skinny(a, w, 2000, False, True), ref.linear(a, w, out_float32=True), dtype, "skinny, 32-bit out", rel=2e-3)
        close(ops._skinny(a, w, 1000, True, False), ref.linear_swiglu(a, w), dtype, "skinny + swiglu")
    finally:
        ops.force_skinny = None


@pytest.mark.parametrize("M", [1, 5, 8, 11, 16])
@pytest.mark.parametrize("splits,tiled,warps", [(1, False, 8), (1, True, 4), (3, True, 8), (2, False, 4), (11, True, 4)])
def test_skinny_product_with_norm_and_sum_inside(ops, ref, M, splits, tiled, warps):
    """The decode product with the RMSNorm of its rows in the prologue and the residual sum in the epilogue, against
    the norm kernel followed by the plain product and a 32-bit sum.  Rows have very different sizes, so that a row
    normed with another row's statistics would show; the widths are no multiples of the kernel's tiles."""
    dtype = torch.bfloat16
    K, N = 1000, 328
    try:
        ops.force_skinny = (splits, tiled, warps)
        x = rand((M, K), dtype, 90) * torch.logspace(-2, 2, M).cuda().to(dtype)[:, None]
        gamma = (1.0 + rand((K,), dtype, 91, 0.3).float()).to(dtype)
        w, w_pairs = rand((N, K), dtype, 92, 0.05), rand((2 * N, K), dtype, 93, 0.05)
        if tiled:
            ops.prepare_matrix(w)
            ops.prepare_matrix(w_pairs, halves=2)
        eps = 1e-5
        normed = ops.rmsnorm(x, gamma, eps)
        close(normed, ref.rmsnorm(x, gamma, eps), dtype, "norm kernel")
        # the norm inside: the same bits as norm kernel + product almost everywhere (the statistics are summed in
        # another order, which can move a rounding), and close to the restatement
        want = ops._skinny(normed, w, N, False, False)
        got = ops._skinny(x, w, N, False, False, norm=(gamma, eps))
        close(got, ref.linear(ref.rmsnorm(x, gamma, eps), w), dtype, "product of the norm")
        assert float((got == want).float().mean()) >= 0.99
        want_act = ops._skinny(normed, w_pairs, N, True, False)
        got_act = ops._skinny(x, w_pairs, N, True, False, norm=(gamma, eps))
        close(got_act, ref.linear_swiglu(ref.rmsnorm(x, gamma, eps), w_pairs), dtype, "swiglu of the product of the norm")
        assert float((got_act == want_act).float().mean()) >= 0.99
        # the sum inside: exactly the 32-bit sum of the residual and the rounded product, rounded once
        a = rand((M, K), dtype, 94)
        w_back = rand((K, K), dtype, 95, 0.05)
        if tiled:
            ops.prepare_matrix(w_back)
        residual = rand((M, K), dtype, 96, 2.0)
        product = ops._skinny(a, w_back, K, False, False)
        summed = residual.clone()
        assert ops._skinny(a, w_back, K, False, False, add_to=summed) is summed
        assert torch.equal(summed, (residual.float() + product.float()).to(dtype))
        # both at once, as a layer's branch uses them
        both = residual[:, :N].clone()
        ops._skinny(x, w, N, False, False, norm=(gamma, eps), add_to=both)
        assert torch.equal(both, (residual[:, :N].float() + got.float()).to(dtype))
        # the statistics that the sum leaves for the next product's norm: the squares of the new rows, 16 columns a
        # piece; a product that reads them gives what a product that reads the rows gives
        from types import SimpleNamespace
        stream = SimpleNamespace(x=residual.clone(), stats=None)
        ops._skinny(a, w_back, K, False, False, add_to=stream)
        assert torch.equal(stream.x, summed) and tuple(stream.stats.shape) == (M, -(-K // 16))
        pieces = torch.nn.functional.pad(summed.float() ** 2, (0, -K % 16)).view(M, -1, 16).sum(-1)
        assert torch.allclose(stream.stats, pieces, rtol=1e-5, atol=0)
        with_stats = ops._skinny(summed, w, N, False, False, norm=(gamma, eps, stream.stats))
        without = ops._skinny(summed, w, N, False, False, norm=(gamma, eps))
        close(with_stats, ref.linear(ref.rmsnorm(summed, gamma, eps), w), dtype, "product of the norm from statistics")
        assert float((with_stats == without).float().mean()) >= 0.99
    finally:
        ops.force_skinny = None
    with pytest.raises(Exception, match="16 rows"):
        ops._skinny(rand((17, K), dtype, 97), w, N, False, False, norm=(gamma, eps))
    with pytest.raises(Exception, match="bfloat16"):
        ops._skinny(x, w, N, False, False, norm=(gamma.float(), eps))
    with pytest.raises(Exception, match="adds to"):
        ops._skinny(x, w, N, False, False, add_to=residual)


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(8, 2, 128, None), (3, 1, 64, 150)])
def test_prefill_attention_over_many_pages(ops, ref, heads, kv_heads, head_dim, window):
    """Long pieces appended to contexts that already hold tokens; one far key is made to stand out."""
    dtype = torch.bfloat16
    caches = [Cache([KVRequest(kv_heads, head_dim, window)], n_slots=3, max_tokens=64 * 40, dtype=dtype, device="cuda",
                    max_step_tokens=512) for _ in range(2)]
    for step, q_lens in enumerate([(200, 64), (450, 333)]):
        outs = []
        qkv = rand((sum(q_lens), (heads + 2 * kv_heads) * head_dim), dtype, 80 + step, 0.5)
        if step == 0:
            qkv[37, heads * head_dim:(heads + 1) * head_dim] = 3.0     # key 37 of sequence 0 is large ...
        elif window is None:
            qkv[449, :head_dim] = 3.0                                  # ... and a late query of head 0 points at it
        for c, o in zip(caches, (ops, ref)):
            sl = [0, 1]
            if step == 0:
                assert [c.alloc(), c.alloc()] == sl
            for s_, n in zip(sl, q_lens):
                c.reserve(s_, c.lengths_host[s_] + n)
            c.flush()
            ctx = make_ctx(c, ops, sl, q_lens, dtype)
            q = o.qk_norm_rope_store(ctx, qkv, c.layers[0], heads, kv_heads, head_dim, None, None, 0.0, None)
            outs.append(o.attention(ctx, q, c.layers[0], heads, 1.0 / math.sqrt(head_dim), window))
            o.advance_lengths(ctx)
            for s_, n in zip(sl, q_lens):
                c.advance_host(s_, n)
        close(outs[0], outs[1], dtype, f"prefill attention, step {step}")
    if window is None:
        want = caches[0].groups[0].v[0, int(caches[0].groups[0].table_host[0, 0]), 0, 37].float()
        got = outs[0][449, :head_dim].float()
        assert float((got - want).abs().max()) < 0.05 * float(want.abs().max())


def test_prefill_attention_far_into_a_long_context(ops, ref):
    """A piece appended after 9,000 cached tokens: more pages than the kernel keeps ids for at a time (its
    ring of page ids is refilled on the way), and products that run a page ahead of the softmax throughout."""
    dtype, heads, kv_heads, head_dim = torch.bfloat16, 8, 2, 128
    cache = Cache([KVRequest(kv_heads, head_dim, None)], n_slots=2, max_tokens=64 * 150, dtype=dtype, device="cuda",
                  max_step_tokens=512)
    g = cache.groups[0]
    g.k.copy_(rand(tuple(g.k.shape), dtype, 90))
    g.v.copy_(rand(tuple(g.v.shape), dtype, 91))
    slot = cache.alloc()
    cache.reserve(slot, 9000 + 300)
    cache.assume_length(slot, 9000)
    cache.flush()
    poison_beyond(cache, [slot], [9300])
    ctx = make_ctx(cache, ops, [slot], [300], dtype)
    qkv = rand((300, (heads + 2 * kv_heads) * head_dim), dtype, 92, 0.5)
    page = int(g.table_host[slot, 8500 // 64])
    g.k[0, page, 0, 8500 % 64] = 3.0          # key 8,500 is large and the last query of head 0 points at it
    qkv[-1, :head_dim] = 3.0
    outs = []
    k0, v0 = g.k.clone(), g.v.clone()
    for o in (ops, ref):
        q = o.qk_norm_rope_store(ctx, qkv, cache.layers[0], heads, kv_heads, head_dim, None, None, 0.0, None)
        outs.append(o.attention(ctx, q, cache.layers[0], heads, 1.0 / math.sqrt(head_dim), None))
        g.k.copy_(k0)
        g.v.copy_(v0)
    close(outs[0], outs[1], dtype, "prefill attention, long context")
    want = g.v[0, page, 0, 8500 % 64].float()
    assert float((outs[0][-1, :head_dim].float() - want).abs().max()) < 0.05 * float(want.abs().max())
    assert ops.read_kernel_status() == 0


@pytest.mark.parametrize("shape", [(1, 6144, 2560), (8, 2560, 9728), (16, 1000, 4104), (33, 2560, 4096), (20, 700, 520),
                                   (64, 151936, 256), (5, 130, 72)])
def test_stream_product(ops, ref, shape):
    """The TMA + tcgen05 weight-streaming product: tiles split between blocks, ragged edges in every dimension."""
    M, N, K = shape
    dtype = torch.bfloat16
    a, w = rand((M, K), dtype, 90), rand((N, K), dtype, 91, 0.05)
    close(ops._stream_product(a, w, N, False, False), ref.linear(a, w), dtype, "stream")
    close(ops._stream_product(a, w, N, False, True), ref.linear(a, w, out_float32=True), dtype, "stream, 32-bit out", rel=2e-3)
    assert ops.read_kernel_status() == 0


@pytest.mark.parametrize("shape", [(8, 9728, 2560), (30, 1000, 1160), (1, 200, 64)])
def test_stream_product_with_swiglu(ops, ref, shape):
    M, I, K = shape
    dtype = torch.bfloat16
    h, w = rand((M, K), dtype, 92), rand((2 * I, K), dtype, 93, 0.05)
    close(ops._stream_product(h, w, I, True, False), ref.linear_swiglu(h, w), dtype, "stream + swiglu")
    close(ops._stream_product(h, w, I, True, False), ref.linear_swiglu(h, w), dtype, "stream + swiglu, again")  # counters were left zero
    assert ops.read_kernel_status() == 0


def test_rope_store_head_128_with_32_bit_norm_weights(ops, ref):
    """The vectorised rope-and-store kernel (bfloat16, head size 128) with norm weights kept in 32-bit."""
    dtype, heads, kv_heads, D = torch.bfloat16, 4, 2, 128
    caches = [Cache([KVRequest(kv_heads, D)], n_slots=2, max_tokens=64 * 4, dtype=dtype, device="cuda") for _ in range(2)]
    ang = torch.arange(200, dtype=torch.float32)[:, None] / (10000.0 ** (torch.arange(64).float() / 64))[None]
    rotary = (ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda(), D)
    qn, kn = 1 + 0.1 * rand((D,), torch.float32, 100), 1 + 0.1 * rand((D,), torch.float32, 101)
    qkv = rand((70, (heads + 2 * kv_heads) * D), dtype, 102)
    outs = []
    for c, o in zip(caches, (ops, ref)):
        slot = c.alloc()
        c.reserve(slot, 70)
        c.flush()
        ctx = make_ctx(c, ops, [slot], [70], dtype)
        outs.append(o.qk_norm_rope_store(ctx, qkv, c.layers[0], heads, kv_heads, D, qn, kn, 1e-6, rotary))
        assert int(ctx.status) == 0
    close(outs[0], outs[1], dtype, "q", rel=8e-3)
    close(caches[0].groups[0].k, caches[1].groups[0].k, dtype, "stored keys", rel=8e-3)
    assert torch.equal(caches[0].groups[0].v, caches[1].groups[0].v)


@pytest.mark.parametrize("dtype,head_dim", [(torch.float32, 32), (torch.bfloat16, 128), (torch.bfloat16, 64)])
def test_attention_respects_the_window_edge(ops, dtype, head_dim):
    """A huge key just outside the window must not count; the same key just inside must win.
    Checked for a long piece (prefill kernels) and for a single new token (decode kernels)."""
    heads, window, n = 4, 70, 200
    for q_len in (n, 1):
        for inside in (False, True):
            cache = Cache([KVRequest(1, head_dim, window)], n_slots=1, max_tokens=64 * 5, dtype=dtype, device="cuda",
                          max_step_tokens=256)
            slot = cache.alloc()
            cache.reserve(slot, n)
            cache.flush()
            qkv = rand((n, (heads + 2) * head_dim), dtype, 110, 0.05)
            edge = n - 1 - window + (1 if inside else 0)         # the last query sees keys edge+1 .. n-1 (or edge .. n-1)
            qkv[edge, heads * head_dim:(heads + 1) * head_dim] = 6.0
            qkv[-1, :heads * head_dim] = 6.0
            if q_len == n:
                ctx = make_ctx(cache, ops, [slot], [n], dtype)
                q = ops.qk_norm_rope_store(ctx, qkv, cache.layers[0], heads, 1, head_dim, None, None, 0.0, None)
                a = ops.attention(ctx, q, cache.layers[0], heads, 1.0, window)
            else:
                ctx = make_ctx(cache, ops, [slot], [n - 1], dtype)
                ops.qk_norm_rope_store(ctx, qkv[:-1].contiguous(), cache.layers[0], heads, 1, head_dim, None, None, 0.0, None)
                ops.advance_lengths(ctx)
                cache.advance_host(slot, n - 1)
                ctx = make_ctx(cache, ops, [slot], [1], dtype)
                q = ops.qk_norm_rope_store(ctx, qkv[-1:].contiguous(), cache.layers[0], heads, 1, head_dim, None, None, 0.0, None)
                a = ops.attention(ctx, q, cache.layers[0], heads, 1.0, window)
            value_at_edge = qkv[edge, (heads + 1) * head_dim:].float()
            got = a[-1, :head_dim].float()
            is_edge_value = float((got - value_at_edge).abs().max()) < 0.05 * float(value_at_edge.abs().max()) + 1e-3
            assert is_edge_value == inside, f"q_len {q_len}, key {'inside' if inside else 'outside'} the window"


@pytest.mark.parametrize("width", [520, 1000, 2560, 3080, 4096])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_rmsnorm_of_many_rows(ops, ref, width, wdtype):
    """From 128 rows on the bfloat16 norm runs a warp per row (1 to 16 vectors of eight values per lane): same bits in
    the residual sum, and the norm within a rounding step, for widths that fill the last vector and that do not."""
    dtype, rows = torch.bfloat16, 301
    x = rand((rows, width), dtype, 70, 3.0)
    w = (1 + 0.1 * rand((width,), torch.float32, 71)).to(wdtype)
    close(ops.rmsnorm(x, w, 1e-5), ref.rmsnorm(x, w, 1e-5), dtype, "rmsnorm", rel=8e-3)
    d = rand((rows, width), dtype, 72)
    x1, x2 = x.clone(), x.clone()
    y1, y2 = ops.add_rmsnorm(x1, d, w, 1e-6), ref.add_rmsnorm(x2, d, w, 1e-6)
    assert torch.equal(x1, x2), "residual sum"
    close(y1, y2, dtype, "add_rmsnorm", rel=8e-3)
    same = float((y1 == y2).float().mean())       # the same roundings: only a last bit of the sum of squares can move a value
    assert same >= 0.999, f"only {same:.5f} of the normed values have the restatement's bits"
    few = ops.add_rmsnorm(x.clone()[:7], d[:7], w, 1e-6)      # the block-per-row kernel on the same rows
    assert float((few.float() - y1[:7].float()).abs().max()) <= 8e-3 * float(y1.float().abs().max())


@pytest.mark.parametrize("heads,kv_heads", [(4, 2), (12, 3), (44, 4), (5, 1)])
def test_rope_store_of_many_rows(ops, ref, heads, kv_heads):
    """From 256 rows on, head size 128: a block per row, each warp with several heads' rows in flight.  Head counts
    that fill the warps' turns and that do not, three sequences at unequal positions."""
    dtype, D = torch.bfloat16, 128
    caches = [Cache([KVRequest(kv_heads, D)], n_slots=3, max_tokens=64 * 10, dtype=dtype, device="cuda", max_step_tokens=400)
              for _ in range(2)]
    ang = torch.arange(500, dtype=torch.float32)[:, None] / (10000.0 ** (torch.arange(64).float() / 64))[None]
    rotary = (ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda(), D)
    qn, kn = (1 + 0.1 * rand((D,), torch.float32, 100)).to(dtype), (1 + 0.1 * rand((D,), torch.float32, 101)).to(dtype)
    q_lens, starts = (200, 70, 31), (0, 65, 130)
    qkv = rand((sum(q_lens), (heads + 2 * kv_heads) * D), dtype, 102)
    outs = []
    for c, o in zip(caches, (ops, ref)):
        slots = [c.alloc() for _ in q_lens]
        for s, n, st in zip(slots, q_lens, starts):
            c.assume_length(s, st)
            c.reserve(s, st + n)
        c.flush()
        ctx = make_ctx(c, ops, slots, list(q_lens), dtype)
        outs.append(o.qk_norm_rope_store(ctx, qkv, c.layers[0], heads, kv_heads, D, qn, kn, 1e-6, rotary))
        assert int(ctx.status) == 0
    close(outs[0], outs[1], dtype, "q", rel=8e-3)
    close(caches[0].groups[0].k, caches[1].groups[0].k, dtype, "stored keys", rel=8e-3)
    assert torch.equal(caches[0].groups[0].v, caches[1].groups[0].v)
    # The kernel rounds where the formula rounds (five roundings a value), so nearly every value has the restatement's
    # bits; the rest sit one bfloat16 step away, where the two sums of squares differ in their last bit.
    same = float((outs[0] == outs[1]).float().mean())
    assert same >= 0.995, f"only {same:.5f} of the values have the restatement's bits"
