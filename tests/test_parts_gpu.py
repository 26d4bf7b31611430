"""Each part of a layer alone, built from its spec with random weights, against the plain formula."""

import math

import pytest
import torch

from plain import qwen3_plain as plain
from starter_b200.cache import Cache
from starter_b200.config import AttentionSpec, BlockSpec, GatedMLPSpec, NormSpec, RopeSpec
from starter_b200.engine.context import ResidualStream, Runtime, StepContext
from starter_b200.parts import build_part

pytestmark = pytest.mark.gpu
MODES = ["float32", "bfloat16"]


def runtime(mode):
    from starter_b200.csrc.ops import get_ops
    return Runtime(dtype=getattr(torch, mode), device=torch.device("cuda"), ops=get_ops(verbose=False))


def rand(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, mode, what, rel=None):
    rel = rel or (2e-5 if mode == "float32" else 2e-2)
    scale = float(want.abs().max())
    err = float((got.float().cpu() - want).abs().max())
    assert err <= rel * scale, f"{what}: {err:.3g} > {rel * scale:.3g}"


def one_sequence_ctx(rt, cache, n):
    slot = cache.alloc()
    cache.reserve(slot, n)
    cache.flush()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return StepContext(runtime=rt, cache=cache, n_seqs=1, n_rows=n, max_q_len=n, kv_bound=n, seq_slot=i32([slot]),
                       cu_q=i32([0, n]), row_seq=i32([0] * n), lengths=cache.lengths,
                       status=torch.zeros(1, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("mode", MODES)
def test_norm_part(mode):
    rt, rnd = runtime(mode), plain._rounder(mode)
    w = (1 + 0.1 * rand((200,), 1, dtype=torch.float32)).to(torch.bfloat16)
    part = build_part("norm", NormSpec(size=200, eps=3e-5), {"weight": w.to(rt.dtype).cuda()}, rt)
    x, d = rand((9, 200), 2, 2.0), rand((9, 200), 3)
    close(part.forward(x.to(rt.dtype).cuda()), plain.rms_norm(x.float(), w.float(), 3e-5, rnd), mode, "norm")
    xx = x.to(rt.dtype).cuda()
    y = part.add_forward(xx, d.to(rt.dtype).cuda())
    want_x = rnd(x.float() + d.float())
    close(xx, want_x, mode, "residual sum", rel=1e-6 if mode == "float32" else 4e-3)
    close(y, plain.rms_norm(want_x, w.float(), 3e-5, rnd), mode, "norm after add")


@pytest.mark.parametrize("mode", MODES)
def test_rope_part_tables(mode):
    rt = runtime(mode)
    part = build_part("position", RopeSpec(theta=123456.0, rotary_dim=48), {}, rt)
    part.prepare(300)
    cos, sin = plain.rope_tables(123456.0, 48, 300, plain._rounder(mode))
    got_cos, got_sin, dim = part.fused_rotary()
    assert dim == 48 and tuple(got_cos.shape) == (300, 24)
    assert torch.equal(got_cos.float().cpu(), cos[:, :24]) and torch.equal(got_sin.float().cpu(), sin[:, :24])
    assert torch.equal(cos[:, :24], cos[:, 24:])       # columns d and d + D/2 share an angle (engine/model.py:91)


@pytest.mark.parametrize("mode", MODES)
def test_gated_mlp_part(mode):
    rt, rnd = runtime(mode), plain._rounder(mode)
    spec = GatedMLPSpec(hidden_size=72, intermediate_size=200)
    w = {"gate": rand((200, 72), 4, 0.1), "up": rand((200, 72), 5, 0.1), "down": rand((72, 200), 6, 0.1)}
    part = build_part("ff", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    for rows in (3, 40):
        h = rand((rows, 72), 7)
        want = plain.mlp(h.float(), w["gate"].float(), w["up"].float(), w["down"].float(), rnd)
        close(part.forward(None, h.to(rt.dtype).cuda()), want, mode, f"mlp, {rows} rows")


def attention_weights(hq, hkv, d, hidden, seed):
    return {"q": rand((hq * d, hidden), seed, 0.1), "k": rand((hkv * d, hidden), seed + 1, 0.1),
            "v": rand((hkv * d, hidden), seed + 2, 0.1), "o": rand((hidden, hq * d), seed + 3, 0.1),
            "q_norm": (1 + 0.1 * rand((d,), seed + 4, dtype=torch.float32)).to(torch.bfloat16),
            "k_norm": (1 + 0.1 * rand((d,), seed + 5, dtype=torch.float32)).to(torch.bfloat16)}


def plain_attention_branch(h, w, hq, hkv, d, eps, theta, scale, window, rnd):
    T = h.shape[0]
    f = {k: v.float() for k, v in w.items()}
    q = plain.linear(h, f["q"], rnd).view(T, hq, d)
    k = plain.linear(h, f["k"], rnd).view(T, hkv, d)
    v = plain.linear(h, f["v"], rnd).view(T, hkv, d)
    q, k = plain.rms_norm(q, f["q_norm"], eps, rnd), plain.rms_norm(k, f["k_norm"], eps, rnd)
    cos, sin = plain.rope_tables(theta, d, T, rnd)
    q, k = plain.apply_rope(q, cos, sin, rnd), plain.apply_rope(k, cos, sin, rnd)
    return plain.linear(plain.attention(q, k, v, scale, window, rnd), f["o"], rnd)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("hq,hkv,d,window", [(6, 2, 32, None), (4, 4, 64, 50), (8, 2, 128, None)])
def test_attention_part(mode, hq, hkv, d, window):
    rt, rnd = runtime(mode), plain._rounder(mode)
    hidden, eps, theta, scale = 88, 2e-6, 50000.0, 0.7 / math.sqrt(d)
    spec = AttentionSpec(hidden_size=hidden, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=scale,
                         qk_norm=NormSpec(size=d, eps=eps), position=RopeSpec(theta=theta, rotary_dim=d), window=window)
    w = attention_weights(hq, hkv, d, hidden, 10)
    part = build_part("mixer", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    cache = Cache([part.cache_request()], n_slots=2, max_tokens=64 * 4, dtype=rt.dtype, device="cuda")
    part.prepare(cache)
    T = 150
    h = rand((T, hidden), 20)
    ctx = one_sequence_ctx(rt, cache, T)
    got = part.forward(ctx, h.to(rt.dtype).cuda(), cache.layers[0])
    assert int(ctx.status) == 0
    want = plain_attention_branch(rnd(h.float()), w, hq, hkv, d, eps, theta, scale, window, rnd)
    close(got, want, mode, "attention branch")


@pytest.mark.parametrize("mode", MODES)
def test_block_part(mode):
    """A whole pre-norm layer against plain.decoder_layer, through the tensor names of the plain model."""
    rt, rnd = runtime(mode), plain._rounder(mode)
    cfg = dict(hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=16, intermediate_size=96,
               rms_norm_eps=1e-5, rope_theta=10000.0)
    norm = NormSpec(size=80, eps=1e-5)
    spec = BlockSpec(mixer_norm=norm,
                     mixer=AttentionSpec(hidden_size=80, num_heads=5, num_kv_heads=5, head_dim=16, scale=0.25,
                                         qk_norm=NormSpec(size=16, eps=1e-5), position=RopeSpec(theta=10000.0, rotary_dim=16)),
                     ff_norm=norm, ff=GatedMLPSpec(hidden_size=80, intermediate_size=96))
    aw = attention_weights(5, 5, 16, 80, 30)
    names = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
             "o": "self_attn.o_proj.weight", "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight"}
    tensors = {"model.layers.0." + names[k]: v.float() for k, v in aw.items()}
    mw = {"gate": rand((96, 80), 40, 0.1), "up": rand((96, 80), 41, 0.1), "down": rand((80, 96), 42, 0.1)}
    for k, v in mw.items():
        tensors[f"model.layers.0.mlp.{k}_proj.weight"] = v.float()
    n1 = (1 + 0.1 * rand((80,), 43, dtype=torch.float32)).to(torch.bfloat16)
    n2 = (1 + 0.1 * rand((80,), 44, dtype=torch.float32)).to(torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = n1.float()
    tensors["model.layers.0.post_attention_layernorm.weight"] = n2.float()
    dev = lambda d: {k: v.to(rt.dtype).cuda() for k, v in d.items()}
    block = build_part("block", spec, {"mixer_norm": dev({"weight": n1}), "mixer": dev(aw), "ff_norm": dev({"weight": n2}),
                                       "ff": dev(mw)}, rt)
    cache = Cache([block.cache_request()], n_slots=1, max_tokens=128, dtype=rt.dtype, device="cuda")
    block.prepare(cache)
    T = 70
    x = rand((T, 80), 50)
    ctx = one_sequence_ctx(rt, cache, T)
    stream = ResidualStream(x.to(rt.dtype).cuda())
    block.forward(ctx, stream, cache.layers[0])
    got = stream.x.float().cpu() + stream.pending.float().cpu()   # the second branch is still waiting to be added
    cos, sin = plain.rope_tables(10000.0, 16, T, rnd)
    want = plain.decoder_layer(rnd(x.float()), 0, cfg, tensors, cos, sin, rnd)
    close(got, want, mode, "layer", rel=2e-5 if mode == "float32" else 2e-2)
