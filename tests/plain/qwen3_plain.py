"""Plain, slow Qwen3 forward pass: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the
package under test: it reads ``config.json`` and ``model.safetensors`` through
the ``safetensors`` library, and every function restates one formula of the
reference engine (IshaanBansal2006/starter), cited as ``file:line`` of that
project.  The reference's forward pass itself cannot run without a CUDA
device (its kernels are Triton), so this file rests on the formulas; the
pieces of the reference that do run on a CPU (rotary tables, fused weight
layout, the attention mask) are compared once in ``tests/golden``.

Two numeric modes:

* ``"float32"``: every product, sum and table in 32-bit, no rounding.
* ``"bfloat16"``: weights are bfloat16 and every intermediate is rounded to
  bfloat16 at exactly the places where the reference rounds; sums, softmax,
  norms and angles stay in 32-bit.  Logits are returned unrounded (32-bit).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def _rounder(mode: str):
    if mode == "float32":
        return lambda t: t
    if mode == "bfloat16":
        return lambda t: t.to(torch.bfloat16).to(torch.float32)
    raise ValueError(mode)


def read_folder(folder):
    """config.json as a dict and every tensor of every *.safetensors file of the folder, sorted
    (engine/model.py:67-75), widened to float32."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = {}
    for path in sorted(folder.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name).to(torch.float32)
    return cfg, tensors


def head_dim_of(cfg) -> int:
    """engine/model.py:47: head_dim, or hidden_size // num_attention_heads when absent."""
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg, layer: int):
    """Window of one layer in tokens, or None for full attention.

    The reference runs full causal attention only (OPTIMIZATION_GUIDE.md:43).
    The Qwen3 configuration keys ``use_sliding_window``, ``sliding_window``,
    ``max_window_layers`` and ``layer_types`` name a window for some layers;
    a query at position p then sees the keys n with p - window < n <= p.
    """
    types = cfg.get("layer_types")
    if types is not None:
        sliding = types[layer] == "sliding_attention"
    else:
        sliding = bool(cfg.get("use_sliding_window", False)) and layer >= cfg.get("max_window_layers", 0)
    if sliding and cfg.get("sliding_window"):
        return int(cfg["sliding_window"])
    return None


def embedding(table, ids):
    """engine/model.py:287: x[r, :] = embed[ids[r], :]."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, weight, eps, rnd):
    """engine/kernels/rmsnorm.py:31-45: 32-bit mean of squares over the last axis;
    the normalised value is rounded before the weight multiply, the product again."""
    x = x.to(torch.float32)
    variance = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    normed = rnd(x * torch.rsqrt(variance + eps))
    return rnd(normed * weight)


def linear(x, weight, rnd):
    """engine/model.py:291,295,297: y = x @ W.T with W as [out, in], 32-bit sum, rounded output."""
    return rnd(x.to(torch.float32) @ weight.to(torch.float32).T)


def rope_tables(theta, head_dim, n_pos, rnd):
    """engine/model.py:78-93: inv_freq[j] = 1 / theta**(2j/D) in 32-bit, angle = p * inv_freq[j]
    in 32-bit, the table is cat(angle, angle) so columns d and d + D/2 share an angle,
    and cos/sin are rounded after they are taken."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    positions = torch.arange(n_pos, dtype=torch.float32)
    freqs = positions[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return rnd(emb.cos()), rnd(emb.sin())


def apply_rope(y, cos, sin, rnd):
    """engine/kernels/rope.py:26-30: out = y*cos + rotate_half(y)*sin with
    rotate_half(y) = cat(-y[D/2:], y[:D/2]); each product and the sum are rounded.
    y: [T, heads, D]; cos, sin: [T, D]."""
    half = y.shape[-1] // 2
    rotated = torch.cat((-y[..., half:], y[..., :half]), dim=-1)
    return rnd(rnd(y * cos[:, None, :]) + rnd(rotated * sin[:, None, :]))


def attention(q, k, v, scale, window, rnd):
    """engine/kernels/attention.py:63-87 and engine/model.py:268-274: query head h reads
    key/value head h // (HQ/HKV); scores (q.k)*scale, softmax statistics in 32-bit; the
    probabilities exp(s - max) are rounded before they meet V, the 32-bit sum of the
    unrounded probabilities divides once at the end.  Key n is visible to the query at
    position p when n <= p (attention.py:75) and, with a window, p - n < window.
    q: [T, HQ, D]; k, v: [T, HKV, D] -> [T, HQ*D]."""
    T, HQ, D = q.shape
    group = HQ // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * scale
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= (pos[:, None] - pos[None, :]) < window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    top = scores.max(dim=-1, keepdim=True).values
    p = torch.exp(scores - top)
    total = p.sum(dim=-1, keepdim=True)
    out = torch.einsum("hts,shd->htd", rnd(p), v) / total
    return rnd(out.permute(1, 0, 2).reshape(T, HQ * D))


def swiglu(gate, up, rnd):
    """engine/kernels/swiglu.py:21-24: silu(g) = g / (1 + exp(-g)) in 32-bit, rounded, times up, rounded."""
    return rnd(rnd(gate / (1.0 + torch.exp(-gate))) * up)


def mlp(h, w_gate, w_up, w_down, rnd):
    """engine/model.py:297: down(swiglu(gate(h), up(h))); gate and up are rounded outputs of
    their products (engine/kernels/gemm.py:116-121)."""
    return linear(swiglu(linear(h, w_gate, rnd), linear(h, w_up, rnd), rnd), w_down, rnd)


def decoder_layer(x, layer, cfg, tensors, cos, sin, rnd):
    """OPTIMIZATION_GUIDE.md:60-69 and engine/model.py:289-298: two pre-norm residual
    branches; the residual sums are taken in 32-bit and rounded (add_rmsnorm.py:21-24)."""
    p = f"model.layers.{layer}."
    T = x.shape[0]
    HQ, HKV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, tensors[p + "input_layernorm.weight"], eps, rnd)
    q = linear(h, tensors[p + "self_attn.q_proj.weight"], rnd).view(T, HQ, D)
    k = linear(h, tensors[p + "self_attn.k_proj.weight"], rnd).view(T, HKV, D)
    v = linear(h, tensors[p + "self_attn.v_proj.weight"], rnd).view(T, HKV, D)
    # engine/kernels/rope.py:19-25: RMSNorm over each head vector, weight shared by the heads.
    q = rms_norm(q, tensors[p + "self_attn.q_norm.weight"], eps, rnd)
    k = rms_norm(k, tensors[p + "self_attn.k_norm.weight"], eps, rnd)
    q = apply_rope(q, cos, sin, rnd)
    k = apply_rope(k, cos, sin, rnd)
    a = attention(q, k, v, 1.0 / math.sqrt(D), layer_window(cfg, layer), rnd)  # scale: engine/model.py:130
    x = rnd(x + linear(a, tensors[p + "self_attn.o_proj.weight"], rnd))
    h = rms_norm(x, tensors[p + "post_attention_layernorm.weight"], eps, rnd)
    d = mlp(h, tensors[p + "mlp.gate_proj.weight"], tensors[p + "mlp.up_proj.weight"],
            tensors[p + "mlp.down_proj.weight"], rnd)
    return rnd(x + d)


def lm_head_weight(cfg, tensors):
    """engine/model.py:103-107: lm_head.weight when present, else the embedding when tied."""
    if "lm_head.weight" in tensors:
        return tensors["lm_head.weight"]
    if not cfg.get("tie_word_embeddings", False):
        raise KeyError("lm_head.weight missing and embeddings are not tied")
    return tensors["model.embed_tokens.weight"]


def forward(cfg, tensors, ids, mode="float32"):
    """Logits [T, V] (32-bit) at every position of one whole sequence.

    engine/model.py:280-299: embedding, the layers in order, final RMSNorm, LM head.
    The reference rounds its logits to bfloat16; here the last product is left in 32-bit."""
    rnd = _rounder(mode)
    if mode == "bfloat16":
        tensors = {n: rnd(t) for n, t in tensors.items()}
    x = embedding(tensors["model.embed_tokens.weight"], ids)
    cos, sin = rope_tables(cfg["rope_theta"], head_dim_of(cfg), len(ids), rnd)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, layer, cfg, tensors, cos, sin, rnd)
    h = rms_norm(x, tensors["model.norm.weight"], cfg["rms_norm_eps"], rnd)
    return h @ lm_head_weight(cfg, tensors).T


# ---------------------------------------------------------------------------------------
# sampling and the generation loop, restated plainly


def greedy(logits):
    """engine/engine.py:204,207 with the tie rule of engine/kernels/topk.py:4-5,27:
    the largest logit, the lowest index among equals."""
    logits = torch.as_tensor(logits, dtype=torch.float32)
    best = logits.max()
    return int(torch.nonzero(logits == best)[0, 0])


def uniform_from_counter(seed: int, request: int, step: int) -> float:
    """The sampler's uniform number in [0, 1): a splitmix64 finaliser over the three keys,
    top 24 bits.  The reference samples greedily only; this definition is the library's own
    and is restated here in integer arithmetic."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample(logits, temperature: float, top_k: int, u: float):
    """Temperature / top-k draw as a pure function of 32-bit logits and one uniform u.

    Kept set: the top_k largest logits (all when top_k == 0), ties at the edge resolved
    toward lower indices.  Weights exp((l - max) / T); the token is the first index, in
    index order over the kept set, whose running sum reaches u * total.  Returns the token
    and the distance of u * total from the nearest edge of the running sum, relative to
    total, so a caller can tell a draw that 32-bit rounding could flip."""
    logits = torch.as_tensor(logits, dtype=torch.float64)
    if temperature <= 0.0:
        return greedy(logits), 1.0
    V = logits.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        order = sorted(range(V), key=lambda i: (-float(logits[i]), i))[:top_k]
        keep[:] = False
        keep[order] = True
    w = torch.where(keep, torch.exp((logits - logits[keep].max()) / temperature), torch.zeros((), dtype=torch.float64))
    running = torch.cumsum(w, 0)
    total = float(running[-1])
    target = u * total
    token = int(torch.nonzero(running > target)[0, 0]) if target < total else int(torch.nonzero(keep)[-1, 0])
    edges = torch.cat([torch.zeros(1, dtype=torch.float64), running[keep]])
    margin = float((edges - target).abs().min()) / total
    return token, margin


def generate(cfg, tensors, prompts, max_new_tokens, mode="float32", temperature=0.0, top_k=0, seed=0,
             stop_token_ids=()):
    """One list of new tokens per prompt: whole-sequence forward for every new token
    (README.md:54-66: one token per sequence per step; stop tokens are this library's addition:
    a sequence ends with its first stop token, which is part of its output)."""
    outs = []
    for r, prompt in enumerate(prompts):
        seq, new = list(prompt), []
        for step in range(max_new_tokens):
            logits = forward(cfg, tensors, seq, mode)[-1]
            if temperature > 0.0:
                tok, _ = sample(logits, temperature, top_k, uniform_from_counter(seed, r, step))
            else:
                tok = greedy(logits)
            seq.append(tok)
            new.append(tok)
            if tok in stop_token_ids:
                break
        outs.append(new)
    return outs
