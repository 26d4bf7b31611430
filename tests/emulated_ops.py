"""A torch stand-in for the CUDA extension's call table, for tests without a GPU.

It gives every call of ``starter_b200.csrc.ops.Ops`` the same meaning in slow
torch code on whatever device the tensors are on, so that the host side of the
library (cache, paging, step cutting, generation loop) can be driven on a CPU.
It is test equipment: the library never falls back to it.  The GPU tests also
use these functions as the plain reference of each kernel.
"""

from __future__ import annotations

import math

import torch

from starter_b200.cache.cache import PAGE


def _rnd(t, dtype):
    return t.to(dtype).to(torch.float32)


class EmulatedOps:
    name = "emulated"

    def prepare_matrix(self, w, halves=1):
        return w

    # ---- rows ---------------------------------------------------------------------------

    def embed(self, tokens, table, status):
        bad = (tokens < 0) | (tokens >= table.shape[0])
        if bool(bad.any()):
            status |= 1
        return table[tokens.long().clamp(0, table.shape[0] - 1)].clone()

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def rmsnorm(self, x, w, eps):
        xf = x.float()
        n = xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
        return (_rnd(n, x.dtype) * w.float()).to(x.dtype)

    def add_rmsnorm(self, x, delta, w, eps):
        x.copy_((x.float() + delta.float()).to(x.dtype))
        return self.rmsnorm(x, w, eps)

    def linear(self, a, w, out_float32=False):
        out = a.float() @ w.float().T
        return out if out_float32 else out.to(a.dtype)

    def swiglu(self, gu):
        inter = gu.shape[1] // 2
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
        s = _rnd(g / (1.0 + torch.exp(-g)), gu.dtype)
        return (s * u).to(gu.dtype)

    def linear_swiglu(self, h, w_gate_up):
        return self.swiglu(self.linear(h, w_gate_up))

    # ---- cache --------------------------------------------------------------------------

    @staticmethod
    def _positions(ctx):
        slots = ctx.seq_slot.long()[ctx.row_seq.long()]
        first = ctx.cu_q.long()[ctx.row_seq.long()]
        rows = torch.arange(ctx.n_rows, device=slots.device)
        return slots, ctx.lengths.long()[slots] + rows - first

    @staticmethod
    def _physical(group, slots, pos):
        logical = pos // PAGE
        if group.ring_pages:
            logical = logical % group.ring_pages
        return group.table.long()[slots, logical], pos % PAGE

    def qk_norm_rope_store(self, ctx, qkv, layer_cache, n_heads, n_kv_heads, head_dim, q_norm, k_norm, eps, rotary):
        M, D, dt = qkv.shape[0], head_dim, qkv.dtype
        slots, pos = self._positions(ctx)
        q = qkv[:, :n_heads * D].float().reshape(M, n_heads, D)
        k = qkv[:, n_heads * D:(n_heads + n_kv_heads) * D].float().reshape(M, n_kv_heads, D)
        v = qkv[:, (n_heads + n_kv_heads) * D:].reshape(M, n_kv_heads, D)

        def norm(t, w):
            if w is None:
                return t
            n = _rnd(t * torch.rsqrt((t * t).sum(-1, keepdim=True) / D + eps), dt)
            return _rnd(n * w.float(), dt)

        def rope(t):
            if rotary is None:
                return t
            cos, sin, rd = rotary
            half = rd // 2
            c = cos.float()[pos][:, None, :]
            s = sin.float()[pos][:, None, :]
            t1, t2 = t[..., :half], t[..., half:rd]
            o1 = _rnd(_rnd(t1 * c, dt) + _rnd(-t2 * s, dt), dt)
            o2 = _rnd(_rnd(t2 * c, dt) + _rnd(t1 * s, dt), dt)
            return torch.cat([o1, o2, t[..., rd:]], dim=-1)

        q = rope(norm(q, q_norm))
        if n_kv_heads:
            k = rope(norm(k, k_norm))
            group = layer_cache.group
            page, off = self._physical(group, slots, pos)
            if bool((page < 0).any()):
                ctx.status |= 2
            ok = page >= 0
            layer_cache.k[page[ok], :, off[ok]] = k[ok].to(dt)
            layer_cache.v[page[ok], :, off[ok]] = v[ok].to(dt)
        return q.reshape(M, n_heads * D).to(dt)

    def attention(self, ctx, q, layer_cache, n_heads, scale, window):
        group = layer_cache.group
        M, dt = q.shape[0], q.dtype
        D = group.request.head_dim
        hkv = group.request.num_kv_heads
        rep = n_heads // hkv
        slots, pos = self._positions(ctx)
        out = torch.empty(M, n_heads * D, dtype=dt, device=q.device)
        qf = q.float().reshape(M, n_heads, D)
        for r in range(M):
            p = int(pos[r])
            lo = 0 if window is None else max(0, p - window + 1)
            keys = torch.arange(lo, p + 1, device=q.device)
            page, off = self._physical(group, slots[r].expand(keys.numel()), keys)
            kk = layer_cache.k[page, :, off].float().repeat_interleave(rep, dim=1)  # [n, HQ, D]
            vv = layer_cache.v[page, :, off].float().repeat_interleave(rep, dim=1)
            s = torch.einsum("hd,nhd->hn", qf[r], kk) * scale
            pr = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            total = pr.sum(-1, keepdim=True)
            pv = torch.einsum("hn,nhd->hd", _rnd(pr, dt), vv) / total
            out[r] = pv.reshape(-1).to(dt)
        return out

    def advance_lengths(self, ctx):
        counts = (ctx.cu_q[1:] - ctx.cu_q[:-1]).to(ctx.lengths.dtype)
        slots = ctx.seq_slot.long()
        real = slots < ctx.cache.null_slot
        ctx.lengths[slots[real]] += counts[real]

    # ---- sampling -----------------------------------------------------------------------

    def argmax(self, logits):
        return logits.float().argmax(dim=-1).to(torch.int32)

    def sample(self, logits, temperature, top_k, seed, request_ids, steps, advance=False, device_params=None):
        from plain import qwen3_plain as plain
        if device_params is not None:
            import struct
            words = [int(v) & 0xffffffff for v in device_params.tolist()]
            (temperature,) = struct.unpack("<f", struct.pack("<I", words[0]))
            top_k, seed = words[1], words[2] | (words[3] << 32)
        out = []
        for r in range(logits.shape[0]):
            req = int(request_ids[r]) if request_ids is not None else r
            step = int(steps[r]) if steps is not None else 0
            tok, _ = plain.sample(logits[r].float().cpu(), temperature, top_k, plain.uniform_from_counter(seed, req, step))
            out.append(tok)
        if advance and steps is not None:
            steps += 1
        return torch.tensor(out, dtype=torch.int32, device=logits.device)
