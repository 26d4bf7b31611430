"""Times one kernel on one of the decode shapes: replay of a CUDA graph that walks through copies of the
weights (more bytes than L2 holds), median of several replays.  The reference times its candidate
kernels the same way (engine/kernels/gemm.py:477-513).

    python -m starter_b200.csrc.microbench --kernel stream --shape gateup --rows 8
    python -m starter_b200.csrc.microbench --kernel attn_decode --rows 8 --context 4096
    python -m starter_b200.csrc.microbench --kernel attn_prefill --tokens 2048 --context 2048
    python -m starter_b200.csrc.microbench --kernel rope_store --rows 2048      (also rmsnorm, swiglu)
"""

from __future__ import annotations

import argparse
import json
import math

import torch

SHAPES = {"qkv": (6144, 2560, False), "o": (2560, 4096, False), "gateup": (9728, 2560, True),
          "down": (2560, 9728, False), "lm_head": (151936, 2560, False)}


def time_graph(calls, replays: int = 5) -> float:
    """Microseconds per call: the calls are captured in one graph, the median replay is reported."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in calls[:2]:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in calls:
            f()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1000.0 / len(calls))
    return sorted(times)[len(times) // 2]


def bench_product(ops, kernel: str, shape: str, rows: int, copies: int):
    n_out, K, gate_up = SHAPES[shape]
    w_rows = 2 * n_out if gate_up else n_out
    copies = min(copies, max(2, (1 << 31) // (w_rows * K * 2)))
    ws = [torch.randn(w_rows, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    a = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
    if kernel == "skinny":   # as the parts do it: the decode product reads the tile-major copy when there is one
        ws = [ops.prepare_matrix(w, halves=2 if gate_up else 1) for w in ws]
    if kernel == "stream":
        calls = [lambda w=w: ops._stream_product(a, w, n_out, gate_up, False) for w in ws]
    elif kernel == "skinny":
        calls = [lambda w=w: ops._skinny(a, w, n_out, gate_up, False) for w in ws]
    elif kernel == "cublas":
        calls = [lambda w=w: torch.mm(a, w.t()) for w in ws]
    else:
        raise SystemExit(f"unknown product kernel {kernel!r}")
    us = time_graph(calls)
    nbytes = w_rows * K * 2
    return {"kernel": kernel, "shape": shape, "rows": rows, "us": round(us, 2), "weight_bytes": nbytes,
            "GB/s": round(nbytes / us / 1e3, 1)}


def bench_attn_decode(ops, rows: int, context: int, heads: int, kv_heads: int, head_dim: int, layers: int, long_context: int = 0):
    """One new token per sequence over caches of ``context`` tokens; with ``long_context`` the first sequence holds
    that many instead, and the step's context carries the hint that the lengths are very unequal when they are."""
    from ..cache import Cache, KVRequest
    from ..engine.context import Runtime, StepContext, lengths_uneven
    dtype = torch.bfloat16
    lengths = [max(long_context, 1) if long_context and i == 0 else context for i in range(rows)]
    cache = Cache([KVRequest(kv_heads, head_dim)] * layers, n_slots=rows, max_tokens=sum(-(-n // 64) * 64 for n in lengths),
                  dtype=dtype, device="cuda", max_seq_tokens=max(lengths))
    cache.groups[0].k.normal_()
    cache.groups[0].v.normal_()
    slots = [cache.alloc() for _ in range(rows)]
    for s, n in zip(slots, lengths):
        cache.assume_length(s, n - 1)
    cache.flush()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    ctx = StepContext(runtime=Runtime(dtype, torch.device("cuda"), ops), cache=cache, n_seqs=rows, n_rows=rows, max_q_len=1,
                      kv_bound=max(lengths), seq_slot=i32(slots), cu_q=i32(list(range(rows + 1))), row_seq=i32(list(range(rows))),
                      lengths=cache.lengths, status=torch.zeros(1, dtype=torch.int32, device="cuda"),
                      uneven=lengths_uneven(lengths))
    q = torch.randn(rows, heads * head_dim, device="cuda", dtype=dtype)
    calls = [lambda lc=lc: ops.attention(ctx, q, lc, heads, 1.0 / math.sqrt(head_dim), None) for lc in cache.layers]
    us = time_graph(calls)
    nbytes = sum(lengths) * kv_heads * head_dim * 2 * 2
    out = {"kernel": "attn_decode", "rows": rows, "context": context, "us": round(us, 2), "cache_bytes": nbytes,
           "GB/s": round(nbytes / us / 1e3, 1)}
    if long_context:
        out.update(long_context=long_context, uneven=ctx.uneven)
    return out


def bench_attn_prefill(ops, tokens: int, context: int, heads: int, kv_heads: int, head_dim: int, layers: int):
    """One sequence that holds ``context - tokens`` tokens and brings ``tokens`` new ones."""
    from ..cache import Cache, KVRequest
    from ..engine.context import Runtime, StepContext
    dtype = torch.bfloat16
    cache = Cache([KVRequest(kv_heads, head_dim)] * layers, n_slots=1, max_tokens=context, dtype=dtype, device="cuda",
                  max_seq_tokens=context, max_step_tokens=tokens)
    cache.groups[0].k.normal_()
    cache.groups[0].v.normal_()
    slot = cache.alloc()
    cache.reserve(slot, context)
    cache.assume_length(slot, context - tokens)
    cache.flush()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    ctx = StepContext(runtime=Runtime(dtype, torch.device("cuda"), ops), cache=cache, n_seqs=1, n_rows=tokens, max_q_len=tokens,
                      kv_bound=context, seq_slot=i32([slot]), cu_q=i32([0, tokens]), row_seq=i32([0] * tokens),
                      lengths=cache.lengths, status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    q = torch.randn(tokens, heads * head_dim, device="cuda", dtype=dtype)
    calls = [lambda lc=lc: ops.attention(ctx, q, lc, heads, 1.0 / math.sqrt(head_dim), None) for lc in cache.layers]
    us = time_graph(calls)
    start = context - tokens
    flops = 4.0 * head_dim * heads * (tokens * start + tokens * (tokens + 1) / 2.0)
    return {"kernel": "attn_prefill", "tokens": tokens, "context": context, "us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1)}


def bench_rows(ops, kernel: str, rows: int, copies: int = 6):
    """The row-wise kernels of a prefill at the 4B layer sizes: add + norm, q/k norm + rotary + cache store, SwiGLU."""
    from ..cache import Cache, KVRequest
    from ..engine.context import Runtime, StepContext
    dt = torch.bfloat16
    H, I, HQ, HKV, D = 2560, 9728, 32, 8, 128
    if kernel == "rmsnorm":
        xs = [torch.randn(rows, H, device="cuda", dtype=dt) for _ in range(copies)]
        d = torch.randn(rows, H, device="cuda", dtype=dt)
        w = torch.ones(H, device="cuda", dtype=dt)
        calls = [lambda x=x: ops.add_rmsnorm(x, d, w, 1e-6) for x in xs]
        nbytes = 4 * rows * H * 2
    elif kernel == "swiglu":
        gus = [torch.randn(rows, 2 * I, device="cuda", dtype=dt) for _ in range(copies)]
        calls = [lambda g=g: ops.swiglu(g) for g in gus]
        nbytes = 3 * rows * I * 2
    else:
        cache = Cache([KVRequest(HKV, D)] * copies, n_slots=1, max_tokens=rows, dtype=dt, device="cuda", max_seq_tokens=rows,
                      max_step_tokens=rows)
        slot = cache.alloc()
        cache.reserve(slot, rows)
        cache.flush()
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        ctx = StepContext(runtime=Runtime(dt, torch.device("cuda"), ops), cache=cache, n_seqs=1, n_rows=rows, max_q_len=rows,
                          kv_bound=rows, seq_slot=i32([slot]), cu_q=i32([0, rows]), row_seq=i32([0] * rows), lengths=cache.lengths,
                          status=torch.zeros(1, dtype=torch.int32, device="cuda"))
        qkvs = [torch.randn(rows, (HQ + 2 * HKV) * D, device="cuda", dtype=dt) for _ in range(copies)]
        qn = torch.ones(D, device="cuda", dtype=dt)
        ang = torch.arange(rows, dtype=torch.float32)[:, None] / (5e6 ** (torch.arange(D // 2).float() / (D // 2)))[None]
        rotary = (ang.cos().to(dt).cuda(), ang.sin().to(dt).cuda(), D)
        calls = [lambda q=q, lc=lc: ops.qk_norm_rope_store(ctx, q, lc, HQ, HKV, D, qn, qn, 1e-6, rotary)
                 for q, lc in zip(qkvs, cache.layers)]
        nbytes = rows * ((HQ + 2 * HKV) + HQ + 2 * HKV) * D * 2
    us = time_graph(calls)
    return {"kernel": kernel, "rows": rows, "us": round(us, 2), "bytes": nbytes, "GB/s": round(nbytes / us / 1e3, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--kernel", required=True, choices=["stream", "skinny", "cublas", "attn_decode", "attn_prefill", "rmsnorm", "rope_store", "swiglu"])
    ap.add_argument("--shape", default="gateup", choices=sorted(SHAPES))
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--copies", type=int, default=12, help="copies of the weights the graph walks through")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--long-context", type=int, default=0, help="attn_decode: the first sequence holds this many tokens instead")
    ap.add_argument("--tokens", type=int, default=2048, help="attn_prefill: new tokens of the sequence")
    ap.add_argument("--layers", type=int, default=8, help="attn_decode: layers of cache the graph walks through")
    ap.add_argument("--dependent-launch", action="store_true", help="launch with programmatic dependent launch")
    args = ap.parse_args(argv)
    from .ops import get_ops
    ops = get_ops(verbose=False)
    ops.set_dependent_launch(args.dependent_launch)
    if args.kernel in ("rmsnorm", "rope_store", "swiglu"):
        out = bench_rows(ops, args.kernel, args.rows)
    elif args.kernel == "attn_prefill":
        out = bench_attn_prefill(ops, args.tokens, max(args.context, args.tokens), 32, 8, 128, args.layers)
    elif args.kernel == "attn_decode":
        out = bench_attn_decode(ops, args.rows, args.context, 32, 8, 128, args.layers, args.long_context)
    else:
        out = bench_product(ops, args.kernel, args.shape, args.rows, args.copies)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
