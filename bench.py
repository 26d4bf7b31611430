#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-4B shape on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences at a context of 4,096
tokens.  Prints one JSON line: ``value`` = decoded tokens per second timed on
the device over exactly K graph-replayed steps; ``e2e`` = the same through
``Engine.generate`` with host token lists in and out; ``prefill`` = one prompt
of 2,048 tokens; ``roofline`` = bytes the decode step has to read (every
weight once, the cache of the live sequences) over its time, against the
measured copy bandwidth; ``points`` = decode at batch 1 and 64.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rms_norm_eps=1e-6,
                rope_theta=5000000.0, tie_word_embeddings=True)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            peaks = {k: float(raw[k]) for k in FALLBACK_PEAKS if k in raw}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int = 0):
        self.proc = None
        self.lines = []
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, max_mhz, reasons = [], 0, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(int(float(parts[0])))
                max_mhz = max(max_mhz, int(float(parts[1])))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def model_numbers(cfg, n_layers):
    """Bytes of the weights a decode step reads, cache bytes per token, and prefill flops per token."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    HQ, HKV, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    layer_params = (HQ + 2 * HKV) * D * H + H * HQ * D + 2 * I * H + H * I
    weight_bytes = 2 * (n_layers * (layer_params + 2 * H + 2 * D) + V * H + H)
    kv_bytes_per_token = n_layers * 2 * HKV * D * 2
    return layer_params, weight_bytes, kv_bytes_per_token


def time_decode(session, sampling, batch, context, steps, warmup, torch):
    """Device time of exactly ``steps`` decode steps of ``batch`` sequences that end at ``context`` tokens."""
    from starter_b200.engine.graph import GraphDecoder
    cache = session.cache
    decoder = GraphDecoder(session, sampling)
    slots = [cache.alloc() for _ in range(batch)]
    try:
        start = context - steps - warmup
        for s in slots:
            cache.reserve(s, context)
            cache.assume_length(s, start)
        bucket = decoder.bucket(batch)
        cache.flush()
        g = torch.Generator().manual_seed(0)
        tokens = torch.randint(0, session.vocab_size, (batch,), generator=g).tolist()
        bucket.load(slots, tokens, list(range(batch)), 0)
        for _ in range(warmup):
            bucket.graph.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            bucket.graph.replay()
        t1.record()
        torch.cuda.synchronize()
        for s in slots:
            cache.advance_host(s, steps + warmup)
        session.stepper.raise_on_status()
        ms = t0.elapsed_time(t1) / steps
        return ms, start + warmup + steps / 2.0
    finally:
        for s in slots:
            cache.free(s)


def count_step_launches(session, sampling, batch, torch):
    """Kernels of this library in one decode step (counted on an eager pass over the null slot)."""
    from starter_b200.engine.graph import _Bucket
    b = _Bucket(session, batch, sampling)
    before = session.runtime.ops.launches
    b.body()
    torch.cuda.synchronize()
    return session.runtime.ops.launches - before


def time_prefill(session, n_tokens, repeats, torch):
    from starter_b200.engine.step import StepEntry
    cache = session.cache
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, session.vocab_size, (n_tokens,), generator=g).tolist()
    times = []
    for _ in range(repeats + 1):
        slot = cache.alloc()
        try:
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            session.stepper.step([StepEntry(slot, prompt, [n_tokens - 1])])
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1))
        finally:
            cache.free(slot)
    times = sorted(times[1:])  # the first pass warms libraries up
    return times[len(times) // 2]


def time_e2e(engine, batch, context, steps, torch):
    """Decoded tokens per second as a caller of Engine.generate sees them: host token lists in,
    host token lists out, timed on the host from the first step's tokens to the last's."""
    g = torch.Generator().manual_seed(2)
    prompt_len = context - steps - 1
    prompts = [torch.randint(0, engine.session.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch)]
    for _ in engine.generate([p[:64] for p in prompts], 4):  # untimed: captures the decode graph of this batch size
        pass
    it = engine.generate(prompts, steps + 1)
    next(it)
    t0 = time.perf_counter()
    n = 0
    for out in it:
        n += 1
    dt = time.perf_counter() - t0
    assert n == steps
    return batch * steps / dt, prompt_len


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    ap.add_argument("--skip-e2e", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "IshaanBansal2006/starter has no setup.py or pyproject.toml: pip reports 'Directory is not "
                          "installable', so baseline/_ref cannot be made"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library does not run on {args.gpus} GPUs")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from starter_b200.config import config_from_dict
    from starter_b200.engine.engine import Engine
    from starter_b200.engine.session import Session
    from starter_b200.sampling import SamplingParams
    from starter_b200.weights import RandomSource

    peaks, peak_source = load_peaks()
    raw = dict(QWEN3_4B)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    n_layers = cfg.num_hidden_layers
    layer_params, weight_bytes, kv_per_token = model_numbers(cfg, n_layers)
    torch.cuda.set_device(0)
    source = RandomSource(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    T = 2048   # tokens of the prefill that is timed
    session = Session((cfg, source), dtype="bfloat16", max_tokens=max(max_batch * args.context, T), max_seqs=max_batch,
                      max_seq_tokens=max(args.context, T), device="cuda:0", verbose=True)
    for group in session.cache.groups:  # a context of random keys and values stands in for real prompts
        group.k.normal_()
        group.v.normal_()
    sampling = SamplingParams()
    ops = session.runtime.ops

    with ClockSampler() as clocks:
        ms_step, mean_ctx = time_decode(session, sampling, args.batch, args.context, args.steps, args.warmup, torch)
    clock_summary = clocks.summary()
    per_step_launches = count_step_launches(session, sampling, args.batch, torch)
    value = args.batch * 1000.0 / ms_step
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_per_token
    achieved_gbs = step_bytes / (ms_step * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms, _ = time_decode(session, sampling, b, args.context, args.steps, args.warmup, torch)
            points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)

    prefill_ms = time_prefill(session, T, repeats=3, torch=torch)
    D, HQ = cfg.head_dim, cfg.num_attention_heads
    prefill_flops = 2.0 * T * layer_params * n_layers + 4.0 * D * HQ * (T * (T + 1) / 2.0) * n_layers \
        + 2.0 * cfg.vocab_size * cfg.hidden_size
    prefill_frac = prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)

    e2e = None
    if not args.skip_e2e:
        engine = Engine.__new__(Engine)  # the entry point's object around the session that is already loaded
        from starter_b200.engine.generate import Generator
        engine.model_path, engine.session, engine.generator = None, session, Generator(session, use_graphs=True)
        e2e_value, prompt_len = time_e2e(engine, args.batch, args.context, args.steps, torch)
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": round(4.0 * args.batch * (prompt_len + 4) / args.steps, 1),
               "d2h_bytes_per_step": 4 * args.batch}

    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} (Qwen3-4B shape, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0, N(0,0.02)), random token ids, random cache contents",
        "impl": "ours",
        "config": {"model": "Qwen3-4B shape", "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.context,
                   "prefill_tokens": T, "parallelism": "single GPU", "cuda_graphs": True,
                   "l2": "each step reads all weights (larger than L2)", "peaks": peak_source,
                   "decode_weight_copy_gb": round(getattr(ops, "_tiled_bytes", 0) / 1e9, 2)},
        "e2e": e2e,
        "prefill": {"value": round(T * 1000.0 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
        "gpu_launches": per_step_launches * args.steps,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
