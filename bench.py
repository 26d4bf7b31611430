#!/usr/bin/env python3
"""Decode and prefill throughput of Qwen3-shaped models on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 4b|1.7b|8b] [--check]

The default run (``--config 4b``) is the headline: a step is one decode step of
a batch of 8 sequences at a context of 4,096 tokens.  Prints one JSON line:
``value`` = decoded tokens per second timed on the device over exactly K
graph-replayed steps; ``e2e`` = the same through ``Engine.generate`` with host
token lists in and out; ``prefill`` = one prompt of 2,048 tokens; ``roofline``
= bytes the decode step has to read (every weight once, the cache of the live
sequences) over its time, against the measured copy bandwidth; ``points`` =
decode at batch 1 and 64, at context 2,048, and averaged over the sweep from
2,048 to 4,096 positions.

``--config 1.7b``: 16 sequences with prompt lengths drawn uniformly from
[64, 2048] (seeded), 256 decode steps.  ``--config 8b``: an untied head, 32
prompts of 1,024 tokens, 512 decode steps, a cache of 8,192 tokens per
sequence.  ``--check`` decodes nothing for speed: it runs the same layer
sizes with 2 layers in bfloat16 and in true 32-bit and prints how far the
logits are apart.

``--impl reference`` drives the unmodified engine of IshaanBansal2006/starter
from ``baseline/_ref/engine`` (a plain copy of its ``engine/`` folder) through
its own ``Engine(model_path).generate(input_ids, max_new_tokens)``.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_COMMON = dict(architectures=["Qwen3ForCausalLM"], num_key_value_heads=8, head_dim=128, vocab_size=151936,
               rms_norm_eps=1e-6)
CONFIGS = {
    # name: (config.json, workload)
    "4b": (dict(_COMMON, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32,
                rope_theta=5000000.0, tie_word_embeddings=True),
           dict(model="Qwen3-4B shape", batch=8, context=4096, steps=256, prompts="decode ends at the context")),
    "1.7b": (dict(_COMMON, hidden_size=2048, intermediate_size=6144, num_hidden_layers=28, num_attention_heads=16,
                  rope_theta=1000000.0, tie_word_embeddings=True),
             dict(model="Qwen3-1.7B shape", batch=16, context=2048 + 256, steps=256, prompts="uniform[64,2048]")),
    "8b": (dict(_COMMON, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                rope_theta=1000000.0, tie_word_embeddings=False),
           dict(model="Qwen3-8B shape", batch=32, context=8192, steps=512, prompts="1024 each")),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PREFILL_TOKENS = 2048
LONG_PREFILL_TOKENS = 8192   # a second prefill point, where attention is a third of the work


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


def model_numbers(raw, n_layers):
    """Parameters of one layer's matrices, bytes of the weights a decode step reads (the embedding
    table only where it is the output head as well), and cache bytes per token."""
    H, I, V = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    HQ, HKV, D = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    layer_params = (HQ + 2 * HKV) * D * H + H * HQ * D + 2 * I * H + H * I
    weight_bytes = 2 * (n_layers * (layer_params + 2 * H + 2 * D) + V * H + H)
    kv_bytes_per_token = n_layers * 2 * HKV * D * 2
    return layer_params, weight_bytes, kv_bytes_per_token


def prefill_flops(raw, n_layers, lengths):
    """Flops of a prefill of prompts of these lengths with logits at each prompt's last token."""
    layer_params, _, _ = model_numbers(raw, n_layers)
    D, HQ = raw["head_dim"], raw["num_attention_heads"]
    linear = 2.0 * sum(lengths) * layer_params * n_layers
    attention = sum(4.0 * D * HQ * (t * (t + 1) / 2.0) for t in lengths) * n_layers
    return linear + attention + 2.0 * len(lengths) * raw["vocab_size"] * raw["hidden_size"]


def prefill_point(points, name, raw, n_layers, lengths, ms, peaks):
    """A further prefill measurement as flat numbers: tokens a second under ``name``, its time under
    ``name_ms`` and its flops / time / the sustained bf16 peak under ``name_frac_of_sustained``."""
    points[name] = round(sum(lengths) * 1000.0 / ms, 1)
    points[name + "_ms"] = round(ms, 3)
    points[name + "_frac_of_sustained"] = round(
        prefill_flops(raw, n_layers, lengths) / (ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)


def prompt_lengths(workload, seed=4):
    import torch
    B = workload["batch"]
    if workload["prompts"] == "uniform[64,2048]":
        g = torch.Generator().manual_seed(seed)
        return torch.randint(64, 2049, (B,), generator=g).tolist()
    if workload["prompts"] == "1024 each":
        return [1024] * B
    return [workload["context"] - workload["steps"] - 1] * B


# ---- this library ---------------------------------------------------------------------------------

def time_decode(session, sampling, starts, steps, warmup, torch):
    """Device time per step of exactly ``steps`` decode steps of len(starts) sequences; sequence b
    holds starts[b] tokens when the warm-up begins.  Returns (ms per step, mean context while timed)."""
    from starter_b200.engine.graph import GraphDecoder
    cache = session.cache
    decoder = GraphDecoder(session, sampling)
    batch = len(starts)
    slots = [cache.alloc() for _ in range(batch)]
    try:
        for s, start in zip(slots, starts):
            cache.reserve(s, start + warmup + steps)
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
        return ms, sum(starts) / batch + warmup + steps / 2.0
    finally:
        for s in slots:
            cache.free(s)


def count_step_launches(session, sampling, batch, torch):
    """Kernels of this library in one decode step (counted on an eager pass over the null slot)."""
    from starter_b200.engine.graph import GraphDecoder
    b = GraphDecoder(session, sampling).new_bucket(batch)
    before = session.runtime.ops.launches
    b.body()
    torch.cuda.synchronize()
    return session.runtime.ops.launches - before


def time_prefill(session, lengths, repeats, torch):
    """Median device time of one step that runs prompts of these lengths, logits at each one's end."""
    from starter_b200.engine.step import StepEntry
    cache = session.cache
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, session.vocab_size, (n,), generator=g).tolist() for n in lengths]
    times = []
    for _ in range(repeats + 1):
        slots = [cache.alloc() for _ in prompts]
        try:
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            session.stepper.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1))
        finally:
            for s in slots:
                cache.free(s)
    times = sorted(times[1:])  # the first pass warms libraries up
    return times[len(times) // 2]


def time_e2e(engine, lengths, steps, torch):
    """Decoded tokens per second as a caller of Engine.generate sees them: host token lists in, host
    token lists out.  Returns (tokens/s from the first step's tokens to the last's, seconds from the
    call to the first step's tokens: upload of the prompts, their prefill, the first selection)."""
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, engine.session.vocab_size, (n,), generator=g).tolist() for n in lengths]
    for _ in engine.generate(prompts, 4):  # untimed, the same prompts: the library's first call at these shapes and
        pass                               # the capture of this batch size's decode graph (the reference arm does the same)
    torch.cuda.synchronize()
    t_call = time.perf_counter()
    it = engine.generate(prompts, steps + 1)
    next(it)
    t0 = time.perf_counter()
    n = 0
    for out in it:
        n += 1
    dt = time.perf_counter() - t0
    assert n == steps
    return len(lengths) * steps / dt, t0 - t_call


def run_ours(args, raw, workload) -> int:
    import torch
    from starter_b200.config import config_from_dict
    from starter_b200.engine.engine import Engine
    from starter_b200.engine.session import Session
    from starter_b200.sampling import SamplingParams
    from starter_b200.weights import RandomSource

    peaks, peak_source = load_peaks()
    raw = dict(raw)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    n_layers = cfg.num_hidden_layers
    layer_params, weight_bytes, kv_per_token = model_numbers(raw, n_layers)
    batch, context, steps, warmup = args.batch, args.context, args.steps, args.warmup
    torch.cuda.set_device(0)
    source = RandomSource(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    headline = args.config == "4b"
    max_batch = max(batch, 64 if headline and not args.skip_points else 1)
    lengths = prompt_lengths(dict(workload, batch=batch, context=context, steps=steps))
    long_prefill = LONG_PREFILL_TOKENS if headline and not args.skip_points else 0
    session = Session((cfg, source), dtype="bfloat16", max_tokens=max(max_batch * context, PREFILL_TOKENS, long_prefill),
                      max_seqs=max_batch, max_seq_tokens=max(context, PREFILL_TOKENS, long_prefill), device="cuda:0",
                      verbose=True)
    for group in session.cache.groups:  # a context of random keys and values stands in for real prompts
        group.k.normal_()
        group.v.normal_()
    sampling = SamplingParams()
    ops = session.runtime.ops

    # The step that is timed: the workload's own decode steps.  4b: the last `steps` positions before the
    # context's end; the others: the `steps` positions after the prompts.
    starts = [context - steps - warmup] * batch if headline else [n - warmup for n in lengths]
    with ClockSampler() as clocks:
        ms_step, mean_ctx = time_decode(session, sampling, starts, steps, warmup, torch)
    clock_summary = clocks.summary()
    per_step_launches = count_step_launches(session, sampling, batch, torch)
    value = batch * 1000.0 / ms_step
    step_bytes = weight_bytes + batch * mean_ctx * kv_per_token
    achieved_gbs = step_bytes / (ms_step * 1e-3) / 1e9

    def rate(b, ms):
        return round(b * 1000.0 / ms, 1)

    points = {}
    if not args.skip_points:
        if headline:
            for b in (1, 64):
                ms, _ = time_decode(session, sampling, [context - steps - warmup] * b, steps, warmup, torch)
                points[f"decode_b{b}"] = rate(b, ms)
            half = context // 2
            for b in (1, batch, 64):
                ms, _ = time_decode(session, sampling, [half - steps // 2 - warmup] * b, steps, warmup, torch)
                points[f"decode_b{b}_ctx{half}"] = rate(b, ms)
                ms, _ = time_decode(session, sampling, [half - warmup] * b, context - half, warmup, torch)
                points[f"decode_b{b}_sweep_{half}_{context}"] = rate(b, ms)
        else:
            ms, ctx = time_decode(session, sampling, [context - steps - warmup] * batch, steps, warmup, torch)
            points[f"decode_b{batch}_ctx{context}"] = rate(batch, ms)
            points[f"decode_b{batch}_ctx{context}_hbm_frac"] = round(
                (weight_bytes + batch * ctx * kv_per_token) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)

    prefill_ms = time_prefill(session, [PREFILL_TOKENS], repeats=3, torch=torch)
    prefill_frac = prefill_flops(raw, n_layers, [PREFILL_TOKENS]) / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    prefill = {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4)}
    if long_prefill:
        ms = time_prefill(session, [long_prefill], repeats=2, torch=torch)
        prefill_point(points, f"prefill_{long_prefill}", raw, n_layers, [long_prefill], ms, peaks)
    if not headline:  # the workload's own prompts, all in one step
        ms = time_prefill(session, lengths, repeats=2, torch=torch)
        prefill_point(points, "prefill_workload", raw, n_layers, lengths, ms, peaks)
        points["prefill_workload_tokens"] = sum(lengths)

    e2e = None
    if not args.skip_e2e:
        engine = Engine.from_session(session)
        e2e_value, first_s = time_e2e(engine, lengths, steps, torch)
        # Timed from the first step's tokens to the last's: inside that region a step's input (the token
        # chosen one step before) is already on the device, so nothing goes up; its tokens come down.
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
               "d2h_bytes_per_step": 4 * batch, "first_tokens_s": round(first_s, 4),
               "prompt_upload_bytes": 4 * (sum(lengths) + 4 * batch),
               "region": "decode steps; prompt upload and prefill are in first_tokens_s"}

    line = {
        "metric": f"decode tok/s at batch {batch}, context {round(mean_ctx + steps / 2.0)} ({workload['model']}, bf16, "
                  "random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0, N(0,0.02)), random token ids, random cache contents",
        "impl": "ours",
        "config": {"model": workload["model"], "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": batch, "seq_len": context,
                   "prompts": workload["prompts"], "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "each step reads all weights (larger than L2)", "peaks": peak_source,
                   "decode_weight_copy_gb": round(getattr(ops, "_tiled_bytes", 0) / 1e9, 2)},
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
        "gpu_launches": per_step_launches * steps,
    }
    print(json.dumps(line))
    return 0


def run_check(args, raw, workload) -> int:
    """The 32-bit check path at the benchmark's layer sizes: 2 layers, the shape rules as they are."""
    import torch
    from starter_b200.config import config_from_dict
    from starter_b200.engine.check import compare_dtypes
    cfg = config_from_dict(dict(raw, num_hidden_layers=args.layers or 2))
    report = compare_dtypes(cfg, seed=0, prompt_lengths=(300, 2048), decode_batches=(1, 8, 64), decode_steps=6,
                            device="cuda:0", verbose=True)
    report.update(impl="ours", check="bfloat16 engine against the float32 engine, same weights",
                  config={"model": workload["model"], "layers": cfg.num_hidden_layers,
                          "layers_of_model": raw["num_hidden_layers"]})
    print(json.dumps(report))
    return 0 if report["within_tolerance"] else 1


# ---- the reference --------------------------------------------------------------------------------

def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def run_reference(args, raw, workload) -> int:
    """Drive the reference's own Engine from baseline/_ref/engine, unmodified.

    Its switches (engine/engine.py:437-454): ENGINE_RECYCLE=0 turns its speculative decoding off (not
    part of this comparison: both arms decode one token per sequence per step), ENGINE_SELF_CHECK=0
    skips its comparison with the Transformers library.  Every other switch keeps its default, so its
    start-up pickers choose its kernels by timing, as in a stock run.
    """
    ref_engine = os.path.join(ROOT, "baseline", "_ref", "engine")
    if not os.path.isfile(os.path.join(ref_engine, "engine.py")):
        return _unavailable("baseline/_ref/engine/engine.py is absent: copy the reference's engine/ folder there")
    if workload["prompts"] == "uniform[64,2048]":
        return _unavailable("the reference rejects prompts of unequal length (engine/engine.py:584-585: "
                            "'all prompts in a batch must have the same length'), which this workload is made of")
    os.environ.setdefault("ENGINE_RECYCLE", "0")
    os.environ.setdefault("ENGINE_SELF_CHECK", "0")
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device: the reference's kernels need one")
        from starter_b200.config import config_from_dict
        from starter_b200.weights import write_model_folder
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"set-up failed: {exc!r}")

    peaks, peak_source = load_peaks()
    raw = dict(raw)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    n_layers = raw["num_hidden_layers"]
    _, weight_bytes, kv_per_token = model_numbers(raw, n_layers)
    batch, context, steps, warmup = args.batch, args.context, args.steps, args.warmup
    headline = args.config == "4b"
    lengths = prompt_lengths(dict(workload, batch=batch, context=context, steps=steps))
    T = lengths[0]
    folder = tempfile.mkdtemp(prefix="starter_ref_model_")
    try:
        # Data only: the same kind of folder the reference is given in a stock run, with seeded random weights.
        write_model_folder(config_from_dict(raw), 0, folder, device="cuda:0")
        torch.cuda.empty_cache()
        sys.path.insert(0, ref_engine)
        try:
            from engine import Engine  # the reference's engine/engine.py
        except Exception as exc:  # noqa: BLE001
            return _unavailable(f"importing the reference's engine failed: {exc!r}")

        def fresh_engine():
            # A new engine per measurement: its pickers share one 60 s budget that starts with the object.
            gc.collect()
            torch.cuda.empty_cache()
            eng = Engine(folder)
            if eng.fallback is not None or eng.model is None:
                raise RuntimeError("the reference fell back to its Transformers baseline (its model did not load)")
            return eng

        def generate_timed(eng, B, T, n_new, seed):
            """(tokens/s between the first and the last yield, seconds to the first yield) of one call."""
            g = torch.Generator().manual_seed(seed)
            ids = torch.randint(0, raw["vocab_size"], (B, T), generator=g).tolist()
            for _ in eng.generate(ids, n_new):  # untimed: builds the plan, runs the pickers, captures the graphs
                pass
            if eng.fallback is not None:
                raise RuntimeError("the reference fell back to its Transformers baseline during generate")
            torch.cuda.synchronize()
            t_call = time.perf_counter()
            it = eng.generate(ids, n_new)
            next(it)
            t0 = time.perf_counter()
            n = sum(1 for _ in it)
            dt = time.perf_counter() - t0
            assert n == n_new - 1
            return B * n / dt, t0 - t_call

        def replay_decode(eng, key, start, n_steps):
            """Device time per step of its captured decode graph, the sequences set to ``start`` tokens."""
            plan = eng.plans[key]
            if plan.g_decode is None:
                raise RuntimeError("the reference did not capture its decode graph")
            if start + warmup + n_steps > plan.plan.cap:
                raise RuntimeError(f"its plan holds {plan.plan.cap} tokens per sequence")
            plan.plan.pos.fill_(start)
            for _ in range(warmup):
                plan._step_decode()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(n_steps):
                plan._step_decode()
            t1.record()
            torch.cuda.synchronize()
            return t0.elapsed_time(t1) / n_steps

        try:
            eng = fresh_engine()
            with ClockSampler() as clocks:
                e2e_value, first_s = generate_timed(eng, batch, T, steps + 1, seed=2)
                start = (context - steps - warmup) if headline else T - warmup
                ms_step = replay_decode(eng, (batch, T), start, steps)
            clock_summary = clocks.summary()
            mean_ctx = start + warmup + steps / 2.0
            points = {}
            if not headline:
                points["prefill_workload"] = {"tokens": batch * T, "first_tokens_s": round(first_s, 4)}
            if headline and not args.skip_points:
                for b in (1, 64):
                    del eng
                    eng = fresh_engine()
                    # a short prompt, a plan that holds the whole context; positions are then set on its plan
                    short, n_new = 64, context - 64
                    g = torch.Generator().manual_seed(3)
                    ids = torch.randint(0, raw["vocab_size"], (b, short), generator=g).tolist()
                    it = eng.generate(ids, n_new)
                    for _ in range(4):
                        next(it)
                    it.close()
                    torch.cuda.synchronize()
                    ms = replay_decode(eng, (b, short), context - steps - warmup, steps)
                    points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
                    half = context // 2   # the same plan at half the context, as this library's arm measures it
                    ms = replay_decode(eng, (b, short), half - steps // 2 - warmup, steps)
                    points[f"decode_b{b}_ctx{half}"] = round(b * 1000.0 / ms, 1)
            del eng

            def prefill_ms_of(n_tokens, repeats):
                eng = fresh_engine()
                g = torch.Generator().manual_seed(1)
                ids = torch.randint(0, raw["vocab_size"], (1, n_tokens), generator=g).tolist()
                list(eng.generate(ids, 1))
                plan = eng.plans[(1, n_tokens)]
                times = []
                for _ in range(repeats + 1):
                    torch.cuda.synchronize()
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0.record()
                    plan._step_prefill()
                    t1.record()
                    torch.cuda.synchronize()
                    times.append(t0.elapsed_time(t1))
                times = sorted(times[1:])
                return times[len(times) // 2]

            prefill_ms = prefill_ms_of(PREFILL_TOKENS, 3)
            if headline and not args.skip_points:
                ms = prefill_ms_of(LONG_PREFILL_TOKENS, 2)
                prefill_point(points, f"prefill_{LONG_PREFILL_TOKENS}", raw, n_layers, [LONG_PREFILL_TOKENS], ms, peaks)
        except Exception as exc:  # noqa: BLE001
            return _unavailable(f"the reference's engine failed on this box: {exc!r}")
    finally:
        shutil.rmtree(folder, ignore_errors=True)

    step_bytes = weight_bytes + batch * mean_ctx * kv_per_token
    achieved_gbs = step_bytes / (ms_step * 1e-3) / 1e9
    prefill_frac = prefill_flops(raw, n_layers, [PREFILL_TOKENS]) / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    line = {
        "metric": f"decode tok/s at batch {batch}, context {round(mean_ctx + steps / 2.0)} ({workload['model']}, bf16, "
                  "random weights)",
        "value": round(batch * 1000.0 / ms_step, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0, N(0,0.02)), random token ids",
        "impl": "reference",
        "config": {"model": workload["model"], "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
                   "tied": raw["tie_word_embeddings"], "global_batch": batch, "seq_len": context,
                   "prompts": workload["prompts"], "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "each step reads all weights (larger than L2)", "peaks": peak_source,
                   "switches": f"ENGINE_RECYCLE={os.environ['ENGINE_RECYCLE']} ENGINE_SELF_CHECK={os.environ['ENGINE_SELF_CHECK']}",
                   "value_is": "its captured decode graph replayed with plan.pos set; e2e is Engine.generate alone"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 8 * batch, "first_tokens_s": round(first_s, 4),
                "region": "decode steps; prompt upload and prefill are in first_tokens_s"},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps that are timed (default: the workload's)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="4b", choices=sorted(CONFIGS))
    ap.add_argument("--check", action="store_true", help="compare bfloat16 with 32-bit logits at these layer sizes")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--context", type=int, default=0)
    ap.add_argument("--skip-points", action="store_true", help="leave out the further decode points")
    ap.add_argument("--skip-e2e", action="store_true")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library does not run on {args.gpus} GPUs")
        return 2
    raw, workload = CONFIGS[args.config]
    args.batch = args.batch or workload["batch"]
    args.context = args.context or workload["context"]
    args.steps = args.steps or workload["steps"]
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args, raw, workload)
    import torch
    if not torch.cuda.is_available():   # no fallback: the library's kernels are the thing measured
        print("bench.py needs a CUDA device (sm_100a) and found none", file=sys.stderr)
        return 1
    if args.check:
        return run_check(args, raw, workload)
    return run_ours(args, raw, workload)


if __name__ == "__main__":
    sys.exit(main())
