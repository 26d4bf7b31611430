"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives the same model, step function, cache and kernels that generation uses.
The reference's nearest thing is its teacher-forced self-check
(engine/engine.py:474-516), which pushes given tokens through ``prefill`` and
``decode`` and compares logits.

Input, one JSON object a line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: each request's next tokens and the places among them whose logits
are wanted; a request that appears for the first time takes a cache slot.
``end``: requests that are finished after this step; their slots and pages
are given back.  For a step with wanted places, ``<out>/<step>.f32`` receives
the logits [wanted, vocab] as little-endian 32-bit floats, in the order of the
entries and of ``want``.  After every step a line ``done <step>`` is printed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from ..cache.cache import PAGE
from .session import Session
from .step import StepEntry


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                   help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help=f"the most tokens live requests hold at any time, each rounded up to {PAGE}; sizes the cache")
    return p


def run(args, stdin=None, stdout=None) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    session = Session(args.model, dtype=args.dtype, max_tokens=args.max_tokens)
    slots = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for e in record.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = session.cache.alloc()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        logits = session.stepper.step(entries) if entries else None
        session.stepper.raise_on_status()
        if logits is not None:
            data = logits.float().cpu().contiguous().numpy().astype("<f4", copy=False)
            data.tofile(out_dir / f"{step}.f32")
        for rid in record.get("end", []):
            if rid in slots:
                session.cache.free(slots.pop(rid))
        stdout.write(f"done {step}\n")
        stdout.flush()
    return 0


def main(argv=None) -> int:
    return run(build_parser().parse_args(argv))
