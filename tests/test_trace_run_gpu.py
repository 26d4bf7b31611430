"""bin/trace_run as a user drives it: steps on standard input, logits in files."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import TINY, random_tokens
from helpers import TOLERANCE, plain_logits

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(folder, dtype, steps, out_dir, max_tokens):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    return proc


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "W"])
def test_replay_in_three_cuttings(tiny_folders, tmp_path, name, dtype):
    folder, vocab = tiny_folders.for_dtype(name, dtype), TINY[name]["vocab_size"]   # float32: 32-bit weights in three shards
    seqs = random_tokens(vocab, (40, 130, 7, 64), seed=21)
    ref = plain_logits(folder, seqs, dtype)
    scale = max(float(r.abs().max()) for r in ref)
    tol = TOLERANCE[dtype] * scale

    # 1. each request alone and whole; its slot is given back and used by the next
    steps = [{"step": i, "entries": [{"id": f"r{i}", "tokens": s, "want": list(range(len(s)))}], "end": [f"r{i}"]}
             for i, s in enumerate(seqs)]
    replay(folder, dtype, steps, tmp_path / "whole", 192)
    for i, r in enumerate(ref):
        assert float((read(tmp_path / "whole", i, vocab) - r).abs().max()) <= tol, f"whole, request {i}"

    # 2. the last 32 tokens one by one
    steps, n = [], 0
    for i, s in enumerate(seqs):
        cut = max(1, len(s) - 32)
        steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": s[:cut], "want": [cut - 1]}], "end": []})
        n += 1
        for t in range(cut, len(s)):
            steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": [s[t]], "want": [0]}],
                          "end": [f"r{i}"] if t == len(s) - 1 else []})
            n += 1
        if cut == len(s):
            steps[-1]["end"] = [f"r{i}"]
    replay(folder, dtype, steps, tmp_path / "tail", 192)
    n = 0
    for i, (s, r) in enumerate(zip(seqs, ref)):
        cut = max(1, len(s) - 32)
        for t in range(cut - 1, len(s)):
            got = read(tmp_path / "tail", n, vocab)
            assert got.shape[0] == 1 and float((got[0] - r[t]).abs().max()) <= tol, f"tail, request {i}, position {t}"
            n += 1

    # 3. two batches of unequal lengths, one after another; the shorter request ends earlier;
    #    a step with nothing wanted writes no file
    steps, n, expect = [], 0, []
    for batch in ([0, 1, 2], [3, 2]):
        cut = {i: max(1, len(seqs[i]) // 2) for i in batch}
        steps.append({"step": n, "entries": [{"id": f"b{n}-{i}", "tokens": seqs[i][:cut[i]], "want": []} for i in batch], "end": []})
        ids = {i: f"b{n}-{i}" for i in batch}
        expect.append(None)
        n += 1
        t = 0
        while True:
            live = [i for i in batch if cut[i] + t < len(seqs[i])]
            if not live:
                break
            steps.append({"step": n, "entries": [{"id": ids[i], "tokens": [seqs[i][cut[i] + t]], "want": [0]} for i in live],
                          "end": [ids[i] for i in live if cut[i] + t + 1 == len(seqs[i])]})
            expect.append([(i, cut[i] + t) for i in live])
            n += 1
            t += 1
    replay(folder, dtype, steps, tmp_path / "ragged", 64 * 5)
    for step, exp in enumerate(expect):
        if exp is None:
            assert not (tmp_path / "ragged" / f"{step}.f32").exists()
            continue
        got = read(tmp_path / "ragged", step, vocab)
        assert got.shape[0] == len(exp)
        for row, (i, pos) in enumerate(exp):
            assert float((got[row] - ref[i][pos]).abs().max()) <= tol, f"ragged, step {step}, request {i}, position {pos}"


def test_too_small_a_cache_is_an_error(tiny_folders, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": list(range(130)), "want": [0]}], "end": []}]
    text = json.dumps(steps[0]) + "\n"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tiny_folders["A"]), "--dtype",
                           "float32", "--out", str(tmp_path), "--max-tokens", "128"], input=text, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode != 0 and "cache" in proc.stderr
