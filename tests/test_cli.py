"""The command line, run as a user runs it: ``python -m starter_b200 ...`` in a process of its own."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import TINY, random_tokens, tiny_raw

ROOT = Path(__file__).resolve().parent.parent


def cli(*args, env=None, timeout=600):
    full_env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    full_env.update(env or {})
    return subprocess.run([sys.executable, "-m", "starter_b200", *map(str, args)], capture_output=True, text=True,
                          timeout=timeout, env=full_env, cwd=str(ROOT))


def test_random_weights_writes_a_folder_that_loads(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_raw("B")))
    proc = cli("random-weights", "--config", tmp_path / "config.json", "--seed", 5, "--out", tmp_path / "one")
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "model.safetensors" in proc.stdout and (tmp_path / "one" / "model.safetensors").is_file()
    proc = cli("random-weights", "--config", tmp_path / "config.json", "--seed", 5, "--out", tmp_path / "three", "--shards", 3,
               "--dtype", "float32")
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert len(list((tmp_path / "three").glob("model-*-of-00003.safetensors"))) == 3
    assert json.loads((tmp_path / "three" / "config.json").read_text())["num_key_value_heads"] == 1


def test_generate_without_a_gpu_says_so_in_one_line(tiny_folders):
    """No CUDA device: the library's own message and exit code 1, not a traceback from deep inside torch."""
    proc = cli("generate", "--model", tiny_folders["A"], "--input-ids", "1,2,3", "--max-new-tokens", 2,
               env={"CUDA_VISIBLE_DEVICES": ""})
    assert proc.returncode == 1
    assert "no CUDA device" in proc.stderr and "Traceback" not in proc.stderr


def test_faults_of_the_input_are_messages(tiny_folders, tmp_path):
    proc = cli("random-weights", "--config", tmp_path / "nowhere.json", "--out", tmp_path / "out")
    assert proc.returncode == 1 and "nowhere.json" in proc.stderr and "Traceback" not in proc.stderr
    proc = cli("generate", "--model", tiny_folders["A"], "--max-new-tokens", 2)
    assert proc.returncode == 2 and "--input-ids" in proc.stderr


@pytest.mark.gpu
def test_generate_gives_the_entry_point_s_tokens(tiny_folders, tmp_path):
    from starter_b200.engine import Engine
    prompts = random_tokens(TINY["B"]["vocab_size"], (5, 20, 1, 9, 14), seed=8)
    folder = tiny_folders.for_dtype("B", "float32")            # three shard files, 32-bit weights
    eng = Engine(folder, dtype="float32", max_batch=4, max_context=128)
    want = eng.generate_all(prompts, 6)
    ids = ";".join(",".join(map(str, p)) for p in prompts)

    proc = cli("generate", "--model", folder, "--dtype", "float32", "--input-ids", ids, "--max-new-tokens", 6, "--max-batch", 4,
               "--max-context", 128)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [json.loads(line) for line in proc.stdout.splitlines()] == want   # five requests, two batches one after another

    (tmp_path / "prompts.json").write_text(json.dumps(prompts[:3]))
    proc = cli("generate", "--model", folder, "--dtype", "float32", "--input-file", tmp_path / "prompts.json",
               "--max-new-tokens", 6, "--max-batch", 4, "--max-context", 128, "--stream", "--no-graphs")
    assert proc.returncode == 0, proc.stderr[-2000:]
    steps = [json.loads(line) for line in proc.stdout.splitlines()]
    assert len(steps) == 6 and [[s[b] for s in steps] for b in range(3)] == want[:3]

    stop = want[1][2]
    expect = eng.generate_all(prompts[:3], 6, stop_token_ids=[stop], temperature=0.7, top_k=20, seed=3)
    proc = cli("generate", "--model", folder, "--dtype", "float32", "--input-ids", ";".join(ids.split(";")[:3]),
               "--max-new-tokens", 6, "--max-batch", 4, "--max-context", 128, "--stop-token", stop, "--temperature", 0.7,
               "--top-k", 20, "--seed", 3)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [json.loads(line) for line in proc.stdout.splitlines()] == expect

    proc = cli("generate", "--model", tmp_path / "nowhere", "--input-ids", "1,2", "--max-new-tokens", 2)
    assert proc.returncode == 1 and "config.json" in proc.stderr and "Traceback" not in proc.stderr
    proc = cli("generate", "--model", folder, "--dtype", "float32", "--input-ids", "1,2,9999", "--max-new-tokens", 2)
    assert proc.returncode == 1 and "outside the vocabulary" in proc.stderr and "Traceback" not in proc.stderr
