"""The benchmark script's host side: what it refuses, and the arithmetic behind its roofline and prefill figures.

The numbers are worked out again here from the layer formulas of the reference (engine/model.py:102-126 for the
tensors of a layer, OPTIMIZATION_GUIDE.md:104-112 for the cache bytes per token), not from the script's own helpers.
"""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def run_bench(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, env=env,
                          timeout=300)


def test_more_than_one_gpu_is_one_line_and_exit_code_2():
    done = run_bench("--gpus", "2")
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1 and "one GPU" in done.stdout


def test_reference_arm_without_a_device_says_unavailable_and_exits_0():
    done = run_bench("--impl", "reference")
    assert done.returncode == 0
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_reference_arm_names_the_workload_it_cannot_run():
    done = run_bench("--impl", "reference", "--config", "1.7b")
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert done.returncode == 0 and "same length" in line["unavailable"]


def test_own_arm_without_a_device_is_one_line_and_no_traceback():
    done = run_bench()
    assert done.returncode == 1 and done.stdout == ""
    assert "CUDA device" in done.stderr and "Traceback" not in done.stderr


def test_bytes_of_a_decode_step_at_the_headline_sizes():
    raw, workload = bench.CONFIGS["4b"]
    H, I, V, L = 2560, 9728, 151936, 36
    q, kv = 32 * 128, 8 * 128
    matrices = H * (q + 2 * kv) + q * H + 3 * H * I        # q/k/v, output, gate, up, down
    vectors = 2 * H + 2 * 128                              # two norms of the width, q and k norms of a head
    weights = 2 * (L * (matrices + vectors) + V * H + H)   # tied: the table is read once, as the head; the last norm
    params, weight_bytes, per_token = bench.model_numbers(raw, L)
    assert params == matrices and weight_bytes == weights
    assert per_token == 147456                             # 2 (k, v) x 36 layers x 8 heads x 128 x 2 bytes
    assert round(weight_bytes / 1e9, 2) == 8.04


def test_prefill_flops_count_the_causal_half_and_one_head_row():
    raw, _ = bench.CONFIGS["4b"]
    params, _, _ = bench.model_numbers(raw, 36)
    T = 2048
    want = 36 * (2.0 * T * params + 4.0 * 128 * 32 * T * (T + 1) / 2) + 2.0 * 151936 * 2560
    assert bench.prefill_flops(raw, 36, [T]) == pytest.approx(want, rel=1e-12)
    two = bench.prefill_flops(raw, 36, [T, T])
    assert two == pytest.approx(2 * want, rel=1e-12)       # prompts do not see one another


def test_further_prefill_points_are_flat_numbers():
    raw, _ = bench.CONFIGS["4b"]
    points = {}
    bench.prefill_point(points, "prefill_8192", raw, 36, [8192], 80.0, {"bf16_tflops_sustained": 1400.0})
    assert set(points) == {"prefill_8192", "prefill_8192_ms", "prefill_8192_frac_of_sustained"}
    assert all(isinstance(v, float) for v in points.values())
    assert points["prefill_8192"] == 102400.0 and points["prefill_8192_ms"] == 80.0
    flops = bench.prefill_flops(raw, 36, [8192])
    assert points["prefill_8192_frac_of_sustained"] == pytest.approx(flops / 0.080 / 1.4e15, abs=1e-4)


def test_prompt_lengths_of_the_three_workloads():
    for name, (raw, workload) in bench.CONFIGS.items():
        lengths = bench.prompt_lengths(workload)
        assert len(lengths) == workload["batch"]
        if name == "4b":      # decoding ends at the context: prompt + steps + the first token = context
            assert set(lengths) == {workload["context"] - workload["steps"] - 1}
        elif name == "1.7b":
            assert all(64 <= n <= 2048 for n in lengths) and len(set(lengths)) > 1
            assert lengths == bench.prompt_lengths(workload)   # seeded
        else:
            assert set(lengths) == {1024}


def test_peaks_come_from_the_measured_file_or_the_stated_fallback(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.load_peaks() == (bench.FALLBACK_PEAKS, "fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6500.0, "bf16_tflops": 1600.0}))
    peaks, source = bench.load_peaks()
    assert source == "measured" and peaks["hbm_gbs"] == 6500.0 and peaks["bf16_tflops_sustained"] == 1600.0
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.load_peaks()[1] == "fallback"
