"""The benchmark's command-line contract that can be checked without a GPU: the reference arm runs
the CPU oracle on the headline workload and prints exactly one JSON line with the agreed keys, ranks
other than 0 print nothing, and the GPU arm refuses to run without a device instead of falling back."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def run_bench(*arguments, env=None):
    merged = dict(os.environ, **(env or {}))
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *arguments], capture_output=True, text=True,
                          env=merged, timeout=600)


def test_reference_arm_prints_one_line_on_rank_zero_only():
    result = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert result.returncode == 0, result.stderr
    lines = [line for line in result.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "causal_prefill_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["ms_per_step"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] and "sample" in line["cpu_baseline"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]
    sys.path.insert(0, str(ROOT))
    import bench

    assert line["config"] == bench.bench_config(1)  # both arms state one and the same workload
    assert "whole config-2 prefill batch" in line["cpu_baseline"]["sample"]

    other = run_bench("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
                      env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert other.returncode == 0 and other.stdout.strip() == ""


def test_benchmark_inputs_are_the_oracles_inputs():
    """The package's generator (what the GPU arm draws from) and the oracle's give the same bits."""
    import torch

    from oracle import attention as oracle
    from tilecadence_b200.synthetic import seeded_normal

    shapes = ((1, 64, 32, 128), (1, 64, 8, 128), (3, 5))
    for ours, theirs in zip(seeded_normal(1, *shapes), oracle.seeded_normal(1, *shapes)):
        assert ours.dtype == torch.bfloat16 and torch.equal(ours.view(torch.int16), theirs.view(torch.int16))
    half = seeded_normal(0, (4, 4), dtype=torch.float16)[0]
    assert torch.equal(half, oracle.seeded_normal(0, (4, 4), dtype=torch.float16)[0])


def test_gpu_arm_fails_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        return  # on a GPU box the arm runs; the GPU tests cover it
    result = run_bench("--steps", "1", "--warmup", "3", "--no-cpu-baseline")
    assert result.returncode != 0
    assert result.stdout.strip() == ""  # no JSON line is ever printed from a fallback
