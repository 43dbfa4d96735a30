"""CPU checks of the benchmark drivers: argument surface, the reference arm's "unavailable" line,
the clock sampler against a fake ``nvidia-smi`` (reference tests/test_training_matrix_harness.py
tests its drivers the same way: on CPU, without a GPU)."""
import json
import os
import stat
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable_instead_of_crashing_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        import pytest

        pytest.skip("CPU-only check")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_bench_argument_surface():
    sys.path.insert(0, ROOT)
    import importlib

    bench = importlib.import_module("bench")
    argv = sys.argv
    try:
        sys.argv = ["bench.py"]
        a = bench.parse_args()
        assert (a.gpus, a.impl, a.model) == (1, "ours", "llama3-8b") and a.warmup >= 3 and a.steps >= 1
        sys.argv = ["bench.py", "--gpus", "8", "--steps", "5", "--warmup", "3", "--impl", "reference"]
        a = bench.parse_args()
        assert (a.gpus, a.steps, a.warmup, a.impl) == (8, 5, 3, "reference")
    finally:
        sys.argv = argv
    assert bench.METRIC == "fsdp2_full_ft_tokens_per_sec" and bench.BATCH_PER_GPU["llama3-8b"] == 2


def test_clock_sampler_parses_a_fake_nvidia_smi(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "echo '0, 1500, 1965, 950.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "sleep 0.05\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ.get("PATH", ""))
    sys.path.insert(0, ROOT)
    from gefen_x_b200.utils.clocks import ClockSampler

    s = ClockSampler(gpu_index=0)
    s.start()
    import time

    time.sleep(0.6)
    out = s.stop()
    assert out.get("samples", 0) >= 1 and out["sm_mhz"] == 1500.0 and out["sm_max_mhz"] == 1965.0
    assert "sw_power_cap" in out["reasons"] and "hw_slowdown" not in out["reasons"]
