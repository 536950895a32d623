"""The JSON line ``bench.py`` prints: the keys a harness reads, on both arms."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def run_bench(*args, timeout=900):
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=str(ROOT),
                          timeout=timeout)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [line for line in proc.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, "exactly one JSON line on stdout"
    return json.loads(lines[0])


def test_reference_arm_prints_the_same_metric_on_the_cpu(built_libs):
    """``--impl reference`` times the CPU restatement of the reference's torch path: no GPU needed."""
    line = run_bench("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert line["impl"] == "reference" and line["metric"] == "decode_attn_kv_read_gbs" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["config"]["workload"] == "qwen2.5-coder-3b-b64"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["gpu_launches"] == 0


@pytest.mark.gpu
def test_own_arm_prints_the_contract_keys(built_libs):
    line = run_bench("--steps", "10", "--warmup", "3", "--repeats", "2", "--no-per-config", "--with-producer")
    assert "impl" not in line or line["impl"] != "reference"
    assert line["metric"] == "decode_attn_kv_read_gbs" and line["unit"] == "GB/s" and line["n_gpus"] == 1
    assert line["steps"] == 10 and line["warmup"] == 3 and line["scaling"] == "weak" and line["data"] == "synthetic"
    assert line["correct"] is True and line["max_abs_error"] < 0.05
    assert line["value"] > 0 and abs(line["ms_per_step"] * 1e3 - line["us_per_layer_step"]) < 1e-2
    roof = line["roofline"]
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s" and 0 < roof["frac"] < 1.5
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-3
    assert roof["traffic"] is None or roof["traffic"] > 0
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["value"] < line["value"]  # copies in and out every step
    assert line["gpu_launches"] >= 10 and line["cpu_baseline"]["kind"] == "port"
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(line["clocks"])
    both = line["with_producer"]
    assert both["status"] == 0 and both["us_per_layer_step"] > both["producer_alone_us"] > 0
