"""The reference arm of bench.py runs on the host cores and needs no GPU: its JSON line must carry
the keys the measurement contract names."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    result = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload",
                             "gemm_bias_1024", "--steps", "1", "--warmup", "1"],
                            capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert result.returncode == 0, result.stderr[-2000:]
    lines = [line for line in result.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "bf16_gemm_epilogue_tflops"
    assert line["unit"] == "TFLOP/s" and line["higher_is_better"] is True and line["value"] > 0
    baseline = line["cpu_baseline"]
    assert baseline["kind"] in ("port", "reference") and baseline["cores"] >= 1 and baseline["sample"]
    assert baseline["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("gemm_bias")
