"""bench.py's reference arm runs on the host alone: one JSON line with the contract's keys, the CPU
oracle as the thing timed, no GPU launches."""
import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    j = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in j, key
    assert j["impl"] == "reference" and j["unit"] == "GB/s" and j["value"] > 0 and j["steps"] == 2
    assert j["gpu_launches"] == 0 and j["vs_baseline"] is None
    assert "workload" in j["config"] and "model" not in j["config"]
    assert j["cpu_baseline"]["kind"] == "port" and j["cpu_baseline"]["cores"] >= 1
    assert j["e2e"] == {"value": j["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_algorithmic_bytes_formula():
    """bytes(M, N, K) = N*K/2 + N*K/16 + 2*M*K + 2*M*N + 4, the figure the roofline uses."""
    sys.path.insert(0, str(ROOT))
    import bench
    assert bench.algo_bytes(1, 4096, 4096) == 9_453_572
    assert bench.algo_bytes(1, 28672, 4096) == 66_125_828
    assert bench.algo_bytes(1, 4096, 14336) == 33_067_012
    assert bench.algo_bytes(64, 4096, 4096) == 4096 * 4096 * 9 // 16 + 2 * 64 * 8192 + 4
