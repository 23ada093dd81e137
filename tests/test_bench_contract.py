"""The CPU (`--impl reference`) arm of bench.py end to end on the small configuration 1:
it needs no GPU, so the shape of its JSON line is checked here."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    j = json.loads(lines[0])
    assert j["impl"] == "reference" and j["metric"] == "dnpeff_nmf_iterations_per_s" and j["unit"] == "iter/s"
    assert j["steps"] == 2 and j["warmup"] == 1 and j["higher_is_better"] is True and j["gpu_launches"] == 0
    assert abs(j["value"] - 1000.0 / j["ms_per_step"]) < 1e-9 * j["value"]
    cb = j["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == j["value"] and cb["extrapolated"] is False
    assert "all 2048 of 2048 rows" in cb["sample"]
    assert j["e2e"] == {"value": j["value"], "unit": "iter/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert j["config"]["workload"].startswith("config1:")


def test_reference_arm_other_ranks_of_a_torchrun_job_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "1",
                          "--gpus", "2", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120,
                         cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
