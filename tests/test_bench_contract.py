"""The reference arm of bench.py needs no GPU: its JSON line carries the keys
the measurement contract names, on the smallest workload."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         cwd=ROOT, timeout=600, env={**os.environ, **(env or {})})
    assert out.returncode == 0, out.stderr[-2000:]
    return [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]


def test_reference_arm_line():
    (line,) = _run("--impl", "reference", "--workload", "cora", "--steps", "2", "--warmup", "1")
    assert line["impl"] == "reference" and line["unit"] == "ms/epoch" and line["higher_is_better"] is False
    assert line["value"] > 0 and line["ms_per_step"] == line["value"] and line["n_gpus"] == 1
    assert line["vs_baseline"] is None and line["data"] == "synthetic" and line["dtype"] == "f32"
    assert "workload" in line["config"] and "model" not in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "ms/epoch", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_runs_on_rank_zero_only():
    assert _run("--impl", "reference", "--workload", "cora", "--steps", "1", "--warmup", "1",
                env={"RANK": "1", "WORLD_SIZE": "2"}) == []
    (line,) = _run("--impl", "reference", "--workload", "rmat24")
    assert line == {"impl": "reference", "unavailable": line["unavailable"]} and "GPU" in line["unavailable"]


def test_small_workloads_are_timed_behind_an_l2_flush():
    """A workload whose forward inputs would stay in the 126 MB L2 from one step to the next is timed
    behind a flush; the large ones read more than L2 holds.  Both arms print the same wording."""
    import bench
    note, fits = bench.l2_policy(2708, 13264, [16, 22])
    assert fits and "flushed" in note
    note, fits = bench.l2_policy(2_097_152, 35_651_584, [16, 22])
    assert not fits and "exceed" in note
