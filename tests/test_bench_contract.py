"""The reference arm of bench.py runs without a GPU: one JSON line on stdout with the keys the
benchmark contract asks for (the GPU arm prints the same keys plus the roofline and clocks)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, res.stdout
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "compound-optree effective HBM GB/s"
    for key in ("value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["unit"] == "GB/s" and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["steps"] == 1 and line["warmup"] == 1 and line["value"] > 0
    # neon's own NervanaCPU where a neon source tree can be imported, else its numpy restatement
    from oracle import neon_ref
    assert line["cpu_baseline"]["kind"] == ("reference" if neon_ref.find_reference() else "port")
    assert line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["single_process"]["cores"] == 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "model" not in line["config"]


def test_reference_arm_other_ranks_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == "", res.stdout + res.stderr[-1000:]
