"""The benchmark's CPU arm (`--impl reference`) runs without a GPU and prints the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-seq", "256", "--workload", "cogvideox"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    for key in ("metric", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "config"):
        assert key in d


def test_reference_arm_runs_the_executed_reference_when_its_copy_is_present():
    """With oracle/_ref/ (made by oracle/make_ref.py from a checkout of the reference) the arm times the
    reference's own proAttention.attn on gloo ranks and adds benchmark configuration 1 at full size."""
    import pytest
    from oracle import ref_runner
    if not ref_runner.available():
        pytest.skip("no copy of the reference under oracle/_ref")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0", "--cpu-seq", "512", "--workload", "cogvideox"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT,
                         env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE")})
    assert out.returncode == 0, out.stderr[-2000:]
    d = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][0])
    assert d["cpu_baseline"]["kind"] == "reference" and d["value"] > 0
    c1 = d["cpu_baseline"]["config1"]
    assert c1["ranks"] == 2 and c1["ms_per_step"] > 0


def test_other_ranks_of_the_reference_arm_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""
