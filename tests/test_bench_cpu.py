"""CPU: what bench.py can do without a GPU.  The reference arm falls back to the float64 CPU port when no GPU (or no built
reference extension) is there and must still print ONE JSON line with the contract's keys; this library's own arm must refuse
to run, loudly, because the CUDA path has no CPU fallback."""
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), *args], capture_output=True, text=True, env=env, cwd=REPO, timeout=600)


def test_reference_arm_on_cpu_prints_one_json_line():
    p = _run("--impl", "reference", "--reference-kind", "cpu", "--n-gaussians", "2000", "--steps", "1", "--warmup", "0", "--cpu-sample-views", "1")
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "frames/s" and d["unit"] == "frames/s" and d["higher_is_better"] is True
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "VARIANT" in d["config"]["workload"]          # a reduced scene never carries the benchmark's name


def test_own_arm_refuses_to_run_without_a_gpu():
    p = _run("--n-gaussians", "2000", "--steps", "1", "--warmup", "0")
    assert p.returncode != 0
    assert "no CPU fallback" in (p.stderr + p.stdout)
