"""What bench.py promises without a GPU: one line and exit code 2 for more than one GPU, the
reference arm's `unavailable` line, and a `config` that is flat and short."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = run("--gpus", "2")
    assert r.returncode == 2
    lines = [l for l in (r.stdout + r.stderr).splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_config_record_is_flat_and_short():
    sys.path.insert(0, ROOT)
    import bench

    cfg = bench.config_record(32, 8, "fallback")
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    assert cfg["layers"] == cfg["layers_of_config"] == 32 and cfg["global_batch"] == 8
