"""bench.py's command-line contract, as far as it can be checked without a GPU:
the reference arm (the C port of the reference kernel on the host cores) prints
exactly one JSON line with the agreed keys, and the product arm refuses to run
without a device instead of falling back to the CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, env=e,
                          capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_one_json_line(built):
    r = run(["--impl", "reference", "--steps", "1", "--warmup", "0", "--rows", "1024"],
            env={"OMP_NUM_THREADS": "1"})       # what torch.distributed.run exports
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 0 and d["value"] > 0
    assert d["vs_baseline"] is None and d["dtype"] == "f32" and d["data"] == "synthetic"
    # `config` holds the workload only (it must equal the product arm's); the sample and
    # the thread team are described under cpu_baseline
    assert "MAXANDARGMAX" in d["config"]["workload"] and d["config"]["rows_per_gpu"] == 1024
    assert set(d["config"]) == {"workload", "rows_per_gpu", "bytes_per_step_per_gpu", "l2"}
    assert d["cpu_baseline"]["kind"] == "port" and "all 1024 rows" in d["cpu_baseline"]["sample"]
    # the team is every core the process may use, whatever OMP_NUM_THREADS said
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert d["cpu_baseline"]["omp_num_threads_env"] == "1"
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_under_a_multi_rank_launch_runs_on_rank_zero_only(built):
    r0 = run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", "--rows", "1024"],
             env={"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "2"})
    r1 = run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
             env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert r0.returncode == 0 and r1.returncode == 0
    assert json.loads(r0.stdout.strip())["n_gpus"] == 2
    assert r1.stdout.strip() == ""


def test_product_arm_fails_loudly_without_a_device(built):
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    r = run(["--steps", "1", "--warmup", "1"])
    assert r.returncode != 0
    assert "no CUDA device" in (r.stderr + r.stdout)
    assert r.stdout.strip() == ""                      # nothing that could be taken for a result
