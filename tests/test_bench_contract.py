"""The benchmark's command-line contract, as far as it can be checked without a
GPU: the reference arm (CPU oracle on a bounded sample) prints one JSON line
with the agreed keys, the optional arm for the reference's own CUDA kernels
reports `unavailable` instead of failing, and the main arm refuses to run
without a CUDA device (there is no CPU fallback to time)."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*argv, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *argv], capture_output=True, text=True,
                          cwd=ROOT, env=e, timeout=600)


def test_reference_arm_line():
    r = run("--impl", "reference", "--steps", "1", "--warmup", "0", "--op", "mamba2")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["vs_baseline"] is None
    # the reference's own jit.naive when an install of it is present beside the repository, else the port
    have_ref = os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "flex_rnn"))
    assert line["cpu_baseline"]["kind"] == ("reference" if have_ref else "port") and line["cpu_baseline"]["cores"] >= 1
    assert "B=1,H=32" in line["cpu_baseline"]["sample"]          # one batch element, all heads: the cpu_baseline sample
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0


def test_other_ranks_of_the_reference_arm_do_nothing():
    r = run("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_reference_cuda_arm_reports_unavailable_without_a_gpu():
    if torch.cuda.is_available():
        return
    r = run("--impl", "reference_cuda", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference_cuda" and "unavailable" in line


def test_gpu_count_must_match_the_launch():
    """--gpus N without N launched processes is refused (it would silently time one GPU)."""
    r = run("--gpus", "8", "--steps", "1", "--warmup", "1")
    assert r.returncode != 0 and "torch.distributed.run" in r.stderr


def test_main_arm_needs_a_gpu():
    if torch.cuda.is_available():
        return
    r = run("--steps", "1", "--warmup", "1")
    assert r.returncode != 0 and "CUDA device" in r.stderr
