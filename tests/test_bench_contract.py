"""``bench.py`` on a machine without a GPU: the reference arm prints one JSON line with the
contract's keys; the GPU arm refuses to run (there is no CPU path to fall back to)."""

from __future__ import annotations

import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _run(*args, env=None):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_the_contract_line():
    done = _run("--impl", "reference", "--workload", "cfg0_cpu_fp32", "--steps", "2",
                "--warmup", "1")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "MSDA fwd+bwd queries/sec"
    assert line["unit"] == "queries/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["vs_baseline"] is None
    assert line["steps"] == 2 and line["warmup"] == 1 and line["n_gpus"] == 1
    assert line["config"]["workload"] == "cfg0_cpu_fp32" and line["data"] == "synthetic"
    # same configuration keys as the GPU arm prints
    for key in ("batch_per_gpu", "queries", "levels", "heads", "head_dim", "points"):
        assert key in line["config"]
    base = line["cpu_baseline"]
    # the reference's own eager backend where its package was staged, else the restatement of it
    from oracle import build_ref

    assert base["kind"] == ("reference" if build_ref.staged_package() else "port")
    assert base["cores"] >= 1 and base["value"] == line["value"]
    assert "sample" in base and base["unit"] == line["unit"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"],
                           "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_arm_under_a_launcher_only_rank_zero_reports():
    import os

    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    done = _run("--impl", "reference", "--workload", "cfg0_cpu_fp32", "--steps", "1",
                "--warmup", "1", "--gpus", "2", env=env)
    assert done.returncode == 0 and done.stdout.strip() == ""


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        import pytest

        pytest.skip("a GPU is present")
    done = _run("--steps", "1", "--warmup", "1")
    assert done.returncode != 0
    assert "CUDA" in done.stderr
