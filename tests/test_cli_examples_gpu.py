"""The command-line entry points and the examples run end to end on a GPU."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
ENV = dict(os.environ, PYTHONPATH=str(ROOT / "sm120-nvfp4-training_b200") + os.pathsep + os.environ.get("PYTHONPATH", ""))


def run(*args, timeout=600):
    res = subprocess.run([sys.executable, *args], cwd=ROOT, env=ENV, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout


def test_list_profiles_cli():
    out = run("-m", "nvfp4_training", "list").split()
    assert out == ["balanced", "short128", "conservative", "same_as_v5", "experimental_m4v4", "experimental_fp8_master"]


@pytest.mark.parametrize("profile", ["balanced", "experimental_fp8_master"])
def test_check_cli_one_profile(tmp_path, profile):
    target = tmp_path / "check.json"
    run("-m", "nvfp4_training", "check", "--profile", profile, "--output", str(target))
    report = json.loads(target.read_text())
    assert report["status"] == "passed" and len(report["cases"]) == 4 and all(c["exact_resume"] for c in report["cases"])
    assert all((c["gemms"], c["sr"], c["rht"], c["final_step"]) == (9, 6, 6, 7) for c in report["cases"])


def test_bench_cli_small(tmp_path):
    target = tmp_path / "bench.json"
    run("-m", "nvfp4_training", "bench", "--warmup", "2", "--steps", "3", "--rounds", "2", "--output", str(target))
    report = json.loads(target.read_text())
    assert report["sr_calls"] == 128 and report["tokens_s"] > 0 and len(report["rounds_ms"]) == 2


@pytest.mark.parametrize("script,args", [("train.py", []), ("train.py", ["--eager", "--profile", "conservative"]),
                                         ("frozen.py", []), ("lora.py", ["nvfp4"]), ("lora.py", ["preserve"])])
def test_examples(script, args):
    out = run(str(ROOT / "examples" / script), *args)
    assert "loss" in out
    if script == "lora.py":
        assert "restored adapters identical: True" in out
