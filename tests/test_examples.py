"""The example scripts still run end to end (each in its own process: they create their own fake process groups).
(Reference: its CI runs the examples on every change, .github/workflows/test_cuda.yml:55-60.)"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,expect", [
    ("example_autoparallel.py", "ran one local step"),
    ("example_moe_planner.py", "collectives:"),
    ("example_fp8_linear.py", "scaled_mm"),
    ("example_flex_attention.py", "gradients: 5 of 5"),
])
def test_example_runs(script, expect):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script)], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-3000:]
    assert expect in out.stdout, out.stdout[-2000:]
