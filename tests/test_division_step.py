"""The reciprocal-multiply-correct sequence that replaces the division instruction in the Normalize
and row-norm kernels gives the IEEE quotient: checked on the host with the same three operations
(float multiply, two fused multiply-adds) over ten million operand pairs inside the range the
kernels' guard admits."""
import os
import shutil
import subprocess

import pytest

SRC = os.path.join(os.path.dirname(__file__), "support", "division_step.c")


def test_division_step_matches_ieee_division(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("gcc not available")
    exe = str(tmp_path / "division_step")
    # -ffp-contract=off: the three operations must stay exactly as written
    build = subprocess.run([gcc, "-O2", "-ffp-contract=off", "-o", exe, SRC, "-lm"], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    out = subprocess.run([exe, "10000000"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == "0", out.stdout
