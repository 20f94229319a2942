"""Host replay of the fixed-column float4 walk that the strided Softmax, the Normalize family and the
inner-kept Reduce share (shadow_b200/csrc/colwalk.cuh): every thread of every block is replayed on the
CPU for a list of geometries - ragged `inner` (49, 3, 5), even and multiple-of-4 `inner`, planes smaller
than a block, rows longer than a block, the benchmark shapes - and coverage (each float4 exactly once),
fixed columns per lane, row arithmetic and shared-memory slot layout are checked."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(os.path.dirname(__file__), "support", "colwalk_cover.cu")

GEOMETRIES = [
    (3, 1000, 49), (40, 1000, 49), (2, 21, 4096), (1, 21, 262144), (4, 512, 1444), (3, 4, 3), (2, 6, 6), (3, 8, 5),
    (7, 1, 8), (2, 2, 2), (1, 1, 4), (2, 3, 4100), (2, 64, 50), (2, 12, 1028), (5, 512, 196), (600, 64, 196),
    (3, 17, 36), (9, 4, 1), (2, 100, 1026), (1, 4, 2049), (3, 33, 12), (11, 8, 7), (2, 40, 1023), (1, 7, 2052),
    # long columns: too many float4 per thread for the patch-in-registers kernels
    (3, 1000, 49), (2, 4000, 49), (2, 3000, 196), (1, 9000, 1444), (2, 2002, 6),
]


@pytest.mark.parametrize("passes", [0, 1, 2])
def test_every_float4_once_and_lanes_stay_on_their_columns(tmp_path, passes):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    exe = str(tmp_path / "colwalk_cover")
    build = subprocess.run([nvcc, "-O1", "-std=c++17", "-I" + os.path.join(ROOT, "include"),
                            "-I" + os.path.join(ROOT, "shadow_b200", "csrc"), "-o", exe, SRC], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    args = [str(passes)] + [str(v) for g in GEOMETRIES for v in g]
    out = subprocess.run([exe] + args, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = out.stdout.strip().splitlines()
    assert len(lines) == len(GEOMETRIES)
    assert sum(1 for ln in lines if ln.startswith("ok")) >= len(GEOMETRIES) - (12 if passes == 2 else 6), out.stdout
