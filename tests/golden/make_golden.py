"""Generate tests/golden/small_cases.npz: outputs of the COMPILED REFERENCE (its own CPU kernels,
built by oracle/build.py into oracle/_ref/) on every case of tests/cases.py:small_cases().

Inputs are not stored: they are seeded draws that tests/cases.py regenerates bit-identically.
Outputs above cases.GOLDEN_FULL_LIMIT elements are stored as a SHA-256 digest of their bytes.
Run from the repository root on a machine that has the reference tree:
    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import build as obuild  # noqa: E402
from oracle import oracle as orc  # noqa: E402
import cases  # noqa: E402


def main():
    obuild.build_ref()
    lib = orc.ref_library()
    assert lib is not None, "reference tree not available"
    out = {}
    for case in cases.small_cases():
        y = cases.run_net(lib, case)
        if y.size > cases.GOLDEN_FULL_LIMIT:
            # large outputs are pinned by digest only, to keep the fixture small
            out[case["name"] + "/sha256"] = np.frombuffer(hashlib.sha256(y.tobytes()).digest(), dtype=np.uint8)
        else:
            out[case["name"]] = y
        out[case["name"] + "/shape"] = np.array(y.shape, dtype=np.int32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "small_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", sum(k.endswith("/shape") for k in out), "cases")


if __name__ == "__main__":
    main()
