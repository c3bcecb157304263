"""The reference's own test file, run unmodified against this library's drop-in module.

``tests/test_q8_1.py`` of the reference imports ``q8_1_me`` and checks ``quantize`` / ``parse`` against its
NumPy restatement (seed 24, ``randn(2048, 13, 1, 1)``; ``qs`` exact, scales 1e-5, sums 1e-2).  Here the file is
run as it lies in the reference checkout, in a subprocess whose module path leads to
``jjjetson_ops_b200/python`` - nothing of it is copied or restated.  The checkout is found through the
JQ_REFERENCE_ROOT environment variable or the ``reference_path`` entry of BASELINE.json; where there is none
(the checkout does not travel to every machine) the test is skipped.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_root():
    candidates = [os.environ.get("JQ_REFERENCE_ROOT")]
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            candidates.append(json.load(f).get("reference_path"))
    except (OSError, ValueError):
        pass
    for c in candidates:
        if c and os.path.isfile(os.path.join(c, "tests", "test_q8_1.py")):
            return c
    return None


def test_reference_test_q8_1_passes_unmodified(native_lib, cuda_device, tmp_path):
    ref = _reference_root()
    if ref is None:
        pytest.skip("no reference checkout on this machine (JQ_REFERENCE_ROOT)")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.path.join(ROOT, "jjjetson_ops_b200", "python") + os.pathsep + env.get("PYTHONPATH", "")
    env["PYTHONDONTWRITEBYTECODE"] = "1"  # the checkout may be read-only
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", os.path.join(ref, "tests", "test_q8_1.py"), "-q", "-p", "no:cacheprovider",
         "--rootdir", str(tmp_path)],
        cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "1 passed" in proc.stdout, proc.stdout[-2000:]
