"""Regenerates ``q8_1_ref_seed24.npz`` from the reference's own NumPy restatement.

Run where the reference checkout is mounted::

    python tests/golden/make_q8_1_ref_golden.py /path/to/JJJetson_Ops

It imports ``q8_1_ref`` from the reference's ``tests/test_q8_1.py`` (:5-62) with the compiled
``q8_1_me`` module stubbed out (the function itself is pure NumPy), feeds it the exact input of
the reference test (:71-73: ``np.random.seed(24)``, ``randn(2048, 13, 1, 1)``, Fortran order) and a
second, smaller seeded case, and stores what it returns.  The inputs are not stored: the legacy
``np.random.seed`` stream is stable across NumPy versions, and the tests regenerate them.
"""
import importlib.util
import os
import sys
import types

import numpy as np


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: %s /path/to/JJJetson_Ops" % sys.argv[0])
    ref_root = sys.argv[1]
    sys.modules["q8_1_me"] = types.ModuleType("q8_1_me")  # only the GPU entry points live there
    spec = importlib.util.spec_from_file_location(
        "ref_test_q8_1", os.path.join(ref_root, "tests", "test_q8_1.py")
    )
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    out = {}
    for tag, seed, ne1 in (("a", 24, 13), ("b", 7, 3)):
        np.random.seed(seed)
        x = np.asfortranarray(np.random.randn(2048, ne1, 1, 1).astype(np.float32))
        qs, d, s = mod.q8_1_ref(x)
        out[f"{tag}_seed"] = np.int64(seed)
        out[f"{tag}_ne1"] = np.int64(ne1)
        out[f"{tag}_qs"] = qs
        out[f"{tag}_scale"] = d
        out[f"{tag}_sum"] = s
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "q8_1_ref_seed24.npz"), **out)
    print("wrote", os.path.join(here, "q8_1_ref_seed24.npz"))


if __name__ == "__main__":
    main()
